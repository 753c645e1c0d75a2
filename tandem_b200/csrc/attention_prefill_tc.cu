// Paged causal attention for prompt portions on the fifth-generation tensor cores (tcgen05), head
// size TB_HD (64 or 128) fixed at compile time.  Same contract as attention_prefill.cu (query tiles
// of 128 rows = (token, query head of the group) pairs, one block per tile and kv head, keys and
// values streamed from the request's pages by the TMA unit); what differs is who does the math:
//
//   warp 9   issues S = Q K^T (tcgen05.mma, M = 128 rows, N = 64 keys) into one of two score
//            buffers in tensor memory;
//   warp 10  issues O += P V (M = 128, N = head size) into the output accumulator, also in tensor
//            memory (a thread of its own, so that the scores of the next block never queue behind
//            a wait for this block's probabilities).
//            The A operands of both products live in tensor memory too: the query tile (stored
//            there once, by the threads that own its rows) and the probabilities (two buffers).
//            Shared memory then carries only what it must, the keys and values: with Q and P in
//            shared memory its bandwidth (128 bytes a cycle) was what bounded the kernel;
//   warps 0-7  a row of the MMA is a lane of tensor memory, and a warp reaches the 32 lanes of its
//            number modulo 4: warps 0-3 take the even blocks of keys and warps 4-7 the odd ones,
//            one query row per thread, so that on every scheduler one warp exponentiates (the
//            special-function unit is the narrow resource: 64 x 128 exp2 per block) while the
//            other loads, masks and waits.  The two threads of a row hand the row's reference
//            maximum to each other through shared memory, block by block.  They
//            read a row of S with tcgen05.ld, mask it, keep the running maximum and sum in
//            float32 (exp2), write the probabilities as bfloat16 pairs into tensor memory
//            (tcgen05.st), the A operand of the second MMA, and rescale O in tensor memory when
//            the reference maximum has to move (only when a row's maximum grew by more than 2^8
//            since the reference was set: the sum is kept against the same reference, so the
//            result is exact);
//   warps 8 and 11  are the producers (bulk copies of cache tiles, completing on mbarriers), one
//            for the even stages and one for the odd ones: a stage costs a warp about a thousand
//            cycles of dependent instructions, more than the tensor cores need for it.
//
// While the softmax warps work on block j, the tensor cores already compute the scores of block
// j + 1.  The cache's own tile layout (cache_layout.cuh) is the 128-byte-swizzled layout that
// tcgen05 reads: K is a K-major B operand as it lies, V an MN-major one.
//
// It stands where 12vivi/tandem calls FlashInfer's paged prefill wrapper
// (python/tandem/layers/flashinfer_attention.py:167-171,194-209); the arithmetic is
// python/tandem/layers/attention.py:46-56 of the reference.
#include "attention_common.cuh"

namespace tb {

static_assert(HD == 64 || HD == 128, "the tcgen05 prefill kernel takes head sizes 64 and 128");
constexpr int BM = 128;            // rows of a query tile
constexpr int BLOCK_KEYS = 64;     // keys per stage
#ifndef TB_PF_STAGES
#define TB_PF_STAGES (TB_HD == 128 ? 6 : 8)
#endif
constexpr int STAGES = TB_PF_STAGES;  // one block per SM
constexpr int SOFTMAX_WARPS = 8, PRODUCER_WARP = 8, SCORE_WARP = 9, OUTPUT_WARP = 10, PRODUCER_WARP_2 = 11;
constexpr int THREADS = 384;
constexpr int TILE_INTS = 4;       // first token row, request, first position, number of tokens
constexpr int K_BYTES = BLOCK_KEYS * HD * 2, STAGE_BYTES = 2 * K_BYTES;
constexpr int TMEM_COLS = 512;     // S0 at 0, S1 at 64, O at 128, P0 at 256, P1 at 288, Q at 320 (bfloat16 pairs per column)
constexpr int TMEM_O = 128, TMEM_P = 256, TMEM_Q = 320;
constexpr float RESCALE_AT = 8.f;  // move a row's reference maximum when it has grown by 2^8

struct PrefillArgs {
  const __nv_bfloat16* q;
  int q_stride;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_table;
  int table_stride;
  const int* tiles;
  __nv_bfloat16* out;
  int* status;
  int nh, nkv, page_size, window;
  float scale_log2;
};

// ------------------------------------------------------------------------------------------- tcgen05
// Shared-memory operand descriptors, 128-byte swizzle: rows of 128 bytes in groups of eight.
__device__ __forceinline__ uint64_t desc_k_major(const void* p, uint32_t group_stride_bytes) {  // 8-row groups that far apart
  return (uint64_t)((smem_u32(p) & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(group_stride_bytes >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
__device__ __forceinline__ uint64_t desc_mn_major(const void* p, uint32_t block_stride_bytes, uint32_t group_stride_bytes) {
  // rows of 64 contiguous N elements; groups of 8 K-rows group_stride apart, 64-element N blocks block_stride apart
  return (uint64_t)((smem_u32(p) & 0x3FFFFu) >> 4) | ((uint64_t)(block_stride_bytes >> 4) << 16) |
         ((uint64_t)(group_stride_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Four MMAs along K (16 elements each) in one straight line: A moves on by 8 columns of tensor
// memory, B's descriptor by BSTEP (in 16-byte units).  One thread issues all MMAs of the kernel,
// and what it computes between two of them is what bounds their rate: measured 96 cycles per MMA
// with the operands worked out in between, 46 (N = 64) and 64 (N = 128, the nominal rate) without.
template <int BSTEP>
__device__ __forceinline__ void umma_ts_x4(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t.reg .b32 a1, a2, a3;\n\t.reg .b64 b1, b2, b3;\n\t"
      "setp.ne.b32 p0, %4, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
      "add.u32 a1, %1, 8;\n\tadd.u32 a2, %1, 16;\n\tadd.u32 a3, %1, 24;\n\t"
      "add.s64 b1, %2, %5;\n\tadd.s64 b2, %2, %6;\n\tadd.s64 b3, %2, %7;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], b2, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], b3, %3, p1;\n\t}" ::"r"(d),
      "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate_first), "n"(BSTEP), "n"(2 * BSTEP), "n"(3 * BSTEP)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, float* v) {  // tmem_ld_wait() before v is read
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
      "%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  tmem_ld32_issue(taddr, v);
  tmem_ld_wait();
}
__device__ __forceinline__ float fast_exp2(float x) {  // 2^x, -inf -> 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_st32_words(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
      "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};" ::"r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
      "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
      "r"(v[30]), "r"(v[31]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
      "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};" ::"r"(__float_as_uint(v[0])),
      "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])),
      "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
      "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])),
      "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])),
      "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])),
      "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])),
      "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])),
      "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31])), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ------------------------------------------------------------------------------------------- kernel
__global__ void __launch_bounds__(THREADS, 1) attention_prefill_tc_kernel(const PrefillArgs a) {
  extern __shared__ unsigned char smem_unaligned[];
  pdl_wait();
  unsigned char* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
  unsigned char* stage_mem = smem;                 // [STAGES][K | V]
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(stage_mem + STAGES * STAGE_BYTES);
  uint64_t* kv_empty = kv_full + STAGES;
  uint64_t* s_full = kv_empty + STAGES;   // [2]
  uint64_t* s_empty = s_full + 2;         // [2]
  uint64_t* p_full = s_empty + 2;         // [2]
  uint64_t* pv_done = p_full + 2;         // [2]
  uint64_t* pair_bar = pv_done + 2;       // [4]: the two warps that share 32 rows hand the reference maximum over
  uint64_t* q_full = pair_bar + 4;        // the query tile stands in tensor memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* m_s = reinterpret_cast<float*>(const_cast<int*>(abort_flag) + 1);  // [2 blocks][128 rows] reference maxima
  float* l_s = m_s + 4 * BM;                                                // [2 groups][128 rows] sums, then [2][128] their references
  int* table_s = reinterpret_cast<int*>(l_s + 4 * BM);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int* tile = a.tiles + (size_t)blockIdx.x * TILE_INTS;
  const int t0 = tile[0], req = tile[1], p0 = tile[2], ntok = tile[3];
  const int kvh = blockIdx.y, G = a.nh / a.nkv, ps = a.page_size, W = a.window;
  const int kb = W > 0 ? max(0, p0 - W + 1) : 0, ke = p0 + ntok;
  const int s0 = (kb / BLOCK_KEYS) * BLOCK_KEYS;
  const int num_blocks = (ke - s0 + BLOCK_KEYS - 1) / BLOCK_KEYS;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(kv_full + s, 1); mbar_init(kv_empty + s, 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_full + b, 1); mbar_init(s_empty + b, 4);
      mbar_init(p_full + b, 4); mbar_init(pv_done + b, 1);
    }
    for (int q = 0; q < 4; ++q) mbar_init(pair_bar + q, 1);
    mbar_init(q_full, 4);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  {  // the request's page numbers for this tile's keys
    const int* table = a.block_table + (size_t)req * a.table_stride;
    const int first = s0 / ps, count = (ke + ps - 1) / ps - first;
    if (count <= TABLE_CACHE)
      for (int i = tid; i < count; i += THREADS) table_s[i] = table[first + i];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // Only now may the kernel behind this one become resident: it may hold tensor memory while it
  // waits for this grid to end, so every block of this grid must have its own columns first.
  pdl_launch_dependents();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + TMEM_O;

  if (warp == PRODUCER_WARP || warp == PRODUCER_WARP_2) {
    const int* table = a.block_table + (size_t)req * a.table_stride;
    const int first = s0 / ps, count = (ke + ps - 1) / ps - first;
    stream_kv(a.k_cache, a.v_cache, count <= TABLE_CACHE ? table_s - first : table, kvh, a.nkv, ps, kb, ke, s0, num_blocks,
              STAGES, reinterpret_cast<__nv_bfloat16*>(stage_mem), kv_full, kv_empty, abort_flag, a.status, lane,
              warp == PRODUCER_WARP ? 0 : 1, 2);
  } else if (warp == SCORE_WARP) {
    // ------------------------------------------------------------------ S_j = Q K_j^T
    if (lane == 0) {
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BLOCK_KEYS >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      bool ok = mbar_wait(q_full, 0, abort_flag, a.status);
      for (int j = 0; j < num_blocks && ok; ++j) {
        const int slot = j % STAGES;
        if (!mbar_wait(kv_full + slot, (j / STAGES) & 1, abort_flag, a.status)) break;
        if (j >= 2 && !mbar_wait(s_empty + (j & 1), ((j >> 1) & 1) ^ 1, abort_flag, a.status)) break;
        tc_fence_after();
        const unsigned char* ks = stage_mem + (size_t)slot * STAGE_BYTES;
        const uint64_t kd = desc_k_major(ks, NB * 1024);
#pragma unroll
        for (int b = 0; b < NB; ++b)  // 64 elements of the head: 32 columns of Q, the next column block of K (1,024 bytes on)
          umma_ts_x4<2>(tmem_base + (uint32_t)((j & 1) * BLOCK_KEYS), tmem_base + (uint32_t)(TMEM_Q + b * 32), kd + b * 64, idesc_s, b ? 1u : 0u);
        umma_commit(s_full + (j & 1));
      }
    }
  } else if (warp == OUTPUT_WARP) {
    // ------------------------------------------------------------------ O += P_i V_i
    if (lane == 0) {
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      for (int i = 0; i < num_blocks; ++i) {
        const int slot = i % STAGES;
        // the probabilities exist only after the scores, which needed the stage's keys: its values have landed too
        if (!mbar_wait(p_full + (i & 1), (i >> 1) & 1, abort_flag, a.status)) break;
        tc_fence_after();
        const unsigned char* vs = stage_mem + (size_t)slot * STAGE_BYTES + K_BYTES;
        // 16 keys a step: 8 columns of P, two row groups (2 x NB x 1,024 bytes) down V
        umma_ts_x4<NB * 128>(tmem_o, tmem_base + (uint32_t)(TMEM_P + (i & 1) * 32), desc_mn_major(vs, 1024, NB * 1024), idesc_o, i ? 1u : 0u);
        umma_commit(kv_empty + slot);  // the scores of this stage completed before its probabilities were made
        umma_commit(pv_done + (i & 1));
      }
    }
  } else if (warp < SOFTMAX_WARPS) {
    // ------------------------------------------------------------------ softmax: one row per thread, every other block
    const int quarter = warp & 3, group = warp >> 2;
    const int row = quarter * 32 + lane;  // = lane of tensor memory
    const int tl = row / G;
    const bool live = tl < ntok;
    const int qpos = p0 + min(tl, ntok - 1);
    const int lo = W > 0 ? max(0, qpos - W + 1) : 0;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    uint64_t* pair = pair_bar + quarter;  // phase j completes when block j's reference maximum stands in m_s
    if (group == 0) {  // this thread's row of the query tile goes to tensor memory: two elements per column
      const __nv_bfloat16* src = a.q + (size_t)(t0 + tl) * a.q_stride + (size_t)(kvh * G + row % G) * HD;
#pragma unroll
      for (int c0 = 0; c0 < HD / 2; c0 += 32) {
        uint32_t w[32];
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          const uint4 v = live ? *reinterpret_cast<const uint4*>(src + (c0 + c) * 2) : make_uint4(0, 0, 0, 0);
          w[c] = v.x; w[c + 1] = v.y; w[c + 2] = v.z; w[c + 3] = v.w;
        }
        tmem_st32_words(tmem_base + lane_base + (uint32_t)(TMEM_Q + c0), w);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_full);
    }
    // m_mine: the reference this thread's sum l is kept against (the one of its last block)
    float m_mine = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = group; j < num_blocks && ok; j += 2) {
      const int base = s0 + j * BLOCK_KEYS;
      // every give-up below is taken by the whole warp or by none of it: the tensor-memory
      // instructions and __syncwarp that follow a wait want all 32 lanes
      ok = __all_sync(0xffffffffu, mbar_wait(s_full + (j & 1), (j >> 1) & 1, abort_flag, a.status));
      if (!ok) break;
      tc_fence_after();
      float s[64];
      tmem_ld32_issue(tmem_base + lane_base + (uint32_t)((j & 1) * BLOCK_KEYS), s);
      tmem_ld32_issue(tmem_base + lane_base + (uint32_t)((j & 1) * BLOCK_KEYS + 32), s + 32);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty + (j & 1));
      if (base + BLOCK_KEYS - 1 > qpos || base < lo) {  // a block at the causal or the window's edge
#pragma unroll
        for (int c = 0; c < 64; ++c)
          if (base + c > qpos || base + c < lo) s[c] = -INFINITY;
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 64; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], s[c]);
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;  // the scale is positive
      // the row's reference after the block before this one, from the thread that had that block
      float m_prev = -INFINITY;
      if (j >= 1) {
        ok = __all_sync(0xffffffffu, mbar_wait(pair, (j - 1) & 1, abort_flag, a.status));
        if (!ok) break;
        m_prev = m_s[((j - 1) & 1) * BM + row];
      }
      // move the reference only when it pays (any row of the warp: the tensor-memory instructions
      // below are executed by whole warps)
      const bool warp_need = __any_sync(0xffffffffu, mx > m_prev + RESCALE_AT);
      const float m_new = warp_need ? fmaxf(m_prev, mx) : m_prev;
      m_s[(j & 1) * BM + row] = m_new;
      __syncwarp();
      if (lane == 0) mbar_arrive(pair);
      l *= m_mine == -INFINITY ? 0.f : exp2f(m_mine - m_new);  // every move since this thread's last block
      m_mine = m_new;
      if (j >= 2) {  // this block's buffer of P is free once O += P V of the block before the last has completed
        ok = __all_sync(0xffffffffu, mbar_wait(pv_done + (j & 1), ((j - 2) >> 1) & 1, abort_flag, a.status));
        if (!ok) break;
      }
      if (j >= 1 && warp_need) {  // O is touched only between two of the tensor cores' updates; this move is this thread's
        ok = __all_sync(0xffffffffu, mbar_wait(pv_done + ((j - 1) & 1), ((j - 1) >> 1) & 1, abort_flag, a.status));
        if (!ok) break;
        tc_fence_after();
        const float corr = m_prev == -INFINITY ? 0.f : exp2f(m_prev - m_new);
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          float o[32];
          tmem_ld32(tmem_o + lane_base + c0, o);
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] *= corr;
          tmem_st32(tmem_o + lane_base + c0, o);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      const float neg_m = m_new == -INFINITY ? 0.f : -m_new;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pw[32];  // the row of P, two probabilities per word
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        const float p0 = fast_exp2(fmaf(s[c], a.scale_log2, neg_m)), p1 = fast_exp2(fmaf(s[c + 1], a.scale_log2, neg_m));
        sum4[c & 3] += p0;
        sum4[(c + 1) & 3] += p1;
        pw[c >> 1] = pack_bf16(p0, p1);
      }
      tmem_st32_words(tmem_base + lane_base + (uint32_t)(TMEM_P + (j & 1) * 32), pw);
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      if (base < kb || base + BLOCK_KEYS > ke) {
        // an edge block: value rows of keys outside [kb, ke) get zero weights, but must not hold NaN
        // patterns (they were not copied, or came along with their row group): this warp clears its quarter
        unsigned char* vs = stage_mem + (size_t)(j % STAGES) * STAGE_BYTES + K_BYTES;
        for (int i = lane; i < 16 * NB * 8; i += 32) {
          const int r = quarter * 16 + i / (NB * 8), bc = i % (NB * 8);
          if (base + r < kb || base + r >= ke)
            *reinterpret_cast<uint4*>(vs + ((r >> 3) * NB + (bc >> 3)) * 1024 + (r & 7) * 128 + ((bc & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();  // the cleared rows are read by the tensor cores through the async proxy
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + (j & 1));
    }
    // ------------------------------------------------------------------ epilogue
    // The last block's thread knows the final reference; both sums are brought to it and added.
    // Each of the two threads of a row then writes half of the row's output columns.
    constexpr int OC = HD / 2;
    const int last_group = (num_blocks - 1) & 1;
    if (ok) {
      l_s[group * BM + row] = l;
      l_s[(2 + group) * BM + row] = m_mine;
    }
    tc_fence_before();
    asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_WARPS * 32) : "memory");  // all softmax warps (every path reaches it)
    if (ok && !*abort_flag) ok = mbar_wait(pv_done + ((num_blocks - 1) & 1), ((num_blocks - 1) >> 1) & 1, abort_flag, a.status);
    ok = __all_sync(0xffffffffu, ok && !*abort_flag);  // the loads from tensor memory below are the whole warp's or nobody's
    if (ok) {
      tc_fence_after();
      const float m_final = l_s[(2 + last_group) * BM + row];
      float total = 0.f;
#pragma unroll
      for (int gg = 0; gg < 2; ++gg) {
        const float mg = l_s[(2 + gg) * BM + row];
        total += mg == -INFINITY ? 0.f : l_s[gg * BM + row] * exp2f(mg - m_final);
      }
      const float inv = total > 0.f ? 1.f / total : 0.f;
      __nv_bfloat16* dst = a.out + (size_t)(t0 + tl) * a.nh * HD + (size_t)(kvh * G + row % G) * HD + group * OC;
#pragma unroll
      for (int c0 = 0; c0 < OC; c0 += 32) {
        float o[32];
        tmem_ld32(tmem_o + lane_base + (uint32_t)(group * OC + c0), o);
        if (live) {
#pragma unroll
          for (int c = 0; c < 32; c += 8)
            *reinterpret_cast<uint4*>(dst + c0 + c) = make_uint4(pack_bf16(o[c] * inv, o[c + 1] * inv), pack_bf16(o[c + 2] * inv, o[c + 3] * inv),
                                                                 pack_bf16(o[c + 4] * inv, o[c + 5] * inv), pack_bf16(o[c + 6] * inv, o[c + 7] * inv));
        }
      }
    }
  }
  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) for (int i = 0; i < 2000; ++i) __nanosleep(100);
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

constexpr size_t smem_bytes() { return 1024 + (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 13) * 8 + 16 + 8 * BM * 4 + TABLE_CACHE * 4; }

}  // namespace tb

extern "C" {

int tb_attention_prefill_tc_tile_rows() { return tb::BM; }

// tiles: [num_tiles, 4] int32 on the device; grid = (num_tiles, nkv).  Pages of 8 keys or a multiple of 16.
int tb_attention_prefill_tc(void* stream, const void* q, int q_stride, const void* k_cache, const void* v_cache,
                            const int* block_table, int table_stride, const int* tiles, int num_tiles, void* out,
                            int* status, int nh, int nkv, int page_size, int window, float scale) {
  if (num_tiles <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || nh / nkv > tb::BM || !(scale > 0.f)) return TB_ERR_BAD_SIZE;
  if (!(page_size == 8 || (page_size > 0 && page_size % 16 == 0))) return TB_ERR_BAD_SIZE;
  tb::PrefillArgs a;
  a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride;
  a.k_cache = (const __nv_bfloat16*)k_cache; a.v_cache = (const __nv_bfloat16*)v_cache;
  a.block_table = block_table; a.table_stride = table_stride;
  a.tiles = tiles; a.out = (__nv_bfloat16*)out; a.status = status;
  a.nh = nh; a.nkv = nkv; a.page_size = page_size; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  static bool configured = false;
  const size_t smem = tb::smem_bytes();
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(tb::attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return tb::launch(tb::attention_prefill_tc_kernel, dim3(num_tiles, nkv), dim3(tb::THREADS), smem, stream, a);
}

}  // extern "C"
