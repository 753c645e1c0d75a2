// Paged causal attention for prompt portions (any number of new tokens per request, at any offset
// into the request) in bfloat16, head size TB_HD fixed at compile time: flash attention on the
// tensor cores, keys and values streamed from the pages by the TMA unit.
//
// The host cuts every request's new tokens into query tiles; one block runs one tile for one kv
// head.  A tile's 128 rows are (token, query head of the group) pairs, token-major, so one pass
// over the keys serves all the query heads that share the kv head.  Each of the eight consumer
// warps owns 16 rows; per stage of 64 keys it computes S = Q K^T with mma.sync, masks (causal
// with the row's own position, optional window), runs the online softmax in float32 with exp2
// and accumulates O += P V.  A ninth warp is the producer (attention_common.cuh).  Keys a portion
// needs from earlier steps and its own keys come from the cache alike: the step wrote them there
// before this kernel runs.
//
// It stands where 12vivi/tandem calls FlashInfer's paged prefill wrapper
// (python/tandem/layers/flashinfer_attention.py:167-171,194-209); the arithmetic is
// python/tandem/layers/attention.py:46-56 of the reference.
#include "attention_common.cuh"

namespace tb {

#ifndef TB_PF_WARPS
#define TB_PF_WARPS 8  // consumer warps: a query tile of 128 rows shares every stage of keys and values
#endif
#ifndef TB_PF_STAGES
#define TB_PF_STAGES (TB_HD <= 64 ? 4 : (TB_HD <= 192 ? 3 : 2))
#endif
constexpr int WARPS = TB_PF_WARPS;
constexpr int BM = WARPS * 16;  // rows of a query tile
constexpr int STAGES = TB_PF_STAGES;
constexpr int QS = HD + 8;
constexpr int THREADS = (WARPS + 1) * 32;
constexpr int TILE_INTS = 4;  // first token row, request, first position, number of tokens

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

__global__ void __launch_bounds__(THREADS) attention_prefill_kernel(const PrefillArgs a) {
  extern __shared__ unsigned char smem_unaligned[];
  pdl_launch_dependents();
  pdl_wait();
  unsigned char* smem_raw = smem_unaligned + ((128u - (smem_u32(smem_unaligned) & 127u)) & 127u);
  __nv_bfloat16* stage_mem = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* q_s = stage_mem + STAGES * STAGE_ELEMS;  // [BM][QS]
  uint64_t* full = reinterpret_cast<uint64_t*>(q_s + BM * QS);
  uint64_t* empty = full + STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + STAGES);
  int* table_s = const_cast<int*>(abort_flag) + 2;  // [TABLE_CACHE] the request's page numbers for this tile's keys

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int* tile = a.tiles + (size_t)blockIdx.x * TILE_INTS;
  const int t0 = tile[0], req = tile[1], p0 = tile[2], ntok = tile[3];
  const int kvh = blockIdx.y, G = a.nh / a.nkv, ps = a.page_size, W = a.window;
  const int xmask = min(7, ps - 1);
  const int kb = W > 0 ? max(0, p0 - W + 1) : 0, ke = p0 + ntok;  // keys any row of the tile can see
  const int s0 = (kb / STAGE_KEYS) * STAGE_KEYS;
  const int num_stages = (ke - s0 + STAGE_KEYS - 1) / STAGE_KEYS;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, WARPS); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  for (int i = tid; i < BM * (HD / 8); i += THREADS) {  // the query tile: row = token * G + head of the group
    const int row = i / (HD / 8), c = i % (HD / 8);
    const int tl = row / G, g = row % G;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tl < ntok)
      v = *reinterpret_cast<const uint4*>(a.q + (size_t)(t0 + tl) * a.q_stride + (size_t)(kvh * G + g) * HD + c * 8);
    *reinterpret_cast<uint4*>(q_s + row * QS + c * 8) = v;
  }
  const int* table = cache_table(a.block_table + (size_t)req * a.table_stride, table_s, s0, ke, ps, tid, THREADS);
  fence_proxy_async();
  __syncthreads();

  if (warp == WARPS) {
    stream_kv(a.k_cache, a.v_cache, table, kvh, a.nkv, ps, kb, ke, s0,
              num_stages, STAGES, stage_mem, full, empty, abort_flag, a.status, lane);
    return;
  }

  // ------------------------------------------------------------------ consumers
  int tl_row[2], qpos[2];  // the two rows this thread holds pieces of: lane/4 and lane/4 + 8 of the warp's 16
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    tl_row[r] = (warp * 16 + (lane >> 2) + r * 8) / G;
    qpos[r] = p0 + min(tl_row[r], ntok - 1);  // rows past the last token copy its mask; they are not written
  }
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks)
    ldmatrix_x4(qf[ks], smem_u32(q_s + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * QS + ks * 16 + (lane >> 4) * 8));

  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int warp_first_pos = p0 + min((warp * 16) / G, ntok - 1);       // lowest position among the warp's rows
  const int warp_last_pos = p0 + min((warp * 16 + 15) / G, ntok - 1);   // highest

  for (int it = 0; it < num_stages; ++it) {
    const int slot = it % STAGES;
    if (!__all_sync(0xffffffffu, mbar_wait(full + slot, (it / STAGES) & 1, abort_flag, a.status))) break;  // the whole warp or nobody
    const int base = s0 + it * STAGE_KEYS;
    __nv_bfloat16* kt = stage_mem + slot * STAGE_ELEMS;
    __nv_bfloat16* vt = kt + STAGE_KEYS * HD;
    if (base < kb || base + STAGE_KEYS > ke) {  // an edge stage: every warp cleans one sub-tile, then all read all
      if (warp < 4) zero_value_rows(vt + warp * TILE * HD, base + warp * TILE, kb, ke, lane);
      asm volatile("bar.sync 1, %0;" ::"n"(WARPS * 32) : "memory");
    }
    // keys of this stage that no row of the warp can see need no arithmetic at all
    const bool skip = base > warp_last_pos || (W > 0 && base + STAGE_KEYS <= warp_first_pos - W + 1);
    if (!skip) {
      float s[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
        for (int sub = 0; sub < 4; ++sub) {
          uint32_t b[4];
          ldmatrix_x4(b, smem_u32(kt + sub * TILE * HD + tile_elem((lane & 7) + (lane >> 4) * 8, ks * 16 + ((lane >> 3) & 1) * 8, xmask)));
          mma_bf16_16816(s[2 * sub], qf[ks], b[0], b[1]);
          mma_bf16_16816(s[2 * sub + 1], qf[ks], b[2], b[3]);
        }
      }
      // all keys of the stage visible to all rows of the warp: no mask
      const bool full_stage = base + STAGE_KEYS - 1 <= warp_first_pos && (W <= 0 || base > warp_last_pos - W);
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[nt][e] * a.scale_log2;
          if (!full_stage) {
            const int key = base + nt * 8 + (lane & 3) * 2 + (e & 1), q = qpos[e >> 1];
            if (key > q || (W > 0 && key <= q - W)) v = -INFINITY;
          }
          s[nt][e] = v;
          tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
        }
      float corr[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float mx = tile_max[r];
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[r], mx);
        const float m_safe = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen no key yet
        corr[r] = exp2f(m_run[r] - m_safe);
        m_run[r] = m_new;
        l_run[r] *= corr[r];
        tile_max[r] = m_safe;
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[nt][e] = exp2f(s[nt][e] - tile_max[e >> 1]);
          l_run[e >> 1] += s[nt][e];
        }
#pragma unroll
      for (int j = 0; j < HD / 8; ++j) { o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1]; }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint32_t pf[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                                pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
        for (int j = 0; j < HD / 8; j += 2) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, smem_u32(vt + kk * TILE * HD + tile_elem((lane & 7) + ((lane >> 3) & 1) * 8, j * 8 + (lane >> 4) * 8, xmask)));
          mma_bf16_16816(o[j], pf, b[0], b[1]);
          mma_bf16_16816(o[j + 1], pf, b[2], b[3]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty + slot);
  }
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
    return;
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    if (tl_row[r] >= ntok) continue;
    const int g = (warp * 16 + (lane >> 2) + r * 8) % G;
    const float inv = 1.f / l_run[r];
    __nv_bfloat16* dst = a.out + (size_t)(t0 + tl_row[r]) * a.nh * HD + (size_t)(kvh * G + g) * HD + (lane & 3) * 2;
#pragma unroll
    for (int j = 0; j < HD / 8; ++j)
      *reinterpret_cast<__nv_bfloat162*>(dst + j * 8) = __floats2bfloat162_rn(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
  }
}

constexpr size_t prefill_smem_bytes() { return 128 + (size_t)STAGES * STAGE_ELEMS * 2 + (size_t)BM * QS * 2 + 2 * STAGES * 8 + 16 + TABLE_CACHE * 4; }

}  // namespace tb

extern "C" {

// How many tokens one query tile takes for `groups` query heads per kv head (0: the kernel does not
// take that many heads per kv head).
int tb_attention_prefill_tile_tokens(int groups) { return groups > 0 && groups <= tb::BM ? tb::BM / groups : 0; }
int tb_attention_prefill_tile_rows() { return tb::BM; }

// tiles: [num_tiles, 4] int32 on the device; grid = (num_tiles, nkv).
int tb_attention_prefill(void* stream, const void* q, int q_stride, const void* k_cache, const void* v_cache,
                         const int* block_table, int table_stride, const int* tiles, int num_tiles, void* out,
                         int* status, int nh, int nkv, int page_size, int window, float scale) {
  if (num_tiles <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || nh / nkv > tb::BM || page_size <= 0) return TB_ERR_BAD_SIZE;
  if (!(page_size == 1 || page_size == 2 || page_size == 4 || page_size == 8 || page_size % 16 == 0))
    return TB_ERR_BAD_SIZE;
  tb::PrefillArgs a;
  a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride;
  a.k_cache = (const __nv_bfloat16*)k_cache; a.v_cache = (const __nv_bfloat16*)v_cache;
  a.block_table = block_table; a.table_stride = table_stride;
  a.tiles = tiles; a.out = (__nv_bfloat16*)out; a.status = status;
  a.nh = nh; a.nkv = nkv; a.page_size = page_size; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  static bool configured = false;
  const size_t smem = tb::prefill_smem_bytes();
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(tb::attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return tb::launch(tb::attention_prefill_kernel, dim3(num_tiles, nkv), dim3(tb::THREADS), smem, stream, a);
}

}  // extern "C"
