// Y[M, N] = X[M, K] * W[N, K]^T for few rows (M <= 64) in bfloat16 with float32 accumulation: the
// matrix product of a decode step, which is one pass over the weights at memory speed.
//
// Blackwell-native: the weights are the *A* operand of tcgen05.mma (128 rows of W per tile, so the
// rows of W fill the 128 lanes of tensor memory), the M activation rows are the B operand (N of the
// MMA = M padded to 16, 32 or 64); TMA brings [128 x 64] weight boxes and [Mpad x 64] activation
// boxes into a ring of shared-memory stages in the 128-byte-swizzled layout the MMA reads; the
// accumulator lives in tensor memory, double-buffered so that the epilogue of one tile overlaps
// the main loop of the next.  Warps: 0-3 epilogue (tcgen05.ld, each warp its quarter of the
// lanes), 4 TMA producer, 5 MMA issuer.
//
// Work is cut stream-K fashion: the (N tile, K chunk) pairs are dealt to one persistent block per
// SM in contiguous, equal ranges, so every SM streams the same number of bytes whatever N and K
// are.  A tile whose K range is shared by several blocks is summed by the block that arrives last
// (an atomic counter per tile, reset by that block), from float32 partials in scratch memory, in
// block order: the result does not depend on timing.
//
// 12vivi/tandem has Triton weight-streaming kernels for batch <= 8 in this place
// (python/tandem/layers/triton_gemv.py:26-87,285-297) and cuBLAS beyond.
#include <cuda.h>

#include "common.cuh"
#include "sm100_primitives.cuh"

namespace tb {

constexpr int BN = 128;  // rows of W per tile (the M of the MMA)
constexpr int BOX_K = 64;  // K elements per TMA box: 128 bytes, one swizzle row
constexpr int BOXES = 2;   // boxes per stage, next to each other along K (256 contiguous bytes per row of W)
constexpr int BK = BOX_K * BOXES;  // K elements per stage
constexpr int SK_THREADS = 192;

// first chunk of block p when `total` chunks are dealt to `blocks` blocks
__host__ __device__ __forceinline__ long long range_start(long long p, long long total, long long blocks) { return p * total / blocks; }

__host__ __device__ __forceinline__ int block_of_chunk(long long c, long long total, long long blocks) {
  long long p = c * blocks / total;
  while (p + 1 < blocks && range_start(p + 1, total, blocks) <= c) ++p;
  while (p > 0 && range_start(p, total, blocks) > c) --p;
  return (int)p;
}

struct SkinnyArgs {
  void* y;         // [M, N] bf16 or f32
  float* partial;  // [grid][2][Mpad][BN] float32
  int* counters;   // [tiles * 4], zero between launches
  int* status;
  int M, N, K, mpad, out_f32, stages;
};

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                   smem_u32(dst)),
               "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ uint64_t smem_desc_sw128(const void* p) {
  // K-major operand tile of 128-byte rows, 8-row groups 1024 bytes apart, 128-byte swizzle
  return (uint64_t)((smem_u32(p) & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Four MMAs along the 64 K elements of a box (16 each = 32 bytes = 2 descriptor units) in one
// straight line: what the issuing thread computes between two MMAs bounds their rate (measured: 96
// cycles per MMA with the descriptors worked out in between, under 50 without), and after the
// first bytes of a launch have arrived, all stages are full at once and the MMAs are what is waited for.
__device__ __forceinline__ void umma_bf16_x4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
      "setp.ne.b32 p0, %4, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
      "add.s64 a1, %1, 2;\n\tadd.s64 a2, %1, 4;\n\tadd.s64 a3, %1, 6;\n\t"
      "add.s64 b1, %2, 2;\n\tadd.s64 b2, %2, 4;\n\tadd.s64 b3, %2, 6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, p1;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate_first)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_load_16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__global__ void __launch_bounds__(SK_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const SkinnyArgs a) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
  const int stages = a.stages, mpad = a.mpad;
  const int stage_bytes = BN * BK * 2 + mpad * BK * 2;  // W boxes, then X boxes
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)stages * stage_bytes);
  uint64_t* empty = full + stages;
  uint64_t* acc_full = empty + stages;   // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long KC = (a.K + BK - 1) / BK, NT = (a.N + BN - 1) / BN, total = KC * NT, blocks = gridDim.x;
  const long long c_begin = range_start(blockIdx.x, total, blocks), c_end = range_start(blockIdx.x + 1, total, blocks);

  // The producer's first lane sets the barriers up and starts the first loads at once; everything
  // else of the prologue (tensor memory, the block-wide sync) hides behind their latency.
  pdl_launch_dependents();  // by every thread: the kernel behind this one may become resident
  int produced = 0;
  if (warp == 4 && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    for (int s = 0; s < stages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 4); }
    *abort_flag = 0;
    mbar_fence_init();
    // weights are written by no kernel: their first stages are on their way before the kernel in
    // front of this one has finished; the activations follow once it has
    for (long long c = c_begin; c < c_end && produced < stages; ++c, ++produced) {
      const int tile = (int)(c / KC), kc = (int)(c % KC);
      unsigned char* ws = smem + (size_t)produced * stage_bytes;
      mbar_arrive_expect_tx(full + produced, (uint32_t)stage_bytes);
#pragma unroll
      for (int b = 0; b < BOXES; ++b)
        tma_load_2d(ws + b * BN * BOX_K * 2, &map_w, kc * BK + b * BOX_K, tile * BN, full + produced);
    }
    pdl_wait();
    int s = 0;
    for (long long c = c_begin; s < produced; ++c, ++s) {
      const int kc = (int)(c % KC);
      unsigned char* ws = smem + (size_t)s * stage_bytes;
#pragma unroll
      for (int b = 0; b < BOXES; ++b)
        tma_load_2d(ws + BN * BK * 2 + b * mpad * BOX_K * 2, &map_x, kc * BK + b * BOX_K, 0, full + s);
    }
  }
  if (warp == 0) {  // tensor memory for two accumulators of mpad columns (128 columns cover 2 x 64)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(128) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  pdl_wait();  // (the producer's first lane has waited already)
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int it = produced;
      for (long long c = c_begin + produced; c < c_end; ++c, ++it) {
        const int slot = it % stages;
        if (!mbar_wait(empty + slot, ((it / stages) & 1) ^ 1, abort_flag, a.status)) break;
        const int tile = (int)(c / KC), kc = (int)(c % KC);
        unsigned char* ws = smem + (size_t)slot * stage_bytes;
        mbar_arrive_expect_tx(full + slot, (uint32_t)stage_bytes);
#pragma unroll
        for (int b = 0; b < BOXES; ++b) {
          tma_load_2d(ws + b * BN * BOX_K * 2, &map_w, kc * BK + b * BOX_K, tile * BN, full + slot);
          tma_load_2d(ws + BN * BK * 2 + b * mpad * BOX_K * 2, &map_x, kc * BK + b * BOX_K, 0, full + slot);
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(mpad >> 3) << 17) | ((uint32_t)(BN >> 4) << 24);
      int it = 0, seg = 0;
      long long c = c_begin;
      while (c < c_end) {
        const long long tile = c / KC;
        const long long seg_end = min(c_end, (tile + 1) * KC);
        const int buf = seg & 1;
        if (seg >= 2 && !mbar_wait(acc_empty + buf, ((seg >> 1) & 1) ^ 1, abort_flag, a.status)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d = tmem_base + (uint32_t)(buf * mpad);
        bool ok = true;
        for (bool first = true; c < seg_end; ++c, ++it, first = false) {
          const int slot = it % stages;
          if (!mbar_wait(full + slot, (it / stages) & 1, abort_flag, a.status)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned char* ws = smem + (size_t)slot * stage_bytes;
          static_assert(BOX_K == 64, "four MMAs of 16 K elements per box");
#pragma unroll
          for (int b = 0; b < BOXES; ++b)
            umma_bf16_x4(d, smem_desc_sw128(ws + b * BN * BOX_K * 2), smem_desc_sw128(ws + BN * BK * 2 + b * mpad * BOX_K * 2), idesc,
                         (first && b == 0) ? 0u : 1u);
          umma_commit(empty + slot);  // the stage is free once these MMAs have read it
        }
        if (!ok) break;
        umma_commit(acc_full + buf);
        ++seg;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 0-3)
    int seg = 0;
    long long c = c_begin;
    const int col = warp * 32 + lane;  // this thread's row of W inside the tile = TMEM lane
    while (c < c_end) {
      const long long tile = c / KC;
      const long long seg_begin = c, seg_end = min(c_end, (tile + 1) * KC);
      c = seg_end;
      const int buf = seg & 1;
      // the whole warp gives up or none of it: the loads from tensor memory below want all 32 lanes
      if (!__all_sync(0xffffffffu, mbar_wait(acc_full + buf, (seg >> 1) & 1, abort_flag, a.status))) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool whole = seg_begin == tile * KC && seg_end == (tile + 1) * KC;
      const long long n = tile * BN + col;
      float* part = a.partial + ((size_t)blockIdx.x * 2 + (seg == 0 ? 0 : 1)) * mpad * BN;
      for (int t0 = 0; t0 < mpad; t0 += 16) {
        float v[16];
        tmem_load_16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(buf * mpad + t0), v);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int t = t0 + j;
          if (t >= a.M) continue;
          if (!whole) part[(size_t)t * BN + col] = v[j];
          else if (n < a.N) {
            if (a.out_f32) reinterpret_cast<float*>(a.y)[(size_t)t * a.N + n] = v[j];
            else reinterpret_cast<__nv_bfloat16*>(a.y)[(size_t)t * a.N + n] = __float2bfloat16_rn(v[j]);
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + buf);
      ++seg;
      if (whole) continue;
      // A shared tile: each warp owns 32 of the tile's columns in every block that works on the tile;
      // the warp that arrives last for its quarter adds up that quarter's partials, in block order.
      __syncwarp();
      const int p_lo = block_of_chunk(tile * KC, total, blocks), p_hi = block_of_chunk((tile + 1) * KC - 1, total, blocks);
      int last = 0;
      if (lane == 0) last = arrive_acq_rel(a.counters + tile * 4 + warp) == p_hi - p_lo;
      last = __shfl_sync(0xffffffffu, last, 0);
      if (!last) continue;
      // 16 tokens at a time, so that 16 loads are in flight per contributor
      for (int t0 = 0; t0 < a.M; t0 += 16) {
        float sum[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) sum[j] = 0.f;
        for (int q0 = p_lo; q0 <= p_hi; q0 += 4) {  // four contributors' loads in flight, summed in block order
          float v[4][16];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int q = q0 + i;
            const int slot = range_start(q, total, blocks) >= tile * KC ? 0 : 1;
            const float* src = a.partial + ((size_t)q * 2 + slot) * mpad * BN + (size_t)t0 * BN + col;
#pragma unroll
            for (int j = 0; j < 16; ++j) v[i][j] = (q <= p_hi && t0 + j < a.M) ? __ldcg(src + (size_t)j * BN) : 0.f;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 16; ++j) sum[j] += v[i][j];
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int t = t0 + j;
          if (t >= a.M || n >= a.N) continue;
          if (a.out_f32) reinterpret_cast<float*>(a.y)[(size_t)t * a.N + n] = sum[j];
          else reinterpret_cast<__nv_bfloat16*>(a.y)[(size_t)t * a.N + n] = __float2bfloat16_rn(sum[j]);
        }
      }
      if (lane == 0) a.counters[tile * 4 + warp] = 0;
    }
  }
  // ------------------------------------------------------------------ teardown
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*abort_flag) for (int i = 0; i < 2000; ++i) __nanosleep(100);  // let copies in flight land
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(128) : "memory");
  }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_tiled() {
  static EncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(p);
  }
  return fn;
}

// [rows, K] bf16 row-major, boxes of [box_rows x 64 elements] with the 128-byte swizzle
static int make_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows) {
  EncodeTiled enc = encode_tiled();
  if (!enc) return TB_ERR_BAD_SIZE;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BOX_K, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 20000 + (int)r;
}

}  // namespace tb

extern "C" {

// Scratch the caller provides: partial >= blocks * 2 * 64 * 128 floats, counters >= 4 * ceil(N / 128)
// ints that are zero (the kernel leaves them zero).  `blocks`: persistent blocks (one per SM).
int tb_gemm_skinny(void* stream, const void* x, const void* w, void* y, float* partial, int* counters, int* status,
                   int M, int N, int K, int out_f32, int blocks) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || K % 8 != 0 || blocks <= 0) return TB_ERR_BAD_SIZE;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return TB_ERR_BAD_SIZE;
  const int mpad = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  CUtensorMap map_w, map_x;
  int e = tb::make_map(&map_w, w, N, K, tb::BN);
  if (e) return e;
  e = tb::make_map(&map_x, x, M, K, mpad);
  if (e) return e;
  const int stage_bytes = tb::BN * tb::BK * 2 + mpad * tb::BK * 2;
  const int stages = mpad == 64 ? 4 : 5;
  const size_t smem = 1024 + (size_t)stages * stage_bytes + (2 * stages + 4) * 8 + 16;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t ce = cudaFuncSetAttribute(tb::gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    configured = smem;
  }
  const long long total = (long long)((K + tb::BK - 1) / tb::BK) * ((N + tb::BN - 1) / tb::BN);
  tb::SkinnyArgs a;
  a.y = y; a.partial = partial; a.counters = counters; a.status = status;
  a.M = M; a.N = N; a.K = K; a.mpad = mpad; a.out_f32 = out_f32; a.stages = stages;
  const int grid = (int)(total < blocks ? total : blocks);
  return tb::launch(tb::gemm_skinny_kernel, dim3(grid), dim3(tb::SK_THREADS), smem, stream, map_w, map_x, a);
}

}  // extern "C"
