// Y[M, N] = X[M, K] * W[N, K]^T for many rows in bfloat16 with float32 accumulation, computed by
// pairs of blocks on neighbouring SMs (tcgen05 with cta_group::2): the matrix product of a prefill
// step where the single-block kernel (gemm_wide.cu) is bound by what its SM can bring in.
//
// A pair of blocks (a cluster of two) computes output tiles of 256 rows of X by up to 256 rows of
// W.  Each block brings its own 128 rows of X and its own HALF of the tile's rows of W (ordinary 2-D
// TMA into its own shared memory; no load is multicast), K in stages of 64.  One thread of the
// pair's first block issues the MMAs for both: M = 256 is split over the two blocks' tensor cores,
// each of which reads its block's rows of X and both blocks' halves of W, and accumulates its 128
// rows x 256 columns in its own tensor memory (twice, so that the epilogue of one tile overlaps
// the main loop of the next).  Against gemm_wide a block moves 32 KB a stage through its shared
// memory and from the L2 instead of 48 KB for the same 512 cycles of tensor-core time, and six
// stages fit where four did.
//
// Barriers.  `full` (first block only): both blocks' producers announce their bytes there (the
// second block's copies complete on the first block's barrier: cp.async.bulk.tensor with
// cta_group::2) and the issuing thread waits on it.  `empty` and `acc_full` exist in both blocks
// and are completed in both by one tcgen05.commit with a two-block mask.  `acc_empty` (first
// block only) counts the epilogue warps of both blocks (the second block's arrive remotely).
// Every wait is bounded (sm100_primitives.cuh); the two cluster-wide meetings (after set-up, and
// before the blocks leave: neither may go while the other still signals into its shared memory
// or its tensor cores read its operands) are reached by every thread on every path.
//
// With `gated` the rows of W are [gate | up] halves of I rows each: the first block brings the tile's
// gate rows, the second its up rows, and the epilogue writes silu(gate) * up, [M, I].
//
// Warps: 0-3 epilogue (each its 32 lanes of tensor memory), 4 and 6 TMA producers (even and odd
// stages), 5 MMA issuer (first block only).
// 12vivi/tandem runs these products through cuBLAS (python/tandem/layers/linear.py:14) and the
// activation as its own kernel (python/tandem/layers/mlp.py:36-44).
#include <cuda.h>

#include "common.cuh"
#include "sm100_primitives.cuh"

namespace tb {

constexpr int PM = 128;  // rows of X per block (256 per pair)
constexpr int PN = 256;  // most rows of W per tile; a launch uses a.wn of them, each block half
constexpr int PK = 64;   // K elements per stage: 128 bytes, one swizzle row
constexpr int P_STAGES = 6;
constexpr int P_STAGE_BYTES = (PM + PN / 2) * PK * 2;
constexpr int P_THREADS = 224;

// With -DTB_PAIR_TRACE the first block adds up where its issuing thread and one producer spend their
// cycles (tb_gemm_wide_pair_trace reads the sums): what showed that a remote arrival with release
// semantics held the producers for 1,500 cycles a stage.
#ifdef TB_PAIR_TRACE
__device__ long long tb_pair_trace[16];
#define PTRACE(i, v) do { if (blockIdx.x == 0) tb_pair_trace[i] += (v); } while (0)
#else
#define PTRACE(i, v) do { } while (0)
#endif

struct PairArgs {
  void* y;
  int* status;
  int M, N, K;  // N: rows of W; with `gated`, N = 2 I
  int out_f32, gated;
  int m_tiles, n_tiles;  // tiles of 256 rows of X, of wn rows of W
  int wn;  // rows of W per tile: a multiple of 32 from 128 to 256 (with `gated` a multiple of 64: half gate rows, half up rows)
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_meet() {  // every thread of both blocks
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address, in the cluster's shared-memory window, of this block's `p` as it stands in block `rank`
__device__ __forceinline__ uint32_t in_block(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void remote_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void remote_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.relaxed.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");  // announces bytes, publishes nothing
}
// 2-D tensor copy into this block's shared memory that completes on a barrier of either block of the pair
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                   smem_u32(dst)),
               "l"(map), "r"(bar), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ uint64_t pair_desc_sw128(const void* p) {
  // K-major operand tile of 128-byte rows, 8-row groups 1024 bytes apart, 128-byte swizzle
  return (uint64_t)((smem_u32(p) & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// Four MMAs of the pair along the 64 K elements of a stage (16 each = 32 bytes = 2 descriptor
// units), both operands in shared memory (at the same places in both blocks).
__device__ __forceinline__ void umma_pair_x4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
      "setp.ne.b32 p0, %4, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
      "add.s64 a1, %1, 2;\n\tadd.s64 a2, %1, 4;\n\tadd.s64 a3, %1, 6;\n\t"
      "add.s64 b1, %2, 2;\n\tadd.s64 b2, %2, 4;\n\tadd.s64 b3, %2, 6;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], a1, b1, %3, p1;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], a2, b2, %3, p1;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], a3, b3, %3, p1;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate_first)
      : "memory");
}
// arrives, once the MMAs issued so far have completed, on the barrier at this place in both blocks
__device__ __forceinline__ void umma_commit_both(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "h"((uint16_t)3)
               : "memory");
}

__device__ __forceinline__ void pair_tmem_load_32(uint32_t taddr, float (&v)[32]) {
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

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gemm_wide_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const PairArgs a) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)P_STAGES * P_STAGE_BYTES);  // used in the first block
  uint64_t* empty = full + P_STAGES;
  uint64_t* acc_full = empty + P_STAGES;  // [2]
  uint64_t* acc_empty = acc_full + 2;     // [2], used in the first block
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int KC = (a.K + PK - 1) / PK;
  const int tiles = a.m_tiles * a.n_tiles;
  const int half = a.wn / 2;  // rows of W a block brings per tile

  if (warp == 4 && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    for (int s = 0; s < P_STAGES; ++s) { mbar_init(full + s, 2); mbar_init(empty + s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 8); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {  // one warp of each block of the pair, together
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_meet();  // both blocks' barriers stand and both have their tensor memory
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  pdl_launch_dependents();  // every block of this grid holds its tensor memory now
  pdl_wait();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4 || warp == 6) {
    // ------------------------------------------------------------------ TMA producers (both blocks)
    if (lane == 0) {
      const int mine = warp == 4 ? 0 : 1;
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += pairs) {
        const int mt = tile % a.m_tiles, nt = tile / a.m_tiles;
        // this block's rows of W: with `gated` the first block has the gate rows, the second the up rows
        const int w_row = a.gated ? (int)rank * (a.N / 2) + nt * half : nt * a.wn + (int)rank * half;
        for (int kc = 0; kc < KC; ++kc, ++it) {
          if ((it & 1) != mine) continue;
          const int slot = it % P_STAGES;
          const long long tp0 = clock64();
          if (it >= P_STAGES && !mbar_wait(empty + slot, ((it / P_STAGES) & 1) ^ 1, abort_flag, a.status)) { ok = false; break; }
          const long long tp1 = clock64();
          if (mine == 0) PTRACE(4, tp1 - tp0);
          unsigned char* xs = smem + (size_t)slot * P_STAGE_BYTES;
          unsigned char* ws = xs + PM * PK * 2;
          const uint32_t bar = in_block(full + slot, 0);
          remote_arrive_expect_tx(bar, (uint32_t)((PM + half) * PK * 2));
          tma_load_2d_pair(xs, &map_x, kc * PK, mt * 2 * PM + (int)rank * PM, bar);
          tma_load_2d_pair(ws, &map_w, kc * PK, w_row, bar);
          if (mine == 0) { PTRACE(5, clock64() - tp1); PTRACE(6, 1); }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer (first block only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(a.wn >> 3) << 17) | ((uint32_t)((2 * PM) >> 4) << 24);
      int it = 0, local = 0;
      for (int tile = pair; tile < tiles; tile += pairs, ++local) {
        const int buf = local & 1;
        const long long ta0 = clock64();
        if (local >= 2 && !mbar_wait(acc_empty + buf, ((local >> 1) & 1) ^ 1, abort_flag, a.status)) break;
        PTRACE(0, clock64() - ta0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d = tmem_base + (uint32_t)(buf * PN);
        bool ok = true;
        for (int kc = 0; kc < KC; ++kc, ++it) {
          const int slot = it % P_STAGES;
          const long long tf0 = clock64();
          if (!mbar_wait(full + slot, (it / P_STAGES) & 1, abort_flag, a.status)) { ok = false; break; }
          const long long tf1 = clock64();
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned char* xs = smem + (size_t)slot * P_STAGE_BYTES;
          umma_pair_x4(d, pair_desc_sw128(xs), pair_desc_sw128(xs + PM * PK * 2), idesc, kc ? 1u : 0u);
          umma_commit_both(empty + slot);  // the stage is free in both blocks once these MMAs have read it
          PTRACE(1, tf1 - tf0); PTRACE(2, clock64() - tf1); PTRACE(3, 1);
        }
        if (!ok) break;
        umma_commit_both(acc_full + buf);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 0-3 of both blocks): one row of X per thread
    int local = 0;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    for (int tile = pair; tile < tiles; tile += pairs, ++local) {
      const int mt = tile % a.m_tiles, nt = tile / a.m_tiles;
      const int buf = local & 1;
      // the whole warp gives up or none of it: the loads from tensor memory below want all 32 lanes
      if (!__all_sync(0xffffffffu, mbar_wait(acc_full + buf, (local >> 1) & 1, abort_flag, a.status))) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = mt * 2 * PM + (int)rank * PM + warp * 32 + lane;
      const uint32_t acc = tmem_base + lane_base + (uint32_t)(buf * PN);
      if (a.gated) {
        const int out_n = a.N / 2;
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.y) + (size_t)row * out_n + nt * half;
#pragma unroll 1
        for (int c0 = 0; c0 < half; c0 += 32) {
          float g[32], u[32];
          pair_tmem_load_32(acc + c0, g);
          pair_tmem_load_32(acc + half + c0, u);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (row < a.M) {
#pragma unroll
            for (int c = 0; c < 32; c += 8) {
              if (nt * half + c0 + c >= out_n) break;  // I is a multiple of 8
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                // the gate and up products are rounded to bfloat16 first, as when they are stored and read back
                const float g0 = __bfloat162float(__float2bfloat16_rn(g[c + 2 * j])), g1 = __bfloat162float(__float2bfloat16_rn(g[c + 2 * j + 1]));
                const float u0 = __bfloat162float(__float2bfloat16_rn(u[c + 2 * j])), u1 = __bfloat162float(__float2bfloat16_rn(u[c + 2 * j + 1]));
                w[j] = pack2(__fdividef(g0, 1.f + __expf(-g0)) * u0, __fdividef(g1, 1.f + __expf(-g1)) * u1);
              }
              *reinterpret_cast<uint4*>(dst + c0 + c) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < a.wn; c0 += 32) {
          float v[32];
          pair_tmem_load_32(acc + c0, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          const int n0 = nt * a.wn + c0;
          if (row < a.M && n0 < a.N) {
            if (a.out_f32) {
              float* dst = reinterpret_cast<float*>(a.y) + (size_t)row * a.N + n0;
#pragma unroll
              for (int c = 0; c < 32; c += 4)
                if (n0 + c < a.N) *reinterpret_cast<float4*>(dst + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);  // N is a multiple of 8
            } else {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.y) + (size_t)row * a.N + n0;
#pragma unroll
              for (int c = 0; c < 32; c += 8)
                if (n0 + c < a.N)
                  *reinterpret_cast<uint4*>(dst + c) = make_uint4(pack2(v[c], v[c + 1]), pack2(v[c + 2], v[c + 3]), pack2(v[c + 4], v[c + 5]), pack2(v[c + 6], v[c + 7]));
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) remote_arrive(in_block(acc_empty + buf, 0));
    }
  }
  // ------------------------------------------------------------------ teardown
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*abort_flag) for (int i = 0; i < 2000; ++i) __nanosleep(100);  // let copies in flight land
  cluster_meet();  // neither block leaves while the other may still signal into it or have its operands read
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
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

// [rows, K] bf16 row-major, boxes of [box_rows x 64 elements] with the 128-byte swizzle; rows and
// columns beyond the tensor read as zeros
static int make_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows) {
  EncodeTiled enc = encode_tiled();
  if (!enc) return TB_ERR_BAD_SIZE;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)PK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 20000 + (int)r;
}

}  // namespace tb

extern "C" {

// y [M, N] (bf16, or float32 with out_f32) = x [M, K] w[N, K]^T; with gated (bf16 only, N = 2 I even,
// I a multiple of 8): y [M, I] = silu(x w[:I]^T) * (x w[I:]^T).  K and N multiples of 8.  `blocks`: SMs of the device.
#ifdef TB_PAIR_TRACE
int tb_gemm_wide_pair_trace(long long* host, int reset) {
  if (reset) { long long z[16] = {0}; return (int)cudaMemcpyToSymbol(tb::tb_pair_trace, z, sizeof(z)); }
  return (int)cudaMemcpyFromSymbol(host, tb::tb_pair_trace, sizeof(tb::tb_pair_trace));
}
#endif
int tb_gemm_wide_pair(void* stream, const void* x, const void* w, void* y, int* status, int M, int N, int K, int out_f32,
                      int gated, int blocks) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || N % 8 != 0 || blocks < 2) return TB_ERR_BAD_SIZE;
  if (gated && (out_f32 || N % 16 != 0)) return TB_ERR_BAD_SIZE;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)y & 15)) return TB_ERR_BAD_SIZE;
  const int pairs = blocks / 2;
  // rows of W per tile: the candidate with the fewest waves' worth of time, useful columns only
  const int m_tiles = (M + 2 * tb::PM - 1) / (2 * tb::PM), out_cols = gated ? N / 2 : N;
  int wn = tb::PN;
  double best = 1e300;
  for (int cand = tb::PN; cand >= 128; cand -= gated ? 64 : 32) {  // gated: both halves multiples of 32
    const int per_tile = gated ? cand / 2 : cand;
    const long long tiles = (long long)m_tiles * ((out_cols + per_tile - 1) / per_tile);
    const double cost = (double)((tiles + pairs - 1) / pairs) * (160 + cand);  // waves x time of a tile (measured: a fixed part too)
    if (cost < best - 1e-9) { best = cost; wn = cand; }
  }
  CUtensorMap map_x, map_w;
  int e = tb::make_map(&map_x, x, M, K, tb::PM);
  if (e) return e;
  e = tb::make_map(&map_w, w, N, K, wn / 2);
  if (e) return e;
  const size_t smem = 1024 + (size_t)tb::P_STAGES * tb::P_STAGE_BYTES + (2 * tb::P_STAGES + 4) * 8 + 16;
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(tb::gemm_wide_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  tb::PairArgs a;
  a.y = y; a.status = status; a.M = M; a.N = N; a.K = K; a.out_f32 = out_f32; a.gated = gated;
  a.wn = wn;
  a.m_tiles = m_tiles;
  a.n_tiles = gated ? (N / 2 + wn / 2 - 1) / (wn / 2) : (N + wn - 1) / wn;
  const int tiles = a.m_tiles * a.n_tiles;
  const int grid = 2 * (tiles < pairs ? tiles : pairs);
  return tb::launch(tb::gemm_wide_pair_kernel, dim3(grid), dim3(tb::P_THREADS), smem, stream, map_x, map_w, a);
}

}  // extern "C"
