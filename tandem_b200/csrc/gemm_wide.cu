// Y[M, N] = X[M, K] * W[N, K]^T for many rows (a prompt portion) in bfloat16 with float32
// accumulation on the fifth-generation tensor cores: the matrix product of a prefill step.
//
// Output tiles of 128 rows of X (the M of tcgen05.mma: a token is a lane of tensor memory) by up to
// 256 rows of W (the N of the MMA; the launcher picks the multiple of 32 from 128 to 256 that
// wastes least of the last wave of tiles), K in stages of 64: TMA brings a [128 x 64] box of X and a
// [256 x 64] box of W per stage into a ring of four 48 KB stages in the 128-byte-swizzled layout
// the MMA reads; one thread issues the four MMAs of a stage in a straight line (what it computes
// between two MMAs bounds their rate); the accumulator [128 x 256] float32 lives in tensor memory,
// twice, so that the epilogue of one tile (tcgen05.ld, conversion, 64-byte row pieces to global
// memory) overlaps the main loop of the next.  One persistent block per SM walks the tiles with the
// rows of X changing fastest, so that the blocks running at one time share few tiles of W and
// every tile of W comes from HBM once.
//
// With `gated` the rows of W are [gate | up] halves of I rows each, a tile holds 128 rows of each
// half, and the epilogue writes silu(gate) * up, [M, I]: the activation kernel and one trip of
// the intermediate through memory are saved.
//
// Measured on a B200 (2,048 rows, Qwen3-8B widths): 1.27 - 1.37 PFLOP/s, 85 - 90 % of cuBLAS.  What
// bounds it is shared memory: a stage is written once by TMA and read once by the MMAs, 96 KB
// through a 128-byte-a-cycle port = 768 cycles against 508 of tensor-core time; pairs of blocks
// that share their operands (cta_group::2) are what lifts that, and they are not built.  With the
// activation in the epilogue it is faster than the library product followed by the activation
// kernel (289 against 297 us for gate_up at 2,048 rows), which is where it is used.
//
// Warps: 0-3 epilogue (each its 32 lanes of tensor memory), 4 and 6 TMA producers (even and odd
// stages: a stage costs a thread some 700 cycles of waits and copy instructions, more than the
// tensor cores need for it), 5 MMA issuer.
// 12vivi/tandem runs these products through cuBLAS (python/tandem/layers/linear.py:14) and the
// activation as its own kernel (python/tandem/layers/mlp.py:36-44).
#include <cuda.h>

#include "common.cuh"
#include "sm100_primitives.cuh"

namespace tb {

constexpr int WM = 128;  // rows of X per tile
constexpr int WN = 256;  // most rows of W per tile; a launch uses a.wn of them
constexpr int WK = 64;   // K elements per stage: 128 bytes, one swizzle row
constexpr int W_STAGES = 4;
constexpr int W_STAGE_BYTES = (WM + WN) * WK * 2;
constexpr int W_THREADS = 224;

struct WideArgs {
  void* y;
  int* status;
  int M, N, K;       // N: rows of W; with `gated`, N = 2 I
  int out_f32, gated;
  int m_tiles, n_tiles;
  int wn;  // rows of W per tile: a multiple of 32 from 128 to 256 (with `gated`: half of them gate rows, half up rows)
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

// Four MMAs along the 64 K elements of a stage (16 each = 32 bytes = 2 descriptor units), both
// operands in shared memory.
__device__ __forceinline__ void umma_ss_x4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate_first) {
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

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, float (&v)[32]) {
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

__global__ void __launch_bounds__(W_THREADS, 1)
gemm_wide_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const WideArgs a) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)W_STAGES * W_STAGE_BYTES);
  uint64_t* empty = full + W_STAGES;
  uint64_t* acc_full = empty + W_STAGES;  // [2]
  uint64_t* acc_empty = acc_full + 2;     // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int KC = (a.K + WK - 1) / WK;
  const int tiles = a.m_tiles * a.n_tiles;

  if (warp == 4 && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    for (int s = 0; s < W_STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 4); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  pdl_launch_dependents();  // every block of this grid holds its tensor memory now
  pdl_wait();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4 || warp == 6) {
    // ------------------------------------------------------------------ TMA producers
    if (lane == 0) {
      const int mine = warp == 4 ? 0 : 1;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int mt = tile % a.m_tiles, nt = tile / a.m_tiles;
        for (int kc = 0; kc < KC; ++kc, ++it) {
          if ((it & 1) != mine) continue;
          const int slot = it % W_STAGES;
          if (it >= W_STAGES && !mbar_wait(empty + slot, ((it / W_STAGES) & 1) ^ 1, abort_flag, a.status)) { ok = false; break; }
          unsigned char* xs = smem + (size_t)slot * W_STAGE_BYTES;
          unsigned char* ws = xs + WM * WK * 2;
          mbar_arrive_expect_tx(full + slot, (uint32_t)((WM + a.wn) * WK * 2));
          tma_load_2d(xs, &map_x, kc * WK, mt * WM, full + slot);
          if (a.gated) {  // rows of the gate half, then the rows of the up half that go with them
            tma_load_2d(ws, &map_w, kc * WK, nt * (a.wn / 2), full + slot);
            tma_load_2d(ws + (a.wn / 2) * WK * 2, &map_w, kc * WK, a.N / 2 + nt * (a.wn / 2), full + slot);
          } else {
            tma_load_2d(ws, &map_w, kc * WK, nt * a.wn, full + slot);
          }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(a.wn >> 3) << 17) | ((uint32_t)(WM >> 4) << 24);
      int it = 0, local = 0;
      for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        if (local >= 2 && !mbar_wait(acc_empty + buf, ((local >> 1) & 1) ^ 1, abort_flag, a.status)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d = tmem_base + (uint32_t)(buf * WN);
        bool ok = true;
        for (int kc = 0; kc < KC; ++kc, ++it) {
          const int slot = it % W_STAGES;
          if (!mbar_wait(full + slot, (it / W_STAGES) & 1, abort_flag, a.status)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned char* xs = smem + (size_t)slot * W_STAGE_BYTES;
          umma_ss_x4(d, smem_desc_sw128(xs), smem_desc_sw128(xs + WM * WK * 2), idesc, kc ? 1u : 0u);
          umma_commit(empty + slot);  // the stage is free once these MMAs have read it
        }
        if (!ok) break;
        umma_commit(acc_full + buf);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 0-3): one row of X per thread
    int local = 0;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
      const int mt = tile % a.m_tiles, nt = tile / a.m_tiles;
      const int buf = local & 1;
      // the whole warp gives up or none of it: the loads from tensor memory below want all 32 lanes
      if (!__all_sync(0xffffffffu, mbar_wait(acc_full + buf, (local >> 1) & 1, abort_flag, a.status))) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = mt * WM + warp * 32 + lane;
      const uint32_t acc = tmem_base + lane_base + (uint32_t)(buf * WN);
      if (a.gated) {
        const int out_n = a.N / 2, half = a.wn / 2;
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.y) + (size_t)row * out_n + nt * half;
#pragma unroll 1
        for (int c0 = 0; c0 < half; c0 += 32) {
          float g[32], u[32];
          tmem_load_32(acc + c0, g);
          tmem_load_32(acc + half + c0, u);
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
          tmem_load_32(acc + c0, v);
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
      if (lane == 0) mbar_arrive(acc_empty + buf);
    }
  }
  // ------------------------------------------------------------------ teardown
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*abort_flag) for (int i = 0; i < 2000; ++i) __nanosleep(100);  // let copies in flight land
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
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
  const cuuint32_t box[2] = {(cuuint32_t)WK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 20000 + (int)r;
}

}  // namespace tb

extern "C" {

// y [M, N] (bf16, or float32 with out_f32) = x [M, K] w[N, K]^T; with gated (bf16 only, N = 2 I even,
// I a multiple of 8): y [M, I] = silu(x w[:I]^T) * (x w[I:]^T).  K and N multiples of 8.
int tb_gemm_wide(void* stream, const void* x, const void* w, void* y, int* status, int M, int N, int K, int out_f32,
                 int gated, int blocks) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || N % 8 != 0 || blocks <= 0) return TB_ERR_BAD_SIZE;
  if (gated && (out_f32 || N % 16 != 0)) return TB_ERR_BAD_SIZE;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)y & 15)) return TB_ERR_BAD_SIZE;
  // rows of W per tile: the candidate with the fewest waves' worth of time, useful columns only
  const int m_tiles = (M + tb::WM - 1) / tb::WM, out_cols = gated ? N / 2 : N;
  int wn = tb::WN;
  double best = 1e300;
  for (int cand = tb::WN; cand >= 128; cand -= gated ? 64 : 32) {  // gated: both halves multiples of 32
    const int per_tile = gated ? cand / 2 : cand;
    const long long tiles = (long long)m_tiles * ((out_cols + per_tile - 1) / per_tile);
    const double cost = (double)((tiles + blocks - 1) / blocks) * (160 + cand);  // waves x time of a tile (measured: a fixed part too)
    if (cost < best - 1e-9) { best = cost; wn = cand; }
  }
  CUtensorMap map_x, map_w;
  int e = tb::make_map(&map_x, x, M, K, tb::WM);
  if (e) return e;
  e = tb::make_map(&map_w, w, N, K, gated ? wn / 2 : wn);
  if (e) return e;
  const size_t smem = 1024 + (size_t)tb::W_STAGES * tb::W_STAGE_BYTES + (2 * tb::W_STAGES + 4) * 8 + 16;
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(tb::gemm_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  tb::WideArgs a;
  a.y = y; a.status = status; a.M = M; a.N = N; a.K = K; a.out_f32 = out_f32; a.gated = gated;
  a.wn = wn;
  a.m_tiles = m_tiles;
  a.n_tiles = gated ? (N / 2 + wn / 2 - 1) / (wn / 2) : (N + wn - 1) / wn;
  const int tiles = a.m_tiles * a.n_tiles;
  return tb::launch(tb::gemm_wide_kernel, dim3(tiles < blocks ? tiles : blocks), dim3(tb::W_THREADS), smem, stream, map_x, map_w, a);
}

}  // extern "C"
