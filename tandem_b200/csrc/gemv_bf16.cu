// y[m, n] = sum_k x[m, k] * w[n, k] for up to eight rows of x (a batch of so many decoding
// requests), or up to sixteen where they fit into shared memory beside the L1: bfloat16 in,
// float32 sums, bfloat16 or float32 out.
//
// With so few rows the product is a stream of weights and nothing else, and what decides its time
// is how soon the stream starts and how little happens after it ends.  So: no shared-memory ring
// for the weights, no tensor memory, no split of K between blocks and hence no merge between
// blocks.  A block of 16 warps takes 16 rows of the weight matrix at a time; its warps share the
// K range, each streams its slice of the 16 rows straight from global memory into registers
// (16 bytes a load, eight loads in flight per lane and the next eight issued before the last
// eight are used) and multiplies with `mma.sync` m16n8k16: the weights are the A operand (16
// rows), the rows of x the B operand (8 columns; rows that x does not have are zeros; with nine to
// sixteen rows of x every weight fragment goes into two MMAs, one per eight rows).  The
// registers that a lane loads are not in the order the instruction names, but a sum over k does
// not care in which order k is walked as long as A and B walk it alike: the lane with thread
// index t in its group takes, of every 64 k, the eight at 8 t and the eight at 32 + 8 t, for A
// from global memory and for B from the copy of x in shared memory (where x is too large for a
// copy that leaves the L1 cache enough room to keep the loads in flight, 164 KB, B comes from
// global memory too, along with the weights of its round).  The 16 partial tiles of a
// block are added in warp order by 128 of its threads.  The first loads are on their way before
// the kernel in front of this one has finished, two rounds of them (weights are written by no kernel).  Every sum is
// taken in one fixed order whatever the grid and however many rows x has.
// With `gated` the rows of w are [gate | up] halves of I rows each and y [M, I] = silu(x gate^T) *
// (x up^T): the 16 rows a block takes at a time are 8 gate rows (the upper half of the MMA tile)
// and the 8 up rows that go with them (the lower half), and the thread that adds a place's gate
// sum up adds its up sum up too (both rounded to bfloat16, as the product alone would store them).
//
// The residual add and the RMSNorm that stand between two products of a decoder layer can ride along,
// so that they need no launch of their own.  RMSNorm scales row m by one number,
// s[m] = rsqrt(mean(r[m]^2) + eps), and a product is linear in its rows:
//     (s[m] r[m, :] * g) W^T  =  s[m] ((r[m, :] * g) W^T)        (g: the norm's weight)
// so the product in front (mode ADD) adds its result into the float32 residual r instead of storing
// it, writes r * g rounded to bfloat16 beside it, and leaves, per block, the sums of squares of the
// entries it wrote; the product behind (mode SCALE) reads those rows as its x, adds the partial
// sums up in block order while its weights stream, and multiplies row m of its result by s[m] in
// float32 before anything else is done to it.  No block reads a row twice and no block waits.
// 12vivi/tandem has kernels of this kind for the same case (python/tandem/layers/triton_gemv.py:25-88),
// with the norm in the product's prologue (triton_gemv.py:92-145).
#include "common.cuh"

namespace tb {

constexpr int GV_WARPS = 16, GV_THREADS = GV_WARPS * 32;
constexpr int GV_STEPS = 2;  // steps of 64 k per round: 2 rows x 2 pieces x 2 steps = 8 loads of 16 bytes in flight per lane

__device__ __forceinline__ uint4 load_weights(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int MODE_PLAIN = 0, MODE_ADD = 1, MODE_SCALE = 2;

struct GemvFuse {
  // MODE_ADD (not gated): the product is not stored but added
  float* residual;         // [M, N] float32: residual += bfloat16(product)
  const float* norm_w;     // [N]: the weight of the norm behind the add
  __nv_bfloat16* scaled;   // [M, N] out: bfloat16(residual * norm_w)
  float* partials_out;     // [gridDim.x, 8 NT] out: this block's sums of squares of the residual entries it wrote
  // MODE_SCALE: row m of the product is multiplied by rsqrt(sum_p partials[p][m] / K + eps)
  const float* partials;   // [parts, 8 NT]
  int parts;
  float eps;
};
// (NT: tiles of eight rows of x, 1 or 2; the rows of `partials` and `partials_out` have 8 NT entries)

template <bool X_IN_SMEM>
struct Round {  // what a lane holds of one round: [step][row g | row g + 8][piece t | piece 4 + t]
  uint4 w[GV_STEPS][2][2];
  uint4 b[X_IN_SMEM ? 1 : GV_STEPS][2];  // the lane's pieces of row g of x, where x is not in shared memory
};

template <bool X_IN_SMEM, int MODE, int NT>
__global__ void __launch_bounds__(GV_THREADS, 1)
gemv_kernel(const uint4* __restrict__ x, const uint4* __restrict__ w, void* __restrict__ y, int M, int N, int pieces,
            int x_stride, int out_f32, int gated, int sets, const GemvFuse f) {
  static_assert(NT == 1 || X_IN_SMEM, "more than eight rows of x are taken from shared memory only");
  constexpr int TILE = 128 * NT;  // floats of a warp's partial tile: 16 rows of w by 8 NT rows of x, [NT][16][8]
  // Two sets of partial tiles, used in turn, so that a group needs one meeting of the block.  With sixteen rows of x
  // the second set is given up where it would push the block into the next carve-out of shared memory (`sets` = 1:
  // a second meeting per group instead): what the copy of x leaves of the SM's memory is the L1, which bounds the
  // loads in flight.  Measured at K = 4096: 9 to 14 rows (132 KB) stream within 2 to 7 % of 8 rows' time (100 KB),
  // 15 and 16 rows (164 KB) 15 % behind it; the second meeting costs 1 % of a decode step.
  const int SETS = NT == 1 ? 2 : sets;
  extern __shared__ uint4 smem[];
  __shared__ float row_scale[8 * NT];  // MODE_SCALE: the rows' rsqrt(mean square + eps)
  __shared__ float ssq_s[4 * NT][8];   // MODE_ADD: sums of squares of what this block wrote, per warp and row
  uint4* xs = smem;                                                    // [M][x_stride] pieces of 8 k
  float* red = reinterpret_cast<float*>(smem + (X_IN_SMEM ? (size_t)M * x_stride : 0));  // [SETS][GV_WARPS][NT][16 rows][8 columns]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int steps = (pieces + 7) >> 3;  // steps of 64 k
  const int s0 = warp * steps / GV_WARPS, s1 = (warp + 1) * steps / GV_WARPS;  // this warp's part of K
  // groups of 16 rows; gated: 8 gate rows and their 8 up rows, I = N / 2 a multiple of 8
  const int half_rows = N >> 1;
  const int groups = gated ? half_rows >> 3 : (N + 15) >> 4;
  const int my_groups = ((int)blockIdx.x < groups) ? (groups - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int group_rows = gated ? 8 : 16, second_half = gated ? half_rows : 8;  // rows g and g + 8 of the tile in w

  auto load_x = [&](int s, Round<X_IN_SMEM>& r) {
    if (X_IN_SMEM) return;
#pragma unroll
    for (int u = 0; u < GV_STEPS; ++u)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int c = (s + u) * 8 + h * 4 + t;
        r.b[X_IN_SMEM ? 0 : u][h] = (g < M && s + u < s1 && c < pieces) ? __ldcg(x + (size_t)g * pieces + c) : make_uint4(0, 0, 0, 0);
      }
  };
  auto load_round = [&](int j, int s, Round<X_IN_SMEM>& r) {  // group number j of this block, steps s .. s + GV_STEPS - 1
    const int row_a = ((int)blockIdx.x + j * (int)gridDim.x) * group_rows + g, row_b = row_a + second_half;
    const uint4* wa = w + (size_t)row_a * pieces;
    const uint4* wb = w + (size_t)row_b * pieces;
#pragma unroll
    for (int u = 0; u < GV_STEPS; ++u) {
      const bool live = s + u < s1;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int c = (s + u) * 8 + h * 4 + t;
        const bool in_k = live && c < pieces;
        r.w[u][0][h] = (in_k && row_a < N) ? load_weights(wa + c) : make_uint4(0, 0, 0, 0);
        r.w[u][1][h] = (in_k && row_b < N) ? load_weights(wb + c) : make_uint4(0, 0, 0, 0);
      }
    }
  };

  Round<X_IN_SMEM> cur, nxt;
  const bool streams = s0 < s1 && my_groups > 0;
  // Two rounds of weights are on their way before this kernel waits for the one in front (weights are
  // written by no kernel): what the registers hold anyway, a round in use and the next one.
  bool second_ahead = false;
  if (streams) {
    load_round(0, s0, cur);
    int nj = 0, ns = s0 + GV_STEPS;
    if (ns >= s1) { ns = s0; ++nj; }
    if (nj < my_groups) { load_round(nj, ns, nxt); second_ahead = true; }
  }
  pdl_wait();  // x is the output of the kernel in front
  if (X_IN_SMEM) {
    // a warp reads only its own part of K of every row: it copies that part and meets nobody but itself
    const int c0 = s0 * 8, width = min(pieces, s1 * 8) - c0;
    for (int i = lane; i < M * width; i += 32) {
      const int row = i / width, c = c0 + i % width;
      xs[row * x_stride + c] = x[(size_t)row * pieces + c];
    }
    __syncwarp();
  } else if (streams) {
    load_x(s0, cur);
  }

  if (MODE == MODE_SCALE && warp < M) {
    // one warp per row: the partial sums in block order, lane by lane, then the lanes in a fixed tree; the result is
    // first read in an epilogue, behind the block-wide barrier in front of it
    float ss = 0.f;
    for (int p = lane; p < f.parts; p += 32) ss += __ldcg(f.partials + p * (8 * NT) + warp);
    ss = warp_sum(ss);
    if (lane == 0) row_scale[warp] = rsqrtf(ss / (float)(pieces * 8) + f.eps);
  }
  float wrote_sq = 0.f;  // MODE_ADD: squares of the residual entries this thread wrote
  // MODE_ADD: the residual entry and the norm weight of the place this thread finishes in a group are fetched when
  // the group begins, not when its sums are ready: a round trip to the L2 less at the end of every group
  float res_old = 0.f, gain = 0.f;
  auto fetch_place = [&](int jj) {
    if (MODE == MODE_ADD && threadIdx.x < TILE && jj < my_groups) {
      const int n = ((int)blockIdx.x + jj * (int)gridDim.x) * group_rows + ((threadIdx.x & 127) >> 3);
      const int col = (threadIdx.x & 7) + 8 * (threadIdx.x >> 7);
      if (col < M && n < N) {
        res_old = __ldcg(f.residual + (size_t)col * N + n);
        gain = f.norm_w[n];
      }
    }
  };
  fetch_place(0);
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
  int j = 0, s = s0;
  while (j < my_groups) {
    int nj = j, ns = s + GV_STEPS;
    if (ns >= s1) { ns = s0; ++nj; }
    // Once the block's last loads are on their way the kernel behind this one may begin to launch: its
    // blocks find room only as these exit, but the launch itself is out of the way by then.  All blocks
    // of this kernel are resident from the start (one per SM), so none of them can be kept out by a
    // dependent that has moved in early.  Measured on a decode step at batch 8, Qwen3-8B sizes: 3.57 ms
    // against 3.63 ms with the trigger at the very end.  The kernel behind must want the same split of
    // the SM's memory into shared memory and L1 as this one (another streaming product does): see the
    // note in attention_decode.cu on what happens otherwise.
    if (nj >= my_groups) pdl_launch_dependents();
    if (streams) {
      if (nj < my_groups) {
        if (!second_ahead) load_round(nj, ns, nxt);
        load_x(ns, nxt);
      }
      second_ahead = false;
#pragma unroll
      for (int u = 0; u < GV_STEPS; ++u) {
        if (s + u < s1) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int c = (s + u) * 8 + h * 4 + t;
            const uint4 &a0 = cur.w[u][0][h], &a1 = cur.w[u][1][h];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              uint4 b = make_uint4(0, 0, 0, 0);
              if (X_IN_SMEM) {
                if (g + 8 * nt < M && c < pieces) b = xs[(g + 8 * nt) * x_stride + c];
              } else {
                b = cur.b[X_IN_SMEM ? 0 : u][h];
              }
              mma_16816(acc[nt], a0.x, a1.x, a0.y, a1.y, b.x, b.y);
              mma_16816(acc[nt], a0.z, a1.z, a0.w, a1.w, b.z, b.w);
            }
          }
        }
      }
    }
    if (nj != j) {  // the group is complete as far as this warp goes: the block adds its 16 partial tiles up
      float* mine = red + ((size_t)(j & (SETS - 1)) * GV_WARPS + warp) * TILE;
      if (SETS == 1) __syncthreads();  // the sums of the group before have been taken (a group of streaming ago)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        *reinterpret_cast<float2*>(mine + nt * 128 + g * 8 + 2 * t) = make_float2(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<float2*>(mine + nt * 128 + (g + 8) * 8 + 2 * t) = make_float2(acc[nt][2], acc[nt][3]);
        acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
      }
      __syncthreads();
      if (threadIdx.x < TILE) {  // a thread per place of the tile: (row of w, row of x)
        const int row = (threadIdx.x & 127) >> 3, col = (threadIdx.x & 7) + 8 * (threadIdx.x >> 7);
        const float* part = red + (size_t)(j & (SETS - 1)) * GV_WARPS * TILE + threadIdx.x;
        float sum = 0.f, second = 0.f;
#pragma unroll
        for (int q = 0; q < GV_WARPS; ++q) sum += part[q * TILE];
        const int n = ((int)blockIdx.x + j * (int)gridDim.x) * group_rows + row;
        const float scale = (MODE == MODE_SCALE && col < M) ? row_scale[col] : 1.f;
        if (MODE == MODE_SCALE) sum *= scale;
        if (!gated) {
          if (MODE == MODE_ADD) {
            if (col < M && n < N) {  // residual += the product as bfloat16 would have stored it
              const float v = res_old + __bfloat162float(__float2bfloat16_rn(sum));
              f.residual[(size_t)col * N + n] = v;
              f.scaled[(size_t)col * N + n] = __float2bfloat16_rn(v * gain);
              wrote_sq += v * v;
            }
            fetch_place(nj);
          } else if (col < M && n < N) {
            if (out_f32) reinterpret_cast<float*>(y)[(size_t)col * N + n] = sum;
            else reinterpret_cast<__nv_bfloat16*>(y)[(size_t)col * N + n] = __float2bfloat16_rn(sum);
          }
        } else if (row < 8) {  // the formula of the activation kernel (tokenwise.cu), on the values it would read
#pragma unroll
          for (int q = 0; q < GV_WARPS; ++q) second += part[q * TILE + 64];
          if (MODE == MODE_SCALE) second *= scale;
          const float gate = __bfloat162float(__float2bfloat16_rn(sum)), up = __bfloat162float(__float2bfloat16_rn(second));
          if (col < M)
            reinterpret_cast<__nv_bfloat16*>(y)[(size_t)col * half_rows + n] =
                __float2bfloat16_rn(__fdividef(gate, 1.f + __expf(-gate)) * up);
        }
      }
    }
    if (streams) cur = nxt;
    j = nj;
    s = ns;
  }
  if (MODE == MODE_ADD) {  // threads 0 .. 128 NT - 1 hold (row of w = (tid % 128) / 8, row of x = tid % 8 + 8 (tid / 128)): rows of w summed in a fixed order
    if (threadIdx.x < TILE) {
      wrote_sq += __shfl_xor_sync(0xffffffffu, wrote_sq, 8);
      wrote_sq += __shfl_xor_sync(0xffffffffu, wrote_sq, 16);
      if (lane < 8) ssq_s[warp][lane] = wrote_sq;
    }
    __syncthreads();
    if (threadIdx.x < 8 * NT) {
      const int w0 = 4 * (threadIdx.x >> 3), c = threadIdx.x & 7;  // the four warps that hold this row of x
      f.partials_out[(size_t)blockIdx.x * (8 * NT) + threadIdx.x] = ssq_s[w0][c] + ssq_s[w0 + 1][c] + ssq_s[w0 + 2][c] + ssq_s[w0 + 3][c];
    }
  }
  pdl_launch_dependents();  // (blocks without work)
}

}  // namespace tb

extern "C" {

// Rows of x the kernel takes, and the shared memory up to which x is copied there (the next
// larger carve-out of the SM's memory leaves the L1 cache 28 KB, and the loads in flight halve).
// More than 8 rows are taken only from shared memory, and only up to the carve-out below that one:
// measured at K = 4096, 9 to 14 rows stream within 2 to 7 % of 8 rows' time, 15 and 16 (164 KB) 15 % behind it.
int tb_gemv_max_rows() { return 16; }
int tb_gemv_max_smem_bytes() { return 164 * 1024; }
int tb_gemv_max_smem_bytes_two_tiles() { return 130 * 1024; }

// Pieces (of 8 k) between two rows of x in shared memory: four more than a multiple of eight, so that
// the 16-byte reads of a quarter warp (two rows, four pieces each) fall into eight different bank groups.
static int x_stride_of(int pieces) { return pieces + ((4 - pieces % 8) + 8) % 8; }

// The sets of partial tiles: two, or with more than 8 rows one where two do not fit beside x.
static int x_bytes(int M, int K) { return M * x_stride_of(K / 8) * 16; }
static int sets_of(int M, int K) {
  return (M <= 8 || x_bytes(M, K) + 2 * tb::GV_WARPS * 256 * 4 <= tb_gemv_max_smem_bytes_two_tiles()) ? 2 : 1;
}
static int reduce_bytes(int M, int K) { return sets_of(M, K) * tb::GV_WARPS * (M > 8 ? 256 : 128) * 4; }

// Whether the kernel takes M rows of K: up to 8 always, up to 16 if x fits into shared memory.
int tb_gemv_takes(int M, int K) {
  if (M <= 0 || M > tb_gemv_max_rows() || K <= 0 || (K & 7)) return 0;
  return M <= 8 || x_bytes(M, K) + reduce_bytes(M, K) <= tb_gemv_max_smem_bytes_two_tiles();
}

// The number of blocks a launch with these sizes uses: the rows of `partials_out` that MODE_ADD writes.
int tb_gemv_grid(int N, int gated, int blocks) {
  const int groups = gated ? N / 16 : (N + 15) / 16;
  return blocks < groups ? blocks : groups;
}

static int launch_gemv(void* stream, const void* x, const void* w, void* y, int M, int N, int K, int out_f32, int gated, int blocks,
                       int mode, const tb::GemvFuse& f) {
  if (M <= 0 || N <= 0) return 0;
  if (!tb_gemv_takes(M, K) || blocks <= 0) return TB_ERR_BAD_SIZE;
  if (gated && (out_f32 || N % 16 != 0)) return TB_ERR_BAD_SIZE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return TB_ERR_BAD_SIZE;
  const int stride = x_stride_of(K / 8), with_x = x_bytes(M, K) + reduce_bytes(M, K);
  const bool in_smem = with_x <= tb_gemv_max_smem_bytes();
  const bool two = M > 8;  // two tiles of eight rows of x (in shared memory then, tb_gemv_takes)
  typedef void (*Kernel)(const uint4*, const uint4*, void*, int, int, int, int, int, int, int, const tb::GemvFuse);
  Kernel kernel =
      two ? (mode == tb::MODE_ADD ? (Kernel)tb::gemv_kernel<true, tb::MODE_ADD, 2>
             : mode == tb::MODE_SCALE ? (Kernel)tb::gemv_kernel<true, tb::MODE_SCALE, 2> : (Kernel)tb::gemv_kernel<true, tb::MODE_PLAIN, 2>)
      : mode == tb::MODE_ADD   ? (in_smem ? (Kernel)tb::gemv_kernel<true, tb::MODE_ADD, 1> : (Kernel)tb::gemv_kernel<false, tb::MODE_ADD, 1>)
      : mode == tb::MODE_SCALE ? (in_smem ? (Kernel)tb::gemv_kernel<true, tb::MODE_SCALE, 1> : (Kernel)tb::gemv_kernel<false, tb::MODE_SCALE, 1>)
                               : (in_smem ? (Kernel)tb::gemv_kernel<true, tb::MODE_PLAIN, 1> : (Kernel)tb::gemv_kernel<false, tb::MODE_PLAIN, 1>);
  static bool allowed[64][12] = {};  // the larger shared memory is asked for once per device and kernel
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= 64) return TB_ERR_BAD_SIZE;
  const int which = (two ? 6 : 0) + mode * 2 + in_smem;
  if (!allowed[device][which]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tb_gemv_max_smem_bytes());
    if (e != cudaSuccess) return (int)e;
    allowed[device][which] = true;
  }
  const int groups = gated ? N / 16 : (N + 15) / 16;
  return tb::launch(kernel, dim3(blocks < groups ? blocks : groups), dim3(tb::GV_THREADS),
                    (size_t)(in_smem ? with_x : reduce_bytes(M, K)), stream, (const uint4*)x, (const uint4*)w, y, M, N, K / 8, stride,
                    out_f32, gated, sets_of(M, K), f);
}

// x [M, K] and w [N, K] bfloat16, both contiguous and 16-byte aligned, K a multiple of 8; y [M, N], or with
// gated (bfloat16 out only, N = 2 I with I a multiple of 8) y [M, I] = silu(x w[:I]^T) * (x w[I:]^T).
int tb_gemv(void* stream, const void* x, const void* w, void* y, int M, int N, int K, int out_f32, int gated, int blocks) {
  return launch_gemv(stream, x, w, y, M, N, K, out_f32, gated, blocks, tb::MODE_PLAIN, tb::GemvFuse{});
}

// residual [M, N] float32 += bfloat16(x w^T); scaled [M, N] = bfloat16(residual * norm_w); partials_out
// [tb_gemv_grid(N, 0, blocks), 8 or, with more than 8 rows, 16] = every block's sums of squares of the residual entries it wrote (rows beyond M: zero).
int tb_gemv_add(void* stream, const void* x, const void* w, float* residual, const float* norm_w, void* scaled, float* partials_out,
                int M, int N, int K, int blocks) {
  if (!residual || !norm_w || !scaled || !partials_out) return TB_ERR_BAD_SIZE;
  tb::GemvFuse f{};
  f.residual = residual; f.norm_w = norm_w; f.scaled = (__nv_bfloat16*)scaled; f.partials_out = partials_out;
  return launch_gemv(stream, x, w, nullptr, M, N, K, 0, 0, blocks, tb::MODE_ADD, f);
}

// As tb_gemv, with row m of the product multiplied by rsqrt(sum_p partials[p][m] / K + eps) before it is rounded (or,
// with gated, before the activation): x holds rows r * g of which the norm's scale has been left out.
int tb_gemv_scaled(void* stream, const void* x, const void* w, void* y, int M, int N, int K, int out_f32, int gated, int blocks,
                   const float* partials, int parts, float eps) {
  if (!partials || parts <= 0) return TB_ERR_BAD_SIZE;
  tb::GemvFuse f{};
  f.partials = partials; f.parts = parts; f.eps = eps;
  return launch_gemv(stream, x, w, y, M, N, K, out_f32, gated, blocks, tb::MODE_SCALE, f);
}

}  // extern "C"
