// A matrix product's output whose shared tiles are still in pieces.
//
// The skinny product (gemm_skinny.cu) deals (N tile, K chunk) pairs to its blocks in contiguous
// ranges; a tile of 128 output columns whose K range several blocks share exists as one float32
// partial per block until somebody adds them up.  Adding them inside the product costs three trips
// to the L2 at the end of every launch (store, count, load).  With a *split output* the product
// just stores the partials, and the kernel that reads the output anyway (residual add + RMSNorm,
// q/k norm + rotary, SiLU * up) adds them on the way in: same order (block order), same float32
// sums, same rounding to bfloat16, so the values are bit for bit those of the in-kernel reduction.
//
//   y        [M, N] bfloat16: columns of tiles that one block computed alone are final here
//   partial  [blocks][2][mpad][128] float32: slot 0 = a block's first tile, slot 1 = its last
//   tiles    [N tiles][3] int32: first and last contributing block, and the first one's slot
//            (every later contributor starts inside the tile: slot 0)
//
// It has no counterpart in 12vivi/tandem, whose split-K kernels reduce in a second launch
// (python/tandem/layers/triton_gemv.py:89-118).
#pragma once

#include <cuda_bf16.h>

namespace tb {

constexpr int SPLIT_BN = 128;  // output columns per tile

struct SplitView {
  const float* partial;  // null: a plain tensor, nothing to add up
  const int* tiles;
  int mpad;
};

// first chunk of block p when `total` chunks are dealt to `blocks` blocks
__host__ __device__ __forceinline__ long long range_start(long long p, long long total, long long blocks) { return p * total / blocks; }

__host__ __device__ __forceinline__ int block_of_chunk(long long c, long long total, long long blocks) {
  long long p = c * blocks / total;
  while (p + 1 < blocks && range_start(p + 1, total, blocks) <= c) ++p;
  while (p > 0 && range_start(p, total, blocks) > c) --p;
  return (int)p;
}

// Who contributes to the tile of column n0.  The table is written by the host, not by a kernel:
// it may be read before the dependency wait.
struct SplitTile {
  int p_lo, p_hi, slot;
};
__device__ __forceinline__ SplitTile split_tile(const SplitView& sv, int n0) {
  SplitTile s{0, 0, 0};
  if (sv.partial) {
    const int* info = sv.tiles + 3 * (n0 / SPLIT_BN);
    s.p_lo = __ldg(info); s.p_hi = __ldg(info + 1); s.slot = __ldg(info + 2);
  }
  return s;
}

// Eight neighbouring columns n0 .. n0+7 (n0 a multiple of 8) of token row t, as floats that are
// exactly representable in bfloat16.  y_row points at row t of y.  Partials are added in block
// order, eight contributors' loads in flight at a time (absent ones count as zeros), as the
// product's own reduction does.
__device__ __forceinline__ void split_load8(const __nv_bfloat16* y_row, const SplitView& sv, const SplitTile& st, int t, int n0,
                                            float (&out)[8]) {
  const int p_lo = st.p_lo, p_hi = st.p_hi, slot = st.slot;
  if (p_lo == p_hi) {
    const uint4 raw = *reinterpret_cast<const uint4*>(y_row + n0);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); out[2 * j] = f.x; out[2 * j + 1] = f.y; }
    return;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) out[j] = 0.f;
  const int col = n0 % SPLIT_BN;
  for (int q0 = p_lo; q0 <= p_hi; q0 += 8) {
    float4 a[8], b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int q = q0 + i;
      a[i] = b[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (q <= p_hi) {
        const float* src = sv.partial + (((size_t)q * 2 + (q == p_lo ? slot : 0)) * sv.mpad + t) * SPLIT_BN + col;
        a[i] = __ldcg(reinterpret_cast<const float4*>(src));
        b[i] = __ldcg(reinterpret_cast<const float4*>(src + 4));
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      out[0] += a[i].x; out[1] += a[i].y; out[2] += a[i].z; out[3] += a[i].w;
      out[4] += b[i].x; out[5] += b[i].y; out[6] += b[i].z; out[7] += b[i].w;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) out[j] = __bfloat162float(__float2bfloat16_rn(out[j]));
}
__device__ __forceinline__ void split_load8(const __nv_bfloat16* y_row, const SplitView& sv, int t, int n0, float (&out)[8]) {
  split_load8(y_row, sv, split_tile(sv, n0), t, n0, out);
}

}  // namespace tb
