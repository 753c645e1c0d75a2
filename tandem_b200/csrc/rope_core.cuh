// Per-head RMSNorm and rotary encoding of one q or k row in bfloat16, as the lanes of a head do it.
//
// A head of `hd` elements (a power of two, 16 to 256, all of it rotating) takes hd / 16 neighbouring
// lanes of a warp.  Lane `sub` holds a[0..8) = x[8 sub .. 8 sub + 8) of the lower half and
// b[0..8) = x[hd/2 + 8 sub ..) of the upper half: the eight pairs (a[i], b[i]) it rotates.
// Both the stand-alone kernel (tokenwise.cu) and decode attention (attention_decode.cu), which
// does the same to its own query rows and to the newest key, go through this function, so that
// they give the same bits.
//
// Formulas: 12vivi/tandem python/tandem/layers/ops.py:29-34,51-61 (norm in float32, rotate_half).
#pragma once

#include "common.cuh"

namespace tb {

__device__ __forceinline__ void unpack8(const uint4& raw, float (&out)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

// w: this lane's sixteen norm weights (w[i] for a[i], w[8 + i] for b[i]); `normed`: whether to normalise.
// cc, ssn: cos and sin of the lane's eight angles.  head_lanes: mask of the lanes of this lane's head.
__device__ __forceinline__ void norm_rope_pairs(float (&a)[8], float (&b)[8], const float (&w)[16], bool normed, const float (&cc)[8],
                                                const float (&ssn)[8], int hd, float eps, unsigned head_lanes, int lanes_per_head,
                                                uint4& lo_out, uint4& hi_out) {
  if (normed) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += a[i] * a[i] + b[i] * b[i];
    for (int o = lanes_per_head >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(head_lanes, ss, o);
    const float inv = rsqrtf(ss / (float)hd + eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) { a[i] = a[i] * inv * w[i]; b[i] = b[i] * inv * w[8 + i]; }
  }
  uint32_t lo[4], hi[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    lo[i] = pack2(a[2 * i] * cc[2 * i] - b[2 * i] * ssn[2 * i], a[2 * i + 1] * cc[2 * i + 1] - b[2 * i + 1] * ssn[2 * i + 1]);
    hi[i] = pack2(b[2 * i] * cc[2 * i] + a[2 * i] * ssn[2 * i], b[2 * i + 1] * cc[2 * i + 1] + a[2 * i + 1] * ssn[2 * i + 1]);
  }
  lo_out = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  hi_out = make_uint4(hi[0], hi[1], hi[2], hi[3]);
}

// cos and sin of a lane's eight angles from the table row of its position: [0, hd/2) cos, [hd/2, hd) sin.
__device__ __forceinline__ void load_angles(const float* row, int half, int j, float (&cc)[8], float (&ssn)[8]) {
  const float4 c0 = *reinterpret_cast<const float4*>(row + j), c1 = *reinterpret_cast<const float4*>(row + j + 4);
  const float4 s0 = *reinterpret_cast<const float4*>(row + half + j), s1 = *reinterpret_cast<const float4*>(row + half + j + 4);
  cc[0] = c0.x; cc[1] = c0.y; cc[2] = c0.z; cc[3] = c0.w; cc[4] = c1.x; cc[5] = c1.y; cc[6] = c1.z; cc[7] = c1.w;
  ssn[0] = s0.x; ssn[1] = s0.y; ssn[2] = s0.z; ssn[3] = s0.w; ssn[4] = s1.x; ssn[5] = s1.y; ssn[6] = s1.z; ssn[7] = s1.w;
}

}  // namespace tb
