// Per-token kernels: embedding gather, residual-add + RMSNorm, q/k-norm + rotary + cache write,
// SiLU-and-multiply.  All arithmetic is float32; T is the storage type of activations and caches.
//
// Formulas: 12vivi/tandem python/tandem/layers/ops.py:29-61 (norm, fused add+norm, silu_and_mul,
// rotate_half), python/tandem/layers/triton_ops.py:21-113 (the fused prologue and the fused
// add+norm, which add in float32 and round once, as these kernels do).
#include "cache_layout.cuh"
#include "common.cuh"
#include "rope_core.cuh"

namespace tb {

// ---------------------------------------------------------------------------------------------
// Embedding: out[t, :] = scale * float(table[ids[t], :]) (+ float(pos_table[positions[t], :]) where
// the model has a learned table of absolute positions).  The residual stream is float32 in both modes.
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int H, int V, float scale, const int* __restrict__ positions,
                                 const T* __restrict__ pos_table, int max_pos) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* o = out + (size_t)t * H;
  if (id < 0 || id >= V) {  // the host checks ids; never read outside the table
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * H;
  if (pos_table || scale != 1.f) {
    const T* prow = nullptr;
    if (pos_table) {
      int pos = positions[t];
      pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);  // the host checks positions
      prow = pos_table + (size_t)pos * H;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = scale * to_float(row[i]) + (prow ? to_float(prow[i]) : 0.f);
    return;
  }
  if (sizeof(T) == 2 && (H & 7) == 0) {  // 16 bytes in, two 16-byte stores out
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(row + i);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]), c = __bfloat1622float2(p[2]), d = __bfloat1622float2(p[3]);
      *reinterpret_cast<float4*>(o + i) = make_float4(a.x, a.y, b.x, b.y);
      *reinterpret_cast<float4*>(o + i + 4) = make_float4(c.x, c.y, d.x, d.y);
    }
    return;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]);
}

// ---------------------------------------------------------------------------------------------
// ids[i] = tokens[source[i]] where source[i] >= 0: token ids that the step before sampled and that
// have not travelled to the host yet go straight into this step's batch.  It stands where
// 12vivi/tandem gathers the in-flight step's tokens on the device
// (python/tandem/executor/model_runner.py:118-126).
__global__ void take_tokens_kernel(int* __restrict__ ids, const int* __restrict__ source, const int* __restrict__ tokens,
                                   int n, int num_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int s = source[i];
  if (s >= 0 && s < num_tokens) ids[i] = tokens[s];
}

// Eight neighbouring bfloat16 values (16-byte aligned) as floats.
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&out)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); out[2 * j] = f.x; out[2 * j + 1] = f.y; }
}

// ---------------------------------------------------------------------------------------------
// residual[src] += x[src] (if x); y[r] = residual[src] * rsqrt(mean(residual[src]^2) + eps) * w
// with src = rows ? rows[r] : r.  One block per output row.
template <typename T>
__global__ void add_rmsnorm_kernel(const T* __restrict__ x, float* __restrict__ residual,
                                   const float* __restrict__ weight, T* __restrict__ y,
                                   const int* __restrict__ rows, int H, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* res = residual + (size_t)src * H;
  const T* xr = x ? x + (size_t)src * H : nullptr;
  float ss = 0.f;
  if (sizeof(T) == 2 && (H & 7) == 0 && H <= (int)blockDim.x * 8) {  // one turn: the sums stay in registers
    const int i = threadIdx.x * 8;
    float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
    if (i < H) {
      s0 = *reinterpret_cast<const float4*>(res + i);
      s1 = *reinterpret_cast<const float4*>(res + i + 4);
      if (xr) {
        float v[8];
        load8(reinterpret_cast<const __nv_bfloat16*>(xr) + i, v);
        s0.x += v[0]; s0.y += v[1]; s0.z += v[2]; s0.w += v[3];
        s1.x += v[4]; s1.y += v[5]; s1.z += v[6]; s1.w += v[7];
        *reinterpret_cast<float4*>(res + i) = s0;
        *reinterpret_cast<float4*>(res + i + 4) = s1;
      }
      ss = s0.x * s0.x + s0.y * s0.y + s0.z * s0.z + s0.w * s0.w + s1.x * s1.x + s1.y * s1.y + s1.z * s1.z + s1.w * s1.w;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    if (i < H) {
      const float4 w0 = *reinterpret_cast<const float4*>(weight + i), w1 = *reinterpret_cast<const float4*>(weight + i + 4);
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(y) + (size_t)r * H + i) =
          make_uint4(pack2(s0.x * inv * w0.x, s0.y * inv * w0.y), pack2(s0.z * inv * w0.z, s0.w * inv * w0.w),
                     pack2(s1.x * inv * w1.x, s1.y * inv * w1.y), pack2(s1.z * inv * w1.z, s1.w * inv * w1.w));
    }
    return;
  }
  if (sizeof(T) == 2 && (H & 7) == 0) {  // eight elements per thread and turn: 16-byte loads and stores
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float4 s0 = *reinterpret_cast<const float4*>(res + i), s1 = *reinterpret_cast<const float4*>(res + i + 4);
      if (xr) {
        float v[8];
        load8(reinterpret_cast<const __nv_bfloat16*>(xr) + i, v);
        s0.x += v[0]; s0.y += v[1]; s0.z += v[2]; s0.w += v[3];
        s1.x += v[4]; s1.y += v[5]; s1.z += v[6]; s1.w += v[7];
        *reinterpret_cast<float4*>(res + i) = s0;
        *reinterpret_cast<float4*>(res + i + 4) = s1;
      }
      ss += s0.x * s0.x + s0.y * s0.y + s0.z * s0.z + s0.w * s0.w + s1.x * s1.x + s1.y * s1.y + s1.z * s1.z + s1.w * s1.w;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    __nv_bfloat16* yr = reinterpret_cast<__nv_bfloat16*>(y) + (size_t)r * H;
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {  // each thread re-reads only what it wrote itself
      const float4 s0 = *reinterpret_cast<const float4*>(res + i), s1 = *reinterpret_cast<const float4*>(res + i + 4);
      const float4 w0 = *reinterpret_cast<const float4*>(weight + i), w1 = *reinterpret_cast<const float4*>(weight + i + 4);
      *reinterpret_cast<uint4*>(yr + i) =
          make_uint4(pack2(s0.x * inv * w0.x, s0.y * inv * w0.y), pack2(s0.z * inv * w0.z, s0.w * inv * w0.w),
                     pack2(s1.x * inv * w1.x, s1.y * inv * w1.y), pack2(s1.z * inv * w1.z, s1.w * inv * w1.w));
    }
    return;
  }
  if ((H & 3) == 0) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 s = *reinterpret_cast<const float4*>(res + i);
      if (xr) {
        s.x += to_float(xr[i]); s.y += to_float(xr[i + 1]); s.z += to_float(xr[i + 2]); s.w += to_float(xr[i + 3]);
        *reinterpret_cast<float4*>(res + i) = s;
      }
      ss += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float s = res[i];
      if (xr) { s += to_float(xr[i]); res[i] = s; }
      ss += s * s;
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  T* yr = y + (size_t)r * H;
  // each thread re-reads only what it wrote itself above
  if ((H & 3) == 0) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      const float4 s = *reinterpret_cast<const float4*>(res + i);
      const float4 w = *reinterpret_cast<const float4*>(weight + i);
      yr[i] = from_float<T>(s.x * inv * w.x);
      yr[i + 1] = from_float<T>(s.y * inv * w.y);
      yr[i + 2] = from_float<T>(s.z * inv * w.z);
      yr[i + 3] = from_float<T>(s.w * inv * w.w);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) yr[i] = from_float<T>(res[i] * inv * weight[i]);
  }
}

// The same for many rows of bfloat16 whose width fits one turn of the block (H <= 8 * threads):
// a block takes two neighbouring rows and issues the loads of both before it uses any, so twice
// as many bytes are on their way per thread (the kernel is bound by memory latency: a row is
// loaded, reduced, stored).
__global__ void add_rmsnorm_rows2_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ residual,
                                         const float* __restrict__ weight, __nv_bfloat16* __restrict__ y, int num_rows, int H,
                                         float eps) {
  __shared__ float scratch[2][33];
  pdl_launch_dependents();
  const int i = threadIdx.x * 8;
  const bool on = i < H;
  float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f), w1 = w0;
  if (on) { w0 = *reinterpret_cast<const float4*>(weight + i); w1 = *reinterpret_cast<const float4*>(weight + i + 4); }  // written by no kernel
  pdl_wait();
  const int r0 = blockIdx.x * 2;
  float4 s[2][2];
  uint4 xv[2];
  bool have[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    have[k] = on && r0 + k < num_rows;
    s[k][0] = s[k][1] = make_float4(0.f, 0.f, 0.f, 0.f);
    xv[k] = make_uint4(0, 0, 0, 0);
    if (have[k]) {
      const float* res = residual + (size_t)(r0 + k) * H + i;
      s[k][0] = *reinterpret_cast<const float4*>(res);
      s[k][1] = *reinterpret_cast<const float4*>(res + 4);
      if (x) xv[k] = *reinterpret_cast<const uint4*>(x + (size_t)(r0 + k) * H + i);
    }
  }
  float ss[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    if (x && have[k]) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&xv[k]);
      const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]), c = __bfloat1622float2(h[2]), d = __bfloat1622float2(h[3]);
      s[k][0].x += a.x; s[k][0].y += a.y; s[k][0].z += b.x; s[k][0].w += b.y;
      s[k][1].x += c.x; s[k][1].y += c.y; s[k][1].z += d.x; s[k][1].w += d.y;
      float* res = residual + (size_t)(r0 + k) * H + i;
      *reinterpret_cast<float4*>(res) = s[k][0];
      *reinterpret_cast<float4*>(res + 4) = s[k][1];
    }
    ss[k] = s[k][0].x * s[k][0].x + s[k][0].y * s[k][0].y + s[k][0].z * s[k][0].z + s[k][0].w * s[k][0].w +
            s[k][1].x * s[k][1].x + s[k][1].y * s[k][1].y + s[k][1].z * s[k][1].z + s[k][1].w * s[k][1].w;
  }
  ss[0] = block_sum(ss[0], scratch[0]);
  ss[1] = block_sum(ss[1], scratch[1]);
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    if (!have[k]) continue;
    const float inv = rsqrtf(ss[k] / (float)H + eps);
    *reinterpret_cast<uint4*>(y + (size_t)(r0 + k) * H + i) =
        make_uint4(pack2(s[k][0].x * inv * w0.x, s[k][0].y * inv * w0.y), pack2(s[k][0].z * inv * w0.z, s[k][0].w * inv * w0.w),
                   pack2(s[k][1].x * inv * w1.x, s[k][1].y * inv * w1.y), pack2(s[k][1].z * inv * w1.z, s[k][1].w * inv * w1.w));
  }
}

// ---------------------------------------------------------------------------------------------
// One warp per (token, head) of the fused projection qkv [T, (nh + 2 nkv) * hd]:
//   q heads: optional RMSNorm over hd, rotary, written back in place;
//   k heads: optional RMSNorm, rotary, written to the key cache at the token's slot;
//   v heads: copied to the value cache.
// Cache tiles [page][kv head] of page_size x hd elements laid out as cache_layout.cuh says;
// slot = page * page_size + offset; a negative slot (padding row) or write_kv == 0 (the run reads
// another run's cache) writes nothing.
// Rotary: pairs (j, j + rd/2), j < rd/2, angle table cs[pos][0..rd/2) = cos, [rd/2..rd) = sin.
template <typename T>
__global__ void qk_norm_rope_kv_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                       const int* __restrict__ slots, const float* __restrict__ q_w,
                                       const float* __restrict__ k_w, const float* __restrict__ cos_sin,
                                       T* __restrict__ k_cache, T* __restrict__ v_cache, int T_tokens, int nh,
                                       int nkv, int hd, int rd, int page_size, float eps, int write_kv,
                                       int max_pos) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int heads = nh + 2 * nkv;
  const long long g = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (g >= (long long)T_tokens * heads) return;
  const int t = (int)(g / heads), h = (int)(g % heads);
  T* x = qkv + (size_t)t * heads * hd + (size_t)h * hd;
  const int slot = slots ? slots[t] : -1;
  const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
  if (!is_q && (slot < 0 || !write_kv)) return;
  T* dst = x;   // q: in place.  k, v: the tile of (page, kv head); `row` is the token's row in it
  int row = -1;
  if (!is_q) {
    const int kvh = is_k ? h - nh : h - nh - nkv;
    row = slot % page_size;
    dst = (is_k ? k_cache : v_cache) + cache_tile(slot / page_size, kvh, nkv, page_size, hd);
  }
  auto at = [&](int d) { return row < 0 ? d : cache_offset<T>(row, d, page_size, hd); };
  if (!is_q && !is_k) {  // v: plain copy
    if (sizeof(T) == 2) {
      for (int d = lane * 2; d < hd; d += 64) *reinterpret_cast<uint32_t*>(dst + at(d)) = *reinterpret_cast<const uint32_t*>(x + d);
    } else {
      for (int d = lane; d < hd; d += 32) dst[at(d)] = x[d];
    }
    return;
  }
  const float* w = is_q ? q_w : k_w;
  float inv = 1.f;
  if (w) {
    float ss = 0.f;
    for (int d = lane; d < hd; d += 32) { const float v = to_float(x[d]); ss += v * v; }
    ss = warp_sum(ss);
    inv = rsqrtf(ss / (float)hd + eps);
  }
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);  // the host checks positions
  const int half = rd >> 1;
  const float* cs = cos_sin + (size_t)pos * rd;
  if (sizeof(T) == 2 && (half & 1) == 0) {  // two neighbouring pairs per lane: 4-byte loads and stores
    for (int j = lane * 2; j < half; j += 64) {
      const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + j));
      const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + j + half));
      float a0 = lo.x * inv, a1 = lo.y * inv, b0 = hi.x * inv, b1 = hi.y * inv;
      if (w) { a0 *= w[j]; a1 *= w[j + 1]; b0 *= w[j + half]; b1 *= w[j + half + 1]; }
      const float2 c = *reinterpret_cast<const float2*>(cs + j), sn = *reinterpret_cast<const float2*>(cs + half + j);
      *reinterpret_cast<__nv_bfloat162*>(dst + at(j)) = __floats2bfloat162_rn(a0 * c.x - b0 * sn.x, a1 * c.y - b1 * sn.y);
      *reinterpret_cast<__nv_bfloat162*>(dst + at(j + half)) = __floats2bfloat162_rn(b0 * c.x + a0 * sn.x, b1 * c.y + a1 * sn.y);
    }
    for (int d = rd + lane; d < hd; d += 32) {
      float a = to_float(x[d]) * inv;
      if (w) a *= w[d];
      dst[at(d)] = from_float<T>(a);
    }
    return;
  }
  for (int j = lane; j < half; j += 32) {
    float a = to_float(x[j]) * inv, b = to_float(x[j + half]) * inv;
    if (w) { a *= w[j]; b *= w[j + half]; }
    const float c = cs[j], s = cs[half + j];
    dst[at(j)] = from_float<T>(a * c - b * s);
    dst[at(j + half)] = from_float<T>(b * c + a * s);
  }
  for (int d = rd + lane; d < hd; d += 32) {  // dims beyond the rotary part pass through
    float a = to_float(x[d]) * inv;
    if (w) a *= w[d];
    dst[at(d)] = from_float<T>(a);
  }
}

// The same for bfloat16 when the whole head rotates (rd == hd) and hd is a power of two from 16 to
// 256: a head takes hd / 16 lanes, each with eight neighbouring elements of the lower half and the
// eight they pair with in the upper half (16-byte loads and stores), so a warp does 512 / hd heads
// at a time; a block of four warps does `heads_per_block` heads of one token, and every lane loads
// its sixteen angles once for all of them.
__global__ void qk_norm_rope_kv_bf16_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                            const int* __restrict__ slots, const float* __restrict__ q_w,
                                            const float* __restrict__ k_w, const float* __restrict__ cos_sin,
                                            __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                            int nh, int nkv, int hd, int page_size, float eps, int write_kv, int max_pos,
                                            int heads_per_block) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int heads = nh + 2 * nkv, half = hd >> 1;
  const int lanes_per_head = hd >> 4, heads_per_warp = 32 / lanes_per_head;
  const int sub = lane % lanes_per_head, j = sub * 8;  // elements j..j+7 and half+j..half+j+7
  // the lanes of this lane's head: they take every branch below together, other heads of the warp may not
  const unsigned head_lanes = (lanes_per_head == 32 ? 0xffffffffu : ((1u << lanes_per_head) - 1u)) << (lane - sub);
  const int t = blockIdx.x, h_begin = blockIdx.y * heads_per_block, h_end = min(heads, h_begin + heads_per_block);
  float wq[16], wk[16];
#pragma unroll
  for (int i = 0; i < 8; ++i) {  // norm weights are written by no kernel
    wq[i] = q_w ? q_w[j + i] : 1.f; wq[8 + i] = q_w ? q_w[half + j + i] : 1.f;
    wk[i] = k_w ? k_w[j + i] : 1.f; wk[8 + i] = k_w ? k_w[half + j + i] : 1.f;
  }
  pdl_wait();
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);  // the host checks positions
  float cc[8], ssn[8];
  load_angles(cos_sin + (size_t)pos * hd, half, j, cc, ssn);
  const int slot = slots ? slots[t] : -1;
  __nv_bfloat16* row = qkv + (size_t)t * heads * hd;
  for (int h = h_begin + warp * heads_per_warp + lane / lanes_per_head; h < h_end; h += 4 * heads_per_warp) {
    const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
    if (!is_q && (slot < 0 || !write_kv)) continue;
    __nv_bfloat16* x = row + (size_t)h * hd;
    const uint4 lo_raw = *reinterpret_cast<const uint4*>(x + j), hi_raw = *reinterpret_cast<const uint4*>(x + half + j);
    __nv_bfloat16* dst = x;
    int at_lo = j, at_hi = half + j;
    if (!is_q) {
      const int kvh = is_k ? h - nh : h - nh - nkv, r = slot % page_size;
      dst = (is_k ? k_cache : v_cache) + cache_tile(slot / page_size, kvh, nkv, page_size, hd);
      at_lo = cache_offset<__nv_bfloat16>(r, j, page_size, hd);
      at_hi = cache_offset<__nv_bfloat16>(r, half + j, page_size, hd);
    }
    if (!is_q && !is_k) {  // v: plain copy
      *reinterpret_cast<uint4*>(dst + at_lo) = lo_raw;
      *reinterpret_cast<uint4*>(dst + at_hi) = hi_raw;
      continue;
    }
    float a[8], b[8];
    unpack8(lo_raw, a);
    unpack8(hi_raw, b);
    uint4 lo_out, hi_out;
    norm_rope_pairs(a, b, is_q ? wq : wk, is_q ? q_w != nullptr : k_w != nullptr, cc, ssn, hd, eps, head_lanes, lanes_per_head, lo_out, hi_out);
    *reinterpret_cast<uint4*>(dst + at_lo) = lo_out;
    *reinterpret_cast<uint4*>(dst + at_hi) = hi_out;
  }
}

// ---------------------------------------------------------------------------------------------
// out[t, i] = silu(gu[t, i]) * gu[t, I + i]
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long long total, int I) {
  pdl_launch_dependents();
  pdl_wait();
  if (sizeof(T) == 2 && (I & 7) == 0) {  // two groups of eight per thread and turn, four loads in flight
    const long long groups = total / 8, stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < groups; e += 2 * stride) {
      uint4 g4[2], u4[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const long long ek = e + k * stride;
        g4[k] = u4[k] = make_uint4(0, 0, 0, 0);
        if (ek < groups) {
          const long long t = (ek * 8) / I;
          const int i = (int)((ek * 8) % I);
          const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(gu) + t * 2 * I;
          g4[k] = *reinterpret_cast<const uint4*>(row + i);
          u4[k] = *reinterpret_cast<const uint4*>(row + I + i);
        }
      }
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const long long ek = e + k * stride;
        if (ek >= groups) continue;
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4[k]);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4[k]);
        uint4 r;
        uint32_t* r2 = reinterpret_cast<uint32_t*>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
          // the result is rounded to bfloat16: the fast exponential and division are exact enough by far
          r2[j] = pack2(__fdividef(g.x, 1.f + __expf(-g.x)) * u.x, __fdividef(g.y, 1.f + __expf(-g.y)) * u.y);
        }
        *reinterpret_cast<uint4*>(out + ek * 8) = r;
      }
    }
    return;
  }
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    const long long t = e / I;
    const int i = (int)(e % I);
    const float g = to_float(gu[t * 2 * I + i]);
    const float u = to_float(gu[t * 2 * I + I + i]);
    out[e] = from_float<T>(g / (1.f + expf(-g)) * u);
  }
}

// ---------------------------------------------------------------------------------------------
// Output-head hooks of architectures that scale or cap their logits: x <- scale * x, then
// x <- cap * tanh(x / cap) where cap > 0.
__global__ void scale_softcap_kernel(float* __restrict__ x, long long n, float scale, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v = x[i] * scale;
    if (cap > 0.f) v = cap * tanhf(v / cap);
    x[i] = v;
  }
}

}  // namespace tb

extern "C" {

// positions / pos_table [max_pos, H] may be null (no learned absolute positions).
int tb_embedding(void* stream, const int* ids, const void* table, float* out, int T_tokens, int H, int V,
                 int dtype, float scale, const int* positions, const void* pos_table, int max_pos) {
  if (T_tokens <= 0) return 0;
  if (pos_table && (!positions || max_pos <= 0)) return TB_ERR_BAD_SIZE;
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::embedding_kernel<T>, dim3(T_tokens), dim3(256), 0, stream, ids, (const T*)table, out, H, V,
                                      scale, positions, (const T*)pos_table, max_pos));
}

// logits = scale * logits, then cap * tanh(logits / cap) where cap > 0 (in place, float32).
int tb_scale_softcap(void* stream, float* logits, long long n, float scale, float cap) {
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return tb::launch(tb::scale_softcap_kernel, dim3((int)blocks), dim3(256), 0, stream, logits, n, scale, cap);
}

int tb_take_tokens(void* stream, int* ids, const int* source, const int* tokens, int n, int num_tokens) {
  if (n <= 0) return 0;
  return tb::launch(tb::take_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, ids, source, tokens, n, num_tokens);
}

int tb_add_rmsnorm(void* stream, const void* x, float* residual, const float* weight, void* y, const int* rows,
                   int num_rows, int H, float eps, int dtype) {
  if (num_rows <= 0) return 0;
  const int threads = H >= 4096 ? 512 : 256;
  if (dtype == TB_BF16 && !rows && num_rows >= 512 && (H & 7) == 0 && H <= threads * 8)
    return tb::launch(tb::add_rmsnorm_rows2_kernel, dim3((num_rows + 1) / 2), dim3(threads), 0, stream, (const __nv_bfloat16*)x,
                      residual, weight, (__nv_bfloat16*)y, num_rows, H, eps);
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::add_rmsnorm_kernel<T>, dim3(num_rows), dim3(threads), 0, stream, (const T*)x, residual,
                                      weight, (T*)y, rows, H, eps));
}

int tb_qk_norm_rope_kv(void* stream, void* qkv, const int* positions, const int* slots, const float* q_w,
                       const float* k_w, const float* cos_sin, void* k_cache, void* v_cache, int T_tokens, int nh,
                       int nkv, int hd, int rd, int page_size, float eps, int write_kv, int max_pos, int dtype) {
  if (T_tokens <= 0) return 0;
  if (rd < 0 || rd > hd || (rd & 1) || page_size <= 0) return TB_ERR_BAD_SIZE;
  const bool pow2 = hd >= 16 && hd <= 256 && (hd & (hd - 1)) == 0;
  if (dtype == TB_BF16 && rd == hd && pow2 && T_tokens <= 65535 * 32) {
    const int heads = nh + 2 * nkv, per_warp = 512 / hd;
    // few tokens: spread a token's heads over several blocks; many: one block keeps its angles for 8 x more heads
    const int heads_per_block = T_tokens >= 256 ? 8 * 4 * per_warp : 4 * per_warp;
    dim3 grid(T_tokens, (heads + heads_per_block - 1) / heads_per_block);
    return tb::launch(tb::qk_norm_rope_kv_bf16_kernel, grid, dim3(128), 0, stream, (__nv_bfloat16*)qkv, positions, slots, q_w, k_w,
                      cos_sin, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nh, nkv, hd, page_size, eps, write_kv, max_pos,
                      heads_per_block);
  }
  const long long warps = (long long)T_tokens * (nh + 2 * nkv);
  const int blocks = (int)((warps + 3) / 4);
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::qk_norm_rope_kv_kernel<T>, dim3(blocks), dim3(128), 0, stream, (T*)qkv, positions, slots,
                                      q_w, k_w, cos_sin, (T*)k_cache, (T*)v_cache, T_tokens, nh, nkv, hd, rd, page_size, eps,
                                      write_kv, max_pos));
}

int tb_silu_mul(void* stream, const void* gu, void* out, int T_tokens, int I, int dtype) {
  const long long total = (long long)T_tokens * I;
  if (total <= 0) return 0;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::silu_mul_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (const T*)gu, (T*)out, total, I));
}

}  // extern "C"
