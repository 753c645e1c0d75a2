// Paged causal attention on the CUDA cores, for any head size and either storage type: the
// attention of the 32-bit path, and the fallback of the bfloat16 path for shapes its tensor-core
// kernels refuse.  One warp per (token, query head); scores, running maximum and sum, and the
// output accumulator are float32; keys are visited in ascending order in chunks of 32, so a
// token's result does not depend on the batch it is in, bit for bit.
//
// A query at position p of its request sees keys max(0, p - window + 1) .. p (window 0: all of
// 0 .. p), read from the request's pages: key j lives in page table[j / page_size] at offset
// j % page_size, tiles laid out as cache_layout.cuh says.  Query head h reads kv head
// h / (nh / nkv).  Formula: 12vivi/tandem python/tandem/layers/attention.py:46-56,
// python/tandem/executor/forward_context.py:70-74; online softmax as in
// python/tandem/layers/triton_decode_attn.py:52-76 (with exp, not exp2).
#include "cache_layout.cuh"
#include "common.cuh"

namespace tb {

constexpr int MAX_HD = 512;
constexpr int WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                      const T* __restrict__ v_cache, const int* __restrict__ block_table, int table_stride,
                      const int* __restrict__ seq_of_token, const int* __restrict__ positions, T* __restrict__ out,
                      int T_tokens, int nh, int nkv, int hd, int page_size, int window, float scale) {
  extern __shared__ float smem[];  // WARPS * hd floats: the scaled query of each warp
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long g = (long long)blockIdx.x * WARPS + warp;
  if (g >= (long long)T_tokens * nh) return;
  const int t = (int)(g / nh), h = (int)(g % nh);
  const int kvh = h / (nh / nkv);
  const int pos = positions[t];
  const int* table = block_table + (size_t)seq_of_token[t] * table_stride;
  float* qs = smem + warp * hd;
  const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
  for (int d = lane; d < hd; d += 32) qs[d] = to_float(qrow[d]) * scale;
  __syncwarp();

  constexpr int MAX_OWN = MAX_HD / 32;  // dims d = lane + 32 * i owned by this lane
  float acc[MAX_OWN];
#pragma unroll
  for (int i = 0; i < MAX_OWN; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;

  for (int base = lo; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key <= pos;
    long long row = -1;  // element offset of the (page, kv head) tile of this lane's key, and its row in it
    int r_in = 0;
    float s = -INFINITY;
    if (valid) {
      const int page = table[key / page_size];
      if (page >= 0) {
        row = cache_tile(page, kvh, nkv, page_size, hd);
        r_in = key % page_size;
        const T* kr = k_cache + row;
        float dot = 0.f;
        for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], to_float(kr[cache_offset<T>(r_in, d, page_size, hd)]), dot);
        s = dot;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float p = (row >= 0) ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < MAX_OWN; ++i) acc[i] *= corr;
    const int count = min(32, pos - base + 1);
    for (int j = 0; j < count; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const long long rj = __shfl_sync(0xffffffffu, row, j);
      const int rin = __shfl_sync(0xffffffffu, r_in, j);
      if (rj < 0) continue;  // uniform across the warp
      const T* vr = v_cache + rj;
#pragma unroll
      for (int i = 0; i < MAX_OWN; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pj, to_float(vr[cache_offset<T>(rin, d, page_size, hd)]), acc[i]);
      }
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T* orow = out + (size_t)t * nh * hd + (size_t)h * hd;
#pragma unroll
  for (int i = 0; i < MAX_OWN; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) orow[d] = from_float<T>(acc[i] * inv);
  }
}

}  // namespace tb

extern "C" int tb_attention_simt(void* stream, const void* q, int q_stride, const void* k_cache,
                                 const void* v_cache, const int* block_table, int table_stride,
                                 const int* seq_of_token, const int* positions, void* out, int T_tokens, int nh,
                                 int nkv, int hd, int page_size, int window, float scale, int dtype) {
  if (T_tokens <= 0) return 0;
  if (hd <= 0 || hd > tb::MAX_HD || nkv <= 0 || nh % nkv != 0 || page_size <= 0) return TB_ERR_BAD_SIZE;
  const long long warps = (long long)T_tokens * nh;
  const int blocks = (int)((warps + tb::WARPS - 1) / tb::WARPS);
  const size_t smem = (size_t)tb::WARPS * hd * sizeof(float);
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::attention_simt_kernel<T>, dim3(blocks), dim3(tb::WARPS * 32), smem, stream, (const T*)q,
                                      q_stride, (const T*)k_cache, (const T*)v_cache, block_table, table_stride, seq_of_token,
                                      positions, (T*)out, T_tokens, nh, nkv, hd, page_size, window, scale));
}
