// Sampling over logits [R, V] float32: argmax, and temperature sampling with the top-k, top-p and
// min-p filters of 12vivi/tandem (python/tandem/layers/sampler.py:19-64), one thread block per row.
//
// Where tandem sorts the row, these kernels find the same cut by bisection on the bit pattern of
// the values (non-negative floats and their order-preserving keys compare like unsigned
// integers), 32 counting passes over a row that stays in L2.  Where tandem draws with
// torch.multinomial, the draw here is the inverse CDF in vocabulary order at u * total for a
// uniform number u that the caller supplies per row, so a draw is a pure function of
// (logits, options, u).  Tokens whose value equals the cut are all kept (a sort keeps as many
// of them as fit); the outcomes differ only for exact ties at the cut.
//
// The filtered probabilities of a row are built in `probs` [R, V], scratch memory that the caller
// provides.
#include "argmax_static.h"
#include "common.cuh"

namespace tb {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ unsigned ordered_key(float x) {  // monotone map float -> unsigned
  const unsigned b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ int block_sum_int(int v, int* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int t = lane < nwarps ? scratch[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Index of the largest value, the lowest index among equals.
__device__ int row_argmax(const float* __restrict__ x, int V, float* fscratch, int* iscratch) {
  float best = -INFINITY;
  int best_i = V;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = x[i];
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
  const float top = block_max(best, fscratch);
  int cand = (best == top) ? best_i : V;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) iscratch[warp] = cand;
  __syncthreads();
  if (warp == 0) {
    int t = lane < nwarps ? iscratch[lane] : V;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = min(t, __shfl_xor_sync(0xffffffffu, t, o));
    if (lane == 0) iscratch[32] = t;
  }
  __syncthreads();
  return min(iscratch[32], V - 1);
}

__global__ void __launch_bounds__(SAMPLE_THREADS) argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V) {
  __shared__ float fs[33];
  __shared__ int is[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int idx = row_argmax(logits + (size_t)r * V, V, fs, is);
  if (threadIdx.x == 0) out[r] = idx;
}

// Argmax of long rows with many blocks per row: every block folds its chunk into one 64-bit word
// (ordered key of the value above, inverted index below, so the largest word is the largest value
// at its lowest index), merges it into best[row] with atomicMax, and the block that arrives last
// writes the index and puts best[row] and arrivals[row] back to zero for the next launch.
__global__ void __launch_bounds__(256)
argmax_split_kernel(const float* __restrict__ logits, int* __restrict__ out, unsigned long long* __restrict__ best,
                    int* __restrict__ arrivals, int V, int chunks) {
  __shared__ unsigned long long warp_best[8];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.y, len = (V + chunks - 1) / chunks;
  const int begin = blockIdx.x * len, end = min(V, begin + len);
  const float* x = logits + (size_t)r * V;
  unsigned long long mine = 0ull;
  for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const unsigned long long cand = ((unsigned long long)ordered_key(x[i]) << 32) | (0xFFFFFFFFu - (unsigned)i);
    mine = cand > mine ? cand : mine;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, mine, o);
    mine = other > mine ? other : mine;
  }
  if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) mine = warp_best[w] > mine ? warp_best[w] : mine;
    if (mine) atomicMax(best + r, mine);
    __threadfence();
    if (atomicAdd(arrivals + r, 1) == chunks - 1) {
      __threadfence();
      const unsigned long long top = atomicExch(best + r, 0ull);
      out[r] = (int)(0xFFFFFFFFu - (unsigned)(top & 0xFFFFFFFFull));
      arrivals[r] = 0;
    }
  }
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p, const float* __restrict__ uniform,
              float* __restrict__ probs, int* __restrict__ out, int V) {
  __shared__ float fs[33];
  __shared__ int is[33];
  __shared__ float prefix[SAMPLE_THREADS];
  __shared__ int chosen;
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* x = logits + (size_t)r * V;
  float* p = probs + (size_t)r * V;
  const float temp = temperature[r];
  if (temp < 1e-5f) {  // greedy row (sampling_params.py:35-37)
    const int idx = row_argmax(x, V, fs, is);
    if (tid == 0) out[r] = idx;
    return;
  }
  const float inv_t = 1.f / fmaxf(temp, 1e-5f);

  // 1) scaled maximum
  float mx = -INFINITY;
  for (int i = tid; i < V; i += blockDim.x) mx = fmaxf(mx, x[i] * inv_t);
  mx = block_max(mx, fs);

  // 2) top-k: the k-th largest scaled logit, by bisection on the ordered keys
  unsigned kth_key = 0;
  const int k = top_k[r];
  if (k > 0 && k < V) {
    for (int b = 31; b >= 0; --b) {
      const unsigned cand = kth_key | (1u << b);
      int c = 0;
      for (int i = tid; i < V; i += blockDim.x) c += ordered_key(x[i] * inv_t) >= cand;
      if (block_sum_int(c, is) >= k) kth_key = cand;
    }
  }

  // 3) probabilities of the kept tokens
  float z = 0.f;
  for (int i = tid; i < V; i += blockDim.x) {
    const float s = x[i] * inv_t;
    const float e = ordered_key(s) >= kth_key ? expf(s - mx) : 0.f;
    p[i] = e;
    z += e;
  }
  z = block_sum(z, fs);
  const float inv_z = 1.f / z;
  for (int i = tid; i < V; i += blockDim.x) p[i] *= inv_z;  // each thread rewrites its own elements

  // 4) top-p: keep a token iff the mass of strictly larger probabilities is <= top_p
  unsigned cut = 0;  // keep probabilities whose bits are >= cut
  const float tp = top_p[r];
  if (tp < 1.f) {
    unsigned below = 0;  // the largest bit pattern t with mass(p > t) > top_p; t = 0 qualifies
    for (int b = 30; b >= 0; --b) {  // probabilities are non-negative: the sign bit is never set
      const unsigned cand = below | (1u << b);
      float mass = 0.f;
      for (int i = tid; i < V; i += blockDim.x) mass += __float_as_uint(p[i]) > cand ? p[i] : 0.f;
      if (block_sum(mass, fs) > tp) below = cand;
    }
    cut = below + 1;
  }

  // 5) min-p relative to the largest probability (always kept: it is exp(0) / z)
  const float mp = min_p[r];
  const float floor_p = mp > 0.f ? mp * inv_z : 0.f;

  // 6) inverse CDF in vocabulary order: thread t owns the contiguous chunk [t*chunk, (t+1)*chunk)
  __syncthreads();  // the chunks below were written by other threads above
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int begin = min(V, tid * chunk), end = min(V, begin + chunk);
  float mine = 0.f;
  for (int i = begin; i < end; ++i) {
    float v = p[i];
    if (__float_as_uint(v) < cut || v < floor_p) v = 0.f;
    p[i] = v;
    mine += v;
  }
  __syncthreads();
  prefix[tid] = mine;
  __syncthreads();
  for (int o = 1; o < SAMPLE_THREADS; o <<= 1) {  // inclusive scan over the thread sums
    const float add = tid >= o ? prefix[tid - o] : 0.f;
    __syncthreads();
    prefix[tid] += add;
    __syncthreads();
  }
  const float total = prefix[SAMPLE_THREADS - 1];
  const float target = uniform[r] * total;
  if (tid == 0) chosen = V;
  __syncthreads();
  const float before = tid > 0 ? prefix[tid - 1] : 0.f;  // the intervals of the threads tile [0, total)
  if (mine > 0.f && before <= target && target < prefix[tid]) {
    float c = before;
    int pick = -1, last = -1;
    for (int i = begin; i < end; ++i) {
      if (p[i] > 0.f) {
        last = i;
        c += p[i];
        if (c > target) { pick = i; break; }
      }
    }
    atomicMin(&chosen, pick >= 0 ? pick : last);
  }
  __syncthreads();
  if (chosen == V) {  // rounding pushed the target past the end: the last kept token
    int last = -1;
    for (int i = begin; i < end; ++i) if (p[i] > 0.f) last = i;
    int m = last;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & 31) == 0) is[tid >> 5] = m;
    __syncthreads();
    if (tid == 0) {
      int best = 0;
      for (int w = 0; w < SAMPLE_THREADS / 32; ++w) best = max(best, is[w]);
      chosen = best;
    }
    __syncthreads();
  }
  if (tid == 0) out[r] = chosen;
}

}  // namespace tb

extern "C" {

int tb_argmax(void* stream, const float* logits, int* out, int R, int V) {
  if (R <= 0) return 0;
  if (V <= 0) return TB_ERR_BAD_SIZE;
  return tb::launch(tb::argmax_kernel, dim3(R), dim3(tb::SAMPLE_THREADS), 0, stream, logits, out, V);
}

// The same result with `chunks` blocks per row; best [R] (64-bit) and arrivals [R] are scratch that
// is zero before the call and zero again after it.
int tb_argmax_split(void* stream, const float* logits, int* out, void* best, int* arrivals, int R, int V,
                    int chunks) {
  if (R <= 0) return 0;
  if (V <= 0 || chunks <= 0 || R > 65535) return TB_ERR_BAD_SIZE;
  return tb::launch(tb::argmax_split_kernel, dim3(chunks, R), dim3(256), 0, stream, logits, out, (unsigned long long*)best,
                    arrivals, V, chunks);
}

int tb_sample(void* stream, const float* logits, const float* temperature, const int* top_k, const float* top_p,
              const float* min_p, const float* uniform, float* probs_scratch, int* out, int R, int V) {
  if (R <= 0) return 0;
  if (V <= 0) return TB_ERR_BAD_SIZE;
  return tb::launch(tb::sample_kernel, dim3(R), dim3(tb::SAMPLE_THREADS), 0, stream, logits, temperature, top_k, top_p, min_p,
                    uniform, probs_scratch, out, V);
}

// ---------------------------------------------------------------------------------------------
// The variant of tb_argmax_split whose scratch lives in this library (argmax_static.h).
// Layout of the array: best[MAX_ROWS] (64-bit words), then arrivals[MAX_ROWS] (32-bit).
static __device__ __align__(256) unsigned char tb_argmax_static_scratch[TB_ARGMAX_STATIC_MAX_ROWS * 16];

int tb_argmax_static(void* stream, const float* logits, int* out, int R, int V, int chunks) {
  if (R <= 0) return 0;
  if (V <= 0 || chunks <= 0) return TB_ERR_BAD_SIZE;
  if (R > TB_ARGMAX_STATIC_MAX_ROWS) return TB_ERR_TOO_LARGE;
  // In host code the array's name is only a handle: the kernel needs its device address, which
  // differs from device to device.  Looked up once per device, with that device current.
  static unsigned char* address[64] = {};
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= 64) return TB_ERR_BAD_SIZE;
  if (address[device] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, tb_argmax_static_scratch);
    if (e != cudaSuccess) return (int)e;
    address[device] = static_cast<unsigned char*>(p);
  }
  unsigned char* scratch = address[device];
  // best and arrivals must be zero when the kernel starts; the kernel also leaves them zero, but a
  // call does not rely on how the one before it ended
  e = cudaMemsetAsync(scratch, 0, (size_t)R * 8, (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemsetAsync(scratch + (size_t)TB_ARGMAX_STATIC_MAX_ROWS * 8, 0, (size_t)R * 4, (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  tb::argmax_split_kernel<<<dim3(chunks, R), 256, 0, (cudaStream_t)stream>>>(
      logits, out, reinterpret_cast<unsigned long long*>(scratch),
      reinterpret_cast<int*>(scratch + (size_t)TB_ARGMAX_STATIC_MAX_ROWS * 8), V, chunks);
  return tb::launch_status();
}

}  // extern "C"
