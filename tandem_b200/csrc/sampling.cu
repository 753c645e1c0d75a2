// Sampling over logits [R, V] float32: argmax, and temperature sampling with the top-k, top-p and
// min-p filters of 12vivi/tandem (python/tandem/layers/sampler.py:19-64).
//
// Where tandem sorts the row, these kernels find the same cut by radix selection on the bit
// pattern of the values (non-negative floats and their order-preserving keys compare like
// unsigned integers), eight bits a pass: a pass builds a histogram of the next digit among the
// values that share the digits found so far, counts for top-k and probability mass for top-p (in
// 52-bit fixed point, so that the sums are integers and do not depend on the order of the atomic
// additions), and the next pass reads off the digit.  A row is cut into chunks that many blocks
// work on at once (a row of 150,000 logits is more than one SM should walk a dozen times), one
// small launch per pass; sums that stay floating point (the normaliser, the kept mass per chunk)
// are taken per chunk and added in chunk order.  Where tandem draws with torch.multinomial, the
// draw here is the inverse CDF in vocabulary order at u * total for a uniform number u that the
// caller supplies per row, so a draw is a pure function of (logits, options, u).  Tokens whose
// value equals the cut are all kept (a sort keeps as many of them as fit); the outcomes differ only
// for exact ties at the cut.
//
// Scratch per row (zero before the first pass): see RowScratch.
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
  const int r = blockIdx.y, len = ((V + chunks - 1) / chunks + 3) & ~3;  // chunks start on 16-byte boundaries of the row
  const int begin = min(V, (int)blockIdx.x * len), end = min(V, begin + len);
  const float* x = logits + (size_t)r * V;
  unsigned long long mine = 0ull;
  auto take = [&](float v, int i) {
    const unsigned long long cand = ((unsigned long long)ordered_key(v) << 32) | (0xFFFFFFFFu - (unsigned)i);
    mine = cand > mine ? cand : mine;
  };
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {  // four logits a load, two loads in flight
    const int quads = (end - begin) >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x + begin);
    int q = threadIdx.x;
    for (; q + (int)blockDim.x < quads; q += 2 * blockDim.x) {
      const float4 a = x4[q], b = x4[q + blockDim.x];
      const int ia = begin + 4 * q, ib = ia + 4 * blockDim.x;
      take(a.x, ia), take(a.y, ia + 1), take(a.z, ia + 2), take(a.w, ia + 3);
      take(b.x, ib), take(b.y, ib + 1), take(b.z, ib + 2), take(b.w, ib + 3);
    }
    if (q < quads) {
      const float4 a = x4[q];
      const int ia = begin + 4 * q;
      take(a.x, ia), take(a.y, ia + 1), take(a.z, ia + 2), take(a.w, ia + 3);
    }
    for (int i = begin + 4 * quads + threadIdx.x; i < end; i += blockDim.x) take(x[i], i);
  } else {
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) take(x[i], i);
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

// ------------------------------------------------------------------------------------------------
// Temperature sampling, many blocks per row.
constexpr int SP_THREADS = 256;
constexpr int SP_MAX_CHUNKS = 64;
constexpr int SP_FIXED_BITS = 52;  // probability mass as an integer multiple of 2^-52

struct RowScratch {
  unsigned long long best;             // argmax word: ordered key above, inverted index below
  unsigned long long mass[4][256];     // top-p passes: mass per digit
  int count[4][256];                   // top-k passes: tokens per digit
  float z_part[SP_MAX_CHUNKS];         // normaliser per chunk
  float kept_part[SP_MAX_CHUNKS];      // kept mass per chunk
  // what the passes have found, by number of digits known (written by block 0 of the pass that works it out)
  unsigned long long p_above[5];       // top-p: mass above the digits found
  unsigned p_prefix[5];                // top-p: digits of the cut
  unsigned k_prefix[5];                // top-k: digits of the k-th largest key
  int k_left[5];                       // top-k: how many of the k lie among the keys that share those digits
  int pad;
};

struct SampleArgs {
  const float* logits;
  const float* temperature;
  const int* top_k;
  const float* top_p;
  const float* min_p;
  const float* uniform;
  RowScratch* scratch;
  int* out;
  int V, chunks;
};

// What every pass needs of a row: its options, its largest logit, and the bounds of this block's chunk.
struct RowView {
  const float* x;
  RowScratch* rs;
  float inv_t, mx, tp, mp;
  int k, begin, end, argmax;
  bool greedy, use_k, use_p;
};

__device__ __forceinline__ RowView row_view(const SampleArgs& a) {
  RowView v;
  const int r = blockIdx.y;
  v.x = a.logits + (size_t)r * a.V;
  v.rs = a.scratch + r;
  const float temp = a.temperature[r];
  v.greedy = temp < 1e-5f;  // sampling_params.py:35-37
  v.inv_t = 1.f / fmaxf(temp, 1e-5f);
  v.k = a.top_k[r];
  v.tp = a.top_p[r];
  v.mp = a.min_p[r];
  v.use_k = !v.greedy && v.k > 0 && v.k < a.V;
  v.use_p = !v.greedy && v.tp < 1.f;
  const int len = ((a.V + a.chunks - 1) / a.chunks + 3) & ~3;
  v.begin = min(a.V, (int)blockIdx.x * len);
  v.end = min(a.V, v.begin + len);
  v.argmax = 0;
  v.mx = 0.f;
  return v;
}

// f(i, x[i]) for this thread's share of the block's chunk: 16-byte loads where the row allows them
// (a chunk starts at a multiple of four).
template <typename F>
__device__ __forceinline__ void chunk_for_each(const RowView& v, int V, F f) {
  if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(v.x) & 15) == 0) {
#pragma unroll 2
    for (int i = v.begin + 4 * (int)threadIdx.x; i < v.end; i += 4 * SP_THREADS) {  // v.end is V or a multiple of four
      const float4 q = *reinterpret_cast<const float4*>(v.x + i);
      f(i, q.x); f(i + 1, q.y); f(i + 2, q.z); f(i + 3, q.w);
    }
  } else {
#pragma unroll 4
    for (int i = v.begin + (int)threadIdx.x; i < v.end; i += SP_THREADS) f(i, v.x[i]);
  }
}

// After the first pass: the index of the largest logit (lowest index among equals) and the largest scaled logit.
__device__ __forceinline__ void read_max(RowView& v) {
  const unsigned long long top = __ldcg(&v.rs->best);
  v.argmax = (int)(0xFFFFFFFFu - (unsigned)(top & 0xFFFFFFFFull));
  v.mx = v.x[v.argmax] * v.inv_t;  // scaling by a positive number keeps the order
}

// Suffix sums over the 256 bins of a histogram (thread b = bin b, 256 threads): sum of bins >= b.
template <typename T>
__device__ T suffix_sum_256(T mine, T* scratch /* [8] */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T v = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {  // inclusive suffix scan inside the warp
    const T up = __shfl_down_sync(0xffffffffu, v, o);
    if (lane + o < 32) v += up;
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = v;  // the warp's total
  __syncthreads();
  T above = 0;
  for (int w = warp + 1; w < 8; ++w) above += scratch[w];
  return v + above;
}

// The key of the k-th largest scaled logit after `digits` digits (the lower digits are zero), and how
// many of the k lie among the keys that share them.  A pass knows the digits before it from the
// record of the pass before, reads the last one off that pass's histogram (the largest digit with
// at least k keys at or above it: one bin has suffix >= k > suffix of the next bin), and its block
// 0 records the result for the passes behind it.
__device__ unsigned top_k_state(const RowView& v, int digits, int* k_left, int* iscratch, int* ishare) {
  if (digits == 0) { *k_left = v.k; return 0u; }
  const int q = digits - 1;
  const unsigned before = q ? __ldcg(&v.rs->k_prefix[q]) : 0u;
  const int k = q ? __ldcg(&v.rs->k_left[q]) : v.k;
  const int mine = __ldcg(&v.rs->count[q][threadIdx.x]);
  const int suffix = suffix_sum_256(mine, iscratch);
  if (threadIdx.x == 0) { ishare[0] = 0; ishare[1] = k; }
  __syncthreads();
  if (suffix >= k && suffix - mine < k) { ishare[0] = threadIdx.x; ishare[1] = k - (suffix - mine); }
  __syncthreads();
  const unsigned key = before | ((unsigned)ishare[0] << (24 - 8 * q));
  *k_left = ishare[1];
  if (blockIdx.x == 0 && threadIdx.x == 0) { v.rs->k_prefix[digits] = key; v.rs->k_left[digits] = ishare[1]; }
  __syncthreads();
  return key;
}

// The cut of top-p after `digits` digits: the largest pattern v (lower digits zero) with
// mass(bits >= v) > top_p, and the mass that lies above the digits found; worked out and recorded
// like top_k_state (the largest digit d with above + mass(digit >= d) > top_p; none: digit 0).
__device__ unsigned top_p_state(const RowView& v, int digits, unsigned long long tp_fixed, unsigned long long* above_out,
                                unsigned long long* lscratch, unsigned long long* lshare) {
  if (digits == 0) { *above_out = 0ull; return 0u; }
  const int q = digits - 1;
  const unsigned before = q ? __ldcg(&v.rs->p_prefix[q]) : 0u;
  const unsigned long long above = q ? __ldcg(&v.rs->p_above[q]) : 0ull;
  const unsigned long long mine = __ldcg(&v.rs->mass[q][threadIdx.x]);
  const unsigned long long suffix = suffix_sum_256(mine, lscratch);
  if (threadIdx.x == 0) { lshare[0] = 0; lshare[1] = 0; }
  __syncthreads();
  if (above + suffix > tp_fixed && !(above + suffix - mine > tp_fixed)) { lshare[0] = threadIdx.x; lshare[1] = suffix - mine; }
  __syncthreads();
  const unsigned cut = before | ((unsigned)lshare[0] << (24 - 8 * q));
  *above_out = above + lshare[1];
  if (blockIdx.x == 0 && threadIdx.x == 0) { v.rs->p_prefix[digits] = cut; v.rs->p_above[digits] = above + lshare[1]; }
  __syncthreads();
  return cut;
}

// p in [0, 1] as a multiple of 2^-52: scaling by a power of two and the conversion are exact
__device__ __forceinline__ unsigned long long to_fixed(float p) { return __float2ull_rz(p * 4503599627370496.f); }
static_assert(SP_FIXED_BITS == 52, "4503599627370496 = 2^52");

// pass 0: the largest logit of every row and its index
__global__ void __launch_bounds__(SP_THREADS) sample_max_kernel(const SampleArgs a) {
  __shared__ unsigned long long warp_best[SP_THREADS / 32];
  pdl_launch_dependents();
  pdl_wait();
  const RowView v = row_view(a);
  unsigned long long mine = 0ull;
  chunk_for_each(v, a.V, [&](int i, float x) {
    const unsigned long long cand = ((unsigned long long)ordered_key(x) << 32) | (0xFFFFFFFFu - (unsigned)i);
    mine = cand > mine ? cand : mine;
  });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, mine, o);
    mine = other > mine ? other : mine;
  }
  if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < SP_THREADS / 32; ++w) mine = warp_best[w] > mine ? warp_best[w] : mine;
    if (mine) atomicMax(&v.rs->best, mine);
  }
}

// top-k, digit `pass` (0: the top eight bits): how many keys that share the digits found so far have each next digit
__global__ void __launch_bounds__(SP_THREADS) sample_count_kernel(const SampleArgs a, int pass) {
  __shared__ int hist[256];
  __shared__ int iscratch[8];
  __shared__ int ishare[2];
  pdl_launch_dependents();
  pdl_wait();
  RowView v = row_view(a);
  if (!v.use_k) return;
  int k_left;
  const unsigned prefix = top_k_state(v, pass, &k_left, iscratch, ishare);
  const int shift = 24 - 8 * pass;
  hist[threadIdx.x] = 0;
  __syncthreads();
  chunk_for_each(v, a.V, [&](int, float x) {
    const unsigned key = ordered_key(x * v.inv_t);
    if (pass == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8))) atomicAdd(&hist[(key >> shift) & 255u], 1);
  });
  __syncthreads();
  if (hist[threadIdx.x]) atomicAdd(&v.rs->count[pass][threadIdx.x], hist[threadIdx.x]);
}

// the normaliser: sum of exp(s - max) over the tokens that top-k keeps, per chunk
__global__ void __launch_bounds__(SP_THREADS) sample_z_kernel(const SampleArgs a) {
  __shared__ float fs[33];
  __shared__ int iscratch[8];
  __shared__ int ishare[2];
  pdl_launch_dependents();
  pdl_wait();
  RowView v = row_view(a);
  if (v.greedy) return;
  read_max(v);
  int k_left;
  const unsigned kth = v.use_k ? top_k_state(v, 4, &k_left, iscratch, ishare) : 0u;  // the last digit: found and recorded here
  float z = 0.f;
  chunk_for_each(v, a.V, [&](int, float x) {
    const float s = x * v.inv_t;
    z += ordered_key(s) >= kth ? expf(s - v.mx) : 0.f;
  });
  z = block_sum(z, fs);
  if (threadIdx.x == 0) v.rs->z_part[blockIdx.x] = z;
}

__device__ __forceinline__ float sum_parts(const float* parts, int chunks) {  // in chunk order, by every thread alike
  float t = 0.f;
  for (int c = 0; c < chunks; ++c) t += __ldcg(parts + c);
  return t;
}

// top-p, digit `pass`: the probability mass of every next digit among the probabilities that share the digits found
__global__ void __launch_bounds__(SP_THREADS) sample_mass_kernel(const SampleArgs a, int pass) {
  __shared__ unsigned long long hist[256];
  __shared__ unsigned long long lscratch[8];
  __shared__ unsigned long long lshare[2];
  pdl_launch_dependents();
  pdl_wait();
  RowView v = row_view(a);
  if (!v.use_p) return;
  read_max(v);
  const unsigned kth = v.use_k ? __ldcg(&v.rs->k_prefix[4]) : 0u;
  const float inv_z = 1.f / sum_parts(v.rs->z_part, a.chunks);
  unsigned long long above;
  const unsigned prefix = top_p_state(v, pass, to_fixed(v.tp), &above, lscratch, lshare);
  const int shift = 24 - 8 * pass;
  hist[threadIdx.x] = 0ull;
  __syncthreads();
  chunk_for_each(v, a.V, [&](int, float x) {
    const float s = x * v.inv_t;
    const float p = ordered_key(s) >= kth ? expf(s - v.mx) * inv_z : 0.f;
    const unsigned bits = __float_as_uint(p);
    if (p > 0.f && (pass == 0 || (bits >> (shift + 8)) == (prefix >> (shift + 8)))) atomicAdd(&hist[(bits >> shift) & 255u], to_fixed(p));
  });
  __syncthreads();
  if (hist[threadIdx.x]) atomicAdd(&v.rs->mass[pass][threadIdx.x], hist[threadIdx.x]);
}

// The probability a token keeps after all filters (0: dropped).
struct Filter {
  unsigned kth, cut;
  float inv_z, floor_p, inv_t, mx;
  __device__ __forceinline__ float kept(float logit) const {
    const float s = logit * inv_t;
    const float p = ordered_key(s) >= kth ? expf(s - mx) * inv_z : 0.f;
    return (__float_as_uint(p) < cut || p < floor_p) ? 0.f : p;
  }
};

// `recorded`: the last digit of the top-p cut has been worked out by an earlier launch
__device__ Filter make_filter(RowView& v, const SampleArgs& a, bool recorded, unsigned long long* lscratch, unsigned long long* lshare) {
  Filter f;
  read_max(v);
  f.kth = v.use_k ? __ldcg(&v.rs->k_prefix[4]) : 0u;
  f.inv_z = 1.f / sum_parts(v.rs->z_part, a.chunks);
  unsigned long long above;
  // keep a token iff the mass of strictly larger probabilities is <= top_p: bits >= the largest v with mass(bits >= v) > top_p
  f.cut = !v.use_p ? 0u : recorded ? __ldcg(&v.rs->p_prefix[4]) : top_p_state(v, 4, to_fixed(v.tp), &above, lscratch, lshare);
  f.floor_p = v.mp > 0.f ? v.mp * f.inv_z : 0.f;  // min-p relative to the largest probability, exp(0) / z
  f.inv_t = v.inv_t;
  f.mx = v.mx;
  return f;
}

// the mass that survives all filters, per chunk
__global__ void __launch_bounds__(SP_THREADS) sample_kept_kernel(const SampleArgs a) {
  __shared__ float fs[33];
  __shared__ unsigned long long lscratch[8];
  __shared__ unsigned long long lshare[2];
  pdl_launch_dependents();
  pdl_wait();
  RowView v = row_view(a);
  if (v.greedy) return;
  const Filter f = make_filter(v, a, false, lscratch, lshare);
  float m = 0.f;
  chunk_for_each(v, a.V, [&](int, float x) { m += f.kept(x); });
  m = block_sum(m, fs);
  if (threadIdx.x == 0) v.rs->kept_part[blockIdx.x] = m;
}

// the draw: inverse CDF in vocabulary order at u * total; the block whose chunk holds that point picks the token
__global__ void __launch_bounds__(SP_THREADS) sample_pick_kernel(const SampleArgs a) {
  __shared__ float prefix[SP_THREADS];
  __shared__ int ishare[2];
  __shared__ int chosen;
  pdl_launch_dependents();
  pdl_wait();
  RowView v = row_view(a);
  const int r = blockIdx.y, tid = threadIdx.x;
  if (v.greedy) {
    if (blockIdx.x == 0 && tid == 0) { read_max(v); a.out[r] = v.argmax; }
    return;
  }
  // which chunk holds the target (every block finds the same answer); `last`: the last chunk with any mass
  float total = 0.f;
  for (int c = 0; c < a.chunks; ++c) total += __ldcg(v.rs->kept_part + c);
  const float target = a.uniform[r] * total;
  int mine = -1, last = -1;
  float before = 0.f, run = 0.f;
  for (int c = 0; c < a.chunks; ++c) {
    const float m = __ldcg(v.rs->kept_part + c);
    if (m > 0.f) {
      last = c;
      if (mine < 0 && target < run + m) { mine = c; before = run; }
    }
    run += m;
  }
  const bool past_end = mine < 0;  // rounding pushed the target past the end: the last kept token
  if (past_end) mine = last;
  if ((int)blockIdx.x != mine) return;
  const Filter f = make_filter(v, a, true, nullptr, nullptr);
  // thread t owns the contiguous piece [b, e) of the chunk
  const int len = v.end - v.begin, piece = (len + SP_THREADS - 1) / SP_THREADS;
  const int b = min(v.end, v.begin + tid * piece), e = min(v.end, b + piece);
  float sum = 0.f;
  for (int i = b; i < e; ++i) sum += f.kept(v.x[i]);
  prefix[tid] = sum;
  __syncthreads();
  for (int o = 1; o < SP_THREADS; o <<= 1) {  // inclusive scan over the thread sums
    const float add = tid >= o ? prefix[tid - o] : 0.f;
    __syncthreads();
    prefix[tid] += add;
    __syncthreads();
  }
  if (tid == 0) chosen = a.V;
  __syncthreads();
  const float start = before + (tid > 0 ? prefix[tid - 1] : 0.f);
  if (!past_end && sum > 0.f && start <= target && target < before + prefix[tid]) {
    float c = start;
    int pick = -1, seen = -1;
    for (int i = b; i < e; ++i) {
      const float p = f.kept(v.x[i]);
      if (p > 0.f) {
        seen = i;
        c += p;
        if (c > target) { pick = i; break; }
      }
    }
    atomicMin(&chosen, pick >= 0 ? pick : seen);
  }
  __syncthreads();
  if (chosen == a.V) {  // no thread's interval took the target (rounding): the last kept token of the chunk
    int seen = -1;
    for (int i = b; i < e; ++i) if (f.kept(v.x[i]) > 0.f) seen = i;
    if (tid == 0) ishare[0] = -1;
    __syncthreads();
    if (seen >= 0) atomicMax(&ishare[0], seen);
    __syncthreads();
    if (tid == 0) chosen = ishare[0] >= 0 ? ishare[0] : v.argmax;
    __syncthreads();
  }
  if (tid == 0) a.out[r] = chosen;
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

// Bytes of scratch a row needs; the scratch [R rows] must be zero when tb_sample is called.
int tb_sample_scratch_bytes() { return (int)sizeof(tb::RowScratch); }

// One token per row.  top_k_any / top_p_any: whether any row uses that filter (its passes are skipped otherwise).
int tb_sample(void* stream, const float* logits, const float* temperature, const int* top_k, const float* top_p,
              const float* min_p, const float* uniform, void* scratch, int* out, int R, int V, int top_k_any, int top_p_any) {
  if (R <= 0) return 0;
  if (V <= 0 || R > 65535) return TB_ERR_BAD_SIZE;
  tb::SampleArgs a;
  a.logits = logits; a.temperature = temperature; a.top_k = top_k; a.top_p = top_p; a.min_p = min_p; a.uniform = uniform;
  a.scratch = static_cast<tb::RowScratch*>(scratch); a.out = out; a.V = V;
  // chunks of at least 2,048 logits, and about four blocks per SM over all rows
  int chunks = (592 + R - 1) / R;
  if (chunks > V / 2048) chunks = V / 2048;
  a.chunks = chunks < 1 ? 1 : (chunks > tb::SP_MAX_CHUNKS ? tb::SP_MAX_CHUNKS : chunks);
  const dim3 grid(a.chunks, R), block(tb::SP_THREADS);
  int e = tb::launch(tb::sample_max_kernel, grid, block, 0, stream, a);
  if (top_k_any)
    for (int pass = 0; pass < 4 && !e; ++pass) e = tb::launch(tb::sample_count_kernel, grid, block, 0, stream, a, pass);
  if (!e) e = tb::launch(tb::sample_z_kernel, grid, block, 0, stream, a);
  if (top_p_any)
    for (int pass = 0; pass < 4 && !e; ++pass) e = tb::launch(tb::sample_mass_kernel, grid, block, 0, stream, a, pass);
  if (!e) e = tb::launch(tb::sample_kept_kernel, grid, block, 0, stream, a);
  if (!e) e = tb::launch(tb::sample_pick_kernel, grid, block, 0, stream, a);
  return e;
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
