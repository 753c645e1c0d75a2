// Sampling over logits [R, V] float32: argmax, and temperature sampling with the top-k, top-p and
// min-p filters of 12vivi/tandem (python/tandem/layers/sampler.py:19-64).
//
// Where tandem sorts the row, these kernels find the same cut by radix selection on the bit
// pattern of the values (non-negative floats and their order-preserving keys compare like
// unsigned integers), eight bits a pass: a pass builds a histogram of the next digit among the
// values that share the digits found so far, counts for top-k and probability mass for top-p (in
// 52-bit fixed point, so that the sums are integers and do not depend on the order of the atomic
// additions), and the next pass reads off the digit.  A row is cut into eight chunks that the blocks
// of a thread-block cluster work on at once (a row of 150,000 logits is more than one SM should walk
// a dozen times); all passes run in one launch, the cluster meeting between them; sums that stay
// floating point (the normaliser, the kept mass per chunk) are taken per chunk and added in chunk
// order, so a row's token does not depend on how many rows the call has.  Where tandem draws with torch.multinomial, the
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
// Temperature sampling: one cluster of blocks per row, one launch for all passes.
constexpr int SP_THREADS = 1024;
constexpr int SP_MAX_CHUNKS = 8;  // a row is cut into eight chunks; a cluster of 8, 4, 2 or 1 blocks shares them out
constexpr int SP_FIXED_BITS = 52;  // probability mass as an integer multiple of 2^-52
constexpr int SP_LANES = 64;     // private copies of the first top-p histogram (see pass_mass)

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
  int V, cluster;  // blocks per row (gridDim.x)
};

// What every pass needs of a row: its options, its largest logit, and the bounds of this block's chunk.
struct RowView {
  const float* x;
  RowScratch* rs;
  float inv_t, mx, tp, mp, inv_z;
  int k, begin, end, argmax;  // [begin, end): all the chunks of this block
  int first_chunk, num_chunks, chunk_len;
  bool greedy, use_k, use_p;
};

struct SampleShared {
  unsigned long long lanes[32][SP_LANES];  // pass_mass, first digit: private copies of the histogram's upper bins
  unsigned long long lhist[256], lscratch[8], lshare[2], warp_best[SP_THREADS / 32];
  int ihist[256], iscratch[8], ishare[2], chosen;
  float fs[33], parts[SP_MAX_CHUNKS], prefix[SP_THREADS];
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
  v.chunk_len = ((a.V + SP_MAX_CHUNKS - 1) / SP_MAX_CHUNKS + 3) & ~3;
  v.num_chunks = SP_MAX_CHUNKS / a.cluster;
  v.first_chunk = (int)blockIdx.x * v.num_chunks;
  v.begin = min(a.V, v.first_chunk * v.chunk_len);
  v.end = min(a.V, v.begin + v.num_chunks * v.chunk_len);
  v.argmax = 0;
  v.mx = 0.f;
  v.inv_z = 0.f;
  return v;
}

// f(i, x[i]) for this thread's share of [begin, end) of the row: 16-byte loads where the row allows them
// (begin is a multiple of four, end is V or one), four of them in flight.
template <typename F>
__device__ __forceinline__ void range_for_each(const RowView& v, int V, int begin, int end, F f) {
  if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(v.x) & 15) == 0) {
#pragma unroll 4
    for (int i = begin + 4 * (int)threadIdx.x; i < end; i += 4 * SP_THREADS) {
      const float4 q = *reinterpret_cast<const float4*>(v.x + i);
      f(i, q.x); f(i + 1, q.y); f(i + 2, q.z); f(i + 3, q.w);
    }
  } else {
#pragma unroll 4
    for (int i = begin + (int)threadIdx.x; i < end; i += SP_THREADS) f(i, v.x[i]);
  }
}

// All the chunks of this block at once (for what does not depend on the order: maxima, integer sums).
template <typename F>
__device__ __forceinline__ void chunk_for_each(const RowView& v, int V, F f) { range_for_each(v, V, v.begin, v.end, f); }

// Chunk by chunk, g(chunk, sum over the block of f's results in that chunk): sums in floating point are taken per
// chunk by the same threads over the same elements however many chunks a block has, so that a row's
// result does not depend on how many blocks share it (which goes with the number of rows).
template <typename F, typename G>
__device__ __forceinline__ void chunk_sums(const RowView& v, int V, float* scratch33, F f, G g) {
  for (int c = v.first_chunk; c < v.first_chunk + v.num_chunks; ++c) {
    const int begin = min(V, c * v.chunk_len), end = min(V, begin + v.chunk_len);
    float t = 0.f;
    range_for_each(v, V, begin, end, [&](int, float x) { t += f(x); });
    t = block_sum(t, scratch33);
    if (threadIdx.x == 0) g(c, t);
  }
}

// The blocks of a row meet: what each has added to the row's scratch in global memory is seen by all behind it.
__device__ __forceinline__ void row_meet() {  // (every thread releases what it wrote and acquires what the others did)
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// After the first pass: the index of the largest logit (lowest index among equals) and the largest scaled logit.
__device__ __forceinline__ void read_max(RowView& v) {
  const unsigned long long top = __ldcg(&v.rs->best);
  v.argmax = (int)(0xFFFFFFFFu - (unsigned)(top & 0xFFFFFFFFull));
  v.mx = v.x[v.argmax] * v.inv_t;  // scaling by a positive number keeps the order
}

// Suffix sums over the 256 bins of a histogram (thread b = bin b for the block's first 256 threads, the
// others bring zero and get nothing of use back): sum of bins >= b.  Called by the whole block.
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
  if (lane == 0 && warp < 8) scratch[warp] = v;  // the warp's total
  __syncthreads();
  T above = 0;
  for (int w = warp + 1; w < 8; ++w) above += scratch[w];
  return v + above;
}

// The key of the k-th largest scaled logit after `digits` digits (the lower digits are zero), and how
// many of the k lie among the keys that share them.  A pass knows the digits before it from the
// record of the pass before, reads the last one off that pass's histogram (the largest digit with
// at least k keys at or above it: one bin has suffix >= k > suffix of the next bin), and the row's
// first block records the result for the passes behind it.
__device__ unsigned top_k_state(const RowView& v, int digits, int* k_left, int* iscratch, int* ishare) {
  if (digits == 0) { *k_left = v.k; return 0u; }
  const int q = digits - 1;
  const bool bin = threadIdx.x < 256;
  const unsigned before = q ? __ldcg(&v.rs->k_prefix[q]) : 0u;
  const int k = q ? __ldcg(&v.rs->k_left[q]) : v.k;
  const int mine = bin ? __ldcg(&v.rs->count[q][threadIdx.x]) : 0;
  const int suffix = suffix_sum_256(mine, iscratch);
  if (threadIdx.x == 0) { ishare[0] = 0; ishare[1] = k; }
  __syncthreads();
  if (bin && suffix >= k && suffix - mine < k) { ishare[0] = threadIdx.x; ishare[1] = k - (suffix - mine); }
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
  const bool bin = threadIdx.x < 256;
  const unsigned before = q ? __ldcg(&v.rs->p_prefix[q]) : 0u;
  const unsigned long long above = q ? __ldcg(&v.rs->p_above[q]) : 0ull;
  const unsigned long long mine = bin ? __ldcg(&v.rs->mass[q][threadIdx.x]) : 0ull;
  const unsigned long long suffix = suffix_sum_256(mine, lscratch);
  if (threadIdx.x == 0) { lshare[0] = 0; lshare[1] = 0; }
  __syncthreads();
  if (bin && above + suffix > tp_fixed && !(above + suffix - mine > tp_fixed)) { lshare[0] = threadIdx.x; lshare[1] = suffix - mine; }
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

// the largest logit of the row and its index
__device__ void pass_max(const SampleArgs& a, const RowView& v, SampleShared& sh) {
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
  if ((threadIdx.x & 31) == 0) sh.warp_best[threadIdx.x >> 5] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < SP_THREADS / 32; ++w) mine = sh.warp_best[w] > mine ? sh.warp_best[w] : mine;
    if (mine) atomicMax(&v.rs->best, mine);
  }
}

// top-k, digit `pass` (0: the top eight bits): how many keys that share the digits found so far have each next digit
__device__ void pass_count(const SampleArgs& a, const RowView& v, int pass, SampleShared& sh) {
  int k_left;
  const unsigned prefix = top_k_state(v, pass, &k_left, sh.iscratch, sh.ishare);
  const int shift = 24 - 8 * pass;
  if (threadIdx.x < 256) sh.ihist[threadIdx.x] = 0;
  __syncthreads();
  chunk_for_each(v, a.V, [&](int, float x) {
    const unsigned key = ordered_key(x * v.inv_t);
    if (pass == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8))) atomicAdd(&sh.ihist[(key >> shift) & 255u], 1);
  });
  __syncthreads();
  if (threadIdx.x < 256 && sh.ihist[threadIdx.x]) atomicAdd(&v.rs->count[pass][threadIdx.x], sh.ihist[threadIdx.x]);
}

// the normaliser: sum of exp(s - max) over the tokens that top-k keeps, per chunk
__device__ void pass_z(const SampleArgs& a, const RowView& v, SampleShared& sh) {
  int k_left;
  const unsigned kth = v.use_k ? top_k_state(v, 4, &k_left, sh.iscratch, sh.ishare) : 0u;  // the last digit: found and recorded here
  chunk_sums(v, a.V, sh.fs,
             [&](float x) {
               const float s = x * v.inv_t;
               return ordered_key(s) >= kth ? expf(s - v.mx) : 0.f;
             },
             [&](int c, float z) { v.rs->z_part[c] = z; });
}

// The sum of a row's per-chunk parts, in chunk order, by every thread alike.  The parts come through shared
// memory: one round trip to the L2 for all of them.
__device__ __forceinline__ float sum_parts(const float* parts, float* staged) {
  if (threadIdx.x < SP_MAX_CHUNKS) staged[threadIdx.x] = __ldcg(parts + threadIdx.x);
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int c = 0; c < SP_MAX_CHUNKS; ++c) t += staged[c];
  __syncthreads();  // `staged` may be filled again
  return t;
}

// top-p, digit `pass`: the probability mass of every next digit among the probabilities that share the digits found.
// Atomics on one word of shared memory take turns, 64-bit ones by compare-and-swap, and the first digit of a
// probability (a float's top eight bits: its sign and most of its exponent) falls into a handful of bins: with
// one histogram per block that pass took 293 us at 64 rows where the others took 17.  So the first digit is
// counted in SP_LANES private copies of the bins that can hold mass at all (a probability below 2^-52 is zero
// in fixed point, which leaves the top eight bits 32 .. 63), a thread adding to the copy of its lane, where
// it meets only threads of other warps; the copies are added up in a fixed order (the sums are integers).
__device__ void pass_mass(const SampleArgs& a, const RowView& v, int pass, SampleShared& sh) {
  const unsigned kth = v.use_k ? __ldcg(&v.rs->k_prefix[4]) : 0u;
  unsigned long long above;
  const unsigned prefix = top_p_state(v, pass, to_fixed(v.tp), &above, sh.lscratch, sh.lshare);
  const int shift = 24 - 8 * pass;
  if (threadIdx.x < 256) sh.lhist[threadIdx.x] = 0ull;
  if (pass == 0)
    for (int i = threadIdx.x; i < 32 * SP_LANES; i += SP_THREADS) (&sh.lanes[0][0])[i] = 0ull;
  __syncthreads();
  if (pass == 0) {
    const int copy = threadIdx.x & (SP_LANES - 1);
    chunk_for_each(v, a.V, [&](int, float x) {
      const float s = x * v.inv_t;
      const float p = ordered_key(s) >= kth ? expf(s - v.mx) * v.inv_z : 0.f;
      const unsigned long long mass = to_fixed(p);
      const unsigned digit = __float_as_uint(p) >> 24;  // 63 at most: p <= 1
      if (mass) atomicAdd(&sh.lanes[digit & 31u][copy], mass);  // mass > 0: digit >= 32
    });
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;  // warp w adds up the copies of bin 32 + w
    unsigned long long t = sh.lanes[warp][lane] + sh.lanes[warp][lane + 32];
    static_assert(SP_LANES == 64 && SP_THREADS == 1024, "one warp per bin, two copies per lane");
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) sh.lhist[32 + warp] = t;
  } else {
    chunk_for_each(v, a.V, [&](int, float x) {
      const float s = x * v.inv_t;
      const float p = ordered_key(s) >= kth ? expf(s - v.mx) * v.inv_z : 0.f;
      const unsigned bits = __float_as_uint(p);
      if (p > 0.f && (bits >> (shift + 8)) == (prefix >> (shift + 8))) atomicAdd(&sh.lhist[(bits >> shift) & 255u], to_fixed(p));
    });
  }
  __syncthreads();
  if (threadIdx.x < 256 && sh.lhist[threadIdx.x]) atomicAdd(&v.rs->mass[pass][threadIdx.x], sh.lhist[threadIdx.x]);
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

// `recorded`: the last digit of the top-p cut has been worked out by an earlier pass
__device__ Filter make_filter(const RowView& v, bool recorded, SampleShared& sh) {
  Filter f;
  f.kth = v.use_k ? __ldcg(&v.rs->k_prefix[4]) : 0u;
  f.inv_z = v.inv_z;
  unsigned long long above;
  // keep a token iff the mass of strictly larger probabilities is <= top_p: bits >= the largest v with mass(bits >= v) > top_p
  f.cut = !v.use_p ? 0u : recorded ? __ldcg(&v.rs->p_prefix[4]) : top_p_state(v, 4, to_fixed(v.tp), &above, sh.lscratch, sh.lshare);
  f.floor_p = v.mp > 0.f ? v.mp * f.inv_z : 0.f;  // min-p relative to the largest probability, exp(0) / z
  f.inv_t = v.inv_t;
  f.mx = v.mx;
  return f;
}

// the mass that survives all filters, per chunk
__device__ void pass_kept(const SampleArgs& a, const RowView& v, SampleShared& sh) {
  const Filter f = make_filter(v, false, sh);
  chunk_sums(v, a.V, sh.fs, [&](float x) { return f.kept(x); }, [&](int c, float m) { v.rs->kept_part[c] = m; });
}

// the draw: inverse CDF in vocabulary order at u * total; the block whose chunk holds that point picks the token
__device__ void pass_pick(const SampleArgs& a, const RowView& v, SampleShared& sh) {
  const int r = blockIdx.y, tid = threadIdx.x;
  // which chunk holds the target (every block finds the same answer); `last`: the last chunk with any mass
  if (tid < SP_MAX_CHUNKS) sh.parts[tid] = __ldcg(v.rs->kept_part + tid);
  __syncthreads();
  float total = 0.f;
  for (int c = 0; c < SP_MAX_CHUNKS; ++c) total += sh.parts[c];
  const float target = a.uniform[r] * total;
  int mine = -1, last = -1;
  float before = 0.f, run = 0.f;
  for (int c = 0; c < SP_MAX_CHUNKS; ++c) {
    const float m = sh.parts[c];
    if (m > 0.f) {
      last = c;
      if (mine < 0 && target < run + m) { mine = c; before = run; }
    }
    run += m;
  }
  const bool past_end = mine < 0;  // rounding pushed the target past the end: the last kept token
  if (past_end) mine = last;
  if (mine < v.first_chunk || mine >= v.first_chunk + v.num_chunks) return;
  const Filter f = make_filter(v, true, sh);
  // thread t owns the contiguous piece [b, e) of the chunk
  const int c_begin = min(a.V, mine * v.chunk_len), c_end = min(a.V, c_begin + v.chunk_len);
  const int len = c_end - c_begin, piece = (len + SP_THREADS - 1) / SP_THREADS;
  const int b = min(c_end, c_begin + tid * piece), e = min(c_end, b + piece);
  float sum = 0.f;
  for (int i = b; i < e; ++i) sum += f.kept(v.x[i]);
  float* prefix = sh.prefix;
  prefix[tid] = sum;
  __syncthreads();
  for (int o = 1; o < SP_THREADS; o <<= 1) {  // inclusive scan over the thread sums
    const float add = tid >= o ? prefix[tid - o] : 0.f;
    __syncthreads();
    prefix[tid] += add;
    __syncthreads();
  }
  if (tid == 0) sh.chosen = a.V;
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
    atomicMin(&sh.chosen, pick >= 0 ? pick : seen);
  }
  __syncthreads();
  if (sh.chosen == a.V) {  // no thread's interval took the target (rounding): the last kept token of the chunk
    int seen = -1;
    for (int i = b; i < e; ++i) if (f.kept(v.x[i]) > 0.f) seen = i;
    if (tid == 0) sh.ishare[0] = -1;
    __syncthreads();
    if (seen >= 0) atomicMax(&sh.ishare[0], seen);
    __syncthreads();
    if (tid == 0) sh.chosen = sh.ishare[0] >= 0 ? sh.ishare[0] : v.argmax;
    __syncthreads();
  }
  if (tid == 0) a.out[r] = sh.chosen;
}

// One row per cluster: the passes follow one another in one launch, the row's blocks meeting in between
// (as separate launches, twelve of them with every filter on, each cost 10 to 17 us of which the walk
// over the logits was the least part).  A row skips the passes of the filters it does not use.  The
// cluster's size is the launch's (gridDim.x: 8 blocks a row for few rows, fewer for many, so that all
// rows are resident at once).
__global__ void __launch_bounds__(SP_THREADS, 1) sample_kernel(const SampleArgs a) {
  __shared__ SampleShared sh;
  pdl_launch_dependents();
  pdl_wait();
  RowView v = row_view(a);
  pass_max(a, v, sh);
  row_meet();
  read_max(v);
  if (v.greedy) {  // (the whole row, and so the whole cluster)
    if (blockIdx.x == 0 && threadIdx.x == 0) a.out[blockIdx.y] = v.argmax;
    return;
  }
  if (v.use_k)
    for (int pass = 0; pass < 4; ++pass) {
      pass_count(a, v, pass, sh);
      row_meet();
    }
  pass_z(a, v, sh);
  row_meet();
  v.inv_z = 1.f / sum_parts(v.rs->z_part, sh.parts);
  if (v.use_p)
    for (int pass = 0; pass < 4; ++pass) {
      pass_mass(a, v, pass, sh);
      row_meet();
    }
  pass_kept(a, v, sh);
  row_meet();
  pass_pick(a, v, sh);
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

// One token per row.  top_k_any / top_p_any: whether any row uses that filter; kept for callers, since every
// row skips the passes of the filters it does not use by itself.
int tb_sample(void* stream, const float* logits, const float* temperature, const int* top_k, const float* top_p,
              const float* min_p, const float* uniform, void* scratch, int* out, int R, int V, int top_k_any, int top_p_any) {
  (void)top_k_any; (void)top_p_any;
  if (R <= 0) return 0;
  if (V <= 0 || R > 65535) return TB_ERR_BAD_SIZE;
  tb::SampleArgs a;
  a.logits = logits; a.temperature = temperature; a.top_k = top_k; a.top_p = top_p; a.min_p = min_p; a.uniform = uniform;
  a.scratch = static_cast<tb::RowScratch*>(scratch); a.out = out; a.V = V;
  // A block of 1,024 threads has an SM to itself, and a cluster's blocks must find their SMs in one GPC: the most
  // blocks per row with which all rows are resident at once (asked of the driver once per device and size).
  static int resident[64][4] = {};  // clusters of 8, 4, 2, 1 blocks that can run at a time
  int device = 0;
  cudaError_t ce = cudaGetDevice(&device);
  if (ce != cudaSuccess) return (int)ce;
  if (device < 0 || device >= 64) return TB_ERR_BAD_SIZE;
  a.cluster = 1;
  for (int i = 0, size = tb::SP_MAX_CHUNKS; size > 1; ++i, size >>= 1) {
    if (!resident[device][i]) {
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3(size, 1024);
      q.blockDim = dim3(tb::SP_THREADS);
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = size; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
      q.attrs = qa;
      q.numAttrs = 1;
      int n = 0;
      ce = cudaOccupancyMaxActiveClusters(&n, tb::sample_kernel, &q);
      if (ce != cudaSuccess) return (int)ce;
      resident[device][i] = n > 0 ? n : -1;
    }
    if (resident[device][i] >= R) { a.cluster = size; break; }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.cluster, R);
  cfg.blockDim = dim3(tb::SP_THREADS);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = tb::pdl_enabled() ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = a.cluster; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return (int)cudaLaunchKernelEx(&cfg, tb::sample_kernel, a);
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
