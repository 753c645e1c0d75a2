// Paged attention for decoded tokens (one query token per request) in bfloat16, head size TB_HD
// fixed at compile time: split-KV "flash decoding" on the tensor cores, fed by the TMA unit.
//
// Work is cut on the host into items (request, key range); one block runs one item for one kv
// head and all the query heads that share it (rows of a 16-row MMA tile; more than 16 heads per kv
// head take further blocks along grid.z).  A producer warp walks the request's block table and
// issues 1-D bulk copies of cache tiles into a ring of shared-memory stages of 64 keys; the
// cache's own tile layout (cache_layout.cuh) is the swizzled layout ldmatrix wants, so no thread
// touches the data on its way in.  Four consumer warps take 16 keys of a stage each:
// S = Q K^T with mma.sync (bf16 in, float32 out), masking, online softmax in float32 with exp2,
// O += P V.  The warps' partial (max, sum, O) are merged through shared memory.  A request cut
// into several items leaves its partials in scratch memory; the block that arrives last (an
// atomic counter per request and kv head, reset by that block) merges them: nothing waits.
//
// In a step of decoded tokens only, the kernel in front of this one (per-head norm, rotary encoding
// and the cache write of the new token) can be folded in (`DecodeArgs::fresh`): the consumer warps
// normalise and rotate their query rows as they load them, and in the block that holds a request's
// newest key the warp whose 16 keys include it makes that key (and copies its value) itself, into
// its stage of shared memory over the stale row that the bulk copy brought, and into the cache for the
// steps to come.  The arithmetic is the stand-alone kernel's (rope_core.cuh), bit for bit.
//
// It does what 12vivi/tandem's Triton split-KV kernel does
// (python/tandem/layers/triton_decode_attn.py:28-129), and stands where it otherwise calls
// FlashInfer's decode wrapper (python/tandem/layers/flashinfer_attention.py:138-157).
#include "attention_common.cuh"
#include "rope_core.cuh"

namespace tb {

constexpr int WARPS = 4;               // consumer warps
static_assert(WARPS * TILE == STAGE_KEYS, "one sub-tile of a stage per consumer warp");
constexpr int STAGES = HD <= 64 ? 4 : (HD <= 128 ? 3 : 2);
constexpr int QS = HD + 8;             // padded row of the query tile in shared memory
constexpr int OS = HD + 4;             // padded row of a warp's float32 output in the merge buffer
constexpr int THREADS = (WARPS + 1) * 32;
constexpr int MAX_SPLITS = 64;         // items of one request the fast merge takes (48 floats of shared memory each)
constexpr int ITEM_INTS = 6;           // token row, request, key begin, key end, first item of the request, its item count

struct DecodeArgs {
  const __nv_bfloat16* q;  // [T, q_stride], query heads first
  int q_stride;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_table;
  int table_stride;
  const int* items;
  const int* num_items;  // device scalar: blocks beyond it return at once (fixed grids under CUDA graphs)
  __nv_bfloat16* out;    // [T, nh * HD]
  float* part_o;         // [items, nkv, G, HD] unnormalised outputs of split requests
  float* part_ml;        // [items, nkv, G, 2] their running max (log2 domain) and sum
  int* counters;         // [items * nkv * row tiles], zero between launches
  int* status;
  int nh, nkv, page_size;
  float scale_log2;
  // fresh != 0: q is the raw projection [T, (nh + 2 nkv) * HD] (q_stride = that width) and the cache has not got the
  // newest row yet; HD is a power of two and the whole head rotates
  int fresh;
  const float* q_norm_w;  // [HD] or null
  const float* k_norm_w;
  const float* cos_sin;   // [max_pos, HD]: cos of the HD / 2 angles, then their sin
  const int* positions;   // [T]
  const int* slots;       // [T] page * page_size + offset of the new row
  __nv_bfloat16* k_cache_w;
  __nv_bfloat16* v_cache_w;
  float eps;
  int max_pos;
};

// The lanes of a head (HD / 16 of them) load, normalise and rotate one row x[0 .. HD) of the raw projection;
// lane `sub` gets elements [8 sub, 8 sub + 8) in lo and [HD/2 + 8 sub, ...) in hi.  w: norm weight [HD] or null.
__device__ __forceinline__ void fresh_row(const __nv_bfloat16* x, const float* w, const float* angles, int sub, unsigned head_lanes,
                                          float eps, uint4& lo, uint4& hi) {
  constexpr int half = HD / 2, lanes_per_head = HD / 16;
  const int j = sub * 8;
  float a[8], b[8], wv[16], cc[8], ssn[8];
  unpack8(*reinterpret_cast<const uint4*>(x + j), a);
  unpack8(*reinterpret_cast<const uint4*>(x + half + j), b);
#pragma unroll
  for (int i = 0; i < 8; ++i) { wv[i] = w ? w[j + i] : 1.f; wv[8 + i] = w ? w[half + j + i] : 1.f; }
  load_angles(angles, half, j, cc, ssn);
  norm_rope_pairs(a, b, wv, w != nullptr, cc, ssn, HD, eps, head_lanes, lanes_per_head, lo, hi);
}

__global__ void __launch_bounds__(THREADS) attention_decode_kernel(const DecodeArgs a) {
  extern __shared__ unsigned char smem_unaligned[];
  // No early griddepcontrol.launch_dependents here: the kernel behind this one (the output projection)
  // becomes resident as this one's blocks exit.  Measured at Qwen3-8B sizes: with the trigger at the
  // top a decode step takes 3.75 ms at batch 8 and 3.37 ms at batch 1, without it 3.64 and 3.26 ms.  With
  // the trigger behind the last key, in front of the merge, and the streaming products behind letting
  // their own dependents in early (gemv_bf16.cu), *every* streaming product of the rest of the step
  // runs at half its speed, down to the output head (408 against 180 us; 5.5 against 3.45 ms a step,
  // at batch 1 as well, where most SMs hold no block of this kernel): an SM keeps the split between
  // shared memory and L1 that its resident blocks need, this kernel needs nearly all of it as shared
  // memory, and once a block of the streaming product has moved in beside or right behind one of
  // these, the SM is never idle again between two kernels of the chain, so the product's loads in
  // flight stay bounded by a small L1 (the same factor as asking for the largest carve-out for every
  // kernel).  Kernels with different needs of shared memory must not overlap on an SM.
  // The batch's description (items, their number, block tables) is written by the host before the
  // step's first kernel: it is read, and the barriers are set up, while the kernel in front of
  // this one still runs.  The queries and the newest cache rows are that kernel's output.
  const int num_items = *a.num_items;
  // grid = (kv heads, item slots, groups of 16 query heads): the kv heads run fastest, so that the blocks of
  // the plan's items are handed out first and those of the empty slots behind them last
  const int item_index = blockIdx.y;
  const int* item = a.items + (size_t)item_index * ITEM_INTS;
  const int t = item[0], req = item[1], kb = item[2], ke = item[3], first_item = item[4], nsplits = item[5];
  if (item_index >= num_items) return;
  // 128-byte rows of the swizzled tiles must start on 128-byte boundaries
  unsigned char* smem_raw = smem_unaligned + ((128u - (smem_u32(smem_unaligned) & 127u)) & 127u);
  __nv_bfloat16* stage_mem = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [STAGES][K | V][STAGE_KEYS * HD]
  __nv_bfloat16* q_s = stage_mem + STAGES * STAGE_ELEMS;  // [16][QS]
  float* m_s = reinterpret_cast<float*>(q_s + 16 * QS);   // [WARPS][16]
  float* l_s = m_s + WARPS * 16;
  uint64_t* full = reinterpret_cast<uint64_t*>(l_s + WARPS * 16);
  uint64_t* empty = full + STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + STAGES);
  int* last_flag = const_cast<int*>(abort_flag) + 1;
  int* table_s = last_flag + 1;  // [TABLE_CACHE] the request's page numbers for this block's keys

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvh = blockIdx.x, G = a.nh / a.nkv, ps = a.page_size;
  const int row0 = blockIdx.z * 16, rows = min(16, G - row0);  // query heads of this block: kvh*G + row0 + g
  const int xmask = min(7, ps - 1);
  const int s0 = (kb / STAGE_KEYS) * STAGE_KEYS;
  const int num_stages = (ke - s0 + STAGE_KEYS - 1) / STAGE_KEYS;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, WARPS); }
    *abort_flag = 0;
    *last_flag = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  __syncthreads();  // the barriers stand; nothing slow has been waited for yet
  // The producer needs the page numbers only and starts to stream as soon as it has them; the
  // consumers load the query tile meanwhile and meet among themselves.
  const bool newest_block = item_index == first_item + nsplits - 1;  // this block's keys end with the request's newest
  const int* table = nullptr;
  int streamed = 0;
  if (warp == WARPS) {
    table = cache_table(a.block_table + (size_t)req * a.table_stride, table_s, s0, ke, ps, lane, 32);
    __syncwarp();
    // Of the cache, only the request's newest row (key ke - 1 of its last item) is written in this
    // step; every older row was written by steps that ended before this step's description was
    // copied to the device.  So the first stages are on their way before the kernel in front of
    // this one has finished, all but the stage that holds the newest row.
    const bool newest_here = newest_block;
    streamed = min(STAGES, num_stages - ((newest_here && !a.fresh) ? 1 : 0));  // folded in: the stale row is overwritten in shared memory
    stream_kv(a.k_cache, a.v_cache, table, kvh, a.nkv, ps, kb, ke, s0,
              streamed, STAGES, stage_mem, full, empty, abort_flag, a.status, lane);
  }
  pdl_wait();
  if (warp < WARPS) {
    if (!a.fresh) {
      for (int i = tid; i < 16 * (HD / 8); i += WARPS * 32) {  // the query tile, 16 bytes at a time
        const int g = i / (HD / 8), c = i % (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (g < rows) v = *reinterpret_cast<const uint4*>(a.q + (size_t)t * a.q_stride + (size_t)(kvh * G + row0 + g) * HD + c * 8);
        *reinterpret_cast<uint4*>(q_s + g * QS + c * 8) = v;
      }
    } else if constexpr ((HD & (HD - 1)) == 0) {
      // the raw query rows, normalised and rotated on their way in: HD / 16 lanes per head
      constexpr int LPH = HD / 16;
      int pos = a.positions[t];
      pos = pos < 0 ? 0 : (pos >= a.max_pos ? a.max_pos - 1 : pos);
      const float* angles = a.cos_sin + (size_t)pos * HD;
      const int sub = lane % LPH;
      const unsigned head_lanes = (LPH == 32 ? 0xffffffffu : ((1u << LPH) - 1u)) << (lane - sub);
      for (int g0 = 0; g0 < 16; g0 += WARPS * 32 / LPH) {  // whole warps walk the rows together: the shuffles want every lane of a head
        const int g = g0 + tid / LPH;
        uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
        if (g < rows) fresh_row(a.q + (size_t)t * a.q_stride + (size_t)(kvh * G + row0 + g) * HD, a.q_norm_w, angles, sub, head_lanes, a.eps, lo, hi);
        if (g < 16) {
          *reinterpret_cast<uint4*>(q_s + g * QS + sub * 8) = lo;
          *reinterpret_cast<uint4*>(q_s + g * QS + HD / 2 + sub * 8) = hi;
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(WARPS * 32) : "memory");  // the four consumer warps: every path reaches it
  }

  float o[HD / 8][4];
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  if (warp == WARPS) {
    // ------------------------------------------------------------------ producer
    stream_kv(a.k_cache, a.v_cache, table, kvh, a.nkv, ps, kb, ke, s0,
              num_stages, STAGES, stage_mem, full, empty, abort_flag, a.status, lane, streamed);
  } else {
    // ------------------------------------------------------------------ consumers
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
      ldmatrix_x4(qf[ks], smem_u32(q_s + ((lane & 7) + ((lane >> 3) & 1) * 8) * QS + ks * 16 + (lane >> 4) * 8));
    for (int it = 0; it < num_stages; ++it) {
      const int slot = it % STAGES;
      if (!__all_sync(0xffffffffu, mbar_wait(full + slot, (it / STAGES) & 1, abort_flag, a.status))) break;  // the whole warp or nobody
      const int k0 = s0 + it * STAGE_KEYS + warp * TILE;
      if (k0 < ke && k0 + TILE > kb) {
        const __nv_bfloat16* kt = stage_mem + slot * STAGE_ELEMS + warp * TILE * HD;
        __nv_bfloat16* vt = stage_mem + slot * STAGE_ELEMS + STAGE_KEYS * HD + warp * TILE * HD;
        if (k0 < kb || k0 + TILE > ke) zero_value_rows(vt, k0, kb, ke, lane);
        if constexpr ((HD & (HD - 1)) == 0) {
          if (a.fresh && newest_block && ke - 1 >= k0 && ke - 1 < k0 + TILE) {
            // this warp's 16 keys include the request's newest one, which no kernel has made yet: the first
            // HD / 16 lanes make it from the raw projection, for this stage and for the cache
            constexpr int LPH = HD / 16;
            if (lane < LPH) {
              const int i = ke - 1 - k0;  // row in the sub-tile
              int pos = a.positions[t];
              pos = pos < 0 ? 0 : (pos >= a.max_pos ? a.max_pos - 1 : pos);
              const unsigned head_lanes = LPH == 32 ? 0xffffffffu : ((1u << LPH) - 1u);
              const __nv_bfloat16* raw = a.q + (size_t)t * a.q_stride;
              uint4 lo, hi;
              fresh_row(raw + (size_t)(a.nh + kvh) * HD, a.k_norm_w, a.cos_sin + (size_t)pos * HD, lane, head_lanes, a.eps, lo, hi);
              const __nv_bfloat16* vraw = raw + (size_t)(a.nh + a.nkv + kvh) * HD;
              const uint4 vlo = *reinterpret_cast<const uint4*>(vraw + lane * 8), vhi = *reinterpret_cast<const uint4*>(vraw + HD / 2 + lane * 8);
              __nv_bfloat16* ktw = const_cast<__nv_bfloat16*>(kt);
              *reinterpret_cast<uint4*>(ktw + tile_elem(i, lane * 8, xmask)) = lo;
              *reinterpret_cast<uint4*>(ktw + tile_elem(i, HD / 2 + lane * 8, xmask)) = hi;
              *reinterpret_cast<uint4*>(vt + tile_elem(i, lane * 8, xmask)) = vlo;
              *reinterpret_cast<uint4*>(vt + tile_elem(i, HD / 2 + lane * 8, xmask)) = vhi;
              const int slot = a.slots[t];
              if (blockIdx.z == 0 && slot >= 0) {  // one block per (request, kv head) writes the cache
                const long long tile = cache_tile(slot / ps, kvh, a.nkv, ps, HD);
                const int r = slot % ps;
                *reinterpret_cast<uint4*>(a.k_cache_w + tile + cache_offset<__nv_bfloat16>(r, lane * 8, ps, HD)) = lo;
                *reinterpret_cast<uint4*>(a.k_cache_w + tile + cache_offset<__nv_bfloat16>(r, HD / 2 + lane * 8, ps, HD)) = hi;
                *reinterpret_cast<uint4*>(a.v_cache_w + tile + cache_offset<__nv_bfloat16>(r, lane * 8, ps, HD)) = vlo;
                *reinterpret_cast<uint4*>(a.v_cache_w + tile + cache_offset<__nv_bfloat16>(r, HD / 2 + lane * 8, ps, HD)) = vhi;
              }
            }
            __syncwarp();
          }
        }
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          uint32_t b[4];
          ldmatrix_x4(b, smem_u32(kt + tile_elem((lane & 7) + (lane >> 4) * 8, ks * 16 + ((lane >> 3) & 1) * 8, xmask)));
          mma_bf16_16816(s[0], qf[ks], b[0], b[1]);
          mma_bf16_16816(s[1], qf[ks], b[2], b[3]);
        }
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = k0 + nt * 8 + (lane & 3) * 2 + (e & 1);
            const float v = (key >= kb && key < ke) ? s[nt][e] * a.scale_log2 : -INFINITY;
            s[nt][e] = v;
            tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
          }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          float mx = tile_max[r];
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
          const float m_new = fmaxf(m_run[r], mx);  // finite: the tile holds at least one visible key
          corr[r] = exp2f(m_run[r] - m_new);
          m_run[r] = m_new;
          l_run[r] *= corr[r];
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[nt][e] = exp2f(s[nt][e] - m_run[e >> 1]);
            l_run[e >> 1] += s[nt][e];
          }
        uint32_t pf[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]), pack_bf16(s[1][0], s[1][1]),
                          pack_bf16(s[1][2], s[1][3])};
#pragma unroll
        for (int j = 0; j < HD / 8; j += 2) {
          o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1];
          o[j + 1][0] *= corr[0]; o[j + 1][1] *= corr[0]; o[j + 1][2] *= corr[1]; o[j + 1][3] *= corr[1];
          uint32_t b[4];
          ldmatrix_x4_trans(b, smem_u32(vt + tile_elem((lane & 7) + ((lane >> 3) & 1) * 8, j * 8 + (lane >> 4) * 8, xmask)));
          mma_bf16_16816(o[j], pf, b[0], b[1]);
          mma_bf16_16816(o[j + 1], pf, b[2], b[3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty + slot);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
  }
  __syncthreads();  // every stage has been read: the ring becomes the merge buffer
  if (*abort_flag) {  // a wait gave up: let copies in flight land before the block leaves
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
    return;
  }
  float* o_s = reinterpret_cast<float*>(smem_raw);  // [WARPS][16][OS]
  if (warp < WARPS) {
    const int r = lane >> 2, c = (lane & 3) * 2;
    if ((lane & 3) == 0) {
      m_s[warp * 16 + r] = m_run[0]; m_s[warp * 16 + r + 8] = m_run[1];
      l_s[warp * 16 + r] = l_run[0]; l_s[warp * 16 + r + 8] = l_run[1];
    }
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) {
      *reinterpret_cast<float2*>(o_s + (warp * 16 + r) * OS + j * 8 + c) = make_float2(o[j][0], o[j][1]);
      *reinterpret_cast<float2*>(o_s + (warp * 16 + r + 8) * OS + j * 8 + c) = make_float2(o[j][2], o[j][3]);
    }
  }
  __syncthreads();
  const size_t part_row = ((size_t)item_index * a.nkv + kvh) * G + row0;  // + g
  for (int idx = tid; idx < rows * HD; idx += THREADS) {
    const int g = idx / HD, d = idx % HD;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) mx = fmaxf(mx, m_s[w * 16 + g]);
    float acc = 0.f, sum = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float f = exp2f(m_s[w * 16 + g] - mx);  // a warp that saw no key has max -inf: weight 0
      acc += o_s[(w * 16 + g) * OS + d] * f;
      sum += l_s[w * 16 + g] * f;
    }
    if (nsplits == 1) {
      a.out[(size_t)t * a.nh * HD + (size_t)(kvh * G + row0 + g) * HD + d] = __float2bfloat16_rn(acc / sum);
    } else {
      a.part_o[(part_row + g) * HD + d] = acc;
      if (d == 0) { a.part_ml[(part_row + g) * 2] = mx; a.part_ml[(part_row + g) * 2 + 1] = sum; }
    }
  }
  if (nsplits == 1) return;

  // the block that arrives last for this (request, kv head, row tile) merges the request's items
  __syncthreads();
  int* counter = a.counters + ((size_t)first_item * a.nkv + kvh) * gridDim.z + blockIdx.z;
  if (tid == 0) *last_flag = (arrive_acq_rel(counter) == nsplits - 1);
  __syncthreads();
  if (!*last_flag) return;
  if (nsplits <= MAX_SPLITS) {
    // 1) every item's (max, sum) into shared memory, one load per thread at a time
    float* ml = o_s;                       // [nsplits][16][2]
    float* weight = o_s + MAX_SPLITS * 32;  // [nsplits][16]
    for (int idx = tid; idx < nsplits * rows; idx += THREADS) {
      const int s = idx / rows, g = idx % rows;
      const size_t pr = ((size_t)(first_item + s) * a.nkv + kvh) * G + row0 + g;
      ml[(s * 16 + g) * 2] = __ldcg(a.part_ml + pr * 2);
      ml[(s * 16 + g) * 2 + 1] = __ldcg(a.part_ml + pr * 2 + 1);
    }
    __syncthreads();
    // 2) eight lanes per row turn them into the items' weights exp2(m_s - m) / sum (whole warps
    //    run the shuffles; lanes of rows that do not exist idle along)
    if (warp < 4) {
      const int g = tid >> 3, sub = tid & 7;
      const int n = g < rows ? nsplits : 0;
      float mx = -INFINITY, sum = 0.f;
      for (int s = sub; s < n; s += 8) mx = fmaxf(mx, ml[(s * 16 + g) * 2]);
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      for (int s = sub; s < n; s += 8) {
        const float w = exp2f(ml[(s * 16 + g) * 2] - mx);
        weight[s * 16 + g] = w;
        sum += ml[(s * 16 + g) * 2 + 1] * w;
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      const float inv = 1.f / sum;
      for (int s = sub; s < n; s += 8) weight[s * 16 + g] *= inv;
    }
    __syncthreads();
    // 3) the weighted sum of the items' outputs, four columns per thread, eight loads in flight
    for (int idx = tid; idx < rows * (HD / 4); idx += THREADS) {
      const int g = idx / (HD / 4), d = (idx % (HD / 4)) * 4;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s0 = 0; s0 < nsplits; s0 += 8) {
        float4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          v[j] = s0 + j < nsplits
                     ? __ldcg(reinterpret_cast<const float4*>(a.part_o + (((size_t)(first_item + s0 + j) * a.nkv + kvh) * G + row0 + g) * HD + d))
                     : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float w = s0 + j < nsplits ? weight[(s0 + j) * 16 + g] : 0.f;
          acc.x += v[j].x * w; acc.y += v[j].y * w; acc.z += v[j].z * w; acc.w += v[j].w * w;
        }
      }
      __nv_bfloat16* dst = a.out + (size_t)t * a.nh * HD + (size_t)(kvh * G + row0 + g) * HD + d;
      *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
    }
  } else {
    for (int idx = tid; idx < rows * HD; idx += THREADS) {
      const int g = idx / HD, d = idx % HD;
      float mx = -INFINITY;
      for (int s = 0; s < nsplits; ++s)
        mx = fmaxf(mx, __ldcg(a.part_ml + ((((size_t)(first_item + s) * a.nkv + kvh) * G + row0 + g) * 2)));
      float acc = 0.f, sum = 0.f;
      for (int s = 0; s < nsplits; ++s) {
        const size_t pr = ((size_t)(first_item + s) * a.nkv + kvh) * G + row0 + g;
        const float f = exp2f(__ldcg(a.part_ml + pr * 2) - mx);
        acc += __ldcg(a.part_o + pr * HD + d) * f;
        sum += __ldcg(a.part_ml + pr * 2 + 1) * f;
      }
      a.out[(size_t)t * a.nh * HD + (size_t)(kvh * G + row0 + g) * HD + d] = __float2bfloat16_rn(acc / sum);
    }
  }
  if (tid == 0) *counter = 0;
}

constexpr size_t decode_smem_bytes() {
  return 128 + (size_t)STAGES * 2 * STAGE_KEYS * HD * 2 + 16 * QS * 2 + 2 * WARPS * 16 * 4 + 2 * STAGES * 8 + 16 + TABLE_CACHE * 4;
}
static_assert((size_t)WARPS * 16 * OS * 4 <= (size_t)STAGES * 2 * STAGE_KEYS * HD * 2, "merge buffer must fit in the ring");
static_assert((size_t)MAX_SPLITS * 48 * 4 <= (size_t)STAGES * 2 * STAGE_KEYS * HD * 2, "split weights must fit in the ring");

}  // namespace tb

extern "C" {

int tb_attention_decode_head_dim() { return tb::HD; }

// items: [max_items, 6] int32 on the device (max_items <= 65535); grid = (nkv, max_items, ceil(G / 16)).
int tb_attention_decode(void* stream, const void* q, int q_stride, const void* k_cache, const void* v_cache,
                        const int* block_table, int table_stride, const int* items, const int* num_items,
                        int max_items, void* out, float* part_o, float* part_ml, int* counters, int* status, int nh,
                        int nkv, int page_size, float scale, int fresh, const float* q_norm_w, const float* k_norm_w,
                        const float* cos_sin, const int* positions, const int* slots, float eps, int max_pos) {
  if (max_items <= 0) return 0;
  if (max_items > 65535) return TB_ERR_BAD_SIZE;
  if (fresh && ((tb::HD & (tb::HD - 1)) != 0 || !cos_sin || !positions || !slots || max_pos <= 0)) return TB_ERR_BAD_SIZE;
  if (nkv <= 0 || nh % nkv != 0 || page_size <= 0) return TB_ERR_BAD_SIZE;
  if (!(page_size == 1 || page_size == 2 || page_size == 4 || page_size == 8 || page_size % 16 == 0))
    return TB_ERR_BAD_SIZE;
  tb::DecodeArgs a;
  a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride;
  a.k_cache = (const __nv_bfloat16*)k_cache; a.v_cache = (const __nv_bfloat16*)v_cache;
  a.block_table = block_table; a.table_stride = table_stride;
  a.items = items; a.num_items = num_items;
  a.out = (__nv_bfloat16*)out; a.part_o = part_o; a.part_ml = part_ml; a.counters = counters; a.status = status;
  a.nh = nh; a.nkv = nkv; a.page_size = page_size;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.fresh = fresh; a.q_norm_w = q_norm_w; a.k_norm_w = k_norm_w; a.cos_sin = cos_sin; a.positions = positions; a.slots = slots;
  a.k_cache_w = (__nv_bfloat16*)k_cache; a.v_cache_w = (__nv_bfloat16*)v_cache; a.eps = eps; a.max_pos = max_pos;
  static bool configured = false;
  const size_t smem = tb::decode_smem_bytes();
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(tb::attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    // All of an SM's memory as shared memory: two blocks are to fit on an SM whatever split the kernel in front
    // left there (with the default, an SM that still had the split of a kernel with little shared memory took
    // one block, and a step's attention at 16 or 32 requests ran in two rounds, 73 us instead of 47); the
    // keys and values come by bulk copies, which do not pass through the L1.
    e = cudaFuncSetAttribute(tb::attention_decode_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int G = nh / nkv;
  dim3 grid(nkv, max_items, (G + 15) / 16);
  return tb::launch(tb::attention_decode_kernel, grid, dim3(tb::THREADS), smem, stream, a);
}

}  // extern "C"
