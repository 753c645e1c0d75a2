// What the tensor-core attention kernels share: the compile-time head size and the tile geometry
// that follows from it, addressing inside a shared-memory tile, and the producer warp that
// streams a request's keys and values from its pages into a ring of shared-memory stages.
//
// A stage holds STAGE_KEYS = 64 keys, K then V, each laid out like the rows of a cache tile
// (cache_layout.cuh): when the head size is a multiple of 64, [8 row groups][column block][8 rows]
// [64 elements] with 128-byte rows swizzled, else plain [64 rows][head size].  A sub-tile of 16 keys
// is two row groups.  Copies are 1-D bulk copies (the TMA unit) that complete on the stage's
// mbarrier; with pages of 8 keys or more one copy brings all rows that a page has in the stage.
#pragma once

#include "cache_layout.cuh"
#include "common.cuh"
#include "sm100_primitives.cuh"

#ifndef TB_HD
#error "compile with -DTB_HD=<head size, a multiple of 16>"
#endif

namespace tb {

constexpr int HD = TB_HD;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 up to 256");
constexpr bool SWZ = (HD % 64 == 0);
constexpr int NB = SWZ ? HD / 64 : 1;  // column blocks of a cache tile
constexpr int BW = SWZ ? 64 : HD;      // elements per row of a column block
constexpr int TILE = 16;               // keys per sub-tile
constexpr int STAGE_KEYS = 64;
constexpr int STAGE_ELEMS = 2 * STAGE_KEYS * HD;  // K and V of one stage
constexpr int STATUS_BAD_PAGE = 2;
constexpr int TABLE_CACHE = 512;  // page numbers a block keeps in shared memory

__device__ __forceinline__ int tile_elem(int i, int d, int xmask) {  // inside one sub-tile of 16 rows
  if (!SWZ) return i * HD + d;
  const int blk = d >> 6, dd = d & 63;
  return (((i >> 3) * NB + blk) * 8 + (i & 7)) * 64 + ((((dd >> 3) ^ (i & xmask)) << 3) | (dd & 7));
}

__device__ __forceinline__ bool page_size_supported(int ps) {
  return ps == 1 || ps == 2 || ps == 4 || ps == 8 || (ps & 15) == 0;
}

// Copy the page numbers of keys [s0, ke) into shared memory (all threads; the caller synchronises
// afterwards) and return a pointer that is indexed like the global table.  Ranges that do not fit
// keep reading the global table.
__device__ __forceinline__ const int* cache_table(const int* table, int* table_s, int s0, int ke, int ps, int tid,
                                                  int threads) {
  const int first = s0 / ps, count = (ke + ps - 1) / ps - first;
  if (count > TABLE_CACHE) return table;
  for (int i = tid; i < count; i += threads) table_s[i] = table[first + i];
  return table_s - first;
}

// The producer warp: fills stage after stage with keys [s0 + it*64, +64) of the request whose block
// table is `table`, restricted to [kb, ke).  A piece is the rows of one page that fall into the
// stage; with at most 16 pieces per stage (pages of 4 keys or more) lane i brings the keys of
// piece i and lane 16 + i its values, else every lane brings both of its pieces, 32 pieces a
// round.  With swizzled tiles and pages of 8 keys or more a piece is copied in whole row groups
// (rows of a group that lie outside [kb, ke) come along; the consumers mask them and clear their
// values), else row by row.  Pages that were given back are not copied.
//
// One warp's chain of dependent instructions is what bounds a kernel that waits for its stages,
// so everything that does not need the stage itself (page lookup, addresses, byte counts) is done
// *before* the wait for the stage to be free, stages that lie wholly inside [kb, ke) skip the
// byte count's reduction, and all lanes wait on the barrier themselves (one vote, no broadcast).  Two warps
// may share the work: each takes the stages first, first + step, ...
__device__ __forceinline__ void stream_kv(const __nv_bfloat16* k_cache, const __nv_bfloat16* v_cache, const int* table,
                                          int kvh, int nkv, int ps, int kb, int ke, int s0, int num_stages,
                                          int stages, __nv_bfloat16* stage_mem, uint64_t* full, uint64_t* empty,
                                          volatile int* abort_flag, int* status, int lane, int first = 0, int step = 1) {
  const int piece = ps % 64 == 0 ? 64 : ps % 32 == 0 ? 32 : ps % 16 == 0 ? 16 : ps;  // divides the page and the stage
  const int pieces = STAGE_KEYS / piece;
  const bool groups = SWZ && ps >= 8;
  const bool whole_rows = groups || !SWZ;  // rows (or row groups) are contiguous in the page as in the stage
  const int ps_shift = (ps & (ps - 1)) == 0 ? __ffs(ps) - 1 : -1;
  const long long tile_elems = (long long)ps * HD, page_elems = tile_elems * nkv, head_off = (long long)kvh * tile_elems;
  if (pieces <= 16) {
    const int my_piece = lane & 15;
    const __nv_bfloat16* cache = lane < 16 ? k_cache : v_cache;
    const int side = lane < 16 ? 0 : STAGE_KEYS * HD;  // keys, then values
    for (int it = first; it < num_stages; it += step) {
      const int slot = it % stages;
      const int base = s0 + it * STAGE_KEYS;
      const int kp = base + my_piece * piece;
      const bool inside = base >= kb && base + STAGE_KEYS <= ke;  // every row of the stage is wanted
      const bool mine = my_piece < pieces && kp < ke && kp + piece > kb;
      int page = -1;
      if (mine) {
        page = table[ps_shift >= 0 ? kp >> ps_shift : kp / ps];
        if (page < 0) atomicExch(status, STATUS_BAD_PAGE);
      }
      int lo = 0, hi = 0;
      if (page >= 0) {
        lo = max(0, kb - kp);
        hi = min(piece, ke - kp);
        if (groups) { lo &= ~7; hi = (hi + 7) & ~7; }
      }
      const int n = hi - lo;
      uint32_t bytes = (uint32_t)STAGE_ELEMS * 2u;
      if (!inside || __any_sync(0xffffffffu, mine && page < 0)) {
        bytes = (uint32_t)n * HD * 2u;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) bytes += __shfl_xor_sync(0xffffffffu, bytes, o);
      }
      const int r0 = (ps_shift >= 0 ? kp & (ps - 1) : kp % ps) + lo, i0 = kp - base + lo;  // first row in the page, in the stage
      const long long src = (long long)page * page_elems + head_off;
      __nv_bfloat16* dst = stage_mem + slot * STAGE_ELEMS + side;
      // all lanes leave together or not at all: a lane that gave up alone would leave the others at the __syncwarp below
      if (it >= stages && !__all_sync(0xffffffffu, mbar_wait(empty + slot, ((it / stages) & 1) ^ 1, abort_flag, status))) break;
      if (lane == 0) mbar_arrive_expect_tx(full + slot, bytes);
      __syncwarp();
      if (n > 0) {
        if (whole_rows) {
          bulk_load(dst + i0 * HD, cache + src + (long long)r0 * HD, n * HD * 2, full + slot);
        } else {  // a page of fewer than 8 rows is one short group: [column block][rows][64]
#pragma unroll
          for (int b = 0; b < NB; ++b)
            bulk_load(dst + (((i0 >> 3) * NB + b) * 8 + (i0 & 7)) * 64, cache + src + ((long long)b * ps + r0) * 64, n * 128, full + slot);
        }
      }
    }
    return;
  }
  // pages of one or two keys: 32 or 64 pieces a stage, every lane brings keys and values of its pieces
  bool alive = true;
  for (int it = first; it < num_stages && alive; it += step) {
    const int slot = it % stages;
    if (it >= stages) {
      if (lane == 0) alive = mbar_wait(empty + slot, ((it / stages) & 1) ^ 1, abort_flag, status);
      alive = __shfl_sync(0xffffffffu, alive, 0);
      if (!alive) break;
    }
    __nv_bfloat16* ks = stage_mem + slot * STAGE_ELEMS;
    __nv_bfloat16* vs = ks + STAGE_KEYS * HD;
    const int base = s0 + it * STAGE_KEYS;
    for (int p0 = 0; p0 < pieces; p0 += 32) {
      const int kp = base + (p0 + lane) * piece;
      const bool mine = (p0 + lane) < pieces && kp < ke && kp + piece > kb;
      int page = -1;
      if (mine) {
        page = table[kp / ps];
        if (page < 0) atomicExch(status, STATUS_BAD_PAGE);
      }
      int lo = 0, hi = 0;
      if (page >= 0) {
        lo = max(0, kb - kp);
        hi = min(piece, ke - kp);
      }
      const int n = hi - lo;
      uint32_t bytes = 2u * (uint32_t)n * HD * 2u;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) bytes += __shfl_xor_sync(0xffffffffu, bytes, o);
      const bool last_round = p0 + 32 >= pieces;
      if (lane == 0) {  // one arrival per stage: the last round arrives, earlier rounds only add bytes
        if (last_round) mbar_arrive_expect_tx(full + slot, bytes);
        else if (bytes) asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(full + slot)), "r"(bytes) : "memory");
      }
      __syncwarp();
      if (n > 0) {
        const int r0 = kp % ps + lo, i0 = kp - base + lo;
        const long long tile = cache_tile(page, kvh, nkv, ps, HD);
        if (!SWZ) {
          bulk_load(ks + i0 * HD, k_cache + tile + (long long)r0 * HD, n * HD * 2, full + slot);
          bulk_load(vs + i0 * HD, v_cache + tile + (long long)r0 * HD, n * HD * 2, full + slot);
        } else {
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            const long long src = tile + ((long long)b * ps + r0) * 64;
            const int d = (((i0 >> 3) * NB + b) * 8 + (i0 & 7)) * 64;
            bulk_load(ks + d, k_cache + src, n * 128, full + slot);
            bulk_load(vs + d, v_cache + src, n * 128, full + slot);
          }
        }
      }
    }
  }
}

// Value rows of the sub-tile at keys k0..k0+15 whose keys lie outside [kb, ke) get zero weights,
// but may hold whatever shared memory held before (no copy filled them): make them zeros, not
// NaN.  One warp; the generic writes are fenced against the next bulk copy into the stage.
__device__ __forceinline__ void zero_value_rows(__nv_bfloat16* vt, int k0, int kb, int ke, int lane) {
  for (int i = lane; i < TILE * (HD / 8); i += 32) {
    const int row = i / (HD / 8), c = i % (HD / 8);
    if (k0 + row < kb || k0 + row >= ke)
      *reinterpret_cast<uint4*>(vt + (SWZ ? (((row >> 3) * NB + (c >> 3)) * 8 + (row & 7)) * 64 + (c & 7) * 8 : row * HD + c * 8)) = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async();
  __syncwarp();
}

}  // namespace tb
