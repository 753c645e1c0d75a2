// Where element (row r of a page, dim d) of one (page, kv head) tile lives.
//
// The cache is [pages][kv heads] tiles of page_size rows x head_dim elements.  For 16-bit caches
// whose head_dim is a multiple of 64 (and whose page size is below 8 or a multiple of 8) a tile is
// stored the way the tensor cores want to read it from shared memory: rows of 64 elements = 128
// bytes whose eight 16-byte chunks are XOR-ed with (row mod 8) (the "128-byte swizzle"), kept in
// groups of eight rows, [row group][head_dim/64 column blocks][8 rows][64 elements].  Any run of
// whole row groups is then one contiguous block of global memory: a single bulk copy brings 16, 32
// or 64 keys of a page into shared memory, ready for conflict-free ldmatrix reads and for the
// shared-memory descriptors of tcgen05 (8-row groups head_dim/64 * 1024 bytes apart, column blocks
// 1024 bytes apart), with no tensor map and no per-thread shuffling.  Pages of fewer than eight
// rows are one short group.  All other caches (float32, other head sizes) keep plain [row][dim] tiles.
//
// Only kernels of this package read or write the cache, all through these functions;
// tandem_b200/cache/layout.py is the same map in Python for tests and tools.
#pragma once

namespace tb {

template <typename T>
__host__ __device__ __forceinline__ bool cache_swizzled(int hd, int page_size) {
  return sizeof(T) == 2 && (hd & 63) == 0 && (page_size < 8 || (page_size & 7) == 0);
}

// element offset inside the tile
template <typename T>
__device__ __forceinline__ int cache_offset(int r, int d, int page_size, int hd) {
  if (!cache_swizzled<T>(hd, page_size)) return r * hd + d;
  const int block = d >> 6, dd = d & 63;
  const int rows = page_size < 8 ? page_size : 8;  // rows of a group
  const int group = page_size < 8 ? 0 : r >> 3, rr = page_size < 8 ? r : r & 7;
  return ((group * (hd >> 6) + block) * rows + rr) * 64 + ((((dd >> 3) ^ (r & 7)) << 3) | (dd & 7));
}

// element offset of the tile of (page, kv head)
__device__ __forceinline__ long long cache_tile(long long page, int kvh, int nkv, int page_size, int hd) {
  return ((page * nkv + kvh) * page_size) * (long long)hd;
}

}  // namespace tb
