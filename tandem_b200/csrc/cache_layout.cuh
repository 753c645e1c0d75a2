// Where element (row r of a page, dim d) of one (page, kv head) tile lives.
//
// The cache is [pages][kv heads] tiles of page_size rows x head_dim elements.  For 16-bit caches
// whose head_dim is a multiple of 64 a tile is stored the way the tensor cores want to read it
// from shared memory: as head_dim/64 column blocks of [page_size rows][64 elements = 128 bytes],
// the eight 16-byte chunks of each 128-byte row XOR-ed with (row mod 8) (the "128-byte swizzle").
// A plain bulk copy of the tile (one contiguous block of global memory) then lands in shared
// memory ready for conflict-free ldmatrix reads, with no tensor map and no per-thread shuffling.
// All other caches (float32, or other head sizes) keep plain [row][dim] tiles.
//
// Only kernels of this package read or write the cache, all through these functions;
// tandem_b200/cache/layout.py is the same map in Python for tests and tools.
#pragma once

namespace tb {

template <typename T>
__host__ __device__ __forceinline__ bool cache_swizzled(int hd) {
  return sizeof(T) == 2 && (hd & 63) == 0;
}

// element offset inside the tile
template <typename T>
__device__ __forceinline__ int cache_offset(int r, int d, int page_size, int hd) {
  if (!cache_swizzled<T>(hd)) return r * hd + d;
  const int block = d >> 6, dd = d & 63;
  return block * page_size * 64 + r * 64 + ((((dd >> 3) ^ (r & 7)) << 3) | (dd & 7));
}

// element offset of the tile of (page, kv head)
__device__ __forceinline__ long long cache_tile(long long page, int kvh, int nkv, int page_size, int hd) {
  return ((page * nkv + kvh) * page_size) * (long long)hd;
}

}  // namespace tb
