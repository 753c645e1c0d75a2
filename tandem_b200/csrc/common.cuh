// Shared helpers of the sm_100a kernels: element types, warp and block reductions, launch checks.
//
// Every kernel file exports plain C functions (`extern "C" int tb_*`) that take raw device
// pointers, sizes and a stream, launch, and return the CUDA error code of the launch (0 = ok).
// The element type of activations and caches is chosen at run time by `dtype` (TB_F32 / TB_BF16);
// arithmetic inside the kernels is float32 whatever the storage type.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define TB_F32 0
#define TB_BF16 1

#define TB_ERR_BAD_DTYPE 10001
#define TB_ERR_BAD_SIZE 10002

namespace tb {

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Arrival on a counter that publishes what the arriving threads wrote before it and, for the thread
// that turns out to be last, makes visible what the earlier arrivals published: one acquire-release
// atomic instead of fence + atomic + fence (the caller synchronises its threads before and after).
__device__ __forceinline__ int arrive_acq_rel(int* counter) {
  int old;
  asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
  return old;
}

inline int launch_status() { return (int)cudaGetLastError(); }

// Programmatic dependent launch.  Every kernel of this package is launched with the attribute that
// lets it become resident while the kernel before it in the stream is still running, and calls
// pdl_wait() before it reads anything an earlier kernel wrote and before it writes anything at
// all; what it does before that (barrier set-up, tensor memory, prefetching weights, which no
// kernel writes) overlaps the tail of its predecessor.  pdl_launch_dependents() tells the
// scheduler that the kernel after this one may start to become resident.  TANDEM_PDL=0 turns
// the attribute off (the two instructions are then no-ops).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {  // two floats -> bfloat16 pair (lo in the low half)
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

inline bool pdl_enabled() {
  static const bool on = [] { const char* e = getenv("TANDEM_PDL"); return !(e && e[0] == '0'); }();
  return on;
}

template <typename... KArgs, typename... Args>
inline int launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, void* stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace tb

// `return <expression with T>` with T picked by a run-time dtype code.
#define TB_DISPATCH_DTYPE(dtype, ...)                         \
  do {                                                        \
    if ((dtype) == TB_F32) {                                  \
      using T = float;                                        \
      return __VA_ARGS__;                                     \
    } else if ((dtype) == TB_BF16) {                          \
      using T = __nv_bfloat16;                                \
      return __VA_ARGS__;                                     \
    } else {                                                  \
      return TB_ERR_BAD_DTYPE;                                \
    }                                                         \
  } while (0)
