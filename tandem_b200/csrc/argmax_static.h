// tb_argmax_static: row-wise argmax that allocates nothing.
//
// This entry point has no counterpart in 12vivi/tandem.  It exists for programs that want the
// engine's argmax kernel but are not allowed to ask the CUDA allocator for memory at the moment
// they call it: a serving loop that gave every free byte of the device to its own pool at start-up,
// an embedder whose memory budget was fixed before this library was loaded, or code that runs
// where a cudaMalloc would stall or fail.  The regular entry point (tb_argmax_split) needs two
// small scratch arrays that its caller allocates; this variant keeps them inside the library, in
// a file-scope __device__ array, so the caller passes only the input and the output.
//
// Limits and rules:
//  * At most TB_ARGMAX_STATIC_MAX_ROWS rows per call (the scratch holds 16 bytes per row, 64 KiB
//    in all; every GPU that loads the library holds that much until the process exits).  More rows
//    are refused with TB_ERR_TOO_LARGE and nothing is launched.
//  * The first call on a device looks up the device address of the scratch
//    (cudaGetSymbolAddress, with that device current) and keeps it.  Make that first call outside
//    any stream capture.
//  * All calls on a device share the one scratch array.  Each call clears it on the given stream
//    before the kernel runs, so a call never sees what an earlier call left; but two calls whose
//    kernels overlap on the GPU (different streams, no dependency between them) race on it.
//    Serialise them.
//  * No cudaMalloc, cudaFree or any allocating routine is called, here or in the kernel.
#pragma once

#define TB_ARGMAX_STATIC_MAX_ROWS 4096
#define TB_ERR_TOO_LARGE 10003

#ifdef __cplusplus
extern "C" {
#endif

// logits [R, V] float32 (device), out [R] int32 (device): index of the largest value of each row,
// the lowest index among equals.  `chunks` blocks work on each row (1 <= chunks; a good choice is
// about 300 / R, at most V / 2048).  Returns 0, TB_ERR_BAD_SIZE, TB_ERR_TOO_LARGE or a CUDA error code.
int tb_argmax_static(void* stream, const float* logits, int* out, int R, int V, int chunks);

#ifdef __cplusplus
}
#endif
