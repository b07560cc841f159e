// nhv_no_alloc.h: the one entry point of libnhv_kernels that allocates nothing.
//
// This entry point has no counterpart in the reference (Bluexvy/NanoHybrid-VLM); it exists for callers of
// this library that are not allowed to allocate device memory.  Such callers are real: a host program that
// has handed every byte of the GPU to its own pool and treats any cudaMalloc as a bug; code that runs at a
// point where an allocation would stall the whole device (cudaMalloc and cudaFree synchronise it) and so
// break a latency budget; a plugin loaded into a process whose owner forbids allocations after start-up.
// The ordinary entry point, nhv_gemm_stream_k, asks its caller for two scratch buffers (partial sums of the
// output tiles that two thread blocks share, and one arrival counter per tile).  This variant brings its
// own: a fixed array of 1.27 MiB (1.25 MiB of partial sums for up to 160 thread blocks, 16 KiB for 4,096
// tile counters) that lives inside the library.  Every GPU that loads the library holds that array until the
// process exits, whether or not this function is ever called.
//
// What it computes is exactly what nhv_gemm_stream_k computes: y[M, N] = x[M, K] * W[N, K]^T in bfloat16 for
// M <= 16 rows of x (mode 0: y bfloat16; mode 1: y float32, rounded through bfloat16; mode 2: W holds gate
// rows [0, N) and up rows [up_row_offset, up_row_offset + N) and y = silu(x Wg^T) * (x Wu^T)).  The caller
// still passes x, W and y; they must be device memory, x and W 16-byte aligned, K and lda multiples of 8.
//
// Limits and rules:
//  * N may make at most 4,096 output tiles: N <= 262,144 in modes 0 and 1, N <= 131,072 in mode 2.  A larger
//    N is refused with an error (return value 1, text from nhv_last_error()); nothing is launched.
//  * The function calls no cudaMalloc, cudaFree or any other allocating routine, of CUDA or of a framework.
//  * The first call on a device sets the variant up for that device: with that device current it looks up
//    the array's device address (cudaGetSymbolAddress), reads the number of SMs and clears the counters on
//    the given stream.  Make that first call before any stream capture begins.
//  * All calls share the one array, and it keeps what the last call left in it.  The partial sums need no
//    clearing (every block writes its slot before any block reads it); the counters must be zero when a call
//    starts, and every call that runs to completion leaves them zero.  Two calls that overlap on the GPU
//    (different streams, or two host threads) race on the array and give wrong results: serialise them.
//  * Host threads: the per-device set-up is guarded, so first calls from several threads are safe; the calls
//    themselves are safe from several threads only in the sense above (their GPU work must not overlap).
//  * Returns 0 on success, 1 for a refused argument, 2 for a CUDA error.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

__attribute__((visibility("default"))) int nhv_gemm_stream_k_no_alloc(void* y, const void* x, const void* W, int M, int N, int K, int lda, int ldc, int mode,
                               int up_row_offset, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
