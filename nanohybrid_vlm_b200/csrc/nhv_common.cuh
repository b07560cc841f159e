// Shared helpers for the sm_100a kernels of this engine.
//
// Every exported function is `extern "C"`, takes raw device pointers, sizes and the
// CUDA stream to launch on, allocates nothing and returns 0 or an error code; the text
// of the last error is read with nhv_last_error().  Python binds them with ctypes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define NHV_API extern "C" __attribute__((visibility("default")))

enum NhvDtype { NHV_F32 = 0, NHV_BF16 = 1 };

#ifdef NHV_OWN_ERROR_TEXT
// A file compiled into a library of its own (tests do that) keeps the text of its last error itself and exports
// nhv_last_error() for it.
#include <stdarg.h>
static char nhv_own_error_text[512];
static void nhv_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(nhv_own_error_text, sizeof(nhv_own_error_text), fmt, ap);
  va_end(ap);
}
NHV_API const char* nhv_last_error() { return nhv_own_error_text; }
#else
// Defined in elementwise.cu.
void nhv_set_error(const char* fmt, ...);
#endif

#define NHV_REQUIRE(cond, ...)                                  \
  do {                                                          \
    if (!(cond)) {                                              \
      nhv_set_error(__VA_ARGS__);                               \
      return 1;                                                 \
    }                                                           \
  } while (0)

#define NHV_CHECK_LAUNCH(name)                                                        \
  do {                                                                                \
    cudaError_t e_ = cudaPeekAtLastError();                                           \
    if (e_ != cudaSuccess) {                                                          \
      nhv_set_error("%s: launch failed: %s", name, cudaGetErrorString(e_));           \
      return 2;                                                                       \
    }                                                                                 \
  } while (0)

#define NHV_CUDA(call, name)                                                          \
  do {                                                                                \
    cudaError_t e_ = (call);                                                          \
    if (e_ != cudaSuccess) {                                                          \
      nhv_set_error("%s: %s", name, cudaGetErrorString(e_));                          \
      return 2;                                                                       \
    }                                                                                 \
  } while (0)

// Programmatic dependent launch.  Every kernel of this library is launched with the attribute that
// lets it start while the kernel before it in the stream is still running, and every kernel begins
// with pdl_prologue(): it lets the kernel after it start likewise, then waits until the kernel before
// it has completed and its writes are visible.  Nothing may be read that another kernel writes, and
// nothing written at all, before that wait; what a kernel does before it (fetching weights) overlaps
// with its predecessor's tail.  Launch latency and pipeline fill leave the critical path this way.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_prologue() {
  pdl_launch_dependents();
  pdl_wait();
}

template <typename... KArgs, typename... Args>
inline cudaError_t nhv_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Round a float to the storage type and back: the value the next op would read.
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32<T>(from_f32<T>(v)); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
