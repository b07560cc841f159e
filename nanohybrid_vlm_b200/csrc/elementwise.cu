// Row-wise kernels: embedding gather, RMSNorm (plain, with fused residual add, with row
// gather), SiLU-and-multiply, and the error string shared by the whole library.
//
// Formulas follow nanovllm/layers/layernorm.py:16-40 (statistics in fp32, cast to the
// storage type, then multiply by the weight in the storage type; the residual sum is
// rounded once for the new residual while the norm uses the unrounded sum),
// nanovllm/layers/activation.py:9-11 and nanovllm/layers/embed_head.py:38.
#include <stdarg.h>
#include <string.h>

#include "nhv_common.cuh"

static thread_local char g_error[512] = "";

void nhv_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

NHV_API const char* nhv_last_error() { return g_error; }
NHV_API int nhv_abi_version() { return 1; }

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_kernel(T* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                             int width, int vocab) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  const T* src = table + (size_t)(ok ? id : 0) * width;
  T* dst = out + (size_t)t * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = ok ? src[c] : from_f32<T>(0.f);
}

NHV_API int nhv_embed(int dtype, void* out, const void* table, const int* ids, int n_tokens, int width, int vocab,
                      cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  NHV_REQUIRE(n_tokens > 0 && width > 0 && vocab > 0, "embed: bad sizes");
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == NHV_F32)
    nhv_launch(embed_kernel<float>, n_tokens, threads, 0, stream, (float*)out, (const float*)table, ids, width, vocab);
  else if (dtype == NHV_BF16)
    nhv_launch(embed_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (__nv_bfloat16*)out,
               (const __nv_bfloat16*)table, ids, width, vocab);
  else
    NHV_REQUIRE(false, "embed: unknown dtype %d", dtype);
  NHV_CHECK_LAUNCH("embed");
  return 0;
}

// ---------------------------------------------------------------- tokens handed from one step to the next
// token_ids[t] = chosen[feed_src[t]] where feed_src[t] >= 0: a step that was launched before the host read the tokens
// of the step before it takes them from that step's sampler output on the device.  Entries with feed_src[t] < 0 keep
// the value that the host wrote.  A source row beyond the step before, or a token outside the vocabulary (which no
// sampler writes), becomes token 0 rather than an index out of the embedding table.
__global__ void feed_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ feed_src,
                                   const int* __restrict__ chosen, int n_tokens, int n_chosen, int vocab) {
  pdl_prologue();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tokens) return;
  const int src = feed_src[t];
  if (src < 0) return;
  const int tok = src < n_chosen ? chosen[src] : 0;
  token_ids[t] = tok >= 0 && tok < vocab ? tok : 0;
}

NHV_API int nhv_feed_tokens(int* token_ids, const int* feed_src, const int* chosen, int n_tokens, int n_chosen, int vocab,
                            cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  NHV_REQUIRE(n_tokens > 0 && n_chosen > 0 && vocab > 0 && token_ids && feed_src && chosen, "feed_tokens: bad arguments");
  nhv_launch(feed_tokens_kernel, (n_tokens + 127) / 128, 128, 0, stream, token_ids, feed_src, chosen, n_tokens, n_chosen, vocab);
  NHV_CHECK_LAUNCH("feed_tokens");
  return 0;
}

// ---------------------------------------------------------------- RMSNorm
// One block per output row.  Row r reads source row rows[r] (or r when rows is null).
// residual != null: s = x + residual in fp32; if write_residual the rounded s replaces residual.
// The row of fp32 sums lives in shared memory between the two passes.
template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ out, const T* __restrict__ x, T* __restrict__ residual,
                               const T* __restrict__ w, const int* __restrict__ rows, int width, float eps,
                               int write_residual, float weight_offset) {
  extern __shared__ float row[];
  __shared__ float red[33];
  pdl_prologue();
  const int r = blockIdx.x;
  const size_t src = (size_t)(rows ? rows[r] : r) * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float s = to_f32<T>(x[src + c]);
    if (residual) {
      s += to_f32<T>(residual[src + c]);
      if (write_residual) residual[src + c] = from_f32<T>(s);
    }
    row[c] = s;
    ss = fmaf(s, s, ss);
  }
  const float total = block_sum(ss, red);
  const float rstd = 1.0f / sqrtf(total / (float)width + eps);
  T* dst = out + (size_t)r * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float n = round_to<T>(row[c] * rstd);
    dst[c] = from_f32<T>(n * (to_f32<T>(w[c]) + weight_offset));
  }
}

// bfloat16 rows of up to 8,192 elements (a multiple of 8): 16-byte loads and stores, the row's fp32 sums kept
// in registers between the statistics and the scaling, so every element is read once and written once.
constexpr int RN_THREADS = 256;

constexpr int RN_CHUNKS = 4;      // 16-byte chunks per thread

template <int RN_T>
__global__ void __launch_bounds__(RN_T) rmsnorm_bf16x8_kernel(
    __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ residual,
    const __nv_bfloat16* __restrict__ w, const int* __restrict__ rows, int width8, float eps, int write_residual,
    float weight_offset) {
  __shared__ float red[33];
  // the norm's weight is no kernel's output: fetch it while the kernel before this one is still running
  pdl_launch_dependents();
  uint4 wv[RN_CHUNKS];
#pragma unroll
  for (int i = 0; i < RN_CHUNKS; ++i) {
    const int c = threadIdx.x + i * RN_T;
    wv[i] = c < width8 ? reinterpret_cast<const uint4*>(w)[c] : make_uint4(0, 0, 0, 0);
  }
  pdl_wait();
  const int r = blockIdx.x;
  const size_t src = (size_t)(rows ? rows[r] : r) * width8;
  const uint4* x4 = reinterpret_cast<const uint4*>(x) + src;
  uint4* res4 = residual ? reinterpret_cast<uint4*>(residual) + src : nullptr;
  float s[RN_CHUNKS][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < RN_CHUNKS; ++i) {
    const int c = threadIdx.x + i * RN_T;
    if (c < width8) {
      const uint4 xv = x4[c];
      const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(&xv);
      if (res4) {
        const uint4 rv = res4[c];
        const __nv_bfloat16* rb = reinterpret_cast<const __nv_bfloat16*>(&rv);
        uint4 nv;
        __nv_bfloat16* nb = reinterpret_cast<__nv_bfloat16*>(&nv);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          s[i][k] = __bfloat162float(xb[k]) + __bfloat162float(rb[k]);
          nb[k] = __float2bfloat16_rn(s[i][k]);
        }
        if (write_residual) res4[c] = nv;
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) s[i][k] = __bfloat162float(xb[k]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) ss = fmaf(s[i][k], s[i][k], ss);
    }
  }
  const float total = block_sum(ss, red);
  const float rstd = 1.0f / sqrtf(total / (float)(width8 * 8) + eps);
  uint4* out4 = reinterpret_cast<uint4*>(out) + (size_t)r * width8;
#pragma unroll
  for (int i = 0; i < RN_CHUNKS; ++i) {
    const int c = threadIdx.x + i * RN_T;
    if (c < width8) {
      const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(&wv[i]);
      uint4 ov;
      __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&ov);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float n = __bfloat162float(__float2bfloat16_rn(s[i][k] * rstd));
        ob[k] = __float2bfloat16_rn(n * (__bfloat162float(wb[k]) + weight_offset));
      }
      out4[c] = ov;
    }
  }
}

NHV_API int nhv_rmsnorm(int dtype, void* out, const void* x, void* residual, const void* w, const int* rows,
                        int n_rows, int width, float eps, int write_residual, float weight_offset,
                        cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NHV_REQUIRE(n_rows > 0 && width > 0, "rmsnorm: bad sizes");
  const size_t smem = (size_t)width * sizeof(float);
  NHV_REQUIRE(smem <= 200 * 1024, "rmsnorm: width %d is beyond the %d floats a row buffer holds", width,
              200 * 1024 / 4);
  NHV_REQUIRE(!(rows && residual && write_residual), "rmsnorm: a gathered norm cannot write the residual back");
  if (dtype == NHV_BF16 && width % 8 == 0 && width <= RN_THREADS * RN_CHUNKS * 8 && ((uintptr_t)out % 16) == 0 &&
      ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 && (!residual || ((uintptr_t)residual % 16) == 0)) {
    // Many rows of up to 4,096 elements (a prompt's): half the threads, each with four 16-byte chunks on their way,
    // and twice the blocks on an SM (measured on B200, 2,048 rows of 4,096 with residual: 17.0 -> 14.0 us); few rows
    // (a decode step's) keep the most threads per row.
    if (width <= RN_THREADS / 2 * RN_CHUNKS * 8 && n_rows >= 256)
      nhv_launch(rmsnorm_bf16x8_kernel<RN_THREADS / 2>, n_rows, RN_THREADS / 2, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)x,
                 (__nv_bfloat16*)residual, (const __nv_bfloat16*)w, rows, width / 8, eps, write_residual, weight_offset);
    else
      nhv_launch(rmsnorm_bf16x8_kernel<RN_THREADS>, n_rows, RN_THREADS, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)x,
                 (__nv_bfloat16*)residual, (const __nv_bfloat16*)w, rows, width / 8, eps, write_residual, weight_offset);
    NHV_CHECK_LAUNCH("rmsnorm");
    return 0;
  }
  int threads = 32;
  while (threads < 1024 && threads * 4 < width) threads <<= 1;
#define LAUNCH(T)                                                                                          \
  do {                                                                                                     \
    if (smem > 48 * 1024)                                                                                  \
      NHV_CUDA(cudaFuncSetAttribute(rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,        \
                                    (int)smem), "rmsnorm");                                                \
    nhv_launch(rmsnorm_kernel<T>, n_rows, threads, smem, stream, (T*)out, (const T*)x, (T*)residual,    \
               (const T*)w, rows, width, eps, write_residual, weight_offset);                            \
  } while (0)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "rmsnorm: unknown dtype %d", dtype);
#undef LAUNCH
  NHV_CHECK_LAUNCH("rmsnorm");
  return 0;
}

// ---------------------------------------------------------------- SiLU(gate) * up
// gate_up [n, 2*inter] with gate in the first half of each row; out [n, inter].
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter, size_t total) {
  pdl_prologue();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / inter;
    const int c = (int)(i - t * inter);
    const float g = to_f32<T>(gate_up[t * 2 * inter + c]);
    const float u = to_f32<T>(gate_up[t * 2 * inter + inter + c]);
    out[i] = from_f32<T>(g / (1.0f + expf(-g)) * u);
  }
}

// bf16, inter a multiple of 8: 16-byte loads and stores, two of each in flight per thread.  The result is rounded
// to bfloat16, so the fast exponential and division (about 2 ulp of fp32) leave it unchanged but for rare
// values on a rounding boundary; the 32-bit path uses the exact kernel above.
__device__ __forceinline__ uint4 silu_mul8(const uint4& gv, const uint4& uv) {
  const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(&gv);
  const __nv_bfloat16* u = reinterpret_cast<const __nv_bfloat16*>(&uv);
  uint4 ov;
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&ov);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float gf = __bfloat162float(g[k]);
    o[k] = __float2bfloat16_rn(__fdividef(gf, 1.0f + __expf(-gf)) * __bfloat162float(u[k]));
  }
  return ov;
}

__global__ void silu_mul_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gate_up,
                                       int inter8, size_t total8) {
  pdl_prologue();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const uint4* in = reinterpret_cast<const uint4*>(gate_up);
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + stride < total8; i += 2 * stride) {
    const size_t j = i + stride;
    const size_t t0 = i / inter8, t1 = j / inter8;
    const size_t a0 = t0 * 2 * inter8 + (i - t0 * inter8), a1 = t1 * 2 * inter8 + (j - t1 * inter8);
    const uint4 g0 = in[a0], u0 = in[a0 + inter8], g1 = in[a1], u1 = in[a1 + inter8];
    reinterpret_cast<uint4*>(out)[i] = silu_mul8(g0, u0);
    reinterpret_cast<uint4*>(out)[j] = silu_mul8(g1, u1);
  }
  if (i < total8) {
    const size_t t = i / inter8;
    const size_t a = t * 2 * inter8 + (i - t * inter8);
    reinterpret_cast<uint4*>(out)[i] = silu_mul8(in[a], in[a + inter8]);
  }
}

NHV_API int nhv_silu_mul(int dtype, void* out, const void* gate_up, int n_rows, int inter, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NHV_REQUIRE(n_rows > 0 && inter > 0, "silu_mul: bad sizes");
  const size_t total = (size_t)n_rows * inter;
  const int threads = 256;
  if (dtype == NHV_BF16 && inter % 8 == 0 && ((uintptr_t)out % 16 == 0) && ((uintptr_t)gate_up % 16 == 0)) {
    const size_t total8 = total / 8;
    const int blocks = (int)((total8 + threads - 1) / threads < 148 * 16 ? (total8 + threads - 1) / threads : 148 * 16);
    nhv_launch(silu_mul_bf16x8_kernel, blocks, threads, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up,
               inter / 8, total8);
  } else {
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    if (dtype == NHV_F32)
      nhv_launch(silu_mul_kernel<float>, blocks, threads, 0, stream, (float*)out, (const float*)gate_up, inter, total);
    else if (dtype == NHV_BF16)
      nhv_launch(silu_mul_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (__nv_bfloat16*)out,
                 (const __nv_bfloat16*)gate_up, inter, total);
    else
      NHV_REQUIRE(false, "silu_mul: unknown dtype %d", dtype);
  }
  NHV_CHECK_LAUNCH("silu_mul");
  return 0;
}

// ---------------------------------------------------------------- storage type -> fp32 rows
template <typename T>
__global__ void to_f32_kernel(float* __restrict__ out, const T* __restrict__ x, size_t total) {
  pdl_prologue();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    out[i] = to_f32<T>(x[i]);
}

NHV_API int nhv_to_f32(int dtype, float* out, const void* x, size_t total, cudaStream_t stream) {
  if (total == 0) return 0;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == NHV_BF16)
    nhv_launch(to_f32_kernel<__nv_bfloat16>, blocks, threads, 0, stream, out, (const __nv_bfloat16*)x, total);
  else if (dtype == NHV_F32)
    nhv_launch(to_f32_kernel<float>, blocks, threads, 0, stream, out, (const float*)x, total);
  else
    NHV_REQUIRE(false, "to_f32: unknown dtype %d", dtype);
  NHV_CHECK_LAUNCH("to_f32");
  return 0;
}
