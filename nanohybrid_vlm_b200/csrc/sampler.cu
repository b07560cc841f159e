// Token choice from fp32 logits: argmax for temperature 0, else the exponential race of
// nanovllm/layers/sampler.py:12-65: argmax_i softmax(logits / T)_i / noise_i with
// noise ~ Exp(1) clamped at 1e-10.  The softmax's denominator is the same for every i,
// so the race is run on logits_i / T - log(noise_i).
//
// The noise is a counter-based Philox4x32-10 stream keyed by the request's seed, with the
// position of the token being chosen and the vocabulary index as the counter: the same
// request draws the same tokens whatever else is in the batch.
#include <math.h>

#include "nhv_common.cuh"

__device__ __forceinline__ void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

__global__ void __launch_bounds__(1024) sample_kernel(int* __restrict__ out, const float* __restrict__ logits,
                                                      int ld, const float* __restrict__ temperatures,
                                                      const unsigned long long* __restrict__ seeds,
                                                      const int* __restrict__ positions, int vocab) {
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  pdl_prologue();
  const int row = blockIdx.x;
  const float* lg = logits + (size_t)row * ld;
  const float temp = temperatures[row];
  const unsigned long long seed = seeds[row];
  const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  const uint32_t pos = (uint32_t)positions[row];
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  const int n_groups = (vocab + 3) >> 2;
  for (int gidx = threadIdx.x; gidx < n_groups; gidx += blockDim.x) {
    uint32_t c[4] = {(uint32_t)gidx, pos, 0u, 0u};
    if (temp > 0.f) philox4x32_10(c, k0, k1);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = gidx * 4 + k;
      if (i >= vocab) break;
      float s = lg[i];
      if (temp > 0.f) {
        const float u = ((float)(c[k] >> 9) + 0.5f) * (1.0f / 8388608.0f);
        const float noise = fmaxf(-logf(u), 1e-10f);
        s = s / temp - logf(noise);
      }
      if (s > bv || (s == bv && i < bi)) { bv = s; bi = i; }
    }
  }
  // lowest index among equal scores, as a sequential argmax gives
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    bv = lane < nw ? best_v[lane] : -INFINITY;
    bi = lane < nw ? best_i[lane] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
  }
}

NHV_API int nhv_sample(int* out, const float* logits, int ld, const float* temperatures,
                       const unsigned long long* seeds, const int* positions, int n_rows, int vocab,
                       cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NHV_REQUIRE(n_rows > 0 && vocab > 0 && ld >= vocab, "sample: bad sizes");
  int threads = 128;
  while (threads < 1024 && threads * 16 < vocab) threads <<= 1;
  nhv_launch(sample_kernel, n_rows, threads, 0, stream, out, logits, ld, temperatures, seeds, positions, vocab);
  NHV_CHECK_LAUNCH("sample");
  return 0;
}
