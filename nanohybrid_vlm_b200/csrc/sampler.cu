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

// Scores are compared as 64-bit keys: the score's bits made order-preserving in the high word, the complement of
// the index in the low word, so that the largest key is the best score and, among equal scores, the lowest
// index (what a sequential argmax gives).
__device__ __forceinline__ unsigned long long score_key(float s, int i) {
  const uint32_t b = __float_as_uint(s);
  const uint32_t ordered = b ^ ((b >> 31) ? 0xFFFFFFFFu : 0x80000000u);
  return ((unsigned long long)ordered << 32) | (uint32_t)(~(uint32_t)i);
}

// A row is cut into gridDim.y pieces, one block each; the blocks meet at the row's slot of `best` (atomic
// maximum of the keys) and count their arrival; the block that arrives last writes the row's token and
// returns slot and counter to zero for the next launch.  No block waits for another.
//
// The sampler is the last kernel of a step and its result is what the host reads, so it also carries the step's
// health: `error_words` holds device addresses of the error words of kernels with bounded waits (null entries
// are skipped); bit i of *status is set if word i is not zero.  Every kernel of the step has completed when this
// one reads them (it waits for its predecessor before reading anything).
__global__ void __launch_bounds__(256) sample_kernel(int* __restrict__ out, const float* __restrict__ logits,
                                                     int ld, const float* __restrict__ temperatures,
                                                     const unsigned long long* __restrict__ seeds,
                                                     const int* __restrict__ positions, int vocab,
                                                     unsigned long long* __restrict__ best, int* __restrict__ arrived,
                                                     const int* const* __restrict__ error_words, int n_error_words,
                                                     int* __restrict__ status) {
  __shared__ unsigned long long warp_best[8];
  pdl_prologue();
  const int row = blockIdx.x;
  if (status != nullptr && row == 0 && blockIdx.y == 0 && threadIdx.x == 0) {
    int bits = 0;
    for (int i = 0; i < n_error_words && i < 31; ++i) {
      const int* word = error_words[i];
      if (word != nullptr && *reinterpret_cast<const volatile int*>(word) != 0) bits |= 1 << i;
    }
    *status = bits;
  }
  const float* lg = logits + (size_t)row * ld;
  const float temp = temperatures[row];
  const unsigned long long seed = seeds[row];
  const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  const uint32_t pos = (uint32_t)positions[row];
  const int n_groups = (vocab + 3) >> 2;
  const int per = (n_groups + gridDim.y - 1) / gridDim.y;
  const int g_end = min(n_groups, ((int)blockIdx.y + 1) * per);
  const bool vec = (ld & 3) == 0 && ((uintptr_t)logits & 15) == 0;
  unsigned long long key = 0;
  for (int gidx = blockIdx.y * per + threadIdx.x; gidx < g_end; gidx += blockDim.x) {
    uint32_t c[4] = {(uint32_t)gidx, pos, 0u, 0u};
    if (temp > 0.f) philox4x32_10(c, k0, k1);
    float v[4];
    if (vec && gidx * 4 + 3 < vocab) {
      const float4 f = *reinterpret_cast<const float4*>(lg + gidx * 4);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = gidx * 4 + k < vocab ? lg[gidx * 4 + k] : -INFINITY;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = gidx * 4 + k;
      if (i >= vocab) break;
      float s = v[k];
      if (temp > 0.f) {
        const float u = ((float)(c[k] >> 9) + 0.5f) * (1.0f / 8388608.0f);
        const float noise = fmaxf(-logf(u), 1e-10f);
        s = s / temp - logf(noise);
      }
      const unsigned long long kk = score_key(s, i);
      key = kk > key ? kk : key;
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
    key = other > key ? other : key;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) warp_best[warp] = key;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) key = warp_best[w] > key ? warp_best[w] : key;
    atomicMax(best + row, key);
    __threadfence();
    if (atomicAdd(arrived + row, 1) == (int)gridDim.y - 1) {
      __threadfence();
      const unsigned long long win = atomicExch(best + row, 0ull);     // read and return to zero
      const uint32_t idx = ~(uint32_t)win;
      out[row] = win == 0ull || idx >= (uint32_t)vocab ? 0 : (int)idx;
      arrived[row] = 0;
    }
  }
}

// best [n_rows] 64-bit words and arrived [n_rows] ints, all zero (the kernel leaves them zero).  error_words:
// device array of n_error_words device addresses (or null entries), status: one int on the device; both may be
// null, then no health is reported.
NHV_API int nhv_sample(int* out, const float* logits, int ld, const float* temperatures,
                       const unsigned long long* seeds, const int* positions, int n_rows, int vocab,
                       unsigned long long* best, int* arrived, const int* const* error_words, int n_error_words,
                       int* status, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NHV_REQUIRE(n_rows > 0 && vocab > 0 && ld >= vocab && best && arrived, "sample: bad arguments");
  // pieces of about 8,192 scores, but no more blocks than a few per SM
  int pieces = (vocab + 8191) / 8192;
  const int room = 148 * 4 / n_rows;
  if (pieces > room) pieces = room < 1 ? 1 : room;
  nhv_launch(sample_kernel, dim3(n_rows, pieces), 256, 0, stream, out, logits, ld, temperatures, seeds, positions, vocab,
             best, arrived, error_words, error_words ? n_error_words : 0, error_words ? status : (int*)nullptr);
  NHV_CHECK_LAUNCH("sample");
  return 0;
}
