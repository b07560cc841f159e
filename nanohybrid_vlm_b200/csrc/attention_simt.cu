// Causal grouped-query attention over cache pages, for any step shape: one kernel serves
// prompt portions and single decoded tokens alike, in fp32 or bf16 storage with all
// arithmetic in fp32.  It is the exact path (true 32-bit) and the fallback of the bf16
// path for head sizes and page sizes that the tensor-core kernels refuse.
//
// Replaces the two library calls at nanovllm/layers/attention.py:67-74.  Scores are
// (q . k) * scale, softmax over keys 0..pos of the same request (or the last `window`
// of them), query head h reads KV head h / (nq / nkv).
//
// The arithmetic for one (query token, head) is fixed: keys are visited in chunks of 32
// aligned to absolute multiples of 32, each dot product runs over the head size in
// ascending order, and the running maximum / sum / output are rescaled once per chunk.
// So a position's result does not depend on how tokens were cut into steps, on the
// batch around it, or on which pages hold the keys.
//
// Block = (tile of TQ consecutive new tokens of one request) x (one KV head) x (a
// sub-group of GS query heads that share it).  A "pair" is (token of the tile, head of
// the sub-group); pairs are dealt to the 4 warps round-robin, lane <-> key inside a
// chunk for the scores, lane <-> output column for the weighted sum of values.
#include <math.h>

#include "nhv_common.cuh"

constexpr int AT_WARPS = 4;
constexpr int AT_CHUNK = 32;
constexpr int AT_MAX_PAIRS = 32;
constexpr int AT_PAIRS_PER_WARP = AT_MAX_PAIRS / AT_WARPS;  // 8
constexpr int AT_MAX_D = 256;
constexpr int AT_COLS = AT_MAX_D / 32;  // output columns per lane

template <typename T>
__global__ void attn_paged_simt_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                                       const T* __restrict__ kv_pages, const int* __restrict__ block_table,
                                       int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                                       int n_seqs, int nq, int nkv, int d, int page_size, int n_pages, int window,
                                       float scale, int TQ, int GS) {
  extern __shared__ float smem[];
  pdl_prologue();
  const int G = nq / nkv;
  const int kvh = blockIdx.y;
  const int g0 = blockIdx.z * GS;
  const int gs = min(GS, G - g0);

  // Which request and which tile of its new tokens is this block?
  int seq = -1, tile = blockIdx.x;
  for (int s = 0; s < n_seqs; ++s) {
    const int n = cu_q[s + 1] - cu_q[s];
    const int nt = (n + TQ - 1) / TQ;
    if (tile < nt) { seq = s; break; }
    tile -= nt;
  }
  if (seq < 0) return;
  const int n_new = cu_q[seq + 1] - cu_q[seq];
  const int total = kv_len[seq];
  const int q_pos0 = total - n_new;           // position of the request's first new token
  const int t0 = tile * TQ;                   // first token of the tile, within the new tokens
  const int tq_n = min(TQ, n_new - t0);
  const int n_pairs = tq_n * gs;
  const int pos_lo = q_pos0 + t0, pos_hi = q_pos0 + t0 + tq_n - 1;

  const int ks = d + 1;                        // padded key row: lane <-> key reads hit 32 banks
  float* Ks = smem;                            // [32][d+1]
  float* Vs = Ks + AT_CHUNK * ks;              // [32][d]
  float* Qs = Vs + AT_CHUNK * d;               // [pairs][d]
  float* Ps = Qs + AT_MAX_PAIRS * d;           // [warps][32]
  __shared__ int key_ok[AT_CHUNK];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int i = threadIdx.x; i < n_pairs * d; i += blockDim.x) {
    const int p = i / d, c = i - p * d;
    const int tq = p / gs, g = p - tq * gs;
    const size_t tok = (size_t)cu_q[seq] + t0 + tq;
    Qs[p * d + c] = to_f32<T>(q[tok * q_stride + (size_t)(kvh * G + g0 + g) * d + c]);
  }

  float m[AT_PAIRS_PER_WARP], l[AT_PAIRS_PER_WARP], o[AT_PAIRS_PER_WARP][AT_COLS];
#pragma unroll
  for (int i = 0; i < AT_PAIRS_PER_WARP; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < AT_COLS; ++c) o[i][c] = 0.f;
  }

  int first_key = 0;
  if (window > 0) first_key = max(0, pos_lo - window + 1);
  const int c_begin = (first_key / AT_CHUNK) * AT_CHUNK;

  for (int c0 = c_begin; c0 <= pos_hi; c0 += AT_CHUNK) {
    __syncthreads();
    // Stage 32 keys and values (zero where there is no key or its page was given back).
    if (threadIdx.x < AT_CHUNK) {
      const int j = c0 + threadIdx.x;
      int ok = 0;
      if (j <= pos_hi && j < total) {
        const int page = block_table[(size_t)seq * bt_stride + j / page_size];
        ok = page >= 0 && page < n_pages;
      }
      key_ok[threadIdx.x] = ok;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < AT_CHUNK * d; i += blockDim.x) {
      const int r = i / d, c = i - r * d;
      float kx = 0.f, vx = 0.f;
      if (key_ok[r]) {
        const int j = c0 + r;
        const int page = block_table[(size_t)seq * bt_stride + j / page_size];
        const int off = j % page_size;
        const size_t base = ((((size_t)page * 2) * nkv + kvh) * page_size + off) * d + c;
        kx = to_f32<T>(kv_pages[base]);
        vx = to_f32<T>(kv_pages[base + (size_t)nkv * page_size * d]);
      }
      Ks[r * ks + c] = kx;
      Vs[r * d + c] = vx;
    }
    __syncthreads();

#pragma unroll
    for (int i = 0; i < AT_PAIRS_PER_WARP; ++i) {
      const int p = warp + i * AT_WARPS;
      if (p >= n_pairs) break;
      const int tq = p / gs;
      const int pos = pos_lo + tq;
      const int lo = window > 0 ? max(0, pos - window + 1) : 0;
      if (c0 > pos || c0 + AT_CHUNK <= lo) continue;  // no key of this chunk is visible to this query
      const int j = c0 + lane;
      float s = -INFINITY;
      if (j <= pos && j >= lo && key_ok[lane]) {
        const float* qv = Qs + p * d;
        const float* kv = Ks + lane * ks;
        float acc = 0.f;
        for (int c = 0; c < d; ++c) acc = fmaf(qv[c], kv[c], acc);
        s = acc * scale;
      }
      const float cmax = warp_max(s);
      if (cmax == -INFINITY) continue;
      const float m_new = fmaxf(m[i], cmax);
      const float alpha = expf(m[i] - m_new);     // exp(-inf) = 0 on the first chunk
      const float pr = expf(s - m_new);           // 0 for masked keys
      l[i] = l[i] * alpha + warp_sum(pr);
      m[i] = m_new;
      Ps[warp * AT_CHUNK + lane] = pr;
      __syncwarp();
#pragma unroll
      for (int cc = 0; cc < AT_COLS; ++cc) {
        const int c = lane + cc * 32;
        if (c < d) {
          float acc = 0.f;
          for (int r = 0; r < AT_CHUNK; ++r) acc = fmaf(Ps[warp * AT_CHUNK + r], Vs[r * d + c], acc);
          o[i][cc] = o[i][cc] * alpha + acc;
        }
      }
      __syncwarp();
    }
  }

#pragma unroll
  for (int i = 0; i < AT_PAIRS_PER_WARP; ++i) {
    const int p = warp + i * AT_WARPS;
    if (p >= n_pairs) break;
    const int tq = p / gs, g = p - tq * gs;
    const size_t tok = (size_t)cu_q[seq] + t0 + tq;
    T* dst = out + tok * out_stride + (size_t)(kvh * G + g0 + g) * d;
    const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
#pragma unroll
    for (int cc = 0; cc < AT_COLS; ++cc) {
      const int c = lane + cc * 32;
      if (c < d) dst[c] = from_f32<T>(o[i][cc] * inv);
    }
  }
}

// max_tiles: an upper bound on sum over requests of ceil(new tokens / TQ); the caller may pass
// n_tokens / TQ + n_seqs.  Blocks beyond the true count leave at once.
NHV_API int nhv_attention_simt(int dtype, const void* q, int q_stride, void* out, int out_stride,
                               const void* kv_pages, const int* block_table, int bt_stride, const int* cu_q,
                               const int* kv_len, int n_seqs, int n_tokens, int nq, int nkv, int d, int page_size,
                               int n_pages, int window, float scale, cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  NHV_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads do not divide into %d KV heads", nq, nkv);
  NHV_REQUIRE(d > 0 && d <= AT_MAX_D, "attention: head size %d is beyond the supported %d", d, AT_MAX_D);
  NHV_REQUIRE(page_size > 0 && n_pages > 0 && bt_stride > 0, "attention: bad page geometry");
  const int G = nq / nkv;
  const int GS = G < 8 ? G : 8;
  const int TQ = AT_MAX_PAIRS / GS;
  const int max_tiles = n_tokens / TQ + n_seqs;
  const size_t smem = ((size_t)AT_CHUNK * (d + 1) + (size_t)AT_CHUNK * d + (size_t)AT_MAX_PAIRS * d +
                       AT_WARPS * AT_CHUNK) * sizeof(float);
  dim3 grid(max_tiles, nkv, (G + GS - 1) / GS);
#define LAUNCH(T)                                                                                              \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      NHV_CUDA(cudaFuncSetAttribute(attn_paged_simt_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                    (int)smem), "attention");                                                  \
    nhv_launch(attn_paged_simt_kernel<T>, grid, AT_WARPS * 32, smem, stream,                                   \
        (const T*)q, q_stride, (T*)out, out_stride, (const T*)kv_pages, block_table, bt_stride, cu_q, kv_len,  \
        n_seqs, nq, nkv, d, page_size, n_pages, window, scale, TQ, GS);                                        \
  } while (0)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "attention: unknown dtype %d", dtype);
#undef LAUNCH
  NHV_CHECK_LAUNCH("attention");
  return 0;
}
