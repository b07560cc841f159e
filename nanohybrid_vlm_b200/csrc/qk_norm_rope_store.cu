// Fused per-head q/k RMSNorm, rotary position encoding and key/value store into cache pages.
//
// One warp per (token, head) of the packed projection output qkv [T, (nq + 2*nkv) * d]:
//   q heads: norm (weight q_w) -> rotate -> written to q_out [T, nq, d] (row stride q_out_stride)
//   k heads: norm (weight k_w) -> rotate -> written to the token's slot of the K pages
//   v heads: copied to the token's slot of the V pages
// The order norm -> round -> times weight -> round -> rotate in fp32 -> round is that of
// nanovllm/models/qwen3.py:82-85, nanovllm/layers/layernorm.py:16-26 and
// nanovllm/layers/rotary_embedding.py:6-14 (half-split rotation: element i pairs with
// i + rotary_dim/2; elements at and beyond rotary_dim pass through).  The store replaces
// nanovllm/layers/attention.py:10-40.
//
// Cache pages of one layer: [page][K|V][kv_head][slot_in_page][d].
// slot_mapping[t] = page * page_size + slot_in_page, or -1 for "do not store".
#include "nhv_common.cuh"

constexpr int QK_WARPS = 4;
constexpr int QK_MAX_D = 512;

template <typename T>
__global__ void qk_norm_rope_store_kernel(const T* __restrict__ qkv, int qkv_stride, T* __restrict__ q_out,
                                          int q_out_stride, T* __restrict__ kv_pages,
                                          const int* __restrict__ slot_mapping, const int* __restrict__ positions,
                                          const T* __restrict__ q_w, const T* __restrict__ k_w,
                                          const float* __restrict__ cos_sin, int rotary_dim, int max_position,
                                          int n_tokens, int nq, int nkv, int d, int page_size, int n_pages,
                                          float eps, float weight_offset, int heads_per_token) {
  extern __shared__ float smem[];
  pdl_prologue();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * QK_WARPS + warp;
  if (item >= (long)n_tokens * heads_per_token) return;
  const int t = (int)(item / heads_per_token);
  const int head = (int)(item - (long)t * heads_per_token);
  float* v = smem + warp * d;

  const T* src = qkv + (size_t)t * qkv_stride + (size_t)head * d;
  const int kind = head < nq ? 0 : (head < nq + nkv ? 1 : 2);  // q, k, v
  T* dst;
  if (kind == 0) {
    dst = q_out + (size_t)t * q_out_stride + (size_t)head * d;
  } else {
    const int slot = slot_mapping[t];
    if (slot < 0 || slot >= n_pages * page_size) return;  // nothing to store (or a bad slot: never write there)
    const int page = slot / page_size, off = slot - page * page_size;
    const int kvh = kind == 1 ? head - nq : head - nq - nkv;
    dst = kv_pages + ((((size_t)page * 2 + (kind - 1)) * nkv + kvh) * page_size + off) * d;
  }

  float ss = 0.f;
  for (int c = lane; c < d; c += 32) {
    const float x = to_f32<T>(src[c]);
    v[c] = x;
    ss = fmaf(x, x, ss);
  }
  const T* w = kind == 0 ? q_w : (kind == 1 ? k_w : nullptr);
  if (kind != 2 && w) {
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)d + eps);
    for (int c = lane; c < d; c += 32) {
      const float n = round_to<T>(v[c] * rstd);
      v[c] = round_to<T>(n * (to_f32<T>(w[c]) + weight_offset));
    }
  }
  __syncwarp();
  if (kind != 2 && cos_sin) {
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_position ? max_position - 1 : pos);
    const int half = rotary_dim >> 1;
    const float* cs = cos_sin + (size_t)pos * rotary_dim;  // cos[0..half) then sin[0..half)
    for (int c = lane; c < d; c += 32) {
      float y = v[c];
      if (c < half) {
        y = v[c] * cs[c] - v[c + half] * cs[half + c];
      } else if (c < rotary_dim) {
        y = v[c] * cs[c - half] + v[c - half] * cs[c];
      }
      dst[c] = from_f32<T>(y);
    }
  } else {
    for (int c = lane; c < d; c += 32) dst[c] = from_f32<T>(v[c]);
  }
}

NHV_API int nhv_qk_norm_rope_store(int dtype, const void* qkv, int qkv_stride, void* q_out, int q_out_stride,
                                   void* kv_pages, const int* slot_mapping, const int* positions, const void* q_w,
                                   const void* k_w, const float* cos_sin, int rotary_dim, int max_position,
                                   int n_tokens, int nq, int nkv, int d, int page_size, int n_pages, float eps,
                                   float weight_offset, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  NHV_REQUIRE(n_tokens > 0 && nq > 0 && nkv >= 0 && d > 0, "qk_norm_rope_store: bad sizes");
  NHV_REQUIRE(d <= QK_MAX_D, "qk_norm_rope_store: head size %d is beyond the supported %d", d, QK_MAX_D);
  NHV_REQUIRE(!cos_sin || (rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= d),
              "qk_norm_rope_store: rotary_dim %d must be even and at most the head size %d", rotary_dim, d);
  NHV_REQUIRE(kv_pages == nullptr || (page_size > 0 && n_pages > 0 && slot_mapping),
              "qk_norm_rope_store: a key/value store needs pages and a slot mapping");
  NHV_REQUIRE(!cos_sin || positions, "qk_norm_rope_store: rotation needs positions");
  // Without pages only the query heads are processed (a layer that reads another layer's cache).
  const int heads_per_token = kv_pages ? nq + 2 * nkv : nq;
  const long items = (long)n_tokens * heads_per_token;
  const int blocks = (int)((items + QK_WARPS - 1) / QK_WARPS);
  const size_t smem = (size_t)QK_WARPS * d * sizeof(float);
#define LAUNCH(T)                                                                                              \
  nhv_launch(qk_norm_rope_store_kernel<T>, blocks, QK_WARPS * 32, smem, stream,                                \
      (const T*)qkv, qkv_stride, (T*)q_out, q_out_stride, (T*)kv_pages, slot_mapping, positions, (const T*)q_w, \
      (const T*)k_w, cos_sin, rotary_dim, max_position, n_tokens, nq, nkv, d, page_size, n_pages, eps,        \
      weight_offset, heads_per_token)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "qk_norm_rope_store: unknown dtype %d", dtype);
#undef LAUNCH
  NHV_CHECK_LAUNCH("qk_norm_rope_store");
  return 0;
}
