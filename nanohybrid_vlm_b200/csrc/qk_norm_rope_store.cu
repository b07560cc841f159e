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

// bfloat16, head sizes 16/32/64/128/256 with a rotary half that is a multiple of 8: each lane owns 16 bytes of
// a head (d / 8 lanes per head, several heads per warp), so every global access is a 16-byte one; the rotation's
// partner elements come from the lane (rotary_dim / 16) further on by shuffle.  Same arithmetic and rounding
// as the kernel above.
template <int LPH>   // lanes per head = d / 8, a power of two
__global__ void __launch_bounds__(QK_WARPS * 32) qk_norm_rope_store_bf16x8_kernel(
    const __nv_bfloat16* __restrict__ qkv, int qkv_stride, __nv_bfloat16* __restrict__ q_out, int q_out_stride,
    __nv_bfloat16* __restrict__ kv_pages, const int* __restrict__ slot_mapping, const int* __restrict__ positions,
    const __nv_bfloat16* __restrict__ q_w, const __nv_bfloat16* __restrict__ k_w, const float* __restrict__ cos_sin,
    int rotary_dim, int max_position, int n_tokens, int nq, int nkv, int page_size, int n_pages, float eps,
    float weight_offset, int heads_per_token) {
  pdl_prologue();
  constexpr int HPW = 32 / LPH, D = LPH * 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPH, c = lane % LPH;
  const long item = ((long)blockIdx.x * QK_WARPS + warp) * HPW + sub;
  const bool active = item < (long)n_tokens * heads_per_token;
  const int t = active ? (int)(item / heads_per_token) : 0;
  const int head = active ? (int)(item - (long)t * heads_per_token) : 0;
  const int kind = head < nq ? 0 : (head < nq + nkv ? 1 : 2);
  __nv_bfloat16* dst = nullptr;
  if (active) {
    if (kind == 0) {
      dst = q_out + (size_t)t * q_out_stride + (size_t)head * D + c * 8;
    } else {
      const int slot = slot_mapping[t];
      if (slot >= 0 && slot < n_pages * page_size) {
        const int page = slot / page_size, off = slot - page * page_size;
        const int kvh = kind == 1 ? head - nq : head - nq - nkv;
        dst = kv_pages + ((((size_t)page * 2 + (kind - 1)) * nkv + kvh) * page_size + off) * D + c * 8;
      }
    }
  }
  float v[8];
  {
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (active) raw = *reinterpret_cast<const uint4*>(qkv + (size_t)t * qkv_stride + (size_t)head * D + c * 8);
    const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = __bfloat162float(b[k]);
  }
  const __nv_bfloat16* w = kind == 0 ? q_w : (kind == 1 ? k_w : nullptr);
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) ss = fmaf(v[k], v[k], ss);
#pragma unroll
  for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (w) {
    const float rstd = 1.0f / sqrtf(ss / (float)D + eps);
    const uint4 wraw = *reinterpret_cast<const uint4*>(w + c * 8);
    const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(&wraw);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float n = __bfloat162float(__float2bfloat16_rn(v[k] * rstd));
      v[k] = __bfloat162float(__float2bfloat16_rn(n * (__bfloat162float(wb[k]) + weight_offset)));
    }
  }
  const int half_lanes = rotary_dim >> 4;                  // lanes that hold half of the rotary part
  const bool rotate = kind != 2 && cos_sin != nullptr;
  const bool first_half = c < half_lanes, in_rot = c < 2 * half_lanes;
  const int partner = first_half ? lane + half_lanes : lane - half_lanes;
  float other[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) other[k] = __shfl_sync(0xffffffffu, v[k], (partner & 31));
  if (rotate && in_rot && active) {
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_position ? max_position - 1 : pos);
    const int half = rotary_dim >> 1;
    const int i0 = (first_half ? c : c - half_lanes) * 8;   // index into the cos / sin halves
    const float* cs = cos_sin + (size_t)pos * rotary_dim;
    const float4 c0 = *reinterpret_cast<const float4*>(cs + i0), c1 = *reinterpret_cast<const float4*>(cs + i0 + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(cs + half + i0), s1 = *reinterpret_cast<const float4*>(cs + half + i0 + 4);
    const float co[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float si[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
    for (int k = 0; k < 8; ++k)
      v[k] = first_half ? v[k] * co[k] - other[k] * si[k] : v[k] * co[k] + other[k] * si[k];
  }
  if (dst) {
    uint4 o;
    __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
    for (int k = 0; k < 8; ++k) ob[k] = __float2bfloat16_rn(v[k]);
    *reinterpret_cast<uint4*>(dst) = o;
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
  const bool pow2 = (d & (d - 1)) == 0;
  if (dtype == NHV_BF16 && pow2 && d >= 16 && d <= 256 && (!cos_sin || rotary_dim % 16 == 0) && qkv_stride % 8 == 0 &&
      q_out_stride % 8 == 0 && ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)q_out % 16) == 0 &&
      (!kv_pages || ((uintptr_t)kv_pages % 16) == 0) && (!q_w || ((uintptr_t)q_w % 16) == 0) &&
      (!k_w || ((uintptr_t)k_w % 16) == 0) && (!cos_sin || ((uintptr_t)cos_sin % 16) == 0)) {
    const int lph = d / 8, hpw = 32 / lph;
    const int vblocks = (int)((items + (long)QK_WARPS * hpw - 1) / ((long)QK_WARPS * hpw));
#define VLAUNCH(L)                                                                                               \
    nhv_launch(qk_norm_rope_store_bf16x8_kernel<L>, vblocks, QK_WARPS * 32, 0, stream, (const __nv_bfloat16*)qkv, \
               qkv_stride, (__nv_bfloat16*)q_out, q_out_stride, (__nv_bfloat16*)kv_pages, slot_mapping, positions, \
               (const __nv_bfloat16*)q_w, (const __nv_bfloat16*)k_w, cos_sin, rotary_dim, max_position, n_tokens, \
               nq, nkv, page_size, n_pages, eps, weight_offset, heads_per_token)
    if (lph == 2) VLAUNCH(2);
    else if (lph == 4) VLAUNCH(4);
    else if (lph == 8) VLAUNCH(8);
    else if (lph == 16) VLAUNCH(16);
    else VLAUNCH(32);
#undef VLAUNCH
    NHV_CHECK_LAUNCH("qk_norm_rope_store");
    return 0;
  }
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
