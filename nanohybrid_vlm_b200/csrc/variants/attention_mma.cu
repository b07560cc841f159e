// bfloat16 attention over cache pages on the tensor cores, compiled once per head size
// (-DNHV_ATTN_D=<head size>, a multiple of 16 up to 256).
//
// Two kernels share one tile routine (64 keys per tile, cp.async double buffering into
// shared memory, ldmatrix fragments, mma.sync.m16n8k16 bf16 with fp32 accumulation, online
// softmax in fp32 on base-2 exponents):
//
//  * prompt portions (a request brings more than one token): a block owns 64 rows, a row
//    being (new token, query head of one KV head's group), token-major, so the grouped
//    query heads share every key/value tile that is read; each of the 4 warps owns 16 rows
//    and walks all keys up to its rows' positions.
//  * single decoded tokens: the rows are the query heads of one KV head's group, all 4
//    warps hold the same rows and take a quarter of every 64-key tile each; the tiles of all
//    requests are dealt to a fixed grid of blocks in contiguous runs (see the decode kernel).
//
// Requests with one new token are left to the decode kernel, the others to the prefill
// kernel, so a mixed batch is two launches.  Keys and values of one layer:
// [page][K|V][kv_head][slot][d] (bf16); a request's logical page p is block_table[p], -1
// where a window has passed it.  Replaces the library calls at
// nanovllm/layers/attention.py:67-74.
#include <math.h>

#include "../nhv_common.cuh"

#ifndef NHV_ATTN_D
#error "compile with -DNHV_ATTN_D=<head size>"
#endif

namespace {

constexpr int D = NHV_ATTN_D;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16 up to 256");
constexpr int CH = D / 8;          // 16-byte chunks in a row
// ldmatrix reads one chunk column of 8 rows at a time: the 8 rows must fall into 8 different bank groups.
// Rows of a multiple of 128 bytes swap chunks inside each group of 8 (chunk ^ (row & 7)); other head sizes
// pad every row by one chunk, which makes the row stride odd.
constexpr bool SWIZZLE = CH % 8 == 0;
constexpr int ROW_CH = SWIZZLE ? CH : CH + 1;
constexpr int BN = 64;             // keys per tile
constexpr int TILE_ELEMS = BN * ROW_CH * 8;
constexpr int KS = D / 16;         // k-steps of Q.K^T
constexpr int DN = D / 8;          // n-tiles of P.V
constexpr int THREADS = 128;
constexpr float LOG2E = 1.4426950408889634f;

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are filled with zeros and src is not read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// element offset of (row, 16-byte chunk) in a tile
__device__ __forceinline__ int tile_off(int row, int chunk) {
  return (row * ROW_CH + (SWIZZLE ? (chunk ^ (row & 7)) : chunk)) * 8;
}

struct PageGeom {
  const bf16* kv_pages;
  const int* table;     // this request's block table
  int nkv, kvh, page_size, n_pages;
};

// Bring keys [key0, key0 + 64) of one request into a K tile and a V tile; keys outside [lo, hi) or on a
// page that was given back are zero-filled.  `page` >= -1: the whole tile lies on that page (page sizes that
// are a multiple of the tile), looked up by the caller ahead of time; -2: look every row's page up here.
__device__ __forceinline__ void load_kv_tile(bf16* ks, bf16* vs, const PageGeom& g, int key0, int lo, int hi, int page) {
  const size_t v_off = (size_t)g.nkv * g.page_size * D;
  if (page != -2) {
    const bool page_ok = page >= 0 && page < g.n_pages;
    const bf16* base = g.kv_pages + ((((size_t)(page_ok ? page : 0) * 2) * g.nkv + g.kvh) * g.page_size + (key0 % g.page_size)) * D;
#pragma unroll 4
    for (int id = threadIdx.x; id < BN * CH; id += THREADS) {
      const int r = id / CH, c = id - r * CH;
      const int j = key0 + r;
      const bool ok = page_ok && j >= lo && j < hi;
      const bf16* src = ok ? base + (size_t)r * D + c * 8 : g.kv_pages;
      cp_async16(ks + tile_off(r, c), src, ok);
      cp_async16(vs + tile_off(r, c), ok ? src + v_off : src, ok);
    }
    return;
  }
  for (int id = threadIdx.x; id < BN * CH; id += THREADS) {
    const int r = id / CH, c = id - r * CH;
    const int j = key0 + r;
    bool ok = j >= lo && j < hi;
    const bf16* src = g.kv_pages;
    if (ok) {
      const int lp = j / g.page_size;
      const int pg = g.table[lp];
      ok = pg >= 0 && pg < g.n_pages;
      if (ok) src = g.kv_pages + ((((size_t)pg * 2) * g.nkv + g.kvh) * g.page_size + (j - lp * g.page_size)) * D + c * 8;
    }
    cp_async16(ks + tile_off(r, c), src, ok);
    cp_async16(vs + tile_off(r, c), ok ? src + v_off : src, ok);
  }
}

// The page of the tile that starts at key0, for the fast path of load_kv_tile; -2 if tiles may straddle pages.
__device__ __forceinline__ int tile_page(const PageGeom& g, int key0, int hi) {
  if (g.page_size % BN != 0) return -2;
  return key0 < hi ? __ldg(g.table + key0 / g.page_size) : -1;
}

// Running softmax state of the two rows (lane/4 and lane/4 + 8) a thread holds of its warp's 16 rows.
struct RowState {
  float m[2], l[2];
  float o[DN][4];
};

// One warp, 16 rows, NT n-tiles of 8 keys starting at tile row `kb`: scores, mask, online softmax, P.V.
// key_base: absolute index of tile row 0.  Row i (0/1) of this thread sees keys in [row_lo[i], row_hi[i]].
template <int NT>
__device__ __forceinline__ void warp_tile(RowState& st, const uint32_t (&qf)[KS][4], const bf16* ks, const bf16* vs,
                                          int kb, int key_base, const int (&row_lo)[2], const int (&row_hi)[2],
                                          float scale_log2) {
  const int lane = threadIdx.x & 31;
  float s[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
  for (int k = 0; k < KS; ++k) {
#pragma unroll
    for (int j = 0; j < NT; j += 2) {
      uint32_t b[4];
      // matrices: (keys 8j.., chunk 2k), (keys 8j.., 2k+1), (keys 8(j+1).., 2k), (keys 8(j+1).., 2k+1)
      ldmatrix_x4(b, ks + tile_off(kb + 8 * j + (lane & 7) + ((lane >> 4) << 3), 2 * k + ((lane >> 3) & 1)));
      mma_bf16(s[j], qf[k], b[0], b[1]);
      mma_bf16(s[j + 1], qf[k], b[2], b[3]);
    }
  }
  // mask and the tile's row maxima
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key_base + kb + 8 * j + ((lane & 3) << 1) + (e & 1);
      const int i = e >> 1;
      const float v = (key >= row_lo[i] && key <= row_hi[i]) ? s[j][e] * scale_log2 : -INFINITY;
      s[j][e] = v;
      mx[i] = fmaxf(mx[i], v);
    }
  }
  float alpha[2], ref[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
    const float m_new = fmaxf(st.m[i], mx[i]);
    ref[i] = m_new == -INFINITY ? 0.f : m_new;      // a row that has seen no key yet
    alpha[i] = exp2f(st.m[i] - ref[i]);
    st.m[i] = m_new;
    st.l[i] *= alpha[i];
  }
#pragma unroll
  for (int n = 0; n < DN; ++n) {
    st.o[n][0] *= alpha[0]; st.o[n][1] *= alpha[0];
    st.o[n][2] *= alpha[1]; st.o[n][3] *= alpha[1];
  }
  uint32_t pf[NT / 2][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const float p0 = exp2f(s[j][0] - ref[0]), p1 = exp2f(s[j][1] - ref[0]);
    const float p2 = exp2f(s[j][2] - ref[1]), p3 = exp2f(s[j][3] - ref[1]);
    // the sums use the probabilities as rounded for the tensor cores, so numerator and denominator agree
    const uint32_t lo = pack_bf16(p0, p1), hi = pack_bf16(p2, p3);
    const __nv_bfloat162 lo2 = *reinterpret_cast<const __nv_bfloat162*>(&lo);
    const __nv_bfloat162 hi2 = *reinterpret_cast<const __nv_bfloat162*>(&hi);
    st.l[0] += __low2float(lo2) + __high2float(lo2);
    st.l[1] += __low2float(hi2) + __high2float(hi2);
    pf[j >> 1][(j & 1) * 2 + 0] = lo;
    pf[j >> 1][(j & 1) * 2 + 1] = hi;
  }
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
#pragma unroll
    for (int n = 0; n < DN; n += 2) {
      uint32_t b[4];
      // transposed: (keys 16kk.., chunk n), (keys 16kk+8.., chunk n), (keys 16kk.., n+1), (keys 16kk+8.., n+1)
      ldmatrix_x4_trans(b, vs + tile_off(kb + 16 * kk + (lane & 7) + (((lane >> 3) & 1) << 3), n + (lane >> 4)));
      mma_bf16(st.o[n], pf[kk], b[0], b[1]);
      mma_bf16(st.o[n + 1], pf[kk], b[2], b[3]);
    }
  }
}

__device__ __forceinline__ void init_state(RowState& st) {
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;
#pragma unroll
  for (int n = 0; n < DN; ++n) st.o[n][0] = st.o[n][1] = st.o[n][2] = st.o[n][3] = 0.f;
}

// Load 16 rows of Q fragments for this warp from a staged Q tile (rows row0 .. row0+15).
__device__ __forceinline__ void load_q_frags(uint32_t (&qf)[KS][4], const bf16* qs, int row0) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int k = 0; k < KS; ++k)
    ldmatrix_x4(qf[k], qs + tile_off(row0 + (lane & 7) + (((lane >> 3) & 1) << 3), 2 * k + (lane >> 4)));
}

// ------------------------------------------------------------------------------------------------ prefill
// Each warp owns MTW row tiles of 16 rows (two for head sizes up to 128, where the accumulators fit the register
// file; one beyond), so every key and value fragment read from shared memory serves MTW row tiles.  The
// block's queries stay in shared memory and their fragments are fetched per K slice.  A 64-key tile is walked in
// two halves of 32 keys to keep the score registers few.
constexpr int MAX_MTW = D <= 128 ? 2 : 1;

template <int MTW>
struct PrefillState {
  float m[MTW][2], l[MTW][2];
  float o[MTW][DN][4];
};

template <int MTW>
__device__ __forceinline__ void warp_tile_prefill(PrefillState<MTW>& st, const bf16* qs, int qrow0, const bf16* ks, const bf16* vs,
                                                  int key_base, const int (&row_lo)[MTW][2], const int (&row_hi)[MTW][2],
                                                  int w_lo, int w_hi, float scale_log2) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int kb = h * 32;
    if (key_base + kb > w_hi || key_base + kb + 32 <= w_lo) continue;      // no row of this warp sees these keys
    float s[MTW][4][4];
#pragma unroll
    for (int mt = 0; mt < MTW; ++mt)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[mt][j][0] = s[mt][j][1] = s[mt][j][2] = s[mt][j][3] = 0.f;
#pragma unroll
    for (int k = 0; k < KS; ++k) {
      uint32_t a[MTW][4];
#pragma unroll
      for (int mt = 0; mt < MTW; ++mt)
        ldmatrix_x4(a[mt], qs + tile_off(qrow0 + mt * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), 2 * k + (lane >> 4)));
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        uint32_t b[4];
        ldmatrix_x4(b, ks + tile_off(kb + 8 * j + (lane & 7) + ((lane >> 4) << 3), 2 * k + ((lane >> 3) & 1)));
#pragma unroll
        for (int mt = 0; mt < MTW; ++mt) {
          mma_bf16(s[mt][j], a[mt], b[0], b[1]);
          mma_bf16(s[mt][j + 1], a[mt], b[2], b[3]);
        }
      }
    }
    uint32_t pf[MTW][2][4];
#pragma unroll
    for (int mt = 0; mt < MTW; ++mt) {
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key_base + kb + 8 * j + ((lane & 3) << 1) + (e & 1);
          const int i = e >> 1;
          const float v = (key >= row_lo[mt][i] && key <= row_hi[mt][i]) ? s[mt][j][e] * scale_log2 : -INFINITY;
          s[mt][j][e] = v;
          mx[i] = fmaxf(mx[i], v);
        }
      float alpha[2], ref[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        const float m_new = fmaxf(st.m[mt][i], mx[i]);
        ref[i] = m_new == -INFINITY ? 0.f : m_new;
        alpha[i] = exp2f(st.m[mt][i] - ref[i]);
        st.m[mt][i] = m_new;
        st.l[mt][i] *= alpha[i];
      }
#pragma unroll
      for (int n = 0; n < DN; ++n) {
        st.o[mt][n][0] *= alpha[0]; st.o[mt][n][1] *= alpha[0];
        st.o[mt][n][2] *= alpha[1]; st.o[mt][n][3] *= alpha[1];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float p0 = exp2f(s[mt][j][0] - ref[0]), p1 = exp2f(s[mt][j][1] - ref[0]);
        const float p2 = exp2f(s[mt][j][2] - ref[1]), p3 = exp2f(s[mt][j][3] - ref[1]);
        const uint32_t lo = pack_bf16(p0, p1), hi = pack_bf16(p2, p3);
        const __nv_bfloat162 lo2 = *reinterpret_cast<const __nv_bfloat162*>(&lo);
        const __nv_bfloat162 hi2 = *reinterpret_cast<const __nv_bfloat162*>(&hi);
        st.l[mt][0] += __low2float(lo2) + __high2float(lo2);
        st.l[mt][1] += __low2float(hi2) + __high2float(hi2);
        pf[mt][j >> 1][(j & 1) * 2 + 0] = lo;
        pf[mt][j >> 1][(j & 1) * 2 + 1] = hi;
      }
    }
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
      for (int n = 0; n < DN; n += 2) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vs + tile_off(kb + 16 * kk + (lane & 7) + (((lane >> 3) & 1) << 3), n + (lane >> 4)));
#pragma unroll
        for (int mt = 0; mt < MTW; ++mt) {
          mma_bf16(st.o[mt][n], pf[mt][kk], b[0], b[1]);
          mma_bf16(st.o[mt][n + 1], pf[mt][kk], b[2], b[3]);
        }
      }
    }
  }
}

template <int MTW>
__global__ void __launch_bounds__(THREADS, MTW == 2 ? 2 : (D <= 128 ? 3 : 1)) attn_prefill_kernel(
    const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
    const bf16* __restrict__ kv_pages, const int* __restrict__ block_table, int bt_stride,
    const int* __restrict__ cu_q, const int* __restrict__ kv_len, int n_seqs, int nq, int nkv, int page_size,
    int n_pages, int window, float scale_log2, int tokens_per_block) {
  constexpr int PF_ROWS = 64 * MTW;                          // rows (token x head of the group) per block
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qbuf = reinterpret_cast<bf16*>(smem_raw);            // [PF_ROWS rows]
  bf16* kbuf = qbuf + MTW * TILE_ELEMS;                      // [2][tile]
  bf16* vbuf = kbuf + 2 * TILE_ELEMS;                        // [2][tile]
  pdl_prologue();
  const int G = nq / nkv;
  // blocks are numbered KV head fastest, then tile; within a request the last tokens (the longest walks over
  // the keys) get the lowest numbers, so the heavy blocks start first and the light ones fill the tail
  const int kvh = blockIdx.x;
  int seq = -1, tile = blockIdx.y;
  for (int s = 0; s < n_seqs; ++s) {
    const int n = cu_q[s + 1] - cu_q[s];
    if (n == 1) continue;                                    // single tokens belong to the decode kernel
    const int nt = (n + tokens_per_block - 1) / tokens_per_block;
    if (tile < nt) { seq = s; tile = nt - 1 - tile; break; }
    tile -= nt;
  }
  if (seq < 0) return;
  const int n_new = cu_q[seq + 1] - cu_q[seq];
  const int total = kv_len[seq];
  const int t0 = tile * tokens_per_block;
  const int tq_n = min(tokens_per_block, n_new - t0);
  const int pos0 = total - n_new + t0;                       // position of the block's first token
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int WROWS = 16 * MTW;                            // rows per warp

  // stage Q: row R = token * G + head
  for (int id = threadIdx.x; id < PF_ROWS * CH; id += THREADS) {
    const int R = id / CH, c = id - R * CH;
    const int tq = R / G, g = R - tq * G;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tq < tq_n)
      v = *reinterpret_cast<const uint4*>(q + (size_t)(cu_q[seq] + t0 + tq) * q_stride + (size_t)(kvh * G + g) * D + c * 8);
    *reinterpret_cast<uint4*>(qbuf + tile_off(R, c)) = v;
  }

  int row_lo[MTW][2], row_hi[MTW][2];
#pragma unroll
  for (int mt = 0; mt < MTW; ++mt)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int R = warp * WROWS + mt * 16 + (lane >> 2) + 8 * i;
      const int tq = R / G;
      if (tq < tq_n) {
        row_hi[mt][i] = pos0 + tq;
        row_lo[mt][i] = window > 0 ? max(0, row_hi[mt][i] - window + 1) : 0;
      } else {
        row_hi[mt][i] = -1;
        row_lo[mt][i] = 0;
      }
    }
  const int pos_hi = pos0 + tq_n - 1;
  const int first_key = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int key_begin = (first_key / BN) * BN;
  const int n_tiles = (pos_hi - key_begin) / BN + 1;
  // this warp's rows: the span of keys any of them sees (warp-uniform, so whole tiles can be skipped)
  const int w_tq_lo = (warp * WROWS) / G, w_tq_hi = min((warp * WROWS + WROWS - 1) / G, tq_n - 1);
  const int w_hi = w_tq_lo < tq_n ? pos0 + w_tq_hi : -1;
  const int w_lo = window > 0 ? max(0, pos0 + w_tq_lo - window + 1) : 0;

  PageGeom geom{kv_pages, block_table + (size_t)seq * bt_stride, nkv, kvh, page_size, n_pages};
  PrefillState<MTW> st;
#pragma unroll
  for (int mt = 0; mt < MTW; ++mt) {
    st.m[mt][0] = st.m[mt][1] = -INFINITY;
    st.l[mt][0] = st.l[mt][1] = 0.f;
#pragma unroll
    for (int n = 0; n < DN; ++n) st.o[mt][n][0] = st.o[mt][n][1] = st.o[mt][n][2] = st.o[mt][n][3] = 0.f;
  }
  int page_next = tile_page(geom, key_begin + BN, pos_hi + 1);
  load_kv_tile(kbuf, vbuf, geom, key_begin, first_key, pos_hi + 1, tile_page(geom, key_begin, pos_hi + 1));
  cp_async_commit();
  for (int it = 0; it < n_tiles; ++it) {
    const int stage = it & 1;
    if (it + 1 < n_tiles) {
      const int page = page_next;
      page_next = tile_page(geom, key_begin + (it + 2) * BN, pos_hi + 1);     // looked up one tile ahead
      load_kv_tile(kbuf + (stage ^ 1) * TILE_ELEMS, vbuf + (stage ^ 1) * TILE_ELEMS, geom, key_begin + (it + 1) * BN,
                   first_key, pos_hi + 1, page);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();                                          // also makes the staged queries visible (first pass)
    const int key_base = key_begin + it * BN;
    if (key_base <= w_hi && key_base + BN > w_lo)
      warp_tile_prefill<MTW>(st, qbuf, warp * WROWS, kbuf + stage * TILE_ELEMS, vbuf + stage * TILE_ELEMS, key_base, row_lo,
                        row_hi, w_lo, w_hi, scale_log2);
    __syncthreads();
  }
#pragma unroll
  for (int mt = 0; mt < MTW; ++mt)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float l = st.l[mt][i];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      const int R = warp * WROWS + mt * 16 + (lane >> 2) + 8 * i;
      const int tq = R / G, g = R - tq * G;
      if (tq >= tq_n) continue;
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      bf16* dst = out + (size_t)(cu_q[seq] + t0 + tq) * out_stride + (size_t)(kvh * G + g) * D + ((lane & 3) << 1);
#pragma unroll
      for (int n = 0; n < DN; ++n)
        *reinterpret_cast<uint32_t*>(dst + n * 8) = pack_bf16(st.o[mt][n][2 * i] * inv, st.o[mt][n][2 * i + 1] * inv);
    }
}

// ------------------------------------------------------------------------------------------------ decode
// Single decoded tokens, stream-K: the work is the flat list of 64-key tiles of every (request with one new
// token, block of up to 16 query heads of one KV head), request-major.  The grid is a fixed number of blocks
// (a few per SM); block c owns the contiguous tiles [c * T / G, (c + 1) * T / G), so every block reads the
// same number of keys whatever the batch looks like, and a short batch spreads over as many blocks as it has
// tiles.  A block walks its range piece by piece (a piece: its tiles of one (request, head block)).  If a
// piece is the whole of its (request, head block) the block writes the output; otherwise it stores (max,
// sum, unnormalised output) to scratch, and the block that arrives last at that (request, head block)'s
// counter merges all pieces in block order and writes the output.  No block waits for another.
constexpr int MAX_DECODE_SEQS = 512;
constexpr int MIN_TILES = 2;
#ifndef NHV_ATTN_DECODE_STAGES
#define NHV_ATTN_DECODE_STAGES 2
#endif
constexpr int DSTAGES = NHV_ATTN_DECODE_STAGES;              // key/value tiles in the decode kernel's ring
constexpr int Q_ELEMS = 16 * ROW_CH * 8;

__device__ __forceinline__ int tile_owner(long long u, long long total, int G) { return (int)(((u + 1) * G - 1) / total); }

// Decoding straight from the projection's output: with `qkv` set, the kernel itself norms and rotates the new
// token's query and key heads (the arithmetic and rounding of qk_norm_rope_store.cu: per-head RMS in fp32, rounded
// to bfloat16, times the weight, rounded, rotated in fp32, rounded) instead of reading `q` and finding the new
// key and value in the cache; the block that holds a request's last tile puts the new key and value into its
// tile, and one block per (request, KV head) also stores them in the cache for the steps to come (store = 0: a
// layer that reads another layer's cache; its keys and values are in the cache already).  One launch less per layer.  Head sizes that are multiples of 32 with rotary_dim a multiple of D / 16.
struct FusedQK {
  const bf16* qkv;          // [tokens, (nq + 2 nkv) * D]; null: the plain form
  const bf16* q_w;          // [D] or null (no norm)
  const bf16* k_w;
  const float* cos_sin;     // [max_position, rotary_dim]: cos then sin halves; null: nothing rotates
  const int* positions;     // [tokens]
  const int* slot_mapping;  // [tokens] slot of the new key and value in the pool
  int qkv_stride, rotary_dim, max_position, store;
  float eps, weight_offset;
};

constexpr int FVEC = D % 32 == 0 ? D / 32 : 1;               // elements of a head per lane

// One head of the new token in this warp: lane l gets elements [l * FVEC, (l + 1) * FVEC).
__device__ __forceinline__ void fused_head(float (&v)[FVEC], const bf16* src, const bf16* w, const float* cs,
                                           const FusedQK& f, int lane) {
#pragma unroll
  for (int k = 0; k < FVEC; ++k) v[k] = __bfloat162float(src[lane * FVEC + k]);
  if (w) {
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < FVEC; ++k) ss = fmaf(v[k], v[k], ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = 1.0f / sqrtf(ss / (float)D + f.eps);
#pragma unroll
    for (int k = 0; k < FVEC; ++k) {
      const float n = __bfloat162float(__float2bfloat16_rn(v[k] * rstd));
      v[k] = __bfloat162float(__float2bfloat16_rn(n * (__bfloat162float(w[lane * FVEC + k]) + f.weight_offset)));
    }
  }
  if (cs) {
    const int half = f.rotary_dim >> 1, half_lanes = half / FVEC;
    const bool first = lane < half_lanes, in_rot = lane < 2 * half_lanes;
    const int partner = (first ? lane + half_lanes : lane - half_lanes) & 31;
    const int i0 = (first ? lane : lane - half_lanes) * FVEC;
#pragma unroll
    for (int k = 0; k < FVEC; ++k) {
      const float other = __shfl_sync(0xffffffffu, v[k], partner);
      if (in_rot) {
        const float co = cs[i0 + k], si = cs[half + i0 + k];
        v[k] = first ? v[k] * co - other * si : v[k] * co + other * si;
      }
    }
  }
}

__global__ void __launch_bounds__(THREADS, D <= 128 ? (DSTAGES == 2 ? 3 : 2) : 1) attn_decode_kernel(
    const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride, const bf16* __restrict__ kv_pages,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ kv_len,
    float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters, int n_seqs, int nq, int nkv,
    int page_size, int n_pages, int window, float scale_log2, int max_pieces, const FusedQK fq) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* kbuf = reinterpret_cast<bf16*>(smem_raw);
  bf16* vbuf = kbuf + DSTAGES * TILE_ELEMS;
  bf16* qbuf = vbuf + DSTAGES * TILE_ELEMS;                   // [16 rows][padded d]
  __shared__ __align__(16) bf16 s_new[2][D];                  // the new token's key and value (fused form)
  __shared__ unsigned short s_cnt[MAX_DECODE_SEQS];          // tiles of each request (0: not a single-token request)
  __shared__ int s_prefix[MAX_DECODE_SEQS + 1];
  __shared__ int s_flag;
  // The plain form reads the keys that the kernel before it stored, so it waits for that kernel first.  The form
  // that works from the projection's output finds its work and starts fetching the first tiles of old keys
  // (written by earlier steps) while the projection winds down, and waits only before it reads qkv.
  pdl_launch_dependents();
  bool waited = fq.qkv == nullptr || !fq.store;    // a layer that reads another layer's cache reads keys of this step
  if (waited) pdl_wait();
  const int G = nq / nkv;
  const int rows_per = min(G, 16);
  const int chunks = (G + 15) / 16;                          // groups of more than 16 heads: several head blocks
  const int H = nkv * chunks;                                // head blocks per request
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int sq = threadIdx.x; sq < n_seqs; sq += THREADS) {
    int nt = 0;
    if (cu_q[sq + 1] - cu_q[sq] == 1) {
      const int total = kv_len[sq];
      const int lo = window > 0 ? max(0, total - window) : 0;
      nt = (total - 1) / BN - lo / BN + 1;
    }
    s_cnt[sq] = (unsigned short)min(nt, 65535);
  }
  __syncthreads();
  if (warp == 0) {                                           // prefix sums: each lane a run of requests, then a warp scan
    const int per = (n_seqs + 31) / 32;
    const int b0 = min(lane * per, n_seqs), b1 = min(b0 + per, n_seqs);
    int sum = 0;
    for (int i = b0; i < b1; ++i) sum += s_cnt[i];
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - sum;
    for (int i = b0; i < b1; ++i) { s_prefix[i] = run; run += s_cnt[i]; }
    if (lane == 31) s_prefix[n_seqs] = incl;
  }
  __syncthreads();
  const long long T = (long long)H * s_prefix[n_seqs];
  // at least MIN_TILES tiles per block (a short batch uses fewer blocks), so that every block has work, the
  // owners of consecutive tiles are consecutive blocks and a request is cut into few pieces
  const int NB = (int)max(1LL, min((long long)gridDim.x, T / MIN_TILES));
  const int c = blockIdx.x;
  if (c >= NB || T == 0) return;
  const long long u0 = (long long)c * T / NB, u1 = (long long)(c + 1) * T / NB;

  long long u = u0;
  while (u < u1) {
    // which request, head block and tile is u?
    int lo_s = 0, hi_s = n_seqs;
    while (lo_s < hi_s) {
      const int mid = (lo_s + hi_s) >> 1;
      if ((long long)H * s_prefix[mid + 1] > u) hi_s = mid; else lo_s = mid + 1;
    }
    const int seq = lo_s;
    const int nt = s_cnt[seq];
    const long long seq_base = (long long)H * s_prefix[seq];
    const int hb = (int)((u - seq_base) / nt), t_begin = (int)((u - seq_base) - (long long)hb * nt);
    const long long piece_first = seq_base + (long long)hb * nt;          // first tile of this (request, head block)
    const int n_tiles = (int)(min(u1, piece_first + nt) - u);
    const bool whole = t_begin == 0 && n_tiles == nt;
    u += n_tiles;

    const int kvh = hb / chunks, g0 = (hb - kvh * chunks) * 16;
    const int gn = min(rows_per, G - g0);
    const int total = kv_len[seq];
    const int lo = window > 0 ? max(0, total - window) : 0;
    const int key_begin = (lo / BN + t_begin) * BN;
    const size_t tok = cu_q[seq];
    PageGeom geom{kv_pages, block_table + (size_t)seq * bt_stride, nkv, kvh, page_size, n_pages};

    // the first tiles are on their way while q is staged
#pragma unroll
    for (int pre = 0; pre < DSTAGES - 1; ++pre) {
      if (pre < n_tiles)
        load_kv_tile(kbuf + pre * TILE_ELEMS, vbuf + pre * TILE_ELEMS, geom, key_begin + pre * BN, lo, total,
                     tile_page(geom, key_begin + pre * BN, total));
      cp_async_commit();
    }
    int page_next = tile_page(geom, key_begin + (DSTAGES - 1) * BN, total);
    const bool fused = fq.qkv != nullptr;
    const bool has_last = t_begin + n_tiles == nt;            // this piece ends with the request's newest key
    if (!waited) {
      pdl_wait();
      waited = true;
    }
    if (!fused) {
      for (int id = threadIdx.x; id < 16 * CH; id += THREADS) {
        const int R = id / CH, cc = id - R * CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (R < gn) v = *reinterpret_cast<const uint4*>(q + tok * q_stride + (size_t)(kvh * G + g0 + R) * D + cc * 8);
        *reinterpret_cast<uint4*>(qbuf + tile_off(R, cc)) = v;
      }
    } else {
      const bf16* row = fq.qkv + tok * fq.qkv_stride;
      const float* cs = nullptr;
      if (fq.cos_sin) {
        int pos = fq.positions[tok];
        pos = pos < 0 ? 0 : (pos >= fq.max_position ? fq.max_position - 1 : pos);
        cs = fq.cos_sin + (size_t)pos * fq.rotary_dim;
      }
      for (int R = warp; R < 16; R += THREADS / 32) {         // a warp per query head of the group
        float v[FVEC];
        if (R < gn) {
          fused_head(v, row + (size_t)(kvh * G + g0 + R) * D, fq.q_w, cs, fq, lane);
        } else {
#pragma unroll
          for (int k = 0; k < FVEC; ++k) v[k] = 0.f;
        }
        const int e0 = lane * FVEC;
#pragma unroll
        for (int k = 0; k < FVEC; ++k)      // a lane's elements may straddle two 16-byte chunks (head sizes 96, 160, 192, 224)
          qbuf[tile_off(R, (e0 + k) >> 3) + ((e0 + k) & 7)] = __float2bfloat16_rn(v[k]);
      }
      if (has_last && fq.store && warp < 2) {                 // warp 0: the new key; warp 1: the new value
        float v[FVEC];
        const bf16* src = row + (size_t)(nq + (warp == 0 ? 0 : nkv) + kvh) * D;
        fused_head(v, src, warp == 0 ? fq.k_w : nullptr, warp == 0 ? cs : nullptr, fq, lane);
#pragma unroll
        for (int k = 0; k < FVEC; ++k) s_new[warp][lane * FVEC + k] = __float2bfloat16_rn(v[k]);
      }
    }
    __syncthreads();
    if (fused && has_last && fq.store && g0 == 0) {
      // one block per (request, KV head) stores the new key and value for the steps to come
      const int slot = fq.slot_mapping[tok];
      if (slot >= 0 && slot < n_pages * page_size) {
        const int pg = slot / page_size, off = slot - pg * page_size;
        for (int id = threadIdx.x; id < 2 * CH; id += THREADS) {
          const int kv = id / CH, cc = id - kv * CH;
          bf16* dst = const_cast<bf16*>(kv_pages) + ((((size_t)pg * 2 + kv) * nkv + kvh) * page_size + off) * D + cc * 8;
          *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&s_new[kv][cc * 8]);
        }
      }
    }
    uint32_t qf[KS][4];
    load_q_frags(qf, qbuf, 0);
    int row_lo[2], row_hi[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      row_lo[i] = lo;
      row_hi[i] = (lane >> 2) + 8 * i < gn ? total - 1 : -1;
    }
    RowState st;
    init_state(st);
    for (int it = 0; it < n_tiles; ++it) {
      const int stage = it % DSTAGES;
      const int nxt = it + DSTAGES - 1;
      if (nxt < n_tiles) {
        const int page = page_next;
        page_next = tile_page(geom, key_begin + (nxt + 1) * BN, total);          // looked up one tile ahead
        load_kv_tile(kbuf + (nxt % DSTAGES) * TILE_ELEMS, vbuf + (nxt % DSTAGES) * TILE_ELEMS, geom, key_begin + nxt * BN,
                     lo, total, page);
      }
      cp_async_commit();                                       // one group per iteration, empty or not
      cp_async_wait<DSTAGES - 1>();
      __syncthreads();
      const int key_base = key_begin + it * BN;
      if (fused && fq.store && has_last && it == n_tiles - 1) {
        // the cache does not hold the newest key and value yet (or is being written): take them from s_new
        const int r = total - 1 - key_base;
        for (int id = threadIdx.x; id < 2 * CH; id += THREADS) {
          const int kv = id / CH, cc = id - kv * CH;
          *reinterpret_cast<uint4*>((kv == 0 ? kbuf : vbuf) + stage * TILE_ELEMS + tile_off(r, cc)) =
              *reinterpret_cast<const uint4*>(&s_new[kv][cc * 8]);
        }
        __syncthreads();
      }
      if (key_base + warp * 16 < total && key_base + warp * 16 + 16 > lo)
        warp_tile<2>(st, qf, kbuf + stage * TILE_ELEMS, vbuf + stage * TILE_ELEMS, warp * 16, key_base, row_lo, row_hi, scale_log2);
      __syncthreads();
    }
    cp_async_wait<0>();
    // merge the 4 warps (each saw a quarter of every tile) through shared memory
    float* mo = reinterpret_cast<float*>(smem_raw);            // [4 warps][16 rows][D]
    float* mml = mo + 4 * 16 * D;                              // [4][16][2]
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float l = st.l[i];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      const int R = (lane >> 2) + 8 * i;
      float* dst = mo + ((size_t)warp * 16 + R) * D + ((lane & 3) << 1);
#pragma unroll
      for (int n = 0; n < DN; ++n) {
        dst[n * 8] = st.o[n][2 * i];
        dst[n * 8 + 1] = st.o[n][2 * i + 1];
      }
      if ((lane & 3) == 0) {
        mml[(warp * 16 + R) * 2] = st.m[i];
        mml[(warp * 16 + R) * 2 + 1] = l;
      }
    }
    __syncthreads();
    const size_t unit = (size_t)seq * H + hb;                  // this (request, head block)
    int pieces = 1, piece = 0;
    if (!whole) {
      const int first_owner = tile_owner(piece_first, T, NB);
      pieces = tile_owner(piece_first + nt - 1, T, NB) - first_owner + 1;
      piece = min(c - first_owner, max_pieces - 1);          // never beyond the scratch, whatever the caller passed
    }
    float* po = part_o + (unit * max_pieces + piece) * rows_per * D;
    float* pml = part_ml + (unit * max_pieces + piece) * rows_per * 2;
    for (int id = threadIdx.x; id < gn * D; id += THREADS) {
      const int R = id / D, cc = id - R * D;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) M = fmaxf(M, mml[(w * 16 + R) * 2]);
      float acc = 0.f, L = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = mml[(w * 16 + R) * 2];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
        acc += mo[((size_t)w * 16 + R) * D + cc] * f;
        L += mml[(w * 16 + R) * 2 + 1] * f;
      }
      if (whole) {
        out[tok * out_stride + (size_t)(kvh * G + g0 + R) * D + cc] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
      } else {
        po[R * D + cc] = acc;
        if (cc == 0) { pml[R * 2] = M; pml[R * 2 + 1] = L; }
      }
    }
    if (!whole) {
      // the arrival is a release (the barrier before it orders the other threads' stores before it) and an
      // acquire (the last piece to arrive may read the others), so no thread stands at a fence
      __syncthreads();
      if (threadIdx.x == 0) {
        int old;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;\n" : "=r"(old) : "l"(counters + unit) : "memory");
        s_flag = old;
      }
      __syncthreads();
      if (s_flag == pieces - 1) {                              // the last piece to arrive: merge all, in piece order
        const float* bo = part_o + unit * max_pieces * rows_per * D;
        const float* bml = part_ml + unit * max_pieces * rows_per * 2;
        // the pieces' (max, sum) first: few numbers, loaded side by side into shared memory
        float* sml = reinterpret_cast<float*>(smem_raw);       // [pieces][gn][2]
        for (int id = threadIdx.x; id < pieces * gn * 2; id += THREADS) {
          const int pc = id / (gn * 2), rem = id - pc * (gn * 2);
          sml[id] = __ldcg(bml + (size_t)pc * rows_per * 2 + rem);
        }
        __syncthreads();
        for (int id = threadIdx.x; id < gn * (D / 4); id += THREADS) {
          const int R = id / (D / 4), c4 = id - R * (D / 4);
          float M = -INFINITY;
          for (int pc = 0; pc < pieces; ++pc) M = fmaxf(M, sml[(pc * gn + R) * 2]);
          float L = 0.f;
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int p0 = 0; p0 < pieces; p0 += 8) {             // eight independent 16-byte loads in flight
            float4 t[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              t[j] = __ldcg(reinterpret_cast<const float4*>(bo + ((size_t)min(p0 + j, pieces - 1) * rows_per + R) * D) + c4);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (p0 + j >= pieces) break;
              const float m = sml[((p0 + j) * gn + R) * 2];
              if (m == -INFINITY) continue;
              const float f = exp2f(m - M);
              acc.x += t[j].x * f; acc.y += t[j].y * f; acc.z += t[j].z * f; acc.w += t[j].w * f;
              L += sml[((p0 + j) * gn + R) * 2 + 1] * f;
            }
          }
          const float inv = L > 0.f ? 1.0f / L : 0.f;
          bf16* dst = out + tok * out_stride + (size_t)(kvh * G + g0 + R) * D + c4 * 4;
          *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
        }
        if (threadIdx.x == 0) counters[unit] = 0;              // ready for the next launch
      }
    }
    __syncthreads();                                           // the tile buffers are reused by the next piece
  }
}

template <int MTW>
constexpr size_t prefill_smem_bytes() { return (size_t)(MTW + 4) * TILE_ELEMS * sizeof(bf16); }   // the queries, two K and two V tiles
constexpr size_t kDecodeSmemBytes = (size_t)(2 * DSTAGES * TILE_ELEMS + Q_ELEMS) * sizeof(bf16);
static_assert((size_t)4 * TILE_ELEMS * sizeof(bf16) >= (size_t)(4 * 16 * D + 4 * 16 * 2) * sizeof(float),
              "merge buffer must fit the tile buffers");

}  // namespace

#define NHV_CAT2(a, b) a##b
#define NHV_CAT(a, b) NHV_CAT2(a, b)
#define NHV_FN(name) NHV_CAT(name, NHV_ATTN_D)

static char g_err[384] = "";
#define ATT_REQUIRE(cond, ...)                      \
  do {                                              \
    if (!(cond)) {                                  \
      snprintf(g_err, sizeof(g_err), __VA_ARGS__);  \
      return 1;                                     \
    }                                               \
  } while (0)

NHV_API const char* NHV_FN(nhv_attn_mma_last_error_d)() { return g_err; }
NHV_API int NHV_FN(nhv_attn_mma_tile_d)() { return BN; }

// The step's attention in bfloat16: prompt portions, then single tokens.
// n_prefill_tokens / n_decode_seqs: how many of the step's tokens / requests are of each kind (0 skips that
// launch).  Decoding needs scratch: scratch_o [n_seqs * head_blocks * max_pieces * rows * D] floats, scratch_ml
// [... * rows * 2] floats and counters [n_seqs * head_blocks] ints that are zero (the kernel leaves them zero),
// with head_blocks = nkv * ceil(group / 16), rows = min(group, 16), max_pieces >= ceil(longest context / 64) + 1.
// decode_blocks: the grid of the decode kernel (a few blocks per SM).
static int attention_launch(const void* q, int q_stride, void* out, int out_stride, const void* kv_pages,
                            const int* block_table, int bt_stride, const int* cu_q, const int* kv_len,
                            int n_seqs, int n_prefill_tokens, int n_prefill_seqs, int n_decode_seqs, int nq,
                            int nkv, int page_size, int n_pages, int window, float scale, float* scratch_o,
                            float* scratch_ml, int* counters, int max_pieces, int decode_blocks,
                            const FusedQK& fq, cudaStream_t stream) {
  ATT_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads do not divide into %d KV heads", nq, nkv);
  ATT_REQUIRE(page_size > 0 && n_pages > 0 && bt_stride > 0, "attention: bad page geometry");
  ATT_REQUIRE(q_stride % 8 == 0 && out_stride % 4 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)kv_pages % 16) == 0 &&
                  ((uintptr_t)out % 8) == 0,
              "attention: q and the pages must be 16-byte aligned, the output 8-byte aligned");
  const int G = nq / nkv;
  const float scale_log2 = scale * LOG2E;
  static bool attr_set = false;
  static int sms = 0;
  if (!attr_set) {
    bool ok = cudaFuncSetAttribute(attn_prefill_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)prefill_smem_bytes<1>()) == cudaSuccess &&
              cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDecodeSmemBytes) == cudaSuccess;
    if constexpr (MAX_MTW == 2)
      ok = ok && cudaFuncSetAttribute(attn_prefill_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)prefill_smem_bytes<2>()) == cudaSuccess;
    int dev = 0;
    ok = ok && cudaGetDevice(&dev) == cudaSuccess &&
         cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess;
    if (!ok) {
      snprintf(g_err, sizeof(g_err), "attention: cannot reserve %zu bytes of shared memory", prefill_smem_bytes<MAX_MTW>());
      return 2;
    }
    attr_set = true;
  }
  if (n_prefill_tokens > 0) {
    ATT_REQUIRE(G <= 64, "attention: a group of %d query heads is beyond the 64 rows of a block", G);
    // 128 rows a block (every key fragment serves two row tiles) when that still fills the device well;
    // a row's result is the same either way: the same keys in the same order
    bool wide = false;
    if constexpr (MAX_MTW == 2) wide = (long long)nkv * (n_prefill_tokens / (128 / G)) >= 3LL * sms;
    const int tokens_per_block = (wide ? 128 : 64) / G;
    const int max_tiles = n_prefill_tokens / tokens_per_block + n_prefill_seqs;
    ATT_REQUIRE(max_tiles <= 65535, "attention: %d tiles of new tokens are beyond the grid's reach", max_tiles);
    dim3 grid(nkv, max_tiles);
    if constexpr (MAX_MTW == 2) {
      if (wide)
        nhv_launch(attn_prefill_kernel<2>, grid, THREADS, prefill_smem_bytes<2>(), stream,
            (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kv_pages, block_table, bt_stride, cu_q, kv_len,
            n_seqs, nq, nkv, page_size, n_pages, window, scale_log2, tokens_per_block);
    }
    if (!wide)
      nhv_launch(attn_prefill_kernel<1>, grid, THREADS, prefill_smem_bytes<1>(), stream,
          (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kv_pages, block_table, bt_stride, cu_q, kv_len,
          n_seqs, nq, nkv, page_size, n_pages, window, scale_log2, tokens_per_block);
  }
  if (n_decode_seqs > 0) {
    ATT_REQUIRE(scratch_o && scratch_ml && counters && max_pieces > 0 && decode_blocks > 0,
                "attention: decoding needs scratch memory for the pieces of split requests");
    ATT_REQUIRE(n_seqs <= MAX_DECODE_SEQS, "attention: %d requests in a step, the decode kernel plans for up to %d",
                n_seqs, MAX_DECODE_SEQS);
    static int resident = 0;                                   // blocks of the decode kernel that fit the device at once
    if (resident == 0) {
      int per_sm = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_kernel, THREADS, kDecodeSmemBytes) != cudaSuccess || per_sm < 1)
        per_sm = 1;
      resident = per_sm * sms;
    }
    decode_blocks = resident;
    nhv_launch(attn_decode_kernel, dim3(decode_blocks), THREADS, kDecodeSmemBytes, stream,
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kv_pages, block_table, bt_stride, cu_q, kv_len,
        scratch_o, scratch_ml, counters, n_seqs, nq, nkv, page_size, n_pages, window, scale_log2, max_pieces, fq);
  }
  const cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    snprintf(g_err, sizeof(g_err), "attention: launch failed: %s", cudaGetErrorString(e));
    return 2;
  }
  return 0;
}

NHV_API int NHV_FN(nhv_attn_mma_d)(const void* q, int q_stride, void* out, int out_stride, const void* kv_pages,
                                   const int* block_table, int bt_stride, const int* cu_q, const int* kv_len,
                                   int n_seqs, int n_prefill_tokens, int n_prefill_seqs, int n_decode_seqs, int nq,
                                   int nkv, int page_size, int n_pages, int window, float scale, float* scratch_o,
                                   float* scratch_ml, int* counters, int max_pieces, int decode_blocks,
                                   cudaStream_t stream) {
  FusedQK none = {};
  return attention_launch(q, q_stride, out, out_stride, kv_pages, block_table, bt_stride, cu_q, kv_len, n_seqs,
                          n_prefill_tokens, n_prefill_seqs, n_decode_seqs, nq, nkv, page_size, n_pages, window, scale,
                          scratch_o, scratch_ml, counters, max_pieces, decode_blocks, none, stream);
}

// 1 if this head size has the form of the decode kernel that works from the projection's output.
NHV_API int NHV_FN(nhv_attn_mma_can_fuse_d)() { return D % 32 == 0 ? 1 : 0; }

// A step of single tokens only, straight from the projection's output qkv [tokens, (nq + 2 nkv) * D]: the kernel
// norms and rotates the query and key heads itself and (store != 0) puts the new keys and values into the cache;
// what qk_norm_rope_store would have done before it.  q_w / k_w null: no norm; cos_sin null: no rotation.
NHV_API int NHV_FN(nhv_attn_mma_decode_fused_d)(const void* qkv, int qkv_stride, void* out, int out_stride, void* kv_pages,
                                                const int* block_table, int bt_stride, const int* cu_q, const int* kv_len,
                                                int n_seqs, int nq, int nkv, int page_size, int n_pages, int window,
                                                float scale, float* scratch_o, float* scratch_ml, int* counters,
                                                int max_pieces, const void* q_w, const void* k_w, const float* cos_sin,
                                                const int* positions, const int* slot_mapping, int rotary_dim,
                                                int max_position, int store, float eps, float weight_offset,
                                                cudaStream_t stream) {
  ATT_REQUIRE(D % 32 == 0, "attention: the fused decode form takes head sizes in steps of 32, not %d", D);
  ATT_REQUIRE(qkv != nullptr && qkv_stride % 8 == 0 && ((uintptr_t)qkv % 16) == 0, "attention: qkv must be 16-byte aligned");
  ATT_REQUIRE(!cos_sin || (positions && rotary_dim > 0 && rotary_dim <= D && rotary_dim % (2 * FVEC) == 0),
              "attention: the fused decode form rotates in steps of %d elements, rotary_dim is %d", 2 * FVEC, rotary_dim);
  ATT_REQUIRE(!store || slot_mapping, "attention: storing the new keys needs the slot mapping");
  FusedQK fq;
  fq.qkv = (const bf16*)qkv;
  fq.q_w = (const bf16*)q_w;
  fq.k_w = (const bf16*)k_w;
  fq.cos_sin = cos_sin;
  fq.positions = positions;
  fq.slot_mapping = slot_mapping;
  fq.qkv_stride = qkv_stride;
  fq.rotary_dim = rotary_dim;
  fq.max_position = max_position;
  fq.store = store;
  fq.eps = eps;
  fq.weight_offset = weight_offset;
  return attention_launch(qkv, qkv_stride, out, out_stride, kv_pages, block_table, bt_stride, cu_q, kv_len, n_seqs, 0, 0,
                          n_seqs, nq, nkv, page_size, n_pages, window, scale, scratch_o, scratch_ml, counters, max_pieces,
                          1, fq, stream);
}
