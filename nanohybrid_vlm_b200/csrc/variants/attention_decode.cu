// bfloat16 attention of single decoded tokens over cache pages, for head sizes in steps of 64 and pages that are a
// multiple of 32 keys; compiled once per head size (-DNHV_ATTN_D=<head size>).  Replaces the library call at
// nanovllm/layers/attention.py:72-74 (flash_attn_with_kvcache).
//
// Decoding reads every key and value of every live request once and computes almost nothing, so the kernel is built
// around keeping HBM busy:
//
//  * Persistent, one block per SM.  The work is the flat list of 32-key tiles of every (request with one new token,
//    block of up to 16 query heads of one KV head), request-major, each (request, head block) preceded by
//    PIECE_COST places that stand for what a piece costs beside its tiles; block c owns the contiguous places
//    [c * T / NB, (c + 1) * T / NB), so every SM has the same load whether the batch holds a few long requests,
//    many short ones or both.  Entries that only fill a batch up to a fixed shape (their token has no page) take
//    no place at all; their output rows are cleared.
//  * A producer warp streams its block's tiles through a ring of shared-memory stages with TMA tile copies straight
//    from the paged pool, a tile's keys and values in ONE copy: the pool is seen in four dimensions, [keys | values]
//    [column block of 64][row of the pool][64 columns], and a box of 2 x D/64 x 32 x 64 lands as the K tile followed
//    by the V tile, each column block by column block in the 128-byte swizzle (64 columns is the widest box that
//    swizzle takes, and what an SM's TMA unit can take is about nine copies a microsecond whatever they hold: with
//    a copy per 64-column block of K and of V the launch was bound by copies, not bytes).  Plain per-block copies,
//    no multicast; completion counted in bytes on an mbarrier.  The producer looks the pages of 32 tiles up at a
//    time and runs ahead of the consumers across the borders of requests, so the ring never drains: up to 12
//    stages of 2 * 32 * D * 2 bytes (192 KB at head size 128) are in flight per SM.
//  * The consumer warps (four for head sizes up to 128) take whole tiles in turn (tile t of the block goes to warp
//    t % NCW): no warp waits for another while a piece lasts.  mma.sync.m16n8k16 bf16 with fp32 accumulation, online
//    softmax in fp32 on base-2 exponents, the rows being the query heads of the group (padded to 16).  At the end
//    of a piece (a block's tiles of one (request, head block)) the four warps' states are merged through shared
//    memory.
//  * If a piece is the whole of its (request, head block) the block writes the output; otherwise it stores (max,
//    sum, unnormalised output) to scratch (a block has at most two such pieces: its first and its last), and the
//    block that arrives last at that (request, head block)'s counter merges all pieces in block order and writes
//    the output.  No block waits for another.
//
// Keys outside a request's range that a tile brings along (beyond its last key, before its window, stale or never
// written) never reach a result: their scores are replaced, not added to, and their value rows are cleared in
// shared memory before the product.
//
// What a piece costs beside its tiles is kept small: a block finds its first piece by a search and walks on from
// there with a cursor; the plan leaves each request's key count, token row and position in shared memory.
//
// With `qkv` given the kernel works from the projection's output: it norms and rotates the new token's query and key
// heads itself (the arithmetic and rounding of qk_norm_rope_store.cu), puts the new key and value into the tile that
// holds the request's last keys, and one block per (request, KV head) stores them in the cache.  In that form the
// producer starts fetching old keys before the kernel waits for its predecessor (programmatic dependent launch), and
// while a piece is at its tiles the rows of qkv and the cosines of the piece after it are copied to shared memory,
// so that only a block's first piece waits for them.
//
// Every wait on an mbarrier is bounded; one that runs out sets the file's error word.
#include <math.h>

#include <mutex>
#include <unordered_map>
#include <utility>

#define NHV_WAIT_LIMIT (1u << 22)
#include "../nhv_async.cuh"

#ifndef NHV_ATTN_D
#error "compile with -DNHV_ATTN_D=<head size>"
#endif

namespace {

constexpr int D = NHV_ATTN_D;
static_assert(D % 64 == 0 && D >= 64 && D <= 256, "head sizes 64, 128, 192 and 256");
constexpr int CH = D / 8;          // 16-byte chunks in a row
constexpr int DB = D / 64;         // 128-byte column blocks of a head (one TMA box each)
constexpr int BN = 32;             // keys per tile
constexpr int KS = D / 16;         // k-steps of Q.K^T
constexpr int DN = D / 8;          // n-tiles of P.V
constexpr int TILE_BYTES = BN * D * 2;                 // one K tile or one V tile
constexpr int STAGE_BYTES = 2 * TILE_BYTES;
// Consumer warps and ring stages.  A stage is always consumed by the same warp (STAGES is a multiple of NCW and
// tile number t of the block goes to warp t % NCW and stage t % STAGES): a warp's waits on one barrier then follow
// one another, so it can never ask for a phase while the one before it is still filling (a wait by parity cannot
// tell those two apart).  Every warp has two stages, so its next tile is on its way while it works on one.
constexpr int NCW = D <= 128 ? 4 : (D == 192 ? 3 : 2);
constexpr int STAGES_MIN = 2 * NCW;
// Groups of up to 8 query heads need only 8 rows of the merge buffer: the room goes to the ring (three stages a warp).
constexpr int STAGES_DEEP = D <= 128 ? 3 * NCW : STAGES_MIN;
constexpr int THREADS = (NCW + 1) * 32;
constexpr int Q_BYTES = 16 * D * 2;
constexpr int merge_bytes(int mrows) { return NCW * mrows * D * 4 + NCW * mrows * 2 * 4; }
constexpr int MAX_SEQS = 512;
constexpr size_t smem_bytes(int stages, int mrows) { return 1024 + (size_t)stages * STAGE_BYTES + merge_bytes(mrows) + Q_BYTES; }
// what the kernel declares beside that: the new key and value, the rows copied ahead, the plan's numbers per request
// (19 bytes each), barriers and flags
constexpr size_t static_bytes(int stages, int mrows) {
  return 2 * D * 2 + (mrows + 2) * D * 2 + D * 4 + (size_t)MAX_SEQS * 19 + 4 + stages * 20 + 64;
}
static_assert(smem_bytes(STAGES_MIN, 16) + static_bytes(STAGES_MIN, 16) <= 227 * 1024 &&
                  smem_bytes(STAGES_DEEP, 8) + static_bytes(STAGES_DEEP, 8) <= 227 * 1024,
              "ring, merge buffer, queries and the plan must fit one block's shared memory");
constexpr int MIN_TILES = 4;
// What a piece costs a block beside its tiles (the query heads' norm and rotation, the merge of the warps, the
// output), in tiles' worth of time: the blocks' shares are equal in tiles + PIECE_COST per (request, head block),
// so a block that gets many short requests gets fewer of them.
#ifndef NHV_PIECE_COST
#define NHV_PIECE_COST 8
#endif
constexpr int PIECE_COST = NHV_PIECE_COST;
constexpr float LOG2E = 1.4426950408889634f;

typedef __nv_bfloat16 bf16;

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
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(NCW * 32) : "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
// 16 bytes from global to shared memory without passing through registers; the thread goes on and asks later
__device__ __forceinline__ void copy16_async(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copies_async_wait() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

// Element offset of (row, 16-byte chunk) in a tile of `ROWS` rows as TMA lays it out: one box of 64 columns after
// the other, in a box rows of 128 bytes whose chunks are exchanged by chunk ^ (row & 7).
template <int ROWS>
__device__ __forceinline__ int tile_off(int row, int chunk) {
  return (chunk >> 3) * ROWS * 64 + row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
}

__device__ __forceinline__ int tile_owner(long long u, long long total, int G) { return (int)(((u + 1) * G - 1) / total); }

struct FusedQK {
  const bf16* qkv;          // [tokens, (nq + 2 nkv) * D]; null: the plain form, queries in q
  const bf16* q_w;          // [D] or null (no norm)
  const bf16* k_w;
  const float* cos_sin;     // [max_position, rotary_dim]: cos then sin halves; null: nothing rotates
  const int* positions;     // [tokens]
  const int* slot_mapping;  // [tokens] slot of the new key and value in the pool
  int qkv_stride, rotary_dim, max_position, store;
  float eps, weight_offset;
};

constexpr int FVEC = D / 32;                                 // elements of a head per lane

// One head of the new token in this warp: lane l gets elements [l * FVEC, (l + 1) * FVEC).  The load (one access
// of FVEC * 2 bytes) and what follows it (norm, rotation) apart, so that a second head's load can be on its way
// before the first head's is used.
struct alignas((FVEC * 2) & -(FVEC * 2)) HeadChunk { bf16 e[FVEC]; };   // 4, 8, 4 (head size 192) or 16 bytes
__device__ __forceinline__ void head_load(float (&v)[FVEC], const bf16* src, int lane) {
  const HeadChunk c = *reinterpret_cast<const HeadChunk*>(src + lane * FVEC);
#pragma unroll
  for (int k = 0; k < FVEC; ++k) v[k] = __bfloat162float(c.e[k]);
}
__device__ __forceinline__ void head_finish(float (&v)[FVEC], const bf16* w, const float* cs, const FusedQK& f, int lane) {
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
__device__ __forceinline__ void fused_head(float (&v)[FVEC], const bf16* src, const bf16* w, const float* cs,
                                           const FusedQK& f, int lane) {
  head_load(v, src, lane);
  head_finish(v, w, cs, f, lane);
}

// Running softmax state of the two rows (lane/4 and lane/4 + 8) a thread holds of the 16 rows.
struct RowState {
  float m[2], l[2];
  float o[DN][4];
};

// One warp, 16 rows, the 32 keys of a tile starting at tile row `kb`: scores, mask, online softmax, P.V.
// key_base: absolute index of tile row 0.  Row i (0/1) of this thread sees keys in [lo, row_hi[i]].
__device__ __forceinline__ void warp_half_tile(RowState& st, const uint32_t (&qf)[KS][4], const bf16* ks, const bf16* vs,
                                               int kb, int key_base, int lo, const int (&row_hi)[2], float scale_log2) {
  const int lane = threadIdx.x & 31;
  constexpr int NT = 4;
  float s[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
  for (int k = 0; k < KS; ++k) {
#pragma unroll
    for (int j = 0; j < NT; j += 2) {
      uint32_t b[4];
      // matrices: (keys 8j.., chunk 2k), (keys 8j.., 2k+1), (keys 8(j+1).., 2k), (keys 8(j+1).., 2k+1)
      ldmatrix_x4(b, ks + tile_off<BN>(kb + 8 * j + (lane & 7) + ((lane >> 4) << 3), 2 * k + ((lane >> 3) & 1)));
      mma_bf16(s[j], qf[k], b[0], b[1]);
      mma_bf16(s[j + 1], qf[k], b[2], b[3]);
    }
  }
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key_base + kb + 8 * j + ((lane & 3) << 1) + (e & 1);
      const int i = e >> 1;
      // a select, not a sum: whatever a key outside the range holds (stale numbers, NaN) is replaced
      const float v = (key >= lo && key <= row_hi[i]) ? s[j][e] * scale_log2 : -INFINITY;
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
    const uint32_t plo = pack_bf16(p0, p1), phi = pack_bf16(p2, p3);
    const __nv_bfloat162 lo2 = *reinterpret_cast<const __nv_bfloat162*>(&plo);
    const __nv_bfloat162 hi2 = *reinterpret_cast<const __nv_bfloat162*>(&phi);
    st.l[0] += __low2float(lo2) + __high2float(lo2);
    st.l[1] += __low2float(hi2) + __high2float(hi2);
    pf[j >> 1][(j & 1) * 2 + 0] = plo;
    pf[j >> 1][(j & 1) * 2 + 1] = phi;
  }
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
#pragma unroll
    for (int n = 0; n < DN; n += 2) {
      uint32_t b[4];
      // transposed: (keys 16kk.., chunk n), (keys 16kk+8.., chunk n), (keys 16kk.., n+1), (keys 16kk+8.., n+1)
      ldmatrix_x4_trans(b, vs + tile_off<BN>(kb + 16 * kk + (lane & 7) + (((lane >> 3) & 1) << 3), n + (lane >> 4)));
      mma_bf16(st.o[n], pf[kk], b[0], b[1]);
      mma_bf16(st.o[n + 1], pf[kk], b[2], b[3]);
    }
  }
}

struct alignas(64) Params {
  CUtensorMap pool_map;     // the pool in four dimensions: one box is a tile's keys and values (see where it is made)
  const bf16* q;            // plain form: [tokens, nq * D]
  bf16* out;
  bf16* kv_pages;
  const int* block_table;
  const int* cu_q;
  const int* kv_len;
  float* part_o;            // [grid][2][16][D]
  float* part_ml;           // [grid][2][16][2]
  int* counters;            // [n_seqs * head_blocks], zero; left zero
  int q_stride, out_stride, bt_stride, n_seqs, nq, nkv, page_size, n_pages, window;
  float scale_log2;
  FusedQK fq;
};

struct Piece {
  int seq, hb, t_begin, n_tiles, nt;
  int advance;              // how far the piece reaches along the blocks' common axis (tiles and piece costs)
  long long first;          // where this piece's (request, head block) starts on that axis; its tiles follow PIECE_COST later
};

// STAGES: ring stages (a multiple of NCW); MROWS: rows of the merge buffer (16, or 8 for groups of up to 8 heads).
template <int STAGES, int MROWS>
__global__ void __launch_bounds__(THREADS, 1) attn_decode_kernel(const __grid_constant__ Params p) {
  static_assert(STAGES % NCW == 0, "every stage must belong to one consumer warp");
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = smem_unaligned + ((1024 - (smem_u32(smem_unaligned) & 1023)) & 1023);
  unsigned char* ring = smem;                                                   // [STAGES][K tile | V tile]
  float* mo = reinterpret_cast<float*>(smem + (size_t)STAGES * STAGE_BYTES);    // [NCW][MROWS][D]
  float* mml = mo + NCW * MROWS * D;                                            // [NCW][MROWS][2]
  bf16* qbuf = reinterpret_cast<bf16*>(mml + NCW * MROWS * 2);                  // [16][D], chunks exchanged as in a tile
  __shared__ __align__(16) bf16 s_new[2][D];                  // the new token's key and value (fused form)
  // fused form: the rows of qkv that the piece after the one at work needs, as they lie in qkv (the head block's
  // query heads, then the new key and the new value), and the cosines and sines of its position
  __shared__ __align__(16) bf16 s_raw[MROWS + 2][D];
  __shared__ __align__(16) float s_raw_cs[D];
  __shared__ unsigned short s_cnt[MAX_SEQS];                 // tiles of each request (0: not a single-token request, or idle)
  __shared__ unsigned char s_idle[MAX_SEQS];                 // 1: an idle entry (a single token whose newest key has no page)
  __shared__ int s_prefix[MAX_SEQS + 1];
  __shared__ int s_total[MAX_SEQS];                          // keys of each request, its new one included
  __shared__ int s_tok[MAX_SEQS];                            // row of each request's token in q / qkv / out
  __shared__ int s_pos[MAX_SEQS];                            // fused form with rotation: the token's position, clamped
  __shared__ uint64_t full[STAGES], empty[STAGES];
  __shared__ int s_tile_ok[STAGES];                          // 0: the tile's page is not there, nothing of it counts
  __shared__ int s_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const FusedQK& fq = p.fq;
  const bool fused = fq.qkv != nullptr;
  // The form that works from the projection's output and stores the new keys itself reads only keys that earlier
  // steps wrote: it plans and fetches while the projection winds down and waits only before it reads qkv.  The
  // other forms read keys that the kernel before them stored, so they wait first.
  const bool early = fused && fq.store;
  pdl_launch_dependents();
  if (!early) pdl_wait();

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  const int n_seqs = p.n_seqs, nkv = p.nkv, page_size = p.page_size, window = p.window;
  const int G = p.nq / nkv;
  const int rows_per = min(G, 16);
  const int chunks = (G + 15) / 16;                          // groups of more than 16 heads: several head blocks
  const int H = nkv * chunks;                                // head blocks per request
  for (int sq = threadIdx.x; sq < n_seqs; sq += THREADS) {
    // three loads at once, then the two that need their answers (also at once); all of them are the step's input,
    // which no kernel before this one writes
    const int tok = __ldg(p.cu_q + sq), tok_end = __ldg(p.cu_q + sq + 1), total = __ldg(p.kv_len + sq);
    const bool single = tok_end - tok == 1;
    const int newest = single && total > 0 ? __ldg(p.block_table + (size_t)sq * p.bt_stride + (total - 1) / page_size) : -1;
    if (fused && fq.cos_sin) {                               // so that no piece waits for its position before it can ask for its cosines
      const int pos = single ? __ldg(fq.positions + tok) : 0;
      s_pos[sq] = pos < 0 ? 0 : (pos >= fq.max_position ? fq.max_position - 1 : pos);
    }
    int nt = 0, idle = 0;
    if (single) {
      const int lo = window > 0 ? max(0, total - window) : 0;
      nt = total > 0 ? (total - 1) / BN - lo / BN + 1 : 0;
      // An entry that only fills the batch up to a fixed shape has no page for its token: it costs nothing here
      // (no tiles, no piece) and its output rows are cleared.
      if (newest < 0 || newest >= p.n_pages) {
        nt = 0;
        idle = 1;
      }
    }
    s_cnt[sq] = (unsigned short)min(nt, 65535);
    s_idle[sq] = (unsigned char)idle;
    s_total[sq] = total;
    s_tok[sq] = tok;
  }
  __syncthreads();
  // a request's share of the common axis: per head block its tiles and the cost of a piece
  auto weight = [&](int sq) { return s_cnt[sq] ? (int)s_cnt[sq] + PIECE_COST : 0; };
  if (warp == 0) {                                           // prefix sums: each lane a run of requests, then a warp scan
    const int per = (n_seqs + 31) / 32;
    const int b0 = min(lane * per, n_seqs), b1 = min(b0 + per, n_seqs);
    int sum = 0;
    for (int i = b0; i < b1; ++i) sum += weight(i);
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - sum;
    for (int i = b0; i < b1; ++i) { s_prefix[i] = run; run += weight(i); }
    if (lane == 31) s_prefix[n_seqs] = incl;
  }
  __syncthreads();
  const long long T = (long long)H * s_prefix[n_seqs];
  // at least MIN_TILES tiles per block (a short batch uses fewer blocks), so that every block has work, the
  // owners of consecutive tiles are consecutive blocks and a request is cut into few pieces
  const int NB = (int)max(1LL, min((long long)gridDim.x, T / MIN_TILES));
  const int c = blockIdx.x;
  // idle entries' output rows, dealt to the blocks; after the wait for the predecessor, which may still read them
  auto clear_idle_rows = [&](int tid, int n_threads) {
    for (int sq = c; sq < n_seqs; sq += gridDim.x) {
      if (!s_idle[sq]) continue;
      bf16* dst = p.out + (size_t)s_tok[sq] * p.out_stride;
      for (int id = tid; id < p.nq * CH; id += n_threads) reinterpret_cast<uint4*>(dst)[id] = make_uint4(0, 0, 0, 0);
    }
  };
  if (c >= NB || T == 0) {
    if (early) pdl_wait();
    clear_idle_rows(threadIdx.x, THREADS);
    return;
  }
  const long long u0 = (long long)c * T / NB, u1 = (long long)(c + 1) * T / NB;

  // A walk along the block's range, one (request, head block) after the other: `first` is where the span of the
  // current one starts (its cost, then its tiles).  Found once by search, then stepped: a piece costs no search
  // and no 64-bit division.
  struct Cursor {
    int seq, hb;
    long long first;
  };
  auto cursor_at = [&](long long u) {
    int lo_s = 0, hi_s = n_seqs;
    while (lo_s < hi_s) {
      const int mid = (lo_s + hi_s) >> 1;
      if ((long long)H * s_prefix[mid + 1] > u) hi_s = mid; else lo_s = mid + 1;
    }
    Cursor cu;
    cu.seq = lo_s;
    const int w = (int)s_cnt[cu.seq] + PIECE_COST;
    const long long seq_base = (long long)H * s_prefix[cu.seq];
    cu.hb = (int)(u - seq_base) / w;                         // at most H * w places: 32 bits do
    cu.first = seq_base + (long long)cu.hb * w;
    return cu;
  };
  // the piece of the cursor's (request, head block) that starts at place u and ends with it or with the block's
  // range; moves u behind the piece and the cursor on if the (request, head block) ends there
  auto next_piece = [&](Cursor& cu, long long& u) {
    Piece pc;
    pc.seq = cu.seq;
    pc.hb = cu.hb;
    pc.first = cu.first;
    pc.nt = s_cnt[cu.seq];
    const int w = pc.nt + PIECE_COST;                        // the span of one (request, head block): the cost, then its tiles
    const int x0 = (int)(u - cu.first), x1 = (int)(min(u1, cu.first + w) - cu.first);
    pc.advance = x1 - x0;
    pc.t_begin = max(0, x0 - PIECE_COST);
    pc.n_tiles = max(0, x1 - PIECE_COST) - pc.t_begin;      // 0: the block's range ends before this one's first tile
    u += pc.advance;
    if (x1 == w) {                                           // on to the next (request, head block) that has tiles
      cu.first += w;
      if (++cu.hb == H) {
        cu.hb = 0;
        do ++cu.seq; while (cu.seq < n_seqs && s_cnt[cu.seq] == 0);
      }
    }
    return pc;
  };

  if (warp == NCW) {
    // ---------------------------------------------------------------- producer
    uint32_t gi = 0;                                         // tiles sent so far: stage gi % STAGES
    int ok = 1;
    Cursor cur = cursor_at(u0);
    for (long long u = u0; u < u1 && ok;) {
      const Piece pc = next_piece(cur, u);
      if (pc.n_tiles == 0) continue;
      const int kvh = pc.hb / chunks;
      const int total = s_total[pc.seq];
      const int lo = window > 0 ? max(0, total - window) : 0;
      const int key_begin = (lo / BN + pc.t_begin) * BN;
      const int* table = p.block_table + (size_t)pc.seq * p.bt_stride;
      for (int it0 = 0; it0 < pc.n_tiles && ok; it0 += 32) {
        int row = 0, there = 0;
        if (it0 + lane < pc.n_tiles) {                       // the pages of 32 tiles at a time
          const int key0 = key_begin + (it0 + lane) * BN;
          int pg = __ldg(table + key0 / page_size);
          there = pg >= 0 && pg < p.n_pages;
          if (!there) pg = 0;
          row = ((pg * 2) * nkv + kvh) * page_size + key0 % page_size;
        }
        const int n_here = min(32, pc.n_tiles - it0);
        for (int j = 0; j < n_here; ++j) {
          const int rk = __shfl_sync(0xffffffffu, row, j), th = __shfl_sync(0xffffffffu, there, j);
          const int stage = gi % STAGES;
          if (lane == 0) {
            if (gi >= (uint32_t)STAGES) ok = mbar_wait(&empty[stage], ((gi / STAGES) - 1) & 1, 1) ? 1 : 0;
            if (ok) {
              s_tile_ok[stage] = th;
              mbar_expect_tx(&full[stage], STAGE_BYTES);
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
          // the whole tile in one copy: the box holds 64 columns x the tile's keys x the head's column blocks x
          // (keys, values), and arrives in that order (a copy costs the TMA unit about as much whatever it holds)
          if (lane == 0) tma_load_4d(ring + (size_t)stage * STAGE_BYTES, &p.pool_map, 0, rk, 0, 0, &full[stage]);
          ++gi;
        }
      }
    }
    if (!ok) give_up_delay();
    return;
  }

  // ------------------------------------------------------------------ consumers
  bool waited = !early, ok = true;
  uint32_t gi_base = 0;
  // Fused form: while a piece is at its tiles, the rows of qkv of the piece after it (and its cosines and sines) are
  // copied to shared memory as they are, asynchronously, so that only a block's first piece waits for them.
  bool raw_ready = false;                                    // s_raw and s_raw_cs hold the coming piece's rows
  auto fetch_ahead = [&](const Piece& q) {
    const int kvh = q.hb / chunks, g0 = (q.hb - kvh * chunks) * 16;
    const int gn = min(rows_per, G - g0);
    const bf16* row = fq.qkv + (size_t)s_tok[q.seq] * fq.qkv_stride;
    const bool newest = fq.store && q.t_begin + q.n_tiles == q.nt;
    for (int id = threadIdx.x; id < (gn + (newest ? 2 : 0)) * CH; id += NCW * 32) {
      const int R = id / CH, cc = id - R * CH;
      const int head = R < gn ? kvh * G + g0 + R : p.nq + (R == gn ? 0 : nkv) + kvh;
      copy16_async(&s_raw[R < gn ? R : MROWS + (R - gn)][cc * 8], row + (size_t)head * D + cc * 8);
    }
    if (fq.cos_sin) {
      const float* cs = fq.cos_sin + (size_t)s_pos[q.seq] * fq.rotary_dim;
      for (int id = threadIdx.x; id < fq.rotary_dim / 4; id += NCW * 32) copy16_async(&s_raw_cs[id * 4], cs + id * 4);
    }
  };
  Cursor cur = cursor_at(u0);
  for (long long u = u0; u < u1;) {
    const Piece pc = next_piece(cur, u);
    if (pc.n_tiles == 0) continue;
    const int seq = pc.seq, hb = pc.hb, n_tiles = pc.n_tiles, nt = pc.nt;
    const bool whole = pc.t_begin == 0 && n_tiles == nt;
    const int kvh = hb / chunks, g0 = (hb - kvh * chunks) * 16;
    const int gn = min(rows_per, G - g0);
    const int total = s_total[seq];
    const int lo = window > 0 ? max(0, total - window) : 0;
    const int key_begin = (lo / BN + pc.t_begin) * BN;
    const size_t tok = s_tok[seq];
    const bool has_last = pc.t_begin + n_tiles == nt;         // this piece ends with the request's newest key
    if (!waited) {
      pdl_wait();
      waited = true;
    }
    int new_slot = -1;
    if (!fused) {
      for (int id = threadIdx.x; id < 16 * CH; id += NCW * 32) {
        const int R = id / CH, cc = id - R * CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (R < gn) v = *reinterpret_cast<const uint4*>(p.q + tok * p.q_stride + (size_t)(kvh * G + g0 + R) * D + cc * 8);
        *reinterpret_cast<uint4*>(qbuf + tile_off<16>(R, cc)) = v;
      }
    } else {
      // the token's row of qkv, or (any piece but the block's first) what was copied of it while the piece before was at work
      const bf16* row = fq.qkv + tok * fq.qkv_stride;
      const float* cs = nullptr;
      if (fq.cos_sin) cs = raw_ready ? s_raw_cs : fq.cos_sin + (size_t)s_pos[seq] * fq.rotary_dim;
      if (has_last && fq.store && g0 == 0) new_slot = fq.slot_mapping[tok];   // used behind the barrier below
      // warp 0: the new key, warp 1: the new value; asked for before the query heads, used behind them
      const bool has_new = has_last && fq.store && warp < 2;
      float nv[FVEC];
      if (has_new) head_load(nv, raw_ready ? s_raw[MROWS + warp] : row + (size_t)(p.nq + (warp == 0 ? 0 : nkv) + kvh) * D, lane);
      for (int R = warp; R < 16; R += NCW) {                  // the query heads of the group dealt to the warps
        float v[FVEC];
        if (R < gn) {
          fused_head(v, raw_ready ? s_raw[R] : row + (size_t)(kvh * G + g0 + R) * D, fq.q_w, cs, fq, lane);
        } else {
#pragma unroll
          for (int k = 0; k < FVEC; ++k) v[k] = 0.f;
        }
        const int e0 = lane * FVEC;
#pragma unroll
        for (int k = 0; k < FVEC; ++k)      // a lane's elements may straddle two 16-byte chunks (head size 192)
          qbuf[tile_off<16>(R, (e0 + k) >> 3) + ((e0 + k) & 7)] = __float2bfloat16_rn(v[k]);
      }
      if (has_new) {
        head_finish(nv, warp == 0 ? fq.k_w : nullptr, warp == 0 ? cs : nullptr, fq, lane);
#pragma unroll
        for (int k = 0; k < FVEC; ++k) s_new[warp][lane * FVEC + k] = __float2bfloat16_rn(nv[k]);
      }
    }
    consumer_sync();
    raw_ready = false;
    if (fused && u < u1) {                                    // s_raw is free: the barrier above is behind its last reader
      Cursor c2 = cur;
      long long u2 = u;
      const Piece nx = next_piece(c2, u2);
      if (nx.n_tiles > 0) {
        fetch_ahead(nx);
        raw_ready = true;
      }
    }
    if (fused && has_last && fq.store && g0 == 0) {
      // one block per (request, KV head) stores the new key and value for the steps to come
      const int slot = new_slot;
      if (slot >= 0 && slot < p.n_pages * page_size) {
        const int pg = slot / page_size, off = slot - pg * page_size;
        for (int id = threadIdx.x; id < 2 * CH; id += NCW * 32) {
          const int kv = id / CH, cc = id - kv * CH;
          bf16* dst = p.kv_pages + ((((size_t)pg * 2 + kv) * nkv + kvh) * page_size + off) * D + cc * 8;
          *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&s_new[kv][cc * 8]);
        }
      }
    }
    uint32_t qf[KS][4];
#pragma unroll
    for (int k = 0; k < KS; ++k)
      ldmatrix_x4(qf[k], qbuf + tile_off<16>((lane & 7) + (((lane >> 3) & 1) << 3), 2 * k + (lane >> 4)));
    int row_hi[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) row_hi[i] = (lane >> 2) + 8 * i < gn ? total - 1 : -1;
    RowState st;
    st.m[0] = st.m[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.f;
#pragma unroll
    for (int n = 0; n < DN; ++n) st.o[n][0] = st.o[n][1] = st.o[n][2] = st.o[n][3] = 0.f;

    // whole tiles in turn, by their number in the block's run of tiles: no warp waits for another
    for (int it = (warp + NCW - (int)(gi_base % NCW)) % NCW; it < n_tiles && ok; it += NCW) {
      const uint32_t gi = gi_base + it;
      const int stage = gi % STAGES;
      ok = mbar_wait(&full[stage], (gi / STAGES) & 1, 2);
      if (!ok) break;
      bf16* kt = reinterpret_cast<bf16*>(ring + (size_t)stage * STAGE_BYTES);
      bf16* vt = reinterpret_cast<bf16*>(ring + (size_t)stage * STAGE_BYTES + TILE_BYTES);
      const int key_base = key_begin + it * BN;
      const bool there = s_tile_ok[stage] != 0;
      bool wrote = false;
      if (fused && fq.store && has_last && it == n_tiles - 1) {
        // the cache does not hold the newest key and value yet (or is being written): take them from s_new
        const int r = total - 1 - key_base;
        for (int id = lane; id < 2 * CH; id += 32) {
          const int kv = id / CH, cc = id - kv * CH;
          *reinterpret_cast<uint4*>((kv == 0 ? kt : vt) + tile_off<BN>(r, cc)) = *reinterpret_cast<const uint4*>(&s_new[kv][cc * 8]);
        }
        wrote = true;
      }
      // value rows of keys outside [lo, total) are cleared: their weight is zero, but zero times what lies there
      // (stale numbers, NaN of a fresh pool) must be zero too
      const int r_lo = there ? min(BN, max(0, lo - key_base)) : BN;            // rows [0, r_lo) are before the range
      const int r_hi = there ? min(BN, max(0, total - key_base)) : BN;         // rows [r_hi, BN) are beyond it
      if (r_lo > 0 || r_hi < BN) {
        for (int id = lane; id < BN * CH; id += 32) {
          const int r = id / CH, cc = id - r * CH;
          if (r < r_lo || r >= r_hi) *reinterpret_cast<uint4*>(vt + tile_off<BN>(r, cc)) = make_uint4(0, 0, 0, 0);
        }
        wrote = true;
      }
      if (wrote) __syncwarp();
      const int lo_t = there ? lo : 0x7fffffff;               // a tile whose page is missing: no key counts
      if (key_base < total && key_base + BN > lo_t)
        warp_half_tile(st, qf, kt, vt, 0, key_base, lo_t, row_hi, p.scale_log2);
      if (wrote) fence_async_smem();                          // this warp's stores before the next copy into the stage
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);
    }
    gi_base += n_tiles;

    // ---- the end of a piece: merge the warps' states (each saw some of the tiles) through shared memory
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float l = st.l[i];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      const int R = (lane >> 2) + 8 * i;
      if (R >= gn) continue;                                   // rows beyond the group hold nothing
      float* dst = mo + ((size_t)warp * MROWS + R) * D + ((lane & 3) << 1);
#pragma unroll
      for (int n = 0; n < DN; ++n)
        *reinterpret_cast<float2*>(dst + n * 8) = make_float2(st.o[n][2 * i], st.o[n][2 * i + 1]);
      if ((lane & 3) == 0) {
        mml[(warp * MROWS + R) * 2] = st.m[i];
        mml[(warp * MROWS + R) * 2 + 1] = l;
      }
    }
    consumer_sync();
    const size_t unit = (size_t)seq * H + hb;                  // this (request, head block)
    // a block has at most two pieces that are not whole: one that goes on where the block before it stopped (only
    // at the start of its range) and one that its range's end cuts short (only at that end)
    const int slot = pc.t_begin > 0 ? 0 : 1;
    float* po = p.part_o + ((size_t)c * 2 + slot) * 16 * D;
    float* pml = p.part_ml + ((size_t)c * 2 + slot) * 16 * 2;
    for (int id = threadIdx.x; id < gn * (D / 4); id += NCW * 32) {
      const int R = id / (D / 4), c4 = id - R * (D / 4);
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < NCW; ++w) M = fmaxf(M, mml[(w * MROWS + R) * 2]);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      float L = 0.f;
#pragma unroll
      for (int w = 0; w < NCW; ++w) {
        const float mw = mml[(w * MROWS + R) * 2];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
        const float4 t = *reinterpret_cast<const float4*>(mo + ((size_t)w * MROWS + R) * D + c4 * 4);
        acc.x += t.x * f; acc.y += t.y * f; acc.z += t.z * f; acc.w += t.w * f;
        L += mml[(w * MROWS + R) * 2 + 1] * f;
      }
      if (whole) {
        const float inv = L > 0.f ? 1.0f / L : 0.f;
        bf16* dst = p.out + tok * p.out_stride + (size_t)(kvh * G + g0 + R) * D + c4 * 4;
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
      } else {
        *reinterpret_cast<float4*>(po + R * D + c4 * 4) = acc;
        if (c4 == 0) { pml[R * 2] = M; pml[R * 2 + 1] = L; }
      }
    }
    if (!whole) {
      // the arrival is a release (the barrier before it orders the other threads' stores before it) and an
      // acquire (the last piece to arrive may read the others), so no thread stands at a fence
      consumer_sync();
      if (threadIdx.x == 0) {
        int old;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;\n" : "=r"(old) : "l"(p.counters + unit) : "memory");
        s_flag = old;
      }
      consumer_sync();
      const int first_owner = tile_owner(pc.first + PIECE_COST, T, NB);
      const int pieces = tile_owner(pc.first + PIECE_COST + nt - 1, T, NB) - first_owner + 1;
      if (s_flag == pieces - 1) {                              // the last piece to arrive: merge all, in block order
        // the first owner's piece starts with the first tile (slot 1); every other owner's goes on from the block
        // before it (slot 0)
        constexpr int first_slot = 1;
        for (int id = threadIdx.x; id < gn * (D / 4); id += NCW * 32) {
          const int R = id / (D / 4), c4 = id - R * (D / 4);
          // One pass, eight pieces' loads on their way at a time (the pieces lie in L2: what this costs is trips,
          // not bytes): the running maximum moves with every eight, and what is summed so far is rescaled to it.
          float M = -INFINITY, L = 0.f;
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int k0 = 0; k0 < pieces; k0 += 8) {
            float4 t[8];
            float2 ml[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int k = min(k0 + j, pieces - 1);
              const size_t at = ((size_t)(first_owner + k) * 2 + (k == 0 ? first_slot : 0)) * 16;
              t[j] = __ldcg(reinterpret_cast<const float4*>(p.part_o + (at + R) * D) + c4);
              ml[j] = __ldcg(reinterpret_cast<const float2*>(p.part_ml + (at + R) * 2));     // (max, sum)
            }
            float Mb = M;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (k0 + j < pieces) Mb = fmaxf(Mb, ml[j].x);
            if (Mb == -INFINITY) continue;                     // nothing but pieces without a key so far
            const float f0 = M == -INFINITY ? 0.f : exp2f(M - Mb);
            acc.x *= f0; acc.y *= f0; acc.z *= f0; acc.w *= f0;
            L *= f0;
            M = Mb;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (k0 + j >= pieces || ml[j].x == -INFINITY) continue;
              const float f = exp2f(ml[j].x - M);
              acc.x += t[j].x * f; acc.y += t[j].y * f; acc.z += t[j].z * f; acc.w += t[j].w * f;
              L += ml[j].y * f;
            }
          }
          const float inv = L > 0.f ? 1.0f / L : 0.f;
          bf16* dst = p.out + tok * p.out_stride + (size_t)(kvh * G + g0 + R) * D + c4 * 4;
          *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
        }
        if (threadIdx.x == 0) p.counters[unit] = 0;            // ready for the next launch
      }
    }
    copies_async_wait();                                       // what this thread copied for the next piece has landed
    consumer_sync();                                           // the merge buffers and the query are reused by the next piece
  }
  if (!waited) pdl_wait();
  clear_idle_rows(threadIdx.x, NCW * 32);
  if (!ok) give_up_delay();
}

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

NHV_API const char* NHV_FN(nhv_attn_decode_last_error_d)() { return g_err; }
// Reads and clears the error word of the kernel's bounded waits (0: none ran out).  Synchronises the device.
NHV_API int NHV_FN(nhv_attn_decode_error_d)() { return nhv_wait_error_take(); }
// The device address of the error word, for kernels that report it with the step's result.
NHV_API void* NHV_FN(nhv_attn_decode_error_word_d)() { return nhv_wait_error_address(); }
// The most requests one launch plans for.
NHV_API int NHV_FN(nhv_attn_decode_max_seqs_d)() { return MAX_SEQS; }

// The grid (one block per SM) and the scratch a launch needs: part_o [blocks * 2 * 16 * D] floats, part_ml
// [blocks * 2 * 16 * 2] floats, and counters [n_seqs * kv_heads * ceil(group / 16)] ints that are zero (the kernel
// leaves them zero).
NHV_API int NHV_FN(nhv_attn_decode_blocks_d)() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      sms = 0;
  }
  return sms;
}

// Attention of the step's single-token requests (requests that bring more tokens are left alone).
// qkv null: the queries are q [tokens, nq * D], normed and rotated, and the cache holds the new keys and values.
// qkv given: the projection's output [tokens, (nq + 2 nkv) * D]; the kernel norms (q_w / k_w, or null) and rotates
// (cos_sin, or null) the new query and key heads itself and, with store != 0, puts the new keys and values into the
// cache; every request of the step must then bring exactly one token.
NHV_API int NHV_FN(nhv_attn_decode_d)(const void* q, int q_stride, const void* qkv, int qkv_stride, void* out, int out_stride,
                                      void* kv_pages, const int* block_table, int bt_stride, const int* cu_q,
                                      const int* kv_len, int n_seqs, int nq, int nkv, int page_size, int n_pages,
                                      int window, float scale, float* part_o, float* part_ml, int* counters,
                                      const void* q_w, const void* k_w, const float* cos_sin, const int* positions,
                                      const int* slot_mapping, int rotary_dim, int max_position, int store, float eps,
                                      float weight_offset, cudaStream_t stream) {
  ATT_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads do not divide into %d KV heads", nq, nkv);
  ATT_REQUIRE(page_size > 0 && page_size % BN == 0 && n_pages > 0 && bt_stride > 0,
              "attention (decode, TMA): pages must be a multiple of %d keys, got %d", BN, page_size);
  ATT_REQUIRE(n_seqs > 0 && n_seqs <= MAX_SEQS, "attention: %d requests in a step, the decode kernel plans for up to %d", n_seqs, MAX_SEQS);
  ATT_REQUIRE(part_o && part_ml && counters, "attention: decoding needs scratch memory for the pieces of split requests");
  ATT_REQUIRE(out_stride % 8 == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)kv_pages % 16) == 0,
              "attention: the pages, the output and the output's rows must be 16-byte aligned");
  ATT_REQUIRE((long long)n_pages * 2 * nkv * page_size < (1LL << 31), "attention: the pool has more rows than a tensor map's 32-bit coordinate");
  Params p;
  p.fq = FusedQK{};
  if (qkv) {
    ATT_REQUIRE(qkv_stride % 8 == 0 && ((uintptr_t)qkv % 16) == 0, "attention: qkv must be 16-byte aligned");
    ATT_REQUIRE(!cos_sin || (((uintptr_t)cos_sin % 16) == 0 && rotary_dim % 4 == 0),
                "attention: the table of cosines and sines must be 16-byte aligned, its rows too");
    ATT_REQUIRE(!cos_sin || (positions && rotary_dim > 0 && rotary_dim <= D && rotary_dim % (2 * FVEC) == 0),
                "attention: the fused decode form rotates in steps of %d elements, rotary_dim is %d", 2 * FVEC, rotary_dim);
    ATT_REQUIRE(!store || slot_mapping, "attention: storing the new keys needs the slot mapping");
    p.fq.qkv = (const bf16*)qkv;
    p.fq.q_w = (const bf16*)q_w;
    p.fq.k_w = (const bf16*)k_w;
    p.fq.cos_sin = cos_sin;
    p.fq.positions = positions;
    p.fq.slot_mapping = slot_mapping;
    p.fq.qkv_stride = qkv_stride;
    p.fq.rotary_dim = rotary_dim;
    p.fq.max_position = max_position;
    p.fq.store = store;
    p.fq.eps = eps;
    p.fq.weight_offset = weight_offset;
  } else {
    ATT_REQUIRE(q && q_stride % 8 == 0 && ((uintptr_t)q % 16) == 0, "attention: q must be 16-byte aligned");
  }
  static std::mutex mutex;
  static std::unordered_map<const void*, std::pair<long long, CUtensorMap>> maps;   // one per cache pool: pools do not move
  const long long rows = (long long)n_pages * 2 * nkv * page_size;
  {
    std::lock_guard<std::mutex> lock(mutex);
    auto it = maps.find(kv_pages);
    if (it == maps.end() || it->second.first != rows) {
      CUtensorMap m;
      // the pool as [keys or values of a page][column block of 64][row of the pool][64 columns]: the values of a
      // (page, KV head) lie nkv * page_size rows behind its keys
      const long long half = (long long)nkv * page_size;
      const long long dims[4] = {64, rows - half, DB, 2};
      const long long strides[4] = {2, (long long)D * 2, 128, half * D * 2};
      const int box[4] = {64, BN, DB, 2};
      ATT_REQUIRE(nhv_make_map_bf16_nd(&m, kv_pages, 4, dims, strides, box), "attention (decode, TMA): cannot encode the tensor map of the pool");
      maps[kv_pages] = {rows, m};
      it = maps.find(kv_pages);
    }
    p.pool_map = it->second.second;
  }
  const bool deep = nq / nkv <= 8;                           // groups of up to 8 heads: the smaller merge buffer, the deeper ring
  const size_t smem = deep ? smem_bytes(STAGES_DEEP, 8) : smem_bytes(STAGES_MIN, 16);
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_decode_kernel<STAGES_DEEP, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem_bytes(STAGES_DEEP, 8)) != cudaSuccess ||
        cudaFuncSetAttribute(attn_decode_kernel<STAGES_MIN, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem_bytes(STAGES_MIN, 16)) != cudaSuccess) {
      snprintf(g_err, sizeof(g_err), "attention (decode, TMA): cannot reserve %zu bytes of shared memory", smem);
      return 2;
    }
    attr_set = true;
  }
  const int blocks = NHV_FN(nhv_attn_decode_blocks_d)();
  ATT_REQUIRE(blocks > 0, "attention: cannot read the number of SMs");
  p.q = (const bf16*)q;
  p.out = (bf16*)out;
  p.kv_pages = (bf16*)kv_pages;
  p.block_table = block_table;
  p.cu_q = cu_q;
  p.kv_len = kv_len;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.counters = counters;
  p.q_stride = q_stride; p.out_stride = out_stride; p.bt_stride = bt_stride; p.n_seqs = n_seqs; p.nq = nq; p.nkv = nkv;
  p.page_size = page_size; p.n_pages = n_pages; p.window = window;
  p.scale_log2 = scale * LOG2E;
  const cudaError_t launched = deep ? nhv_launch(attn_decode_kernel<STAGES_DEEP, 8>, dim3(blocks), dim3(THREADS), smem, stream, p)
                                    : nhv_launch(attn_decode_kernel<STAGES_MIN, 16>, dim3(blocks), dim3(THREADS), smem, stream, p);
  if (launched != cudaSuccess || cudaPeekAtLastError() != cudaSuccess) {
    snprintf(g_err, sizeof(g_err), "attention (decode, TMA): launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return 2;
  }
  return 0;
}
