// Attention of prompt portions over the paged cache on the 5th-generation tensor cores (tcgen05.mma, accumulators
// in tensor memory, K and V brought by TMA), compiled per head size: -DNHV_ATTN_D=64|128|192|256.
//
// softmax(q k^T * scale) v per query head, causal, optionally within a window, q of a portion's tokens against
// all keys of the request that the cache holds (nanovllm/layers/attention.py:67-70 calls a library for this;
// nanovllm/models/qwen3.py:39 gives the scale).  Scores, softmax, the row sum and the output sum are fp32; the
// probabilities are rounded to bfloat16 for the second product only.
//
// A block owns 128 rows: the 128 / G tokens x G query heads that share one KV head (row = token * G + head), so
// a key tile read once serves the whole group.  It walks the keys in tiles of 64, which never straddle a page
// (the page size must be a multiple of 64; other sizes go to the mma.sync kernel).
//
// Warp roles.  Warp 0, one lane: TMA producer; per tile one box of 64 keys x 64 columns per 64 columns of the
// head, for K and for V, from the pool seen as a matrix [pages * 2 * kv_heads * page_size, D], into two stages
// each.  Warp 1: allocates tensor memory; one lane issues the MMAs: S = Q K^T (M 128, N 64, K = D; Q and K both
// K-major in the 128-byte swizzle) into one of two S buffers, and O += P V (M 128, N = D, K = 64; P read from
// tensor memory, V as it lies in the cache: MN-major).  Warps 2-5: one thread per row; it reads its row of S from
// tensor memory, scales, masks, keeps the running maximum and sum, writes the row of P (bfloat16 pairs) over the
// first half of the S it has just read, and at the end reads its row of O, divides and stores it.  S of tile j+1
// is computed while the rows of tile j are in the softmax.
//
// O stays in tensor memory across tiles.  It is rescaled only when a row's maximum has grown by more than 2^8
// since the reference it uses (the probabilities are then at most 2^8, which bfloat16 and the fp32 sum hold as
// well as values below 1); rows are independent, so a row's result does not depend on what shares its block.
//
// Every wait on an mbarrier is bounded: one that runs out sets an error word (nhv_attn_tcgen05_error_d<D>), the
// roles leave their loops, the producer waits (bounded) for the copies it has in flight, and the block frees
// its tensor memory and returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>
#include <unordered_map>

#define NHV_WAIT_LIMIT (1u << 22)
#include "nhv_async.cuh"

#ifndef NHV_ATTN_D
#error "compile with -DNHV_ATTN_D=<head size>"
#endif
#define NHV_CAT2(a, b) a##b
#define NHV_CAT(a, b) NHV_CAT2(a, b)
#define NHV_FN(name) NHV_CAT(name, NHV_ATTN_D)

namespace {

typedef __nv_bfloat16 bf16;
constexpr int D = NHV_ATTN_D;
static_assert(D % 64 == 0 && D >= 64 && D <= 256, "head sizes 64, 128, 192 and 256");
constexpr int BM = 128;                      // rows of a block = lanes of tensor memory
constexpr int BN = 64;                       // keys per tile
constexpr int DB = D / 64;                   // 128-byte column blocks of a head
constexpr int THREADS = 192;
constexpr int Q_BYTES = DB * BM * 128;
constexpr int T_BYTES = DB * BN * 128;       // one K tile or one V tile
constexpr int STAGES = 2;
constexpr int BAR_BYTES = 128;
constexpr int SMEM_NEED = 1024 + Q_BYTES + 2 * STAGES * T_BYTES;    // barriers live in the first 128 bytes
// at least 80 KB, so that an SM never holds more blocks than its tensor memory serves (two of 256 columns)
constexpr int SMEM_BYTES = SMEM_NEED < 80 * 1024 ? 80 * 1024 : SMEM_NEED;
constexpr uint32_t TMEM_COLS = (2 * BN + D) <= 256 ? 256 : 512;
constexpr uint32_t S_COL = 0, O_COL = 2 * BN;
constexpr float RESCALE_STEP = 8.0f;         // log2 units
constexpr float LOG2E = 1.4426950408889634f;

char g_err[256] = "";

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// ---- tensor memory and tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_in_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(slot_in_smem)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the A operand in tensor memory (one row per lane, two bfloat16 per 32-bit column).
__device__ __forceinline__ void tc_mma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 consecutive columns of this thread's lane (no wait: tmem_ld_wait() before the values are used)
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t (&r)[32], uint32_t taddr) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle.  K-major operand (Q, K, P): rows of 128 bytes, groups of 8
// rows 1024 bytes apart (stride offset), the leading offset unused.  MN-major operand (V as it lies in the cache:
// a row of 128 bytes holds 64 columns of one key): the stride offset is the step between groups of 8 keys (1024),
// the leading offset the step between blocks of 64 columns.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t leading_bytes, uint32_t stride_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((leading_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((stride_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;                            // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                            // 128-byte swizzle
  return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32, A K-major, M x N; B K-major or MN-major.
__device__ __forceinline__ uint32_t instr_desc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ float fast_exp2(float x) {     // 2^x; -inf gives 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct alignas(64) Params {
  CUtensorMap kv_map;     // the pool as [n_pages * 2 * nkv * page_size, D], box 64 columns x 64 rows
  const bf16* q;
  bf16* out;
  const int* block_table;
  const int* cu_q;
  const int* kv_len;
  int q_stride, out_stride, bt_stride, n_seqs, nq, nkv, page_size, n_pages, window, tokens_per_block;
  float scale_log2;
};

__global__ void __launch_bounds__(THREADS, (2 * BN + D) <= 256 ? 2 : 1) attn_tcgen05_kernel(const __grid_constant__ Params p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  // barriers in the first 128 bytes, the tiles from the next 1024-byte boundary on
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);
  uint64_t* k_full = bars;                 // [2]
  uint64_t* k_empty = bars + 2;            // [2]
  uint64_t* v_full = bars + 4;             // [2]
  uint64_t* v_empty = bars + 6;            // [2]
  uint64_t* s_full = bars + 8;             // [2]
  uint64_t* p_ready = bars + 10;           // [1]
  uint64_t* o_full = bars + 11;            // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  int* s_abort = reinterpret_cast<int*>(bars + 13);
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* tiles = smem_raw + (((raw + BAR_BYTES + 1023u) & ~1023u) - raw);
  unsigned char* q_s = tiles;
  unsigned char* k_s = q_s + Q_BYTES;                  // [STAGES][T_BYTES]
  unsigned char* v_s = k_s + STAGES * T_BYTES;         // [STAGES][T_BYTES]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
    }
    mbar_init(p_ready, 128);
    mbar_init(o_full, 1);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"((uint64_t)&p.kv_map) : "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  pdl_prologue();

  // which request and which 128 rows: blocks are numbered KV head fastest, then tile; within a request the last
  // tokens (the longest walks over the keys) get the lowest numbers, so the heavy blocks start first
  const int G = p.nq / p.nkv;
  const int kvh = blockIdx.x;
  int seq = -1, tile = blockIdx.y;
  for (int s = 0; s < p.n_seqs; ++s) {
    const int n = p.cu_q[s + 1] - p.cu_q[s];
    if (n == 1) continue;                                    // single tokens belong to the decode kernel
    const int nt = (n + p.tokens_per_block - 1) / p.tokens_per_block;
    if (tile < nt) { seq = s; tile = nt - 1 - tile; break; }
    tile -= nt;
  }
  const bool active = seq >= 0 && (raw & 127u) == 0;
  if (seq >= 0 && !active && threadIdx.x == 0) wait_error_set(9);
  int n_new = 0, total = 0, t0 = 0, tq_n = 0, pos0 = 0, q_row0 = 0;
  if (active) {
    q_row0 = p.cu_q[seq];
    n_new = p.cu_q[seq + 1] - q_row0;
    total = p.kv_len[seq];
    t0 = tile * p.tokens_per_block;
    tq_n = min(p.tokens_per_block, n_new - t0);
    pos0 = total - n_new + t0;
  }
  const int pos_hi = pos0 + tq_n - 1;
  const int first_key = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int key_begin = (first_key / BN) * BN;
  const int n_tiles = active ? (pos_hi - key_begin) / BN + 1 : 0;

  if (active) {
    // stage Q: row R = token * G + head, 16-byte chunk c of column block b at (c ^ (R & 7)) of the row
    for (int id = threadIdx.x; id < BM * (D / 8); id += THREADS) {
      const int R = id / (D / 8), c = id - R * (D / 8);
      const int tq = R / G, g = R - tq * G;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (tq < tq_n)
        v = *reinterpret_cast<const uint4*>(p.q + (size_t)(q_row0 + t0 + tq) * p.q_stride + (size_t)(kvh * G + g) * D + c * 8);
      const int b = c >> 3, cc = c & 7;
      *reinterpret_cast<uint4*>(q_s + b * (BM * 128) + R * 128 + ((cc ^ (R & 7)) << 4)) = v;
    }
    fence_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_tiles > 0) {
      const int* bt = p.block_table + (size_t)seq * p.bt_stride;
      int issued = 0;
      int page = bt[key_begin / p.page_size];
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j & 1;
        const int key_base = key_begin + j * BN;
        int page_next = 0;
        if (j + 1 < n_tiles) page_next = bt[(key_base + BN) / p.page_size];      // looked up one tile ahead
        const int row_k = ((page * 2) * p.nkv + kvh) * p.page_size + key_base % p.page_size;
        const int row_v = row_k + p.nkv * p.page_size;
        if (j >= STAGES && !mbar_wait(&k_empty[st], (uint32_t)((j >> 1) - 1) & 1, 1)) { *s_abort = 1; break; }
        mbar_expect_tx(&k_full[st], T_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b) tma_load_2d(k_s + st * T_BYTES + b * (BN * 128), &p.kv_map, b * 64, row_k, &k_full[st]);
        if (j >= STAGES && !mbar_wait(&v_empty[st], (uint32_t)((j >> 1) - 1) & 1, 2)) { *s_abort = 1; issued = j; break; }
        mbar_expect_tx(&v_full[st], T_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b) tma_load_2d(v_s + st * T_BYTES + b * (BN * 128), &p.kv_map, b * 64, row_v, &v_full[st]);
        issued = j + 1;
        page = page_next;
      }
      if (*s_abort) {
        // leave only when the copies in flight have landed: the last two tiles' barriers cover them
        for (int j = max(0, issued - STAGES); j < issued; ++j) {
          mbar_wait(&k_full[j & 1], (uint32_t)(j >> 1) & 1, 3);
          mbar_wait(&v_full[j & 1], (uint32_t)(j >> 1) & 1, 3);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_tiles > 0) {
      const uint32_t idesc_s = instr_desc(BM, BN, false);
      const uint32_t idesc_o = instr_desc(BM, D, true);
      // descriptors are made once: a later K slice, column block or stage only moves the start address, which
      // sits in the low bits in units of 16 bytes
      const uint64_t q_desc = smem_desc(smem_u32(q_s), 16, 1024);
      const uint64_t k_desc = smem_desc(smem_u32(k_s), 16, 1024);
      const uint64_t v_desc = smem_desc(smem_u32(v_s), BN * 128, 1024);
      bool ok = true;
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(&k_full[st], (uint32_t)(j >> 1) & 1, 4)) return false;
        tc_fence_after();
        const uint64_t kd = k_desc + (uint64_t)(st * (T_BYTES >> 4));
        const uint32_t d_addr = tmem_base + S_COL + (uint32_t)((j & 1) * BN);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          tc_mma(d_addr, q_desc + (uint64_t)(((kk >> 2) * (BM * 128) + (kk & 3) * 32) >> 4),
                 kd + (uint64_t)(((kk >> 2) * (BN * 128) + (kk & 3) * 32) >> 4), idesc_s, kk > 0 ? 1u : 0u);
        tc_commit(&k_empty[st]);
        tc_commit(&s_full[j & 1]);
        return true;
      };
      ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        if (j + 1 < n_tiles) ok = issue_qk(j + 1);
        if (!ok) break;
        ok = mbar_wait(p_ready, (uint32_t)j & 1, 5) && mbar_wait(&v_full[st], (uint32_t)(j >> 1) & 1, 6);
        if (!ok) break;
        tc_fence_after();
        const uint64_t vd = v_desc + (uint64_t)(st * (T_BYTES >> 4));
        const uint32_t p_addr = tmem_base + S_COL + (uint32_t)((j & 1) * BN);    // P lies over the first half of this tile's S
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)                                       // 8 columns of P and 16 rows of V per 16 keys
          tc_mma_a_tmem(tmem_base + O_COL, p_addr + kk * 8, vd + (uint64_t)((kk * 16 * 128) >> 4), idesc_o,
                        (j > 0 || kk > 0) ? 1u : 0u);
        tc_commit(&v_empty[st]);
        tc_commit(o_full);
      }
      if (!ok) *s_abort = 1;
    }
    __syncwarp();
  } else if (n_tiles > 0) {
    // ------------------------------------------------------------------ softmax and output (warps 2..5)
    const int quarter = warp & 3;                               // the tensor-memory lanes this warp may touch
    const int R = quarter * 32 + lane;
    const int tq = R / G, g = R - tq * G;
    const bool valid = tq < tq_n;
    const int row_hi = valid ? pos0 + tq : -1;
    const int row_lo = p.window > 0 ? max(0, row_hi - p.window + 1) : 0;
    // the block's rows: keys up to pos0 are in sight of every valid row if they are above the highest lower edge
    const int all_hi = (tq_n * G >= BM) ? pos0 : -1;            // with padding rows every tile is masked
    const int all_lo = p.window > 0 ? max(0, pos_hi - p.window + 1) : 0;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    float m_run = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int key_base = key_begin + j * BN;
      ok = mbar_wait(&s_full[j & 1], (uint32_t)(j >> 1) & 1, 7);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[2][32];
      tmem_ld32_nowait(sr[0], lane_addr + S_COL + (uint32_t)((j & 1) * BN));
      tmem_ld32_nowait(sr[1], lane_addr + S_COL + (uint32_t)((j & 1) * BN) + 32);
      tmem_ld_wait();
      // x = score * scale in log2 units; the row maximum is taken over the raw scores (the scale is positive)
      // and the scaling folded into the exponent's multiply-add.  A tile that some row of the block sees only
      // in part takes the masked path.
      const bool masked = !(key_base >= all_lo && key_base + BN - 1 <= all_hi);
      if (masked) {
#pragma unroll
        for (int i = 0; i < BN; ++i) {
          const int key = key_base + i;
          if (!(key >= row_lo && key <= row_hi)) sr[i >> 5][i & 31] = 0xFF800000u;      // -inf
        }
      }
      float mx0 = max3(__uint_as_float(sr[0][0]), __uint_as_float(sr[0][1]), __uint_as_float(sr[0][2]));
      float mx1 = max3(__uint_as_float(sr[0][3]), __uint_as_float(sr[0][4]), __uint_as_float(sr[0][5]));
#pragma unroll
      for (int i = 6; i + 3 < BN; i += 4) {
        mx0 = max3(mx0, __uint_as_float(sr[i >> 5][i & 31]), __uint_as_float(sr[(i + 1) >> 5][(i + 1) & 31]));
        mx1 = max3(mx1, __uint_as_float(sr[(i + 2) >> 5][(i + 2) & 31]), __uint_as_float(sr[(i + 3) >> 5][(i + 3) & 31]));
      }
      const float mx = max3(mx0, mx1, fmaxf(__uint_as_float(sr[1][30]), __uint_as_float(sr[1][31]))) * p.scale_log2;
      float alpha = 1.0f;
      const bool grow = mx > m_run + RESCALE_STEP;              // also the first keys a row sees (m_run = -inf)
      if (grow) {
        alpha = exp2f(m_run - mx);                              // 0 when the row had seen nothing
        m_run = mx;
        l *= alpha;
      }
      const float neg_ref = m_run == -INFINITY ? 0.f : -m_run;
      uint32_t pk[BN / 2];
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
      for (int i = 0; i < BN; i += 4) {
        const float p0 = fast_exp2(fmaf(__uint_as_float(sr[i >> 5][i & 31]), p.scale_log2, neg_ref));
        const float p1 = fast_exp2(fmaf(__uint_as_float(sr[i >> 5][(i & 31) + 1]), p.scale_log2, neg_ref));
        const float p2 = fast_exp2(fmaf(__uint_as_float(sr[i >> 5][(i & 31) + 2]), p.scale_log2, neg_ref));
        const float p3 = fast_exp2(fmaf(__uint_as_float(sr[i >> 5][(i & 31) + 3]), p.scale_log2, neg_ref));
        pk[i >> 1] = pack_bf16(p0, p1);
        pk[(i >> 1) + 1] = pack_bf16(p2, p3);
        l0 += p0; l1 += p1; l2 += p2; l3 += p3;                  // the row sum in fp32, before the rounding to bfloat16
      }
      l += (l0 + l1) + (l2 + l3);
      if (j > 0) {
        // the product of the tile before must be complete: P's buffer is free, and O may be rescaled
        ok = mbar_wait(o_full, (uint32_t)(j - 1) & 1, 8);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, grow)) {
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t o[32];
            tmem_ld32_nowait(o, lane_addr + O_COL + c0);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(lane_addr + O_COL + c0, o);
          }
          tmem_st_wait();
        }
      }
      // this row of P over the first 32 columns of the tile's S (all of which this thread has read): two
      // bfloat16 per column, the second product's A operand straight from tensor memory
      tmem_st32(lane_addr + S_COL + (uint32_t)((j & 1) * BN), pk);
      tmem_st_wait();
      if (key_base + BN > total) {
        // keys beyond the request's last one: their V rows may hold anything (0 * NaN = NaN), so zero them
        ok = mbar_wait(&v_full[j & 1], (uint32_t)(j >> 1) & 1, 10);
        if (!ok) break;
        const int first_bad = total - key_base;                  // 1..63
        for (int id = threadIdx.x - 64; id < (BN - first_bad) * DB * 8; id += 128) {
          const int row = first_bad + id / (DB * 8), rem = id % (DB * 8);
          *reinterpret_cast<uint4*>(v_s + (j & 1) * T_BYTES + (rem >> 3) * (BN * 128) + row * 128 + ((rem & 7) << 4)) =
              make_uint4(0, 0, 0, 0);
        }
        fence_async_smem();
      }
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    if (ok) ok = mbar_wait(o_full, (uint32_t)(n_tiles - 1) & 1, 11);
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      bf16* dst = p.out + (size_t)(q_row0 + t0 + tq) * p.out_stride + (size_t)(kvh * G + g) * D;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t o[32];
        tmem_ld32_nowait(o, lane_addr + O_COL + c0);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c0 + i) = w;
          }
        }
      }
    } else {
      *s_abort = 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

bool make_map(CUtensorMap* map, const void* base, long long rows) {
  return nhv_make_map_bf16(map, base, rows, D, D, 64, BN);
}

struct MapKey {
  const void* base;
  long long rows;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const { return std::hash<const void*>()(k.base) ^ ((size_t)k.rows * 1000003u); }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;   // one per cache pool: pools do not move
std::mutex g_maps_mutex;

// The kernel's shared memory, and the whole of the SM's memory as shared memory so that two blocks fit.
bool set_attributes() {
  static bool done = false;
  if (done) return true;
  if (cudaFuncSetAttribute(attn_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return false;
  if (cudaFuncSetAttribute(attn_tcgen05_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                           cudaSharedmemCarveoutMaxShared) != cudaSuccess) return false;
  done = true;
  return true;
}

}  // namespace

#define ATT_REQUIRE(cond, ...)                      \
  do {                                              \
    if (!(cond)) {                                  \
      snprintf(g_err, sizeof(g_err), __VA_ARGS__);  \
      return 1;                                     \
    }                                               \
  } while (0)

NHV_API const char* NHV_FN(nhv_attn_tcgen05_last_error_d)() { return g_err; }

// Reads and clears the error word of the kernel's bounded waits (0: none ran out).  Synchronises the device.
NHV_API int NHV_FN(nhv_attn_tcgen05_error_d)() { return nhv_wait_error_take(); }
// The device address of the error word, for kernels that report it with the step's result.
NHV_API void* NHV_FN(nhv_attn_tcgen05_error_word_d)() { return nhv_wait_error_address(); }

// Attention of the step's prompt portions (requests with more than one new token); requests with one new token
// are left alone.  The page size must be a multiple of 64.
NHV_API int NHV_FN(nhv_attn_tcgen05_d)(const void* q, int q_stride, void* out, int out_stride, const void* kv_pages,
                                       const int* block_table, int bt_stride, const int* cu_q, const int* kv_len,
                                       int n_seqs, int n_prefill_tokens, int n_prefill_seqs, int nq, int nkv,
                                       int page_size, int n_pages, int window, float scale, cudaStream_t stream) {
  ATT_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads do not divide into %d KV heads", nq, nkv);
  const int G = nq / nkv;
  ATT_REQUIRE(G <= BM, "attention: a group of %d query heads is beyond the %d rows of a block", G, BM);
  ATT_REQUIRE(page_size > 0 && page_size % BN == 0, "attention (tcgen05): the page size %d is no multiple of %d", page_size, BN);
  ATT_REQUIRE(n_pages > 0 && bt_stride > 0, "attention: bad page geometry");
  ATT_REQUIRE(q_stride % 8 == 0 && out_stride % 8 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)kv_pages % 16) == 0 &&
                  ((uintptr_t)out % 16) == 0,
              "attention (tcgen05): q, the output and the pages must be 16-byte aligned");
  const long long rows = (long long)n_pages * 2 * nkv * page_size;
  ATT_REQUIRE(rows < (1LL << 31), "attention (tcgen05): the pool's %lld rows are beyond a 32-bit coordinate", rows);
  if (n_prefill_tokens <= 0) return 0;
  ATT_REQUIRE(set_attributes(), "attention (tcgen05): cannot reserve %d bytes of shared memory", SMEM_BYTES);
  Params p;
  {
    std::lock_guard<std::mutex> lock(g_maps_mutex);
    const MapKey key{kv_pages, rows};
    auto it = g_maps.find(key);
    if (it == g_maps.end()) {
      CUtensorMap m;
      ATT_REQUIRE(make_map(&m, kv_pages, rows), "attention (tcgen05): cannot encode the tensor map of the pool");
      it = g_maps.emplace(key, m).first;
    }
    p.kv_map = it->second;
  }
  p.q = (const bf16*)q;
  p.out = (bf16*)out;
  p.block_table = block_table;
  p.cu_q = cu_q;
  p.kv_len = kv_len;
  p.q_stride = q_stride;
  p.out_stride = out_stride;
  p.bt_stride = bt_stride;
  p.n_seqs = n_seqs;
  p.nq = nq;
  p.nkv = nkv;
  p.page_size = page_size;
  p.n_pages = n_pages;
  p.window = window;
  p.tokens_per_block = BM / G;
  p.scale_log2 = scale * LOG2E;
  const int max_tiles = n_prefill_tokens / p.tokens_per_block + n_prefill_seqs;
  ATT_REQUIRE(max_tiles <= 65535, "attention: %d tiles of new tokens are beyond the grid's reach", max_tiles);
  cudaError_t e = nhv_launch(attn_tcgen05_kernel, dim3(nkv, max_tiles), THREADS, SMEM_BYTES, stream, p);
  if (e != cudaSuccess) {
    snprintf(g_err, sizeof(g_err), "attention (tcgen05): launch failed: %s", cudaGetErrorString(e));
    return 2;
  }
  return 0;
}
