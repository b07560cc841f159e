// y[M,N] = x[M,K] * W[N,K]^T in bfloat16 for 17 to 128 tokens on the 5th-generation tensor cores:
// tcgen05.mma with the accumulator in tensor memory, operands brought by TMA.
//
// This is the regime of a decode step with tens of requests (or a small mixed batch): the job is
// still to read W once at the speed of HBM, but the arithmetic is beyond what mma.sync sustains.
// W sits on the MMA's M axis (128 rows per tile), the tokens on its N axis (NT = 32, 64 or 128
// columns), so D[128 x NT] (fp32) lives in NT columns of tensor memory, one row per lane.
//
// Persistent and stream-K like gemm_stream_k.cu: one block per SM; the units (128 rows of W) x
// (64 columns) are dealt to the blocks in contiguous runs; a tile that two blocks share is finished
// by the block that arrives last at the tile's counter, which adds the partial sums from scratch in
// block order.  No block waits for another.
//
// Warp roles: warp 0 lane 0 issues TMA loads (W box 64 x 128, x box 64 x NT, 128-byte swizzle) into
// a ring of stages and arms each stage's mbarrier with the bytes to come; warp 1 allocates tensor
// memory, and its lane 0 issues the MMAs (four K=16 instructions per stage, shared-memory
// descriptors stepping 32 bytes inside the swizzle atom) and commits them to the stage's "empty"
// barrier, and at the end of a tile piece to the accumulator's "full" barrier; warps 2-5 are the
// epilogue: each reads its quarter of the lanes with tcgen05.ld, parks the numbers in shared
// memory, frees the accumulator (two accumulators alternate, so the next piece's MMAs run
// meanwhile) and then the four warps write the tile, or its partial sums, together.
//
// Launched with programmatic dependent launch: the ring is filled with weights before the kernel
// waits for its predecessor.  Every wait is bounded; a wait that runs out sets an error word
// (nhv_gemm_tcgen05_error) and the block leaves through the common exit, which frees its tensor
// memory.  Modes as in gemm_stream_k.cu: 0 bf16, 1 fp32 through bf16, 2 silu(gate) * up (a tile is
// 64 gate rows and the same 64 rows of up).  W is [out, in] (nanovllm/layers/linear.py:40,66).
#include <mutex>
#include <unordered_map>

#define NHV_WAIT_LIMIT (1u << 22)
#include "nhv_async.cuh"

namespace {

typedef __nv_bfloat16 bf16;
constexpr int TILE_ROWS = 128;         // weight rows per tile = MMA M
constexpr int BK = 64;                 // columns per stage = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;           // producer warp, MMA warp, four epilogue warps
constexpr int EPI_THREADS = 128;
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_in_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(slot_in_smem)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// the MMAs issued so far by this thread arrive (once) on `bar` when they have completed
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, both operands K-major
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 consecutive columns of this thread's lane
__device__ __forceinline__ void tmem_ld32(float (&v)[32], uint32_t taddr) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major bf16 operand tile in the 128-byte swizzle: rows of 128 bytes,
// groups of 8 rows 1024 bytes apart (the tile starts on a 1024-byte boundary; `addr` may point 32, 64 or 96
// bytes into the first row to select the K=16 slice).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);            // start address
  d |= (uint64_t)1 << 16;                            // leading byte offset (unused for swizzled K-major), 16 B
  d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset: 8 rows x 128 B
  d |= (uint64_t)1 << 46;                            // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                            // 128-byte swizzle
  return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32, both K-major, M x N.
__device__ __forceinline__ uint32_t instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(EPI_THREADS) : "memory"); }

struct alignas(64) Params {
  CUtensorMap w_map;    // W [N, K], box 64 columns x 128 rows (mode 2: x 64 rows)
  CUtensorMap x_map;    // x [M, K], box 64 columns x NT rows
  void* y;
  float* scratch;       // [grid][2][128][NT] partial sums
  int* counters;        // [tiles], zero between launches
  int M, N, K, ldc, mode, up_row_offset;
};

__device__ __forceinline__ long long unit_begin(int c, long long total, int G) { return (long long)c * total / G; }
__device__ __forceinline__ int unit_owner(long long u, long long total, int G) { return (int)(((u + 1) * G - 1) / total); }

template <int NT, int STAGES>
__global__ void __launch_bounds__(THREADS, 1) gemm_tcgen05_kernel(const __grid_constant__ Params p) {
  constexpr int W_BYTES = TILE_ROWS * 128, X_BYTES = NT * 128;
  constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  constexpr int OUT_LD = NT + 1;                                     // padded row of the parked accumulator
  constexpr uint32_t TMEM_COLS = 2 * NT < 32 ? 32 : 2 * NT;          // two accumulators; a power of two >= 32
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = smem_unaligned + ((1024 - (smem_u32(smem_unaligned) & 1023)) & 1023);
  unsigned char* ring = smem;
  float* parked = reinterpret_cast<float*>(smem + (size_t)STAGES * STAGE_BYTES);   // [128][NT + 1]
  uint64_t* full = reinterpret_cast<uint64_t*>(parked + TILE_ROWS * OUT_LD);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;      // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  __shared__ int s_flag;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x, c = blockIdx.x;
  const int out_rows = p.mode == 2 ? TILE_ROWS / 2 : TILE_ROWS;
  const int tiles = (p.N + out_rows - 1) / out_rows;
  const int kb = (p.K + BK - 1) / BK;
  const long long total = (long long)tiles * kb;
  const long long u0 = unit_begin(c, total, G), u1 = unit_begin(c + 1, total, G);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const long long n_units = u1 - u0;
      auto issue_w = [&](long long i) {
        const long long u = u0 + i;
        const int tile = (int)(u / kb), k = (int)(u - (long long)tile * kb);
        const int s = (int)(i % STAGES);
        unsigned char* dst = ring + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&full[s], STAGE_BYTES);                  // zero-filled parts of a box count too
        if (p.mode == 2) {
          tma_load_2d(dst, &p.w_map, k * BK, tile * (TILE_ROWS / 2), &full[s]);
          tma_load_2d(dst + W_BYTES / 2, &p.w_map, k * BK, p.up_row_offset + tile * (TILE_ROWS / 2), &full[s]);
        } else {
          tma_load_2d(dst, &p.w_map, k * BK, tile * TILE_ROWS, &full[s]);
        }
      };
      auto issue_x = [&](long long i) {
        const int k = (int)((u0 + i) % kb);
        const int s = (int)(i % STAGES);
        tma_load_2d(ring + (size_t)s * STAGE_BYTES + W_BYTES, &p.x_map, k * BK, 0, &full[s]);
      };
      const int pre = (int)min((long long)STAGES, n_units);
      for (int i = 0; i < pre; ++i) issue_w(i);
      pdl_wait();
      for (int i = 0; i < pre; ++i) issue_x(i);
      for (long long i = STAGES; i < n_units; ++i) {
        const int s = (int)(i % STAGES);
        if (!mbar_wait(&empty[s], (uint32_t)((i / STAGES) - 1) & 1, 1)) { s_abort = 1; break; }
        issue_w(i);
        issue_x(i);
      }
    } else {
      pdl_wait();
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    pdl_wait();
    if (lane == 0) {
      const uint32_t idesc = instr_desc(TILE_ROWS, NT);
      int piece = -1, cur_tile = -1;
      bool ok = true;
      for (long long u = u0; u < u1 && ok; ++u) {
        const long long i = u - u0;
        const int s = (int)(i % STAGES);
        const int tile = (int)(u / kb), k = (int)(u - (long long)tile * kb);
        const bool first = tile != cur_tile;
        if (first) {
          cur_tile = tile;
          ++piece;
          if (piece >= 2) ok = mbar_wait(&acc_empty[piece & 1], (uint32_t)((piece >> 1) - 1) & 1, 3);
          if (!ok) break;
          tc_fence_after();
        }
        ok = mbar_wait(&full[s], (uint32_t)(i / STAGES) & 1, 2);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(ring + (size_t)s * STAGE_BYTES);
        const uint32_t b_addr = a_addr + W_BYTES;
        const uint32_t d_addr = tmem_base + (uint32_t)((piece & 1) * NT);
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk)
          tc_mma(d_addr, smem_desc_sw128(a_addr + kk * UMMA_K * 2), smem_desc_sw128(b_addr + kk * UMMA_K * 2), idesc,
                 (first && kk == 0) ? 0u : 1u);
        tc_commit(&empty[s]);                                   // the stage is free once these MMAs have read it
        if (k == kb - 1 || u == u1 - 1) tc_commit(&acc_full[piece & 1]);
      }
      if (!ok) s_abort = 1;
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, 128 threads)
    pdl_wait();
    const int tid = threadIdx.x - 64;                           // 0..127
    const int quarter = warp & 3;                               // the tensor-memory lanes this warp may read
    const int row = quarter * 32 + lane;
    int piece = 0;
    bool ok = true;
    long long u = u0;
    while (u < u1 && ok) {
      const int tile = (int)(u / kb);
      const long long t_first = (long long)tile * kb, t_last = t_first + kb - 1;
      const long long piece_end = min(u1, t_last + 1);
      const bool whole = u == t_first && piece_end == t_last + 1;
      ok = mbar_wait(&acc_full[piece & 1], (uint32_t)(piece >> 1) & 1, 4);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)((piece & 1) * NT);
#pragma unroll
      for (int c0 = 0; c0 < NT; c0 += 32) {
        float v[32];
        tmem_ld32(v, taddr + c0);
#pragma unroll
        for (int j = 0; j < 32; ++j) parked[row * OUT_LD + c0 + j] = v[j];
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[piece & 1]);        // the next piece may overwrite this accumulator
      epi_sync();

      int pieces = 1, c_first = c;
      bool finisher = whole;
      if (!whole) {
        c_first = unit_owner(t_first, total, G);
        pieces = unit_owner(t_last, total, G) - c_first + 1;
        const int slot = (int)(u0 / kb) == tile ? 0 : 1;
        float* mine = p.scratch + ((size_t)c * 2 + slot) * TILE_ROWS * NT;
        for (int id = tid; id < TILE_ROWS * NT / 4; id += EPI_THREADS) {
          const int e = id * 4;
          const float* src = parked + (e / NT) * OUT_LD + (e % NT);
          reinterpret_cast<float4*>(mine)[id] = make_float4(src[0], src[1], src[2], src[3]);
        }
        __threadfence();
        epi_sync();
        if (tid == 0) s_flag = atomicAdd(&p.counters[tile], 1);
        epi_sync();
        finisher = s_flag == pieces - 1;
        if (finisher) {                                         // the last block to arrive: add all partials in block order
          __threadfence();
          // four outputs of 16 bytes per thread at a time, each with up to four pieces in flight: the loads
          // do not depend on one another, so the L2 latency is paid once per batch and not once per load
          const float4* __restrict__ parts = reinterpret_cast<const float4*>(p.scratch);
          constexpr int PIECE_F4 = TILE_ROWS * NT / 4;
          for (int id0 = tid; id0 < PIECE_F4; id0 += 4 * EPI_THREADS) {
            float4 acc[4];
#pragma unroll
            for (int v = 0; v < 4; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int q0 = 0; q0 < pieces; q0 += 4) {
              float4 t[4][4];
              size_t base[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int cc = c_first + min(q0 + j, pieces - 1);
                const int sl = (int)(unit_begin(cc, total, G) / kb) == tile ? 0 : 1;
                base[j] = ((size_t)cc * 2 + sl) * PIECE_F4;
              }
#pragma unroll
              for (int v = 0; v < 4; ++v)
#pragma unroll
                for (int j = 0; j < 4; ++j) t[v][j] = __ldcg(parts + base[j] + min(id0 + v * EPI_THREADS, PIECE_F4 - 1));
#pragma unroll
              for (int v = 0; v < 4; ++v)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  if (q0 + j < pieces) { acc[v].x += t[v][j].x; acc[v].y += t[v][j].y; acc[v].z += t[v][j].z; acc[v].w += t[v][j].w; }
            }
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int id = id0 + v * EPI_THREADS;
              if (id < PIECE_F4) {
                const int e = id * 4;
                float* dst = parked + (e / NT) * OUT_LD + (e % NT);
                dst[0] = acc[v].x; dst[1] = acc[v].y; dst[2] = acc[v].z; dst[3] = acc[v].w;
              }
            }
          }
          epi_sync();
        }
      }
      if (finisher) {
        // thread = output column n (a weight row), loop over tokens: for one token the threads write one run of bytes
        const int n = tile * out_rows + tid;
        if (tid < out_rows && n < p.N) {
          for (int m = 0; m < p.M; ++m) {
            float v = __bfloat162float(__float2bfloat16_rn(parked[tid * OUT_LD + m]));
            if (p.mode == 2) {
              const float up = __bfloat162float(__float2bfloat16_rn(parked[(TILE_ROWS / 2 + tid) * OUT_LD + m]));
              v = v / (1.0f + expf(-v)) * up;
            }
            if (p.mode == 1)
              reinterpret_cast<float*>(p.y)[(size_t)m * p.ldc + n] = v;
            else
              reinterpret_cast<bf16*>(p.y)[(size_t)m * p.ldc + n] = __float2bfloat16_rn(v);
          }
        }
        if (!whole && tid == 0) p.counters[tile] = 0;           // ready for the next launch
      }
      epi_sync();                                               // `parked` is reused by the next piece
      u = piece_end;
      ++piece;
    }
    if (!ok && lane == 0) s_abort = 1;
  }
  // ------------------------------------------------------------------ common exit
  __syncthreads();
  if (s_abort) give_up_delay();                                 // let copies that may still be in flight land
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int NT, int STAGES>
int launch(const Params& p, int grid, cudaStream_t stream) {
  constexpr size_t smem = 1024 + (size_t)STAGES * (TILE_ROWS + NT) * 128 + (size_t)TILE_ROWS * (NT + 1) * 4 +
                          (2 * STAGES + 4) * 8 + 16;
  static_assert(smem <= 227 * 1024, "the ring, the parked accumulator and the barriers must fit one block's shared memory");
  static bool attr_set = false;
  if (!attr_set) {
    NHV_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<NT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
             "gemm_tcgen05");
    attr_set = true;
  }
  NHV_CUDA(nhv_launch(gemm_tcgen05_kernel<NT, STAGES>, dim3(grid), dim3(THREADS), smem, stream, p), "gemm_tcgen05");
  return 0;
}

bool make_map(CUtensorMap* map, const void* base, int rows, int cols, int row_stride_elems, int box_rows) {
  return nhv_make_map_bf16(map, base, rows, cols, row_stride_elems, BK, box_rows);
}

struct MapKey {
  const void* base;
  int rows, cols, box_rows;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.base) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.cols << 20) ^ (size_t)k.box_rows;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_weight_maps;   // weights do not move: one map per matrix
std::mutex g_maps_mutex;

}  // namespace

// Reads and clears the error word (0: no bounded wait ever ran out).  Synchronises the device.
NHV_API int nhv_gemm_tcgen05_error() { return nhv_wait_error_take(); }
// The device address of the error word, for kernels that report it with the step's result.
NHV_API void* nhv_gemm_tcgen05_error_word() { return nhv_wait_error_address(); }

// Tokens per MMA column tile for a batch of M tokens (the scratch is [grid][2][128][this] floats).
NHV_API int nhv_gemm_tcgen05_token_tile(int M) { return M <= 32 ? 32 : (M <= 64 ? 64 : 128); }

NHV_API int nhv_gemm_tcgen05(void* y, const void* x, const void* W, int M, int N, int K, int lda, int ldc, int mode,
                             int up_row_offset, float* scratch, int* counters, int counters_len, int grid,
                             cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  NHV_REQUIRE(M > 0 && M <= 128, "gemm_tcgen05: takes 1 to 128 tokens, got %d", M);
  NHV_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0 && lda >= K && ldc >= N,
              "gemm_tcgen05: K and the row stride of x must be multiples of 8 (N=%d K=%d lda=%d)", N, K, lda);
  NHV_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)W % 16) == 0, "gemm_tcgen05: x and W must be 16-byte aligned");
  NHV_REQUIRE(mode >= 0 && mode <= 2 && grid > 0 && scratch && counters, "gemm_tcgen05: bad arguments");
  const int out_rows = mode == 2 ? TILE_ROWS / 2 : TILE_ROWS;
  const int tiles = (N + out_rows - 1) / out_rows;
  NHV_REQUIRE(tiles <= counters_len, "gemm_tcgen05: %d tiles but room for %d counters", tiles, counters_len);
  const int nt = nhv_gemm_tcgen05_token_tile(M);
  Params p;
  p.y = y; p.scratch = scratch; p.counters = counters;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.mode = mode; p.up_row_offset = up_row_offset;
  const int w_rows = mode == 2 ? up_row_offset + N : N, w_box = mode == 2 ? TILE_ROWS / 2 : TILE_ROWS;
  {
    std::lock_guard<std::mutex> lock(g_maps_mutex);
    const MapKey key{W, w_rows, K, w_box};
    auto it = g_weight_maps.find(key);
    if (it == g_weight_maps.end()) {
      CUtensorMap m;
      NHV_REQUIRE(make_map(&m, W, w_rows, K, K, w_box), "gemm_tcgen05: cannot encode the tensor map of W [%d, %d]", w_rows, K);
      it = g_weight_maps.emplace(key, m).first;
    }
    p.w_map = it->second;
  }
  NHV_REQUIRE(make_map(&p.x_map, x, M, K, lda, nt), "gemm_tcgen05: cannot encode the tensor map of x [%d, %d]", M, K);
  const long long total = (long long)tiles * ((K + BK - 1) / BK);
  if (grid > total) grid = (int)total;
  if (nt == 32) return launch<32, 8>(p, grid, stream);
  if (nt == 64) return launch<64, 7>(p, grid, stream);
  return launch<128, 5>(p, grid, stream);
}
