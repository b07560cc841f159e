// y[M,N] = x[M,K] * W[N,K]^T in bfloat16 for up to 16 tokens: the decode step's projections,
// where the whole job is to read W once at the speed of HBM.
//
// Persistent, stream-K: the grid is one block per SM.  The work is cut into units of (64 rows
// of W) x (BK columns); unit u = tile * (K / BK) + k-block, and block c owns the contiguous
// units [c * U / G, (c + 1) * U / G), so every SM reads the same number of bytes whatever N and
// K are.  A producer thread streams its units through a ring of shared-memory stages with TMA
// tensor copies (cp.async.bulk.tensor.2d, boxes of 64 columns x 64 rows in the 128-byte swizzle,
// completion counted in bytes on an mbarrier; rows and columns beyond the matrix arrive as
// zeros); four consumer warps take a quarter of each stage's columns
// each (mma.sync.m16n8k16, W rows on the MMA's M axis, tokens on its N axis, fp32
// accumulators).  At the end of a tile the four warps' sums are added through shared memory.  A
// block that owns all k-blocks of a tile writes the result; otherwise it stores its partial sums
// to scratch, and the block that arrives last at the tile's counter adds all partials in block
// order and writes the result: no block ever waits for another, and the order of the sums is
// fixed.
//
// The kernel is launched with programmatic dependent launch: it starts while the kernel before
// it in the stream is still running, fills its ring with weights (which no kernel writes), and
// only then waits for that kernel (griddepcontrol.wait) before it reads x or writes anything.
//
// Modes: 0: y bf16.  1: y fp32, rounded through bf16 as nanovllm/layers/embed_head.py:61 with
// nanovllm/layers/sampler.py:12 gives logits.  2: W = [gate rows; up rows], y = silu(gate) * up
// (nanovllm/layers/activation.py:9-11), both products rounded to bf16 first: a tile is 32 gate
// rows and the same 32 rows of up.  W is [out, in] row-major (nanovllm/layers/linear.py:40,66).
//
// Every wait on an mbarrier is bounded; a wait that runs out sets an error word that the host
// reads with nhv_gemm_stream_k_error().
#include <atomic>
#include <mutex>
#include <unordered_map>

#include "nhv_async.cuh"
#include "nhv_no_alloc.h"

namespace {

typedef __nv_bfloat16 bf16;
constexpr int ROWS = 64;                 // weight rows per tile (4 MMA row tiles)
constexpr int MT = ROWS / 16;
constexpr int CONSUMER_WARPS = 4;
constexpr int THREADS = (CONSUMER_WARPS + 1) * 32;
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Count this block's arrival at a tile: release (what the block wrote before is visible to whoever sees the
// count) and acquire (what earlier arrivals wrote is visible to this block).  Returns the count before.
__device__ __forceinline__ int arrive_acq_rel(int* counter) {
  int old;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;\n" : "=r"(old) : "l"(counter) : "memory");
  return old;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(CONSUMER_WARPS * 32) : "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { pdl_wait(); }
__device__ __forceinline__ void launch_dependents() { pdl_launch_dependents(); }

#ifndef NHV_STREAM_K_BK
#define NHV_STREAM_K_BK 256
#endif
#ifndef NHV_STREAM_K_STAGES
#define NHV_STREAM_K_STAGES 5
#endif
constexpr int BK = NHV_STREAM_K_BK;      // columns per stage
constexpr int BOX_COLS = 64;             // columns per TMA box: 128 bytes, the widest the 128-byte swizzle takes
constexpr int BOXES = BK / BOX_COLS;

struct alignas(64) Params {
  CUtensorMap w_map;    // W [N, K], box 64 columns x 64 rows (mode 2: x 32 rows)
  CUtensorMap x_map;    // x [M, K], box 64 columns x (8 or 16) rows
  void* y;
  const bf16* x;
  const bf16* W;
  float* scratch;       // [grid][2][ROWS][8 * NT] partial sums
  int* counters;        // [tiles], zero between launches
  int M, N, K, lda, ldc, mode, up_row_offset;
};

__device__ __forceinline__ long long unit_begin(int c, long long total, int G) { return (long long)c * total / G; }
__device__ __forceinline__ int unit_owner(long long u, long long total, int G) { return (int)(((u + 1) * G - 1) / total); }

template <int NT, int STAGES>
__global__ void __launch_bounds__(THREADS, NHV_STREAM_K_BK <= 128 ? 2 : 1) gemm_stream_k_kernel(const __grid_constant__ Params p) {
  constexpr int X_ROWS = NT * 8;
  constexpr int W_BOX_BYTES = ROWS * 128, X_BOX_BYTES = X_ROWS * 128;
  constexpr int STAGE_BYTES = BOXES * (W_BOX_BYTES + X_BOX_BYTES);     // W boxes first, then x boxes
  extern __shared__ unsigned char smem_unaligned[];
  // the swizzle pattern repeats every 1024 bytes: boxes must start on such a boundary
  unsigned char* smem = smem_unaligned + ((1024 - (smem_u32(smem_unaligned) & 1023)) & 1023);
  unsigned char* ring = smem;
  float* red = reinterpret_cast<float*>(smem + (size_t)STAGES * STAGE_BYTES);       // [4][ROWS][X_ROWS]
  uint64_t* full = reinterpret_cast<uint64_t*>(red + CONSUMER_WARPS * ROWS * X_ROWS);
  uint64_t* empty = full + STAGES;
  __shared__ int s_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x, c = blockIdx.x;
  const int out_rows = p.mode == 2 ? ROWS / 2 : ROWS;       // result columns per tile
  const int tiles = (p.N + out_rows - 1) / out_rows;
  const int kb = (p.K + BK - 1) / BK;
  const long long total = (long long)tiles * kb;
  const long long u0 = unit_begin(c, total, G), u1 = unit_begin(c + 1, total, G);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], CONSUMER_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  launch_dependents();

  if (warp == CONSUMER_WARPS) {
    // ---------------------------------------------------------------- producer (one thread)
    if (lane == 0) {
      const long long n_units = u1 - u0;
      auto issue_w = [&](long long i) {
        const long long u = u0 + i;
        const int tile = (int)(u / kb), k = (int)(u - (long long)tile * kb);
        const int s = (int)(i % STAGES);
        unsigned char* dst = ring + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&full[s], STAGE_BYTES);                 // zero-filled parts of a box count too
#pragma unroll
        for (int b = 0; b < BOXES; ++b) {
          const int col = k * BK + b * BOX_COLS;
          if (p.mode == 2) {     // 32 gate rows, then the same 32 rows of up
            tma_load_2d(dst + b * W_BOX_BYTES, &p.w_map, col, tile * (ROWS / 2), &full[s]);
            tma_load_2d(dst + b * W_BOX_BYTES + W_BOX_BYTES / 2, &p.w_map, col, p.up_row_offset + tile * (ROWS / 2), &full[s]);
          } else {
            tma_load_2d(dst + b * W_BOX_BYTES, &p.w_map, col, tile * ROWS, &full[s]);
          }
        }
      };
      auto issue_x = [&](long long i) {
        const int k = (int)((u0 + i) % kb);
        const int s = (int)(i % STAGES);
        unsigned char* dst = ring + (size_t)s * STAGE_BYTES + BOXES * W_BOX_BYTES;
#pragma unroll
        for (int b = 0; b < BOXES; ++b) tma_load_2d(dst + b * X_BOX_BYTES, &p.x_map, k * BK + b * BOX_COLS, 0, &full[s]);
      };
      // Fill the ring with weights while the kernel before this one may still be running, then wait for it.
      const int pre = (int)min((long long)STAGES, n_units);
      for (int i = 0; i < pre; ++i) issue_w(i);
      grid_dependency_wait();
      for (int i = 0; i < pre; ++i) issue_x(i);
      bool ok = true;
      for (long long i = STAGES; i < n_units; ++i) {
        const int s = (int)(i % STAGES);
        ok = mbar_wait(&empty[s], (uint32_t)((i / STAGES) - 1) & 1, 1);
        if (!ok) break;
        issue_w(i);
        issue_x(i);
      }
      if (!ok) give_up_delay();
    } else {
      grid_dependency_wait();
    }
  } else {
    // ---------------------------------------------------------------- consumers
    grid_dependency_wait();
    float acc[MT][NT][4];
    auto clear = [&]() {
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
    };
    clear();
    constexpr int KSTEPS = BK / 16 / CONSUMER_WARPS;        // k-steps per warp per stage
    static_assert(KSTEPS >= 1 && BOX_COLS % (KSTEPS * 16) == 0, "a warp's columns of a stage lie inside one box");
    const int tid = threadIdx.x;                              // 0..127
    int deferred_tile = -1, deferred_arrived = 0;
    // the tile's result from red: the four warps' sums (a tile this block computed alone) or red[0] (gathered)
    auto write_tile = [&](int tile, bool whole) {
      for (int id = tid; id < out_rows * X_ROWS; id += CONSUMER_WARPS * 32) {
        const int m = id / out_rows, r = id - m * out_rows;
        const int n = tile * out_rows + r;
        if (m >= p.M || n >= p.N) continue;
        auto value = [&](int row) -> float {
          float v = 0.f;
          if (whole) {
#pragma unroll
            for (int w = 0; w < CONSUMER_WARPS; ++w) v += red[(w * ROWS + row) * X_ROWS + m];
          } else {
            v = red[row * X_ROWS + m];
          }
          return __bfloat162float(__float2bfloat16_rn(v));
        };
        float v = value(r);
        if (p.mode == 2) {
          const float up = value(32 + r);
          v = v / (1.0f + expf(-v)) * up;
        }
        if (p.mode == 1)
          reinterpret_cast<float*>(p.y)[(size_t)m * p.ldc + n] = v;
        else
          reinterpret_cast<bf16*>(p.y)[(size_t)m * p.ldc + n] = __float2bfloat16_rn(v);
      }
    };
    auto tile_pieces = [&](int tile) -> int {
      const long long t_first = (long long)tile * kb;
      return unit_owner(t_first + kb - 1, total, G) - unit_owner(t_first, total, G) + 1;
    };
    // the block that arrived last at a shared tile: add all blocks' sums in block order and write the tile
    auto finish_shared_tile = [&](int tile) {
      const long long t_first = (long long)tile * kb;
      const int c_first = unit_owner(t_first, total, G);
      const int pieces = tile_pieces(tile);
      // gather the partial sums into red[0] first: 16 bytes per thread and piece, four pieces in flight
      float4* sum4 = reinterpret_cast<float4*>(red);
      for (int id = tid; id < ROWS * X_ROWS / 4; id += CONSUMER_WARPS * 32) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q0 = 0; q0 < pieces; q0 += 4) {
          float4 t[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int cc = c_first + min(q0 + j, pieces - 1);
            const int slot = (int)(unit_begin(cc, total, G) / kb) == tile ? 0 : 1;
            t[j] = __ldcg(reinterpret_cast<const float4*>(p.scratch + ((size_t)cc * 2 + slot) * ROWS * X_ROWS) + id);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (q0 + j < pieces) { v.x += t[j].x; v.y += t[j].y; v.z += t[j].z; v.w += t[j].w; }
        }
        sum4[id] = v;
      }
      consumer_sync();
      write_tile(tile, false);
      if (tid == 0) p.counters[tile] = 0;                     // ready for the next launch
      consumer_sync();
    };
    bool ok = true;
    for (long long u = u0; u < u1 && ok; ++u) {
      const long long i = u - u0;
      const int s = (int)(i % STAGES);
      const int tile = (int)(u / kb), k = (int)(u - (long long)tile * kb);
      ok = mbar_wait(&full[s], (uint32_t)(i / STAGES) & 1, 2);
      if (!ok) { give_up_delay(); break; }
      // this warp's box of the stage; inside a box row r holds its 16-byte chunk c at chunk (c ^ (r & 7))
      const int my_box = warp * KSTEPS * 16 / BOX_COLS;
      const unsigned char* ws = ring + (size_t)s * STAGE_BYTES + my_box * W_BOX_BYTES;
      const unsigned char* xs = ring + (size_t)s * STAGE_BYTES + BOXES * W_BOX_BYTES + my_box * X_BOX_BYTES;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        const int c0 = ((warp * KSTEPS + kk) * 2) % (BOX_COLS / 8);
        uint32_t b[4];
        {
          const int r = NT == 1 ? (lane & 7) : (lane & 7) + ((lane >> 4) << 3);
          const int ch = c0 + ((lane >> 3) & 1);
          ldmatrix_x4(b, xs + r * 128 + ((ch ^ (r & 7)) << 4));
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          uint32_t a[4];
          const int r = mt * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          const int ch = c0 + (lane >> 4);
          ldmatrix_x4(a, ws + r * 128 + ((ch ^ (r & 7)) << 4));
          mma_bf16(acc[mt][0], a, b[0], b[1]);
          if (NT == 2) mma_bf16(acc[mt][NT - 1], a, b[2], b[3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);

      const bool tile_ends = k == kb - 1 || u == u1 - 1;
      if (!tile_ends) continue;
      // ------------------------------------------------------------ end of this block's piece of the tile
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int r = mt * 16 + (lane >> 2) + ((e >> 1) << 3);
            const int m = j * 8 + ((lane & 3) << 1) + (e & 1);
            red[(warp * ROWS + r) * X_ROWS + m] = acc[mt][j][e];
          }
      clear();
      consumer_sync();
      const long long t_first = (long long)tile * kb, t_last = t_first + kb - 1;
      const bool whole = u0 <= t_first && u1 > t_last;
      if (whole) {
        write_tile(tile, true);
        consumer_sync();
        continue;
      }
      // A tile shared with other blocks: park this block's sums in scratch and count the arrival.  The arrival
      // is a release (the barrier before it orders the other threads' stores before it) and an acquire (the last
      // block to arrive may read the others' sums), so no thread stands at a fence.
      // slot 0: the tile this block's range starts in; slot 1: a later tile that it only begins
      const int slot = (int)(u0 / kb) == tile ? 0 : 1;
      float* mine = p.scratch + ((size_t)c * 2 + slot) * ROWS * X_ROWS;
      for (int id = tid; id < ROWS * X_ROWS; id += CONSUMER_WARPS * 32) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < CONSUMER_WARPS; ++w) v += red[w * ROWS * X_ROWS + id];
        mine[id] = v;
      }
      consumer_sync();
      int arrived = 0;
      if (tid == 0) arrived = arrive_acq_rel(&p.counters[tile]);
      if (u != u1 - 1) {
        // more units follow: keep the stream going and look at the count when it has ended (only the first tile
        // of a block's range can end in the middle of it)
        deferred_tile = tile;
        deferred_arrived = arrived;
        continue;
      }
      if (tid == 0) s_flag = arrived;
      consumer_sync();
      if (s_flag == tile_pieces(tile) - 1) finish_shared_tile(tile);
      consumer_sync();
    }
    if (deferred_tile >= 0) {
      if (tid == 0) s_flag = deferred_arrived;
      consumer_sync();
      if (s_flag == tile_pieces(deferred_tile) - 1) finish_shared_tile(deferred_tile);
    }
  }
}

template <int NT, int STAGES>
int launch(const Params& p, int grid, cudaStream_t stream) {
  constexpr int X_ROWS = NT * 8;
  constexpr size_t smem = 1024 + (size_t)STAGES * BOXES * (ROWS + X_ROWS) * 128 + (size_t)CONSUMER_WARPS * ROWS * X_ROWS * 4 +
                          2 * STAGES * 8;
  // the attribute belongs to the device that is current: set once for each
  static std::atomic<bool> attr_set[64];
  int dev = 0;
  NHV_CUDA(cudaGetDevice(&dev), "gemm_stream_k");
  if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
    NHV_CUDA(cudaFuncSetAttribute(gemm_stream_k_kernel<NT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)smem), "gemm_stream_k");
    if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  NHV_CUDA(cudaLaunchKernelEx(&cfg, gemm_stream_k_kernel<NT, STAGES>, p), "gemm_stream_k");
  return 0;
}

// ---------------------------------------------------------------- tensor maps (host)
bool make_map(CUtensorMap* map, const void* base, int rows, int cols, int row_stride_elems, int box_rows) {
  return nhv_make_map_bf16(map, base, rows, cols, row_stride_elems, BOX_COLS, box_rows);
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

// How much scratch the kernel wants for a grid of `grid` blocks: floats of partial sums, ints of counters
// (the counters must be zero before the first launch; the kernel leaves them zero).
NHV_API int nhv_gemm_stream_k_scratch(int grid, int max_tiles, size_t* partial_floats, size_t* counter_ints) {
  *partial_floats = (size_t)grid * 2 * ROWS * 16;
  *counter_ints = (size_t)max_tiles;
  return 0;
}

// Reads and clears the error word (0: no bounded wait ever ran out).  Synchronises the device.
NHV_API int nhv_gemm_stream_k_error() { return nhv_wait_error_take(); }
// The device address of the error word, for kernels that report it with the step's result.
NHV_API void* nhv_gemm_stream_k_error_word() { return nhv_wait_error_address(); }

NHV_API int nhv_gemm_stream_k(void* y, const void* x, const void* W, int M, int N, int K, int lda, int ldc, int mode,
                              int up_row_offset, float* scratch, int* counters, int counters_len, int grid,
                              cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  NHV_REQUIRE(M > 0 && M <= 16, "gemm_stream_k: takes 1 to 16 tokens, got %d", M);
  NHV_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0 && lda >= K && ldc >= N,
              "gemm_stream_k: K and the row stride of x must be multiples of 8 (N=%d K=%d lda=%d)", N, K, lda);
  NHV_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)W % 16) == 0, "gemm_stream_k: x and W must be 16-byte aligned");
  NHV_REQUIRE(mode >= 0 && mode <= 2 && grid > 0 && scratch && counters, "gemm_stream_k: bad arguments");
  const int out_rows = mode == 2 ? ROWS / 2 : ROWS;
  const int tiles = (N + out_rows - 1) / out_rows;
  NHV_REQUIRE(tiles <= counters_len, "gemm_stream_k: %d tiles but room for %d counters", tiles, counters_len);
  Params p;
  p.y = y; p.x = (const bf16*)x; p.W = (const bf16*)W; p.scratch = scratch; p.counters = counters;
  p.M = M; p.N = N; p.K = K; p.lda = lda; p.ldc = ldc; p.mode = mode; p.up_row_offset = up_row_offset;
  const int w_rows = mode == 2 ? up_row_offset + N : N, w_box = mode == 2 ? ROWS / 2 : ROWS;
  {
    std::lock_guard<std::mutex> lock(g_maps_mutex);
    const MapKey key{W, w_rows, K, w_box};
    auto it = g_weight_maps.find(key);
    if (it == g_weight_maps.end()) {
      CUtensorMap m;
      NHV_REQUIRE(make_map(&m, W, w_rows, K, K, w_box), "gemm_stream_k: cannot encode the tensor map of W [%d, %d]", w_rows, K);
      it = g_weight_maps.emplace(key, m).first;
    }
    p.w_map = it->second;
  }
  NHV_REQUIRE(make_map(&p.x_map, x, M, K, lda, M <= 8 ? 8 : 16), "gemm_stream_k: cannot encode the tensor map of x [%d, %d]", M, K);
  const long long total = (long long)tiles * ((K + BK - 1) / BK);
  if (grid > total) grid = (int)total;
  if (M <= 8) return launch<1, NHV_STREAM_K_STAGES>(p, grid, stream);
  return launch<2, NHV_STREAM_K_STAGES>(p, grid, stream);
}

// ------------------------------------------------------------------------------------------------
// An entry point that allocates nothing (declared in nhv_no_alloc.h; it has no counterpart in the
// reference).  Same product as nhv_gemm_stream_k, but the partial sums and tile counters live in a
// fixed array inside this library instead of buffers the caller allocates.
namespace {

constexpr int STATIC_MAX_GRID = 160;                                   // blocks (one per SM) the array has room for
constexpr int STATIC_MAX_TILES = 4096;                                 // output tiles it has counters for
constexpr size_t STATIC_PARTIAL_BYTES = (size_t)STATIC_MAX_GRID * 2 * ROWS * 16 * sizeof(float);   // 1.25 MiB
constexpr size_t STATIC_COUNTER_BYTES = (size_t)STATIC_MAX_TILES * sizeof(int);                    // 16 KiB
constexpr int STATIC_MAX_DEVICES = 64;

// Held by every GPU that loads this library, until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_PARTIAL_BYTES + STATIC_COUNTER_BYTES];

struct StaticScratch {
  // device address of g_static_scratch on this device; stored last (release) by the thread that sets the device
  // up, so that a thread that sees it (acquire) also sees `sms`
  std::atomic<unsigned char*> base{nullptr};
  int sms = 0;
};
StaticScratch g_static[STATIC_MAX_DEVICES];
std::mutex g_static_mutex;

}  // namespace

NHV_API int nhv_gemm_stream_k_no_alloc(void* y, const void* x, const void* W, int M, int N, int K, int lda, int ldc,
                                       int mode, int up_row_offset, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  NHV_REQUIRE(M > 0 && M <= 16, "gemm_stream_k_no_alloc: takes 1 to 16 tokens, got %d", M);
  NHV_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0 && lda >= K && ldc >= N,
              "gemm_stream_k_no_alloc: K and the row stride of x must be multiples of 8 (N=%d K=%d lda=%d)", N, K, lda);
  NHV_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)W % 16) == 0, "gemm_stream_k_no_alloc: x and W must be 16-byte aligned");
  NHV_REQUIRE(mode >= 0 && mode <= 2, "gemm_stream_k_no_alloc: unknown mode %d", mode);
  const int out_rows = mode == 2 ? ROWS / 2 : ROWS;
  const int tiles = (N + out_rows - 1) / out_rows;
  NHV_REQUIRE(tiles <= STATIC_MAX_TILES, "gemm_stream_k_no_alloc: N=%d makes %d output tiles, the built-in scratch has "
              "counters for %d (N up to %d)", N, tiles, STATIC_MAX_TILES, STATIC_MAX_TILES * out_rows);
  int dev = 0;
  NHV_CUDA(cudaGetDevice(&dev), "gemm_stream_k_no_alloc");
  NHV_REQUIRE(dev >= 0 && dev < STATIC_MAX_DEVICES, "gemm_stream_k_no_alloc: device %d is beyond the %d this library tracks", dev,
              STATIC_MAX_DEVICES);
  StaticScratch* st = &g_static[dev];
  unsigned char* base = st->base.load(std::memory_order_acquire);
  if (base == nullptr) {
    // Set-up, once per device, with that device current.  In host code the array's name only stands for the
    // symbol; the address a kernel can use comes from cudaGetSymbolAddress.
    std::lock_guard<std::mutex> lock(g_static_mutex);
    base = st->base.load(std::memory_order_acquire);
    if (base == nullptr) {
      unsigned char* ptr = nullptr;
      NHV_CUDA(cudaGetSymbolAddress((void**)&ptr, g_static_scratch), "gemm_stream_k_no_alloc: address of the built-in scratch");
      NHV_REQUIRE(ptr != nullptr, "gemm_stream_k_no_alloc: the built-in scratch has no device address");
      int sms = 0;
      NHV_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "gemm_stream_k_no_alloc");
      // the counters must start at zero (the kernel returns them to zero after every call that completes)
      NHV_CUDA(cudaMemsetAsync(ptr + STATIC_PARTIAL_BYTES, 0, STATIC_COUNTER_BYTES, stream), "gemm_stream_k_no_alloc");
      st->sms = sms;
      st->base.store(ptr, std::memory_order_release);
      base = ptr;
    }
  }
  int grid = st->sms < STATIC_MAX_GRID ? st->sms : STATIC_MAX_GRID;
  Params p;
  p.y = y; p.x = (const bf16*)x; p.W = (const bf16*)W;
  p.scratch = reinterpret_cast<float*>(base);
  p.counters = reinterpret_cast<int*>(base + STATIC_PARTIAL_BYTES);
  p.M = M; p.N = N; p.K = K; p.lda = lda; p.ldc = ldc; p.mode = mode; p.up_row_offset = up_row_offset;
  const int w_rows = mode == 2 ? up_row_offset + N : N, w_box = mode == 2 ? ROWS / 2 : ROWS;
  // both tensor maps are encoded on the stack: no cache, nothing allocated on the host either
  NHV_REQUIRE(make_map(&p.w_map, W, w_rows, K, K, w_box), "gemm_stream_k_no_alloc: cannot encode the tensor map of W [%d, %d]", w_rows, K);
  NHV_REQUIRE(make_map(&p.x_map, x, M, K, lda, M <= 8 ? 8 : 16), "gemm_stream_k_no_alloc: cannot encode the tensor map of x [%d, %d]", M, K);
  const long long total = (long long)tiles * ((K + BK - 1) / BK);
  if (grid > total) grid = (int)total;
  if (M <= 8) return launch<1, NHV_STREAM_K_STAGES>(p, grid, stream);
  return launch<2, NHV_STREAM_K_STAGES>(p, grid, stream);
}

