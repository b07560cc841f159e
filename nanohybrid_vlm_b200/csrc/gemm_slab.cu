// y[M,N] = x[M,K] * W[N,K]^T in bfloat16 for up to 8 tokens, from a copy of W laid out for this kernel: the
// decode step's projections, where the whole job is to read W once at the speed of HBM.
//
// The copy ("slabs", made once when the weights are loaded, ops.slab_weight) cuts W's rows into one share per
// block: G blocks, rpb = ceil(N / G) rows each, so every SM reads the same number of bytes and no output is
// shared between blocks: nothing to add up across blocks, no scratch, no counters, and a block is done when its
// last product is.  (gemm_stream_k.cu balances a row-major matrix by cutting along K instead and pays for it
// with a fix-up at the end of every launch.)  A block's share is walked in sub-tiles of up to 64 rows (mode 2:
// 32 gate rows and the same 32 rows of up), each over all of K in stages of nb * 64 columns; the bytes of one
// stage of one sub-tile are contiguous in the copy and already in the order they take in shared memory (box by
// box of 64 columns; in a box rows of 128 bytes, mode 2: the gate rows then the up rows; the 16-byte chunks of
// row r exchanged by c ^ (r & 7), which is what ldmatrix reads without bank conflicts), so a stage arrives by
// one linear bulk copy of up to 32 KB (cp.async.bulk, completion counted in bytes on an mbarrier).  x comes by TMA
// tensor copies with the same swizzle: a stage's columns in one copy where K is a multiple of 64 (x seen as
// [K / 64][M][64]), since what the TMA unit can take is a number of copies rather than of bytes.
//
// One producer thread streams the stages through a ring; four consumer warps take a quarter of each stage's
// columns each (mma.sync.m16n8k16, W rows on the MMA's M axis, tokens on its N axis, fp32 accumulators) and add
// their sums through shared memory at the end of a sub-tile.  Launched with programmatic dependent launch: the
// ring is filled with weights before the kernel waits for its predecessor.  Every wait on an mbarrier is bounded;
// one that runs out sets an error word (nhv_gemm_slab_error).
//
// Modes: 0: y bf16.  1: y fp32, rounded through bf16 as nanovllm/layers/embed_head.py:61 with
// nanovllm/layers/sampler.py:12 gives logits.  2: y = silu(gate) * up (nanovllm/layers/activation.py:9-11), both
// products rounded to bf16 first.  W is [out, in] (nanovllm/layers/linear.py:40,66).
#include "nhv_async.cuh"

// Test builds only (tests compile this file into a library of its own with a short NHV_WAIT_LIMIT): the producer
// leaves the copies of ring unit NHV_TEST_DROP_UNIT unsent, so that the consumers' wait for it runs out and the
// way out of a run-out wait (error word, delay, ordinary exit) is exercised without a fault or a hang.
#ifdef NHV_TEST_DROP_UNIT
#define NHV_UNIT_IS_SENT(i) ((i) != (NHV_TEST_DROP_UNIT))
#else
#define NHV_UNIT_IS_SENT(i) true
#endif

namespace {

typedef __nv_bfloat16 bf16;
constexpr int ROWS = 64;                 // shared-memory rows of a sub-tile (4 MMA row tiles)
constexpr int MT = ROWS / 16;
constexpr int X_ROWS = 8;                // tokens
constexpr int CONSUMER_WARPS = 4;
constexpr int THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int STAGES = 5;
constexpr int MAX_NB = 8;                // at most 8 boxes of 64 columns per stage
constexpr int W_STAGE_BYTES = 32 * 1024; // rows * nb * 128 bytes never exceeds this
constexpr int X_BOX_BYTES = X_ROWS * 128;
constexpr int STAGE_BYTES = W_STAGE_BYTES + MAX_NB * X_BOX_BYTES;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(CONSUMER_WARPS * 32) : "memory"); }
struct alignas(64) Params {
  CUtensorMap x_map;     // x [M, K]: x3d: as [K / 64][M][64], one box is a stage's columns; else box 64 columns x 8 rows
  const unsigned char* slabs;
  void* y;
  long long slab_bytes;  // one block's share
  int M, N, K, ldc, mode;
  int rpb;               // result columns per block
  int nb;                // boxes of 64 columns per stage
  int ks;                // stages over K (K padded to ks * nb * 64 columns in the copy)
  int x3d;               // K is a multiple of 64: a stage's columns of x come in one copy
  // a hint: the copy that the product after this one will read; block c asks its first bytes into L2 as it sends
  // for its own last stage (null: no hint)
  const unsigned char* next_slabs;
  long long next_slab_bytes;
  int next_bytes, next_blocks;
};

__global__ void __launch_bounds__(THREADS, 1) gemm_slab_kernel(const __grid_constant__ Params p) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = smem_unaligned + ((1024 - (smem_u32(smem_unaligned) & 1023)) & 1023);
  unsigned char* ring = smem;
  float* red = reinterpret_cast<float*>(smem + (size_t)STAGES * STAGE_BYTES);       // [4][ROWS][X_ROWS]
  uint64_t* full = reinterpret_cast<uint64_t*>(red + CONSUMER_WARPS * ROWS * X_ROWS);
  uint64_t* empty = full + STAGES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x;
  const int th = p.mode == 2 ? ROWS / 2 : ROWS;                 // result columns of a full sub-tile
  const int n_sub = (p.rpb + th - 1) / th;
  const int mult = p.mode == 2 ? 2 : 1;                         // rows of W per result column
  const int units = n_sub * p.ks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], CONSUMER_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == CONSUMER_WARPS) {
    // ---------------------------------------------------------------- producer (one thread)
    if (lane == 0) {
      const unsigned char* slab = p.slabs + (size_t)c * p.slab_bytes;
      auto issue_w = [&](int i) {
        const int t = i / p.ks, k = i - t * p.ks;
        const int h = min(th, p.rpb - t * th);                  // result columns of this sub-tile
        const int s = i % STAGES;
        unsigned char* dst = ring + (size_t)s * STAGE_BYTES;
        const uint32_t bytes = (uint32_t)h * mult * p.nb * 128;  // the whole stage of this sub-tile: one linear copy
        // the bytes of earlier sub-tiles (all full), then the earlier stages of this one
        const unsigned char* src = slab + ((size_t)t * th * p.ks + (size_t)k * h) * mult * p.nb * 128;
        mbar_expect_tx(&full[s], bytes + p.nb * X_BOX_BYTES);
        bulk_load(dst, src, bytes, &full[s]);
      };
      auto issue_x = [&](int i) {
        const int k = i % p.ks;
        const int s = i % STAGES;
        unsigned char* dst = ring + (size_t)s * STAGE_BYTES + W_STAGE_BYTES;
        // one copy where it can be (a copy costs the TMA unit about as much whatever it holds): the box holds the
        // stage's nb column blocks one after the other, as the separate copies lay them
        if (p.x3d) {
          tma_load_3d(dst, &p.x_map, 0, 0, k * p.nb, &full[s]);
        } else {
          for (int b = 0; b < p.nb; ++b) tma_load_2d(dst + b * X_BOX_BYTES, &p.x_map, (k * p.nb + b) * 64, 0, &full[s]);
        }
      };
      // Fill the ring with weights while the kernel before this one may still be running, then wait for it.
      const int pre = min(STAGES, units);
      for (int i = 0; i < pre; ++i)
        if (NHV_UNIT_IS_SENT(i)) issue_w(i);
      pdl_wait();
      for (int i = 0; i < pre; ++i)
        if (NHV_UNIT_IS_SENT(i)) issue_x(i);
      bool ok = true;
      for (int i = STAGES; i < units; ++i) {
        const int s = i % STAGES;
        ok = mbar_wait(&empty[s], (uint32_t)((i / STAGES) - 1) & 1, 1);
        if (!ok) break;
        if (NHV_UNIT_IS_SENT(i)) {
          issue_w(i);
          issue_x(i);
        }
      }
      if (p.next_slabs && c < p.next_blocks) {
        const unsigned char* nx = p.next_slabs + (size_t)c * p.next_slab_bytes;
        for (int off = 0; off < p.next_bytes; off += 16384) {
          const int n = min(16384, p.next_bytes - off);
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(nx + off), "r"(n) : "memory");
        }
      }
      if (!ok) give_up_delay();
    } else {
      pdl_wait();
    }
  } else {
    // ---------------------------------------------------------------- consumers
    pdl_wait();
    const int tid = threadIdx.x;                                // 0..127
    float acc[MT][4];
    auto clear = [&]() {
#pragma unroll
      for (int i = 0; i < MT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    };
    clear();
    bool ok = true;
    for (int i = 0; i < units && ok; ++i) {
      const int s = i % STAGES;
      const int t = i / p.ks, k = i - t * p.ks;
      ok = mbar_wait(&full[s], (uint32_t)(i / STAGES) & 1, 2);
      if (!ok) { give_up_delay(); break; }
      const unsigned char* stage = ring + (size_t)s * STAGE_BYTES;
      const int h_now = min(th, p.rpb - t * th);
      const int box_stride = h_now * mult * 128;                  // a box holds the sub-tile's rows and nothing else
      // this warp's k-steps of the stage: nb of the 4 * nb, each 16 columns; box = step / 4
      for (int kk = 0; kk < p.nb; ++kk) {
        const int step = warp * p.nb + kk;
        const int box = step >> 2, c0 = (step & 3) * 2;
        const unsigned char* ws = stage + (size_t)box * box_stride;
        const unsigned char* xs = stage + W_STAGE_BYTES + (size_t)box * X_BOX_BYTES;
        uint32_t b[4];
        {
          const int r = lane & 7;
          const int ch = c0 + ((lane >> 3) & 1);
          ldmatrix_x4(b, xs + r * 128 + ((ch ^ (r & 7)) << 4));
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          uint32_t a[4];
          const int r = mt * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          const int ch = c0 + (lane >> 4);
          ldmatrix_x4(a, ws + r * 128 + ((ch ^ (r & 7)) << 4));
          mma_bf16(acc[mt], a, b[0], b[1]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
      if (k != p.ks - 1) continue;
      // ------------------------------------------------------------ end of the sub-tile: add the four warps' sums
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = mt * 16 + (lane >> 2) + ((e >> 1) << 3);
          const int m = ((lane & 3) << 1) + (e & 1);
          red[(warp * ROWS + r) * X_ROWS + m] = acc[mt][e];
        }
      clear();
      consumer_sync();
      const int h = min(th, p.rpb - t * th);
      for (int id = tid; id < h * X_ROWS; id += CONSUMER_WARPS * 32) {
        const int m = id / h, r = id - m * h;
        const int n = c * p.rpb + t * th + r;
        if (m >= p.M || n >= p.N) continue;
        auto value = [&](int row) -> float {
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < CONSUMER_WARPS; ++w) v += red[(w * ROWS + row) * X_ROWS + m];
          return __bfloat162float(__float2bfloat16_rn(v));
        };
        float v = value(r);
        if (p.mode == 2) {
          const float up = value(h + r);                           // the rows of up follow the rows of gate
          v = v / (1.0f + expf(-v)) * up;
        }
        if (p.mode == 1)
          reinterpret_cast<float*>(p.y)[(size_t)m * p.ldc + n] = v;
        else
          reinterpret_cast<bf16*>(p.y)[(size_t)m * p.ldc + n] = __float2bfloat16_rn(v);
      }
      consumer_sync();
    }
  }
}

bool make_x_map(CUtensorMap* map, const void* base, int rows, int cols, int row_stride_elems) {
  return nhv_make_map_bf16(map, base, rows, cols, row_stride_elems, 64, X_ROWS);
}
// x as [cols / 64][rows][64] (cols a multiple of 64): a box of nb column blocks; blocks beyond the last read as zero
bool make_x_map_3d(CUtensorMap* map, const void* base, int rows, int cols, int row_stride_elems, int nb) {
  const long long dims[3] = {64, rows, cols / 64};
  const long long strides[3] = {2, (long long)row_stride_elems * 2, 128};
  const int box[3] = {64, X_ROWS, nb};
  return nhv_make_map_bf16_nd(map, base, 3, dims, strides, box);
}

}  // namespace

// Reads and clears the error word (0: no bounded wait ever ran out).  Synchronises the device.
NHV_API int nhv_gemm_slab_error() { return nhv_wait_error_take(); }
// The device address of the error word, for kernels that report it with the step's result.
NHV_API void* nhv_gemm_slab_error_word() { return nhv_wait_error_address(); }

// The geometry of the copy for a matrix with N result columns (mode 2: N = half the rows of W) and K columns on a
// device with `sms` SMs: blocks, result columns per block, boxes per stage, stages over K, bytes per block.
NHV_API int nhv_gemm_slab_geometry(int N, int K, int mode, int sms, int* blocks, int* rpb, int* nb, int* ks,
                                   long long* slab_bytes) {
  NHV_REQUIRE(N > 0 && K > 0 && sms > 0 && mode >= 0 && mode <= 2, "gemm_slab: bad sizes (N=%d K=%d)", N, K);
  const int g = N < sms ? N : sms;
  const int r = (N + g - 1) / g;
  const int th = mode == 2 ? ROWS / 2 : ROWS;
  const int mult = mode == 2 ? 2 : 1;
  const int tallest = (r < th ? r : th) * mult;                // rows of W in the tallest sub-tile
  int boxes = W_STAGE_BYTES / (tallest * 128);                 // as many boxes as fill a stage
  if (boxes > MAX_NB) boxes = MAX_NB;
  const int k_boxes = (K + 63) / 64;
  if (boxes > k_boxes) boxes = k_boxes;
  if (boxes < 1) boxes = 1;
  *blocks = (N + r - 1) / r;
  *rpb = r;
  *nb = boxes;
  *ks = (k_boxes + boxes - 1) / boxes;
  *slab_bytes = (long long)r * mult * (*ks) * boxes * 128;
  return 0;
}

// slabs: the copy made by ops.slab_weight for exactly this geometry (nhv_gemm_slab_geometry with the same N, K,
// mode and SM count).
static int gemm_slab_launch(void* y, const void* x, const void* slabs, int M, int N, int K, int lda, int ldc, int mode,
                            int sms, const void* next_slabs, long long next_slab_bytes, int next_bytes, int next_blocks,
                            cudaStream_t stream);
NHV_API int nhv_gemm_slab(void* y, const void* x, const void* slabs, int M, int N, int K, int lda, int ldc, int mode,
                          int sms, cudaStream_t stream) {
  return gemm_slab_launch(y, x, slabs, M, N, K, lda, ldc, mode, sms, nullptr, 0, 0, 0, stream);
}
// The same with a hint: the copy (and its geometry: bytes per block, blocks) that the next product will read, of which
// every block asks `next_bytes` into L2 when it has sent for its own last stage.
NHV_API int nhv_gemm_slab_hint(void* y, const void* x, const void* slabs, int M, int N, int K, int lda, int ldc, int mode,
                               int sms, const void* next_slabs, long long next_slab_bytes, int next_bytes, int next_blocks,
                               cudaStream_t stream) {
  return gemm_slab_launch(y, x, slabs, M, N, K, lda, ldc, mode, sms, next_slabs, next_slab_bytes, next_bytes, next_blocks, stream);
}
static int gemm_slab_launch(void* y, const void* x, const void* slabs, int M, int N, int K, int lda, int ldc, int mode,
                            int sms, const void* next_slabs, long long next_slab_bytes, int next_bytes, int next_blocks,
                            cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  NHV_REQUIRE(M > 0 && M <= X_ROWS, "gemm_slab: takes 1 to %d tokens, got %d", X_ROWS, M);
  NHV_REQUIRE(K % 8 == 0 && lda % 8 == 0 && lda >= K && ldc >= N,
              "gemm_slab: K and the row stride of x must be multiples of 8 (N=%d K=%d lda=%d)", N, K, lda);
  NHV_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)slabs % 16) == 0, "gemm_slab: x and the copy of W must be 16-byte aligned");
  Params p;
  int blocks = 0;
  if (int rc = nhv_gemm_slab_geometry(N, K, mode, sms, &blocks, &p.rpb, &p.nb, &p.ks, &p.slab_bytes)) return rc;
  p.slabs = (const unsigned char*)slabs;
  p.y = y;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.mode = mode;
  p.next_slabs = (const unsigned char*)next_slabs;
  p.next_slab_bytes = next_slab_bytes;
  p.next_bytes = next_bytes < next_slab_bytes ? next_bytes / 16 * 16 : (int)(next_slab_bytes / 16 * 16);
  p.next_blocks = next_blocks;
  p.x3d = K % 64 == 0;
  NHV_REQUIRE(p.x3d ? make_x_map_3d(&p.x_map, x, M, K, lda, p.nb) : make_x_map(&p.x_map, x, M, K, lda),
              "gemm_slab: cannot encode the tensor map of x [%d, %d]", M, K);
  constexpr size_t smem = 1024 + (size_t)STAGES * STAGE_BYTES + (size_t)CONSUMER_WARPS * ROWS * X_ROWS * 4 + 2 * STAGES * 8;
  static_assert(smem <= 227 * 1024, "the ring and the reduction buffer must fit one block's shared memory");
  static bool attr_set = false;
  if (!attr_set) {
    NHV_CUDA(cudaFuncSetAttribute(gemm_slab_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "gemm_slab");
    attr_set = true;
  }
  NHV_CUDA(nhv_launch(gemm_slab_kernel, dim3(blocks), dim3(THREADS), smem, stream, p), "gemm_slab");
  return 0;
}
