// y[M,N] = x[M,K] * W[N,K]^T in bfloat16 for a handful of tokens (M <= 16): the decode step's
// projections.  The work is reading W once at the speed of HBM; the tokens ride along.
//
// A block owns ROWS weight rows (16 or 32) and the whole K: it streams its rows through a ring
// of cp.async stages (256 columns each) next to the matching columns of x, the 4 warps take a
// quarter of every stage each (mma.sync.m16n8k16, W rows on the M axis of the MMA, tokens on
// its N axis, fp32 accumulation) and add their partial sums through shared memory in a fixed
// order at the end, so a result does not depend on the grid.  W is [out, in] row-major as in
// nanovllm/layers/linear.py:40,66.
//
// Variants: plain; fp32 output (logits: rounded to bfloat16 first, then widened, as
// nanovllm/layers/embed_head.py:61 with nanovllm/layers/sampler.py:12 gives them); and the
// feed-forward's first half fused with its activation: the block takes rows n of the gate matrix
// and the same rows of the up matrix and writes silu(gate) * up (nanovllm/layers/activation.py:9-11),
// each product rounded to bfloat16 first as the unfused pair of ops would.
#include "nhv_common.cuh"

namespace {

typedef __nv_bfloat16 bf16;
constexpr int BK = 256;             // columns per stage
constexpr int CH = BK / 8;          // 16-byte chunks per row per stage
constexpr int ROW_CH = CH + 1;      // padded row stride (odd: ldmatrix without bank conflicts)
constexpr int THREADS = 128;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// MT: 16-row tiles of W per block (1 or 2).  NT: 8-token tiles (1 or 2).  STAGES: ring depth.
// MODE 0: y bf16; 1: y fp32 (rounded through bf16); 2: y = silu(gate) * up, tile 0 = gate rows, tile 1 = up rows.
template <int MT, int NT, int STAGES, int MODE>
__global__ void __launch_bounds__(THREADS) gemm_small_m_kernel(void* __restrict__ y, const bf16* __restrict__ x,
                                                               const bf16* __restrict__ W, int M, int N, int K,
                                                               int lda, int ldc, int up_row_offset) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_prologue();
  constexpr int W_ROWS = MT * 16, X_ROWS = NT * 8;
  constexpr int STAGE_ELEMS = (W_ROWS + X_ROWS) * ROW_CH * 8;
  bf16* ring = reinterpret_cast<bf16*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // MODE 2: N counts activation columns; tile 0 reads rows n0.., tile 1 rows up_row_offset + n0..
  const int n0 = blockIdx.x * (MODE == 2 ? 16 : W_ROWS);
  const int n_rows_valid = min(MODE == 2 ? 16 : W_ROWS, N - n0);

  auto load_stage = [&](int stage, int k0) {
    bf16* ws = ring + stage * STAGE_ELEMS;
    bf16* xs = ws + W_ROWS * ROW_CH * 8;
    for (int id = threadIdx.x; id < W_ROWS * CH; id += THREADS) {
      const int r = id / CH, c = id - r * CH;
      const int k = k0 + c * 8;
      int row;
      bool ok;
      if (MODE == 2) {
        const int rr = r & 15;
        row = (r < 16 ? 0 : up_row_offset) + n0 + rr;
        ok = rr < n_rows_valid && k < K;
      } else {
        row = n0 + r;
        ok = r < n_rows_valid && k < K;
      }
      cp_async16(ws + (r * ROW_CH + c) * 8, ok ? W + (size_t)row * K + k : W, ok);
    }
    for (int id = threadIdx.x; id < X_ROWS * CH; id += THREADS) {
      const int r = id / CH, c = id - r * CH;
      const int k = k0 + c * 8;
      const bool ok = r < M && k < K;
      cp_async16(xs + (r * ROW_CH + c) * 8, ok ? x + (size_t)r * lda + k : x, ok);
    }
  };

  float acc[MT][NT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

  const int n_k = (K + BK - 1) / BK;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_k) load_stage(s, s * BK);
    cp_async_commit();
  }
  for (int it = 0; it < n_k; ++it) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    const int nxt = it + STAGES - 1;
    if (nxt < n_k) load_stage(nxt % STAGES, nxt * BK);
    cp_async_commit();
    const bf16* ws = ring + (it % STAGES) * STAGE_ELEMS;
    const bf16* xs = ws + W_ROWS * ROW_CH * 8;
    // this warp's quarter of the stage: columns [warp * 64, warp * 64 + 64) = chunks warp*8 .. +7
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const int c0 = warp * 8 + kk * 2;
      uint32_t a[MT][4];
#pragma unroll
      for (int i = 0; i < MT; ++i)
        ldmatrix_x4(a[i], ws + ((i * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * ROW_CH + c0 + (lane >> 4)) * 8);
      if (NT == 1) {
        // one token tile: lanes 0-15 address (tokens, chunk c0) and (tokens, chunk c0 + 1)
        uint32_t b[4];
        ldmatrix_x4(b, xs + (((lane & 7)) * ROW_CH + c0 + ((lane >> 3) & 1)) * 8);
#pragma unroll
        for (int i = 0; i < MT; ++i) mma_bf16(acc[i][0], a[i], b[0], b[1]);
      } else {
        uint32_t b[4];   // (tokens 0-7, c0), (tokens 0-7, c0+1), (tokens 8-15, c0), (tokens 8-15, c0+1)
        ldmatrix_x4(b, xs + (((lane & 7) + ((lane >> 4) << 3)) * ROW_CH + c0 + ((lane >> 3) & 1)) * 8);
#pragma unroll
        for (int i = 0; i < MT; ++i) {
          mma_bf16(acc[i][0], a[i], b[0], b[1]);
          mma_bf16(acc[i][NT - 1], a[i], b[2], b[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  // add the 4 warps' partial sums in warp order
  float* red = reinterpret_cast<float*>(smem_raw);       // [4][W_ROWS][X_ROWS]
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = i * 16 + (lane >> 2) + ((e >> 1) << 3);
        const int m = j * 8 + ((lane & 3) << 1) + (e & 1);
        red[(warp * W_ROWS + r) * X_ROWS + m] = acc[i][j][e];
      }
  __syncthreads();
  constexpr int OUT_ROWS = MODE == 2 ? 16 : W_ROWS;
  for (int id = threadIdx.x; id < OUT_ROWS * X_ROWS; id += THREADS) {
    const int m = id / OUT_ROWS, r = id - m * OUT_ROWS;   // consecutive threads: consecutive output columns
    if (m >= M || r >= n_rows_valid) continue;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) v += red[(w * W_ROWS + r) * X_ROWS + m];
    v = __bfloat162float(__float2bfloat16_rn(v));
    if (MODE == 2) {
      float u = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) u += red[(w * W_ROWS + 16 + r) * X_ROWS + m];
      u = __bfloat162float(__float2bfloat16_rn(u));
      v = v / (1.0f + expf(-v)) * u;
    }
    if (MODE == 1)
      reinterpret_cast<float*>(y)[(size_t)m * ldc + n0 + r] = v;
    else
      reinterpret_cast<bf16*>(y)[(size_t)m * ldc + n0 + r] = __float2bfloat16_rn(v);
  }
}

template <int MT, int NT, int STAGES, int MODE>
int launch(void* y, const bf16* x, const bf16* W, int M, int N, int K, int lda, int ldc, int up_row_offset,
           cudaStream_t stream) {
  constexpr int W_ROWS = MT * 16, X_ROWS = NT * 8;
  constexpr size_t ring = (size_t)STAGES * (W_ROWS + X_ROWS) * ROW_CH * 16;
  constexpr size_t red = (size_t)4 * W_ROWS * X_ROWS * 4;
  constexpr size_t smem = ring > red ? ring : red;
  static bool attr_set = false;
  if (!attr_set) {
    NHV_CUDA(cudaFuncSetAttribute(gemm_small_m_kernel<MT, NT, STAGES, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)smem), "gemm_small_m");
    attr_set = true;
  }
  const int rows_per_block = MODE == 2 ? 16 : W_ROWS;
  const int blocks = (N + rows_per_block - 1) / rows_per_block;
  nhv_launch(gemm_small_m_kernel<MT, NT, STAGES, MODE>, blocks, THREADS, smem, stream, y, x, W, M, N, K, lda, ldc,
             up_row_offset);
  NHV_CHECK_LAUNCH("gemm_small_m");
  return 0;
}

}  // namespace

// mode 0: y bf16 [M,N]; 1: y fp32 [M,N]; 2: W holds gate rows [0,N) and up rows [up_row_offset, up_row_offset+N),
// y bf16 [M,N] = silu(x Wg^T) * (x Wu^T).
NHV_API int nhv_gemm_small_m(void* y, const void* x, const void* W, int M, int N, int K, int lda, int ldc, int mode,
                             int up_row_offset, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  NHV_REQUIRE(M > 0 && M <= 16, "gemm_small_m: takes 1 to 16 tokens, got %d", M);
  NHV_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0 && lda >= K && ldc >= N,
              "gemm_small_m: K and the row stride of x must be multiples of 8 (N=%d K=%d lda=%d)", N, K, lda);
  NHV_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)W % 16) == 0, "gemm_small_m: x and W must be 16-byte aligned");
  const bf16* xb = (const bf16*)x;
  const bf16* wb = (const bf16*)W;
  const bool wide = N >= 16384;     // enough blocks either way: 32 rows per block halve the re-reads of x
  if (mode == 2) {
    return M <= 8 ? launch<2, 1, 3, 2>(y, xb, wb, M, N, K, lda, ldc, up_row_offset, stream)
                  : launch<2, 2, 3, 2>(y, xb, wb, M, N, K, lda, ldc, up_row_offset, stream);
  }
  if (mode == 1) {
    return M <= 8 ? launch<2, 1, 3, 1>(y, xb, wb, M, N, K, lda, ldc, 0, stream)
                  : launch<2, 2, 3, 1>(y, xb, wb, M, N, K, lda, ldc, 0, stream);
  }
  NHV_REQUIRE(mode == 0, "gemm_small_m: unknown mode %d", mode);
  if (wide)
    return M <= 8 ? launch<2, 1, 3, 0>(y, xb, wb, M, N, K, lda, ldc, 0, stream)
                  : launch<2, 2, 3, 0>(y, xb, wb, M, N, K, lda, ldc, 0, stream);
  return M <= 8 ? launch<1, 1, 5, 0>(y, xb, wb, M, N, K, lda, ldc, 0, stream)
                : launch<1, 2, 4, 0>(y, xb, wb, M, N, K, lda, ldc, 0, stream);
}
