// C[M,N] = A[M,K] * W[N,K]^T on the CUDA cores with fp32 multiply-add: the matrix
// product of the true 32-bit path (no TF32 or other reduced-precision matrix mode), also
// usable with bf16 storage.  W is row-major [out, in] as in nanovllm/layers/linear.py:40,66.
//
// Each output element is one accumulator that adds its K products in ascending k, so the
// value of C[m,n] does not depend on M, on the tile that holds it or on the batch.
#include "nhv_common.cuh"

constexpr int GM = 64, GN = 64, GK = 16;

template <typename T, typename TO>
__global__ void __launch_bounds__(256) gemm_nt_simt_kernel(TO* __restrict__ C, const T* __restrict__ A,
                                                           const T* __restrict__ W, int M, int N, int K, int lda,
                                                           int ldw, int ldc) {
  __shared__ __align__(16) float As[GK][GM + 4];
  __shared__ __align__(16) float Ws[GK][GN + 4];
  pdl_prologue();
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4 x 4 outputs each
  const int m0 = blockIdx.y * GM, n0 = blockIdx.x * GN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += GK) {
    // 64 rows x 16 k per operand = 1024 elements, 4 per thread; consecutive threads read along k.
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = threadIdx.x + i * 256;
      const int r = e >> 4, kk = e & 15;
      const int k = k0 + kk;
      float a = 0.f, w = 0.f;
      if (k < K) {
        if (m0 + r < M) a = to_f32<T>(A[(size_t)(m0 + r) * lda + k]);
        if (n0 + r < N) w = to_f32<T>(W[(size_t)(n0 + r) * ldw + k]);
      }
      As[kk][r] = a;
      Ws[kk][r] = w;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 wv = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
      const float a[4] = {av.x, av.y, av.z, av.w};
      const float w[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = from_f32<TO>(acc[i][j]);
    }
  }
}

// out_f32 != 0: C is fp32 whatever the storage type of A and W (logits).
NHV_API int nhv_gemm_nt_simt(int dtype, void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw,
                             int ldc, int out_f32, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  NHV_REQUIRE(M > 0 && N > 0 && K > 0 && lda >= K && ldw >= K && ldc >= N, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
  dim3 grid((N + GN - 1) / GN, (M + GM - 1) / GM);
  NHV_REQUIRE(grid.y <= 65535, "gemm: M=%d is beyond the grid's reach", M);
  if (dtype == NHV_F32)
    nhv_launch(gemm_nt_simt_kernel<float, float>, grid, 256, 0, stream, (float*)C, (const float*)A, (const float*)W, M, N,
               K, lda, ldw, ldc);
  else if (dtype == NHV_BF16 && out_f32)
    nhv_launch(gemm_nt_simt_kernel<__nv_bfloat16, float>, grid, 256, 0, stream, (float*)C, (const __nv_bfloat16*)A,
               (const __nv_bfloat16*)W, M, N, K, lda, ldw, ldc);
  else if (dtype == NHV_BF16)
    nhv_launch(gemm_nt_simt_kernel<__nv_bfloat16, __nv_bfloat16>, grid, 256, 0, stream, (__nv_bfloat16*)C,
               (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, M, N, K, lda, ldw, ldc);
  else
    NHV_REQUIRE(false, "gemm: unknown dtype %d", dtype);
  NHV_CHECK_LAUNCH("gemm_nt_simt");
  return 0;
}
