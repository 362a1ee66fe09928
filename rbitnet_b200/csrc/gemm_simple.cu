// Plain tiled matrix product on the CUDA cores: C[M,N] (+)= alpha * A[M,K] * W[N,K]^T.
//
// This is the true 32-bit path's product (FFMA with float32 accumulation, no
// tensor-core or reduced-precision mode) and the product for shapes that the
// tensor-core kernel refuses.  W is row-major [out, in], the layout the
// reference indexes as w[i + o*n_in] (crates/bitnet-core/src/llama/model.rs:67-91),
// so no weight is transposed at load.  Each output element is one sequential
// float32 sum over k in ascending order, whatever M is: a row's result does not
// depend on which other rows are in the batch.
#include "rb_common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each

template <typename TA, typename TC>
__global__ void __launch_bounds__(256) gemm_simple_kernel(TC* __restrict__ C, int64_t ldc,
                                                         const TA* __restrict__ A, int64_t lda,
                                                         const TA* __restrict__ W, int64_t ldw, int M, int N,
                                                         int K, int accumulate, float alpha) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  __shared__ float As[BK][BM + 1];
  __shared__ float Ws[BK][BN + 1];
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64x16 elements of each operand, 256 threads -> 4 each
    for (int e = threadIdx.x; e < BM * BK; e += 256) {
      const int r = e / BK, c = e % BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? rb_to_float<TA>(A[(int64_t)gm * lda + gk]) : 0.f;
      Ws[c][r] = (gn < N && gk < K) ? rb_to_float<TA>(W[(int64_t)gn * ldw + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      TC* p = C + (int64_t)gm * ldc + gn;
      float v = alpha == 1.0f ? acc[i][j] : acc[i][j] * alpha;
      if (accumulate) v += rb_to_float<TC>(*p);
      *p = rb_from_float<TC>(v);
    }
  }
}

}  // namespace

// a_dtype: dtype of A and W; c_dtype: dtype of C.  accumulate: C += instead of C =.
// alpha multiplies the finished sum (1.0 leaves it as it is).
RB_EXPORT int rb_gemm_simple(void* C, int64_t ldc, int c_dtype, const void* A, int64_t lda, const void* W,
                             int64_t ldw, int a_dtype, int M, int N, int K, int accumulate,
                             float alpha, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  RB_REQUIRE(M > 0 && N > 0 && K > 0, "rb_gemm_simple: bad sizes M=%d N=%d K=%d", M, N, K);
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  RB_REQUIRE(grid.y <= 65535, "rb_gemm_simple: M=%d too large for one launch", M);
#define LAUNCH(TA, TC)                                                                                     \
  RB_LAUNCH("gemm_simple_kernel", (gemm_simple_kernel<TA, TC>), grid, 256, 0, stream, (TC*)C, ldc, (const TA*)A, \
            lda, (const TA*)W, ldw, M, N, K, accumulate, alpha)
  if (a_dtype == RB_F32 && c_dtype == RB_F32) LAUNCH(float, float);
  else if (a_dtype == RB_BF16 && c_dtype == RB_F32) LAUNCH(__nv_bfloat16, float);
  else if (a_dtype == RB_BF16 && c_dtype == RB_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else RB_FAIL("rb_gemm_simple: unsupported dtypes a=%d c=%d", a_dtype, c_dtype);
#undef LAUNCH
  RB_CHECK_LAUNCH("rb_gemm_simple");
  return 0;
}
