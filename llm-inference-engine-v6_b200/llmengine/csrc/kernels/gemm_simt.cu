// out[m,n] = sum_k a[m,k] * w[n,k]   (W row-major [N,K], as checkpoints store linear layers)
//
// CUDA-core matrix product with float32 accumulation: the true 32-bit path of the engine, and the
// path that takes every shape (any M, N, K and row strides) in bfloat16 when the tensor-core
// kernel refuses one. Each output element is one chain of fused multiply-adds over k = 0..K-1 in
// ascending order, whatever M is and wherever the element lies in a tile, so a row's result does
// not depend on what else is in the batch. This mirrors the serial dot of the reference's
// matmul_f32 (src/kernels.cpp:33-57); no bias (src/engine.cpp:319-341).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TA* __restrict__ a, const TW* __restrict__ w,
                                                        TO* __restrict__ out, int M, int N, int K,
                                                        long long lda, long long ldw, long long ldo) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  dep_launch();
  dep_wait();
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  // loader mapping: 64 rows x 16 k; thread -> row tid/4, k offset (tid%4)*4 .. +3
  const int lr = tid >> 2, lk = (tid & 3) * 4;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    {
      const int m = m0 + lr;
      const TA* src = a + (size_t)m * lda + k0 + lk;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = 0.f;
        if (m < M && k0 + lk + e < K) v = to_f32(src[e]);
        As[lk + e][lr] = v;
      }
      const int n = n0 + lr;
      const TW* wsrc = w + (size_t)n * ldw + k0 + lk;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = 0.f;
        if (n < N && k0 + lk + e < K) v = to_f32(wsrc[e]);
        Ws[lk + e][lr] = v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[TM], wv[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) av[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) wv[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) out[(size_t)m * ldo + n] = from_f32<TO>(acc[i][j]);
    }
  }
}

template <typename TA, typename TW, typename TO>
int launch(const void* a, const void* w, void* out, int M, int N, int K, long long lda, long long ldw,
           long long ldo, cudaStream_t stream) {
  dim3 grid(ceil_div(N, BN), ceil_div(M, BM));
  launch_kernel(gemm_simt_kernel<TA, TW, TO>, grid, 256, 0, stream, (const TA*)a, (const TW*)w, (TO*)out, M, N, K, lda, ldw, ldo);
  return 0;
}

}  // namespace

// in_dtype: element type of both a and w; out_dtype: element type of out.
extern "C" int llm_gemm_simt(const void* a, const void* w, void* out, int M, int N, int K, long long lda,
                             long long ldw, long long ldo, int in_dtype, int out_dtype, cudaStream_t stream) {
  if (M == 0 || N == 0) return LLM_OK;
  LLM_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
  LLM_REQUIRE(lda >= K && ldw >= K && ldo >= N, "gemm_simt: row strides smaller than the rows");
  LLM_REQUIRE(ceil_div(M, BM) <= 65535, "gemm_simt: M=%d too large", M);
  if (in_dtype == LLM_F32 && out_dtype == LLM_F32)
    launch<float, float, float>(a, w, out, M, N, K, lda, ldw, ldo, stream);
  else if (in_dtype == LLM_BF16 && out_dtype == LLM_BF16)
    launch<bf16, bf16, bf16>(a, w, out, M, N, K, lda, ldw, ldo, stream);
  else if (in_dtype == LLM_BF16 && out_dtype == LLM_F32)
    launch<bf16, bf16, float>(a, w, out, M, N, K, lda, ldw, ldo, stream);
  else
    LLM_REQUIRE(false, "gemm_simt: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
  LLM_CHECK_LAUNCH("gemm_simt");
  return LLM_OK;
}
