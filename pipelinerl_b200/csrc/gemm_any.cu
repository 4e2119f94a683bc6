// Shape-agnostic GEMM  C[M,N] = A[M,K] * W[N,K]^T  with fp32 accumulation on the CUDA cores.
//
// The tcgen05 kernels (gemm_tc.cu, gemm_tn.cu) need bf16 operands and K % 8 == 0.  This kernel takes any M, N, K, any
// row strides and fp32 or bf16 operands: it is the GEMM of the true-fp32 serving mode and of layers whose sizes the
// TMA descriptors cannot express (a rank-r bottleneck with r < 8, an odd projection width).  Every output element is
// accumulated by ONE thread over k = 0..K-1 in ascending order with fmaf (in steps of sixteen whose sums are added up), so its value does not depend on M, on the
// position of the row in the batch or on the tile it falls into: a token's logits are bit-identical whether it is
// computed alone, in a chunk or in a mixed batch.
#include "prl_common.cuh"

namespace prl {
namespace {

constexpr int kTile = 64;   // output tile 64 x 64 per CTA of 256 threads, 4 x 4 outputs per thread
constexpr int kStepK = 16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename TA, typename TW>
__global__ void __launch_bounds__(256) gemm_any_kernel(const TA* __restrict__ A, int64_t lda, const TW* __restrict__ W,
                                                       int64_t ldw, int M, int N, int K, float* __restrict__ C,
                                                       int64_t ldc) {
  pdl_wait();   // launched with the programmatic-serialization attribute like the engine's other step kernels; no early
                // trigger: letting the next grid become resident early measured +3 ms on a 4096-token prefill and +-0 on decode
  __shared__ float As[kStepK][kTile + 4];
  __shared__ float Ws[kStepK][kTile + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  // loader: 64 rows x 16 k = 1024 elements per operand, 4 per thread; k fastest so global reads are contiguous
  const int lr = tid / 4;          // 0..63
  const int lk = (tid % 4) * 4;    // 0,4,8,12
  for (int k0 = 0; k0 < K; k0 += kStepK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int m = m0 + lr, n = n0 + lr;
      As[lk + j][lr] = (m < M && k < K) ? to_f32(A[(int64_t)m * lda + k]) : 0.f;
      Ws[lk + j][lr] = (n < N && k < K) ? to_f32(W[(int64_t)n * ldw + k]) : 0.f;
    }
    __syncthreads();
    // two levels: the step's sixteen products are summed on their own, then added to the total, so the rounding error
    // grows with sqrt(16) + sqrt(K / 16) instead of sqrt(K) terms; still one thread, one fixed order per element
    float part[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) part[i][j] = 0.f;
#pragma unroll
    for (int kk = 0; kk < kStepK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tn + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) part[i][j] = fmaf(a[i], w[j], part[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] += part[i][j];
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + tm + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tn + j;
      if (n < N) C[(int64_t)m * ldc + n] = acc[i][j];
    }
  }
}

template <typename TA, typename TW>
int launch_any(const void* A, int64_t lda, const void* W, int64_t ldw, int64_t M, int64_t N, int64_t K, float* C,
               int64_t ldc, cudaStream_t st) {
  dim3 grid((unsigned)((N + kTile - 1) / kTile), (unsigned)((M + kTile - 1) / kTile));
  PRL_CUDA(launch_pdl((gemm_any_kernel<TA, TW>), dim3(grid), dim3(256), (size_t)(0), st, (const TA*)A, lda, (const TW*)W, ldw, (int)M, (int)N, (int)K, C, ldc));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

}  // namespace
}  // namespace prl

using namespace prl;

extern "C" int prl_gemm_any(const void* A, int32_t a_is_f32, int64_t lda, const void* W, int32_t w_is_f32, int64_t ldw,
                            int64_t M, int64_t N, int64_t K, float* C, int64_t ldc, prl_stream_t stream) {
  PRL_CHECK_ARG(A && W && C, "prl_gemm_any: NULL argument");
  PRL_CHECK_ARG(M >= 1 && N >= 1 && K >= 1 && lda >= K && ldw >= K && ldc >= N && M < (1 << 22) && N < (1 << 30),
                "prl_gemm_any: bad shape (M=%lld N=%lld K=%lld lda=%lld ldw=%lld ldc=%lld)", (long long)M, (long long)N,
                (long long)K, (long long)lda, (long long)ldw, (long long)ldc);
  cudaStream_t st = (cudaStream_t)stream;
  if (a_is_f32 && w_is_f32) return launch_any<float, float>(A, lda, W, ldw, M, N, K, C, ldc, st);
  if (a_is_f32) return launch_any<float, __nv_bfloat16>(A, lda, W, ldw, M, N, K, C, ldc, st);
  if (w_is_f32) return launch_any<__nv_bfloat16, float>(A, lda, W, ldw, M, N, K, C, ldc, st);
  return launch_any<__nv_bfloat16, __nv_bfloat16>(A, lda, W, ldw, M, N, K, C, ldc, st);
}

