// C[M,N] = A[M,K] * W[N,K]^T (+ bias, activation, residual) on the CUDA cores with fp32 FMA.
//
// This is the true 32-bit matrix product of the float32 path (tensor cores have no fp32 x fp32
// mode) and the plain on-device reference of the tensor-core kernel in bfloat16. Every output
// element is accumulated over k = 0..K-1 in that order in one fp32 register, whatever M, N or
// the tile it falls in, so a row's result does not depend on what else is in the batch.
// Any M, N, K and leading dimensions; no alignment rule.
#include "common.cuh"

namespace ayk {

constexpr int BM = 64, BN = 64, BK = 16;

// MODE 0: out[m,n] = act(acc + bias[n]) stored as TOut.   MODE 1: out(fp32)[m,n] += acc + bias[n].
template <typename TA, typename TW, typename TOut, int MODE>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ a, int lda, const TW* __restrict__ w, int ldw,
                 const float* __restrict__ bias, TOut* __restrict__ out, int ldo, int M, int N,
                 int K, int act) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  pdl_launch_dependents();
  pdl_wait_for(a);
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int ty = tid >> 4, tx = tid & 15;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    {
      const int m = m0 + lrow;
      const TA* src = a + (size_t)m * lda + k0 + lk;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        As[lk + i][lrow] = (m < M && k0 + lk + i < K) ? ldf(src + i) : 0.f;
      }
      const int n = n0 + lrow;
      const TW* wsrc = w + (size_t)n * ldw + k0 + lk;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        Ws[lk + i][lrow] = (n < N && k0 + lk + i < K) ? ldf(wsrc + i) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
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
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias != nullptr) v += bias[n];
      TOut* dst = out + (size_t)m * ldo + n;
      if (MODE == 1) {
        stf(dst, ldf(dst) + v);
      } else {
        stf(dst, activate(v, act));
      }
    }
  }
}

template <typename TA, typename TW, typename TOut, int MODE>
int gemm_simt(const void* a, int lda, const void* w, int ldw, const float* bias, void* out,
              int ldo, int M, int N, int K, int act, cudaStream_t stream) {
  if (M == 0 || N == 0) return AYK_OK;
  if (M < 0 || N < 0 || K < 1 || lda < K || ldw < K || ldo < N) return AYK_BAD_ARGUMENT;
  if (act < ACT_NONE || act > ACT_GELU_ERF) return AYK_BAD_ARGUMENT;
  const long long gy = (M + BM - 1) / BM;
  if (gy > 65535) return AYK_TOO_LARGE;
  dim3 grid((N + BN - 1) / BN, (unsigned)gy);
  return launch_kernel(gemm_simt_kernel<TA, TW, TOut, MODE>, grid, dim3(256), 0, stream, 1,
                       (const TA*)a, lda, (const TW*)w, ldw, bias, (TOut*)out, ldo, M, N, K, act);
}

}  // namespace ayk

using bf16 = __nv_bfloat16;

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

// in_type / out_type: 0 = float32, 1 = bfloat16. `residual` != 0: out is fp32 and is added to.
AYK_API int ayk_gemm_simt(const void* a, int lda, const void* w, int ldw, const float* bias,
                          void* out, int ldo, int M, int N, int K, int act, int residual,
                          int in_type, int out_type, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (residual) {
    if (out_type != 0 || act != ayk::ACT_NONE) return AYK_BAD_ARGUMENT;
    if (in_type == 0) {
      return ayk::gemm_simt<float, float, float, 1>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, s);
    }
    return ayk::gemm_simt<bf16, bf16, float, 1>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, s);
  }
  if (in_type == 0 && out_type == 0) {
    return ayk::gemm_simt<float, float, float, 0>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, s);
  }
  if (in_type == 1 && out_type == 1) {
    return ayk::gemm_simt<bf16, bf16, bf16, 0>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, s);
  }
  if (in_type == 1 && out_type == 0) {
    return ayk::gemm_simt<bf16, bf16, float, 0>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, s);
  }
  return AYK_BAD_ARGUMENT;
}
