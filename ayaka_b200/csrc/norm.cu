// LayerNorm over fp32 rows of the residual stream: mean, then the biased variance about that
// mean, then (x - mean) * rsqrt(var + eps) * gamma + beta, all in fp32, rounded once to the
// output type. `rows` may gather: output row i normalises input row rows[i] (the final norm
// runs only on the rows whose logits are wanted). Any width.
#include "common.cuh"

namespace ayk {

template <typename TOut>
__global__ void layer_norm_kernel(const float* __restrict__ x, int ld_x,
                                  const int* __restrict__ rows, const float* __restrict__ gamma,
                                  const float* __restrict__ beta, float eps,
                                  TOut* __restrict__ out, int ld_out, int width) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const float* src = x + (size_t)(rows != nullptr ? rows[r] : r) * ld_x;
  float s = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) s += src[c];
  const float mean = block_sum(s, scratch) / (float)width;
  float q = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float dlt = src[c] - mean;
    q += dlt * dlt;
  }
  const float var = block_sum(q, scratch) / (float)width;
  const float inv = rsqrtf(var + eps);
  TOut* dst = out + (size_t)r * ld_out;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = (src[c] - mean) * inv * gamma[c];
    if (beta != nullptr) v += beta[c];
    stf(dst + c, v);
  }
}

template <typename TOut>
int layer_norm(const float* x, int ld_x, const int* rows, const float* gamma, const float* beta,
               float eps, void* out, int ld_out, int n, int width, cudaStream_t stream) {
  if (n == 0) return AYK_OK;
  if (n < 0 || width < 1 || ld_x < width || ld_out < width || !(eps > 0.f)) {
    return AYK_BAD_ARGUMENT;
  }
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  return launch_kernel(layer_norm_kernel<TOut>, dim3(n), dim3(threads), 0, stream, 1, x, ld_x,
                       rows, gamma, beta, eps, (TOut*)out, ld_out, width);
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

AYK_API int ayk_layer_norm_f32(const float* x, int ld_x, const int* rows, const float* gamma,
                               const float* beta, float eps, void* out, int ld_out, int n,
                               int width, void* stream) {
  return ayk::layer_norm<float>(x, ld_x, rows, gamma, beta, eps, out, ld_out, n, width,
                                (cudaStream_t)stream);
}
AYK_API int ayk_layer_norm_bf16(const float* x, int ld_x, const int* rows, const float* gamma,
                                const float* beta, float eps, void* out, int ld_out, int n,
                                int width, void* stream) {
  return ayk::layer_norm<__nv_bfloat16>(x, ld_x, rows, gamma, beta, eps, out, ld_out, n, width,
                                        (cudaStream_t)stream);
}
