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
  pdl_wait_for(x);
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

// four consecutive outputs as one store (the address is a multiple of 4 elements)
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 packed;
  packed.x = *reinterpret_cast<uint32_t*>(&lo);
  packed.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = packed;
}

// The same with the row held in registers: one pass over global memory (all loads in flight
// at once), mean and variance from the registers. For rows of at most THREADS * 4 * VEC floats
// whose addresses allow 16-byte loads.
template <typename TOut, int VEC, int THREADS>
__global__ void __launch_bounds__(THREADS)
layer_norm_held_kernel(const float* __restrict__ x, int ld_x, const int* __restrict__ rows,
                       const float* __restrict__ gamma, const float* __restrict__ beta,
                       float eps, TOut* __restrict__ out, int ld_out, int width,
                       int wide_out) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  // the norm's weights (and the gather index, part of the step's metadata) do not depend on
  // the kernel ahead: they are fetched before the wait, the rows after it
  const int r = blockIdx.x;
  const int row = rows != nullptr ? rows[r] : r;
  float4 g[VEC], b[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = (i * THREADS + threadIdx.x) * 4;
    g[i] = b[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < width) {
      g[i] = __ldg(reinterpret_cast<const float4*>(gamma + c));
      if (beta != nullptr) b[i] = __ldg(reinterpret_cast<const float4*>(beta + c));
    }
  }
  pdl_wait_for(x);
  const float* src = x + (size_t)row * ld_x;
  float4 held[VEC];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = (i * THREADS + threadIdx.x) * 4;
    held[i] = c < width ? *reinterpret_cast<const float4*>(src + c)
                        : make_float4(0.f, 0.f, 0.f, 0.f);
    s += (held[i].x + held[i].y) + (held[i].z + held[i].w);
  }
  const float mean = block_sum(s, scratch) / (float)width;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    if ((i * THREADS + threadIdx.x) * 4 < width) {
      const float a = held[i].x - mean, bb = held[i].y - mean;
      const float c = held[i].z - mean, d = held[i].w - mean;
      q += (a * a + bb * bb) + (c * c + d * d);
    }
  }
  const float inv = rsqrtf(block_sum(q, scratch) / (float)width + eps);
  TOut* dst = out + (size_t)r * ld_out;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = (i * THREADS + threadIdx.x) * 4;
    if (c < width) {
      const float v0 = (held[i].x - mean) * inv * g[i].x + b[i].x;
      const float v1 = (held[i].y - mean) * inv * g[i].y + b[i].y;
      const float v2 = (held[i].z - mean) * inv * g[i].z + b[i].z;
      const float v3 = (held[i].w - mean) * inv * g[i].w + b[i].w;
      if (wide_out) {
        store4(dst + c, v0, v1, v2, v3);
      } else {
        stf(dst + c, v0); stf(dst + c + 1, v1); stf(dst + c + 2, v2); stf(dst + c + 3, v3);
      }
    }
  }
}

template <typename TOut>
int layer_norm(const float* x, int ld_x, const int* rows, const float* gamma, const float* beta,
               float eps, void* out, int ld_out, int n, int width, cudaStream_t stream) {
  if (n == 0) return AYK_OK;
  if (n < 0 || width < 1 || ld_x < width || ld_out < width || !(eps > 0.f)) {
    return AYK_BAD_ARGUMENT;
  }
  const bool vector_ok = width % 4 == 0 && ld_x % 4 == 0 && ((uintptr_t)x % 16) == 0 &&
                         ((uintptr_t)gamma % 16) == 0 && ((uintptr_t)beta % 16) == 0;
  // whole groups of four outputs can be stored at once when the rows start on such groups
  const int wide_out = (ld_out % 4 == 0 && ((uintptr_t)out % (4 * sizeof(TOut))) == 0) ? 1 : 0;
  if (vector_ok && width <= 8192 && width >= 256) {
#define AYK_LN_HELD(VEC, THREADS)                                                              \
  return launch_kernel(layer_norm_held_kernel<TOut, VEC, THREADS>, dim3(n), dim3(THREADS), 0,  \
                       stream, 1, x, ld_x, rows, gamma, beta, eps, (TOut*)out, ld_out, width,  \
                       wide_out)
    // with many rows, CTAs of 128 threads (more of them resident per SM) hide the one memory
    // round trip of a row better; with few rows the wider CTA has the shorter chain
    if (n >= 512 && width <= 2048) AYK_LN_HELD(4, 128);
    if (width <= 1024) AYK_LN_HELD(1, 256);
    if (width <= 2048) AYK_LN_HELD(2, 256);
    if (width <= 4096) AYK_LN_HELD(4, 256);
    AYK_LN_HELD(8, 256);
#undef AYK_LN_HELD
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
