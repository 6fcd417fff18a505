// Shared helpers of the sm_100a kernels: element conversion, warp/block reductions,
// the C ABI's status codes. Every entry point is `extern "C" int ayk_*(..., void* stream)`
// and returns 0, a positive cudaError_t from the launch, or a negative refusal code below.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define AYK_OK 0
#define AYK_BAD_ARGUMENT (-1)   // a size or pointer the kernel does not take
#define AYK_BAD_ALIGNMENT (-2)  // a pointer or stride that breaks a vector or TMA rule
#define AYK_TOO_LARGE (-3)      // beyond a stated maximum
#define AYK_DRIVER (-4)         // a driver entry point is missing or failed
#define AYK_NOT_TAKEN (-6)      // this entry point does not serve the case; nothing ran

#define AYK_API extern "C" __attribute__((visibility("default")))

namespace ayk {

template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) {
    return __bfloat162float(*p);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) {
    *p = __float2bfloat16_rn(v);
  }
};

template <typename T> __device__ __forceinline__ float ldf(const T* p) { return Elem<T>::load(p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v) { Elem<T>::store(p, v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// tanh-form and erf-form GELU in fp32 (torch's `gelu(approximate="tanh")` and `gelu`).
__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float inner = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.f + tanhf(inner));
}
__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
}

enum Activation : int { ACT_NONE = 0, ACT_GELU_TANH = 1, ACT_GELU_ERF = 2 };

// The tanh form with the hardware's approximate tanh (one special-function instruction,
// relative error about 2^-11): for results that are rounded to bfloat16 (2^-8) right after.
__device__ __forceinline__ float gelu_tanh_fast(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(k0 * (x + k1 * x * x * x)));
  return 0.5f * x * (1.f + t);
}

__device__ __forceinline__ float activate(float x, int act) {
  if (act == ACT_GELU_TANH) return gelu_tanh(x);
  if (act == ACT_GELU_ERF) return gelu_erf(x);
  return x;
}

// The same for a result that is stored as bfloat16.
__device__ __forceinline__ float activate_to_bf16(float x, int act) {
  if (act == ACT_GELU_TANH) return gelu_tanh_fast(x);
  if (act == ACT_GELU_ERF) return gelu_erf(x);
  return x;
}

// Programmatic dependent launch: a kernel launched with the attribute may start while its
// predecessor in the stream is still running; pdl_wait() blocks until the predecessor has
// finished and its writes are visible, so everything before it (barrier set-up, tensor-memory
// allocation, weight prefetch) overlaps the predecessor's tail. Every kernel launched through
// launch_kernel() calls pdl_wait() (pdl_wait_for() where it then reads through read-only
// pointers) before it touches anything another kernel produces or reads, which keeps the
// chain transitive.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// The wait, with the pointers to what the kernel ahead wrote passed through it. A load through
// a const __restrict__ pointer (or __ldg) promises the compiler that nothing writes that
// memory while the kernel runs, so it may be started above the wait's "memory" clobber, where
// a kernel that begins before its predecessor ends reads what is not written yet (seen: the
// query loads of the tensor-core decode attention, moved up beside its prefetch of old keys,
// gave wrong rows in about one run of three on a two-layer model). An address that is the
// output of a volatile asm statement behind the wait cannot be formed earlier.
template <typename P>
__device__ __forceinline__ void pdl_behind_wait(P& pointer) {  // P: a (restrict) pointer type
  static_assert(sizeof(P) == 8, "pointers only");
  unsigned long long bits = reinterpret_cast<unsigned long long>(pointer);
  asm volatile("" : "+l"(bits)::"memory");
  pointer = reinterpret_cast<P>(bits);
}
template <typename... P>
__device__ __forceinline__ void pdl_wait_for(P&... pointers) {
  pdl_wait();
  (pdl_behind_wait(pointers), ...);
}
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

inline int& pdl_enabled() {
  static int enabled = 1;
  return enabled;
}

template <typename... KArgs, typename... Args>
inline int launch_kernel_dims(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, int cluster_x, int cluster_y, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attrs[2];
  int n = 0;
  if (cluster_x > 1 || cluster_y > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = cluster_x > 1 ? cluster_x : 1;
    attrs[n].val.clusterDim.y = cluster_y > 1 ? cluster_y : 1;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl_enabled()) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  config.attrs = attrs;
  config.numAttrs = n;
  cudaError_t e = cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) return (int)e;
  e = cudaGetLastError();
  return e == cudaSuccess ? AYK_OK : (int)e;
}

// cluster of `cluster_y` CTAs along grid.y (1: no cluster)
template <typename... KArgs, typename... Args>
inline int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                         cudaStream_t stream, int cluster_y, Args... args) {
  return launch_kernel_dims(kernel, grid, block, smem, stream, 1, cluster_y, args...);
}
// cluster of `cluster_x` CTAs along grid.x
template <typename... KArgs, typename... Args>
inline int launch_kernel_x(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                           cudaStream_t stream, int cluster_x, Args... args) {
  return launch_kernel_dims(kernel, grid, block, smem, stream, cluster_x, 1, args...);
}

// Streaming multiprocessors of the current device (asked once). Grid sizes and tile choices
// are multiples of this, never a number of one GPU model; if the query fails the answer is
// 1, which only makes the choices conservative.
inline int sm_count() {
  static int count = 0;
  if (count == 0) {
    int device = 0, found = 0;
    if (cudaGetDevice(&device) == cudaSuccess &&
        cudaDeviceGetAttribute(&found, cudaDevAttrMultiProcessorCount, device) == cudaSuccess &&
        found > 0) {
      count = found;
    } else {
      return 1;
    }
  }
  return count;
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? AYK_OK : (int)e;
}

}  // namespace ayk
