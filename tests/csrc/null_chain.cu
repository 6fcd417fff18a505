// Test-only kernels: a chain of kernels that do nothing but wait for their predecessor and
// release their successor (programmatic dependent launch as every kernel of the engine uses
// it), to measure what a kernel boundary itself costs inside a CUDA graph.
#include "common.cuh"
namespace {
__global__ void null_kernel(int* sink) {
  ayk::pdl_launch_dependents();
  ayk::pdl_wait();
  if (sink != nullptr && threadIdx.x == 0 && blockIdx.x == 0) sink[0] += 1;
}
__global__ void null_kernel_late(int* sink) {
  ayk::pdl_wait();
  if (sink != nullptr && threadIdx.x == 0 && blockIdx.x == 0) sink[0] += 1;
  ayk::pdl_launch_dependents();
}
}
AYK_API int null_chain(int n, int blocks, int threads, int* sink, int late, void* stream) {
  for (int i = 0; i < n; ++i) {
    int r = late ? ayk::launch_kernel(null_kernel_late, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, 1, sink)
                 : ayk::launch_kernel(null_kernel, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, 1, sink);
    if (r != 0) return r;
  }
  return 0;
}
AYK_API void set_pdl(int on) { ayk::pdl_enabled() = on; }
