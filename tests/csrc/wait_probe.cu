// Test-only kernel: one thread waits on an mbarrier that nothing ever arrives at, with the
// same bounded wait the engine's tensor-core kernels use (tc_common.cuh), compiled with a
// limit of a few milliseconds (-DAYK_WAIT_NS=...). The wait runs out, the thread writes
// AYK_WAIT_TIMEOUT to the status word exactly as those kernels do, and the kernel returns
// normally: no trap, no fault, no copy in flight, nothing left spinning.
#include "tc_common.cuh"

namespace {

__global__ void wait_probe_kernel(int* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    ayk::mbar_init(&bar, 1);
    ayk::mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0 && !ayk::mbar_wait(&bar, 0)) atomicExch(status, AYK_WAIT_TIMEOUT);
}

}  // namespace

AYK_API int ayk_wait_probe(int* status, void* stream) {
  if (status == nullptr) return AYK_BAD_ARGUMENT;
  wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status);
  return ayk::launch_status();
}
