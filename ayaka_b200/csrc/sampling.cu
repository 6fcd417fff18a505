// Token choice from fp32 logits [rows, vocab] (row stride ld, any vocab).
//
// argmax: the largest logit, the smallest id among equals; NaN never wins.
#include "common.cuh"

namespace ayk {

__global__ void __launch_bounds__(256)
argmax_kernel(const float* __restrict__ logits, int ld, int vocab, int* __restrict__ out) {
  __shared__ float best_v[8];
  __shared__ int best_i[8];
  const float* row = logits + (size_t)blockIdx.x * ld;
  float bv = -INFINITY;
  int bi = vocab;
  for (int c = threadIdx.x; c < vocab; c += blockDim.x) {
    const float v = row[c];
    if (v > bv || (v == bv && c < bi)) { bv = v; bi = c; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) {
      if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
    }
    out[blockIdx.x] = bi < vocab ? bi : 0;
  }
}

}  // namespace ayk

AYK_API int ayk_argmax(const float* logits, int ld, int rows, int vocab, int* out, void* stream) {
  if (rows == 0) return AYK_OK;
  if (rows < 0 || vocab < 1 || ld < vocab) return AYK_BAD_ARGUMENT;
  ayk::argmax_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>(logits, ld, vocab, out);
  return ayk::launch_status();
}
