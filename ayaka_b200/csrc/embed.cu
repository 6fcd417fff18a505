// Embedding: out[i, :] = scale * table[index[i], :] (+ add_table[add_index[i], :]) as fp32 rows of the
// residual stream. One gather for the token table, one for an additive per-row table (GPT-2's
// learned positions), one fp32 add, one store: the sum is never rounded to 16 bits.
#include "common.cuh"

namespace ayk {

template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ index,
                                  int table_rows, const T* __restrict__ add_table,
                                  const int* __restrict__ add_index, int add_rows,
                                  float* __restrict__ out, int ld_out, int width, float scale,
                                  int* __restrict__ bad_index) {
  pdl_launch_dependents();
  pdl_wait_for(index, add_index);  // a graph's ids come from the kernel that advanced them
  const int row = blockIdx.x;
  int id = index[row];
  if (id < 0 || id >= table_rows) {
    if (threadIdx.x == 0) atomicExch(bad_index, 1);
    id = 0;
  }
  const T* src = table + (size_t)id * width;
  const T* add = nullptr;
  if (add_table != nullptr) {
    int a = add_index[row];
    if (a < 0 || a >= add_rows) {
      if (threadIdx.x == 0) atomicExch(bad_index, 1);
      a = 0;
    }
    add = add_table + (size_t)a * width;
  }
  float* dst = out + (size_t)row * ld_out;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = ldf(src + c) * scale;  // (a factor of 1 changes no bit)
    if (add != nullptr) v += ldf(add + c);
    dst[c] = v;
  }
}

template <typename T>
int embed_rows(const void* table, const int* index, int table_rows, const void* add_table,
               const int* add_index, int add_rows, float* out, int ld_out, int rows, int width,
               float scale, int* bad_index, cudaStream_t stream) {
  if (rows == 0) return AYK_OK;
  if (rows < 0 || width < 1 || ld_out < width || table_rows < 1) return AYK_BAD_ARGUMENT;
  if (add_table != nullptr && (add_index == nullptr || add_rows < 1)) return AYK_BAD_ARGUMENT;
  const int threads = width >= 1024 ? 256 : 128;
  return launch_kernel(embed_rows_kernel<T>, dim3(rows), dim3(threads), 0, stream, 1,
                       (const T*)table, index, table_rows, (const T*)add_table, add_index,
                       add_rows, out, ld_out, width, scale, bad_index);
}

}  // namespace ayk

// `scale` multiplies the table's row before the additive row is added (1 for GPT-2; some
// architectures scale their embeddings by sqrt(width)). `bad_index` is one device int, set to 1 when an id falls outside its table (the row then
// uses id 0); the host checks ids before the step, this only makes a slip visible.
AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

AYK_API int ayk_embed_rows_f32(const void* table, const int* index, int table_rows,
                               const void* add_table, const int* add_index, int add_rows,
                               float* out, int ld_out, int rows, int width, float scale,
                               int* bad_index, void* stream) {
  return ayk::embed_rows<float>(table, index, table_rows, add_table, add_index, add_rows, out,
                                ld_out, rows, width, scale, bad_index, (cudaStream_t)stream);
}
AYK_API int ayk_embed_rows_bf16(const void* table, const int* index, int table_rows,
                                const void* add_table, const int* add_index, int add_rows,
                                float* out, int ld_out, int rows, int width, float scale,
                                int* bad_index, void* stream) {
  return ayk::embed_rows<__nv_bfloat16>(table, index, table_rows, add_table, add_index, add_rows,
                                        out, ld_out, rows, width, scale, bad_index,
                                        (cudaStream_t)stream);
}
