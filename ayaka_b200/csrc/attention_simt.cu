// Paged attention on the CUDA cores, fp32 arithmetic throughout, plus the KV store.
//
// Cache layout (one tensor for K, one for V, per layer): [page][kv_head][slot][head_dim].
// Page 0 is padding; a block-table entry of 0 means "no page".
//
// attention: one warp per (query row, head). The row of request b at position p attends keys
// max(0, p - window + 1) .. p of that request, read through its block table in tiles of 32
// keys counted from a multiple of 32: lane j scores key t0 + j (q.k in fp32, times scale), the
// warp keeps a running maximum and sum (online softmax, expf), then the lanes split head_dim
// and add p_j * V[j]. The tiling depends only on the position, so a row's output is the same
// whether it arrives alone, in a prompt portion or beside other requests. It serves prefill,
// decode and mixed batches of the float32 path; in bfloat16 it is the plain reference of the
// tensor-core and split-KV kernels. head_dim: a multiple of 8, at most 256. Any number of
// heads and of KV heads that divides it.
#include "common.cuh"

namespace ayk {

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_HD = 256;

template <typename T> struct Vec8;
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, int ld_q, const T* __restrict__ k_pages,
                      const T* __restrict__ v_pages, const int* __restrict__ block_table,
                      int table_stride, const int* __restrict__ request_of_row,
                      const int* __restrict__ positions, T* __restrict__ out, int ld_out,
                      int num_rows, int num_kv_heads, int group, int head_dim, int page_size,
                      float scale, int window) {
  __shared__ __align__(16) float q_s[ATT_WARPS][ATT_MAX_HD];
  __shared__ float p_s[ATT_WARPS][32];
  __shared__ long long off_s[ATT_WARPS][32];
  pdl_launch_dependents();
  pdl_wait_for(q, k_pages, v_pages);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * ATT_WARPS + warp;
  const int head = blockIdx.y;
  if (row >= num_rows) return;
  const int kv_head = head / group;
  const int req = request_of_row[row];
  T* dst = out + (size_t)row * ld_out + (size_t)head * head_dim;
  if (req < 0) {  // a padding row
    for (int d = lane; d < head_dim; d += 32) stf(dst + d, 0.f);
    return;
  }
  const int pos = positions[row];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const T* qsrc = q + (size_t)row * ld_q + (size_t)head * head_dim;
  for (int d = lane; d < head_dim; d += 32) q_s[warp][d] = ldf(qsrc + d);
  __syncwarp();

  const int* table = block_table + (size_t)req * table_stride;
  float acc[ATT_MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < ATT_MAX_HD / 32; ++i) acc[i] = 0.f;
  float run_max = -INFINITY, run_sum = 0.f;

  for (int t0 = (lo / 32) * 32; t0 <= pos; t0 += 32) {
    const int key = t0 + lane;
    const bool valid = key >= lo && key <= pos;
    float s = -INFINITY;
    long long base = 0;
    if (valid) {
      const int page = table[key / page_size];
      base = (((long long)page * num_kv_heads + kv_head) * page_size + key % page_size) *
             head_dim;
      const T* kp = k_pages + base;
      float dot = 0.f;
      for (int d = 0; d < head_dim; d += 8) {
        float kv[8];
        Vec8<T>::load(kp + d, kv);
#pragma unroll
        for (int e = 0; e < 8; ++e) dot = fmaf(q_s[warp][d + e], kv[e], dot);
      }
      s = dot * scale;
    }
    const float new_max = fmaxf(run_max, warp_max(s));
    const float corr = expf(run_max - new_max);  // exp(-inf) = 0 on the first tile
    const float p = valid ? expf(s - new_max) : 0.f;
    run_sum = run_sum * corr + warp_sum(p);
    run_max = new_max;
    p_s[warp][lane] = p;
    off_s[warp][lane] = base;
    __syncwarp();
    const int j_lo = lo > t0 ? lo - t0 : 0;
    const int j_hi = pos - t0 + 1 < 32 ? pos - t0 + 1 : 32;
#pragma unroll
    for (int i = 0; i < ATT_MAX_HD / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < head_dim) {
        float a = acc[i] * corr;
        for (int j = j_lo; j < j_hi; ++j) {
          a = fmaf(p_s[warp][j], ldf(v_pages + off_s[warp][j] + d), a);
        }
        acc[i] = a;
      }
    }
    __syncwarp();
  }
  const float inv = 1.f / run_sum;
#pragma unroll
  for (int i = 0; i < ATT_MAX_HD / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < head_dim) stf(dst + d, acc[i] * inv);
  }
}

// K and V rows of this step, from the fused projection's output into the pages.
// slot_mapping[row] = page * page_size + slot, or negative for a row that stores nothing.
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ k, const T* __restrict__ v, int ld_kv,
                                const int* __restrict__ slot_mapping, T* __restrict__ k_pages,
                                T* __restrict__ v_pages, int num_kv_heads, int head_dim,
                                int page_size) {
  pdl_launch_dependents();
  pdl_wait_for(k, v);
  const int row = blockIdx.x;
  const int slot = slot_mapping[row];
  if (slot < 0) return;
  const int page = slot / page_size, within = slot % page_size;
  const int width = num_kv_heads * head_dim;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const int h = c / head_dim, d = c % head_dim;
    const size_t dst = (((size_t)page * num_kv_heads + h) * page_size + within) * head_dim + d;
    k_pages[dst] = k[(size_t)row * ld_kv + c];
    v_pages[dst] = v[(size_t)row * ld_kv + c];
  }
}

// The same in 16-byte pieces (8 bfloat16 or 4 float32), for rows and pages that start on 16
// bytes: a piece never straddles two heads because head_dim is a multiple of 8. One CTA per
// row; a thread's key and value pieces are all requested before the first is stored.
template <typename T>
__global__ void __launch_bounds__(256)
kv_store_wide_kernel(const T* __restrict__ k, const T* __restrict__ v, int ld_kv,
                     const int* __restrict__ slot_mapping, T* __restrict__ k_pages,
                     T* __restrict__ v_pages, int num_kv_heads, int head_dim, int page_size) {
  constexpr int EL = 16 / sizeof(T);
  pdl_launch_dependents();
  const int row = blockIdx.x;
  const int slot = slot_mapping[row];  // the step's metadata: not written by the kernel ahead
  pdl_wait_for(k, v);
  if (slot < 0) return;
  const int page = slot / page_size, within = slot % page_size;
  const int pieces = num_kv_heads * head_dim / EL;
  const int per_head = head_dim / EL;
  const uint4* k_row = reinterpret_cast<const uint4*>(k + (size_t)row * ld_kv);
  const uint4* v_row = reinterpret_cast<const uint4*>(v + (size_t)row * ld_kv);
  const size_t base = ((size_t)page * num_kv_heads * page_size + within) * per_head;
  const size_t head_step = (size_t)page_size * per_head;
  uint4* k_dst = reinterpret_cast<uint4*>(k_pages);
  uint4* v_dst = reinterpret_cast<uint4*>(v_pages);
  for (int p0 = threadIdx.x; p0 < pieces; p0 += 2 * 256) {
    const int p1 = p0 + 256;
    const uint4 ka = k_row[p0], va = v_row[p0];
    uint4 kb = ka, vb = va;
    if (p1 < pieces) {
      kb = k_row[p1];
      vb = v_row[p1];
    }
    const size_t d0 = base + (size_t)(p0 / per_head) * head_step + p0 % per_head;
    k_dst[d0] = ka;
    v_dst[d0] = va;
    if (p1 < pieces) {
      const size_t d1 = base + (size_t)(p1 / per_head) * head_step + p1 % per_head;
      k_dst[d1] = kb;
      v_dst[d1] = vb;
    }
  }
}

template <typename T>
int attention_simt(const void* q, int ld_q, const void* k_pages, const void* v_pages,
                   const int* block_table, int table_stride, const int* request_of_row,
                   const int* positions, void* out, int ld_out, int num_rows, int num_heads,
                   int num_kv_heads, int head_dim, int page_size, float scale, int window,
                   cudaStream_t stream) {
  if (num_rows == 0) return AYK_OK;
  if (num_rows < 0 || num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads ||
      page_size < 1 || table_stride < 1 || window < 0) {
    return AYK_BAD_ARGUMENT;
  }
  if (head_dim < 8 || head_dim % 8) return AYK_BAD_ARGUMENT;
  if (head_dim > ATT_MAX_HD || num_heads > 65535) return AYK_TOO_LARGE;
  const size_t vec = 8 * sizeof(T);
  if (((uintptr_t)k_pages % vec) || ((uintptr_t)v_pages % vec)) return AYK_BAD_ALIGNMENT;
  dim3 grid((num_rows + ATT_WARPS - 1) / ATT_WARPS, num_heads);
  return launch_kernel(attention_simt_kernel<T>, grid, dim3(ATT_WARPS * 32), 0, stream, 1,
                       (const T*)q, ld_q, (const T*)k_pages, (const T*)v_pages, block_table,
                       table_stride, request_of_row, positions, (T*)out, ld_out, num_rows,
                       num_kv_heads, num_heads / num_kv_heads, head_dim, page_size, scale,
                       window);
}

template <typename T>
int kv_store(const void* k, const void* v, int ld_kv, const int* slot_mapping, void* k_pages,
             void* v_pages, int num_rows, int num_kv_heads, int head_dim, int page_size,
             cudaStream_t stream) {
  if (num_rows == 0) return AYK_OK;
  if (num_rows < 0 || num_kv_heads < 1 || head_dim < 1 || page_size < 1 ||
      ld_kv < num_kv_heads * head_dim) {
    return AYK_BAD_ARGUMENT;
  }
  const size_t el = 16 / sizeof(T);
  const bool wide = head_dim % 8 == 0 && ((uintptr_t)k % 16) == 0 && ((uintptr_t)v % 16) == 0 &&
                    (size_t)ld_kv % el == 0 && ((uintptr_t)k_pages % 16) == 0 &&
                    ((uintptr_t)v_pages % 16) == 0;
  if (wide) {
    return launch_kernel(kv_store_wide_kernel<T>, dim3(num_rows), dim3(256), 0, stream, 1,
                         (const T*)k, (const T*)v, ld_kv, slot_mapping, (T*)k_pages,
                         (T*)v_pages, num_kv_heads, head_dim, page_size);
  }
  return launch_kernel(kv_store_kernel<T>, dim3(num_rows), dim3(256), 0, stream, 1,
                       (const T*)k, (const T*)v, ld_kv, slot_mapping, (T*)k_pages, (T*)v_pages,
                       num_kv_heads, head_dim, page_size);
}

}  // namespace ayk

using bf16 = __nv_bfloat16;

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

// type: 0 = float32, 1 = bfloat16 (queries, pages and output share it).
AYK_API int ayk_attention_simt(const void* q, int ld_q, const void* k_pages, const void* v_pages,
                               const int* block_table, int table_stride,
                               const int* request_of_row, const int* positions, void* out,
                               int ld_out, int num_rows, int num_heads, int num_kv_heads,
                               int head_dim, int page_size, float scale, int window, int type,
                               void* stream) {
  if (type == 0) {
    return ayk::attention_simt<float>(q, ld_q, k_pages, v_pages, block_table, table_stride,
                                      request_of_row, positions, out, ld_out, num_rows, num_heads,
                                      num_kv_heads, head_dim, page_size, scale, window,
                                      (cudaStream_t)stream);
  }
  if (type == 1) {
    return ayk::attention_simt<bf16>(q, ld_q, k_pages, v_pages, block_table, table_stride,
                                     request_of_row, positions, out, ld_out, num_rows, num_heads,
                                     num_kv_heads, head_dim, page_size, scale, window,
                                     (cudaStream_t)stream);
  }
  return AYK_BAD_ARGUMENT;
}

AYK_API int ayk_kv_store(const void* k, const void* v, int ld_kv, const int* slot_mapping,
                         void* k_pages, void* v_pages, int num_rows, int num_kv_heads,
                         int head_dim, int page_size, int type, void* stream) {
  if (type == 0) {
    return ayk::kv_store<float>(k, v, ld_kv, slot_mapping, k_pages, v_pages, num_rows,
                                num_kv_heads, head_dim, page_size, (cudaStream_t)stream);
  }
  if (type == 1) {
    return ayk::kv_store<bf16>(k, v, ld_kv, slot_mapping, k_pages, v_pages, num_rows,
                               num_kv_heads, head_dim, page_size, (cudaStream_t)stream);
  }
  return AYK_BAD_ARGUMENT;
}
