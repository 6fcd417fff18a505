// Paged attention for decode rows: one query row per request, keys split over several CTAs.
//
// A decode step reads every cached key and value of every live request once; with one row
// per request there is no reuse, so the kernel is built to keep many bytes in flight.
// grid = (splits, heads, requests). A CTA of 128 threads takes one contiguous share of the
// request's keys and streams it through a ring of shared-memory stages: one thread issues
// bulk asynchronous copies (cp.async.bulk, a page's run of keys of one head is contiguous in
// the cache) that complete on an mbarrier, several chunks ahead of the arithmetic. TPK threads
// cooperate on one key (each holds 8 of head_dim's elements), so a CTA covers 128 / TPK keys
// per pass. Scores, the running maximum and sum (online softmax) and the weighted sum of
// values are fp32. Every wait is bounded and reports through `status`. Each
// CTA leaves (max, sum, weighted values) of its share in scratch memory; the CTA that
// finishes last for a (request, head) — found with an atomic ticket — merges the shares in
// split order and writes the output row. With splits == 1 nothing goes through scratch.
//
// Scratch: partial [requests * heads * splits * (head_dim + 2)] floats and one int ticket
// per (request, head), zero before the first launch and left zero by every launch.
// Cache layout: [page][kv_head][slot][head_dim]; block-table entry 0 = no page.
#include "tc_common.cuh"

namespace ayk {

constexpr int DEC_THREADS = 128;
constexpr int DEC_STAGES = 4;

template <typename T> struct Frag8;
template <> struct Frag8<float> {
  static __device__ __forceinline__ void copy(float* dst, const float* src) {
    *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
    *reinterpret_cast<float4*>(dst + 4) = *reinterpret_cast<const float4*>(src + 4);
  }
  static __device__ __forceinline__ void load_shared(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p + 4));
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};
template <> struct Frag8<__nv_bfloat16> {
  static __device__ __forceinline__ void copy(__nv_bfloat16* dst, const __nv_bfloat16* src) {
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
  }
  static __device__ __forceinline__ void load_shared(const __nv_bfloat16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

// Merge (max, sum, acc[8]) of `other` into the running triple.
__device__ __forceinline__ void merge_state(float& m, float& l, float* acc, float om, float ol,
                                            const float* oacc) {
  const float nm = fmaxf(m, om);
  if (nm == -INFINITY) return;  // both empty
  const float a = expf(m - nm), b = expf(om - nm);
  l = l * a + ol * b;
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = acc[i] * a + oacc[i] * b;
  m = nm;
}

template <typename T, int TPK>
__global__ void __launch_bounds__(DEC_THREADS)
attention_decode_kernel(const T* __restrict__ q, int ld_q, const T* __restrict__ k_pages,
                        const T* __restrict__ v_pages, const int* __restrict__ block_table,
                        int table_stride, const int* __restrict__ request_of_row,
                        const int* __restrict__ positions, T* __restrict__ out, int ld_out,
                        int num_kv_heads, int group, int head_dim, int page_size, float scale,
                        int window, float* __restrict__ partial, int* __restrict__ tickets,
                        const T* __restrict__ k_new, const T* __restrict__ v_new, int ld_new,
                        T* __restrict__ k_store, T* __restrict__ v_store, int chunk_keys,
                        int* __restrict__ status) {
  constexpr int KEYS_PER_PASS = DEC_THREADS / TPK;
  __shared__ float s_m[DEC_THREADS / 32][TPK], s_l[DEC_THREADS / 32][TPK];
  __shared__ float s_acc[DEC_THREADS / 32][TPK][8];
  __shared__ int s_last;
  __shared__ __align__(8) uint64_t s_full[DEC_STAGES];
  extern __shared__ __align__(128) unsigned char dec_smem[];

  pdl_launch_dependents();
  pdl_wait();
  const int split = blockIdx.x, splits = gridDim.x;
  const int head = blockIdx.y, num_heads = gridDim.y;
  const int row = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sub = tid % TPK;        // which 8 elements of head_dim
  const int key_slot = tid / TPK;   // which key of the pass
  const bool dims_ok = sub * 8 < head_dim;
  const int req = request_of_row[row];
  T* dst = out + (size_t)row * ld_out + (size_t)head * head_dim;
  if (req < 0) {  // a padding row: zeros, no scratch, no ticket
    if (split == 0) {
      for (int d = tid; d < head_dim; d += DEC_THREADS) stf(dst + d, 0.f);
    }
    return;
  }
  const int kv_head = head / group;
  const int pos = positions[row];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int total = pos + 1 - lo;
  int share = (total + splits - 1) / splits;
  share = (share + KEYS_PER_PASS - 1) / KEYS_PER_PASS * KEYS_PER_PASS;
  const int k_lo = lo + split * share;
  const int k_hi = k_lo + share < pos + 1 ? k_lo + share : pos + 1;

  float qf[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) qf[i] = 0.f;
  if (dims_ok) {
    float tmp[8];
    Frag8<T>::load(q + (size_t)row * ld_q + (size_t)head * head_dim + sub * 8, tmp);
#pragma unroll
    for (int i = 0; i < 8; ++i) qf[i] = tmp[i] * scale;
  }
  const int* table = block_table + (size_t)req * table_stride;
  float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;

  // ---- the ring of stages: chunk c holds keys k_lo + c * chunk_keys .. of K, then of V -----
  const int stage_elems = chunk_keys * head_dim;  // elements of K (and of V) per stage
  T* ring = reinterpret_cast<T*>(dec_smem);
  const int num_chunks = k_hi > k_lo ? (k_hi - k_lo + chunk_keys - 1) / chunk_keys : 0;
  if (tid == 0) {
    for (int s = 0; s < DEC_STAGES; ++s) mbar_init(&s_full[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  // one thread copies a chunk: runs of keys inside one page are contiguous in the cache
  auto issue = [&](int c) {
    const int stage = c % DEC_STAGES;
    const int c_lo = k_lo + c * chunk_keys;
    const int c_hi = c_lo + chunk_keys < k_hi ? c_lo + chunk_keys : k_hi;
    const uint32_t row_bytes = (uint32_t)head_dim * sizeof(T);
    mbar_expect_tx(&s_full[stage], 2u * (uint32_t)(c_hi - c_lo) * row_bytes);
    T* k_dst = ring + (size_t)stage * 2 * stage_elems;
    T* v_dst = k_dst + stage_elems;
    for (int key = c_lo; key < c_hi;) {
      const int slot = key % page_size;
      int run = page_size - slot;
      if (run > c_hi - key) run = c_hi - key;
      const int page = table[key / page_size];
      const size_t off = (((size_t)page * num_kv_heads + kv_head) * page_size + slot) * head_dim;
      bulk_load(k_dst + (size_t)(key - c_lo) * head_dim, k_pages + off, run * row_bytes,
                &s_full[stage]);
      bulk_load(v_dst + (size_t)(key - c_lo) * head_dim, v_pages + off, run * row_bytes,
                &s_full[stage]);
      key += run;
    }
  };
  int issued = 0;  // chunks whose copies thread 0 has started
  if (tid == 0) {
    for (int c = 0; c < DEC_STAGES - 1 && c < num_chunks; ++c) issue(c);
    issued = num_chunks < DEC_STAGES - 1 ? num_chunks : DEC_STAGES - 1;
  }
  bool gave_up = false;
  int c = 0;
  for (; c < num_chunks; ++c) {
    // the stage of chunk c + STAGES - 1 was read in the last iteration, which ended with a
    // barrier: it is free
    if (tid == 0 && c + DEC_STAGES - 1 < num_chunks) {
      issue(c + DEC_STAGES - 1);
      issued = c + DEC_STAGES;
    }
    const int stage = c % DEC_STAGES;
    const bool landed = mbar_wait(&s_full[stage], (c / DEC_STAGES) & 1);
    if (__syncthreads_or(!landed)) {  // all threads agree, whoever ran out of patience
      gave_up = true;
      break;
    }
    const int c_lo = k_lo + c * chunk_keys;
    const T* k_src = ring + (size_t)stage * 2 * stage_elems;
    const T* v_src = k_src + stage_elems;
    for (int local = key_slot; local < chunk_keys; local += KEYS_PER_PASS) {
      const int key = c_lo + local;
      const bool valid = key < k_hi;
      float kf[8], vf[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) { kf[i] = 0.f; vf[i] = 0.f; }
      if (valid && dims_ok) {
        if (k_new != nullptr && key == pos) {
          // the row's own key and value come straight from this step's projection; the first
          // head of each group also puts them into the cache (the fused KV store)
          const size_t src = (size_t)row * ld_new + (size_t)kv_head * head_dim + sub * 8;
          Frag8<T>::load(k_new + src, kf);
          Frag8<T>::load(v_new + src, vf);
          if (k_store != nullptr && head % group == 0) {
            const int page = table[key / page_size];
            const size_t off = (((size_t)page * num_kv_heads + kv_head) * page_size +
                                key % page_size) * head_dim + sub * 8;
            Frag8<T>::copy(k_store + off, k_new + src);
            Frag8<T>::copy(v_store + off, v_new + src);
          }
        } else {
          Frag8<T>::load_shared(k_src + (size_t)local * head_dim + sub * 8, kf);
          Frag8<T>::load_shared(v_src + (size_t)local * head_dim + sub * 8, vf);
        }
      }
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) s = fmaf(qf[i], kf[i], s);
#pragma unroll
      for (int o = TPK / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (valid) {
        const float nm = fmaxf(m, s);
        const float corr = expf(m - nm);
        const float p = expf(s - nm);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(p, vf[i], acc[i] * corr);
        m = nm;
      }
    }
    __syncthreads();
  }
  if (gave_up) {
    // leave together, after this CTA's copies in flight have landed (bounded), and say so
    if (tid == 0) {
      for (int w = c; w < issued; ++w) mbar_wait(&s_full[w % DEC_STAGES], (w / DEC_STAGES) & 1);
      atomicExch(status, AYK_WAIT_TIMEOUT);
    }
    return;
  }
  // merge the key slots that share `sub`: first inside the warp, then across warps
#pragma unroll
  for (int o = TPK; o < 32; o <<= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float ol = __shfl_xor_sync(0xffffffffu, l, o);
    float oacc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) oacc[i] = __shfl_xor_sync(0xffffffffu, acc[i], o);
    merge_state(m, l, acc, om, ol, oacc);
  }
  if (lane < TPK) {
    s_m[warp][lane] = m;
    s_l[warp][lane] = l;
#pragma unroll
    for (int i = 0; i < 8; ++i) s_acc[warp][lane][i] = acc[i];
  }
  __syncthreads();
  if (tid < TPK) {
    m = s_m[0][tid];
    l = s_l[0][tid];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = s_acc[0][tid][i];
    for (int w = 1; w < DEC_THREADS / 32; ++w) {
      merge_state(m, l, acc, s_m[w][tid], s_l[w][tid], s_acc[w][tid]);
    }
    if (splits == 1) {
      if (sub * 8 < head_dim) {
        const float inv = 1.f / l;
#pragma unroll
        for (int i = 0; i < 8; ++i) stf(dst + tid * 8 + i, acc[i] * inv);
      }
    } else {
      float* mine = partial + ((size_t)(row * num_heads + head) * splits + split) *
                                  (head_dim + 2);
      if (tid == 0) { mine[0] = m; mine[1] = l; }
      if (sub * 8 < head_dim) {
#pragma unroll
        for (int i = 0; i < 8; ++i) mine[2 + tid * 8 + i] = acc[i];
      }
    }
  }
  if (splits == 1) return;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int ticket = atomicAdd(&tickets[row * num_heads + head], 1);
    s_last = ticket == splits - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* shares = partial + (size_t)(row * num_heads + head) * splits * (head_dim + 2);
  float top = -INFINITY;
  for (int s = 0; s < splits; ++s) top = fmaxf(top, shares[s * (head_dim + 2)]);
  float denom = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float sm = shares[s * (head_dim + 2)];
    if (sm != -INFINITY) denom += shares[s * (head_dim + 2) + 1] * expf(sm - top);
  }
  for (int d = tid; d < head_dim; d += DEC_THREADS) {
    float sum = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float sm = shares[s * (head_dim + 2)];
      if (sm != -INFINITY) sum += shares[s * (head_dim + 2) + 2 + d] * expf(sm - top);
    }
    stf(dst + d, sum / denom);
  }
  if (tid == 0) tickets[row * num_heads + head] = 0;  // ready for the next launch
}

template <typename T, int TPK>
int launch_decode(const void* q, int ld_q, const void* k_pages, const void* v_pages,
                  const int* block_table, int table_stride, const int* request_of_row,
                  const int* positions, void* out, int ld_out, int num_rows, int num_heads,
                  int num_kv_heads, int head_dim, int page_size, float scale, int window,
                  int splits, float* partial, int* tickets, const void* k_new,
                  const void* v_new, int ld_new, int store, int* status, cudaStream_t stream) {
  dim3 grid(splits, num_heads, num_rows);
  // keys per stage: 64 while a stage (K and V) stays within 32 KB, never fewer than a pass
  int chunk_keys = 64;
  while (chunk_keys > DEC_THREADS / TPK && (size_t)chunk_keys * head_dim * sizeof(T) * 2 > 32768) {
    chunk_keys >>= 1;
  }
  if (chunk_keys < DEC_THREADS / TPK) chunk_keys = DEC_THREADS / TPK;
  const size_t smem = (size_t)DEC_STAGES * 2 * chunk_keys * head_dim * sizeof(T);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<T, TPK>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 140 * 1024);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_kernel(attention_decode_kernel<T, TPK>, grid, dim3(DEC_THREADS), smem, stream, 1,
                       (const T*)q, ld_q, (const T*)k_pages, (const T*)v_pages, block_table,
                       table_stride, request_of_row, positions, (T*)out, ld_out, num_kv_heads,
                       num_heads / num_kv_heads, head_dim, page_size, scale, window, partial,
                       tickets, (const T*)k_new, (const T*)v_new, ld_new,
                       store ? (T*)const_cast<void*>(k_pages) : (T*)nullptr,
                       store ? (T*)const_cast<void*>(v_pages) : (T*)nullptr, chunk_keys, status);
}

template <typename T>
int attention_decode(const void* q, int ld_q, const void* k_pages, const void* v_pages,
                     const int* block_table, int table_stride, const int* request_of_row,
                     const int* positions, void* out, int ld_out, int num_rows, int num_heads,
                     int num_kv_heads, int head_dim, int page_size, float scale, int window,
                     int splits, float* partial, int* tickets, const void* k_new,
                     const void* v_new, int ld_new, int store, int* status,
                     cudaStream_t stream) {
  if (num_rows == 0) return AYK_OK;
  if (status == nullptr) return AYK_BAD_ARGUMENT;
  if ((k_new == nullptr) != (v_new == nullptr) || (store && k_new == nullptr)) {
    return AYK_BAD_ARGUMENT;
  }
  if (k_new != nullptr && (((uintptr_t)k_new % (8 * sizeof(T))) ||
                           ((uintptr_t)v_new % (8 * sizeof(T))) ||
                           ((size_t)ld_new * sizeof(T)) % (8 * sizeof(T)))) {
    return AYK_BAD_ALIGNMENT;
  }
  if (num_rows < 0 || num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads ||
      page_size < 1 || table_stride < 1 || window < 0 || splits < 1) {
    return AYK_BAD_ARGUMENT;
  }
  if (head_dim < 8 || head_dim % 8) return AYK_BAD_ARGUMENT;
  if (head_dim > 256 || num_heads > 65535 || num_rows > 65535 || splits > 1024) {
    return AYK_TOO_LARGE;
  }
  if (splits > 1 && (partial == nullptr || tickets == nullptr)) return AYK_BAD_ARGUMENT;
  const size_t vec = 8 * sizeof(T);
  if (((uintptr_t)k_pages % vec) || ((uintptr_t)v_pages % vec) || ((uintptr_t)q % vec) ||
      ((size_t)ld_q * sizeof(T)) % vec) {
    return AYK_BAD_ALIGNMENT;
  }
  const int frags = head_dim / 8;
#define AYK_DECODE(TPK)                                                                        \
  return launch_decode<T, TPK>(q, ld_q, k_pages, v_pages, block_table, table_stride,          \
                               request_of_row, positions, out, ld_out, num_rows, num_heads,   \
                               num_kv_heads, head_dim, page_size, scale, window, splits,      \
                               partial, tickets, k_new, v_new, ld_new, store, status,    \
                               stream)
  if (frags <= 2) AYK_DECODE(2);
  if (frags <= 4) AYK_DECODE(4);
  if (frags <= 8) AYK_DECODE(8);
  if (frags <= 16) AYK_DECODE(16);
  AYK_DECODE(32);
#undef AYK_DECODE
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

// type: 0 = float32, 1 = bfloat16. `partial` holds num_rows * num_heads * splits *
// (head_dim + 2) floats and `tickets` num_rows * num_heads zeroed ints (both unused when
// splits == 1). With k_new/v_new ([rows, kv_heads * head_dim], row stride ld_new) each row's
// own key and value are read from there instead of the cache, and with `store` they are also
// written into the row's cache slot (the step's KV store, fused). `status` is one device int
// that a CTA sets to AYK_WAIT_TIMEOUT if a wait on its copies ran out.
AYK_API int ayk_attention_decode(const void* q, int ld_q, const void* k_pages,
                                 const void* v_pages, const int* block_table, int table_stride,
                                 const int* request_of_row, const int* positions, void* out,
                                 int ld_out, int num_rows, int num_heads, int num_kv_heads,
                                 int head_dim, int page_size, float scale, int window,
                                 int splits, float* partial, int* tickets, const void* k_new,
                                 const void* v_new, int ld_new, int store, int* status,
                                 int type, void* stream) {
  if (type == 0) {
    return ayk::attention_decode<float>(q, ld_q, k_pages, v_pages, block_table, table_stride,
                                        request_of_row, positions, out, ld_out, num_rows,
                                        num_heads, num_kv_heads, head_dim, page_size, scale,
                                        window, splits, partial, tickets, k_new, v_new, ld_new,
                                        store, status, (cudaStream_t)stream);
  }
  if (type == 1) {
    return ayk::attention_decode<__nv_bfloat16>(
        q, ld_q, k_pages, v_pages, block_table, table_stride, request_of_row, positions, out,
        ld_out, num_rows, num_heads, num_kv_heads, head_dim, page_size, scale, window, splits,
        partial, tickets, k_new, v_new, ld_new, store, status, (cudaStream_t)stream);
  }
  return AYK_BAD_ARGUMENT;
}
