// Causal attention for prompt portions in bfloat16 on the tensor cores, over the paged cache.
//
// Flash-attention dataflow with mma.sync.m16n8k16 (bf16 in, fp32 accumulate): a CTA of four
// warps owns 64 consecutive query rows of one request and one head (16 rows per warp) and
// walks that request's keys 64 at a time from position 0 (or from the window's first block)
// up to the tile's last row. K and V blocks are gathered from the pages with 16-byte
// cp.async copies into double-buffered shared memory; scores, the running maximum and sum
// (online softmax, exp2 of log2e-scaled scores) and the output accumulator stay in fp32
// registers; probabilities are rounded to bf16 only as the A operand of P.V. The key walk
// depends only on positions, so a row's output does not depend on how the prompt was cut.
//
// The rows of a step are the last rows[b] positions of each request b (row_start/kv_len);
// tiles of all requests are numbered consecutively along grid.x and each CTA finds its own.
// Compiled for one head size: -DAYK_HEAD_DIM=<multiple of 16, at most 256>.
//
// This kernel uses the legacy warp-level tensor path (not tcgen05): attention is ~5% of a
// prefill step's FLOPs and this dataflow is proven; the matrix products that dominate run on
// tcgen05 (gemm_tc.cu).
#include "common.cuh"

#ifndef AYK_HEAD_DIM
#define AYK_HEAD_DIM 64
#endif

namespace ayk {

constexpr int PF_HD = AYK_HEAD_DIM;
constexpr int PF_BM = 64;               // query rows per CTA
constexpr int PF_BN = 64;               // keys per block
constexpr int PF_STRIDE = PF_HD + 8;    // elements per shared row: one 16-byte chunk of padding
constexpr int PF_TILE = PF_BM * PF_STRIDE;  // elements of one [64][HD] tile
constexpr int PF_CHUNKS = PF_HD / 8;    // 16-byte chunks per row
constexpr int PF_SMEM_BYTES = 5 * PF_TILE * 2;  // Q, 2 x K, 2 x V
static_assert(PF_HD % 16 == 0 && PF_HD >= 16 && PF_HD <= 256, "head size");

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Gather one block of 64 keys (or values) of one head into a [64][HD] shared tile.
__device__ __forceinline__ void load_kv_block(__nv_bfloat16* tile,
                                              const __nv_bfloat16* __restrict__ pages,
                                              const int* __restrict__ table, int key0,
                                              int first_key, int last_key, int num_kv_heads,
                                              int kv_head, int page_size, int page_shift) {
  // keys outside [first_key, last_key] are zero-filled: their pages may be gone (a window)
  // or hold anything, and 0 * NaN would poison the sum
  for (int i = threadIdx.x; i < PF_BN * PF_CHUNKS; i += 128) {
    const int r = i / PF_CHUNKS, c = i % PF_CHUNKS;
    const int key = key0 + r;
    const bool valid = key >= first_key && key <= last_key;
    const __nv_bfloat16* src = pages;
    if (valid) {
      // a shift and a mask when the page size is a power of two: a division costs more
      // instructions than the rest of the address
      const int index = page_shift >= 0 ? key >> page_shift : key / page_size;
      const int slot = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
      const int page = table[index];
      src = pages + (((size_t)page * num_kv_heads + kv_head) * page_size + slot) * PF_HD + c * 8;
    }
    cp_async16(tile + r * PF_STRIDE + c * 8, src, valid);
  }
}

__global__ void __launch_bounds__(128)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int ld_q,
                         const __nv_bfloat16* __restrict__ k_pages,
                         const __nv_bfloat16* __restrict__ v_pages,
                         const int* __restrict__ block_table, int table_stride,
                         const int* __restrict__ row_start, const int* __restrict__ kv_len,
                         __nv_bfloat16* __restrict__ out, int ld_out, int num_requests,
                         int num_kv_heads, int group, int page_size, float scale, int window,
                         int total_tiles, int page_shift) {
  extern __shared__ __align__(16) unsigned char pf_smem[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(pf_smem);
  __nv_bfloat16* k_s = q_s + PF_TILE;       // two stages
  __nv_bfloat16* v_s = k_s + 2 * PF_TILE;   // two stages

  pdl_launch_dependents();
  pdl_wait_for(q, k_pages, v_pages);
  // Which request and which 64-row tile of it. Heads run along grid.x and tiles along grid.y
  // from the last tile down: a tile's work grows with its position in the sequence, and the
  // longest tiles must start first or they finish alone at the end.
  int tile = total_tiles - 1 - (int)blockIdx.y, req = 0, rows_b = 0;
  for (; req < num_requests; ++req) {
    rows_b = row_start[req + 1] - row_start[req];
    const int tiles = (rows_b + PF_BM - 1) / PF_BM;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (req >= num_requests) return;
  const int head = blockIdx.x;
  const int kv_head = head / group;
  const int first_row = row_start[req] + tile * PF_BM;
  const int nrows = rows_b - tile * PF_BM < PF_BM ? rows_b - tile * PF_BM : PF_BM;
  const int length = kv_len[req];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (length == 0) {  // a padding request: zeros
    for (int i = threadIdx.x; i < nrows * PF_HD; i += 128) {
      out[(size_t)(first_row + i / PF_HD) * ld_out + head * PF_HD + i % PF_HD] =
          __float2bfloat16_rn(0.f);
    }
    return;
  }
  const int pos0 = length - rows_b + tile * PF_BM;  // position of the tile's first row
  const int last_key = pos0 + nrows - 1;
  const int lo_min = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int block_lo = lo_min / PF_BN;
  const int block_hi = last_key / PF_BN;  // inclusive
  const int* table = block_table + (size_t)req * table_stride;

  // Q tile and the first K/V block
  for (int i = threadIdx.x; i < PF_BM * PF_CHUNKS; i += 128) {
    const int r = i / PF_CHUNKS, c = i % PF_CHUNKS;
    const bool valid = r < nrows;
    const __nv_bfloat16* src =
        q + (size_t)(first_row + (valid ? r : 0)) * ld_q + head * PF_HD + c * 8;
    cp_async16(q_s + r * PF_STRIDE + c * 8, src, valid);
  }
  load_kv_block(k_s, k_pages, table, block_lo * PF_BN, lo_min, last_key, num_kv_heads,
                kv_head, page_size, page_shift);
  load_kv_block(v_s, v_pages, table, block_lo * PF_BN, lo_min, last_key, num_kv_heads,
                kv_head, page_size, page_shift);
  cp_async_commit();

  float o[PF_HD / 8][4];
#pragma unroll
  for (int t = 0; t < PF_HD / 8; ++t) { o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f; }
  float run_max[2] = {-INFINITY, -INFINITY}, run_sum[2] = {0.f, 0.f};
  const float scale2 = scale * 1.4426950408889634f;  // scores in units of log2
  const int row_a = pos0 + warp * 16 + (lane >> 2);  // position of this thread's first row
  uint32_t q_frag[PF_HD / 16][4];
  bool q_loaded = false;

  for (int block = block_lo; block <= block_hi; ++block) {
    const int stage = (block - block_lo) & 1;
    if (block < block_hi) {  // prefetch the next block into the other stage
      load_kv_block(k_s + (stage ^ 1) * PF_TILE, k_pages, table, (block + 1) * PF_BN, lo_min,
                    last_key, num_kv_heads, kv_head, page_size, page_shift);
      load_kv_block(v_s + (stage ^ 1) * PF_TILE, v_pages, table, (block + 1) * PF_BN, lo_min,
                    last_key, num_kv_heads, kv_head, page_size, page_shift);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (!q_loaded) {
#pragma unroll
      for (int kk = 0; kk < PF_HD / 16; ++kk) {
        ldmatrix_x4(q_frag[kk], q_s + (warp * 16 + (lane & 15)) * PF_STRIDE + kk * 16 +
                                    (lane >> 4) * 8);
      }
      q_loaded = true;
    }
    const __nv_bfloat16* kb = k_s + stage * PF_TILE;
    const __nv_bfloat16* vb = v_s + stage * PF_TILE;

    // S = Q K^T : 16 rows x 64 keys per warp
    float s[PF_BN / 8][4];
#pragma unroll
    for (int t = 0; t < PF_BN / 8; ++t) { s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < PF_HD / 16; ++kk) {
#pragma unroll
      for (int t = 0; t < PF_BN / 16; ++t) {
        uint32_t kf[4];
        // lanes 0-7: keys 16t..+7, d chunk 0; 8-15: same keys, chunk 1; 16-23: keys +8, chunk
        // 0; 24-31: keys +8, chunk 1
        ldmatrix_x4(kf, kb + (t * 16 + (lane & 7) + ((lane >> 4) << 3)) * PF_STRIDE + kk * 16 +
                            ((lane >> 3) & 1) * 8);
        mma_bf16(s[2 * t], q_frag[kk], kf[0], kf[1]);
        mma_bf16(s[2 * t + 1], q_frag[kk], kf[2], kf[3]);
      }
    }
    // mask, online softmax (rows row_a and row_a + 8). A block that lies wholly before the
    // warp's first row (and no window) has nothing to mask: only the scaling remains.
    const int key_base = block * PF_BN + (lane & 3) * 2;
    const bool all_seen = window == 0 && block * PF_BN + PF_BN - 1 <= pos0 + warp * 16;
    float block_max[2] = {-INFINITY, -INFINITY};
    if (all_seen) {
#pragma unroll
      for (int t = 0; t < PF_BN / 8; ++t) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[t][e] *= scale2;
          block_max[e >> 1] = fmaxf(block_max[e >> 1], s[t][e]);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < PF_BN / 8; ++t) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key_base + t * 8 + (e & 1);
          const int pos = row_a + (e >> 1) * 8;
          const bool seen = key <= pos && (window == 0 || key > pos - window);
          const float v = seen ? s[t][e] * scale2 : -INFINITY;
          s[t][e] = v;
          block_max[e >> 1] = fmaxf(block_max[e >> 1], v);
        }
      }
    }
    float corr[2], ref[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      block_max[h] = fmaxf(block_max[h], __shfl_xor_sync(0xffffffffu, block_max[h], 1));
      block_max[h] = fmaxf(block_max[h], __shfl_xor_sync(0xffffffffu, block_max[h], 2));
      const float new_max = fmaxf(run_max[h], block_max[h]);
      ref[h] = new_max == -INFINITY ? 0.f : new_max;
      corr[h] = exp2f(run_max[h] - ref[h]);
      run_max[h] = new_max;
      run_sum[h] *= corr[h];
    }
    float part[2] = {0.f, 0.f};
#pragma unroll
    for (int t = 0; t < PF_BN / 8; ++t) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = exp2f(s[t][e] - ref[e >> 1]);
        s[t][e] = p;
        part[e >> 1] += p;
      }
    }
    run_sum[0] += part[0];
    run_sum[1] += part[1];
#pragma unroll
    for (int t = 0; t < PF_HD / 8; ++t) {
      o[t][0] *= corr[0]; o[t][1] *= corr[0];
      o[t][2] *= corr[1]; o[t][3] *= corr[1];
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < PF_BN / 16; ++kk) {
      uint32_t pf[4];
      pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int t = 0; t < PF_HD / 16; ++t) {
        uint32_t vf[4];
        // transposed load: lanes 0-7: keys 16kk..+7 at d chunk 2t; 8-15: keys +8, same chunk;
        // 16-23: keys 16kk..+7 at chunk 2t+1; 24-31: keys +8, chunk 2t+1
        ldmatrix_x4_trans(vf, vb + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PF_STRIDE +
                                  t * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * t], pf, vf[0], vf[1]);
        mma_bf16(o[2 * t + 1], pf, vf[2], vf[3]);
      }
    }
    __syncthreads();  // everyone is done with this stage before it is refilled
  }

  // normalise; stage the tile through shared memory (Q's space) for 16-byte stores
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    run_sum[h] += __shfl_xor_sync(0xffffffffu, run_sum[h], 1);
    run_sum[h] += __shfl_xor_sync(0xffffffffu, run_sum[h], 2);
  }
  const float inv0 = 1.f / run_sum[0], inv1 = 1.f / run_sum[1];
  const int r0 = warp * 16 + (lane >> 2);
#pragma unroll
  for (int t = 0; t < PF_HD / 8; ++t) {
    const int col = t * 8 + (lane & 3) * 2;
    *reinterpret_cast<uint32_t*>(q_s + r0 * PF_STRIDE + col) =
        pack_bf16(o[t][0] * inv0, o[t][1] * inv0);
    *reinterpret_cast<uint32_t*>(q_s + (r0 + 8) * PF_STRIDE + col) =
        pack_bf16(o[t][2] * inv1, o[t][3] * inv1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nrows * PF_CHUNKS; i += 128) {
    const int r = i / PF_CHUNKS, c = i % PF_CHUNKS;
    const uint4 v = *reinterpret_cast<const uint4*>(q_s + r * PF_STRIDE + c * 8);
    *reinterpret_cast<uint4*>(out + (size_t)(first_row + r) * ld_out + head * PF_HD + c * 8) = v;
  }
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

AYK_API int ayk_attention_prefill_head_dim() { return ayk::PF_HD; }

// bfloat16 only. q/out rows are 16-byte aligned (ld multiples of 8 elements). `total_tiles`
// = sum over requests of ceil(rows / 64), computed by the caller from its host copy of the
// rows.
AYK_API int ayk_attention_prefill(const void* q, int ld_q, const void* k_pages,
                                  const void* v_pages, const int* block_table, int table_stride,
                                  const int* row_start, const int* kv_len, void* out, int ld_out,
                                  int num_requests, int total_tiles, int num_heads,
                                  int num_kv_heads, int head_dim, int page_size, float scale,
                                  int window, void* stream) {
  using namespace ayk;
  if (num_requests == 0 || total_tiles == 0) return AYK_OK;
  if (head_dim != PF_HD) return AYK_BAD_ARGUMENT;
  if (num_requests < 0 || total_tiles < 0 || num_heads < 1 || num_kv_heads < 1 ||
      num_heads % num_kv_heads || page_size < 1 || table_stride < 1 || window < 0) {
    return AYK_BAD_ARGUMENT;
  }
  if (((uintptr_t)q % 16) || ((uintptr_t)out % 16) || ((uintptr_t)k_pages % 16) ||
      ((uintptr_t)v_pages % 16) || (ld_q % 8) || (ld_out % 8)) {
    return AYK_BAD_ALIGNMENT;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         PF_SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (total_tiles > 65535) return AYK_TOO_LARGE;
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0) {
    page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
  }
  return launch_kernel(attention_prefill_kernel, dim3(num_heads, total_tiles), dim3(128),
                       PF_SMEM_BYTES, (cudaStream_t)stream, 1, (const __nv_bfloat16*)q, ld_q,
                       (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table,
                       table_stride, row_start, kv_len, (__nv_bfloat16*)out, ld_out, num_requests,
                       num_kv_heads, num_heads / num_kv_heads, page_size, scale, window,
                       total_tiles, page_shift);
}
