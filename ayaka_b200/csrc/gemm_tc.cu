// C[M,N] = A[M,K] * W[N,K]^T (+ bias, activation, residual) in bfloat16 on the 5th-generation
// tensor cores: TMA -> shared memory (128-byte swizzle) -> tcgen05.mma with the fp32
// accumulator in tensor memory -> tcgen05.ld -> epilogue in registers -> global memory.
//
// One CTA of 128 threads computes one 128 x BN tile of C. Warp 0's elected thread is the TMA
// producer, warp 1's the MMA issuer; a ring of STAGES buffers with a full/empty mbarrier pair
// each decouples them. When the last MMA has been committed all four warps run the epilogue:
// warp w owns tensor-memory lanes 32w..32w+31, i.e. rows 32w..32w+31 of the tile, and each
// thread reads its row 32 columns at a time.
//
// K is walked in blocks of 64 from 0 upward whatever M and N are, so an output element's
// accumulation order does not depend on the batch. Tails in M, N and K are zero-filled by
// TMA and masked at the store. Needs: A and W 16-byte aligned with row strides that are
// multiples of 8 elements (the caller falls back to the CUDA-core kernel otherwise).
//
// Every wait is bounded; a wait that runs out sets *status = AYK_WAIT_TIMEOUT, the CTA skips
// its stores, drains its copies, frees its tensor memory and returns.
#include <mutex>
#include <unordered_map>

#include "tc_common.cuh"

namespace ayk {

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;

enum OutMode : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_RESIDUAL_F32 = 2 };

// tensor-memory columns to allocate for an accumulator `n` wide: a power of two, at least 32
__host__ __device__ constexpr uint32_t tc_tmem_cols(int n) {
  return n <= 32 ? 32 : (n <= 64 ? 64 : (n <= 128 ? 128 : (n <= 256 ? 256 : 512)));
}

// Shared memory the epilogue stages output boxes in: 32 rows x 128 bytes per epilogue warp.
constexpr int EPI_WARP_BYTES = 32 * 128;
constexpr int EPI_BYTES = 4 * EPI_WARP_BYTES;
// ... and each epilogue warp's copy of the tile's bias (BN floats), fetched before the warp
// waits for the accumulator: a load of the bias after the wait would put a trip through the
// (busy) memory system into every 32 columns of the epilogue.
constexpr int epi_bias_bytes(int bn) { return 4 * bn * 4; }

template <int BN, int STAGES>
struct TcSmem {
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = TC_A_BYTES + B_BYTES;
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int BIAS_OFFSET = EPI_OFFSET + EPI_BYTES;
  static constexpr int BAR_OFFSET = BIAS_OFFSET + epi_bias_bytes(BN);
  // full[STAGES], empty[STAGES], accum, then the tmem slot and the failure flag
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 1) * 8 + 16;
  static constexpr int DYNAMIC = TOTAL + 1024;  // room to align the base to 1024 bytes
};

// One output row's 32 consecutive columns n .. n + 31 (fp32 accumulators as raw bits): bias,
// activation or residual sum, and the store; `vec_ok` says that rows start on 16 bytes.
__device__ __forceinline__ void store_row_chunk(const uint32_t* raw, int m, int n, int N,
                                                const float* __restrict__ bias,
                                                void* __restrict__ out, int ldo, int mode,
                                                int act, int vec_ok) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    v[j] = __uint_as_float(raw[j]);
    if (bias != nullptr && n + j < N) v[j] += __ldg(bias + n + j);
  }
  const bool full_chunk = n + 32 <= N;
  if (mode == OUT_BF16) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)m * ldo + n;
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = activate(v[j], act);
    if (vec_ok && full_chunk) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 packed;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j], v[j + 1]);
        __nv_bfloat162 h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
        __nv_bfloat162 h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
        packed.x = *reinterpret_cast<uint32_t*>(&h0);
        packed.y = *reinterpret_cast<uint32_t*>(&h1);
        packed.z = *reinterpret_cast<uint32_t*>(&h2);
        packed.w = *reinterpret_cast<uint32_t*>(&h3);
        *reinterpret_cast<uint4*>(dst + j) = packed;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {  // unrolled: v[] must stay in registers
        if (n + j < N) dst[j] = __float2bfloat16_rn(v[j]);
      }
    }
  } else {
    float* dst = reinterpret_cast<float*>(out) + (size_t)m * ldo + n;
    if (mode == OUT_F32) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = activate(v[j], act);
    }
    if (vec_ok && full_chunk) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        if (mode == OUT_RESIDUAL_F32) {
          const float4 r = *reinterpret_cast<const float4*>(dst + j);
          o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
        }
        *reinterpret_cast<float4*>(dst + j) = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (n + j < N) dst[j] = mode == OUT_RESIDUAL_F32 ? dst[j] + v[j] : v[j];
      }
    }
  }
}

// One epilogue warp's 32 rows of a tile, BN columns from tensor-memory address `acc` (lane
// base included): bias, activation, rounding, then out to global memory. With `vec_ok` (the
// output's base and row stride are multiples of 16 bytes, `map_out` describes it) the rows
// are staged in `staging` (this warp's 32 x 128 bytes, 128-byte swizzle: lane r writes its
// 16-byte piece c at piece c ^ (r & 7), free of bank conflicts) and leave as one TMA store per
// box of 128 bytes x 32 rows — or one TMA reduce-add for the residual sum, which adds in the
// memory system and so never reads the old rows into the SM. TMA clips at the matrix edges.
// A lane storing its own row directly touches 32 different lines per instruction; measured
// on a B200 that made the epilogue of a 128 x 192 tile take 11 microseconds against 8.5 for
// its main loop. Without `vec_ok` that direct path is what remains.
// This warp's copy of the tile's bias (zeros where there is none) into shared memory.
template <int BN>
__device__ __forceinline__ void stage_bias(float* bias_s, const float* __restrict__ bias, int n0,
                                           int N, int lane) {
  for (int i = lane; i < BN; i += 32) {
    bias_s[i] = (bias != nullptr && n0 + i < N) ? __ldg(bias + n0 + i) : 0.f;
  }
  __syncwarp();
}

// The key and value columns of a fused query/key/value projection go into the cache instead
// of the output: columns from q_width on are keys, then values (kv_width of each), heads of head_dim columns; row m is
// stored at slot slots[m] (page * page_size + offset; negative: nowhere) of pages laid out
// [page][kv_head][slot][head_dim]. head_dim and the widths are multiples of 32, so the 32
// columns a warp converts at a time lie in one head.
struct KvScatter {
  const int* slots;
  __nv_bfloat16* k_pages;
  __nv_bfloat16* v_pages;
  int q_width, kv_width, num_kv_heads, head_dim, page_size;
};

// Where row m goes in the cache: the element offset of its slot in head 0, or -1 for a row
// that stores nothing. The slots are the step's metadata, not written by the kernel ahead:
// the epilogue warps fetch this before they wait for the accumulator.
__device__ __forceinline__ long long kv_row_offset(const KvScatter& kv, int m, int M) {
  const int slot = m < M ? __ldg(kv.slots + m) : -1;
  if (slot < 0) return -1;
  const int page = slot / kv.page_size, within = slot - page * kv.page_size;
  return ((long long)page * kv.num_kv_heads * kv.page_size + within) * kv.head_dim;
}

template <int BN, bool SCATTER = false>
__device__ __forceinline__ void epilogue_warp(uint32_t acc, int lane, int m_warp, int n0, int M,
                                              int N, const float* __restrict__ bias,
                                              const float* bias_s, void* __restrict__ out,
                                              int ldo, int mode, int act, int vec_ok,
                                              const CUtensorMap* map_out, uint8_t* staging,
                                              const KvScatter& kv = KvScatter{},
                                              long long kv_row = -1) {
  if (!vec_ok) {
    const int m = m_warp + lane;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      const int n = n0 + c * 32;
      if (n >= N) break;  // uniform over the warp
      uint32_t raw[32];
      tmem_ld_32x32(acc + (uint32_t)(c * 32), raw);
      tmem_ld_wait();
      if (m < M) store_row_chunk(raw, m, n, N, bias, out, ldo, mode, act, 0);
      __syncwarp();  // the next tcgen05.ld needs the whole warp
    }
    return;
  }
  if (m_warp >= M) return;  // nothing of this warp's rows exists (uniform over the warp)
  uint8_t* row = staging + lane * 128;
  const int swz = lane & 7;
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    const int n = n0 + c * 32;
    if (n >= N) break;
    uint8_t* kv_dst = nullptr;  // this chunk's 64 bytes of the row in the cache, if any
    if (SCATTER && n >= kv.q_width && kv_row >= 0) {
      const int col = n - kv.q_width;
      const int value = col >= kv.kv_width ? 1 : 0;
      const int hcol = col - value * kv.kv_width;
      const int head = hcol / kv.head_dim;
      __nv_bfloat16* pages = value ? kv.v_pages : kv.k_pages;
      kv_dst = reinterpret_cast<uint8_t*>(
          pages + (size_t)kv_row + (size_t)head * kv.page_size * kv.head_dim +
          (hcol - head * kv.head_dim));
    }
    // key and value columns go to the cache only (q_width is a multiple of 64: a box of 64
    // columns is all queries or all keys/values)
    const bool to_cache = SCATTER && n >= kv.q_width;
    // a box is 64 bf16 columns (two passes of this loop) or 32 fp32 columns (one)
    const bool opens_box = !to_cache && (mode != OUT_BF16 || (c & 1) == 0);
    if (opens_box) {
      if (lane == 0) bulk_wait_read_all();  // the box before has left the staging rows
      __syncwarp();
    }
    uint32_t raw[32];
    tmem_ld_32x32(acc + (uint32_t)(c * 32), raw);
    tmem_ld_wait();
    float v[32];
#pragma unroll
    for (int q = 0; q < 8; ++q) {  // the bias: the same shared-memory words for every lane
      const float4 b = *reinterpret_cast<const float4*>(bias_s + c * 32 + q * 4);
      v[q * 4] = __uint_as_float(raw[q * 4]) + b.x;
      v[q * 4 + 1] = __uint_as_float(raw[q * 4 + 1]) + b.y;
      v[q * 4 + 2] = __uint_as_float(raw[q * 4 + 2]) + b.z;
      v[q * 4 + 3] = __uint_as_float(raw[q * 4 + 3]) + b.w;
    }
    if (mode == OUT_BF16) {
      // (the tanh of a GELU through the special-function unit: with tanhf the epilogue of a
      // 128 x 256 tile took longer than its main loop)
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = activate_to_bf16(v[j], act);
    } else if (mode == OUT_F32) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = activate(v[j], act);
    }
    if (mode == OUT_BF16) {
      const int piece0 = (c & 1) * 4;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 packed;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(v[q * 8], v[q * 8 + 1]);
        __nv_bfloat162 h1 = __floats2bfloat162_rn(v[q * 8 + 2], v[q * 8 + 3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[q * 8 + 4], v[q * 8 + 5]);
        __nv_bfloat162 h3 = __floats2bfloat162_rn(v[q * 8 + 6], v[q * 8 + 7]);
        packed.x = *reinterpret_cast<uint32_t*>(&h0);
        packed.y = *reinterpret_cast<uint32_t*>(&h1);
        packed.z = *reinterpret_cast<uint32_t*>(&h2);
        packed.w = *reinterpret_cast<uint32_t*>(&h3);
        if (to_cache) {
          if (kv_dst != nullptr) *reinterpret_cast<uint4*>(kv_dst + (q << 4)) = packed;
        } else {
          *reinterpret_cast<uint4*>(row + (((piece0 + q) ^ swz) << 4)) = packed;
        }
      }
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        *reinterpret_cast<float4*>(row + ((q ^ swz) << 4)) =
            make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
      }
    }
    const bool closes_box = !to_cache && (mode != OUT_BF16 || (c & 1) == 1 ||
                                          c + 1 == BN / 32 || n + 32 >= N);
    if (closes_box) {
      fence_proxy_async_shared();
      __syncwarp();
      if (lane == 0) {
        const int x = mode == OUT_BF16 ? n0 + (c & ~1) * 32 : n;
        if (mode == OUT_RESIDUAL_F32) {
          tma_reduce_add_2d(map_out, staging, x, m_warp);
        } else {
          tma_store_2d(map_out, staging, x, m_warp);
        }
        bulk_commit_group();
      }
    }
  }
}

template <int BN, int STAGES, bool SCATTER = false>
__global__ void __launch_bounds__(128)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_out, const float* __restrict__ bias,
               void* __restrict__ out, int ldo, int M, int N, int K, int act, int mode,
               int vec_ok, int* __restrict__ status, KvScatter kv) {
  using L = TcSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* accum = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * TC_BM;
  const int num_kb = (K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum, 1);
    *failed = 0;
    mbar_fence_init();
    tma_prefetch_map(&map_a);
    tma_prefetch_map(&map_w);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, tc_tmem_cols(BN));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_launch_dependents();
  int issued = 0;  // k-blocks whose copies the producer has started
  if (warp == 0 && lane == 0) {
    // weights do not depend on the kernel before this one: fetch the first stages' weight
    // tiles at once, wait for the predecessor, then fetch the activations
    const int ahead = num_kb < STAGES ? num_kb : STAGES;
    for (int kb = 0; kb < ahead; ++kb) {
      uint8_t* a_tile = smem + kb * L::STAGE_BYTES;
      mbar_expect_tx(&full[kb], L::STAGE_BYTES);
      tma_load_2d(a_tile + TC_A_BYTES, &map_w, &full[kb], kb * TC_BK, n0);
    }
    pdl_wait();
    for (int kb = 0; kb < num_kb; ++kb) {
      const int s = kb % STAGES;
      uint8_t* a_tile = smem + s * L::STAGE_BYTES;
      if (kb >= STAGES) {
        if (!mbar_wait(&empty[s], ((kb / STAGES) & 1) ^ 1)) {
          *failed = 1;
          break;
        }
        mbar_expect_tx(&full[s], L::STAGE_BYTES);
        tma_load_2d(a_tile + TC_A_BYTES, &map_w, &full[s], kb * TC_BK, n0);
      }
      tma_load_2d(a_tile, &map_a, &full[s], kb * TC_BK, m0);
      issued = kb + 1;
    }
  } else if (warp == 1 && lane == 0) {
    constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, BN);
    bool ok = true;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % STAGES;
      if (!mbar_wait(&full[s], (kb / STAGES) & 1)) {
        *failed = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      const uint8_t* a_tile = smem + s * L::STAGE_BYTES;
      const uint8_t* b_tile = a_tile + TC_A_BYTES;
#pragma unroll
      for (int k = 0; k < TC_BK / 16; ++k) {
        umma_f16(tmem_base, umma_desc_k128(a_tile, k * 32), umma_desc_k128(b_tile, k * 32),
                 idesc, (kb | k) != 0);
      }
      umma_commit(&empty[s]);  // the stage is free once these MMAs have read it
    }
    if (ok) umma_commit(accum);
  }

  // ---- epilogue: all four warps -----------------------------------------------------
  __syncwarp();
  float* bias_s = reinterpret_cast<float*>(smem + L::BIAS_OFFSET) + warp * BN;
  stage_bias<BN>(bias_s, bias, n0, N, lane);
  const long long kv_row = SCATTER ? kv_row_offset(kv, m0 + warp * 32 + lane, M) : -1;
  pdl_wait();
  bool have = mbar_wait(accum, 0);
  if (!have) *failed = 1;
  tc_fence_after();
  if (have && *failed == 0) {
    epilogue_warp<BN, SCATTER>(tmem_base + ((uint32_t)(warp * 32) << 16), lane, m0 + warp * 32,
                               n0, M, N, bias, bias_s, out, ldo, mode, act, vec_ok, &map_out,
                               smem + L::EPI_OFFSET + warp * EPI_WARP_BYTES, kv, kv_row);
    if (lane == 0) bulk_wait_all();  // the stores are done before the CTA says it is
  }

  // ---- teardown ---------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*failed != 0) {
    if (warp == 0 && lane == 0) {
      // copies this thread started may still be landing: wait for each started stage, bounded
      for (int kb = issued > STAGES ? issued - STAGES : 0; kb < issued; ++kb) {
        mbar_wait(&full[kb % STAGES], (kb / STAGES) & 1);
      }
      atomicExch(status, AYK_WAIT_TIMEOUT);
    }
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tmem_base, tc_tmem_cols(BN));
}

// ---------------------------------------------------------------------------------------
// The same product for a few hundred rows, where 128 x 128 tiles are too few to fill the
// device (288 rows x 1280 columns are 30 tiles on 148 SMs, each walking all of K): the K
// range is split over the 2 or 4 CTAs of a thread-block cluster. Every CTA accumulates its
// share of K for the whole tile in tensor memory, then the cluster does a reduce-scatter
// through distributed shared memory: CTA r owns columns r * 128 / R .. of the tile; every
// CTA writes its partial sums of those columns into a slot of its own in CTA r's shared
// memory (its own slot locally), one cluster barrier makes them visible, and CTA r adds the
// R slots in rank order, so the sum's order is fixed whatever the batch. Then bias,
// activation or residual sum, and the store (or, for the fused query/key/value projection,
// the scatter of key and value columns into the cache), each lane on its own row. No CTA
// reads or writes a peer's memory after the barrier, so nobody has to wait to leave; a CTA
// whose wait ran out still takes part in the barrier (its peers would wait for it for ever
// otherwise), skips its stores and reports through `status`.
constexpr int SK_BN = 128;
template <int STAGES>
struct SplitKSmem {
  static constexpr int STAGE_BYTES = TC_A_BYTES + SK_BN * TC_BK * 2;
  static constexpr int RECV_OFFSET = STAGES * STAGE_BYTES;      // [src rank][row][own columns]
  static constexpr int RECV_BYTES = TC_BM * SK_BN * 4;          // R * 128 * (128 / R) floats
  static constexpr int BAR_OFFSET = RECV_OFFSET + RECV_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 1) * 8 + 16;
  static constexpr int DYNAMIC = TOTAL + 1024;
};

template <int STAGES, bool SCATTER>
__global__ void __launch_bounds__(128)
gemm_tc_splitk_kernel(const __grid_constant__ CUtensorMap map_a,
                      const __grid_constant__ CUtensorMap map_w, const float* __restrict__ bias,
                      void* __restrict__ out, int ldo, int M, int N, int K, int act, int mode,
                      int vec_ok, int kb_per_split, int* __restrict__ status, KvScatter kv) {
  using L = SplitKSmem<STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* accum = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* recv = reinterpret_cast<float*>(smem + L::RECV_OFFSET);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = gridDim.y;                 // the cluster spans grid.y
  const int rank = (int)cluster_rank();    // == blockIdx.y
  const int n0 = blockIdx.x * SK_BN, m0 = blockIdx.z * TC_BM;
  const int num_kb = (K + TC_BK - 1) / TC_BK;
  const int kb0 = rank * kb_per_split;
  const int kb1 = kb0 + kb_per_split < num_kb ? kb0 + kb_per_split : num_kb;
  const int my_kb = kb1 - kb0;             // at least 1 (the host chooses R so)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum, 1);
    *failed = 0;
    mbar_fence_init();
    tma_prefetch_map(&map_a);
    tma_prefetch_map(&map_w);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, tc_tmem_cols(SK_BN));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_launch_dependents();
  cluster_arrive_release();  // "this CTA runs": awaited before anyone writes to it
  int issued = 0;
  if (warp == 0 && lane == 0) {
    const int ahead = my_kb < STAGES ? my_kb : STAGES;
    for (int i = 0; i < ahead; ++i) {  // weight tiles do not depend on the kernel ahead
      mbar_expect_tx(&full[i], L::STAGE_BYTES);
      tma_load_2d(smem + i * L::STAGE_BYTES + TC_A_BYTES, &map_w, &full[i], (kb0 + i) * TC_BK,
                  n0);
    }
    pdl_wait();
    for (int i = 0; i < my_kb; ++i) {
      const int s = i % STAGES;
      uint8_t* a_tile = smem + s * L::STAGE_BYTES;
      if (i >= STAGES) {
        if (!mbar_wait(&empty[s], ((i / STAGES) & 1) ^ 1)) {
          *failed = 1;
          break;
        }
        mbar_expect_tx(&full[s], L::STAGE_BYTES);
        tma_load_2d(a_tile + TC_A_BYTES, &map_w, &full[s], (kb0 + i) * TC_BK, n0);
      }
      tma_load_2d(a_tile, &map_a, &full[s], (kb0 + i) * TC_BK, m0);
      issued = i + 1;
    }
  } else if (warp == 1 && lane == 0) {
    constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, SK_BN);
    bool ok = true;
    for (int i = 0; i < my_kb && ok; ++i) {
      const int s = i % STAGES;
      if (!mbar_wait(&full[s], (i / STAGES) & 1)) {
        *failed = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      const uint8_t* a_tile = smem + s * L::STAGE_BYTES;
      const uint8_t* b_tile = a_tile + TC_A_BYTES;
#pragma unroll
      for (int k = 0; k < TC_BK / 16; ++k) {
        umma_f16(tmem_base, umma_desc_k128(a_tile, k * 32), umma_desc_k128(b_tile, k * 32),
                 idesc, (i | k) != 0);
      }
      umma_commit(&empty[s]);
    }
    if (ok) umma_commit(accum);
  }

  // ---- reduce-scatter: this CTA's partial sums go to the owners of their columns ------
  __syncwarp();
  const int row = warp * 32 + lane;  // the tile row (tensor-memory lane) this thread owns
  const long long kv_row = SCATTER ? kv_row_offset(kv, m0 + row, M) : -1;
  pdl_wait();
  bool have = mbar_wait(accum, 0);
  if (!have) *failed = 1;
  tc_fence_after();
  const int chunks_own = 4 / R;      // 32-column chunks a rank owns (R is 2 or 4)
  const int cols_own = SK_BN / R;
  cluster_wait_acquire();            // every CTA of the cluster has started
  if (have && *failed == 0) {
    const int swz = lane & 7;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t raw[32];
      tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(c * 32), raw);
      tmem_ld_wait();
      const int owner = c / chunks_own;
      // slot [rank][row][(c % chunks_own) * 32 ..]; the eight 16-byte pieces of a chunk are
      // permuted by the row so that a warp's stores spread over the banks
      float* local = recv + ((size_t)rank * TC_BM + row) * cols_own + (c % chunks_own) * 32;
      const uint32_t base = peer_address(local, (uint32_t)owner);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        st_cluster_v4(base + (uint32_t)(((q ^ swz) << 4)), raw[q * 4], raw[q * 4 + 1],
                      raw[q * 4 + 2], raw[q * 4 + 3]);
      }
    }
  }
  cluster_sync_all();  // every CTA, failed or not: the partial sums are visible after it

  // ---- this rank's columns: sum in rank order, then the epilogue ----------------------
  if (have && *failed == 0 && m0 + row < M) {
    const int swz = lane & 7;
#pragma unroll 1
    for (int oc = 0; oc < chunks_own; ++oc) {
      const int n = n0 + rank * cols_own + oc * 32;
      if (n >= N) break;
      uint32_t raw[32];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int src = 0; src < R; ++src) {
          const float4 part = *reinterpret_cast<const float4*>(
              reinterpret_cast<const uint8_t*>(recv + ((size_t)src * TC_BM + row) * cols_own +
                                               oc * 32) + ((q ^ swz) << 4));
          sum.x += part.x; sum.y += part.y; sum.z += part.z; sum.w += part.w;
        }
        raw[q * 4] = __float_as_uint(sum.x);
        raw[q * 4 + 1] = __float_as_uint(sum.y);
        raw[q * 4 + 2] = __float_as_uint(sum.z);
        raw[q * 4 + 3] = __float_as_uint(sum.w);
      }
      if (SCATTER && n >= kv.q_width) {
        // a key or value chunk: bias, round, and into the row's slot of the cache
        if (kv_row >= 0) {
          const int col = n - kv.q_width;
          const int value = col >= kv.kv_width ? 1 : 0;
          const int hcol = col - value * kv.kv_width;
          const int head = hcol / kv.head_dim;
          __nv_bfloat16* dst = (value ? kv.v_pages : kv.k_pages) + (size_t)kv_row +
                               (size_t)head * kv.page_size * kv.head_dim +
                               (hcol - head * kv.head_dim);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              v[j] = __uint_as_float(raw[q * 8 + j]) +
                     (bias != nullptr ? __ldg(bias + n + q * 8 + j) : 0.f);
            }
            uint4 packed;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(v[2], v[3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(v[6], v[7]);
            packed.x = *reinterpret_cast<uint32_t*>(&h0);
            packed.y = *reinterpret_cast<uint32_t*>(&h1);
            packed.z = *reinterpret_cast<uint32_t*>(&h2);
            packed.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(dst + q * 8) = packed;
          }
        }
      } else {
        store_row_chunk(raw, m0 + row, n, N, bias, out, ldo, mode, act, vec_ok);
      }
    }
  }

  // ---- teardown ---------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*failed != 0) {
    if (warp == 0 && lane == 0) {
      for (int i = issued > STAGES ? issued - STAGES : 0; i < issued; ++i) {
        mbar_wait(&full[i % STAGES], (i / STAGES) & 1);
      }
      atomicExch(status, AYK_WAIT_TIMEOUT);
    }
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tmem_base, tc_tmem_cols(SK_BN));
}

// ---------------------------------------------------------------------------------------
// The same product as a persistent kernel: one CTA per SM walks over output tiles, with two
// accumulators in tensor memory so that the epilogue of one tile runs under the main loop of
// the next. Six warps: warp 0's elected thread feeds the shared-memory ring by TMA without
// pausing between tiles, warp 1's issues the MMAs into accumulator (tile & 1), warps 2-5 are
// the epilogue (warp w reads tensor-memory lanes 32 * (w % 4) ..). Barriers: full/empty per
// ring stage, acc_full/acc_empty per accumulator. K is still walked 0 upward in blocks of 64
// for every tile, so results equal the one-tile-per-CTA kernel's bit for bit.
template <int BN, int STAGES>
struct PersistentSmem {
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = TC_A_BYTES + B_BYTES;
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int BIAS_OFFSET = EPI_OFFSET + EPI_BYTES;
  static constexpr int BAR_OFFSET = BIAS_OFFSET + epi_bias_bytes(BN);
  // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], then the tmem slot and the flag
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16;
  static constexpr int DYNAMIC = TOTAL + 1024;
};

template <int BN, int STAGES, bool SCATTER = false>
__global__ void __launch_bounds__(192)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                          const __grid_constant__ CUtensorMap map_w,
                          const __grid_constant__ CUtensorMap map_out,
                          const float* __restrict__ bias, void* __restrict__ out, int ldo, int M,
                          int N, int K, int act, int mode, int vec_ok,
                          int* __restrict__ status, KvScatter kv) {
  using L = PersistentSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + TC_BM - 1) / TC_BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + TC_BK - 1) / TC_BK;
  // two accumulators; the allocation is a power of two, the second starts at column BN
  constexpr uint32_t TMEM_COLS = 2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512));

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);  // the four epilogue warps
    }
    *failed = 0;
    mbar_fence_init();
    tma_prefetch_map(&map_a);
    tma_prefetch_map(&map_w);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();

  // tile t -> (m tile, n tile): consecutive tiles share the weight tile and walk down the rows
  auto tile_origin = [&](int t, int& m0, int& n0) {
    n0 = (t / tiles_m) * BN;
    m0 = (t % tiles_m) * TC_BM;
  };

  if (warp == 0 && lane == 0) {
    // ---- producer: one continuous stream of k-blocks over all of this CTA's tiles. The
    // weight tiles of the first stages do not depend on the kernel ahead: they start before
    // the dependency wait, the activations after it.
    int ahead = 0;
    if (blockIdx.x < num_tiles) {
      int m0, n0;
      tile_origin(blockIdx.x, m0, n0);
      ahead = num_kb < STAGES ? num_kb : STAGES;
      for (int kb = 0; kb < ahead; ++kb) {
        mbar_expect_tx(&full[kb], L::STAGE_BYTES);
        tma_load_2d(smem + kb * L::STAGE_BYTES + TC_A_BYTES, &map_w, &full[kb], kb * TC_BK, n0);
      }
    }
    pdl_wait();
    int it = 0;  // k-blocks issued so far
    for (int t = blockIdx.x; t < num_tiles && *failed == 0; t += gridDim.x) {
      int m0, n0;
      tile_origin(t, m0, n0);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % STAGES;
        uint8_t* a_tile = smem + s * L::STAGE_BYTES;
        if (it >= ahead) {
          if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1)) {
            *failed = 1;
            break;
          }
          mbar_expect_tx(&full[s], L::STAGE_BYTES);
          tma_load_2d(a_tile + TC_A_BYTES, &map_w, &full[s], kb * TC_BK, n0);
        }
        tma_load_2d(a_tile, &map_a, &full[s], kb * TC_BK, m0);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer
    constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, BN);
    int it = 0, local = 0;
    for (int t = blockIdx.x; t < num_tiles && *failed == 0; t += gridDim.x, ++local) {
      const int buf = local & 1;
      // the accumulator must have been drained by the epilogue of two tiles ago
      if (local >= 2 && !mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1)) {
        *failed = 1;
        break;
      }
      tc_fence_after();
      const uint32_t acc = tmem_base + (uint32_t)(buf * BN);
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % STAGES;
        if (!mbar_wait(&full[s], (it / STAGES) & 1)) {
          *failed = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint8_t* a_tile = smem + s * L::STAGE_BYTES;
        const uint8_t* b_tile = a_tile + TC_A_BYTES;
#pragma unroll
        for (int k = 0; k < TC_BK / 16; ++k) {
          umma_f16(acc, umma_desc_k128(a_tile, k * 32), umma_desc_k128(b_tile, k * 32), idesc,
                   (kb | k) != 0);
        }
        umma_commit(&empty[s]);
      }
      if (!ok) break;
      umma_commit(&acc_full[buf]);
    }
  } else if (warp >= 2) {
    // ---- epilogue: four warps, each on its quarter of the tensor-memory lanes
    pdl_wait();
    const int quarter = warp & 3;
    int local = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++local) {
      const int buf = local & 1;
      int m0, n0;
      tile_origin(t, m0, n0);
      float* bias_s = reinterpret_cast<float*>(smem + L::BIAS_OFFSET) + quarter * BN;
      stage_bias<BN>(bias_s, bias, n0, N, lane);
      const long long kv_row = SCATTER ? kv_row_offset(kv, m0 + quarter * 32 + lane, M) : -1;
      bool have = true;
      if (lane == 0) have = mbar_wait(&acc_full[buf], (local >> 1) & 1);
      have = __shfl_sync(0xffffffffu, have, 0);
      if (!have || *failed != 0) {
        if (lane == 0) *failed = 1;
        break;
      }
      tc_fence_after();
      epilogue_warp<BN, SCATTER>(
          tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(quarter * 32) << 16), lane,
          m0 + quarter * 32, n0, M, N, bias, bias_s, out, ldo, mode, act, vec_ok, &map_out,
          smem + L::EPI_OFFSET + quarter * EPI_WARP_BYTES, kv, kv_row);
      // this warp has read its lanes of the accumulator: hand it back
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (lane == 0) bulk_wait_all();  // the stores are done before the CTA says it is
  }

  // ---- teardown ---------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*failed != 0 && threadIdx.x == 0) atomicExch(status, AYK_WAIT_TIMEOUT);
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------
// The same persistent kernel for CTA pairs (tcgen05 cta_group::2): the two CTAs of a cluster
// work on one 256 x BN tile. Each loads its own 128 rows of the activations and its own half
// (BN / 2 rows) of the weight tile, so a stage of the ring is a third smaller than for a
// 128 x BN tile while the pair's MMA does twice the work: shared-memory traffic per FLOP,
// which bounds the single-CTA kernels, drops by a third. Only the even CTA (rank 0) issues
// MMAs; its `full` barriers count the bytes of both CTAs' copies (the odd CTA's copies name
// the even CTA's barrier), its commits arrive on the `empty` and `acc_full` barriers of both,
// and both CTAs' epilogue warps arrive on its `acc_empty`. Each CTA's epilogue reads its own
// 128 lanes of tensor memory. No copy is multicast. K is walked as in the other kernels, so
// the results are the same bit for bit.
template <int BN, int STAGES>
struct PairSmem {
  static constexpr int B_BYTES = (BN / 2) * TC_BK * 2;
  static constexpr int STAGE_BYTES = TC_A_BYTES + B_BYTES;
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int BIAS_OFFSET = EPI_OFFSET + EPI_BYTES;
  static constexpr int BAR_OFFSET = BIAS_OFFSET + epi_bias_bytes(BN);
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16;
  static constexpr int DYNAMIC = TOTAL + 1024;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(192)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_out, const float* __restrict__ bias,
                    void* __restrict__ out, int ldo, int M, int N, int K, int act, int mode,
                    int vec_ok, int* __restrict__ status) {
  using L = PairSmem<BN, STAGES>;
  static_assert(BN % 32 == 0 && BN <= 256, "tile width");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_rank();  // 0 issues the MMAs
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  constexpr int PAIR_BM = 2 * TC_BM;
  const int tiles_m = (M + PAIR_BM - 1) / PAIR_BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + TC_BK - 1) / TC_BK;
  constexpr uint32_t TMEM_COLS = 2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512));

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);  // four epilogue warps in each CTA (used in rank 0 only)
    }
    *failed = 0;
    mbar_fence_init();
    tma_prefetch_map(&map_a);
    tma_prefetch_map(&map_w);
  }
  if (warp == 0) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();

  auto tile_origin = [&](int t, int& m0, int& n0) {
    n0 = (t / tiles_m) * BN;
    m0 = (t % tiles_m) * PAIR_BM;
  };

  if (warp == 0 && lane == 0) {
    // ---- producer (in both CTAs): this CTA's rows of A and its half of the weight tile
    const uint32_t leader_full = peer_address(&full[0], 0);
    int ahead = 0;
    if (pair < num_tiles) {
      int m0, n0;
      tile_origin(pair, m0, n0);
      ahead = num_kb < STAGES ? num_kb : STAGES;
      for (int kb = 0; kb < ahead; ++kb) {
        if (rank == 0) mbar_expect_tx(&full[kb], 2 * L::STAGE_BYTES);
        tma_load_2d_pair(smem + kb * L::STAGE_BYTES + TC_A_BYTES, &map_w,
                         leader_full + 8u * (uint32_t)kb, kb * TC_BK, n0 + rank * (BN / 2));
      }
    }
    pdl_wait();
    int it = 0;
    for (int t = pair; t < num_tiles && *failed == 0; t += num_pairs) {
      int m0, n0;
      tile_origin(t, m0, n0);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % STAGES;
        uint8_t* a_tile = smem + s * L::STAGE_BYTES;
        if (it >= ahead) {
          if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1)) {
            *failed = 1;
            break;
          }
          if (rank == 0) mbar_expect_tx(&full[s], 2 * L::STAGE_BYTES);
          tma_load_2d_pair(a_tile + TC_A_BYTES, &map_w, leader_full + 8u * (uint32_t)s,
                           kb * TC_BK, n0 + rank * (BN / 2));
        }
        tma_load_2d_pair(a_tile, &map_a, leader_full + 8u * (uint32_t)s, kb * TC_BK,
                         m0 + rank * TC_BM);
      }
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---- MMA issuer: the even CTA, for both
    constexpr uint32_t idesc = umma_idesc_bf16(PAIR_BM, BN);
    int it = 0, local = 0;
    for (int t = pair; t < num_tiles && *failed == 0; t += num_pairs, ++local) {
      const int buf = local & 1;
      if (local >= 2 && !mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1)) {
        *failed = 1;
        break;
      }
      tc_fence_after();
      const uint32_t acc = tmem_base + (uint32_t)(buf * BN);
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % STAGES;
        if (!mbar_wait(&full[s], (it / STAGES) & 1)) {
          *failed = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint8_t* a_tile = smem + s * L::STAGE_BYTES;
        const uint8_t* b_tile = a_tile + TC_A_BYTES;
#pragma unroll
        for (int k = 0; k < TC_BK / 16; ++k) {
          umma_f16_pair(acc, umma_desc_k128(a_tile, k * 32), umma_desc_k128(b_tile, k * 32),
                        idesc, (kb | k) != 0);
        }
        umma_commit_pair(&empty[s], 3);
      }
      if (!ok) break;
      umma_commit_pair(&acc_full[buf], 3);
    }
  } else if (warp >= 2) {
    // ---- epilogue (in both CTAs): this CTA's 128 rows of the tile
    pdl_wait();
    const int quarter = warp & 3;
    int local = 0;
    for (int t = pair; t < num_tiles; t += num_pairs, ++local) {
      const int buf = local & 1;
      int m0, n0;
      tile_origin(t, m0, n0);
      float* bias_s = reinterpret_cast<float*>(smem + L::BIAS_OFFSET) + quarter * BN;
      stage_bias<BN>(bias_s, bias, n0, N, lane);
      bool have = true;
      if (lane == 0) have = mbar_wait(&acc_full[buf], (local >> 1) & 1);
      have = __shfl_sync(0xffffffffu, have, 0);
      if (!have || *failed != 0) {
        if (lane == 0) *failed = 1;
        break;
      }
      tc_fence_after();
      epilogue_warp<BN>(tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(quarter * 32) << 16), lane,
                        m0 + rank * TC_BM + quarter * 32, n0, M, N, bias, bias_s, out, ldo, mode,
                        act, vec_ok, &map_out, smem + L::EPI_OFFSET + quarter * EPI_WARP_BYTES);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) {
          mbar_arrive(&acc_empty[buf]);
        } else {
          mbar_arrive_cluster(peer_address(&acc_empty[buf], 0));
        }
      }
    }
    if (lane == 0) bulk_wait_all();  // the stores are done before the CTA says it is
  }

  // ---- teardown: nobody leaves while the peer may still signal it or read its operands
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (*failed != 0 && threadIdx.x == 0) atomicExch(status, AYK_WAIT_TIMEOUT);
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------
// Few rows (decode): the weight is the 128-row operand and the tokens are the narrow one
// ("swap A and B"): D[n, m] = sum_k W[n, k] * A[m, k], with m padded to MP in {16, 32, 64}.
// A step with a handful of tokens is pure weight streaming, and N / 128 CTAs are too few to
// pull the weights at HBM speed, so K is split over the CTAs of a thread-block cluster
// (grid.y = cluster size S). Each CTA accumulates its K range in tensor memory, parks the
// partial [MP, 128] tile in its shared memory, and after a cluster barrier CTA r sums columns
// r*MP/S .. (r+1)*MP/S over all peers through distributed shared memory in rank order 0..S-1
// (a fixed order: the result does not change from run to run), applies the epilogue and
// stores. Thread t owns output column n0 + t, so a warp's stores are contiguous.
template <int MP, int STAGES>
struct SmallSmem {
  static constexpr int W_BYTES = TC_BM * TC_BK * 2;
  static constexpr int A_BYTES = MP * TC_BK * 2;
  static constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
  static constexpr int PARTIAL_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int PARTIAL_BYTES = MP * TC_BM * 4;
  static constexpr int BAR_OFFSET = PARTIAL_OFFSET + PARTIAL_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 1) * 8 + 16;
  static constexpr int DYNAMIC = TOTAL + 1024;
};

__device__ __forceinline__ void store_output(void* out, int ldo, int m, int n, float v, int mode,
                                             int act) {
  if (mode == OUT_BF16) {
    reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + n] =
        __float2bfloat16_rn(activate_to_bf16(v, act));
  } else if (mode == OUT_F32) {
    reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = activate(v, act);
  } else {
    float* dst = reinterpret_cast<float*>(out) + (size_t)m * ldo + n;
    *dst = *dst + v;
  }
}

template <int MP, int STAGES>
__global__ void __launch_bounds__(128)
gemm_tc_small_kernel(const __grid_constant__ CUtensorMap map_w,
                     const __grid_constant__ CUtensorMap map_a, const float* __restrict__ bias,
                     void* __restrict__ out, int ldo, int M, int N, int K, int act, int mode,
                     int kb_per_split, int* __restrict__ status) {
  using L = SmallSmem<MP, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  float* partial = reinterpret_cast<float*>(smem + L::PARTIAL_OFFSET);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* accum = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * TC_BM;
  const int splits = gridDim.y;
  const int rank = blockIdx.y;  // cluster = (1, splits, 1): the rank inside the cluster
  const int num_kb = (K + TC_BK - 1) / TC_BK;
  const int kb_lo = rank * kb_per_split;
  const int kb_hi = kb_lo + kb_per_split < num_kb ? kb_lo + kb_per_split : num_kb;
  const int my_kb = kb_hi > kb_lo ? kb_hi - kb_lo : 0;
  constexpr uint32_t TMEM_COLS = MP < 32 ? 32 : MP;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum, 1);
    *failed = 0;
    mbar_fence_init();
    tma_prefetch_map(&map_w);
    tma_prefetch_map(&map_a);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_launch_dependents();
  // this thread's output column and its bias: a weight, so fetched before any wait
  const int t = threadIdx.x;
  const int n = n0 + t;
  const float b = (bias != nullptr && n < N) ? __ldg(bias + n) : 0.f;
  int issued = 0;
  if (warp == 0 && lane == 0) {
    // the weight tiles of the first stages start before the kernel ahead has finished
    const int ahead = my_kb < STAGES ? my_kb : STAGES;
    for (int i = 0; i < ahead; ++i) {
      uint8_t* w_tile = smem + i * L::STAGE_BYTES;
      mbar_expect_tx(&full[i], L::STAGE_BYTES);
      tma_load_2d(w_tile, &map_w, &full[i], (kb_lo + i) * TC_BK, n0);
    }
    pdl_wait();
    for (int i = 0; i < my_kb; ++i) {
      const int s = i % STAGES;
      uint8_t* w_tile = smem + s * L::STAGE_BYTES;
      if (i >= STAGES) {
        if (!mbar_wait(&empty[s], ((i / STAGES) & 1) ^ 1)) {
          *failed = 1;
          break;
        }
        mbar_expect_tx(&full[s], L::STAGE_BYTES);
        tma_load_2d(w_tile, &map_w, &full[s], (kb_lo + i) * TC_BK, n0);
      }
      tma_load_2d(w_tile + L::W_BYTES, &map_a, &full[s], (kb_lo + i) * TC_BK, 0);
      issued = i + 1;
    }
  }
  if (warp == 1 && lane == 0) {
    constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, MP);
    bool ok = true;
    for (int i = 0; i < my_kb; ++i) {
      const int s = i % STAGES;
      if (!mbar_wait(&full[s], (i / STAGES) & 1)) {
        *failed = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      const uint8_t* w_tile = smem + s * L::STAGE_BYTES;
      const uint8_t* a_tile = w_tile + L::W_BYTES;
#pragma unroll
      for (int k = 0; k < TC_BK / 16; ++k) {
        umma_f16(tmem_base, umma_desc_k128(w_tile, k * 32), umma_desc_k128(a_tile, k * 32),
                 idesc, (i | k) != 0);
      }
      umma_commit(&empty[s]);
    }
    if (ok && my_kb > 0) umma_commit(accum);
  }
  __syncwarp();
  pdl_wait();
  // The residual rows this CTA will add to (its share of the rows after a K split, when that
  // is at most 8): requested now, so that they arrive while the MMAs finish instead of
  // after the reduction.
  const int cols = MP / splits;  // the host picks splits that divide MP
  const bool early_rows = mode == OUT_RESIDUAL_F32 && splits > 1 && cols <= 8;
  float old_row[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int m = rank * cols + j;
    old_row[j] = (early_rows && j < cols && m < M && n < N)
                     ? reinterpret_cast<const float*>(out)[(size_t)m * ldo + n] : 0.f;
  }
  bool have = true;
  if (my_kb > 0) {
    have = mbar_wait(accum, 0);
    if (!have) *failed = 1;
  }
  tc_fence_after();

  // this CTA's partial sums: thread t holds output column n0 + t for every padded row
  if (splits == 1) {
    if (have && *failed == 0) {
#pragma unroll
      for (int c = 0; c < MP / 16; ++c) {
        uint32_t raw[16];
        tmem_ld_32x16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(c * 16), raw);
        tmem_ld_wait();
        if (n < N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = c * 16 + j;
            if (m < M) store_output(out, ldo, m, n, __uint_as_float(raw[j]) + b, mode, act);
          }
        }
        __syncwarp();
      }
    }
  } else {
#pragma unroll
    for (int c = 0; c < MP / 16; ++c) {
      uint32_t raw[16];
      if (my_kb > 0 && have) {
        tmem_ld_32x16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(c * 16), raw);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) raw[j] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) partial[(c * 16 + j) * TC_BM + t] = __uint_as_float(raw[j]);
      __syncwarp();
    }
    __syncthreads();
    cluster_sync_all();
    if (*failed == 0 && n < N) {
      // remote addresses of this thread's column in every peer's tile
      uint32_t peer_base[8];
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        peer_base[p] = p < splits ? peer_address(partial + t, (uint32_t)p) : 0u;
      }
      // four rows at a time: all of their loads are issued before the first sum, so the
      // distributed-shared-memory latency is paid once per group, not once per load
      auto group = [&](int j0, const float* old4) {
        float v[4][8];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int m = rank * cols + j0 + jj;
#pragma unroll
          for (int p = 0; p < 8; ++p) {
            v[jj][p] = (p < splits && j0 + jj < cols && m < M)
                           ? ld_cluster_f32(peer_base[p] + (uint32_t)(m * TC_BM * 4)) : 0.f;
          }
        }
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int m = rank * cols + j0 + jj;
          if (j0 + jj < cols && m < M) {
            float sum = v[jj][0];
#pragma unroll
            for (int p = 1; p < 8; ++p) {
              if (p < splits) sum += v[jj][p];
            }
            if (old4 != nullptr) {
              reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = old4[jj] + (sum + b);
            } else {
              store_output(out, ldo, m, n, sum + b, mode, act);
            }
          }
        }
      };
      if (early_rows) {
        group(0, old_row);
        if (cols > 4) group(4, old_row + 4);
      } else {
        for (int j0 = 0; j0 < cols; j0 += 4) group(j0, nullptr);
      }
    }
    cluster_sync_all();  // nobody leaves while a peer may still read its tile
  }

  tc_fence_before();
  __syncthreads();
  if (*failed != 0) {
    if (warp == 0 && lane == 0) {
      for (int i = issued > STAGES ? issued - STAGES : 0; i < issued; ++i) {
        mbar_wait(&full[i % STAGES], (i / STAGES) & 1);
      }
      atomicExch(status, AYK_WAIT_TIMEOUT);
    }
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace ayk

#include "gemm_stream.cuh"

namespace ayk {

// Tensor maps are cached by what they describe: weights are static and activations live in
// persistent buffers, so a serving process encodes each map once.
struct MapKey {
  const void* base;
  uint64_t rows, cols, ld;
  uint32_t box_rows, elem_bytes;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld &&
           box_rows == o.box_rows && elem_bytes == o.elem_bytes;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.base;
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.cols;
    h = h * 1000003u ^ k.ld;
    h = h * 1000003u ^ k.box_rows;
    h = h * 1000003u ^ k.elem_bytes;
    return h;
  }
};

static int cached_map(const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, CUtensorMap* out, int elem_bytes = 2) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  std::lock_guard<std::mutex> lock(mu);
  const MapKey key{base, rows, cols, ld, box_rows, (uint32_t)elem_bytes};
  auto it = cache.find(key);
  if (it == cache.end()) {
    CUtensorMap map;
    const int r = make_map_128b(&map, base, rows, cols, ld, box_rows, elem_bytes);
    if (r != AYK_OK) return r;
    if (cache.size() > 4096) cache.clear();
    it = cache.emplace(key, map).first;
  }
  *out = it->second;
  return AYK_OK;
}

// The output's map for the epilogue's TMA stores (boxes of 32 rows x 128 bytes), when its base
// and row stride allow one; otherwise `vec_ok` = 0 and the kernel stores row by row.
static int output_map(void* out, int ldo, int M, int N, int mode, const CUtensorMap& fallback,
                      CUtensorMap* map_out, int* vec_ok) {
  const size_t elem = mode == OUT_BF16 ? 2 : 4;
  *vec_ok = (((uintptr_t)out % 16) == 0 && ((size_t)ldo * elem) % 16 == 0) ? 1 : 0;
  *map_out = fallback;  // unused without vec_ok
  if (!*vec_ok) return AYK_OK;
  return cached_map(out, (uint64_t)M, (uint64_t)N, (uint64_t)ldo, 32, map_out, (int)elem);
}

template <int BN, int STAGES, bool SCATTER = false>
int launch_gemm_tc(const void* a, int lda, const void* w, int ldw, const float* bias, void* out,
                   int ldo, int M, int N, int K, int act, int mode, int* status,
                   cudaStream_t stream, const KvScatter& kv = KvScatter{}) {
  using L = TcSmem<BN, STAGES>;
  CUtensorMap map_a, map_w;
  int r = cached_map(a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, TC_BM, &map_a);
  if (r != AYK_OK) return r;
  r = cached_map(w, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, BN, &map_w);
  if (r != AYK_OK) return r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, SCATTER>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYNAMIC);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap map_out;
  int vec_ok = 0;
  r = output_map(out, ldo, M, N, mode, map_a, &map_out, &vec_ok);
  if (r != AYK_OK) return r;
  const long long gy = (M + TC_BM - 1) / TC_BM;
  if (gy > 65535) return AYK_TOO_LARGE;
  dim3 grid((N + BN - 1) / BN, (unsigned)gy);
  if (SCATTER && !vec_ok) return AYK_BAD_ALIGNMENT;  // (the caller checks before it asks)
  return launch_kernel(gemm_tc_kernel<BN, STAGES, SCATTER>, grid, dim3(128), L::DYNAMIC, stream,
                       1, map_a, map_w, map_out, bias, out, ldo, M, N, K, act, mode, vec_ok,
                       status, kv);
}

template <int BN, int STAGES, bool SCATTER = false>
int launch_gemm_tc_persistent(const void* a, int lda, const void* w, int ldw, const float* bias,
                              void* out, int ldo, int M, int N, int K, int act, int mode,
                              int* status, cudaStream_t stream,
                              const KvScatter& kv = KvScatter{}) {
  using L = PersistentSmem<BN, STAGES>;
  CUtensorMap map_a, map_w;
  int r = cached_map(a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, TC_BM, &map_a);
  if (r != AYK_OK) return r;
  r = cached_map(w, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, BN, &map_w);
  if (r != AYK_OK) return r;
  static bool configured = false;
  static int num_sms = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, STAGES, SCATTER>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYNAMIC);
    if (e != cudaSuccess) return (int)e;
    int device = 0;
    e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    e = cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap map_out;
  int vec_ok = 0;
  r = output_map(out, ldo, M, N, mode, map_a, &map_out, &vec_ok);
  if (r != AYK_OK) return r;
  const long long tiles = (long long)((M + TC_BM - 1) / TC_BM) * ((N + BN - 1) / BN);
  if (tiles > 0x7fffffffLL) return AYK_TOO_LARGE;
  const int grid = tiles < num_sms ? (int)tiles : num_sms;
  if (SCATTER && !vec_ok) return AYK_BAD_ALIGNMENT;  // (the caller checks before it asks)
  return launch_kernel(gemm_tc_persistent_kernel<BN, STAGES, SCATTER>, dim3(grid), dim3(192),
                       L::DYNAMIC, stream, 1, map_a, map_w, map_out, bias, out, ldo, M, N, K, act,
                       mode, vec_ok, status, kv);
}

template <int BN, int STAGES>
int launch_gemm_tc_pair(const void* a, int lda, const void* w, int ldw, const float* bias,
                        void* out, int ldo, int M, int N, int K, int act, int mode, int* status,
                        cudaStream_t stream) {
  using L = PairSmem<BN, STAGES>;
  CUtensorMap map_a, map_w;
  int r = cached_map(a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, TC_BM, &map_a);
  if (r != AYK_OK) return r;
  r = cached_map(w, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, BN / 2, &map_w);
  if (r != AYK_OK) return r;
  static bool configured = false;
  static int num_sms = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<BN, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYNAMIC);
    if (e != cudaSuccess) return (int)e;
    int device = 0;
    e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    e = cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap map_out;
  int vec_ok = 0;
  r = output_map(out, ldo, M, N, mode, map_a, &map_out, &vec_ok);
  if (r != AYK_OK) return r;
  const long long tiles = (long long)((M + 2 * TC_BM - 1) / (2 * TC_BM)) * ((N + BN - 1) / BN);
  if (tiles > 0x7fffffffLL) return AYK_TOO_LARGE;
  const int pairs = tiles < num_sms / 2 ? (int)tiles : num_sms / 2;
  return launch_kernel_x(gemm_tc_pair_kernel<BN, STAGES>, dim3(2 * pairs), dim3(192), L::DYNAMIC,
                         stream, 2, map_a, map_w, map_out, bias, out, ldo, M, N, K, act, mode,
                         vec_ok, status);
}

// K splits for a product of more than 64 rows whose 128 x 128 tiles would leave most of the
// device idle and whose K is long: the largest of 4, 2 that leaves every CTA of the cluster
// at least SK_MIN_BLOCKS blocks of K and keeps all CTAs resident at once (one per SM: the
// exchange buffer takes the room of a second); 1 when the plain kernels are the better
// choice. Measured at 288 rows (GPT-2 large's sizes): K = 5120 over 4 CTAs 23 against 33
// microseconds; K = 1280 over 4 CTAs 19 against 17, the exchange costs more than it saves.
constexpr int SK_MIN_BLOCKS = 16;
inline int splitk_ranks(int M, int N, int K) {
  const long long tiles = (long long)((M + TC_BM - 1) / TC_BM) * ((N + SK_BN - 1) / SK_BN);
  const int num_kb = (K + TC_BK - 1) / TC_BK;
  const int sms = sm_count();
  for (int r : {4, 2}) {
    const int per = (num_kb + r - 1) / r;
    if (per >= SK_MIN_BLOCKS && per * (r - 1) < num_kb && tiles * r <= sms) return r;
  }
  return 1;
}

template <int STAGES, bool SCATTER>
int launch_gemm_tc_splitk(const void* a, int lda, const void* w, int ldw, const float* bias,
                          void* out, int ldo, int M, int N, int K, int act, int mode, int ranks,
                          int* status, cudaStream_t stream, const KvScatter& kv = KvScatter{}) {
  using L = SplitKSmem<STAGES>;
  if (ranks != 2 && ranks != 4) return AYK_BAD_ARGUMENT;
  const int num_kb = (K + TC_BK - 1) / TC_BK;
  const int per = (num_kb + ranks - 1) / ranks;
  if (per * (ranks - 1) >= num_kb) return AYK_BAD_ARGUMENT;  // a rank without a block of K
  CUtensorMap map_a, map_w;
  int r = cached_map(a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, TC_BM, &map_a);
  if (r != AYK_OK) return r;
  r = cached_map(w, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, SK_BN, &map_w);
  if (r != AYK_OK) return r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_splitk_kernel<STAGES, SCATTER>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYNAMIC);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const size_t elem = mode == OUT_BF16 ? 2 : 4;
  const int vec_ok = (((uintptr_t)out % 16) == 0 && ((size_t)ldo * elem) % 16 == 0) ? 1 : 0;
  const long long gz = (M + TC_BM - 1) / TC_BM;
  if (gz > 65535) return AYK_TOO_LARGE;
  dim3 grid((N + SK_BN - 1) / SK_BN, ranks, (unsigned)gz);
  return launch_kernel(gemm_tc_splitk_kernel<STAGES, SCATTER>, grid, dim3(128), L::DYNAMIC,
                       stream, ranks, map_a, map_w, bias, out, ldo, M, N, K, act, mode, vec_ok,
                       per, status, kv);
}

template <int MP, int STAGES>
int launch_gemm_tc_small(const void* a, int lda, const void* w, int ldw, const float* bias,
                         void* out, int ldo, int M, int N, int K, int act, int mode, int splits,
                         int* status, cudaStream_t stream) {
  using L = SmallSmem<MP, STAGES>;
  CUtensorMap map_a, map_w;
  int r = cached_map(w, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, TC_BM, &map_w);
  if (r != AYK_OK) return r;
  r = cached_map(a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, MP, &map_a);
  if (r != AYK_OK) return r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_small_kernel<MP, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYNAMIC);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int num_kb = (K + TC_BK - 1) / TC_BK;
  if (splits < 1) splits = 1;
  while (splits > 1 && (splits > num_kb || splits > 8 || MP % splits)) splits >>= 1;
  const int kb_per_split = (num_kb + splits - 1) / splits;
  return launch_kernel(gemm_tc_small_kernel<MP, STAGES>,
                       dim3((N + TC_BM - 1) / TC_BM, splits, 1), dim3(128), L::DYNAMIC, stream,
                       splits, map_w, map_a, bias, out, ldo, M, N, K, act, mode, kb_per_split,
                       status);
}

inline int pick_splits(int tile_n, int N, int M) {
  // -1: choose; -2, -4, -8: that many K splits; -100: one split
  if (tile_n == -100) return 1;
  if (tile_n != -1) return -tile_n;
  const int tiles = (N + TC_BM - 1) / TC_BM;
  // More than 16 rows: a CTA takes most of an SM's shared memory and a cluster lies inside
  // one GPC, so a GPC of 18 SMs holds two clusters of eight or four of four at a time, and
  // clusters beyond one round wait for a whole round. Eight splits while the tiles are at
  // most 16, four up to 32, else none: the reduction (each rank fetches its rows of every
  // peer's tile) costs more the fewer ranks share the rows, which is why two splits lose to
  // none. Measured in a chain of such products at 64 rows, microseconds with 1 / 2 / 4 / 8
  // splits: GPT-2 small's QKV (18 tiles, K 768) 7.9 / 10.3 / 7.6 / 12.1 and its output
  // projection (6 tiles) 16.6 / 13.7 / 9.2 / 5.7; GPT-2 large's QKV at 32 rows (30 tiles)
  // 8.6 / 8.9 / 7.4 / 12.3 and its feed-forward (40 tiles) 8.7 / 9.3 / 13.1 / 17.6; GPT-2
  // XL's QKV (38 tiles) 11.4 / 13.1 / 17.3 / 21.1 and its output projection (13 tiles) 37 /
  // 24 / 14 / 7.6.
  if (M > 16) return tiles <= 16 ? 8 : (tiles <= 32 ? 4 : 1);
  // as many K splits as still leave two CTAs' worth of tiles per SM
  int splits = 1;
  while (splits < 8 && tiles * splits * 2 <= 2 * sm_count()) splits <<= 1;
  return splits;
}

// The tile code (see ayk_gemm_bf16_tc) for a product with more than 64 rows.
inline int choose_tile(int M, int N) {
  // measured at GPT-2 XL's shapes: with more 128 x 256 tiles than SMs the persistent kernel
  // wins (its epilogues hide under the next tile's main loop); with fewer, one tile per CTA
  const int num_sms = sm_count();
  // tile width 256, 192 or 128: the one with the least (rounds over the SMs) x (time of a
  // round). Measured at K = 1600: a round of 256-wide tiles takes only 7 % longer than one
  // of 192-wide tiles (9.8 against 9.2 microseconds), i.e. about (width + 768) units, so
  // the number of rounds decides and the width breaks ties. One tile per CTA while
  // everything fits one round, else the persistent kernel.
  const long long tiles_m = (M + TC_BM - 1) / TC_BM;
  long long best_cost = -1;
  int best_bn = 256;
  for (int bn : {256, 192, 128}) {
    const long long tiles = tiles_m * ((N + bn - 1) / bn);
    const long long cost = ((tiles + num_sms - 1) / num_sms) * (bn + 768);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best_bn = bn;
    }
  }
  const long long tiles = tiles_m * ((N + best_bn - 1) / best_bn);
  return tiles > num_sms ? 1000 + best_bn : best_bn;
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

namespace ayk {
// Products of up to this many rows go to gemm_stream_kernel when nothing else is asked for.
inline int& stream_rows() {
  static int rows = ST_MAX_ROWS;
  return rows;
}
}  // namespace ayk
// For measurements: 0 sends every product of at most 64 rows to the cluster split-K kernel.
AYK_API void ayk_set_stream_rows(int rows) {
  ayk::stream_rows() = rows < 0 ? 0 : (rows > ayk::ST_MAX_ROWS ? ayk::ST_MAX_ROWS : rows);
}

// mode: 0 = bf16 out with activation, 1 = fp32 out with activation, 2 = fp32 out += (residual).
// tile_n: 0 = choose; 64, 128, 192, 256 = one tile of that width per CTA; 1128, 1192,
// 1256 = the persistent kernel with tiles 128, 192 or 256 wide; 2192, 2256 = the persistent
// kernel for CTA pairs (256-row tiles, 192 or 256 wide; measured level with 1192 / 1256 at
// GPT-2 XL's shapes, so the choice never picks it); negative = the few-rows kernel (see
// pick_splits; -200 = the kernel for at most 16 rows that holds its weights on chip before the
// rows arrive, gemm_stream.cuh; -201 / -202 = the same with one / two column tiles per CTA);
// 3002, 3004 = 128 x 128 tiles with K split over a cluster of 2 or 4 CTAs (chosen for a few
// hundred rows, where whole tiles would leave most SMs idle). `status` is one device int that a CTA sets to AYK_WAIT_TIMEOUT if a wait ran
// out; the host reads it when it checks a step.
AYK_API int ayk_gemm_bf16_tc(const void* a, int lda, const void* w, int ldw, const float* bias,
                             void* out, int ldo, int M, int N, int K, int act, int mode,
                             int tile_n, int* status, void* stream) {
  using namespace ayk;
  if (M == 0 || N == 0) return AYK_OK;
  if (M < 0 || N < 0 || K < 1 || lda < K || ldw < K || ldo < N || status == nullptr) {
    return AYK_BAD_ARGUMENT;
  }
  if (mode < OUT_BF16 || mode > OUT_RESIDUAL_F32 || act < ACT_NONE || act > ACT_GELU_ERF ||
      (mode == OUT_RESIDUAL_F32 && act != ACT_NONE)) {
    return AYK_BAD_ARGUMENT;
  }
  if (((uintptr_t)a % 16) || ((uintptr_t)w % 16) || (lda % 8) || (ldw % 8)) {
    return AYK_BAD_ALIGNMENT;
  }
  cudaStream_t s = (cudaStream_t)stream;
  // at most 16 rows: the kernel that holds its weights on chip; with more than 8 rows (two
  // row tiles, one after the other) only while its CTAs fit the SMs in one round (the head
  // of GPT-2 XL at 16 rows: 43 microseconds against 33.5 with the cluster split-K kernel)
  if (tile_n == 0 && M <= stream_rows() && stream_splits(M, K) > 0 &&
      (M <= 8 || stream_one_round(N))) {
    tile_n = -200;
  }
  if (tile_n <= -200 && tile_n >= -202) {
    const int splits = stream_splits(M, K);
    if (splits == 0) return AYK_BAD_ARGUMENT;
    return launch_gemm_stream(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode, splits,
                              tile_n == -200 ? -1 : (tile_n == -202 ? 1 : 0), s);
  }
  // 33 to 64 rows of a product so wide that the weight-streaming kernel would run it without
  // a K split (more than 32 tiles of 128 columns), while its 64-column tiles are still one
  // round: the rows as the 128-row operand and one 64-column tile per CTA, which has twice
  // the CTAs and needs no cluster. Measured, a decode step of 64 requests with and without
  // this choice: GPT-2 XL 4.22 against 4.58 ms, GPT-2 large 3.02 against 3.18; of 48 requests
  // 3.78 against 4.18 and 2.40 against 2.54, of 36 requests (GPT-2 XL) 3.38 against 3.69.
  // Where the weight-streaming kernel splits K in four (GPT-2 small and medium: at most 32
  // tiles) it stays ahead (0.77 against 0.79 ms, 1.56 against 1.60), and up to 32 rows, where
  // its rows operand is 32 wide, everywhere (GPT-2 XL's QKV at 32 rows in a chain: 9.9
  // against 10.6 us, its feed-forward 10.3 against 12.3).
  if (tile_n == 0 && M > 32 && M <= 64 && (N + TC_BM - 1) / TC_BM > 32 &&
      (N + 63) / 64 <= sm_count()) {
    tile_n = 64;
  }
  if (tile_n == 0 && M <= 64) tile_n = -1;  // few rows: the weight-streaming kernel
  if (tile_n < 0) {
    if (M > 64) return AYK_BAD_ARGUMENT;
    const int splits = pick_splits(tile_n, N, M);
    if (M <= 16) {
      return launch_gemm_tc_small<16, 5>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode,
                                         splits, status, s);
    }
    if (M <= 32) {
      return launch_gemm_tc_small<32, 6>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode,
                                         splits, status, s);
    }
    return launch_gemm_tc_small<64, 6>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode,
                                       splits, status, s);
  }
  if (tile_n == 0) {
    const int ranks = splitk_ranks(M, N, K);
    if (ranks > 1) tile_n = 3000 + ranks;
  }
  if (tile_n == 3002 || tile_n == 3004) {
    return launch_gemm_tc_splitk<4, false>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode,
                                           tile_n - 3000, status, s);
  }
  if (tile_n == 0) tile_n = choose_tile(M, N);
  switch (tile_n) {
    case 192:
      return launch_gemm_tc<192, 5>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode, status, s);
    case 1192:
      return launch_gemm_tc_persistent<192, 5>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode,
                                               status, s);
    case 1128:
      return launch_gemm_tc_persistent<128, 6>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode,
                                               status, s);
    case 1256:
      return launch_gemm_tc_persistent<256, 4>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode,
                                               status, s);
    case 2192:
      return launch_gemm_tc_pair<192, 7>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode,
                                         status, s);
    case 2256:
      return launch_gemm_tc_pair<256, 6>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode,
                                         status, s);
    case 64:
      return launch_gemm_tc<64, 8>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode, status, s);
    case 128:
      return launch_gemm_tc<128, 6>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode, status, s);
    case 256:
      return launch_gemm_tc<256, 4>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode, status, s);
    default:
      return AYK_BAD_ARGUMENT;
  }
}

// The fused query/key/value projection of a step of more than 64 rows: bf16 a w^T + bias as
// above, of which the query columns go to `out` and the key and value columns (from q_width
// on: kv_width of keys, then of values) of every row m go to the cache at slot slots[m] (see
// KvScatter; a negative slot stores nothing) and *not* to `out`: the attention kernels for
// prompt portions read them from the cache. Returns AYK_OK when it ran; AYK_NOT_TAKEN when this product
// cannot carry the store (few rows, a head size that is no multiple of 32, a query width that
// is no multiple of 64, an output TMA cannot write): nothing ran then and the caller does the
// product and the store on their own.
AYK_API int ayk_gemm_bf16_tc_kv(const void* a, int lda, const void* w, int ldw,
                                const float* bias, void* out, int ldo, int M, int N, int K,
                                const int* slots, void* k_pages, void* v_pages, int q_width,
                                int kv_width, int num_kv_heads, int head_dim, int page_size,
                                int* status, void* stream) {
  using namespace ayk;
  if (M < 0 || N < 1 || K < 1 || lda < K || ldw < K || ldo < N || status == nullptr ||
      slots == nullptr || k_pages == nullptr || v_pages == nullptr || num_kv_heads < 1 ||
      page_size < 1 || head_dim < 1 || kv_width != num_kv_heads * head_dim ||
      N != q_width + 2 * kv_width) {
    return AYK_BAD_ARGUMENT;
  }
  if (M <= 64 || head_dim % 32 || q_width % 64 || ((uintptr_t)a % 16) || ((uintptr_t)w % 16) ||
      (lda % 8) || (ldw % 8) || ((uintptr_t)out % 16) || (ldo % 8) ||
      ((uintptr_t)k_pages % 16) || ((uintptr_t)v_pages % 16)) {
    return AYK_NOT_TAKEN;
  }
  const KvScatter kv{slots, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, q_width, kv_width,
                     num_kv_heads, head_dim, page_size};
  cudaStream_t s = (cudaStream_t)stream;
  const int ranks = splitk_ranks(M, N, K);
  if (ranks > 1) {
    return launch_gemm_tc_splitk<4, true>(a, lda, w, ldw, bias, out, ldo, M, N, K, ACT_NONE,
                                          OUT_BF16, ranks, status, s, kv);
  }
  switch (choose_tile(M, N)) {
    case 128:
      return launch_gemm_tc<128, 6, true>(a, lda, w, ldw, bias, out, ldo, M, N, K, ACT_NONE,
                                          OUT_BF16, status, s, kv);
    case 192:
      return launch_gemm_tc<192, 5, true>(a, lda, w, ldw, bias, out, ldo, M, N, K, ACT_NONE,
                                          OUT_BF16, status, s, kv);
    case 256:
      return launch_gemm_tc<256, 4, true>(a, lda, w, ldw, bias, out, ldo, M, N, K, ACT_NONE,
                                          OUT_BF16, status, s, kv);
    case 1128:
      return launch_gemm_tc_persistent<128, 6, true>(a, lda, w, ldw, bias, out, ldo, M, N, K,
                                                     ACT_NONE, OUT_BF16, status, s, kv);
    case 1192:
      return launch_gemm_tc_persistent<192, 5, true>(a, lda, w, ldw, bias, out, ldo, M, N, K,
                                                     ACT_NONE, OUT_BF16, status, s, kv);
    case 1256:
      return launch_gemm_tc_persistent<256, 4, true>(a, lda, w, ldw, bias, out, ldo, M, N, K,
                                                     ACT_NONE, OUT_BF16, status, s, kv);
    default:
      return AYK_NOT_TAKEN;
  }
}
