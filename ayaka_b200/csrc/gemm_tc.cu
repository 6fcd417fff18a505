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

template <int BN, int STAGES>
struct TcSmem {
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = TC_A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  // full[STAGES], empty[STAGES], accum, then the tmem slot and the failure flag
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 1) * 8 + 16;
  static constexpr int DYNAMIC = TOTAL + 1024;  // room to align the base to 1024 bytes
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(128)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const float* __restrict__ bias, void* __restrict__ out, int ldo, int M, int N,
               int K, int act, int mode, int vec_ok, int* __restrict__ status) {
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
  pdl_wait();
  bool have = mbar_wait(accum, 0);
  if (!have) *failed = 1;
  tc_fence_after();
  if (have && *failed == 0) {
    const int m = m0 + warp * 32 + lane;
    const bool row_ok = m < M;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      const int n = n0 + c * 32;
      if (n >= N) break;  // uniform over the CTA
      uint32_t raw[32];
      tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(c * 32), raw);
      tmem_ld_wait();
      if (row_ok) {
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
          for (int j = 0; j < 32 && n + j < N; ++j) dst[j] = __float2bfloat16_rn(v[j]);
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
          for (int j = 0; j < 32 && n + j < N; ++j) {
            dst[j] = mode == OUT_RESIDUAL_F32 ? dst[j] + v[j] : v[j];
          }
        }
      }
      }  // row_ok
      __syncwarp();  // the next tcgen05.ld needs the whole warp
    }
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
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], then the tmem slot and the flag
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16;
  static constexpr int DYNAMIC = TOTAL + 1024;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(192)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                          const __grid_constant__ CUtensorMap map_w,
                          const float* __restrict__ bias, void* __restrict__ out, int ldo, int M,
                          int N, int K, int act, int mode, int vec_ok,
                          int* __restrict__ status) {
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
      bool have = true;
      if (lane == 0) have = mbar_wait(&acc_full[buf], (local >> 1) & 1);
      have = __shfl_sync(0xffffffffu, have, 0);
      if (!have || *failed != 0) {
        if (lane == 0) *failed = 1;
        break;
      }
      tc_fence_after();
      const int m = m0 + quarter * 32 + lane;
      const bool row_ok = m < M;
      const uint32_t acc = tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int n = n0 + c * 32;
        if (n >= N) break;  // uniform over the warp
        uint32_t raw[32];
        tmem_ld_32x32(acc + (uint32_t)(c * 32), raw);
        tmem_ld_wait();
        if (row_ok) {
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
              for (int j = 0; j < 32 && n + j < N; ++j) dst[j] = __float2bfloat16_rn(v[j]);
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
              for (int j = 0; j < 32 && n + j < N; ++j) {
                dst[j] = mode == OUT_RESIDUAL_F32 ? dst[j] + v[j] : v[j];
              }
            }
          }
        }
        __syncwarp();  // the next tcgen05.ld needs the whole warp
      }
      // this warp has read its lanes of the accumulator: hand it back
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
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
        __float2bfloat16_rn(activate(v, act));
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
  bool have = true;
  if (my_kb > 0) {
    have = mbar_wait(accum, 0);
    if (!have) *failed = 1;
  }
  tc_fence_after();

  // this CTA's partial sums: thread t holds output column n0 + t for every padded row
  const int t = threadIdx.x;
  const int n = n0 + t;
  if (splits == 1) {
    if (have && *failed == 0) {
#pragma unroll
      for (int c = 0; c < MP / 16; ++c) {
        uint32_t raw[16];
        tmem_ld_32x16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(c * 16), raw);
        tmem_ld_wait();
        if (n < N) {
          const float b = bias != nullptr ? __ldg(bias + n) : 0.f;
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
    const int cols = MP / splits;  // the host picks splits that divide MP
    if (*failed == 0 && n < N) {
      const float b = bias != nullptr ? __ldg(bias + n) : 0.f;
      // remote addresses of this thread's column in every peer's tile
      uint32_t peer_base[8];
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        peer_base[p] = p < splits ? peer_address(partial + t, (uint32_t)p) : 0u;
      }
      // four rows at a time: all of their loads are issued before the first sum, so the
      // distributed-shared-memory latency is paid once per group, not once per load
      for (int j0 = 0; j0 < cols; j0 += 4) {
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
            store_output(out, ldo, m, n, sum + b, mode, act);
          }
        }
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

// Tensor maps are cached by what they describe: weights are static and activations live in
// persistent buffers, so a serving process encodes each map once.
struct MapKey {
  const void* base;
  uint64_t rows, cols, ld;
  uint32_t box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld &&
           box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.base;
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.cols;
    h = h * 1000003u ^ k.ld;
    h = h * 1000003u ^ k.box_rows;
    return h;
  }
};

static int cached_map(const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  std::lock_guard<std::mutex> lock(mu);
  const MapKey key{base, rows, cols, ld, box_rows};
  auto it = cache.find(key);
  if (it == cache.end()) {
    CUtensorMap map;
    const int r = make_map_bf16_k64(&map, base, rows, cols, ld, box_rows);
    if (r != AYK_OK) return r;
    if (cache.size() > 4096) cache.clear();
    it = cache.emplace(key, map).first;
  }
  *out = it->second;
  return AYK_OK;
}

template <int BN, int STAGES>
int launch_gemm_tc(const void* a, int lda, const void* w, int ldw, const float* bias, void* out,
                   int ldo, int M, int N, int K, int act, int mode, int* status,
                   cudaStream_t stream) {
  using L = TcSmem<BN, STAGES>;
  CUtensorMap map_a, map_w;
  int r = cached_map(a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, TC_BM, &map_a);
  if (r != AYK_OK) return r;
  r = cached_map(w, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, BN, &map_w);
  if (r != AYK_OK) return r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYNAMIC);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const size_t elem = mode == OUT_BF16 ? 2 : 4;
  const int vec_ok = (((uintptr_t)out % 16) == 0 && ((size_t)ldo * elem) % 16 == 0) ? 1 : 0;
  const long long gy = (M + TC_BM - 1) / TC_BM;
  if (gy > 65535) return AYK_TOO_LARGE;
  dim3 grid((N + BN - 1) / BN, (unsigned)gy);
  return launch_kernel(gemm_tc_kernel<BN, STAGES>, grid, dim3(128), L::DYNAMIC, stream, 1, map_a,
                       map_w, bias, out, ldo, M, N, K, act, mode, vec_ok, status);
}

template <int BN, int STAGES>
int launch_gemm_tc_persistent(const void* a, int lda, const void* w, int ldw, const float* bias,
                              void* out, int ldo, int M, int N, int K, int act, int mode,
                              int* status, cudaStream_t stream) {
  using L = PersistentSmem<BN, STAGES>;
  CUtensorMap map_a, map_w;
  int r = cached_map(a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, TC_BM, &map_a);
  if (r != AYK_OK) return r;
  r = cached_map(w, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, BN, &map_w);
  if (r != AYK_OK) return r;
  static bool configured = false;
  static int num_sms = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYNAMIC);
    if (e != cudaSuccess) return (int)e;
    int device = 0;
    e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    e = cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const size_t elem = mode == OUT_BF16 ? 2 : 4;
  const int vec_ok = (((uintptr_t)out % 16) == 0 && ((size_t)ldo * elem) % 16 == 0) ? 1 : 0;
  const long long tiles = (long long)((M + TC_BM - 1) / TC_BM) * ((N + BN - 1) / BN);
  if (tiles > 0x7fffffffLL) return AYK_TOO_LARGE;
  const int grid = tiles < num_sms ? (int)tiles : num_sms;
  return launch_kernel(gemm_tc_persistent_kernel<BN, STAGES>, dim3(grid), dim3(192), L::DYNAMIC,
                       stream, 1, map_a, map_w, bias, out, ldo, M, N, K, act, mode, vec_ok,
                       status);
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
  // measured on GPT-2 XL's shapes: with more than 32 rows the cluster reduction of a
  // [64, 128] tile costs more than it buys unless the tiles are very few
  if (M > 32) return tiles >= 32 ? 1 : 8;
  int splits = 1;
  while (splits < 8 && tiles * splits * 2 <= 296) splits <<= 1;
  return splits;
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

// mode: 0 = bf16 out with activation, 1 = fp32 out with activation, 2 = fp32 out += (residual).
// tile_n: 0 = choose; 32, 64, 128, 192, 256 = one tile of that width per CTA; 1128, 1192, 1256 = the
// persistent kernel with tiles 128, 192 or 256 wide; negative = the few-rows kernel (see below). `status` is one device int that a CTA sets to
// AYK_WAIT_TIMEOUT if a wait ran out; the host reads it when it checks a step.
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
    // measured at GPT-2 XL's shapes: with more 128 x 256 tiles than SMs the persistent kernel
    // wins (its epilogues hide under the next tile's main loop); with fewer, one tile per CTA
    static int num_sms = 0;
    if (num_sms == 0) {
      int device = 0;
      if (cudaGetDevice(&device) != cudaSuccess ||
          cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, device) !=
              cudaSuccess) {
        num_sms = 148;
      }
    }
    // tile width 256, 192 or 128: the one that needs the least (rounds over the SMs) x (work
    // of a tile); one tile per CTA while everything fits one round, else the persistent kernel
    const long long tiles_m = (M + TC_BM - 1) / TC_BM;
    long long best_cost = -1;
    int best_bn = 256;
    for (int bn : {256, 192, 128}) {
      const long long tiles = tiles_m * ((N + bn - 1) / bn);
      const long long cost = ((tiles + num_sms - 1) / num_sms) * bn;
      if (best_cost < 0 || cost < best_cost) {
        best_cost = cost;
        best_bn = bn;
      }
    }
    const long long tiles = tiles_m * ((N + best_bn - 1) / best_bn);
    tile_n = tiles > num_sms ? 1000 + best_bn : best_bn;
  }
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
    case 32:
      return launch_gemm_tc<32, 8>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode, status, s);
    case 64:
      return launch_gemm_tc<64, 4>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode, status, s);
    case 128:
      return launch_gemm_tc<128, 4>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode, status, s);
    case 256:
      return launch_gemm_tc<256, 4>(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode, status, s);
    default:
      return AYK_BAD_ARGUMENT;
  }
}
