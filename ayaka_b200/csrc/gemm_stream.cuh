// The product for at most 16 rows (a decode step of a few requests): C[M,N] = A[M,K] W[N,K]^T.
//
// Such a product is one pass over the weights and nothing else, and in a chain of kernels a
// layer long its time is the chain of dependent steps after the kernel ahead has finished,
// not the bytes. So this kernel does everything that does not depend on the rows *before*
// the dependency wait, and keeps what follows the wait as short as it can be:
//
//   before the wait   every thread copies the weights it will multiply, all of them, into
//                     shared-memory slots of its own with cp.async (up to 56 KB per column
//                     tile, about 220 KB per SM: the whole matrix of a GPT-2 XL product is in
//                     flight or on chip when the rows arrive); bias
//   after the wait    the rows' fragments straight from L1/L2 into registers (no staging, no
//                     barrier), the old values of a residual sum, cp.async.wait_group,
//                     mma.sync from the thread's own slots, a sum over the eight warps through
//                     shared memory in warp order, (K split over a cluster: the partial sums
//                     pushed into rank 0's shared memory, one cluster barrier,) epilogue, store.
//
// A CTA owns 16 output columns (32 as two tiles for wide products, see CT) and a range of K;
// its eight warps take the 32-wide steps of
// that range in turn (warp w: steps w, w + 8, ...). The tensor-core shape is m16n8k16 with the
// weights as the 16-row operand and eight rows of A as the 8-column one. A lane's 16-byte
// pieces are eight consecutive k of one weight row, used as the operands of two MMAs; the k
// order inside a step is permuted the same way for both operands, which a sum over k does not
// see. Nine to sixteen rows run as two row tiles, one after the other, over the same weights.
// This is the legacy tensor path on purpose: at 8 rows the arithmetic is 0.1 % of the time,
// and what counts is that a fragment needs no shared-memory layout, no descriptor and no
// barrier. Products of more rows go to the tcgen05 kernels.
//
// The order of the sums is fixed (steps of a warp in order, warps in order, cluster ranks in
// order) and does not depend on M or on which row of the step a token is.
#pragma once

#include "tc_common.cuh"

namespace ayk {

constexpr int ST_THREADS = 256;
constexpr int ST_WARPS = ST_THREADS / 32;
constexpr int ST_COLS = 16;        // output columns per column tile
constexpr int ST_STEP_K = 32;      // k per step
constexpr int ST_STEPS_PER_WARP = 7;
constexpr int ST_MAX_STEPS = ST_WARPS * ST_STEPS_PER_WARP;  // per CTA: 56 KB of weights
constexpr int ST_MAX_ROWS = 16;
constexpr int ST_RED_BYTES = ST_WARPS * 32 * 16;

__device__ __forceinline__ void cp_async_16_zfill(void* dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1,
                                               uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 16 bytes of the rows the kernel ahead wrote: an ordinary load after the dependency wait,
// cached in L1, where the CTAs of an SM (all of which read the same rows) find each other's.
// Measured in a decode layer of GPT-2 XL at 8 rows: 34.9 microseconds a layer against 37.4
// with loads that go to L2 every time (ld.global.cg).
__device__ __forceinline__ uint4 ld_rows_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.ca.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t address, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(address), "f"(v) : "memory");
}

// grid (ceil(N / (16 CT)), splits), cluster (1, splits): CTA (x, y) owns CT tiles of 16
// columns from column 16 CT x on and the steps y * steps_per_split .. of K. With CT = 2 (wide
// products, no split) a lane's row fragments serve two column tiles: half the loads of rows
// per byte of weights. Dynamic shared memory: CT * steps_per_split KB of weight slots, CT *
// ST_RED_BYTES for the sum over warps, and with a split splits * 1 KB where rank 0 receives
// the partial sums.
template <int CT>
__global__ void __launch_bounds__(ST_THREADS, 4 / CT)
gemm_stream_kernel(const __nv_bfloat16* __restrict__ a, int lda,
                   const __nv_bfloat16* __restrict__ w, int ldw, const float* __restrict__ bias,
                   void* __restrict__ out, int ldo, int M, int N, int K, int act, int mode,
                   int steps_per_split) {
  extern __shared__ __align__(16) uint8_t st_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int splits = gridDim.y;
  const int rank = blockIdx.y;
  const int n0 = blockIdx.x * (ST_COLS * CT);
  const int total_steps = (K + ST_STEP_K - 1) / ST_STEP_K;
  const int step_lo = rank * steps_per_split;
  const int step_hi = min(step_lo + steps_per_split, total_steps);
  const int my_steps = max(step_hi - step_lo, 0);

  uint4* slots = reinterpret_cast<uint4*>(st_smem);
  float* red = reinterpret_cast<float*>(st_smem + (size_t)steps_per_split * 1024 * CT);
  float* recv = red + CT * ST_RED_BYTES / 4;

  if (splits > 1) cluster_arrive();  // "this CTA runs": awaited before anyone writes to it

  // ---- everything that is a weight: requested now, whatever the kernel ahead is doing
#pragma unroll
  for (int ct = 0; ct < CT; ++ct) {
    const int row0 = n0 + ct * ST_COLS + g, row1 = row0 + 8;
    const __nv_bfloat16* src0 = w + (size_t)(row0 < N ? row0 : 0) * ldw;
    const __nv_bfloat16* src1 = w + (size_t)(row1 < N ? row1 : 0) * ldw;
#pragma unroll
    for (int j = 0; j < ST_STEPS_PER_WARP; ++j) {
      const int local = warp + ST_WARPS * j;
      if (local < my_steps) {
        const int k = (step_lo + local) * ST_STEP_K + 8 * q;
        const bool in_k = k < K;  // K is a multiple of 8: a piece is inside or outside
        uint4* slot = slots + ((size_t)local * CT + ct) * 64 + lane;
        cp_async_16_zfill(slot, in_k ? src0 + k : w, (in_k && row0 < N) ? 16u : 0u);
        cp_async_16_zfill(slot + 32, in_k ? src1 + k : w, (in_k && row1 < N) ? 16u : 0u);
      }
    }
  }
  pdl_launch_dependents();
  // the thread that writes output (row m, column n) of each tile of eight rows
  const int t = threadIdx.x;
  const int c = t & 15, m_in_tile = (t >> 4) & 7, tile_of_t = t >> 7;
  const int n = n0 + tile_of_t * ST_COLS + c;
  const bool writer = t < 128 * CT && rank == 0 && n < N;
  const float b = (writer && bias != nullptr) ? __ldg(bias + n) : 0.f;

  pdl_wait();

  const int row_tiles = (M + 7) >> 3;
  float old_value[2] = {0.f, 0.f};
  if (writer && mode == OUT_RESIDUAL_F32) {
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      const int m = mt * 8 + m_in_tile;
      if (mt < row_tiles && m < M) {
        old_value[mt] = __ldcg(reinterpret_cast<const float*>(out) + (size_t)m * ldo + n);
      }
    }
  }

  float total[2] = {0.f, 0.f};
  for (int mt = 0; mt < row_tiles; ++mt) {
    // the rows' fragments: lane (g, q) needs A[8 mt + g][k .. k + 8) of each of its steps
    uint4 x[ST_STEPS_PER_WARP];
    const int m_frag = mt * 8 + g;
    const __nv_bfloat16* a_row = a + (size_t)(m_frag < M ? m_frag : 0) * lda;
#pragma unroll
    for (int j = 0; j < ST_STEPS_PER_WARP; ++j) {
      const int local = warp + ST_WARPS * j;
      const int k = (step_lo + local) * ST_STEP_K + 8 * q;
      x[j] = (local < my_steps && k < K && m_frag < M)
                 ? ld_rows_16(a_row + k) : make_uint4(0u, 0u, 0u, 0u);
    }
    if (mt == 0) cp_async_commit_wait_all();
    float acc0[CT][4], acc1[CT][4];
#pragma unroll
    for (int ct = 0; ct < CT; ++ct) {
#pragma unroll
      for (int i = 0; i < 4; ++i) acc0[ct][i] = acc1[ct][i] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < ST_STEPS_PER_WARP; ++j) {
      const int local = warp + ST_WARPS * j;
      if (local < my_steps) {
#pragma unroll
        for (int ct = 0; ct < CT; ++ct) {
          const uint4 p0 = slots[((size_t)local * CT + ct) * 64 + lane];
          const uint4 p1 = slots[((size_t)local * CT + ct) * 64 + 32 + lane];
          mma_bf16_16816(acc0[ct], p0.x, p1.x, p0.y, p1.y, x[j].x, x[j].y);
          mma_bf16_16816(acc1[ct], p0.z, p1.z, p0.w, p1.w, x[j].z, x[j].w);
        }
      }
    }
    // lane (g, q) holds columns g and g + 8 of rows 2q and 2q + 1 of each column tile
    if (mt > 0) __syncthreads();  // the last tile's sums have been read
#pragma unroll
    for (int ct = 0; ct < CT; ++ct) {
      reinterpret_cast<float4*>(red)[(ct * ST_WARPS + warp) * 32 + lane] =
          make_float4(acc0[ct][0] + acc1[ct][0], acc0[ct][1] + acc1[ct][1],
                      acc0[ct][2] + acc1[ct][2], acc0[ct][3] + acc1[ct][3]);
    }
    __syncthreads();
    if (t < 128 * CT) {
      const int from_lane = 4 * (c & 7) + (m_in_tile >> 1);
      const int index = tile_of_t * (ST_WARPS * 128) + from_lane * 4 + (c >> 3) * 2 +
                        (m_in_tile & 1);
      float sum = red[index];
#pragma unroll
      for (int v = 1; v < ST_WARPS; ++v) sum += red[v * 128 + index];
      if (mt == 0) total[0] = sum; else total[1] = sum;
    }
  }

  if (CT == 1 && splits > 1) {
    cluster_wait();  // every CTA of the cluster has started
    if (t < 128) {
      const uint32_t mine = peer_address(recv + rank * 256 + t, 0u);
      st_cluster_f32(mine, total[0]);
      if (row_tiles > 1) st_cluster_f32(mine + 128 * 4, total[1]);
    }
    cluster_arrive();
    cluster_wait();
    if (writer) {
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        if (mt < row_tiles) {
          float sum = recv[mt * 128 + t];
          for (int r = 1; r < splits; ++r) sum += recv[r * 256 + mt * 128 + t];
          total[mt] = sum;
        }
      }
    }
  }
  if (writer) {
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      const int m = mt * 8 + m_in_tile;
      if (mt < row_tiles && m < M) {
        const float v = total[mt] + b;
        if (mode == OUT_RESIDUAL_F32) {
          reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = old_value[mt] + v;
        } else {
          store_output(out, ldo, m, n, v, mode, act);
        }
      }
    }
  }
}

// How many CTAs of a cluster share K so that each holds at most ST_MAX_STEPS steps: 1, 2, 4
// or 8; 0 when the product is not this kernel's (more than 16 rows, K no multiple of 8 or
// beyond 8 * 56 * 32).
inline int stream_splits(int M, int K) {
  if (M < 1 || M > ST_MAX_ROWS || K % 8 != 0) return 0;
  const int steps = (K + ST_STEP_K - 1) / ST_STEP_K;
  for (int splits = 1; splits <= 8; splits <<= 1) {
    if ((steps + splits - 1) / splits <= ST_MAX_STEPS) return splits;
  }
  return 0;
}

// From this many columns on, and while one column tile per CTA would still fit the SMs in
// one round (four CTAs each), a product without a K split runs with two column tiles per CTA:
// half the CTAs, twice the weights each (GPT-2 XL: the query/key/value projection and the
// feed-forward's first product; measured 34.2 against 34.9 microseconds a layer at 8 rows).
// Over several rounds the narrow CTAs win (the head, 50,257 columns: 29.7 against 30.8
// microseconds at 8 rows).
#ifndef AYK_STREAM_WIDE_FROM
#define AYK_STREAM_WIDE_FROM 4096
#endif

inline int stream_sms() { return sm_count(); }
// Whether one column tile per CTA fits the SMs in one round.
inline bool stream_one_round(int N) { return (N + ST_COLS - 1) / ST_COLS <= 4 * stream_sms(); }

// wide: 0 = one column tile per CTA, 1 = two (refused with a K split), -1 = choose
inline int launch_gemm_stream(const void* a, int lda, const void* w, int ldw, const float* bias,
                              void* out, int ldo, int M, int N, int K, int act, int mode,
                              int splits, int wide, cudaStream_t stream) {
  const int steps = (K + ST_STEP_K - 1) / ST_STEP_K;
  const int steps_per_split = (steps + splits - 1) / splits;
  if (wide < 0) {
    wide = (splits == 1 && N >= AYK_STREAM_WIDE_FROM && stream_one_round(N)) ? 1 : 0;
  }
  if (wide && splits != 1) return AYK_BAD_ARGUMENT;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<1>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         ST_MAX_STEPS * 1024 + ST_RED_BYTES + 8 * 1024);
    if (e == cudaSuccess) {
      e = cudaFuncSetAttribute(gemm_stream_kernel<2>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                               2 * (ST_MAX_STEPS * 1024 + ST_RED_BYTES));
    }
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const __nv_bfloat16* a16 = reinterpret_cast<const __nv_bfloat16*>(a);
  const __nv_bfloat16* w16 = reinterpret_cast<const __nv_bfloat16*>(w);
  if (wide) {
    const size_t smem = 2 * ((size_t)steps_per_split * 1024 + ST_RED_BYTES);
    return launch_kernel(gemm_stream_kernel<2>, dim3((N + 2 * ST_COLS - 1) / (2 * ST_COLS), 1, 1),
                         dim3(ST_THREADS), smem, stream, 1, a16, lda, w16, ldw, bias, out, ldo,
                         M, N, K, act, mode, steps_per_split);
  }
  const size_t smem = (size_t)steps_per_split * 1024 + ST_RED_BYTES +
                      (splits > 1 ? (size_t)splits * 1024 : 0);
  return launch_kernel(gemm_stream_kernel<1>, dim3((N + ST_COLS - 1) / ST_COLS, splits, 1),
                       dim3(ST_THREADS), smem, stream, splits, a16, lda, w16, ldw, bias, out,
                       ldo, M, N, K, act, mode, steps_per_split);
}

}  // namespace ayk
