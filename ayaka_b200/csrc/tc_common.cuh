// Inline-PTX wrappers for the Blackwell (sm_100a) data path: mbarriers with bounded waits,
// TMA tensor copies, tcgen05 tensor-memory allocation, MMA issue, commit and loads, and the
// host side of tensor maps. No wait in here can spin forever: every one gives up after
// AYK_WAIT_NS nanoseconds and tells its caller.
#pragma once

#include <cuda.h>

#include "common.cuh"

#define AYK_WAIT_TIMEOUT (-5)
#ifndef AYK_WAIT_NS
#define AYK_WAIT_NS 2000000000ull  // 2 s; a legitimate wait is microseconds
#endif
#ifndef AYK_SUSPEND_NS
#define AYK_SUSPEND_NS 4000  // longest park of one mbarrier.try_wait, in nanoseconds
#endif

namespace ayk {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier -------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)
               : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One attempt: true if the phase with the given parity has completed. The hardware may park
// the thread for up to `suspend_ns` while the phase is pending and wakes it when the phase
// completes, so a waiting warp does not take issue slots from the warps that work.
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity,
                                         uint32_t suspend_ns = AYK_SUSPEND_NS) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(suspend_ns)
      : "memory");
  return ok != 0;
}
// Wait for the phase with the given parity to complete; false if it did not within the limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (int i = 0; i < 1024; ++i) {
    if (mbar_try(bar, parity)) return true;
  }
  const uint64_t start = global_ns();
  while (true) {
    for (int i = 0; i < 256; ++i) {
      if (mbar_try(bar, parity)) return true;
    }
    if (global_ns() - start > AYK_WAIT_NS) return false;
  }
}

// ---- TMA ------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// 2-D tiled load: x = innermost coordinate (elements), y = row. x * elemsize must be a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Untiled bulk copy global -> shared: both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// ---- tcgen05 --------------------------------------------------------------------------
// One warp allocates `cols` (a power of two >= 32) columns; the base address lands in *slot.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(slot)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]^T, kind::f16 (bf16/f16 inputs, fp32 accumulate).
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Make `bar` receive one arrival when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::
                   "r"(smem_u32(bar))
               : "memory");
}
// ---- stores through TMA: a tile staged in shared memory goes to global memory as one
// coalesced bulk copy, clipped at the tensor's edges. x * element size must be a multiple
// of 16 bytes; never start at a negative coordinate.
__device__ __forceinline__ void fence_proxy_async_shared() {
  // generic-proxy writes to shared memory become visible to the async proxy (TMA, tcgen05)
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x,
                                             int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::
                   "l"(map), "r"(smem_u32(src)), "r"(x), "r"(y)
               : "memory");
}
// global[tile] += shared[tile], element by element (fp32 adds done by the memory system).
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* src,
                                                  int x, int y) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
      ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// This thread's bulk stores have finished reading shared memory (it may be overwritten) ...
__device__ __forceinline__ void bulk_wait_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// ... and have finished altogether (their writes are done).
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// ---- CTA pairs (cta_group::2): two CTAs of a cluster, on neighbouring SMs, run one MMA of
// 256 rows. Each holds its own 128 rows of A and half of the rows of B in shared memory and
// its own 128 lanes of the accumulator in tensor memory; the even CTA of the pair issues.
// One warp of each CTA allocates (same warp index, same shared-memory slot in both).
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::
                   "r"(smem_u32(slot)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols)
               : "memory");
}
// The descriptors name shared-memory offsets that hold this CTA's operand parts; the peer's
// parts lie at the same offsets of its shared memory.
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at this shared-memory offset in every CTA of `cta_mask` when all
// MMAs issued so far by this thread have finished (an arrival sent to several CTAs, not a
// copy of data: no load is multicast).
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}
// 2-D tiled load into this CTA's shared memory whose bytes are counted on a barrier that may
// lie in the peer CTA (`bar_cluster_address` from peer_address()). No multicast: every CTA
// fetches its own tile.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map,
                                                 uint32_t bar_cluster_address, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(bar_cluster_address), "r"(x), "r"(y)
      : "memory");
}
// One arrival on a barrier of another CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_address) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::
                   "r"(bar_cluster_address)
               : "memory");
}
// 32 lanes x 32 columns of 32-bit cells: thread i of the warp gets lane (base lane + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]),
        "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]),
        "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 16 columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bf16) wide,
// written by TMA with the 128-byte swizzle; the tile starts on a 1024-byte boundary. Groups
// of 8 rows are 1024 bytes apart (stride byte offset); the leading offset is unused (1).
// `byte_offset` advances along K inside the 128-byte row (32 bytes per 16 bf16).
__device__ __forceinline__ uint64_t umma_desc_k128(const void* tile, uint32_t byte_offset) {
  const uint32_t addr = smem_u32(tile) + byte_offset;
  uint64_t desc = 0;
  desc |= (uint64_t)((addr & 0x3FFFFu) >> 4);  // start address
  desc |= (uint64_t)1 << 16;                   // leading byte offset (ignored with swizzle)
  desc |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset
  desc |= (uint64_t)1 << 46;                   // descriptor version of sm_100
  desc |= (uint64_t)2 << 61;                   // 128-byte swizzle
  return desc;
}
// Instruction descriptor: bf16 A and B (both K-major), fp32 accumulator, tile M x N.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

// ---- thread-block clusters ------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;"
               ::: "memory");
}
// Read a float from the same shared-memory offset in CTA `rank` of this cluster.
__device__ __forceinline__ float ld_peer_f32(const float* local, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)),
               "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// The shared::cluster address of `local` in CTA `rank`, and a load through such an address.
__device__ __forceinline__ uint32_t peer_address(const void* local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)),
               "r"(rank));
  return remote;
}
// 16 bytes into shared memory of this or another CTA of the cluster (a shared::cluster
// address from peer_address()).
__device__ __forceinline__ void st_cluster_v4(uint32_t address, uint32_t a, uint32_t b,
                                              uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(address), "r"(a),
               "r"(b), "r"(c), "r"(d)
               : "memory");
}
__device__ __forceinline__ void st_cluster_b32(uint32_t address, uint32_t v) {
  asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(address), "r"(v) : "memory");
}
// The two halves of a cluster barrier, for CTAs that have something to do in between.
__device__ __forceinline__ void cluster_arrive_release() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t address) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(address) : "memory");
  return v;
}

// ---- host: tensor maps ----------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    return (EncodeTiledFn)p;
  }();
  return fn;
}

// Map of a row-major matrix [rows, cols] of 2-byte (bf16) or 4-byte (fp32) elements with row
// stride ld (elements); box = box_rows x 128 bytes (64 or 32 columns), 128-byte swizzle, zero
// fill outside on loads, clipping on stores. Needs a 16-byte aligned base and row stride.
inline int make_map_128b(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                         uint64_t ld, uint32_t box_rows, int elem_bytes) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return AYK_DRIVER;
  if (elem_bytes != 2 && elem_bytes != 4) return AYK_BAD_ARGUMENT;
  if (((uintptr_t)base & 15) || ((ld * elem_bytes) % 16)) return AYK_BAD_ALIGNMENT;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {ld * (uint64_t)elem_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                       : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                  2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? AYK_OK : AYK_DRIVER;
}

inline int make_map_bf16_k64(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                             uint64_t ld, uint32_t box_rows) {
  return make_map_128b(map, base, rows, cols, ld, box_rows, 2);
}

}  // namespace ayk
