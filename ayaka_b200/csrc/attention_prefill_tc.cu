// Causal attention for prompt portions in bfloat16 over the paged cache, head size 64, with
// both products on the 5th-generation tensor cores (tcgen05) and their accumulators in tensor
// memory.
//
// A CTA owns 256 consecutive query rows of one request and one head, as two groups of 128,
// and walks that request's keys 128 at a time from position 0 (or the window's first block)
// up to the tile's last row. The (group, block) pairs are worked on in one order, group 0
// before group 1 for every block; pair i has its scores in slot i mod 3 of a ring in tensor
// memory, its P in the same slot of a ring in shared memory, and the slot's three mbarriers
// (scores ready, P handed over, product finished). Sixteen warps, by role:
//   warps 0-3, 4-7  softmax of group 0 and of group 1: a thread owns one query row. For every
//              block it reads its row of S = Q K^T from tensor memory, keeps the running
//              reference maximum and sum in fp32 registers, writes P = exp2(S * scale * log2e
//              - reference) as bf16 into shared memory in the layout the tensor core reads
//              (128-byte swizzle), and rescales its group's output accumulator in tensor
//              memory when the reference moved;
//   warp 8     one thread issues S = Q K^T (4 x 128x128x16 per pair). The scores of pair i + 3
//              go out as soon as pair i has been handed over (its slot is free): they are the
//              *other* group's next block, while the group that just finished finds the
//              scores of its own next block (pair i + 2) waiting, so the round trip through
//              the issuing threads is off the softmax's path;
//   warp 9     one thread issues O += P V (8 x 128x64x16 per pair; V is read as stored,
//              [key][64], as an MN-major operand) when a pair is handed over. Two issuing
//              threads because one is too slow: with these small MMAs a single thread spent
//              1.2 microseconds per pair on waits, descriptors, issue and commits;
//   warps 10-15  gather Q with 16-byte cp.async copies; then warp 10 brings the K blocks and
//              warp 13 the V blocks into rings of three shared-memory stages (both groups
//              share them) by TMA, one box per page (a head's slots of a page are contiguous
//              rows of 128 bytes; page sizes 8, 16, 32, ... only). With other page sizes warps
//              10-12 and 13-15 gather the blocks with cp.async instead. Measured at 8,192
//              tokens: 435 against 513 microseconds for the kernel.
// mbarriers connect the roles; every wait is bounded (tc_common.cuh) and a wait that runs out
// sets the status word. No barrier can complete two phases unseen by a waiter: a slot's next
// tenant is admitted only after the hand-over of the present one has been seen, and a pair is
// handed over only after the product that last read its P slot has finished. One CTA per SM:
// 224 KB of shared memory and all 512 tensor-memory columns (three score tiles of 128; O0,
// O1: 64 each).
//
// The reference maximum moves only when the block's maximum exceeds it by more than 8 (in
// log2 units; a row's first reference is 0 if its first maximum lies within 8 of that), so
// most blocks do not touch the accumulator; probabilities stay below 2^8 and
// the final division by the running sum makes the result the same function of the scores. A
// row's blocks are aligned to absolute key positions, so its result does not depend on how
// the prompt was cut or on the rows that share its tile.
#include <cuda.h>

#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "tc_common.cuh"

namespace ayk {

constexpr int FA_GM = 128;                  // query rows per group
constexpr int FA_BM = 2 * FA_GM;            // query rows per CTA
constexpr int FA_BN = 128;                  // keys per block
constexpr int FA_HD = 64;                   // head size: one 128-byte swizzle row
constexpr int FA_TILE = FA_GM * FA_HD * 2;  // bytes of a [128][64] bf16 tile
constexpr int FA_STAGES = 3;                // K and V blocks in flight
constexpr int FA_PRODUCERS = 3;              // warps that gather K, and as many for V
constexpr int FA_FIRST_PRODUCER = 10;        // warps 0-7 softmax, 8 and 9 issue the MMAs
constexpr int FA_THREADS = (FA_FIRST_PRODUCER + 2 * FA_PRODUCERS) * 32;
constexpr int FA_RING = 3;                  // score tiles (tensor memory) and P tiles (shared)
constexpr float FA_LAZY = 8.f;              // how far a block's maximum may exceed the reference

struct FaSmem {
  static constexpr int Q = 0;                // two groups
  static constexpr int K = Q + 2 * FA_TILE;          // FA_STAGES stages
  static constexpr int V = K + FA_STAGES * FA_TILE;  // FA_STAGES stages
  static constexpr int P = V + FA_STAGES * FA_TILE;  // FA_RING x [128 rows][128 keys] (two tiles)
  static constexpr int BAR = P + FA_RING * 2 * FA_TILE;
  static constexpr int NUM_BARS = 2 + 4 * FA_STAGES + 3 * FA_RING;
  static constexpr int DYNAMIC = BAR + NUM_BARS * 8 + 16 + 1024;  // room to align the base
};

__device__ __forceinline__ void fa_cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void fa_cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N> __device__ __forceinline__ void fa_cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// 32 lanes x 32 columns back into tensor memory (the inverse of tmem_ld_32x32).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(
          taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),
      "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]),
      "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]),
      "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
// 2^x in one special-function instruction (2 ulp; exp2(-inf) = 0).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// max(a, b, c) in one instruction (three-input max, sm_100).
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Two fp32 lanes in one instruction (sm_100): a * b + c and a + b on register pairs.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n.reg .b64 ra, rb, rc, rd;\n"
      "mov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\nmov.b64 rc, {%6, %7};\n"
      "fma.rn.f32x2 rd, ra, rb, rc;\nmov.b64 {%0, %1}, rd;\n}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("{\n.reg .b64 ra, rb, rd;\n"
      "mov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\n"
      "add.rn.f32x2 rd, ra, rb;\nmov.b64 {%0, %1}, rd;\n}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// Descriptor of an MN-major operand stored as rows of 128 bytes (64 bf16 along MN) with the
// 128-byte swizzle, one row per K index: groups of 8 rows (8 values of K) are 1024 bytes
// apart. `tile` points at the first of the 16 rows one MMA reads.
__device__ __forceinline__ uint64_t umma_desc_mn128(const void* tile) {
  const uint32_t addr = smem_u32(tile);
  uint64_t desc = 0;
  desc |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  desc |= (uint64_t)1 << 16;            // leading offset: between 64-wide MN groups (one here)
  desc |= (uint64_t)(1024 >> 4) << 32;  // stride offset: between groups of 8 rows
  desc |= (uint64_t)1 << 46;
  desc |= (uint64_t)2 << 61;
  return desc;
}

// FA_PRODUCERS warps (this one is number `part`) gather a block of 128 keys (or values) of one
// head into a [128][64] tile: a warp's copies complete one after the other, at about one
// 512-byte instruction per memory round trip (measured: 32 of them took 4.7 microseconds), so
// several warps share a block. Row =
// key, 16-byte piece c of row r at piece c ^ (r & 7). Keys outside [first_key, last_key] are
// zero-filled: their pages may be gone (a window) or hold anything, and 0 * NaN would poison
// the sum.
__device__ __forceinline__ void fa_gather_block(uint8_t* tile,
                                                const __nv_bfloat16* __restrict__ pages,
                                                const int* __restrict__ table, int key0,
                                                int first_key, int last_key, int num_kv_heads,
                                                int kv_head, int page_size, int page_shift,
                                                int lane, int part) {
  const int piece = lane & 7;
#pragma unroll 4
  for (int t = part; t < FA_BN / 4; t += FA_PRODUCERS) {
    const int r = t * 4 + (lane >> 3);
    const int key = key0 + r;
    const bool valid = key >= first_key && key <= last_key;
    const __nv_bfloat16* src = pages;
    if (valid) {
      const int index = page_shift >= 0 ? key >> page_shift : key / page_size;
      const int slot = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
      const int page = table[index];
      src = pages + (((size_t)page * num_kv_heads + kv_head) * page_size + slot) * FA_HD +
            piece * 8;
    }
    fa_cp_async16(tile + r * 128 + ((piece ^ (r & 7)) << 4), src, valid);
  }
}

__global__ void __launch_bounds__(FA_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, int box_rows,
                            const __nv_bfloat16* __restrict__ q, int ld_q,
                            const __nv_bfloat16* __restrict__ k_pages,
                            const __nv_bfloat16* __restrict__ v_pages,
                            const int* __restrict__ block_table, int table_stride,
                            const int* __restrict__ row_start, const int* __restrict__ kv_len,
                            __nv_bfloat16* __restrict__ out, int ld_out, int num_requests,
                            int num_kv_heads, int group, int page_size, float scale, int window,
                            int total_tiles, int page_shift, int* __restrict__ status) {
  extern __shared__ uint8_t fa_raw[];
  uint8_t* smem = fa_raw + ((1024 - (smem_u32(fa_raw) & 1023)) & 1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FaSmem::BAR);
  uint64_t* q_full = bars;        // one arrival per producer warp
  uint64_t* k_full = bars + 1;                   // [stage], one arrival per producer warp
  uint64_t* k_empty = k_full + FA_STAGES;        // [stage], MMA commits
  uint64_t* v_full = k_empty + FA_STAGES;        // [stage]
  uint64_t* v_empty = v_full + FA_STAGES;        // [stage]
  uint64_t* s_full = v_empty + FA_STAGES;  // [ring slot] MMA commit: S is in tensor memory
  // [ring slot], like s_full: the next use of a slot's barriers belongs to the pair three
  // further on, whose scores are issued only after this pair's hand-over has been seen, so no
  // waiter ever has two phases of one barrier to tell apart
  uint64_t* p_full = s_full + FA_RING;   // 4 arrivals: S is read, P is in shared memory
  uint64_t* pv_done = p_full + FA_RING;  // MMA commit: O += P V (and all before it) has finished
  uint64_t* v_land = pv_done + FA_RING;  // TMA: a V block that needs rows zeroed lands here first
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + FaSmem::NUM_BARS);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 512;  // S ring: 3 x 128 columns; O0: 384..447, O1: 448..511
  constexpr uint32_t O_COL = FA_RING * FA_BN;

  if (threadIdx.x == 0) {
    // a block is published by its gathering warps, or (TMA) by one arrival with the bytes
    const uint32_t publishers = box_rows > 0 ? 1 : FA_PRODUCERS;
    mbar_init(q_full, 2 * FA_PRODUCERS);
    mbar_init(v_land, 1);
    for (int s = 0; s < FA_STAGES; ++s) {
      mbar_init(&k_full[s], publishers);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], publishers);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < FA_RING; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 4);
      mbar_init(&pv_done[s], 1);
    }
    *failed = 0;
    mbar_fence_init();
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait_for(q, k_pages, v_pages);

  // Which request and which 256-row tile of it: heads along grid.x, tiles along grid.y from
  // the last one down (the longest first). (The tiles ranked by the keys they reach, so that
  // the order holds across requests too, made the prologue two trips to memory longer and
  // a step of two prompts of 1,024 tokens 1 % slower.)
  int tile = total_tiles - 1 - (int)blockIdx.y, req = 0, rows_b = 0;
  for (; req < num_requests; ++req) {
    rows_b = row_start[req + 1] - row_start[req];
    const int tiles = (rows_b + FA_BM - 1) / FA_BM;
    if (tile < tiles) break;
    tile -= tiles;
  }
  const int head = blockIdx.x;
  const int kv_head = head / group;
  bool work = req < num_requests;
  int first_row = 0, nrows = 0, length = 0;
  if (work) {
    first_row = row_start[req] + tile * FA_BM;
    nrows = rows_b - tile * FA_BM < FA_BM ? rows_b - tile * FA_BM : FA_BM;
    length = kv_len[req];
    if (length == 0) {  // a padding request: zeros
      for (int i = threadIdx.x; i < nrows * (FA_HD / 8); i += FA_THREADS) {
        *reinterpret_cast<uint4*>(out + (size_t)(first_row + i / (FA_HD / 8)) * ld_out +
                                  head * FA_HD + (i % (FA_HD / 8)) * 8) =
            make_uint4(0u, 0u, 0u, 0u);
      }
      work = false;
    }
  }
  if (work) {
    const int pos0 = length - rows_b + tile * FA_BM;  // position of the tile's first row
    const int last_key = pos0 + nrows - 1;
    const int lo_min = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    // Each group's blocks: from the block of its first row's first visible key to the block
    // of its last row. Group 1 has none when the tile has at most 128 rows.
    int blo[2], bhi[2];
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      const int g_pos0 = pos0 + g * FA_GM;
      const int g_rows = nrows - g * FA_GM < FA_GM ? nrows - g * FA_GM : FA_GM;
      const int g_lo = (window > 0 && g_pos0 - window + 1 > 0) ? g_pos0 - window + 1 : 0;
      blo[g] = g_lo / FA_BN;
      bhi[g] = g_rows > 0 ? (g_pos0 + g_rows - 1) / FA_BN : blo[g] - 1;
    }
    const int jlo = blo[0];  // group 0 starts first and group 1 (if any) ends last
    const int jhi = bhi[1] >= blo[1] ? bhi[1] : bhi[0];
    const int num_blocks = jhi - jlo + 1;
    const int* table = block_table + (size_t)req * table_stride;
    uint8_t* q_s = smem + FaSmem::Q;
    uint8_t* p_s = smem + FaSmem::P;

    // The (group, block) pairs in the order they are worked on: block by block, group 0
    // before group 1. Pair number i has its scores in ring slot i % FA_RING of tensor memory
    // and its P in the same slot of shared memory.
    auto active = [&](int g, int j) { return j >= blo[g] && j <= bhi[g]; };
    auto advance = [&](int& g, int& j) {
      do {
        if (g == 0) {
          g = 1;
        } else {
          g = 0;
          ++j;
        }
      } while (j <= jhi && !active(g, j));
    };

    if (warp >= FA_FIRST_PRODUCER) {
      // ---- producers: all of them bring Q; then the first FA_PRODUCERS warps bring the K
      // blocks and the others the V blocks
      const bool keys = warp < FA_FIRST_PRODUCER + FA_PRODUCERS;
      const int part = (warp - FA_FIRST_PRODUCER) % FA_PRODUCERS;
      uint64_t* full = keys ? k_full : v_full;
      uint64_t* empty = keys ? k_empty : v_empty;
      uint8_t* stages = smem + (keys ? FaSmem::K : FaSmem::V);
      const __nv_bfloat16* pages = keys ? k_pages : v_pages;
      {
        const int piece = lane & 7;
        for (int t = warp - FA_FIRST_PRODUCER; t < FA_BM / 4; t += 2 * FA_PRODUCERS) {
          const int r = t * 4 + (lane >> 3);
          const bool valid = r < nrows;
          const __nv_bfloat16* src =
              q + (size_t)(first_row + (valid ? r : 0)) * ld_q + head * FA_HD + piece * 8;
          fa_cp_async16(q_s + r * 128 + ((piece ^ (r & 7)) << 4), src, valid);
        }
        fa_cp_async_commit();
      }
      bool ok = true;
      if (box_rows > 0) {
        // ---- TMA: a page's [slots][64] of one head is contiguous, so a block of 128 keys is
        // 128 / box_rows boxes of box_rows rows (box_rows = min(page size, 128)); lane t
        // fetches box t. Boxes wholly outside [lo_min, last_key] are left out (their pages
        // may be gone); rows outside it inside a fetched box hold whatever the page holds.
        // For K that is harmless (their scores are masked). For V they must be zero (0 * NaN
        // would poison the sum): such a block lands on a barrier of this warp first, which
        // zeroes the rows and then publishes the block.
        // Q is published once the first K or V block of this warp is on its way: the block
        // does not wait for Q (that order cost a CTA the time of one more trip to memory
        // before its first product)
        auto publish_q = [&]() {
          fa_cp_async_wait<0>();
          fence_proxy_async_shared();
          __syncwarp();
          if (lane == 0) mbar_arrive(q_full);
        };
        if (part != 0) publish_q();
        if (part == 0) {
          const CUtensorMap* map = keys ? &map_k : &map_v;
          const int boxes = FA_BN / box_rows;
          const uint32_t box_bytes = (uint32_t)box_rows * 128u;
          int landed = 0, issued = 0;
          for (int jj = 0; jj < num_blocks && ok; ++jj) {
            const int stage = jj % FA_STAGES;
            if (jj >= FA_STAGES) {  // the stage's last tenant must have been read by its MMAs
              if (lane == 0) ok = mbar_wait(&empty[stage], (uint32_t)(jj / FA_STAGES - 1) & 1u);
              ok = __shfl_sync(0xffffffffu, ok, 0);
              if (!ok) break;
            }
            const int key0 = (jlo + jj) * FA_BN;
            const int key = key0 + lane * box_rows;
            const bool fetch = lane < boxes && key + box_rows - 1 >= lo_min && key <= last_key;
            const uint32_t count = (uint32_t)__popc(__ballot_sync(0xffffffffu, fetch));
            const bool fix = !keys && (key0 < lo_min || key0 + FA_BN - 1 > last_key);
            uint64_t* lands = fix ? v_land : &full[stage];
            uint8_t* tile = stages + stage * FA_TILE;
            if (lane == 0) mbar_expect_tx(lands, count * box_bytes);
            __syncwarp();
            if (fetch) {
              const int index = page_shift >= 0 ? key >> page_shift : key / page_size;
              const int slot = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
              const int page = table[index];
              tma_load_2d(tile + (size_t)lane * box_bytes, map, lands, 0,
                          (page * num_kv_heads + kv_head) * page_size + slot);
            }
            if (jj == 0) publish_q();
            if (fix) {
              if (lane == 0) ok = mbar_wait(v_land, (uint32_t)landed & 1u);
              ok = __shfl_sync(0xffffffffu, ok, 0);
              if (!ok) break;
              ++landed;
              // rows of keys outside [lo_min, last_key]: eight 16-byte pieces each
              for (int i = lane; i < FA_BN * 8; i += 32) {
                const int r = i >> 3;
                if (key0 + r < lo_min || key0 + r > last_key) {
                  *reinterpret_cast<uint4*>(tile + r * 128 + ((i & 7) << 4)) =
                      make_uint4(0u, 0u, 0u, 0u);
                }
              }
              fence_proxy_async_shared();
              __syncwarp();
              if (lane == 0) mbar_arrive(&full[stage]);
            }
            issued = jj + 1;
          }
          // nothing of this warp's is in flight when it leaves: the last blocks have landed
          if (lane == 0) {
            for (int jj = issued > FA_STAGES ? issued - FA_STAGES : 0; jj < issued; ++jj) {
              mbar_wait(&full[jj % FA_STAGES], (uint32_t)(jj / FA_STAGES) & 1u);
            }
          }
          __syncwarp();
        }
      } else {
        for (int jj = 0; jj < num_blocks && ok; ++jj) {
          const int stage = jj % FA_STAGES;
          if (jj >= FA_STAGES) {  // the stage's last tenant must have been read by its MMAs
            if (lane == 0) ok = mbar_wait(&empty[stage], (uint32_t)(jj / FA_STAGES - 1) & 1u);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
          }
          fa_gather_block(stages + stage * FA_TILE, pages, table, (jlo + jj) * FA_BN, lo_min,
                          last_key, num_kv_heads, kv_head, page_size, page_shift, lane, part);
          fa_cp_async_commit();
          // The block before has landed once only this one is still in flight: publish it.
          // (With three stages the wait for this block's stage, above, concerns a block the
          // consumer finished two blocks ago, so it never holds a publication back.) Q was
          // committed before the first block.
          fa_cp_async_wait<1>();
          fence_proxy_async_shared();
          __syncwarp();
          if (lane == 0) {
            if (jj == 0) mbar_arrive(q_full);
            if (jj > 0) mbar_arrive(&full[(jj - 1) % FA_STAGES]);
          }
        }
        fa_cp_async_wait<0>();
        fence_proxy_async_shared();
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(&full[(num_blocks - 1) % FA_STAGES]);
      }
      if (!ok && lane == 0) *failed = 1;
    } else if (warp == 8) {
      // ---- issuer of S = Q K^T -------------------------------------------------------------
      if (lane == 0) {
        constexpr uint32_t idesc_s = umma_idesc_bf16(FA_GM, FA_BN);
        int sg = 0, sj = jlo, si = 0;  // the next pair
        if (!active(0, jlo)) advance(sg, sj);
        bool ok = mbar_wait(q_full, 0);
        while (ok && sj <= jhi) {
          const int jj = sj - jlo, stage = jj % FA_STAGES, slot = si % FA_RING;
          // the slot's tenant three pairs ago has been read
          if (si >= FA_RING) {
            ok = mbar_wait(&p_full[slot], (uint32_t)(si / FA_RING - 1) & 1u);
          }
          if (ok) {
            ok = mbar_wait(&k_full[stage], (uint32_t)(jj / FA_STAGES) & 1u);
          }
          if (!ok) break;
          tc_fence_after();
          const uint8_t* k_tile = smem + FaSmem::K + stage * FA_TILE;
          const uint8_t* q_tile = q_s + sg * FA_TILE;
#pragma unroll
          for (int k = 0; k < FA_HD / 16; ++k) {
            umma_f16(tmem_base + (uint32_t)(slot * FA_BN), umma_desc_k128(q_tile, k * 32),
                     umma_desc_k128(k_tile, k * 32), idesc_s, k != 0);
          }
          umma_commit(&s_full[slot]);
          if (sg == 1 || !active(1, sj)) umma_commit(&k_empty[stage]);  // the block's last reader
          ++si;
          advance(sg, sj);
        }
        if (!ok) *failed = 1;
      }
      __syncwarp();
    } else if (warp == 9) {
      // ---- issuer of O += P V --------------------------------------------------------------
      if (lane == 0) {
        constexpr uint32_t idesc_o = umma_idesc_bf16(FA_GM, FA_HD) | (1u << 16);  // B: MN-major
        int pg = 0, pj = jlo, pi = 0, npv[2] = {0, 0};
        if (!active(0, jlo)) advance(pg, pj);
        bool ok = true;
        while (ok && pj <= jhi) {
          const int jj = pj - jlo, stage = jj % FA_STAGES, slot = pi % FA_RING;
          ok = mbar_wait(&v_full[stage], (uint32_t)(jj / FA_STAGES) & 1u);
          if (ok) {
            ok = mbar_wait(&p_full[slot], (uint32_t)(pi / FA_RING) & 1u);
          }
          if (!ok) break;
          tc_fence_after();
          const uint8_t* v_tile = smem + FaSmem::V + stage * FA_TILE;
          const uint8_t* p_tile = p_s + slot * 2 * FA_TILE;
#pragma unroll
          for (int k = 0; k < FA_BN / 16; ++k) {
            umma_f16(tmem_base + O_COL + (uint32_t)(pg * FA_HD),
                     umma_desc_k128(p_tile + (k >> 2) * FA_TILE, (k & 3) * 32),
                     umma_desc_mn128(v_tile + k * 16 * 128), idesc_o, (npv[pg] | k) != 0);
          }
          umma_commit(&pv_done[slot]);
          if (pg == 1 || !active(1, pj)) umma_commit(&v_empty[stage]);
          ++npv[pg];
          ++pi;
          advance(pg, pj);
        }
        if (!ok) *failed = 1;
      }
      __syncwarp();
    } else if (bhi[warp >> 2] >= blo[warp >> 2]) {
      // ---- softmax: warps 0-3 own the rows of group 0, warps 4-7 those of group 1 ----------
      const int g = warp >> 2;
      const int r = threadIdx.x & (FA_GM - 1);  // the row inside the group
      const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
      const uint32_t o_acc = tmem_base + O_COL + (uint32_t)(g * FA_HD) + lane_base;
      const int g_pos0 = pos0 + g * FA_GM;
      const int pos = g_pos0 + r;
      const int after = window > 0 ? pos - window : -2147483647 - 1;  // keys > after are seen
      const float scale2 = scale * 1.4426950408889634f;  // scores in units of log2
      float ref = -INFINITY, sum = 0.f;
      const int swz = r & 7;
      const int my_blocks = bhi[g] - blo[g] + 1;
      const int other = g ^ 1;
      const int other_blocks = bhi[other] >= blo[other] ? bhi[other] - blo[other] + 1 : 0;
      bool ok = true;
      // The number of this group's block n in the order of work (see the MMA issuer): its own
      // blocks so far plus the other group's blocks that come before it.
      auto pair_of = [&](int n) {
        int before = blo[g] + n - blo[other] + (other < g ? 1 : 0);
        before = before < 0 ? 0 : (before > other_blocks ? other_blocks : before);
        return n + before;
      };
      // Wait until the product O += P V of a pair of this group has finished (and with it
      // every product issued before). The slot's barrier was last used three pairs earlier,
      // by a product that finished before this pair's scores were committed.
      auto wait_pv = [&](int pair) {
        if (lane == 0) ok = mbar_wait(&pv_done[pair % FA_RING], (uint32_t)(pair / FA_RING) & 1u);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        tc_fence_after();
      };
      for (int n = 0; n < my_blocks; ++n) {
        const int key0 = (blo[g] + n) * FA_BN;
        const int pair = pair_of(n), slot = pair % FA_RING;
        const uint32_t s_acc = tmem_base + (uint32_t)(slot * FA_BN) + lane_base;
        uint8_t* p_row = p_s + slot * 2 * FA_TILE + r * 128;
        if (lane == 0) ok = mbar_wait(&s_full[slot], (uint32_t)(pair / FA_RING) & 1u);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        tc_fence_after();
        // the slot's P was last read by the product of three pairs ago, handed over more than
        // a block ago
        if (pair >= FA_RING) {
          wait_pv(pair - FA_RING);
          if (!ok) break;
        }
        // A block wholly before the group's first row (and no window) has nothing to mask.
        // The masked variant selects without branching: per element it is two integer
        // compares and a select.
        const bool all_seen = window == 0 && key0 + FA_BN - 1 <= g_pos0;
        // One pass over the scores: exponentiate against the reference the row already has
        // and find the block's maximum on the way. Only if that maximum leaves the reference
        // more than FA_LAZY behind (the first block, and now and then an early one) does the
        // reference move; then the accumulator is rescaled and the pass runs a second time.
        float part = 0.f;
        for (int attempt = 0;; ++attempt) {
          const float offset = ref == -INFINITY ? 0.f : ref;
          float2 part01 = make_float2(0.f, 0.f), part23 = make_float2(0.f, 0.f);
          float t0 = -INFINITY, t1 = -INFINITY, t2 = -INFINITY, t3 = -INFINITY;
          constexpr int CW = 32;  // columns of the row worked on at a time
          float p[CW];
          // scale and reference for two scores an instruction
          const float2 scale_2 = make_float2(scale2, scale2), offset_2 = make_float2(-offset, -offset);
          // the columns' scores (masked) against the reference, the block's maximum on the way
          auto select = [&](const uint32_t* raw, int c) {
            if (all_seen) {
#pragma unroll
              for (int i = 0; i < CW; i += 8) {
                t0 = fmax3(t0, __uint_as_float(raw[i]), __uint_as_float(raw[i + 1]));
                t1 = fmax3(t1, __uint_as_float(raw[i + 2]), __uint_as_float(raw[i + 3]));
                t2 = fmax3(t2, __uint_as_float(raw[i + 4]), __uint_as_float(raw[i + 5]));
                t3 = fmax3(t3, __uint_as_float(raw[i + 6]), __uint_as_float(raw[i + 7]));
              }
#pragma unroll
              for (int i = 0; i < CW; i += 2) {
                const float2 x = fma2(
                    make_float2(__uint_as_float(raw[i]), __uint_as_float(raw[i + 1])), scale_2,
                    offset_2);
                p[i] = x.x;
                p[i + 1] = x.y;
              }
            } else {
              const int key = key0 + c * CW;
#pragma unroll
              for (int i = 0; i < CW; i += 4) {
                const bool a0 = (key + i <= pos) & (key + i > after);
                const bool a1 = (key + i + 1 <= pos) & (key + i + 1 > after);
                const bool a2 = (key + i + 2 <= pos) & (key + i + 2 > after);
                const bool a3 = (key + i + 3 <= pos) & (key + i + 3 > after);
                const float x0 = a0 ? __uint_as_float(raw[i]) : -INFINITY;
                const float x1 = a1 ? __uint_as_float(raw[i + 1]) : -INFINITY;
                const float x2 = a2 ? __uint_as_float(raw[i + 2]) : -INFINITY;
                const float x3 = a3 ? __uint_as_float(raw[i + 3]) : -INFINITY;
                t0 = fmaxf(t0, x0);
                t1 = fmaxf(t1, x1);
                t2 = fmaxf(t2, x2);
                t3 = fmaxf(t3, x3);
                const float2 x01 = fma2(make_float2(x0, x1), scale_2, offset_2);
                const float2 x23 = fma2(make_float2(x2, x3), scale_2, offset_2);
                p[i] = x01.x;  // -inf for a masked key: exp2(-inf) = 0
                p[i + 1] = x01.y;
                p[i + 2] = x23.x;
                p[i + 3] = x23.y;
              }
            }
          };
          auto weigh = [&](int c) {
#pragma unroll
            for (int i = 0; i < CW; ++i) p[i] = fast_exp2(p[i]);
#pragma unroll
            for (int i = 0; i < CW; i += 4) {
              part01 = add2(part01, make_float2(p[i], p[i + 1]));
              part23 = add2(part23, make_float2(p[i + 2], p[i + 3]));
            }
            // 64 keys make a tile of 128-byte rows; eight keys a 16-byte piece of it
            uint8_t* dst = p_row + ((c * CW) >> 6) * FA_TILE;
            const int piece0 = ((c * CW) & 63) >> 3;
#pragma unroll
            for (int h = 0; h < CW / 8; ++h) {
              uint4 packed;
              __nv_bfloat162 h0 = __floats2bfloat162_rn(p[h * 8], p[h * 8 + 1]);
              __nv_bfloat162 h1 = __floats2bfloat162_rn(p[h * 8 + 2], p[h * 8 + 3]);
              __nv_bfloat162 h2 = __floats2bfloat162_rn(p[h * 8 + 4], p[h * 8 + 5]);
              __nv_bfloat162 h3 = __floats2bfloat162_rn(p[h * 8 + 6], p[h * 8 + 7]);
              packed.x = *reinterpret_cast<uint32_t*>(&h0);
              packed.y = *reinterpret_cast<uint32_t*>(&h1);
              packed.z = *reinterpret_cast<uint32_t*>(&h2);
              packed.w = *reinterpret_cast<uint32_t*>(&h3);
              *reinterpret_cast<uint4*>(dst + (((piece0 + h) ^ swz) << 4)) = packed;
            }
          };
          // One load and one copy of the arithmetic. Loading the next columns while these are
          // worked on measured no faster, neither with two register buffers and the arithmetic
          // twice in the loop (426 against 408 microseconds at 8,192 tokens) nor with the next
          // load issued once these columns have left its registers (384 against 379): the
          // other group's warps fill the gap.
          uint32_t raw[CW];
#pragma unroll 1
          for (int c = 0; c < FA_BN / CW; ++c) {
            tmem_ld_32x32(s_acc + (uint32_t)(c * CW), raw);
            tmem_ld_wait();
            select(raw, c);
            weigh(c);
          }
          part = (part01.x + part01.y) + (part23.x + part23.y);
          const float top = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3)) * scale2;
          // A row without a reference ran this pass against 0 (see offset): that stands as
          // its reference if its maximum is within FA_LAZY of it, and the first block then
          // needs no second pass either.
          const bool fresh = ref == -INFINITY;
          const bool moves = fresh ? (top > FA_LAZY || (top < -FA_LAZY && top > -INFINITY))
                                   : top > ref + FA_LAZY;
          if (fresh && !moves && top > -INFINITY) ref = 0.f;
          if (attempt == 1 || !__any_sync(0xffffffffu, moves)) break;
          float alpha = 1.f;
          if (moves) {
            alpha = fast_exp2(ref - top);  // 0 when there was no reference yet
            ref = top;
          }
          if (n > 0) {
            // the accumulator is whole once this group's product before has finished
            // (issued a whole softmax ago: over long since)
            wait_pv(pair_of(n - 1));  // (issued a whole softmax ago: over long since)
            if (!ok) break;
#pragma unroll 1
            for (int c = 0; c < FA_HD / 32; ++c) {
              uint32_t raw[32];
              tmem_ld_32x32(o_acc + (uint32_t)(c * 32), raw);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * alpha);
              tmem_st_32x32(o_acc + (uint32_t)(c * 32), raw);
            }
            tmem_st_wait();
          }
          sum *= alpha;
        }
        if (!ok) break;
        sum += part;
        // S has been read for the last time and P is written (generic-proxy writes that the
        // tensor core reads): one arrival says both
        tc_fence_before();
        fence_proxy_async_shared();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[slot]);
      }
      // (no pair three further on exists: the other group ends at most a block later)
      if (ok) wait_pv(pair_of(my_blocks - 1));
      if (ok) {
        tc_fence_after();
        const float inv = 1.f / sum;
        const int row = g * FA_GM + r;  // inside the tile
        __nv_bfloat16* dst = out + (size_t)(first_row + row) * ld_out + head * FA_HD;
#pragma unroll 1
        for (int c = 0; c < FA_HD / 32; ++c) {
          uint32_t raw[32];
          tmem_ld_32x32(o_acc + (uint32_t)(c * 32), raw);
          tmem_ld_wait();
          if (row < nrows) {
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              uint4 packed;
              __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(raw[h * 8]) * inv,
                                                        __uint_as_float(raw[h * 8 + 1]) * inv);
              __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(raw[h * 8 + 2]) * inv,
                                                        __uint_as_float(raw[h * 8 + 3]) * inv);
              __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(raw[h * 8 + 4]) * inv,
                                                        __uint_as_float(raw[h * 8 + 5]) * inv);
              __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(raw[h * 8 + 6]) * inv,
                                                        __uint_as_float(raw[h * 8 + 7]) * inv);
              packed.x = *reinterpret_cast<uint32_t*>(&h0);
              packed.y = *reinterpret_cast<uint32_t*>(&h1);
              packed.z = *reinterpret_cast<uint32_t*>(&h2);
              packed.w = *reinterpret_cast<uint32_t*>(&h3);
              *reinterpret_cast<uint4*>(dst + c * 32 + h * 8) = packed;
            }
          }
          __syncwarp();
        }
      } else if (lane == 0) {
        *failed = 1;
      }
    }
  }

  // ---- teardown ---------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*failed != 0 && threadIdx.x == 0) atomicExch(status, AYK_WAIT_TIMEOUT);
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Tensor maps of the caches' page tensors, kept by base address: a serving process has two
// per layer and encodes each once.
static int pages_map(const void* base, uint64_t rows, uint32_t box_rows, CUtensorMap* out) {
  struct Entry {
    const void* base;
    uint64_t rows;
    uint32_t box_rows;
    CUtensorMap map;
  };
  static std::mutex mu;
  static std::vector<Entry> cache;
  std::lock_guard<std::mutex> lock(mu);
  for (const Entry& e : cache) {
    if (e.base == base && e.rows == rows && e.box_rows == box_rows) {
      *out = e.map;
      return AYK_OK;
    }
  }
  Entry e{base, rows, box_rows, {}};
  const int r = make_map_bf16_k64(&e.map, base, rows, FA_HD, FA_HD, box_rows);
  if (r != AYK_OK) return r;
  if (cache.size() >= 1024) cache.clear();
  cache.push_back(e);
  *out = e.map;
  return AYK_OK;
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

// Query rows per CTA: the caller sizes the grid with it.
AYK_API int ayk_attention_prefill_tc_rows() { return ayk::FA_BM; }

// bfloat16, head size 64 and a positive scale only (AYK_BAD_ARGUMENT otherwise: use the
// mma.sync kernel). q/out
// rows are 16-byte aligned (ld multiples of 8 elements). `total_tiles` = sum over requests of
// ceil(rows / 256), from the caller's host copy of the rows. `status` is one device int that
// the kernel sets to AYK_WAIT_TIMEOUT if a wait ran out.
AYK_API int ayk_attention_prefill_tc(const void* q, int ld_q, const void* k_pages,
                                     const void* v_pages, const int* block_table,
                                     int table_stride, const int* row_start, const int* kv_len,
                                     void* out, int ld_out, int num_requests, int total_tiles,
                                     int num_heads, int num_kv_heads, int head_dim, int page_size,
                                     int num_pages, float scale, int window, int* status,
                                     void* stream) {
  using namespace ayk;
  if (num_requests == 0 || total_tiles == 0) return AYK_OK;
  if (head_dim != FA_HD || status == nullptr || !(scale > 0.f)) return AYK_BAD_ARGUMENT;
  if (num_requests < 0 || total_tiles < 0 || num_heads < 1 || num_kv_heads < 1 ||
      num_heads % num_kv_heads || page_size < 1 || table_stride < 1 || window < 0) {
    return AYK_BAD_ARGUMENT;
  }
  if (total_tiles > 65535) return AYK_TOO_LARGE;
  if (((uintptr_t)q % 16) || ((uintptr_t)out % 16) || ((uintptr_t)k_pages % 16) ||
      ((uintptr_t)v_pages % 16) || (ld_q % 8) || (ld_out % 8)) {
    return AYK_BAD_ALIGNMENT;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FaSmem::DYNAMIC);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0) {
    page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
  }
  // Pages of a power-of-two size from 8 slots up are fetched by TMA: one head's slots of a
  // page are contiguous rows of 128 bytes, so the pages tensor is a matrix of
  // pages * heads * slots rows to the tensor map. Other page sizes are gathered by cp.async.
  CUtensorMap map_k, map_v;
  memset(&map_k, 0, sizeof(map_k));
  memset(&map_v, 0, sizeof(map_v));
  int box_rows = 0;
  const unsigned long long cache_rows = (unsigned long long)num_pages * num_kv_heads * page_size;
  if (page_shift >= 3 && num_pages > 0 && cache_rows < 2147483648ull) {
    box_rows = page_size < FA_BN ? page_size : FA_BN;
    int r = pages_map(k_pages, cache_rows, (uint32_t)box_rows, &map_k);
    if (r == AYK_OK) r = pages_map(v_pages, cache_rows, (uint32_t)box_rows, &map_v);
    if (r != AYK_OK) return r;
  }
  return launch_kernel(attention_prefill_tc_kernel, dim3(num_heads, total_tiles),
                       dim3(FA_THREADS), FaSmem::DYNAMIC, (cudaStream_t)stream, 1, map_k, map_v,
                       box_rows, (const __nv_bfloat16*)q, ld_q, (const __nv_bfloat16*)k_pages,
                       (const __nv_bfloat16*)v_pages, block_table, table_stride, row_start,
                       kv_len, (__nv_bfloat16*)out, ld_out, num_requests, num_kv_heads,
                       num_heads / num_kv_heads, page_size, scale, window, total_tiles,
                       page_shift, status);
}
