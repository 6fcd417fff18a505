// Decode attention (one row a request), bfloat16, head size 64 or 128, with both products on
// the warp-level tensor cores.
//
// The split-KV kernel of attention_decode.cu does its dot products on the CUDA cores: eight
// conversions and eight multiply-adds per 16 bytes of keys, and again per 16 bytes of values.
// With 64 requests x 25 heads that binds it to instruction issue (measured on a B200: issue
// slots 68 % busy, DRAM at 55 %), and with a few requests it spreads a pair over a cluster,
// whose launch and barrier cost about 3 microseconds in a chain of dependent kernels. Here a
// warp takes tiles of 16 keys: S = q K^T as m16n8k16 MMAs whose 16 query rows are the one
// real row and 15 rows of zeros (the tensor pipe has room for that many times over), the
// softmax on the four lanes that hold the real row, O += P V as MMAs whose A operand is the
// score accumulator as it lies in registers. About 30 instructions per 16 keys instead of
// about 180, and one CTA per (row, head) at every batch size.
//
// A CTA of four, eight or sixteen warps serves one (row, head); warp w takes tiles w,
// w + WARPS, ... of the row's keys, each with its own ring of three 16-key stages of K and V
// in shared memory (128-byte rows with the usual XOR swizzle for ldmatrix), all three started
// before the dependency wait for the keys of earlier steps (when the row's own key comes from
// k_new) and each refilled as soon as its tile has been used. Where the layout allows (head
// size 64, pages of a multiple of 16 tokens, no window, the caller names the number of pages)
// a tile is two TMA boxes of 16 rows, one of K and one of V, issued by one lane and awaited
// on a barrier per stage; else every lane copies its 16-byte pieces with cp.async. Cycle
// stamps in the kernel showed why that matters: issuing one tile's 256 cp.async took 0.75
// microseconds each time, with the table lookup ahead of it or without (the SM's queue of
// outstanding requests was full), five times in a row for a warp of a 528-key context; a TMA
// box costs its issuer nothing. A decode step of GPT-2 XL at 8 requests: 1.40 against 1.49 ms.
// The row's pages are read once into shared memory (up to DM_TABLE_ROOM entries). The warps' partial results merge through shared memory in warp order. More warps
// finish a pair sooner and fewer such CTAs fit an SM; the host picks by the number of pairs
// (decode_mma_warps). The row's own key and value come from the projection's output (k_new /
// v_new) and, with `store`, are written to the cache by the warp that owns the last tile.
#pragma once

#include <mutex>
#include <unordered_map>

#include "tc_common.cuh"

namespace ayk {

constexpr int DM_STAGES = 3;
constexpr int DM_TILE = 16;  // keys per tile
constexpr int DM_TABLE_ROOM = 512;  // table entries a CTA holds in shared memory (2 KB)

__device__ __forceinline__ void dm_cp_async_16(void* dst, const void* src, bool valid) {
  const uint32_t bytes = valid ? 16u : 0u;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(
                   (uint32_t)__cvta_generic_to_shared(dst)),
               "l"(src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void dm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void dm_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void dm_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void dm_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void dm_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t dm_pack(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// grid (num_heads, num_rows); HD = head size (64 or 128). Shared memory: DM_WARPS rings of
// DM_STAGES x (K tile + V tile) of 16 x HD bfloat16, then the merge area.
template <int HD, int DM_WARPS, bool TMA>
__global__ void __launch_bounds__(DM_WARPS * 32)
attention_decode_mma_kernel(const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, int* status,
                            const __nv_bfloat16* __restrict__ q, int ld_q,
                            const __nv_bfloat16* __restrict__ k_pages,
                            const __nv_bfloat16* __restrict__ v_pages,
                            const int* __restrict__ block_table, int table_stride,
                            const int* __restrict__ request_of_row,
                            const int* __restrict__ positions, __nv_bfloat16* __restrict__ out,
                            int ld_out, int num_kv_heads, int group, int page_size,
                            int page_shift, float scale, int window,
                            const __nv_bfloat16* __restrict__ k_new,
                            const __nv_bfloat16* __restrict__ v_new, int ld_new,
                            __nv_bfloat16* __restrict__ k_store,
                            __nv_bfloat16* __restrict__ v_store, int table_room) {
  constexpr int ROW_BYTES = HD * 2;          // one key's bytes
  constexpr int PIECES = ROW_BYTES / 16;     // 16-byte pieces per key
  constexpr int TILE_BYTES = DM_TILE * ROW_BYTES;
  constexpr int KSTEPS = HD / 16;            // k-steps of S = q K^T
  constexpr int NT = HD / 8;                 // 8-wide tiles of O
  extern __shared__ __align__(128) uint8_t dm_raw[];
  // (tiles start on 1024 bytes: the 128-byte swizzle of a TMA box is a function of the
  // shared-memory address, and the index arithmetic below assumes a tile starts a pattern)
  uint8_t* dm_smem = dm_raw + ((1024 - (smem_u32(dm_raw) & 1023)) & 1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, qd = lane & 3;
  const int head = blockIdx.x, row = blockIdx.y;
  const int kv_head = head / group;

  uint8_t* ring = dm_smem + (size_t)warp * DM_STAGES * 2 * TILE_BYTES;
  float* merge = reinterpret_cast<float*>(dm_smem + (size_t)DM_WARPS * DM_STAGES * 2 * TILE_BYTES);
  int* table_s = reinterpret_cast<int*>(merge + DM_WARPS * (HD + 2));  // table_room entries
  // one barrier per stage of this warp's ring (TMA only), behind the table on 8 bytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(table_s + DM_TABLE_ROOM) + warp * DM_STAGES;
  bool gave_up = false;
  if (TMA) {
    if (lane == 0) {
#pragma unroll
      for (int st = 0; st < DM_STAGES; ++st) mbar_init(&bars[st], 1);
      mbar_fence_init();
    }
    __syncwarp();
  }

  pdl_launch_dependents();
  const int req = __ldg(request_of_row + row);
  __nv_bfloat16* dst = out + (size_t)row * ld_out + (size_t)head * HD;
  if (req < 0) {  // a padding row: zeros (uniform over the CTA)
    pdl_wait();
    for (int d = threadIdx.x; d < HD; d += DM_WARPS * 32) dst[d] = __float2bfloat16(0.f);
    return;
  }
  const int pos = __ldg(positions + row);
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int nkeys = pos + 1 - lo;
  const int tiles = (nkeys + DM_TILE - 1) / DM_TILE;
  const int my_tiles = tiles > warp ? (tiles - warp + DM_WARPS - 1) / DM_WARPS : 0;
  const int* table = block_table + (size_t)req * table_stride;
  // The row's pages, once, into shared memory: a table entry fetched where a tile's copies
  // are issued is a trip to L2 (0.7 microseconds, measured with cycle stamps) ahead of every
  // tile, five times in a row for a warp of a 528-key context. Contexts of more pages than
  // the launch made room for keep the direct lookups.
  const int page_lo = page_shift >= 0 ? lo >> page_shift : lo / page_size;
  const int page_hi = page_shift >= 0 ? pos >> page_shift : pos / page_size;
  const bool table_held = page_hi - page_lo < table_room;
  if (table_held) {
    for (int i = threadIdx.x; i <= page_hi - page_lo; i += DM_WARPS * 32) {
      table_s[i] = __ldg(table + page_lo + i);
    }
    __syncthreads();
  }
  auto page_at = [&](int page_index) {
    return table_held ? table_s[page_index - page_lo] : __ldg(table + page_index);
  };
  const size_t head_off = (size_t)kv_head * page_size * HD;
  const size_t page_elems = (size_t)num_kv_heads * page_size * HD;
  const bool patch = k_new != nullptr;  // the row's own key and value are not in the cache yet

  // tile i of this warp -> stage i % DM_STAGES: each lane copies PIECES / 2 pieces of K and of
  // V (16 keys x PIECES pieces over 32 lanes), rows swizzled by piece ^ (key & 7)
  auto issue = [&](int i) {
    const int tile = warp + i * DM_WARPS;
    uint8_t* k_tile = ring + (size_t)(i % DM_STAGES) * 2 * TILE_BYTES;
    uint8_t* v_tile = k_tile + TILE_BYTES;
    if (TMA) {
      // the tile's 16 keys lie in one page (a page is a multiple of 16 keys and the first key
      // is key 0): one box of 16 rows of K and one of V, whatever of them is beyond the row
      if (lane == 0) {
        const int key = tile * DM_TILE;
        const int page_index = page_shift >= 0 ? key >> page_shift : key / page_size;
        const int slot = key - page_index * page_size;
        const int first = (page_at(page_index) * num_kv_heads + kv_head) * page_size + slot;
        uint64_t* bar = &bars[i % DM_STAGES];
        mbar_expect_tx(bar, 2 * TILE_BYTES);
        tma_load_2d(k_tile, &map_k, bar, 0, first);
        tma_load_2d(v_tile, &map_v, bar, 0, first);
      }
      return;
    }
#pragma unroll
    for (int j = 0; j < PIECES / 2; ++j) {
      const int idx = j * 32 + lane;
      const int key_in_tile = idx / PIECES, piece = idx % PIECES;
      const int key = lo + tile * DM_TILE + key_in_tile;
      // outside the row's keys, and the row's own key when it comes from k_new: zero fill
      const bool valid = key <= pos && !(patch && key == pos);
      size_t off = 0;
      if (valid) {
        const int page_index = page_shift >= 0 ? key >> page_shift : key / page_size;
        const int slot = page_shift >= 0 ? key & (page_size - 1) : key - page_index * page_size;
        off = (size_t)page_at(page_index) * page_elems + head_off + (size_t)slot * HD +
              (size_t)piece * 8;
      }
      const int swz = (piece & ~7) | ((piece ^ key_in_tile) & 7);
      const int at = key_in_tile * ROW_BYTES + swz * 16;
      dm_cp_async_16(k_tile + at, k_pages + off, valid);
      dm_cp_async_16(v_tile + at, v_pages + off, valid);
    }
  };

  // Keys of earlier steps do not depend on the kernel ahead: the first stages start before
  // the wait. That holds only while the row's own key comes from k_new; when it is read from
  // the cache, the kernel ahead is the one that wrote it there, and the wait comes first.
  if (!patch) pdl_wait_for(q, k_pages, v_pages);
#pragma unroll
  for (int i = 0; i < DM_STAGES; ++i) {  // every stage: a stage is refilled once it is used
    if (i < my_tiles) issue(i);
    if (!TMA) dm_commit();
  }
  if (patch) pdl_wait_for(q, k_new, v_new);

  // the query row as the A operand: rows other than row 0 of the 16 are zero
  uint32_t qa[KSTEPS][2];
  {
    const __nv_bfloat16* q_row = q + (size_t)row * ld_q + (size_t)head * HD;
#pragma unroll
    for (int s = 0; s < KSTEPS; ++s) {
      qa[s][0] = g == 0 ? *reinterpret_cast<const uint32_t*>(q_row + s * 16 + 2 * qd) : 0u;
      qa[s][1] = g == 0 ? *reinterpret_cast<const uint32_t*>(q_row + s * 16 + 8 + 2 * qd) : 0u;
    }
  }
  const float scale_log2 = scale * 1.4426950408889634f;

  float o[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  float run_max = -INFINITY, run_sum = 0.f;

  for (int i = 0; i < my_tiles; ++i) {
    const int tile = warp + i * DM_WARPS;
    uint8_t* k_tile = ring + (size_t)(i % DM_STAGES) * 2 * TILE_BYTES;
    uint8_t* v_tile = k_tile + TILE_BYTES;
    if (TMA) {
      if (!mbar_wait(&bars[i % DM_STAGES], (uint32_t)(i / DM_STAGES) & 1u)) gave_up = true;
      if (tile == tiles - 1) {
        // what the boxes brought from beyond the row (slots not written yet, or another
        // request's leavings) must not meet the zero weights of its keys: 0 x NaN is NaN
        const int have = pos - tile * DM_TILE + 1;  // keys of the row in this tile, 1 to 16
#pragma unroll
        for (int j = 0; j < PIECES / 2; ++j) {
          const int idx = j * 32 + lane;
          if (idx / PIECES >= have) {
            *reinterpret_cast<uint4*>(k_tile + idx * 16) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(v_tile + idx * 16) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
    } else {
      dm_wait<DM_STAGES - 1>();  // DM_STAGES + i groups committed: the first i + 1 are done
    }
    __syncwarp();  // every lane's copies of this tile have landed
    if (patch && tile == tiles - 1) {
      // the row's own key and value: from the projection's output into the tile (and the
      // cache); the copy above left their 16-byte pieces zero
      const int key_in_tile = pos - lo - tile * DM_TILE;
      if (lane < PIECES) {
        const uint4 kv = *reinterpret_cast<const uint4*>(k_new + (size_t)row * ld_new +
                                                         (size_t)kv_head * HD + lane * 8);
        const uint4 vv = *reinterpret_cast<const uint4*>(v_new + (size_t)row * ld_new +
                                                         (size_t)kv_head * HD + lane * 8);
        const int swz = (lane & ~7) | ((lane ^ key_in_tile) & 7);
        *reinterpret_cast<uint4*>(k_tile + key_in_tile * ROW_BYTES + swz * 16) = kv;
        *reinterpret_cast<uint4*>(v_tile + key_in_tile * ROW_BYTES + swz * 16) = vv;
        if (k_store != nullptr && head == kv_head * group) {  // one head of a group stores
          const int page_index = page_shift >= 0 ? pos >> page_shift : pos / page_size;
          const int slot = pos - page_index * page_size;
          const size_t off = (size_t)page_at(page_index) * page_elems + head_off +
                             (size_t)slot * HD + (size_t)lane * 8;
          *reinterpret_cast<uint4*>(k_store + off) = kv;
          *reinterpret_cast<uint4*>(v_store + off) = vv;
        }
      }
    }
    __syncwarp();

    // ---- S = q K^T: two tiles of 8 keys, KSTEPS k-steps each ---------------------------
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      // four 8x8 matrices: keys 0-7 dims 16ks..+7, keys 0-7 dims 16ks+8.., keys 8-15 likewise
      uint32_t b[4];
      const int m = lane >> 3, r = lane & 7;
      const int key_in_tile = (m >> 1) * 8 + r;
      const int piece = ks * 2 + (m & 1);
      const int swz = (piece & ~7) | ((piece ^ key_in_tile) & 7);
      dm_ldmatrix_x4(b, k_tile + key_in_tile * ROW_BYTES + swz * 16);
      dm_mma(s0, qa[ks][0], 0u, qa[ks][1], 0u, b[0], b[1]);
      dm_mma(s1, qa[ks][0], 0u, qa[ks][1], 0u, b[2], b[3]);
    }
    // lanes 0-3 hold the real row: keys 2qd, 2qd + 1 (s0) and 8 + 2qd, 8 + 2qd + 1 (s1)
    const int base = lo + tile * DM_TILE;
    float p[4];
    p[0] = base + 2 * qd <= pos ? s0[0] * scale_log2 : -INFINITY;
    p[1] = base + 2 * qd + 1 <= pos ? s0[1] * scale_log2 : -INFINITY;
    p[2] = base + 8 + 2 * qd <= pos ? s1[0] * scale_log2 : -INFINITY;
    p[3] = base + 8 + 2 * qd + 1 <= pos ? s1[1] * scale_log2 : -INFINITY;
    float tile_max = fmaxf(fmaxf(p[0], p[1]), fmaxf(p[2], p[3]));
    tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
    tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
    // (every tile a warp is given holds at least one key of the row, so the maximum of the
    // real row is finite; the other quads work on rows of zeros and are never read)
    const float new_max = fmaxf(run_max, tile_max);
    const float alpha = exp2f(run_max - new_max);
    run_max = new_max;
#pragma unroll
    for (int j = 0; j < 4; ++j) p[j] = exp2f(p[j] - new_max);
    run_sum = run_sum * alpha + (p[0] + p[1] + p[2] + p[3]);
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      o[t][0] *= alpha;
      o[t][1] *= alpha;
    }
    // ---- O += P V: P is the score accumulator where it lies (rows 8-15 are never read) ---
    const uint32_t pa0 = dm_pack(p[0], p[1]), pa2 = dm_pack(p[2], p[3]);
#pragma unroll
    for (int t2 = 0; t2 < NT / 2; ++t2) {
      // transposed 8x8 matrices: keys 0-7 / 8-15 of dims 16 t2 .. + 7 and 16 t2 + 8 .. + 15
      uint32_t b[4];
      const int m = lane >> 3, r = lane & 7;
      const int key_in_tile = (m & 1) * 8 + r;
      const int piece = t2 * 2 + (m >> 1);
      const int swz = (piece & ~7) | ((piece ^ key_in_tile) & 7);
      dm_ldmatrix_x4_trans(b, v_tile + key_in_tile * ROW_BYTES + swz * 16);
      dm_mma(o[2 * t2], pa0, 0u, pa2, 0u, b[0], b[1]);
      dm_mma(o[2 * t2 + 1], pa0, 0u, pa2, 0u, b[2], b[3]);
    }
    __syncwarp();  // every lane has read the stage: it takes the tile DM_STAGES on
    if (i + DM_STAGES < my_tiles) issue(i + DM_STAGES);
    if (!TMA) dm_commit();
  }

  // ---- merge the warps' shares (warp order) -----------------------------------------
  run_sum += __shfl_xor_sync(0xffffffffu, run_sum, 1);
  run_sum += __shfl_xor_sync(0xffffffffu, run_sum, 2);
  float* mine = merge + warp * (HD + 2);
  if (g == 0) {
    if (qd == 0) {
      mine[0] = run_max;
      mine[1] = run_sum;
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      mine[2 + t * 8 + 2 * qd] = o[t][0];
      mine[2 + t * 8 + 2 * qd + 1] = o[t][1];
    }
  }
  __syncthreads();
  for (int d = threadIdx.x; d < HD; d += DM_WARPS * 32) {
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) top = fmaxf(top, merge[w * (HD + 2)]);
    float denom = 0.f, sum = 0.f;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) {
      const float wm = merge[w * (HD + 2)];
      if (wm != -INFINITY) {
        const float f = exp2f(wm - top);
        denom += merge[w * (HD + 2) + 1] * f;
        sum += merge[w * (HD + 2) + 2 + d] * f;
      }
    }
    dst[d] = __float2bfloat16_rn(sum / denom);
  }
  if (TMA && gave_up) atomicExch(status, AYK_WAIT_TIMEOUT);
}

// Tensor maps of the cache pages as rows of one key each ([pages * kv_heads * page_size,
// head size], 128-byte swizzle, boxes of 16 rows), encoded once per cache tensor.
struct DmMapKey {
  const void* base;
  uint64_t rows;
  bool operator==(const DmMapKey& o) const { return base == o.base && rows == o.rows; }
};
struct DmMapKeyHash {
  size_t operator()(const DmMapKey& k) const { return (size_t)k.base * 1000003u ^ k.rows; }
};
inline int dm_cached_map(const void* base, uint64_t rows, int head_dim, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<DmMapKey, CUtensorMap, DmMapKeyHash> cache;
  std::lock_guard<std::mutex> lock(mu);
  const DmMapKey key{base, rows};
  auto it = cache.find(key);
  if (it == cache.end()) {
    CUtensorMap map;
    const int r = make_map_128b(&map, base, rows, (uint64_t)head_dim, (uint64_t)head_dim,
                                DM_TILE, 2);
    if (r != AYK_OK) return r;
    if (cache.size() > 4096) cache.clear();
    it = cache.emplace(key, map).first;
  }
  *out = it->second;
  return AYK_OK;
}

// `num_pages` (0 if the caller does not know): with it, head size 64, pages of a multiple of
// 16 tokens and no window, the tiles come by TMA.
template <int HD, int DM_WARPS>
int launch_decode_mma(const void* q, int ld_q, const void* k_pages, const void* v_pages,
                      const int* block_table, int table_stride, const int* request_of_row,
                      const int* positions, void* out, int ld_out, int num_rows, int num_heads,
                      int num_kv_heads, int page_size, float scale, int window,
                      const void* k_new, const void* v_new, int ld_new, int store,
                      int num_pages, int* status, cudaStream_t stream) {
  using bf = __nv_bfloat16;
  // room for the pages of a row: the table's width, up to DM_TABLE_ROOM entries
  const int table_room = table_stride < DM_TABLE_ROOM ? table_stride : DM_TABLE_ROOM;
  const size_t smem = (size_t)DM_WARPS * DM_STAGES * 2 * DM_TILE * HD * 2 +
                      (size_t)DM_WARPS * (HD + 2) * sizeof(float) +
                      (size_t)DM_TABLE_ROOM * sizeof(int) + (size_t)DM_WARPS * DM_STAGES * 8 +
                      1024;
  const long long rows_of_cache = (long long)num_pages * num_kv_heads * page_size;
  const bool tma = HD == 64 && num_pages > 0 && page_size % DM_TILE == 0 && window == 0 &&
                   status != nullptr && rows_of_cache < (1ll << 31) &&
                   ((uintptr_t)k_pages % 128) == 0 && ((uintptr_t)v_pages % 128) == 0;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_mma_kernel<HD, DM_WARPS, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess && HD == 64) {
      e = cudaFuncSetAttribute(attention_decode_mma_kernel<HD, DM_WARPS, HD == 64>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0) {
    page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
  }
  CUtensorMap map_k = {}, map_v = {};
  if (tma) {
    int r = dm_cached_map(k_pages, (uint64_t)rows_of_cache, HD, &map_k);
    if (r == AYK_OK) r = dm_cached_map(v_pages, (uint64_t)rows_of_cache, HD, &map_v);
    if (r != AYK_OK) return r;
  }
  auto kernel = tma ? attention_decode_mma_kernel<HD, DM_WARPS, HD == 64>
                    : attention_decode_mma_kernel<HD, DM_WARPS, false>;
  return launch_kernel(kernel, dim3(num_heads, num_rows), dim3(DM_WARPS * 32), smem, stream, 1,
                       map_k, map_v, status, (const bf*)q, ld_q, (const bf*)k_pages,
                       (const bf*)v_pages, block_table, table_stride, request_of_row, positions,
                       (bf*)out, ld_out, num_kv_heads, num_heads / num_kv_heads, page_size,
                       page_shift, scale, window, (const bf*)k_new, (const bf*)v_new, ld_new,
                       store ? (bf*)const_cast<void*>(k_pages) : (bf*)nullptr,
                       store ? (bf*)const_cast<void*>(v_pages) : (bf*)nullptr, table_room);
}

// Warps per (row, head). While one round of sixteen-warp CTAs holds every pair (at most one
// pair an SM), sixteen: the pair's keys are then spread over as many warps as one CTA can hold
// rings for. Else four or eight: the CTAs of either kind make ceil(pairs / resident) rounds
// over the device (shared memory allows 4 four-warp or 2 eight-warp CTAs of head size 64 per
// SM, half as many of head size 128), and a round of eight-warp CTAs takes about 0.7 of a
// round of four-warp ones. Measured with the tiles fetched by TMA, GPT-2 XL (25 heads, 528
// keys), decode step in ms with four / eight / sixteen warps: 1 request 1.27 / 1.19 / 1.15,
// 2: 1.29 / 1.19 / 1.20, 4: 1.33 / 1.28 / 1.26, 8: 1.51 / 1.41 / 1.54, 12: 1.98 / 1.99 / 2.14,
// 16: 2.03 / 2.17 / 2.38, 24: 2.97 / 3.03 / 3.27, 32: 3.17 / 3.30 / 3.64, 64: 4.13 / 4.37 /
// 5.15; the rule picks the fastest of each but at 2 requests (level).
inline int decode_mma_warps(long long pairs, int head_dim) {
  const long long sms = sm_count();
  if (head_dim <= 64 && pairs <= sms) return 16;
  const long long per_sm4 = head_dim <= 64 ? 4 : 2, per_sm8 = head_dim <= 64 ? 2 : 1;
  const long long rounds4 = (pairs + per_sm4 * sms - 1) / (per_sm4 * sms);
  const long long rounds8 = (pairs + per_sm8 * sms - 1) / (per_sm8 * sms);
  return rounds8 * 70 < rounds4 * 100 ? 8 : 4;
}

}  // namespace ayk
