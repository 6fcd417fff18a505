// Paged attention for decode rows: one query row per request, keys split over several CTAs.
//
// A decode step reads every cached key and value of every live request once; with one row
// per request there is no reuse, so the kernel is built to keep many loads in flight and to
// spend few instructions per key. grid = (splits, heads, requests). The request's keys are cut
// into splits * 4 contiguous shares, one per warp; the four warps of a CTA never wait for one
// another. TPK lanes of a warp share one key (8 elements of head_dim each, one 16-byte piece
// of the key and one of the value); a lane works on a batch of keys at a time — scores, one
// update of its running maximum and sum (online softmax) and the weighted values, all in fp32
// — while cp.async copies of the next three batches are in flight into the lane's own strip
// of shared memory (a queue nobody else reads, so it needs no barrier). Block-table entries sit one per lane and travel by shuffle, so no load of a key
// waits on a load of a table entry. Only at the end are the lanes', then the warps' shares
// folded together.
//
// Each CTA ends with (max, sum, weighted values) of its share. Up to 8 splits form a
// thread-block cluster and rank 0 merges the shares through distributed shared memory after
// one cluster barrier. With scratch memory (required beyond 8 splits) every CTA writes its
// share there and the CTA that finishes last for a (request, head) — found with an atomic
// ticket — merges them. Either way the shares are merged in split order. With splits == 1
// nothing is merged.
//
// Scratch: partial [requests * heads * splits * (head_dim + 2)] floats and one int ticket
// per (request, head), zero before the first launch and left zero by every launch.
// Cache layout: [page][kv_head][slot][head_dim]; block-table entry 0 = no page.
#include <mutex>

#include "tc_common.cuh"
#include "attention_decode_mma.cuh"

namespace ayk {

constexpr int DEC_WARPS = 4;
constexpr int DEC_THREADS = DEC_WARPS * 32;
// Batches whose copies are in flight ahead of the arithmetic. Measured on a B200 inside a
// decode layer (GPT-2 XL shapes, 768 keys): one batch ahead beats two and three at 8 and 64
// rows (47 / 124 against 51 / 140 microseconds a layer) — a shallow queue is 32 KB of shared
// memory per CTA, six CTAs per SM, and the many resident warps hide more latency than a
// deep queue of few warps does. Filling both stages of the strip before the wait (and
// requesting a batch's successor only once the batch is in registers) was slower too: 39.4
// against 37.5 microseconds a layer at 8 rows, 129 against 113 at 64.
#ifndef AYK_DEC_DEPTH
#define AYK_DEC_DEPTH 1
#endif
constexpr int DEC_DEPTH = AYK_DEC_DEPTH;
// Resident CTAs per SM the register allocation is held to: 80 registers a thread at six (a
// few spilled words), 94 unbounded, which leaves room for five. Measured in a decode layer of
// GPT-2 XL: 34.2 against 36.8 microseconds at 8 rows, 112.9 against 116.5 at 64.
#ifndef AYK_DEC_MIN_CTAS
#define AYK_DEC_MIN_CTAS 6
#endif

template <typename T> struct Frag8;
template <> struct Frag8<float> {
  static __device__ __forceinline__ void copy(float* dst, const float* src) {
    *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
    *reinterpret_cast<float4*>(dst + 4) = *reinterpret_cast<const float4*>(src + 4);
  }
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void load2(const float* p, float& a, float& b) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x;
    b = v.y;
  }
};
template <> struct Frag8<__nv_bfloat16> {
  static __device__ __forceinline__ void copy(__nv_bfloat16* dst, const __nv_bfloat16* src) {
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
  }
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void load2(const __nv_bfloat16* p, float& a, float& b) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
    a = __uint_as_float(w << 16);
    b = __uint_as_float(w & 0xffff0000u);
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

// 8 consecutive elements as they lie in memory (16 bytes of bfloat16, 32 bytes of float32).
template <typename T> struct Raw8;
template <> struct Raw8<__nv_bfloat16> {
  uint4 v;
  __device__ __forceinline__ void fetch(const __nv_bfloat16* p) {
    v = __ldg(reinterpret_cast<const uint4*>(p));
  }
  // `stride`: 16-byte units between the pieces of one value (one piece here)
  __device__ __forceinline__ void from_shared(const uint4* p, int stride) { v = p[0]; }
  __device__ __forceinline__ void zero() { v = make_uint4(0u, 0u, 0u, 0u); }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const {
    *reinterpret_cast<uint4*>(p) = v;
  }
  __device__ __forceinline__ void widen(float* f) const {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};
template <> struct Raw8<float> {
  float4 a, b;
  __device__ __forceinline__ void fetch(const float* p) {
    a = __ldg(reinterpret_cast<const float4*>(p));
    b = __ldg(reinterpret_cast<const float4*>(p + 4));
  }
  __device__ __forceinline__ void from_shared(const uint4* p, int stride) {
    const uint4 lo = p[0], hi = p[stride];
    a = make_float4(__uint_as_float(lo.x), __uint_as_float(lo.y), __uint_as_float(lo.z),
                    __uint_as_float(lo.w));
    b = make_float4(__uint_as_float(hi.x), __uint_as_float(hi.y), __uint_as_float(hi.z),
                    __uint_as_float(hi.w));
  }
  __device__ __forceinline__ void zero() {
    a = make_float4(0.f, 0.f, 0.f, 0.f);
    b = a;
  }
  __device__ __forceinline__ void store(float* p) const {
    *reinterpret_cast<float4*>(p) = a;
    *reinterpret_cast<float4*>(p + 4) = b;
  }
  __device__ __forceinline__ void widen(float* f) const {
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
};

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N> __device__ __forceinline__ void cp_async_wait_group() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void dec_cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void dec_cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void dec_st_cluster(uint32_t address, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(address), "f"(v) : "memory");
}

template <typename T, int TPK, int BATCH>
__global__ void __launch_bounds__(DEC_THREADS, AYK_DEC_MIN_CTAS)
attention_decode_kernel(const T* __restrict__ q, int ld_q, const T* __restrict__ k_pages,
                        const T* __restrict__ v_pages, const int* __restrict__ block_table,
                        int table_stride, const int* __restrict__ request_of_row,
                        const int* __restrict__ positions, T* __restrict__ out, int ld_out,
                        int num_kv_heads, int group, int head_dim, int page_size, float scale,
                        int window, float* __restrict__ partial, int* __restrict__ tickets,
                        const T* __restrict__ k_new, const T* __restrict__ v_new, int ld_new,
                        T* __restrict__ k_store, T* __restrict__ v_store, int clustered,
                        int page_shift) {
  constexpr int SLOTS = 32 / TPK;          // keys a warp covers per pass
  constexpr int STEP = SLOTS * BATCH;      // keys a warp covers per batch
  __shared__ float s_m[DEC_WARPS][TPK], s_l[DEC_WARPS][TPK];  // each warp's (max, sum) ...
  __shared__ float s_wacc[DEC_WARPS][TPK][8];                 // ... and weighted values
  __shared__ float c_share[2 + 256];         // this CTA's (max, sum, weighted values)
  __shared__ int s_last;

  pdl_launch_dependents();
  // Before the wait for the kernel ahead, only what no kernel of this step writes is touched:
  // the step's metadata (copied in before the step's first kernel) and the keys and values
  // of earlier steps. The queries, the step's own key and value, and every store come after.
  const int split = blockIdx.x, splits = gridDim.x;
  const int head = blockIdx.y, num_heads = gridDim.y;
  const int row = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sub = lane % TPK;   // which 8 elements of head_dim
  const int slot = lane / TPK;  // which key of a pass
  const bool dims_ok = sub * 8 < head_dim;
  const int req = request_of_row[row];
  const int pos = positions[row];
  T* dst = out + (size_t)row * ld_out + (size_t)head * head_dim;
  if (req < 0) {  // a padding row: zeros, no scratch, no ticket
    pdl_wait();
    if (split == 0) {
      for (int d = tid; d < head_dim; d += DEC_THREADS) stf(dst + d, 0.f);
    }
    return;
  }
  // "this CTA runs": awaited before any CTA of the cluster writes into another's shared memory
  if (clustered) dec_cluster_arrive();
  const int kv_head = head / group;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  // the request's keys lo..pos are cut into splits * warps contiguous shares, a multiple of
  // a batch each (so every warp but the last works on full batches)
  const int num_shares = splits * DEC_WARPS;
  int share = (pos + 1 - lo + num_shares - 1) / num_shares;
  share = (share + STEP - 1) / STEP * STEP;
  const int k_lo = lo + (split * DEC_WARPS + warp) * share;
  const int k_hi = k_lo + share < pos + 1 ? k_lo + share : pos + 1;
  const int* table = block_table + (size_t)req * table_stride;

  // key -> (page index, slot): a shift and a mask when the page size is a power of two (an
  // integer division costs more instructions than all the arithmetic on a key)
  const int page_mask = page_size - 1;
  auto page_of = [&](int key) { return page_shift >= 0 ? key >> page_shift : key / page_size; };
  auto slot_of = [&](int key) { return page_shift >= 0 ? key & page_mask : key % page_size; };
  // the warp's slice of the block table: one entry per lane, handed around by shuffles, so
  // that no load of a key waits on a load of a table entry (refilled every 32 pages)
  int first_page = page_of(k_lo);
  int my_entry = 0;
  auto refill_table = [&](int from_page) {
    first_page = from_page;
    // (a warp whose share holds no key loads nothing: its first page may lie beyond the
    // request's row of the table)
    const int last_page = k_hi > k_lo ? page_of(k_hi - 1) : from_page - 1;
    my_entry = from_page + lane <= last_page ? table[from_page + lane] : 0;
  };
  refill_table(first_page);

  float run_max = -INFINITY, run_sum = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  const size_t head_off = (size_t)kv_head * page_size * head_dim + (size_t)sub * 8;
  const size_t page_elems = (size_t)num_kv_heads * page_size * head_dim;
  const bool patch = k_new != nullptr && pos >= k_lo && pos < k_hi;

  // Each lane copies exactly the 16-byte pieces it will read itself (its keys' and values'
  // 8 elements) with cp.async into a private strip of shared memory, DEC_DEPTH batches ahead
  // of the arithmetic: a first-in-first-out queue that needs no barrier, because nobody else
  // ever looks at a lane's strip. Strip layout: [stage][key of batch][K, V][lane], 16-byte
  // pieces (two per lane and kind for float32), so copies and reads are conflict-free.
  constexpr int PIECES = sizeof(T) == 2 ? 1 : 2;  // 16-byte pieces per 8 elements
  extern __shared__ __align__(16) unsigned char dec_smem[];
  uint4* strip = reinterpret_cast<uint4*>(dec_smem) +
                 (size_t)warp * (DEC_DEPTH + 1) * BATCH * 2 * PIECES * 32;
  // where rank 0 of a cluster receives the CTAs' shares: [split][2 + head_dim] floats
  float* recv = reinterpret_cast<float*>(reinterpret_cast<uint4*>(dec_smem) +
                                         (size_t)DEC_WARPS * (DEC_DEPTH + 1) * BATCH * 2 *
                                             PIECES * 32);
  auto piece = [&](int stage, int u, int kind, int part) {
    return strip + ((((size_t)stage * BATCH + u) * 2 + kind) * PIECES + part) * 32 + lane;
  };
  auto issue = [&](int base, int stage) {
    // all lanes take part in the shuffles; a batch never spans more than 32 pages
    if (page_of(base + STEP - 1) - first_page >= 32) refill_table(page_of(base));
#pragma unroll
    for (int u = 0; u < BATCH; ++u) {
      const int key = base + u * SLOTS + slot;
      const int page = __shfl_sync(0xffffffffu, my_entry, (page_of(key) - first_page) & 31);
      const bool valid = key < k_hi && dims_ok;
      const bool own = patch && key == pos;  // this row's own key: from the projection
      const size_t off = (size_t)page * page_elems + head_off + (size_t)slot_of(key) * head_dim;
      const size_t fresh = (size_t)row * ld_new + (size_t)kv_head * head_dim + sub * 8;
      const T* k_from = own ? k_new + fresh : k_pages + (valid ? off : 0);
      const T* v_from = own ? v_new + fresh : v_pages + (valid ? off : 0);
#pragma unroll
      for (int part = 0; part < PIECES; ++part) {
        cp_async_16(piece(stage, u, 0, part), reinterpret_cast<const uint4*>(k_from) + part,
                    valid);
        cp_async_16(piece(stage, u, 1, part), reinterpret_cast<const uint4*>(v_from) + part,
                    valid);
      }
      if (own && valid && k_store != nullptr && head % group == 0) {
        // the fused KV store: the first head of a group also puts them into the cache
        Raw8<T> kr, vr;
        kr.fetch(k_new + fresh);
        vr.fetch(v_new + fresh);
        kr.store(k_store + off);
        vr.store(v_store + off);
      }
    }
    cp_async_commit_group();
  };
  const int num_batches = k_hi > k_lo ? (k_hi - k_lo + STEP - 1) / STEP : 0;
  // The first batches start before the wait. This step's token (position pos, the last key of
  // the share that holds it, so in that share's last batch) is written during this step, by
  // this kernel or by the one that fills the cache this run reads: its batch waits.
  const bool newest_here = pos >= k_lo && pos < k_hi;
  const int early = newest_here ? num_batches - 1 : num_batches;
#pragma unroll
  for (int b = 0; b < DEC_DEPTH; ++b) {
    if (b < early) issue(k_lo + b * STEP, b);
  }
  // The strip's last stage is free until the loop's first pass would fill it: when that batch
  // is an earlier step's too and the share is short, it goes out now, before the wait, and the
  // first pass skips it. Measured in a decode layer of GPT-2 XL: 24.4 against 25.0
  // microseconds at 1 row (shares of 2 batches), level at 8 rows (3 batches), and a loss at
  // 64 rows (12 batches a share: 114.4 against 113.0), hence the limit.
  const bool one_more = DEC_DEPTH < early && num_batches <= 4;
  if (one_more) issue(k_lo + DEC_DEPTH * STEP, DEC_DEPTH);
  pdl_wait_for(q, k_new, v_new, k_pages, v_pages);
  Raw8<T> q_raw;
  q_raw.zero();
  if (dims_ok) q_raw.fetch(q + (size_t)row * ld_q + (size_t)head * head_dim + sub * 8);
#pragma unroll
  for (int b = 0; b < DEC_DEPTH; ++b) {
    if (b >= early) {
      if (b < num_batches) issue(k_lo + b * STEP, b); else cp_async_commit_group();
    }
  }
  float qf[8];
  q_raw.widen(qf);
#pragma unroll
  for (int i = 0; i < 8; ++i) qf[i] *= scale;
  for (int b = 0; b < num_batches; ++b) {
    const int base = k_lo + b * STEP;
    const int stage = b % (DEC_DEPTH + 1);
    if (b + DEC_DEPTH < num_batches && !(one_more && b == 0)) {
      issue(k_lo + (b + DEC_DEPTH) * STEP, (b + DEC_DEPTH) % (DEC_DEPTH + 1));
    } else {
      cp_async_commit_group();  // keeps the group count in step
    }
    cp_async_wait_group<DEC_DEPTH>();  // batch b has landed (this lane's own pieces)
    float s[BATCH], vf[BATCH][8];
#pragma unroll
    for (int u = 0; u < BATCH; ++u) {
      Raw8<T> kr, vr;
      kr.from_shared(piece(stage, u, 0, 0), 32);
      vr.from_shared(piece(stage, u, 1, 0), 32);
      float kf[8];
      kr.widen(kf);
      vr.widen(vf[u]);
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) dot = fmaf(qf[i], kf[i], dot);
      s[u] = dot;
    }
#pragma unroll
    for (int o = TPK / 2; o > 0; o >>= 1) {
#pragma unroll
      for (int u = 0; u < BATCH; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
    }
    float top = run_max;
#pragma unroll
    for (int u = 0; u < BATCH; ++u) {
      if (base + u * SLOTS + slot >= k_hi) s[u] = -INFINITY;
      top = fmaxf(top, s[u]);
    }
    const float ref = top == -INFINITY ? 0.f : top;
    const float corr = expf(run_max - ref);
    run_max = top;
    run_sum *= corr;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= corr;
#pragma unroll
    for (int u = 0; u < BATCH; ++u) {
      const float p = expf(s[u] - ref);  // exp(-inf) = 0 for the keys that are not there
      run_sum += p;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(p, vf[u][i], acc[i]);
    }
  }
  cp_async_wait_group<0>();
  // the key slots of the warp that share `sub` fold together
#pragma unroll
  for (int o = TPK; o < 32; o <<= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, run_max, o);
    const float ol = __shfl_xor_sync(0xffffffffu, run_sum, o);
    float oacc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) oacc[i] = __shfl_xor_sync(0xffffffffu, acc[i], o);
    merge_state(run_max, run_sum, acc, om, ol, oacc);
  }
  if (lane < TPK) {
    s_m[warp][lane] = run_max;
    s_l[warp][lane] = run_sum;
#pragma unroll
    for (int i = 0; i < 8; ++i) s_wacc[warp][lane][i] = acc[i];
  }
  __syncthreads();
  if (clustered) dec_cluster_wait();  // every CTA of the cluster has started
  // fold the warps' shares, in warp order, into (max, sum, weighted values[head_dim]): into
  // c_share, or with a cluster straight into this CTA's row of rank 0's `recv`
  const uint32_t remote = clustered
      ? peer_address(recv + (size_t)split * (head_dim + 2), 0u) : 0u;
  if (tid < TPK) {
    float m = -INFINITY, l = 0.f, total[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) total[i] = 0.f;
    for (int w = 0; w < DEC_WARPS; ++w) {
      merge_state(m, l, total, s_m[w][tid], s_l[w][tid], s_wacc[w][tid]);
    }
    if (clustered) {
      if (tid == 0) {
        dec_st_cluster(remote, m);
        dec_st_cluster(remote + 4, l);
      }
      if (tid * 8 < head_dim) {
#pragma unroll
        for (int i = 0; i < 8; ++i) dec_st_cluster(remote + (2 + tid * 8 + i) * 4, total[i]);
      }
    } else {
      if (tid == 0) { c_share[0] = m; c_share[1] = l; }
      if (tid * 8 < head_dim) {
#pragma unroll
        for (int i = 0; i < 8; ++i) c_share[2 + tid * 8 + i] = total[i];
      }
    }
  }
  if (clustered) {
    // the splits of one (request, head) are the CTAs of one cluster: every CTA has written
    // its share into rank 0's shared memory, and after one cluster barrier rank 0 merges them
    // from there, in rank order; no scratch, no tickets, no remote load
    dec_cluster_arrive();
    dec_cluster_wait();
    if (split != 0) return;
    float m[8], l[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      m[s] = s < splits ? recv[s * (head_dim + 2)] : -INFINITY;
      l[s] = s < splits ? recv[s * (head_dim + 2) + 1] : 0.f;
    }
    float top = -INFINITY;
#pragma unroll
    for (int s = 0; s < 8; ++s) top = fmaxf(top, m[s]);
    float w[8], denom = 0.f;
#pragma unroll
    for (int s = 0; s < 8; ++s) {  // rank order: the sum does not change from run to run
      w[s] = m[s] == -INFINITY ? 0.f : expf(m[s] - top);
      denom += l[s] * w[s];
    }
    const float inv = 1.f / denom;
    for (int d = tid; d < head_dim; d += DEC_THREADS) {
      float sum = 0.f;
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        if (s < splits) sum += recv[s * (head_dim + 2) + 2 + d] * w[s];
      }
      stf(dst + d, sum * inv);
    }
    return;
  }
  __syncthreads();
  if (splits == 1) {
    const float inv = 1.f / c_share[1];
    for (int d = tid; d < head_dim; d += DEC_THREADS) stf(dst + d, c_share[2 + d] * inv);
    return;
  }
  // through scratch: every CTA stores its share; the last one to finish merges them
  float* mine = partial + (((size_t)row * num_heads + head) * splits + split) * (head_dim + 2);
  for (int d = tid; d < head_dim + 2; d += DEC_THREADS) mine[d] = c_share[d];
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int ticket = atomicAdd(&tickets[(size_t)row * num_heads + head], 1);
    s_last = ticket == splits - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* shares = partial + ((size_t)row * num_heads + head) * splits * (head_dim + 2);
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
  if (tid == 0) tickets[(size_t)row * num_heads + head] = 0;  // ready for the next launch
}

template <typename T, int TPK>
int launch_decode(const void* q, int ld_q, const void* k_pages, const void* v_pages,
                  const int* block_table, int table_stride, const int* request_of_row,
                  const int* positions, void* out, int ld_out, int num_rows, int num_heads,
                  int num_kv_heads, int head_dim, int page_size, float scale, int window,
                  int splits, float* partial, int* tickets, const void* k_new,
                  const void* v_new, int ld_new, int store, cudaStream_t stream) {
  constexpr int BATCH = sizeof(T) == 2 ? 4 : 2;  // keys a lane works on at a time
  dim3 grid(splits, num_heads, num_rows);
  // up to 8 splits given no scratch run as one thread-block cluster and merge on chip; with
  // scratch (needed beyond 8 splits) the shares go through global memory and a ticket
  const int clustered = (splits > 1 && splits <= 8 && partial == nullptr) ? 1 : 0;
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0) {
    page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
  }
  // every lane's strip: (depth + 1) stages x batch keys x (K, V) x 16 or 32 bytes
  const size_t strips = (size_t)DEC_THREADS * (DEC_DEPTH + 1) * BATCH * 2 * 8 * sizeof(T);
  // ... and with a cluster the room where rank 0 receives the shares
  const size_t smem = strips + (clustered ? (size_t)splits * (head_dim + 2) * sizeof(float) : 0);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<T, TPK, BATCH>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(strips + 8 * (256 + 2) * sizeof(float)));
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_kernel_x(attention_decode_kernel<T, TPK, BATCH>, grid, dim3(DEC_THREADS), smem,
                         stream, clustered ? splits : 1, (const T*)q, ld_q, (const T*)k_pages,
                         (const T*)v_pages, block_table, table_stride, request_of_row, positions,
                         (T*)out, ld_out, num_kv_heads, num_heads / num_kv_heads, head_dim,
                         page_size, scale, window, partial, tickets, (const T*)k_new,
                         (const T*)v_new, ld_new,
                         store ? (T*)const_cast<void*>(k_pages) : (T*)nullptr,
                         store ? (T*)const_cast<void*>(v_pages) : (T*)nullptr, clustered,
                         page_shift);
}

// bfloat16 rows with a head size the tensor-core kernel is built for go there
// (attention_decode_mma.cuh) whatever their number: it needs no cluster to merge its shares
// and a sixth of the instructions. Measured, GPT-2 XL decode step in ms against the split-KV
// kernel above: 1 request 1.16 / 1.22, 2: 1.20 / 1.27, 4: 1.32 / 1.50, 8: 1.48 / 1.64, 64:
// 4.61 / 4.82. The split-KV kernel serves float32, the other head sizes and callers that bring
// scratch.

// Off: every call goes to the split-KV kernel (tests of that kernel at the sizes the
// tensor-core kernel would take; measurements of one against the other).
inline int& decode_tensor_cores() {
  static int on = 1;
  return on;
}

template <typename T>
int attention_decode(const void* q, int ld_q, const void* k_pages, const void* v_pages,
                     const int* block_table, int table_stride, const int* request_of_row,
                     const int* positions, void* out, int ld_out, int num_rows, int num_heads,
                     int num_kv_heads, int head_dim, int page_size, float scale, int window,
                     int splits, float* partial, int* tickets, const void* k_new,
                     const void* v_new, int ld_new, int store, int* status, int num_pages,
                     cudaStream_t stream) {
  if (num_rows == 0) return AYK_OK;
  if ((k_new == nullptr) != (v_new == nullptr) || (store && k_new == nullptr)) {
    return AYK_BAD_ARGUMENT;
  }
  if (k_new != nullptr && (((uintptr_t)k_new % (8 * sizeof(T))) ||
                           ((uintptr_t)v_new % (8 * sizeof(T))) ||
                           ((size_t)ld_new * sizeof(T)) % (8 * sizeof(T)))) {
    return AYK_BAD_ALIGNMENT;
  }
  if (num_rows < 0 || num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads ||
      page_size < 1 || table_stride < 1 || window < 0 ||
      (splits < 1 && splits != -1 && splits != -4 && splits != -8 && splits != -16)) {
    return AYK_BAD_ARGUMENT;
  }
  if (head_dim < 16 || head_dim % 16) return AYK_BAD_ARGUMENT;
  if (head_dim > 256 || num_heads > 65535 || num_rows > 65535 || splits > 1024) {
    return AYK_TOO_LARGE;
  }
  if ((partial == nullptr) != (tickets == nullptr)) return AYK_BAD_ARGUMENT;
  if (splits > 8 && partial == nullptr) return AYK_BAD_ARGUMENT;
  const size_t vec = 8 * sizeof(T);
  if (((uintptr_t)k_pages % 16) || ((uintptr_t)v_pages % 16) || ((uintptr_t)q % vec) ||
      ((size_t)ld_q * sizeof(T)) % vec) {
    return AYK_BAD_ALIGNMENT;
  }
  // splits == -1 (or -4, -8, -16: with that many warps per CTA) asks for the tensor-core
  // kernel and fails if it does not serve the case (tests); otherwise it is taken whenever
  // it serves the case, whatever `splits` says
  const long long pairs = (long long)num_rows * num_heads;
  const bool asked = splits == -1 || splits == -4 || splits == -8 || splits == -16;
  if (asked || (partial == nullptr && decode_tensor_cores())) {
    if (sizeof(T) == 2 && (head_dim == 64 || head_dim == 128) && partial == nullptr) {
      int warps = splits < -1 ? -splits : decode_mma_warps(pairs, head_dim);
      if (head_dim > 64 && warps > 8) warps = 8;  // sixteen rings of head size 128 do not fit
#define AYK_DECODE_MMA(HD, W)                                                                  \
  return launch_decode_mma<HD, W>(q, ld_q, k_pages, v_pages, block_table, table_stride,       \
                                  request_of_row, positions, out, ld_out, num_rows, num_heads, \
                                  num_kv_heads, page_size, scale, window, k_new, v_new,        \
                                  ld_new, store, num_pages, status, stream)
      if (head_dim == 64 && warps == 16) AYK_DECODE_MMA(64, 16);
      if (head_dim == 64 && warps == 8) AYK_DECODE_MMA(64, 8);
      if (head_dim == 64) AYK_DECODE_MMA(64, 4);
      if (warps == 8) AYK_DECODE_MMA(128, 8);
      AYK_DECODE_MMA(128, 4);
#undef AYK_DECODE_MMA
    }
    if (asked) return AYK_BAD_ARGUMENT;  // asked for, but not this kernel's case
  }
  const int frags = head_dim / 8;
#define AYK_DECODE(TPK)                                                                        \
  return launch_decode<T, TPK>(q, ld_q, k_pages, v_pages, block_table, table_stride,          \
                               request_of_row, positions, out, ld_out, num_rows, num_heads,   \
                               num_kv_heads, head_dim, page_size, scale, window, splits,      \
                               partial, tickets, k_new, v_new, ld_new, store, stream)
  if (frags <= 2) AYK_DECODE(2);
  if (frags <= 4) AYK_DECODE(4);
  if (frags <= 8) AYK_DECODE(8);
  if (frags <= 16) AYK_DECODE(16);
  AYK_DECODE(32);
#undef AYK_DECODE
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }
AYK_API void ayk_set_decode_tensor_cores(int on) { ayk::decode_tensor_cores() = on; }

// type: 0 = float32, 1 = bfloat16. Up to 8 splits need no scratch (pass null for `partial`
// and `tickets`); with scratch, `partial` holds num_rows * num_heads * splits * (head_dim + 2)
// floats and `tickets` num_rows * num_heads zeroed ints. With k_new/v_new ([rows, kv_heads *
// head_dim], row stride ld_new) each row's own key and value are read from there instead of
// the cache, and with `store` they are also written into the row's cache slot (the step's KV
// store, fused). `num_pages` is the number of pages k_pages and v_pages hold (0 if the caller
// does not know): with it the tensor-core kernel fetches its tiles by TMA where the layout
// allows, and a wait of that path that runs out is reported through `status`.
AYK_API int ayk_attention_decode(const void* q, int ld_q, const void* k_pages,
                                 const void* v_pages, const int* block_table, int table_stride,
                                 const int* request_of_row, const int* positions, void* out,
                                 int ld_out, int num_rows, int num_heads, int num_kv_heads,
                                 int head_dim, int page_size, float scale, int window,
                                 int splits, float* partial, int* tickets, const void* k_new,
                                 const void* v_new, int ld_new, int store, int* status,
                                 int type, void* stream, int num_pages) {
  if (type == 0) {
    return ayk::attention_decode<float>(q, ld_q, k_pages, v_pages, block_table, table_stride,
                                        request_of_row, positions, out, ld_out, num_rows,
                                        num_heads, num_kv_heads, head_dim, page_size, scale,
                                        window, splits, partial, tickets, k_new, v_new, ld_new,
                                        store, status, num_pages, (cudaStream_t)stream);
  }
  if (type == 1) {
    return ayk::attention_decode<__nv_bfloat16>(
        q, ld_q, k_pages, v_pages, block_table, table_stride, request_of_row, positions, out,
        ld_out, num_rows, num_heads, num_kv_heads, head_dim, page_size, scale, window, splits,
        partial, tickets, k_new, v_new, ld_new, store, status, num_pages, (cudaStream_t)stream);
  }
  return AYK_BAD_ARGUMENT;
}

// ---- an entry point that allocates nothing (see attention_decode_noalloc.h) ---------------
#include "attention_decode_noalloc.h"

namespace ayk {

constexpr size_t NOALLOC_PARTIAL_FLOATS = size_t(1) << 20;  // 4 MiB of partial results
constexpr size_t NOALLOC_TICKETS = size_t(1) << 14;         // one int per (row, head)
constexpr size_t NOALLOC_BYTES = NOALLOC_PARTIAL_FLOATS * sizeof(float) +
                                 NOALLOC_TICKETS * sizeof(int);

// The scratch itself: part of the library's device image, so loading the library is what
// reserves it. In host code this name is only a handle for cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char decode_scratch[NOALLOC_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;

// The array's address on the current device, looked up once per device.
static int noalloc_scratch(unsigned char** out) {
  static std::mutex mu;
  static unsigned char* address[NOALLOC_MAX_DEVICES] = {};
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= NOALLOC_MAX_DEVICES) return AYK_TOO_LARGE;
  std::lock_guard<std::mutex> lock(mu);
  if (address[device] == nullptr) {
    void* found = nullptr;
    e = cudaGetSymbolAddress(&found, decode_scratch);
    if (e != cudaSuccess) return (int)e;
    if (found == nullptr) return AYK_DRIVER;
    address[device] = static_cast<unsigned char*>(found);
  }
  *out = address[device];
  return AYK_OK;
}

}  // namespace ayk

AYK_API void ayk_attention_decode_noalloc_limits(size_t* partial_floats, size_t* tickets) {
  if (partial_floats != nullptr) *partial_floats = ayk::NOALLOC_PARTIAL_FLOATS;
  if (tickets != nullptr) *tickets = ayk::NOALLOC_TICKETS;
}

AYK_API int ayk_attention_decode_noalloc(const void* q, int ld_q, const void* k_pages,
                                         const void* v_pages, const int* block_table,
                                         int table_stride, const int* request_of_row,
                                         const int* positions, void* out, int ld_out,
                                         int num_rows, int num_heads, int num_kv_heads,
                                         int head_dim, int page_size, float scale, int window,
                                         int splits, int type, void* stream) {
  using namespace ayk;
  if (num_rows == 0) return AYK_OK;
  if (num_rows < 0 || num_heads < 1 || head_dim < 1 || splits < 1) return AYK_BAD_ARGUMENT;
  const size_t pairs = (size_t)num_rows * (size_t)num_heads;
  const size_t floats = pairs * (size_t)splits * (size_t)(head_dim + 2);
  if (pairs > NOALLOC_TICKETS || floats > NOALLOC_PARTIAL_FLOATS) return AYK_TOO_LARGE;
  unsigned char* base = nullptr;
  const int found = noalloc_scratch(&base);
  if (found != AYK_OK) return found;
  float* partial = reinterpret_cast<float*>(base);
  int* tickets = reinterpret_cast<int*>(base + NOALLOC_PARTIAL_FLOATS * sizeof(float));
  cudaStream_t s = (cudaStream_t)stream;
  // the tickets must start at zero whatever an earlier call (perhaps one that failed) left
  cudaError_t e = cudaMemsetAsync(tickets, 0, pairs * sizeof(int), s);
  if (e != cudaSuccess) return (int)e;
  int unused_status = 0;  // the kernel never touches it
  if (type == 0) {
    return attention_decode<float>(q, ld_q, k_pages, v_pages, block_table, table_stride,
                                   request_of_row, positions, out, ld_out, num_rows, num_heads,
                                   num_kv_heads, head_dim, page_size, scale, window, splits,
                                   partial, tickets, nullptr, nullptr, 0, 0, &unused_status, 0, s);
  }
  if (type == 1) {
    return attention_decode<__nv_bfloat16>(
        q, ld_q, k_pages, v_pages, block_table, table_stride, request_of_row, positions, out,
        ld_out, num_rows, num_heads, num_kv_heads, head_dim, page_size, scale, window, splits,
        partial, tickets, nullptr, nullptr, 0, 0, &unused_status, 0, s);
  }
  return AYK_BAD_ARGUMENT;
}
