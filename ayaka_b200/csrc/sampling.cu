// Token choice from fp32 logits [rows, vocab] (row stride ld, any vocab).
//
// argmax: the largest logit, the smallest id among equals; NaN never wins.
//
// sample: per row, temperature, top-k, top-p, min-p and one draw by the inverse CDF over the
// canonical order (probability descending, id ascending), with the random number computed
// in the kernel from (seed, position) by Philox-4x32-10: u = (word0 >> 8) / 2^24.
// No sort: the order is walked by radix selection. Every logit x/T maps to an order-preserving
// 32-bit key; a selection descends the key 8 bits at a time over per-warp histograms of
// (count, mass) and stops at the element where the running count or mass passes a target.
// Mass is exp(x/T - max) as a 2^40 fixed-point integer, so sums are exact and do not depend
// on the order of addition: the same row and the same u always give the same token.
//   top-k  : the k-th element by count; its prefix has mass Z_k.
//   top-p  : the first element whose cumulative mass reaches top_p * Z_k ends the prefix.
//   min-p  : elements with mass below min_p * (largest mass) are dropped.
//   draw   : the first element whose cumulative mass exceeds u * (mass of the kept prefix).
// Equal keys (equal logits) are ordered by id. A row with temperature < 1e-5 or top_k == 1 is
// greedy.
#include "common.cuh"

namespace ayk {

constexpr int SMP_THREADS = 512;
constexpr int SMP_WARPS = SMP_THREADS / 32;
constexpr float SMP_ONE = 1099511627776.0f;  // 2^40

__device__ __forceinline__ void better(float& bv, int& bi, float ov, int oi) {
  if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
}

// Block-wide argmax with the smallest id on ties; result valid in every thread.
__device__ int block_argmax(const float* row, int vocab, float* sv, int* si) {
  float bv = -INFINITY;
  int bi = vocab;
  for (int c = threadIdx.x; c < vocab; c += blockDim.x) better(bv, bi, row[c], c);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    better(bv, bi, ov, oi);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < nwarps; ++w) better(bv, bi, sv[w], si[w]);
    si[0] = bi < vocab ? bi : 0;
  }
  __syncthreads();
  const int out = si[0];
  __syncthreads();
  return out;
}

__global__ void __launch_bounds__(256)
argmax_kernel(const float* __restrict__ logits, int ld, int vocab, int* __restrict__ out) {
  __shared__ float sv[8];
  __shared__ int si[8];
  pdl_launch_dependents();
  pdl_wait_for(logits);
  const int best = block_argmax(logits + (size_t)blockIdx.x * ld, vocab, sv, si);
  if (threadIdx.x == 0) out[blockIdx.x] = best;
}

// Two-stage argmax for steps where one CTA per row is too slow (a vocabulary of 50k floats is
// 200 KB per row): stage 1 splits every row over `parts` CTAs that each leave (value, id) of
// their slice; stage 2 folds the parts of a row. Ties go to the smaller id in both stages.
__global__ void __launch_bounds__(256)
argmax_parts_kernel(const float* __restrict__ logits, int ld, int vocab, int parts,
                    float* __restrict__ part_value, int* __restrict__ part_id) {
  __shared__ float sv[8];
  __shared__ int si[8];
  pdl_launch_dependents();
  pdl_wait_for(logits);
  const int row = blockIdx.x, part = blockIdx.y;
  const int span = (vocab + parts - 1) / parts;
  const int lo = part * span;
  const int hi = lo + span < vocab ? lo + span : vocab;
  const float* src = logits + (size_t)row * ld;
  float bv = -INFINITY;
  int bi = vocab;
  for (int c = lo + threadIdx.x; c < hi; c += blockDim.x) better(bv, bi, src[c], c);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    better(bv, bi, ov, oi);
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) better(bv, bi, sv[w], si[w]);
    part_value[row * parts + part] = bv;
    part_id[row * parts + part] = bi;
  }
}

__global__ void __launch_bounds__(32)
argmax_fold_kernel(const float* __restrict__ part_value, const int* __restrict__ part_id,
                   int parts, int vocab, int* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait_for(part_value, part_id);
  const int row = blockIdx.x;
  float bv = -INFINITY;
  int bi = vocab;
  for (int p = threadIdx.x; p < parts; p += 32) {
    better(bv, bi, part_value[row * parts + p], part_id[row * parts + p]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    better(bv, bi, ov, oi);
  }
  if (threadIdx.x == 0) out[row] = bi < vocab ? bi : 0;
}

// ---- Philox-4x32-10 -------------------------------------------------------------------
__device__ __forceinline__ uint32_t philox_word0(uint64_t seed, uint64_t position,
                                                 uint32_t stream, uint32_t sequence) {
  uint32_t c0 = (uint32_t)position, c1 = (uint32_t)(position >> 32), c2 = stream, c3 = sequence;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    if (r) { k0 += 0x9E3779B9u; k1 += 0xBB67AE85u; }
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    const uint32_t n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    const uint32_t n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
  }
  return c0;
}

// ---- keys and masses ------------------------------------------------------------------
__device__ __forceinline__ uint32_t order_key(float x) {
  if (x != x) return 0u;  // NaN sorts last
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ unsigned long long mass_of(float x, float top) {
  if (x != x) return 0ull;
  return (unsigned long long)(expf(x - top) * SMP_ONE);
}

struct SampleShared {
  unsigned long long mass[SMP_WARPS][256];
  unsigned int count[SMP_WARPS][256];
  unsigned long long scan_mass;
  unsigned int scan_count;
  unsigned int picked;
  unsigned int picked_count;
  unsigned long long red64[SMP_WARPS];
  unsigned int red32[SMP_WARPS];
  float sv[SMP_WARPS];
  int si[SMP_WARPS];
};

struct Found {
  uint32_t key;                    // key of the element found
  unsigned long long mass_above;   // mass of all elements with a larger key
  unsigned int count_above;        // their number
  unsigned int count_eq;           // elements with exactly this key
  unsigned long long mass_one;     // mass of one such element
};

// Find the element where the running (count or mass) first exceeds `target`, walking keys
// from the largest down. by_mass: running mass > target; else running count > target.
__device__ Found descend(const float* row, int vocab, float temp, float top, bool by_mass,
                         unsigned long long target, SampleShared& sh) {
  const int warp = threadIdx.x >> 5;
  uint32_t prefix = 0, mask = 0;
  unsigned long long mass_above = 0;
  unsigned int count_above = 0, count_eq = 0;
  for (int level = 0; level < 4; ++level) {
    const int shift = 24 - 8 * level;
    for (int i = threadIdx.x; i < SMP_WARPS * 256; i += blockDim.x) {
      (&sh.mass[0][0])[i] = 0ull;
      (&sh.count[0][0])[i] = 0u;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < vocab; c += blockDim.x) {
      const float x = __fdiv_rn(row[c], temp);
      const uint32_t key = order_key(x);
      if ((key & mask) == prefix) {
        const uint32_t digit = (key >> shift) & 255u;
        atomicAdd(&sh.count[warp][digit], 1u);
        atomicAdd(&sh.mass[warp][digit], mass_of(x, top));
      }
    }
    __syncthreads();
    if (threadIdx.x < 256) {
      unsigned long long m = 0;
      unsigned int n = 0;
      for (int w = 0; w < SMP_WARPS; ++w) {
        m += sh.mass[w][threadIdx.x];
        n += sh.count[w][threadIdx.x];
      }
      sh.mass[0][threadIdx.x] = m;
      sh.count[0][threadIdx.x] = n;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long run_mass = mass_above;
      unsigned int run_count = count_above;
      int pick = -1;
      for (int d = 255; d >= 0; --d) {
        const unsigned long long m = sh.mass[0][d];
        const unsigned int n = sh.count[0][d];
        if (n == 0) continue;
        const bool crosses = by_mass ? (run_mass + m > target)
                                     : ((unsigned long long)run_count + n > target);
        if (crosses) { pick = d; break; }
        run_mass += m;
        run_count += n;
      }
      if (pick < 0) {
        // the target lies beyond everything (rounding at the very end): take the last
        // non-empty bucket, i.e. the smallest keys
        run_mass = mass_above;
        run_count = count_above;
        for (int d = 255; d >= 0; --d) {
          if (sh.count[0][d] == 0) continue;
          if (pick >= 0) { run_mass += sh.mass[0][pick]; run_count += sh.count[0][pick]; }
          pick = d;
        }
        if (pick < 0) pick = 0;
      }
      sh.scan_mass = run_mass;
      sh.scan_count = run_count;
      sh.picked = (unsigned int)pick;
      sh.picked_count = sh.count[0][pick];
    }
    __syncthreads();
    mass_above = sh.scan_mass;
    count_above = sh.scan_count;
    count_eq = sh.picked_count;
    prefix |= sh.picked << shift;
    mask |= 255u << shift;
    __syncthreads();
  }
  Found f;
  f.key = prefix;
  f.mass_above = mass_above;
  f.count_above = count_above;
  f.count_eq = count_eq;
  f.mass_one = mass_of(key_value(prefix), top);
  return f;
}

__device__ unsigned long long block_sum_u64(unsigned long long v, SampleShared& sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh.red64[threadIdx.x >> 5] = v;
  __syncthreads();
  unsigned long long total = 0;
  for (int w = 0; w < SMP_WARPS; ++w) total += sh.red64[w];
  __syncthreads();
  return total;
}
__device__ unsigned int block_sum_u32(unsigned int v, SampleShared& sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh.red32[threadIdx.x >> 5] = v;
  __syncthreads();
  unsigned int total = 0;
  for (int w = 0; w < SMP_WARPS; ++w) total += sh.red32[w];
  __syncthreads();
  return total;
}

// The id of the (index)-th element, by ascending id, whose key equals `key`.
__device__ int nth_with_key(const float* row, int vocab, float temp, uint32_t key,
                            unsigned int index, SampleShared& sh) {
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int lo = threadIdx.x * chunk;
  const int hi = lo + chunk < vocab ? lo + chunk : vocab;
  unsigned int mine = 0;
  for (int c = lo; c < hi; ++c) mine += order_key(__fdiv_rn(row[c], temp)) == key;
  // exclusive prefix over threads: inside the warp by shuffles, across warps through shared
  unsigned int incl = mine;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned int up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  __syncthreads();
  if (lane == 31) sh.red32[warp] = incl;
  if (threadIdx.x == 0) sh.si[0] = -1;
  __syncthreads();
  unsigned int before = incl - mine;
  for (int w = 0; w < warp; ++w) before += sh.red32[w];
  if (index >= before && index < before + mine) {
    unsigned int seen = before;
    for (int c = lo; c < hi; ++c) {
      if (order_key(__fdiv_rn(row[c], temp)) == key) {
        if (seen == index) { sh.si[0] = c; break; }
        ++seen;
      }
    }
  }
  __syncthreads();
  const int out = sh.si[0];
  __syncthreads();
  return out;
}

__global__ void __launch_bounds__(SMP_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int vocab,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p,
              const long long* __restrict__ seeds, const long long* __restrict__ positions,
              int* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char sample_smem[];
  SampleShared& sh = *reinterpret_cast<SampleShared*>(sample_smem);
  pdl_launch_dependents();
  pdl_wait_for(logits);
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * ld;
  const float temp = temperature[r];
  int k = top_k != nullptr ? top_k[r] : 0;
  if (temp < 1e-5f || k == 1) {
    const int best = block_argmax(row, vocab, sh.sv, sh.si);
    if (threadIdx.x == 0) out[r] = best;
    return;
  }
  // the largest x / T
  float top = -INFINITY;
  for (int c = threadIdx.x; c < vocab; c += blockDim.x) {
    const float x = __fdiv_rn(row[c], temp);
    if (x > top) top = x;
  }
  top = warp_max(top);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh.sv[threadIdx.x >> 5] = top;
  __syncthreads();
  top = sh.sv[0];
  for (int w = 1; w < SMP_WARPS; ++w) top = fmaxf(top, sh.sv[w]);
  __syncthreads();

  const float pp = top_p != nullptr ? top_p[r] : 1.f;
  const float mp = min_p != nullptr ? min_p[r] : 0.f;

  // mass of the top-k prefix (or of everything)
  unsigned long long kept_mass;
  unsigned long long kept_count;
  if (k > 1 && k < vocab) {
    const Found f = descend(row, vocab, temp, top, false, (unsigned long long)(k - 1), sh);
    kept_mass = f.mass_above + (unsigned long long)(k - f.count_above) * f.mass_one;
    kept_count = (unsigned long long)k;
  } else {
    unsigned long long mine = 0;
    for (int c = threadIdx.x; c < vocab; c += blockDim.x) {
      mine += mass_of(__fdiv_rn(row[c], temp), top);
    }
    kept_mass = block_sum_u64(mine, sh);
    kept_count = (unsigned long long)vocab;
  }
  const unsigned long long mass_k = kept_mass;
  if (pp < 1.f) {
    unsigned long long want = (unsigned long long)((double)pp * (double)mass_k);
    if (want < 1) want = 1;
    if (want > mass_k) want = mass_k;
    const Found f = descend(row, vocab, temp, top, true, want - 1, sh);
    unsigned long long j = f.mass_one ? (want - 1 - f.mass_above) / f.mass_one : 0;
    if (j >= f.count_eq) j = f.count_eq ? f.count_eq - 1 : 0;
    const unsigned long long n = (unsigned long long)f.count_above + j + 1;
    if (n < kept_count) {
      kept_count = n;
      kept_mass = f.mass_above + (j + 1) * f.mass_one;
    }
  }
  if (mp > 0.f) {
    const unsigned long long floor_mass = (unsigned long long)ceil((double)mp * (double)SMP_ONE);
    unsigned long long m = 0;
    unsigned int n = 0;
    for (int c = threadIdx.x; c < vocab; c += blockDim.x) {
      const unsigned long long w = mass_of(__fdiv_rn(row[c], temp), top);
      if (w >= floor_mass) { m += w; ++n; }
    }
    m = block_sum_u64(m, sh);
    n = block_sum_u32(n, sh);
    if (n >= 1 && (unsigned long long)n < kept_count) {
      kept_count = n;
      kept_mass = m;
    }
  }
  // the draw: u = word >> 8 over 2^24; target = floor(u * kept_mass) in exact integers
  const uint32_t word = philox_word0((uint64_t)seeds[r], (uint64_t)positions[r], 0u, 0u);
  const unsigned long long u24 = (unsigned long long)(word >> 8);
  const unsigned long long hi = __umul64hi(kept_mass, u24);
  const unsigned long long lo = kept_mass * u24;
  const unsigned long long target = (hi << 40) | (lo >> 24);
  const Found f = descend(row, vocab, temp, top, true, target, sh);
  unsigned long long j = f.mass_one ? (target - f.mass_above) / f.mass_one : 0;
  if (j >= f.count_eq) j = f.count_eq ? f.count_eq - 1 : 0;
  // never past the kept prefix
  if ((unsigned long long)f.count_above + j >= kept_count) {
    j = kept_count > f.count_above ? kept_count - 1 - f.count_above : 0;
  }
  const int token = nth_with_key(row, vocab, temp, f.key, (unsigned int)j, sh);
  if (threadIdx.x == 0) out[r] = token >= 0 ? token : 0;
}

// ---------------------------------------------------------------------------------------
// What a request may ask to have done to its logits before the token is chosen, in the
// reference's fixed order (python/ayaka/ops/sampling.py:10-20, 166-200): a mask (only the
// allowed ids survive; banned ids — the stop ids while fewer than min_tokens tokens exist —
// go to -inf), then additive biases, then the three penalties from the request's own tokens:
//   x = x > 0 ? x / r : x * r   for tokens that occur in prompt or output   (repetition)
//   x = x - f * (occurrences in the output)                                   (frequency)
//   x = x - s                   for tokens that occur in the output           (presence)
// -inf stays -inf throughout. One CTA per adjusted row. A row is described by 16 int32 words
// in `desc` followed (anywhere in `desc`) by its lists; offsets are word indices into `desc`:
//   0 row of `logits`          1 history offset   2 history length   3 prompt length
//   4 bias offset              5 bias count (ids, then as many float values)
//   6 allowed offset           7 allowed count (-1: every id is allowed)
//   8 banned offset            9 banned count
//   10 repetition  11 frequency  12 presence (float bits)      13-15 unused
// The history is the request's prompt followed by its output. Counting is quadratic in the
// history (each thread looks for earlier copies of its tokens): a few microseconds at a
// thousand tokens, and nothing is kept between steps.
constexpr int ADJ_THREADS = 256;
constexpr int ADJ_WORDS = 16;

__global__ void __launch_bounds__(ADJ_THREADS)
logits_adjust_kernel(float* __restrict__ logits, int ld, int vocab,
                     const int* __restrict__ desc, unsigned* __restrict__ mask_scratch,
                     int mask_words) {
  pdl_launch_dependents();
  pdl_wait();
  const int* d = desc + blockIdx.x * ADJ_WORDS;
  float* x = logits + (size_t)d[0] * ld;
  const int* hist = desc + d[1];
  const int hist_len = d[2], prompt_len = d[3];
  const int* bias_ids = desc + d[4];
  const int bias_n = d[5];
  const float* bias_values = reinterpret_cast<const float*>(bias_ids + bias_n);
  const int* allowed = desc + d[6];
  const int allowed_n = d[7];
  const int* banned = desc + d[8];
  const int banned_n = d[9];
  const float rep = __int_as_float(d[10]), freq = __int_as_float(d[11]),
              pres = __int_as_float(d[12]);
  const int tid = threadIdx.x;

  if (allowed_n >= 0) {
    unsigned* mask = mask_scratch + (size_t)blockIdx.x * mask_words;
    for (int w = tid; w < mask_words; w += ADJ_THREADS) mask[w] = 0u;
    __syncthreads();
    for (int i = tid; i < allowed_n; i += ADJ_THREADS) {
      const int id = allowed[i];
      if (id >= 0 && id < vocab) atomicOr(&mask[id >> 5], 1u << (id & 31));
    }
    __syncthreads();
    for (int v = tid; v < vocab; v += ADJ_THREADS) {
      if (((mask[v >> 5] >> (v & 31)) & 1u) == 0u) x[v] = -INFINITY;
    }
    __syncthreads();
  }
  for (int i = tid; i < banned_n; i += ADJ_THREADS) {
    const int id = banned[i];
    if (id >= 0 && id < vocab) x[id] = -INFINITY;
  }
  __syncthreads();
  for (int i = tid; i < bias_n; i += ADJ_THREADS) {  // an id appears once
    const int id = bias_ids[i];
    if (id >= 0 && id < vocab) x[id] += bias_values[i];
  }
  __syncthreads();
  if (rep != 1.f || freq != 0.f || pres != 0.f) {
    for (int i = tid; i < hist_len; i += ADJ_THREADS) {
      const int token = hist[i];
      if (token < 0 || token >= vocab) continue;
      bool first = true;
      for (int j = 0; j < i; ++j) {
        if (hist[j] == token) {
          first = false;
          break;
        }
      }
      if (!first) continue;  // the thread of the first copy speaks for the token
      int in_output = i >= prompt_len ? 1 : 0;
      for (int j = i + 1; j < hist_len; ++j) {
        if (hist[j] == token && j >= prompt_len) ++in_output;
      }
      float v = x[token];
      v = v > 0.f ? v / rep : v * rep;
      v -= freq * (float)in_output;
      if (in_output > 0) v -= pres;
      x[token] = v;
    }
  }
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

AYK_API int ayk_argmax(const float* logits, int ld, int rows, int vocab, int* out, void* stream) {
  if (rows == 0) return AYK_OK;
  if (rows < 0 || vocab < 1 || ld < vocab) return AYK_BAD_ARGUMENT;
  return ayk::launch_kernel(ayk::argmax_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream,
                            1, logits, ld, vocab, out);
}

// The same result through two small kernels: `parts` CTAs per row, then a fold. `part_value`
// and `part_id` hold rows * parts entries each (scratch, any contents).
AYK_API int ayk_argmax_split(const float* logits, int ld, int rows, int vocab, int parts,
                             float* part_value, int* part_id, int* out, void* stream) {
  if (rows == 0) return AYK_OK;
  if (rows < 0 || vocab < 1 || ld < vocab || parts < 1 || part_value == nullptr ||
      part_id == nullptr) {
    return AYK_BAD_ARGUMENT;
  }
  if (parts > 65535 || rows > 0x7fffffff / parts) return AYK_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  int r = ayk::launch_kernel(ayk::argmax_parts_kernel, dim3(rows, parts), dim3(256), 0, s, 1,
                             logits, ld, vocab, parts, part_value, part_id);
  if (r != AYK_OK) return r;
  return ayk::launch_kernel(ayk::argmax_fold_kernel, dim3(rows), dim3(32), 0, s, 1,
                            (const float*)part_value, (const int*)part_id, parts, vocab, out);
}

// temperature [rows] fp32; top_k [rows] int32 (<= 0: off) or null; top_p, min_p [rows] fp32 or
// null; seeds, positions [rows] int64 (position = index of the token being produced).
AYK_API int ayk_sample(const float* logits, int ld, int rows, int vocab, const float* temperature,
                       const int* top_k, const float* top_p, const float* min_p,
                       const long long* seeds, const long long* positions, int* out,
                       void* stream) {
  if (rows == 0) return AYK_OK;
  if (rows < 0 || vocab < 1 || ld < vocab || temperature == nullptr || seeds == nullptr ||
      positions == nullptr) {
    return AYK_BAD_ARGUMENT;
  }
  static bool configured = false;
  const int bytes = (int)sizeof(ayk::SampleShared);
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(ayk::sample_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return ayk::launch_kernel(ayk::sample_kernel, dim3(rows), dim3(ayk::SMP_THREADS), bytes,
                            (cudaStream_t)stream, 1, logits, ld, vocab, temperature, top_k,
                            top_p, min_p, seeds, positions, out);
}

namespace ayk {
// x = scale * x, then with cap > 0: x = cap * tanh(x / cap), on rows of fp32 logits in place.
__global__ void logits_scale_cap_kernel(float* __restrict__ logits, int ld, int vocab,
                                        float scale, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  float* row = logits + (size_t)blockIdx.y * ld;
  const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < vocab; c += gridDim.x * blockDim.x) {
    float v = row[c] * scale;
    if (cap > 0.f) v = cap * tanhf(v * inv_cap);
    row[c] = v;
  }
}
}  // namespace ayk

// The head's output as some architectures want it: scaled, then squashed into (-cap, cap).
AYK_API int ayk_logits_scale_cap(float* logits, int ld, int vocab, int num_rows, float scale,
                                 float cap, void* stream) {
  using namespace ayk;
  if (num_rows == 0) return AYK_OK;
  if (num_rows < 0 || num_rows > 65535 || vocab < 1 || ld < vocab || logits == nullptr ||
      cap < 0.f) {
    return AYK_BAD_ARGUMENT;
  }
  const int blocks = (vocab + 1023) / 1024 < 64 ? (vocab + 1023) / 1024 : 64;
  return launch_kernel(logits_scale_cap_kernel, dim3(blocks, num_rows), dim3(256), 0,
                       (cudaStream_t)stream, 1, logits, ld, vocab, scale, cap);
}

// Adjust `num_rows` rows of fp32 logits in place as `desc` says (see logits_adjust_kernel).
// `mask_scratch` holds num_rows * ceil(vocab / 32) words (needed only by rows with an allowed
// list; may be null when no row has one).
AYK_API int ayk_logits_adjust(float* logits, int ld, int vocab, const int* desc, int num_rows,
                              unsigned* mask_scratch, void* stream) {
  using namespace ayk;
  if (num_rows == 0) return AYK_OK;
  if (num_rows < 0 || vocab < 1 || ld < vocab || logits == nullptr || desc == nullptr) {
    return AYK_BAD_ARGUMENT;
  }
  return launch_kernel(logits_adjust_kernel, dim3(num_rows), dim3(ADJ_THREADS), 0,
                       (cudaStream_t)stream, 1, logits, ld, vocab, desc, mask_scratch,
                       (vocab + 31) / 32);
}
