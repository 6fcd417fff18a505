// Host code of a step: the launches of one layer half (norm + attention, norm + feed-forward)
// or of a whole run of layers, issued from C++ instead of one Python call per kernel.
//
// A step of a few hundred rows runs about 340 kernels of a few microseconds each; launched
// one by one through Python and ctypes they cost more on the host than on the device. Here
// a part's static arguments (weights, sizes, scratch buffers, the entry points of the kernels
// it uses) are packed once into a struct, the step's arguments into another, and one call
// walks the layers. The kernels are the same exported entry points the Python functions in
// kernels/ops.py call, reached through function pointers the loader hands over, so this file
// holds no device code and links against nothing; the choice of kernel for a product or an
// attention follows the same rules as ops.linear, ops.attention_prefill and
// parts/mixer.py (which remain for parts that this file does not know, and for tests that
// compare the two paths bit by bit).
//
// The reference keeps this layer in Python (python/ayaka/execution/runner.py:176-259 calls
// the model, which calls torch ops one by one) and hides it behind CUDA graphs for decode
// only; steps that hold prompt portions pay for it there as they did here.
#include <stdint.h>

#include "common.cuh"

namespace {

typedef int (*LayerNormFn)(const float*, int, const int*, const float*, const float*, float,
                           void*, int, int, int, void*);
typedef int (*GemmTcFn)(const void*, int, const void*, int, const float*, void*, int, int, int,
                        int, int, int, int, int*, void*);
typedef int (*GemmTcKvFn)(const void*, int, const void*, int, const float*, void*, int, int, int,
                          int, const int*, void*, void*, int, int, int, int, int, int*, void*);
typedef int (*GemmSimtFn)(const void*, int, const void*, int, const float*, void*, int, int, int,
                          int, int, int, int, int, void*);
typedef int (*KvStoreFn)(const void*, const void*, int, const int*, void*, void*, int, int, int,
                         int, int, void*);
typedef int (*AttnDecodeFn)(const void*, int, const void*, const void*, const int*, int,
                            const int*, const int*, void*, int, int, int, int, int, int, float,
                            int, int, float*, int*, const void*, const void*, int, int, int*,
                            int, void*, int);
typedef int (*AttnSimtFn)(const void*, int, const void*, const void*, const int*, int,
                          const int*, const int*, void*, int, int, int, int, int, int, float, int,
                          int, void*);
typedef int (*AttnPrefillFn)(const void*, int, const void*, const void*, const int*, int,
                             const int*, const int*, void*, int, int, int, int, int, int, int,
                             float, int, void*);
typedef int (*AttnPrefillTcFn)(const void*, int, const void*, const void*, const int*, int,
                               const int*, const int*, void*, int, int, int, int, int, int, int,
                               int, float, int, int*, void*);

}  // namespace

extern "C" {

// One cache group's view of the step (parts/context.py GroupStep).
struct AykGroupStep {
  const int* block_table;
  const int* slot_mapping;
  int table_stride;
  int page_size;
};

// One step (parts/context.py StepContext), plus the switches tests flip in kernels/ops.py.
struct AykStep {
  int num_rows;
  int num_requests;
  int decode_only;
  int max_kv_len;
  int sm_count;
  int decode_ctas_per_sm;
  int bf16_gemm_simt;    // 1: bfloat16 products on the CUDA-core kernel (ops.BF16_GEMM)
  int prefill_mma;       // 1: never the tcgen05 attention kernel (ops.PREFILL_ATTENTION)
  int tile_n;            // gemm_tc.TILE_N
  const int* positions;
  const int* request_of_row;
  const int* row_start;
  const int* kv_len;
  const int* host_rows;  // host copy: rows each request brings (grids are sized from it)
  int* status;
  void* stream;
  int num_groups;
  int launches;          // out: kernels launched through this struct so far
  AykGroupStep groups[8];
};

// Entry points a part may need (null where the library is not loaded: float32 models never
// load the tensor-core libraries).
struct AykKernels {
  void* layer_norm_f32;
  void* layer_norm_bf16;
  void* gemm_tc;
  void* gemm_tc_kv;
  void* gemm_simt;
  void* kv_store;
  void* attention_decode;
  void* attention_simt;
  void* attention_prefill;     // the warp-level kernel compiled for this part's head size
  void* attention_prefill_tc;
  void* attention_prefill_tc_rows;  // query rows per CTA of the kernel above
};

// norm + fused query/key/value projection + attention + output projection (parts/mixer.py)
struct AykAttentionPart {
  AykKernels k;
  int type;  // 0 = float32, 1 = bfloat16
  int width, num_heads, num_kv_heads, head_dim, window;
  float scale;
  float eps;
  int keys_as_projected;
  const float* norm_weight;
  const float* norm_bias;
  const void* qkv_weight;
  const float* qkv_bias;
  const void* out_weight;
  const float* out_bias;
  void* normed;    // [max_rows, width]
  void* qkv;       // [max_rows, q_width + 2 * kv_width]
  void* attended;  // [max_rows, q_width]
};

// norm + up projection with activation + down projection (parts/feed_forward.py)
struct AykMlpPart {
  AykKernels k;
  int type;
  int width, inner, activation;
  float eps;
  const float* norm_weight;
  const float* norm_bias;
  const void* up_weight;
  const float* up_bias;
  const void* down_weight;
  const float* down_bias;
  void* normed;     // [max_rows, width]
  void* inner_buf;  // [max_rows, inner]
};

// One entry of the execution order: a layer's two halves and the cache this run touches.
struct AykLayerRun {
  const AykAttentionPart* attention;
  const AykMlpPart* mlp;
  void* k_pages;
  void* v_pages;
  int num_pages;
  int group;
  int writes;
  int pad;
};

}  // extern "C"

namespace {

inline bool tma_readable(const void* a, int lda, const void* w, int ldw) {
  return ((uintptr_t)a % 16) == 0 && ((uintptr_t)w % 16) == 0 && lda % 8 == 0 && ldw % 8 == 0;
}

// ops.linear: bfloat16 on the tensor cores when TMA can read the operands, else (and for
// float32) the CUDA-core kernel. `residual`: out is fp32 and is added to.
int linear(const AykKernels& k, AykStep* step, int type, const void* a, int lda, const void* w,
           int ldw, const float* bias, void* out, int ldo, int out_type, int M, int N, int K,
           int act, int residual) {
  if (type == 1 && !step->bf16_gemm_simt && tma_readable(a, lda, w, ldw)) {
    if (k.gemm_tc == nullptr) return AYK_DRIVER;
    const int mode = residual ? 2 : (out_type == 1 ? 0 : 1);
    ++step->launches;
    return ((GemmTcFn)k.gemm_tc)(a, lda, w, ldw, bias, out, ldo, M, N, K, act, mode,
                                 step->tile_n, step->status, step->stream);
  }
  if (k.gemm_simt == nullptr) return AYK_DRIVER;
  ++step->launches;
  return ((GemmSimtFn)k.gemm_simt)(a, lda, w, ldw, bias, out, ldo, M, N, K, act, residual, type,
                                   out_type, step->stream);
}

int layer_norm(const AykKernels& k, AykStep* step, int type, const float* x, int ldx,
               const float* gamma, const float* beta, float eps, void* out, int ldo, int n,
               int width) {
  void* fn = type == 1 ? k.layer_norm_bf16 : k.layer_norm_f32;
  if (fn == nullptr) return AYK_DRIVER;
  ++step->launches;
  return ((LayerNormFn)fn)(x, ldx, nullptr, gamma, beta, eps, out, ldo, n, width, step->stream);
}

// parts/mixer.py leading_single_rows: requests at the head of the step that bring one row
// each, if there are at least LEADING_SINGLE_ROWS of them and something else follows
constexpr int LEADING_SINGLE_ROWS = 4;
int leading_single_rows(const AykStep* step) {
  int lead = 0;
  while (lead < step->num_requests && step->host_rows[lead] == 1) ++lead;
  return (lead >= LEADING_SINGLE_ROWS && lead < step->num_requests) ? lead : 0;
}

// sum over the step's requests from `first` on of ceil(rows / tile_rows), and the longest
// portion
int tiles_of(const AykStep* step, int tile_rows, int first) {
  int tiles = 0;
  for (int b = first; b < step->num_requests; ++b) {
    tiles += (step->host_rows[b] + tile_rows - 1) / tile_rows;
  }
  return tiles;
}
int longest_portion(const AykStep* step) {
  int longest = 0;
  for (int b = 0; b < step->num_requests; ++b) {
    if (step->host_rows[b] > longest) longest = step->host_rows[b];
  }
  return longest;
}

// ops.decode_splits
int decode_splits(const AykStep* step, int num_rows, int num_heads, int reach) {
  const int pairs = num_rows * num_heads > 0 ? num_rows * num_heads : 1;
  int splits = step->decode_ctas_per_sm * step->sm_count / pairs;
  const int enough_keys = reach / 128 > 1 ? reach / 128 : 1;
  if (splits > enough_keys) splits = enough_keys;
  if (splits > 8) splits = 8;
  if (splits < 1) splits = 1;
  while (splits & (splits - 1)) --splits;
  return splits;
}

int attention_half(const AykAttentionPart* p, AykStep* step, float* residual, void* k_pages,
                   void* v_pages, int num_pages, int group, int writes) {
  const AykKernels& k = p->k;
  const int n = step->num_rows;
  if (n == 0) return AYK_OK;
  if (group < 0 || group >= step->num_groups) return AYK_BAD_ARGUMENT;
  const AykGroupStep& g = step->groups[group];
  const int q_width = p->num_heads * p->head_dim;
  const int kv_width = p->num_kv_heads * p->head_dim;
  const int ld_qkv = q_width + 2 * kv_width;
  const int elem = p->type == 1 ? 2 : 4;
  int r = layer_norm(k, step, p->type, residual, p->width, p->norm_weight, p->norm_bias, p->eps,
                     p->normed, p->width, n, p->width);
  if (r != AYK_OK) return r;
  // the fused projection; prompt portions in bfloat16 store their keys and values from its
  // epilogue when the kernel can carry that
  bool stored = false;
  if (writes && !step->decode_only && p->keys_as_projected && p->type == 1 &&
      !step->bf16_gemm_simt && k.gemm_tc_kv != nullptr &&
      tma_readable(p->normed, p->width, p->qkv_weight, p->width)) {
    r = ((GemmTcKvFn)k.gemm_tc_kv)(p->normed, p->width, p->qkv_weight, p->width, p->qkv_bias,
                                   p->qkv, ld_qkv, n, ld_qkv, p->width, g.slot_mapping, k_pages,
                                   v_pages, q_width, kv_width, p->num_kv_heads, p->head_dim,
                                   g.page_size, step->status, step->stream);
    if (r == AYK_OK) {
      stored = true;
      ++step->launches;
    } else if (r != AYK_NOT_TAKEN) {
      return r;
    }
  }
  if (!stored) {
    r = linear(k, step, p->type, p->normed, p->width, p->qkv_weight, p->width, p->qkv_bias,
               p->qkv, ld_qkv, p->type, n, ld_qkv, p->width, ayk::ACT_NONE, 0);
    if (r != AYK_OK) return r;
  }
  const char* q = (const char*)p->qkv;
  const char* kk = q + (size_t)q_width * elem;
  const char* vv = kk + (size_t)kv_width * elem;
  if (writes && !step->decode_only && !stored) {
    if (k.kv_store == nullptr) return AYK_DRIVER;
    ++step->launches;
    r = ((KvStoreFn)k.kv_store)(kk, vv, ld_qkv, g.slot_mapping, k_pages, v_pages, n,
                                p->num_kv_heads, p->head_dim, g.page_size, p->type,
                                step->stream);
    if (r != AYK_OK) return r;
  }
  if (!step->decode_only && step->host_rows == nullptr) return AYK_BAD_ARGUMENT;
  if (step->decode_only) {
    int reach = step->max_kv_len;
    if (p->window > 0 && p->window < reach) reach = p->window;
    const int splits = decode_splits(step, n, p->num_heads, reach);
    if (k.attention_decode == nullptr) return AYK_DRIVER;
    ++step->launches;
    r = ((AttnDecodeFn)k.attention_decode)(
        q, ld_qkv, k_pages, v_pages, g.block_table, g.table_stride, step->request_of_row,
        step->positions, p->attended, q_width, n, p->num_heads, p->num_kv_heads, p->head_dim,
        g.page_size, p->scale, p->window, splits, nullptr, nullptr, writes ? kk : nullptr,
        writes ? vv : nullptr, writes ? ld_qkv : 0, writes ? 1 : 0, step->status, p->type,
        step->stream, num_pages);
  } else if (p->type == 1) {
    // leading single-row requests go to the decode kernel (their keys and values are in
    // the cache by now), the rest to a prompt kernel
    const int lead = leading_single_rows(step);
    if (lead > 0) {
      int reach = step->max_kv_len;
      if (p->window > 0 && p->window < reach) reach = p->window;
      if (k.attention_decode == nullptr) return AYK_DRIVER;
      ++step->launches;
      r = ((AttnDecodeFn)k.attention_decode)(
          q, ld_qkv, k_pages, v_pages, g.block_table, g.table_stride, step->request_of_row,
          step->positions, p->attended, q_width, lead, p->num_heads, p->num_kv_heads,
          p->head_dim, g.page_size, p->scale, p->window,
          decode_splits(step, lead, p->num_heads, reach), nullptr, nullptr, nullptr, nullptr, 0,
          0, step->status, p->type, step->stream, num_pages);
      if (r != AYK_OK) return r;
    }
    const int* table = g.block_table + (size_t)lead * g.table_stride;
    const bool tc = p->head_dim == 64 && p->scale > 0.f && !step->prefill_mma &&
                    k.attention_prefill_tc != nullptr &&
                    k.attention_prefill_tc_rows != nullptr && longest_portion(step) >= 256;
    ++step->launches;
    if (tc) {
      r = ((AttnPrefillTcFn)k.attention_prefill_tc)(
          q, ld_qkv, k_pages, v_pages, table, g.table_stride, step->row_start + lead,
          step->kv_len + lead, p->attended, q_width, step->num_requests - lead,
          tiles_of(step, ((int (*)())k.attention_prefill_tc_rows)(), lead), p->num_heads,
          p->num_kv_heads, p->head_dim, g.page_size, num_pages, p->scale, p->window,
          step->status, step->stream);
    } else {
      if (k.attention_prefill == nullptr) return AYK_DRIVER;
      r = ((AttnPrefillFn)k.attention_prefill)(
          q, ld_qkv, k_pages, v_pages, table, g.table_stride, step->row_start + lead,
          step->kv_len + lead, p->attended, q_width, step->num_requests - lead,
          tiles_of(step, 64, lead), p->num_heads, p->num_kv_heads, p->head_dim, g.page_size,
          p->scale, p->window, step->stream);
    }
  } else {
    if (k.attention_simt == nullptr) return AYK_DRIVER;
    ++step->launches;
    r = ((AttnSimtFn)k.attention_simt)(q, ld_qkv, k_pages, v_pages, g.block_table,
                                       g.table_stride, step->request_of_row, step->positions,
                                       p->attended, q_width, n, p->num_heads, p->num_kv_heads,
                                       p->head_dim, g.page_size, p->scale, p->window, p->type,
                                       step->stream);
  }
  if (r != AYK_OK) return r;
  return linear(k, step, p->type, p->attended, q_width, p->out_weight, q_width, p->out_bias,
                residual, p->width, 0, n, p->width, q_width, ayk::ACT_NONE, 1);
}

int mlp_half(const AykMlpPart* p, AykStep* step, float* residual) {
  const int n = step->num_rows;
  if (n == 0) return AYK_OK;
  int r = layer_norm(p->k, step, p->type, residual, p->width, p->norm_weight, p->norm_bias,
                     p->eps, p->normed, p->width, n, p->width);
  if (r != AYK_OK) return r;
  r = linear(p->k, step, p->type, p->normed, p->width, p->up_weight, p->width, p->up_bias,
             p->inner_buf, p->inner, p->type, n, p->inner, p->width, p->activation, 0);
  if (r != AYK_OK) return r;
  return linear(p->k, step, p->type, p->inner_buf, p->inner, p->down_weight, p->inner,
                p->down_bias, residual, p->width, 0, n, p->width, p->inner, ayk::ACT_NONE, 1);
}

}  // namespace

AYK_API void ayk_set_pdl(int) {}  // (every library has it; this one launches through the others)

// The struct sizes, so that the loader can check its mirror of them.
AYK_API void ayk_host_sizes(int* out) {
  out[0] = (int)sizeof(AykStep);
  out[1] = (int)sizeof(AykAttentionPart);
  out[2] = (int)sizeof(AykMlpPart);
  out[3] = (int)sizeof(AykLayerRun);
  out[4] = (int)sizeof(AykKernels);
}

AYK_API int ayk_host_attention(const AykAttentionPart* part, AykStep* step, float* residual,
                               void* k_pages, void* v_pages, int num_pages, int group,
                               int writes) {
  if (part == nullptr || step == nullptr || residual == nullptr) return AYK_BAD_ARGUMENT;
  return attention_half(part, step, residual, k_pages, v_pages, num_pages, group, writes);
}

AYK_API int ayk_host_mlp(const AykMlpPart* part, AykStep* step, float* residual) {
  if (part == nullptr || step == nullptr || residual == nullptr) return AYK_BAD_ARGUMENT;
  return mlp_half(part, step, residual);
}

// The runs of the execution order, one after the other. Returns the first non-zero status;
// *failed_at tells which run gave it.
AYK_API int ayk_host_layers(const AykLayerRun* runs, int count, AykStep* step, float* residual,
                            int* failed_at) {
  if (runs == nullptr || step == nullptr || residual == nullptr || count < 0) {
    return AYK_BAD_ARGUMENT;
  }
  for (int i = 0; i < count; ++i) {
    const AykLayerRun& run = runs[i];
    int r = attention_half(run.attention, step, residual, run.k_pages, run.v_pages,
                           run.num_pages, run.group, run.writes);
    if (r == AYK_OK) r = mlp_half(run.mlp, step, residual);
    if (r != AYK_OK) {
      if (failed_at != nullptr) *failed_at = i;
      return r;
    }
  }
  return AYK_OK;
}
