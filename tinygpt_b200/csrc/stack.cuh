// stack.cuh — launchers of the layer-stack engine's mechanisms (stack_ops.cu): every shape, bf16 or fp32 storage, fp32
// arithmetic wherever a value enters a norm, a softmax, a gate or the residual stream.
#pragma once
#include "common.cuh"

namespace b200 {

// What a general GEMM does with its fp32 row sums  (C[m, n] = Σ_k A[m, k]·W[n, k]).
enum StackEpi : int {
  SEPI_STORE = 0,     // C_T[m, n] = T(acc + bias[n])
  SEPI_STORE_F32 = 1, // C_f32[m, n] = acc + bias[n]
  SEPI_RESIDUAL = 2,  // X_f32[m, n] += mult · acc                  (projection into the residual stream)
  SEPI_ACT_TABLE = 3, // C_T[m, n] = T(gelu_tanh(acc) · table[tok[m]·table_ld + table_col + n])   (gated token table)
  SEPI_LOGITS = 4,    // C_f32[m, n] = acc and C2_bf16[m, n] = bf16(acc)    (fp32 logits + the sampler's bf16 copy)
};

bool stack_pdl();   // kernels of stack_ops.cu are launched under programmatic dependent launch unless B200_NO_PDL=1

struct StackGemm {
  // A is [M, K]: columns [0, k1) come from a, the rest from a2 (the [x; x0] concatenation without a copy).  a_f32: the
  // source is the fp32 residual stream, rounded to T when it is loaded (a bf16 product takes bf16 operands).
  const void* a = nullptr;
  const void* a2 = nullptr;
  int64_t lda = 0, lda2 = 0;
  int k1 = 0;          // columns served by a (= K when a2 is null)
  bool a_f32 = false;
  const void* w = nullptr;   // [N, K] row-major T
  const float* bias = nullptr;
  int M = 0, N = 0, K = 0;
  int epi = SEPI_STORE;
  void* c = nullptr;
  int64_t ldc = 0;
  __nv_bfloat16* c2 = nullptr;   // SEPI_LOGITS
  float mult = 1.f;              // SEPI_RESIDUAL
  const void* table = nullptr;   // SEPI_ACT_TABLE: T [vocab, table_ld]
  const int32_t* tok = nullptr;
  int64_t table_ld = 0;
  int table_col = 0;
  float softcap = 0.f;           // SEPI_LOGITS: > 0: acc <- cap·tanh(acc / cap) before it is stored
  // batched: `batch` independent products, item b reads a + b·sa, w + b·sw and writes c + b·sc (elements)
  int batch = 1;
  int64_t sa = 0, sw = 0, sc = 0;
  // grouped: the rows of A are sorted into groups, group e meets matrix w + e·sw.  The launch has n_tiles row tiles; tile i
  // serves rows [tile_row0[i], min(tile_row0[i] + 64, group_end[e])) of group e = tile_group[i], or nothing (−1).  The
  // three arrays live on the device (written by the routing kernels), so no step of this is decided on the host.
  const int32_t* tile_group = nullptr;
  const int32_t* tile_row0 = nullptr;
  const int32_t* group_end = nullptr;
  int n_tiles = 0;
};
int launch_stack_gemm(const StackGemm& g, int dtype, cudaStream_t st);

// y[r, :] = T(x[rows ? rows[r] : r, :] · rsqrt(mean(x²) + eps) · (offset + w))
int launch_stack_rmsnorm(void* y, const float* x, const float* w, const int32_t* rows_or_null, int64_t n_rows, int dim,
                         float eps, float offset, int dtype, cudaStream_t st);
int launch_stack_rms_add(float* x, const float* y, const float* w, int64_t rows, int dim, float eps, float mult,
                         cudaStream_t st);
int launch_stack_act_mul(void* y, int64_t ld_y, const void* g, const void* u, int64_t ld_gu, int64_t rows, int n, int act,
                         int dtype, cudaStream_t st);
// x0[t, :] = float(embed[tok[t], :]) · scale, and x = x0
int launch_stack_embed(float* x, float* x0, const void* embed, const int32_t* tok, int64_t n_tok, int vocab, int width,
                       float scale, int dtype, cudaStream_t st);

// ---- glue of the bf16 tensor-core / weight-streaming paths (engine_stack.cu picks them per product)
// y[r, j] = bf16(float(y[r, j]) + b[j])
int launch_stack_bias_add(__nv_bfloat16* y, const float* b, int64_t rows, int n, cudaStream_t st);
// x[i] = (add ? x[i] : 0) + mult · float(t[i])
int launch_stack_axpy(float* x, const __nv_bfloat16* t, float mult, bool add, int64_t total, cudaStream_t st);
// cat[r, :] = bf16([a[r, :] | b[r, :]]) (each `width` wide); zero_or_null[r, :] = 0
int launch_stack_cat_cast(__nv_bfloat16* cat, const float* a, const float* b, float* zero_or_null, int64_t rows, int width,
                          cudaStream_t st);

int launch_stack_rms_add_bf16(float* x, const __nv_bfloat16* y, const float* w, int64_t rows, int dim, float eps, float mult,
                              cudaStream_t st);
int launch_stack_cast(__nv_bfloat16* y, const float* x, int64_t total, cudaStream_t st);
// y[r, j] = bf16(gelu_tanh(g[r, j]) · table[tok[r], col + j])
int launch_stack_act_table(__nv_bfloat16* y, const __nv_bfloat16* g, const void* table, const int32_t* tok, int64_t table_ld,
                           int col, int64_t rows, int n, cudaStream_t st);

struct StackAttn {
  b200_attn_desc a{};
  const void* proj = nullptr;   // [n_tok, ld_proj] T: q at off_q (heads·dim), k at off_k, v at off_v, gate logits at off_g
  int64_t ld_proj = 0;
  int off_q = 0, off_k = 0, off_v = 0, off_g = 0;
  void* kcache = nullptr;       // this run's rows of slot 0: [max_ctx, kv_heads·dim]; slot s is s·k_slot_stride further
  void* vcache = nullptr;       // [max_ctx, kv_heads·vdim]
  int64_t k_slot_stride = 0, v_slot_stride = 0;
  const int32_t* slot = nullptr;
  const int32_t* pos = nullptr;
  int n_tok = 0;
  void* out = nullptr;          // [n_tok, ld_out] T, head h at columns h·vdim
  int64_t ld_out = 0;
  // split keys (decode steps over long key lists): nsplit CTAs per (token, head), each over keys_per_split entries of
  // the visible list, partial softmaxes [n_tok·heads][nsplit][2 + vdim] in split_ws; the CTA that finishes a pair last
  // (split_tickets [n_tok·heads], zero-initialised, self-resetting) merges them
  float* split_ws = nullptr;
  unsigned int* split_tickets = nullptr;
  // decode steps (every row the only new row of its sequence): the row's own key / value are read from proj and one
  // CTA per (row, kv head) appends them to the cache in the same launch — no separate kv_store
  int own_from_proj = 0;
  int nsplit = 1, keys_per_split = 0;
};
constexpr int kStackSplitRows = 16;    // most rows a split-key attention launch serves
constexpr int kStackSplitKeys = 128;   // keys per split
constexpr int kStackMaxSplits = 64;
int launch_stack_kv_store(const StackAttn& p, int dtype, cudaStream_t st);
int launch_stack_attention(const StackAttn& p, int dtype, cudaStream_t st);

}  // namespace b200
