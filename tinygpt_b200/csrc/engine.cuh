// engine.cuh — the engine object behind the opaque b200_engine handle, shared by the Llama-family wiring (engine.cu) and
// the layer-stack models (engine_stack.cu).
#pragma once
#include <vector>

#include "gemv.cuh"
#include "ops.cuh"
#include "stack.cuh"

namespace b200 {
struct StackEngine;
static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
}  // namespace b200

struct b200_engine {
  b200_model_desc d{};
  int num_sms = 148;
  int qdim = 0, kvdim = 0, Hq_l = 0, Hkv_l = 0, I_l = 0, V_l = 0;  // local (per-rank) sizes
  // borrowed weights
  const __nv_bfloat16* embed = nullptr;
  const float* rope = nullptr;
  std::vector<b200_layer_weights> lw;
  // owned device memory
  uint8_t* arena = nullptr;
  size_t arena_bytes = 0;
  __nv_bfloat16 *kcache = nullptr, *vcache = nullptr;  // [L][max_ctx][Hkv_l][hd] each
  __nv_bfloat16 *x = nullptr, *qkv = nullptr, *attn = nullptr, *act = nullptr, *logits = nullptr;
  float* attn_ws = nullptr;
  unsigned int* attn_tickets = nullptr;
  void* argmax_ws = nullptr;
  int64_t* cur_tok = nullptr;   // token the next step consumes
  int64_t* gen_log = nullptr;   // ring of generated tokens
  int* pos = nullptr;           // position of the token in flight; advanced by the LAST kernel of each token, so it
                                // is stable (and readable ahead of griddepcontrol.wait) for the whole next token
  unsigned long long* gen_count = nullptr;
  int gen_cap = 0;
  int nsplit = 1;
  // plans
  std::vector<b200::GemvPlan> p_qkv, p_o, p_gu, p_down;
  b200::GemvPlan p_head{};
  // graphs
  cudaGraphExec_t g_step = nullptr;   // full token incl. lm_head + argmax
  cudaGraphExec_t g_body = nullptr;   // embed + layers only (prefill tokens whose logits nobody reads)
  // host mirrors
  int64_t h_pos = 0;
  int64_t h_gen = 0;
  int launches_per_token = 0;   // kernels of a head token (what the graph g_step launches)
  int launches_body = 0;        // kernels of a body-only token (g_body)
  // batched prefill (tcgen05 GEMM path), workspace allocated on first use
  uint8_t* pf_arena = nullptr;
  int pf_chunk = 0;  // tokens the workspace holds
  __nv_bfloat16 *pf_x = nullptr, *pf_h = nullptr, *pf_qkv = nullptr, *pf_attn = nullptr, *pf_gu = nullptr,
                *pf_act = nullptr, *pf_t = nullptr;
  bool use_prefill_gemm = true;
  const void* final_norm_w = nullptr;
  // tensor parallel
  int tp_world = 1, tp_rank = 0;
  bool shard_attn = true;
  uint8_t* win[b200::kMaxTpWorld] = {nullptr};  // exchange windows of every rank as mapped here
  unsigned long long* tp_epoch = nullptr;          // tokens completed (local)
  __nv_bfloat16* x_alt = nullptr;                  // second hidden-state buffer (TP ping-pong)
  const __nv_bfloat16* x_head = nullptr;           // residual the lm_head prologue reads (TP)
  // ---- batched decode (B ≤ 8 sequences at the same position, the reference's left-padded batch): own KV caches and
  // activations for all B sequences, GEMV plans that stream W once for the batch (gemv_batch.cu), own graphs.  Built on
  // the first forward with B > 1 (engine_batch_prepare).
  int batch = 1;                       // sequences of the most recent forward (decode / last_token follow it)
  int b_cap = 0;                       // batch the buffers / plans / graphs below were built for
  uint8_t* b_arena = nullptr;
  __nv_bfloat16 *bk = nullptr, *bv = nullptr;                 // [B][L][max_ctx][Hkv][hd]
  __nv_bfloat16 *bx = nullptr, *bqkv = nullptr, *battn = nullptr, *bact = nullptr, *blogits = nullptr;   // [B][·]
  float* b_attn_ws = nullptr;
  unsigned int* b_tickets = nullptr;
  void* b_argmax_ws = nullptr;
  int64_t* b_tok = nullptr;            // [B] token every sequence consumes next
  int64_t* b_log = nullptr;            // [gen_cap][B] generated tokens
  unsigned long long* b_cnt = nullptr; // [B] tokens generated per sequence (all equal)
  int64_t hb_gen = 0;                  // host mirror of b_cnt
  std::vector<b200::GemvPlan> bp_qkv, bp_o, bp_gu, bp_down;
  b200::GemvPlan bp_head{};
  cudaGraphExec_t gb_step = nullptr, gb_body = nullptr;
  int b_launches = 0, b_launches_body = 0;
  unsigned long long* trace = nullptr;  // B200_TRACE=1: [launch][8] globaltimer stamps of the last token
  bool use_graph = true;
  bool use_pdl = true;
  // sampler (b200_engine_set_sampler): when active the last kernels of a head token are the device sampler instead of
  // the argmax; u = Philox(seed, tokens generated so far)
  bool sampler_on = false;
  float s_temperature = 0.f, s_top_p = 1.f, s_min_p = 0.f;
  int64_t s_top_k = 0;
  unsigned long long s_seed = 0;
  void* sample_ws = nullptr;
  // async token pipeline (b200_engine_set_mailbox): ring in pinned host memory the argmax kernel posts tokens into
  unsigned long long* mailbox = nullptr;
  unsigned long long mailbox_cap = 1;
  // layer-stack model (b200_engine_create_stack): when set, every entry point runs engine_stack.cu's path
  b200::StackEngine* stack = nullptr;
};


namespace b200 {
// engine_stack.cu — the stack engine behind the common entry points
void stack_destroy(b200_engine* e);
int stack_reset(b200_engine* e, cudaStream_t st);
int stack_seek(b200_engine* e, int64_t position, cudaStream_t st);
int stack_forward(b200_engine* e, const int64_t* ids, int64_t B, int64_t S, void* logits_out, int logits_mode,
                  cudaStream_t st);
int stack_decode(b200_engine* e, int64_t n_steps, int64_t* tokens_out, cudaStream_t st);
int stack_last_token(b200_engine* e, int64_t* token_out, cudaStream_t st);
int stack_set_sampler(b200_engine* e, cudaStream_t st);
int64_t stack_bytes_per_token(const b200_engine* e, int64_t ctx);
}  // namespace b200
