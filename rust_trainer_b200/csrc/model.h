// Host-side driver objects behind the level-2 (Linear) and level-3 (Model) C ABI.
// They mirror the reference's Linear (src/linear.rs:38-122), Attention/Mlp/Block
// (src/attention.rs, src/model.rs:92-218) and Model (src/model.rs:292-687), with every
// tensor resident in HBM.
#pragma once
#include "ctx.h"
#include "ops.h"
#include <map>
#include <string>
#include <vector>

struct DevBuf {
  void* p = nullptr;
  size_t bytes = 0;
  // grow-only; returns false on allocation failure
  bool reserve(size_t want, bool zero = false);
  void release();
  template <class T> T* as() const { return (T*)p; }
};

struct LoraDev {
  int rank = 0;
  float alpha = 0.f;
  float *a = nullptr, *b = nullptr, *ga = nullptr, *gb = nullptr;  // views into flat f32 buffers
  __half *a_s = nullptr, *a_h = nullptr, *bp = nullptr, *bt_s = nullptr;  // 16-bit operand copies
  DevBuf shadows;
  bool stale = true;  // operand copies need rebuilding from a, b
  uint64_t version = 1;  // bumped with every change of a, b: stacked copies elsewhere compare it
  float scale() const { return alpha / (float)rank; }
};

struct rt_linear {
  rt_ctx* ctx = nullptr;
  int device = 0;
  std::string name;
  rt_frozen* w = nullptr;
  bool owns_w = false;
  float* bias = nullptr;  // device [out] or null
  bool has_lora = false, lora_enabled = true;
  LoraDev lora;
  DevBuf own_params;  // standalone linears own their a|b|ga|gb; model linears point into the model's buffers
  int in_dim() const { return w->w.cols; }
  int out_dim() const { return w->w.rows; }
  bool lora_active() const { return has_lora && lora_enabled; }
};

// Scratch shared by every Linear call on a ctx (one call at a time per ctx).
struct LinearScratch {
  DevBuf hs, gs, hs2, gs2, smax, grad_ws;
  int hs_rank = -1, gs_rank = -1, hs2_rank = -1, gs2_rank = -1;
};

namespace rt {
// hs_keep: optional [M x 64] f16 buffer (zero beyond the rank) that receives Hs = X.(sA)^T so the
// backward can reuse it instead of recomputing it.
rt_status linear_forward_dev(rt_linear* l, LinearScratch& sc, const __half* x16, int M, void* y, int y_dtype,
                             int accumulate, __half* hs_keep = nullptr, bool hs_ready = false);
// Hs alone (the forward of a linear whose output is not needed).
rt_status linear_lora_h(rt_linear* l, const __half* x16, int M, __half* hs_out);
// dy16 is row-normalised f16 with per-row scales `dscale` (null = all ones).  With
// unscaled_f16_out, dx receives f16 rows WITHOUT their factor dscale[row] (the consumer applies
// it): half the output bytes, no accumulate.
rt_status linear_backward_dev(rt_linear* l, LinearScratch& sc, const __half* x16, const __half* dy16,
                              const float* dscale, int M, void* dx, int accumulate,
                              const __half* hs_saved = nullptr, bool unscaled_f16_out = false);
rt_status lora_refresh(rt_linear* l);
int attn_backward(rt_ctx* c, const __half* q, const __half* k, const __half* v, const __half* o, const __half* dO16,
                  const float* do_scale, const float* row_scale, const float* lse, const int* seq_start, const int* gap, int M,
                  int nh, int nkv, int hd, float* delta, float* dq, float* dk, float* dv);
int attn_forward(rt_ctx* c, const __half* q, const __half* k, const __half* v, const int* seq_start, const int* gap, int M, int nh,
                 int nkv, int hd, __half* o, float* lse);
}  // namespace rt

// Linears that read the same input (q|k|v, gate|up) as ONE matmul: their packed weights lie
// stacked along the output rows in one buffer (the members' own handles point into it), so the
// forward is a single product with the stacked rows as output features and the backward a
// single product contracting over them, instead of one product per member plus accumulating
// passes.  The members' adapters become one stacked low-rank chunk: member i owns columns
// [rank_off[i], rank_off[i] + r_i) of Hs / Gs.
struct LinGroup {
  int n = 0;
  rt_linear* lin[3] = {nullptr, nullptr, nullptr};
  int row_off[3] = {0, 0, 0}, rank_off[3] = {0, 0, 0};
  int rows_total = 0, rank_total = 0;
  bool stacked = false;    // weights share one buffer
  bool lora_ok = false;    // the members' adapters fit one 64-wide chunk (or there are none)
  rt::QWeight w;
  DevBuf store, lora_copies;
  float* bias = nullptr;   // stacked biases (owned), null when no member has one
  __half *a_s = nullptr, *a_h = nullptr, *bp = nullptr, *bt_s = nullptr;
  uint64_t seen[3] = {0, 0, 0};
};

struct BlockDev {
  float *input_norm = nullptr, *post_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
  rt_linear* lin[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};  // q k v o gate up down
  LinGroup qkv, gu;
};

struct rt_model {
  rt_ctx* ctx = nullptr;
  int device = 0;
  rt_model_config cfg;
  bool finalized = false;
  rt_frozen* embed = nullptr;
  rt_frozen* lm_head = nullptr;  // == embed when tied
  float* final_norm = nullptr;
  std::vector<float> rope_factors;  // host copy of rope_freqs.weight
  std::vector<BlockDev> blocks;
  std::vector<void*> owned;  // small device allocations (norms, biases)
  std::vector<rt_linear*> lora_order;  // adapted linears in parameter order

  // flat LoRA state: [A_0 | B_0 | A_1 | B_1 ...] in parameter order
  size_t n_params = 0;
  DevBuf P, G, Mo, Vo, opt_scalars;  // opt_scalars: 1024 f64 partials + 1 f64 sum + 1 f32 norm
  uint64_t opt_t = 0;

  // RoPE tables
  DevBuf inv_freq, rope_cos, rope_sin;
  int rope_max_pos = 0;

  LinearScratch lsc;
  DevBuf hs_keep[7];  // Hs of a block's seven linears, kept from the forward (or its recompute) for the backward
  // What a block's backward needs from its forward is either kept for every layer (180 GB of HBM
  // holds it for the usual fine-tuning shapes) or rebuilt by running the block's forward again
  // just before its backward.  Decided when the token capacity grows; RT_B200_RECOMPUTE=1 forces
  // the second.
  bool store_acts = false;
  int recompute_policy = -1;  // -1: not read yet, 0: automatic, 1: always recompute, 2: always keep
  // activations, sized for `cap_tokens`
  int cap_tokens = 0, cap_targets = 0, cap_head_rows = 0;
  // q_raw holds q|k|v before RoPE (three regions, or one matrix with q, k, v as column slices when the
  // block runs them as a group); g16 holds gate|up the same way; dq16, dg16 likewise for the gradients
  DevBuf tokens, pos, seq_start, x, ckpt, h, n1, n2, q_raw, k_raw, v_raw, q16, k16, v16, o16, lse, delta, g16, u16, hm16;
  DevBuf dx, dy16, sc_y, dhm, dg16, du16, sc_g, sc_u, dn, d_o, dO16, amax, dq, dk, dv, dq16, dk16, dv16, sc_q, sc_k, sc_v;
  DevBuf tpos, ttok, tw, logp, hits, xs, ns16, logits, dl16, sc_l, dns, dxs;
  DevBuf argmax;            // per target, the greedy token of the last pass that asked for it
  bool want_argmax = false;
  std::vector<int> h_pos, h_seq_start, h_gap;
  DevBuf refresh_tab;       // device copy of refresh_sent
  std::vector<rt::LoraRefreshJob> refresh_jobs, refresh_sent;
  DevBuf gap;               // per token (first, end) of the key range hidden from it: packed shared-prompt groups
  bool staged_gap = false;  // the staged batch has such ranges
  int staged_tokens = 0, staged_targets = 0;
  bool staged_has_weights = false;
  // CUDA graphs of the staged step, one per (tokens, targets, backward) once it has run eagerly
  struct GraphEntry { int M, n_targets, backward; uint64_t sig; cudaGraphExec_t exec; unsigned long long kernels; };
  std::vector<GraphEntry> graphs;
  int eager_M = -1, eager_targets = -1, eager_backward = -1;
  uint64_t eager_sig = 0;
  int use_graphs = -1;  // -1: decide from the environment on first use
};
