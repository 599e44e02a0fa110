// C ABI levels 2 and 3: Linear + LoRA and the whole decoder step on the device.
// The arithmetic lives in qgemm.cu (frozen matmuls), attention.cu and ops.cu; this file is the
// sequencing the reference does in src/linear.rs, src/attention.rs, src/model.rs and
// src/optim.rs, plus buffer management.
#include "model.h"
#include <math.h>
#include <algorithm>
#include <stdio.h>
#include <string.h>

bool DevBuf::reserve(size_t want, bool zero) {
  if (want <= bytes) return true;
  if (p) cudaFree(p);
  p = nullptr;
  bytes = 0;
  if (cudaMalloc(&p, want) != cudaSuccess) return false;
  bytes = want;
  if (zero) {
    // the clear runs on the legacy stream, the kernels on the ctx's non-blocking stream: nothing
    // else orders the two, so finish the clear before anyone can launch on the buffer
    cudaMemset(p, 0, want);
    cudaDeviceSynchronize();
  }
  return true;
}
void DevBuf::release() {
  if (p) cudaFree(p);
  p = nullptr;
  bytes = 0;
}

#define RT_TRY(expr)          \
  do {                        \
    rt_status s__ = (expr);   \
    if (s__) return s__;      \
  } while (0)

namespace rt {

rt_status lora_refresh(rt_linear* l) {
  if (!l->has_lora || !l->lora.stale) return RT_OK;
  LoraDev& lo = l->lora;
  launch_lora_refresh(lo.a, lo.b, lo.rank, l->in_dim(), l->out_dim(), lo.scale(), lo.a_s, lo.a_h, lo.bp, lo.bt_s,
                      l->ctx->stream);
  lo.stale = false;
  return RT_OK;
}

// Hs / Gs are [M x 64] f16.  The low-rank chunk of the big matmul reads whole groups of 16
// columns, so columns from `rank` up to the next multiple of 16 must hold zeros (or at least
// finite values against zero weights; zeros keep it exact).  When the rank is not a multiple of
// 16 the buffer is cleared on every call: a decision taken from what earlier calls left behind
// would be frozen into a captured graph and replayed after a different history.  `cur_rank`
// only records that the buffer has been cleared once since it was (re)allocated.
static __half* lowrank_buf(rt_ctx* c, DevBuf& b, int& cur_rank, int M, int rank) {
  const size_t want = (size_t)M * 64 * sizeof(__half);
  bool clear = false;
  if (want > b.bytes) {
    if (!b.reserve(want + want / 2)) return nullptr;
    clear = true;
  }
  if (cur_rank < 0 || rank % 16 != 0) clear = true;
  if (clear) cudaMemsetAsync(b.p, 0, want, c->stream);
  cur_rank = rank;
  return b.as<__half>();
}

int attn_forward(rt_ctx* c, const __half* q, const __half* k, const __half* v, const int* seq_start, const int* gap, int M, int nh,
                 int nkv, int hd, __half* o, float* lse) {
  return launch_attn_fwd_tc(c, q, k, v, seq_start, gap, M, nh, nkv, hd, o, lse);
}
int attn_backward(rt_ctx* c, const __half* q, const __half* k, const __half* v, const __half* o, const __half* dO16,
                  const float* do_scale, const float* row_scale, const float* lse, const int* seq_start, const int* gap, int M,
                  int nh, int nkv, int hd, float* delta, float* dq, float* dk, float* dv) {
  return launch_attn_bwd_tc(c, q, k, v, o, dO16, do_scale, row_scale, lse, seq_start, gap, M, nh, nkv, hd, delta, dq, dk, dv);
}

// out[M x 64] = X[M x K] . Wt[r x K]^T: the tcgen05 stream kernel, or (return 1) a shape it does not take
static int lowrank_product(rt_ctx* c, const __half* X, const __half* Wt, int M, int K, int r, __half* out64) {
  return launch_lowrank_tc(c, X, Wt, M, K, r, out64);
}

static QWeight dense_view(const __half* p, int rows, int cols) {
  QWeight w;
  w.fmt = GGML_F16;
  w.rows = rows;
  w.cols = cols;
  w.dense16 = (void*)p;
  return w;
}

rt_status linear_lora_h(rt_linear* l, const __half* x16, int M, __half* hs_out) {
  rt_ctx* c = l->ctx;
  lora_refresh(l);
  {
    const int rc0 = lowrank_product(c, x16, l->lora.a_s, M, l->in_dim(), l->lora.rank, hs_out);
    if (rc0 == 0) return RT_OK;
    if (rc0 != 1) return c->fail(RT_ERR_CUDA, "lora H kernel launch failed");
  }
  QGemmArgs ha;  // Hs = X . (sA)^T  (general shapes: through the big kernel)
  ha.dir = QG_FWD;
  ha.act = x16;
  ha.act_f16 = 1;
  ha.M = M;
  ha.out = hs_out;
  ha.out_dtype = OUT_F16;
  ha.ld_out = 64;
  ha.aux = 1;
  int rc = qgemm_launch(c, dense_view(l->lora.a_s, l->lora.rank, l->in_dim()), ha);
  if (rc) return c->fail(rc, "lora H matmul launch failed");
  return RT_OK;
}

rt_status linear_forward_dev(rt_linear* l, LinearScratch& sc, const __half* x16, int M, void* y, int y_dtype,
                             int accumulate, __half* hs_keep, bool hs_ready) {
  rt_ctx* c = l->ctx;
  if (M <= 0) return RT_OK;
  QGemmArgs a;
  a.dir = QG_FWD;
  a.act = x16;
  a.act_f16 = 1;
  a.M = M;
  a.out = y;
  a.out_dtype = y_dtype;
  a.accumulate = accumulate;
  a.bias = l->bias;
  if (l->lora_active()) {
    lora_refresh(l);
    const int r = l->lora.rank;
    __half* hs = hs_keep ? hs_keep : lowrank_buf(c, sc.hs, sc.hs_rank, M, r);
    if (!hs) return c->fail(RT_ERR_CUDA, "out of device memory (lora scratch)");
    if (!(hs_keep && hs_ready)) RT_TRY(linear_lora_h(l, x16, M, hs));
    a.lora.act = hs;
    a.lora.w = l->lora.bp;
    a.lora.rank = r;
  }
  int rc = frozen_matmul_launch(c, l->w->w, a);
  if (rc) return c->fail(rc, "frozen forward matmul launch failed");
  return RT_OK;
}

rt_status linear_backward_dev(rt_linear* l, LinearScratch& sc, const __half* x16, const __half* dy16,
                              const float* dscale, int M, void* dx, int accumulate, const __half* hs_saved,
                              bool unscaled_f16_out) {
  rt_ctx* c = l->ctx;
  if (M <= 0) return RT_OK;
  if (unscaled_f16_out && accumulate) return c->fail(RT_ERR_BAD_ARG, "an unscaled f16 gradient cannot accumulate");
  const int K = l->in_dim(), N = l->out_dim();
  QGemmArgs a;
  a.dir = QG_BWD;
  a.act = dy16;
  a.act_f16 = 1;
  a.M = M;
  a.out = dx;
  a.out_dtype = unscaled_f16_out ? OUT_F16 : OUT_F32;
  a.accumulate = accumulate;
  a.row_scale = unscaled_f16_out ? nullptr : dscale;
  if (l->lora_active()) {
    lora_refresh(l);
    const int r = l->lora.rank;
    __half* hs = hs_saved ? const_cast<__half*>(hs_saved) : lowrank_buf(c, sc.hs, sc.hs_rank, M, r);
    __half* gs = lowrank_buf(c, sc.gs, sc.gs_rank, M, r);
    if (!hs || !gs) return c->fail(RT_ERR_CUDA, "out of device memory (lora scratch)");
    // Hs = X . (sA)^T: recomputed as src/linear.rs:105 does, unless the caller kept it
    if (!hs_saved) RT_TRY(linear_lora_h(l, x16, M, hs));
    int rc = lowrank_product(c, dy16, l->lora.bt_s, M, N, r, gs);
    if (rc > 1) return c->fail(RT_ERR_CUDA, "lora G kernel launch failed");
    const bool g_done = rc == 0;
    QGemmArgs ga;  // Gs = dY~ . (sB)   (unit rows: the row scale is applied where Gs is consumed)
    ga.dir = QG_FWD;
    ga.act = dy16;
    ga.act_f16 = 1;
    ga.M = M;
    ga.out = gs;
    ga.out_dtype = OUT_F16;
    ga.ld_out = 64;
    ga.aux = 1;
    if (!g_done) {
      rc = qgemm_launch(c, dense_view(l->lora.bt_s, r, N), ga);
      if (rc) return c->fail(rc, "lora G matmul launch failed");
    }
    // gb[N x r] += dY^T . Hs ; ga[r x K] += Gs^T . X   on the tensor cores, contraction over tokens.
    // The per-token scales of dY move onto the skinny operand (rows * scale / max), the max onto the result.
    const __half *hs_c = hs, *gs_c = gs;
    const float* alpha = nullptr;
    const size_t wsf2 = lora_grads_workspace_floats(M, N, K, r);
    if (!sc.grad_ws.reserve(wsf2 * sizeof(float))) return c->fail(RT_ERR_CUDA, "out of device memory (lora scratch)");
    int rb = launch_lora_grads(c, hs, dy16, N, gs, x16, dscale, M, N, K, r, l->lora.gb, l->lora.ga, sc.grad_ws.as<float>(), c->stream);
    if (rb > 1) return c->fail(RT_ERR_CUDA, "lora gradient kernel launch failed");
    int ra = rb;
    if (rb == 1) {  // shapes the fused kernels do not cover: one product at a time
      if (dscale) {
        if (!sc.smax.reserve(16)) return c->fail(RT_ERR_CUDA, "out of device memory (lora scratch)");
        launch_rowscale_max(dscale, M, sc.smax.as<float>(), c->stream);
        alpha = sc.smax.as<float>();
      }
      const size_t wsf = tok_contract_workspace_floats(M, K > N ? K : N, r);
      if (!sc.grad_ws.reserve(wsf * sizeof(float))) return c->fail(RT_ERR_CUDA, "out of device memory (lora scratch)");
      rb = launch_tok_contract(hs, dy16, dscale, M, N, r, 1, (size_t)r, alpha, l->lora.gb, sc.grad_ws.as<float>(), c->stream);
      ra = launch_tok_contract(gs, x16, dscale, M, K, r, (size_t)K, 1, alpha, l->lora.ga, sc.grad_ws.as<float>(), c->stream);
      if (rb > 1 || ra > 1) return c->fail(RT_ERR_CUDA, "lora gradient kernel launch failed");
    }
    if (dscale && (rb == 1 || ra == 1)) {  // general shapes go through the big kernel and need scaled copies
      __half* hs2 = lowrank_buf(c, sc.hs2, sc.hs2_rank, M, r);
      __half* gs2 = lowrank_buf(c, sc.gs2, sc.gs2_rank, M, r);
      if (!hs2 || !gs2) return c->fail(RT_ERR_CUDA, "out of device memory (lora scratch)");
      launch_scale_lowrank_rows(hs, dscale, sc.smax.as<float>(), M, hs2, c->stream);
      launch_scale_lowrank_rows(gs, dscale, sc.smax.as<float>(), M, gs2, c->stream);
      hs_c = hs2;
      gs_c = gs2;
    }
    QGemmArgs ta;
    ta.dir = QG_BWD;
    ta.tok_mode = 1;
    ta.act_f16 = 1;
    ta.M = r;
    ta.out_dtype = OUT_F32;
    ta.accumulate = 1;
    ta.alpha_dev = alpha;
    ta.aux = 1;
    ta.act = hs_c;  // dB[n, i] += sum_m dY[m, n] Hs[m, i]
    ta.out = l->lora.gb;
    ta.out_s_tok = 1;
    ta.out_s_row = (size_t)r;
    if (rb == 1) {
      rc = qgemm_launch(c, dense_view(dy16, M, N), ta);
      if (rc) return c->fail(rc, "lora dB matmul launch failed");
    }
    ta.act = gs_c;  // dA[i, k] += sum_m Gs[m, i] X[m, k]
    ta.out = l->lora.ga;
    ta.out_s_tok = (size_t)K;
    ta.out_s_row = 1;
    if (ra == 1) {
      rc = qgemm_launch(c, dense_view(x16, M, K), ta);
      if (rc) return c->fail(rc, "lora dA matmul launch failed");
    }
    a.lora.act = gs;
    a.lora.w = l->lora.a_h;
    a.lora.rank = r;
  }
  int rc = frozen_matmul_launch(c, l->w->w, a);
  if (rc) return c->fail(rc, "frozen backward matmul launch failed");
  return RT_OK;
}


// ---- groups of linears that share their input (see LinGroup)
static bool group_lora_on(const LinGroup& g, bool* any) {
  // usable as one product only when every member that has an adapter also has it enabled
  bool on = false, off = false;
  for (int i = 0; i < g.n; ++i)
    if (g.lin[i]->has_lora) (g.lin[i]->lora_enabled ? on : off) = true;
  *any = on;
  return !(on && off);
}
bool group_usable(const LinGroup& g) {
  if (!g.stacked) return false;
  bool any;
  if (!group_lora_on(g, &any)) return false;
  return !any || g.lora_ok;
}

static void group_refresh(LinGroup& g, cudaStream_t st) {
  const size_t K = (size_t)g.w.cols;
  for (int i = 0; i < g.n; ++i) {
    rt_linear* l = g.lin[i];
    if (!l->has_lora || g.seen[i] == l->lora.version) continue;
    LoraDev& lo = l->lora;
    launch_lora_refresh_group(lo.a, lo.b, lo.rank, (int)K, l->out_dim(), lo.scale(), g.a_s + (size_t)g.rank_off[i] * K,
                              g.a_h + (size_t)g.rank_off[i] * K, g.bp + (size_t)g.row_off[i] * 64 + g.rank_off[i],
                              g.bt_s + (size_t)g.rank_off[i] * g.rows_total + g.row_off[i], (size_t)g.rows_total, st);
    g.seen[i] = lo.version;
  }
}

// Rebuilds, in one launch, every 16-bit adapter copy the next pass over the model will read and
// that is older than its adapter: the stacked copies of usable groups, the own copies of the
// linears outside them.  Runs before a pass (never inside a captured one: a copy that happened
// to be fresh at capture time would otherwise never be rebuilt by the replays).
rt_status refresh_adapter_copies(rt_model* m) {
  rt_ctx* c = m->ctx;
  std::vector<LoraRefreshJob>& jobs = m->refresh_jobs;
  jobs.clear();
  unsigned blocks = 0;
  auto add = [&](LoraRefreshJob j) {
    j.first_block = blocks;
    blocks += lora_refresh_job_blocks(j);
    jobs.push_back(j);
  };
  for (auto& b : m->blocks) {
    bool grouped[7] = {false, false, false, false, false, false, false};
    LinGroup* gs[2] = {&b.qkv, &b.gu};
    for (LinGroup* g : gs) {
      if (!group_usable(*g)) continue;
      bool any;
      group_lora_on(*g, &any);
      const size_t K = (size_t)g->w.cols;
      for (int i = 0; i < g->n; ++i) {
        rt_linear* l = g->lin[i];
        for (int k = 0; k < 7; ++k)
          if (b.lin[k] == l) grouped[k] = true;
        if (!any || !l->has_lora || g->seen[i] == l->lora.version) continue;
        const LoraDev& lo = l->lora;
        LoraRefreshJob j{lo.a, lo.b, g->a_s + (size_t)g->rank_off[i] * K, g->a_h + (size_t)g->rank_off[i] * K,
                         g->bp + (size_t)g->row_off[i] * 64 + g->rank_off[i],
                         g->bt_s + (size_t)g->rank_off[i] * g->rows_total + g->row_off[i],
                         (unsigned long long)g->rows_total, lo.rank, (int)K, l->out_dim(), 0, lo.scale(), 0u};
        add(j);
      }
    }
    for (int k = 0; k < 7; ++k) {
      rt_linear* l = b.lin[k];
      if (!l || grouped[k] || !l->lora_active() || !l->lora.stale) continue;
      const LoraDev& lo = l->lora;
      LoraRefreshJob j{lo.a, lo.b, lo.a_s, lo.a_h, lo.bp, lo.bt_s, (unsigned long long)l->out_dim(),
                       lo.rank, l->in_dim(), l->out_dim(), 1, lo.scale(), 0u};
      add(j);
    }
  }
  if (jobs.empty()) return RT_OK;
  const size_t bytes = jobs.size() * sizeof(LoraRefreshJob);
  if (m->refresh_sent.size() != jobs.size() || memcmp(m->refresh_sent.data(), jobs.data(), bytes) != 0) {
    if (!m->refresh_tab.reserve(bytes)) return c->fail(RT_ERR_CUDA, "out of device memory (adapter refresh table)");
    RT_CUDA(c, cudaMemcpyAsync(m->refresh_tab.p, jobs.data(), bytes, cudaMemcpyHostToDevice, c->stream));
    m->refresh_sent = jobs;
  }
  launch_lora_refresh_table(m->refresh_tab.as<LoraRefreshJob>(), (int)jobs.size(), blocks, c->stream);
  for (auto& b : m->blocks) {
    LinGroup* gs[2] = {&b.qkv, &b.gu};
    bool grouped[7] = {false, false, false, false, false, false, false};
    for (LinGroup* g : gs) {
      if (!group_usable(*g)) continue;
      bool any;
      group_lora_on(*g, &any);
      for (int i = 0; i < g->n; ++i) {
        for (int k = 0; k < 7; ++k)
          if (b.lin[k] == g->lin[i]) grouped[k] = true;
        if (any && g->lin[i]->has_lora) g->seen[i] = g->lin[i]->lora.version;
      }
    }
    for (int k = 0; k < 7; ++k)
      if (b.lin[k] && !grouped[k] && b.lin[k]->lora_active()) b.lin[k]->lora.stale = false;
  }
  return RT_OK;
}

// y[M x rows_total] = X . [W_0; W_1; ..]^T (+ stacked bias, + stacked low-rank chunk)
rt_status group_forward_dev(LinGroup& g, LinearScratch& sc, const __half* x16, int M, void* y, int y_dtype, __half* hs_keep,
                            bool hs_ready) {
  rt_ctx* c = g.lin[0]->ctx;
  if (M <= 0) return RT_OK;
  QGemmArgs a;
  a.dir = QG_FWD;
  a.act = x16;
  a.act_f16 = 1;
  a.M = M;
  a.out = y;
  a.out_dtype = y_dtype;
  a.bias = g.bias;
  bool any;
  group_lora_on(g, &any);
  if (any) {
    group_refresh(g, c->stream);
    __half* hs = hs_keep ? hs_keep : lowrank_buf(c, sc.hs, sc.hs_rank, M, g.rank_total);
    if (!hs) return c->fail(RT_ERR_CUDA, "out of device memory (lora scratch)");
    if (!(hs_keep && hs_ready) && lowrank_product(c, x16, g.a_s, M, g.w.cols, g.rank_total, hs))
      return c->fail(RT_ERR_CUDA, "lora H kernel launch failed");
    a.lora.act = hs;
    a.lora.w = g.bp;
    a.lora.rank = g.rank_total;
  }
  int rc = qgemm_launch(c, g.w, a);
  if (rc) return c->fail(rc, "frozen forward matmul launch failed");
  return RT_OK;
}

// dx[M x K] (+)= dY[M x rows_total] . [W_0; W_1; ..] (+ Gs . A), dY row-normalised with ONE factor per token
// for the whole row; each member's dA, dB from its slices.
rt_status group_backward_dev(LinGroup& g, LinearScratch& sc, const __half* x16, const __half* dy16, const float* dscale,
                             int M, float* dx, int accumulate, const __half* hs_saved) {
  rt_ctx* c = g.lin[0]->ctx;
  if (M <= 0) return RT_OK;
  const int K = g.w.cols, NT = g.rows_total;
  QGemmArgs a;
  a.dir = QG_BWD;
  a.act = dy16;
  a.act_f16 = 1;
  a.M = M;
  a.out = dx;
  a.out_dtype = OUT_F32;
  a.accumulate = accumulate;
  a.row_scale = dscale;
  bool any;
  group_lora_on(g, &any);
  if (any) {
    group_refresh(g, c->stream);
    const int R = g.rank_total;
    __half* hs = hs_saved ? const_cast<__half*>(hs_saved) : lowrank_buf(c, sc.hs, sc.hs_rank, M, R);
    __half* gs = lowrank_buf(c, sc.gs, sc.gs_rank, M, R);
    if (!hs || !gs) return c->fail(RT_ERR_CUDA, "out of device memory (lora scratch)");
    if (!hs_saved && lowrank_product(c, x16, g.a_s, M, K, R, hs)) return c->fail(RT_ERR_CUDA, "lora H kernel launch failed");
    if (lowrank_product(c, dy16, g.bt_s, M, NT, R, gs)) return c->fail(RT_ERR_CUDA, "lora G kernel launch failed");
    if (!sc.grad_ws.reserve(lora_grads_workspace_floats(M, NT, K, R) * sizeof(float)))
      return c->fail(RT_ERR_CUDA, "out of device memory (lora scratch)");
    float *gbp[3], *gap[3];
    int roff[3], rws[3], koff[3], rk[3], nm = 0;
    for (int i = 0; i < g.n; ++i) {
      rt_linear* l = g.lin[i];
      if (!l->has_lora) continue;
      gbp[nm] = l->lora.gb; gap[nm] = l->lora.ga;
      roff[nm] = g.row_off[i]; rws[nm] = l->out_dim(); koff[nm] = g.rank_off[i]; rk[nm] = l->lora.rank;
      ++nm;
    }
    if (launch_lora_grads_group(c, hs, dy16, gs, x16, dscale, M, NT, K, R, nm, gbp, gap, roff, rws, koff, rk,
                                sc.grad_ws.as<float>(), c->stream))
      return c->fail(RT_ERR_CUDA, "lora gradient kernel launch failed");
    a.lora.act = gs;
    a.lora.w = g.a_h;
    a.lora.rank = R;
  }
  int rc = qgemm_launch(c, g.w, a);
  if (rc) return c->fail(rc, "frozen backward matmul launch failed");
  return RT_OK;
}

// tensor.rs:155-199 Rng, host side, for Lora::new's A ~ U(-1/sqrt(in), 1/sqrt(in))
struct SplitMix {
  uint64_t state;
  explicit SplitMix(uint64_t seed) : state(seed ^ 0x9E3779B97F4A7C15ull) {}
  uint64_t next() {
    state += 0x9E3779B97F4A7C15ull;
    uint64_t z = state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
  float uniform() { return (float)(next() >> 40) / (float)(1ull << 24); }
  float uniform_sym(float bound) { return (uniform() * 2.0f - 1.0f) * bound; }
};

}  // namespace rt

using namespace rt;

static rt_status attach_views(rt_linear* l, int rank, float alpha, float* a, float* b, float* ga, float* gb) {
  rt_ctx* c = l->ctx;
  const int K = l->in_dim(), N = l->out_dim();
  LoraDev& lo = l->lora;
  lo.rank = rank;
  lo.alpha = alpha;
  lo.a = a;
  lo.b = b;
  lo.ga = ga;
  lo.gb = gb;
  const size_t n_as = (size_t)rank * K, n_bp = (size_t)N * 64, n_bt = (size_t)rank * N;
  // each operand copy starts on a 256-byte boundary (TMA needs 16)
  auto up = [](size_t n) { return (n * 2 + 255) / 256 * 256; };
  const size_t total = 2 * up(n_as) + up(n_bp) + up(n_bt);
  if (!lo.shadows.reserve(total)) return c->fail(RT_ERR_CUDA, "out of device memory (adapter copies)");
  uint8_t* base = (uint8_t*)lo.shadows.p;
  lo.a_s = (__half*)base;
  lo.a_h = (__half*)(base + up(n_as));
  lo.bp = (__half*)(base + 2 * up(n_as));
  lo.bt_s = (__half*)(base + 2 * up(n_as) + up(n_bp));
  lo.stale = true;
  ++lo.version;
  l->has_lora = true;
  return RT_OK;
}

extern "C" {

// ------------------------------------------------------------------ level 2
rt_status rt_linear_create(rt_ctx* c, rt_frozen* w, const float* bias_host, const char* name, rt_linear** out) {
  if (!c || !w || !out) return RT_ERR_BAD_ARG;
  *out = nullptr;
  RT_CUDA(c, cudaSetDevice(c->device));
  rt_linear* l = new rt_linear();
  l->ctx = c;
  l->device = c->device;
  l->w = w;
  l->name = name ? name : "";
  if (bias_host) {
    cudaError_t e = cudaMalloc(&l->bias, (size_t)w->w.rows * sizeof(float));
    if (e == cudaSuccess) e = cudaMemcpy(l->bias, bias_host, (size_t)w->w.rows * sizeof(float), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
      delete l;
      return c->cuda_fail(e, "rt_linear_create");
    }
  }
  *out = l;
  return RT_OK;
}

void rt_linear_destroy(rt_linear* l) {
  if (!l) return;
  cudaSetDevice(l->device);
  if (l->bias) cudaFree(l->bias);
  l->lora.shadows.release();
  l->own_params.release();
  if (l->owns_w) rt_frozen_destroy(l->w);
  delete l;
}

rt_status rt_linear_attach_lora(rt_linear* l, int rank, float alpha, const float* a_host, const float* b_host) {
  if (!l || !a_host || !b_host) return RT_ERR_BAD_ARG;
  rt_ctx* c = l->ctx;
  if (rank <= 0 || rank > 64) return c->fail(RT_ERR_BAD_ARG, "LoRA rank must be in 1..64");
  RT_CUDA(c, cudaSetDevice(c->device));
  const size_t na = (size_t)rank * l->in_dim(), nb = (size_t)l->out_dim() * rank;
  if (!l->own_params.reserve(2 * (na + nb) * sizeof(float))) return c->fail(RT_ERR_CUDA, "out of device memory");
  float* base = l->own_params.as<float>();
  RT_CUDA(c, cudaMemcpyAsync(base, a_host, na * sizeof(float), cudaMemcpyHostToDevice, c->stream));
  RT_CUDA(c, cudaMemcpyAsync(base + na, b_host, nb * sizeof(float), cudaMemcpyHostToDevice, c->stream));
  RT_CUDA(c, cudaMemsetAsync(base + na + nb, 0, (na + nb) * sizeof(float), c->stream));
  RT_CUDA(c, cudaStreamSynchronize(c->stream));
  return attach_views(l, rank, alpha, base, base + na, base + na + nb, base + 2 * na + nb);
}

rt_status rt_linear_set_lora_enabled(rt_linear* l, int on) {
  if (!l) return RT_ERR_BAD_ARG;
  l->lora_enabled = on != 0;
  return RT_OK;
}

static LinearScratch& ctx_scratch(rt_ctx* c) {
  static std::map<rt_ctx*, LinearScratch> m;  // scratch for linears used outside a model
  return m[c];
}

rt_status rt_linear_forward_dev(rt_linear* l, const void* x, size_t t, void* y, int y_dtype, int accumulate) {
  if (!l || !x || !y) return RT_ERR_BAD_ARG;
  rt_ctx* c = l->ctx;
  if (t > (1u << 24)) return c->fail(RT_ERR_BAD_SHAPE, "too many rows");
  if (y_dtype < 0 || y_dtype > 2) return c->fail(RT_ERR_BAD_ARG, "bad output dtype");
  if (accumulate && y_dtype != RT_DT_F32) return c->fail(RT_ERR_BAD_ARG, "accumulate needs an f32 output");
  RT_CUDA(c, cudaSetDevice(c->device));
  return linear_forward_dev(l, ctx_scratch(c), (const __half*)x, (int)t, y, y_dtype, accumulate);
}

rt_status rt_linear_backward_dev(rt_linear* l, const void* x, const void* dy, const float* dscale, size_t t, float* dx,
                                 int accumulate) {
  if (!l || !x || !dy || !dx) return RT_ERR_BAD_ARG;
  rt_ctx* c = l->ctx;
  if (t > (1u << 24)) return c->fail(RT_ERR_BAD_SHAPE, "too many rows");
  RT_CUDA(c, cudaSetDevice(c->device));
  return linear_backward_dev(l, ctx_scratch(c), (const __half*)x, (const __half*)dy, dscale, (int)t, dx, accumulate);
}

rt_status rt_linear_forward(rt_linear* l, const float* x_host, size_t t, float* y_host) {
  if (!l || !x_host || !y_host) return RT_ERR_BAD_ARG;
  rt_ctx* c = l->ctx;
  if (t == 0) return RT_OK;
  if (t > (1u << 24)) return c->fail(RT_ERR_BAD_SHAPE, "too many rows");
  RT_CUDA(c, cudaSetDevice(c->device));
  const size_t K = l->in_dim(), N = l->out_dim();
  float* xf = (float*)c->get_scratch(0, t * K * sizeof(float));
  __half* xh = (__half*)c->get_scratch(1, t * K * sizeof(__half));
  float* yf = (float*)c->get_scratch(2, t * N * sizeof(float));
  if (!xf || !xh || !yf) return c->fail(RT_ERR_CUDA, "out of device memory");
  RT_CUDA(c, cudaMemcpyAsync(xf, x_host, t * K * sizeof(float), cudaMemcpyHostToDevice, c->stream));
  launch_f32_to_16(xf, xh, t * K, true, c->stream);
  rt_status st = linear_forward_dev(l, ctx_scratch(c), xh, (int)t, yf, RT_DT_F32, 0);
  if (st) return st;
  RT_CUDA(c, cudaMemcpyAsync(y_host, yf, t * N * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  return c->check_device_status("rt_linear_forward");
}

rt_status rt_linear_backward(rt_linear* l, const float* x_host, const float* dy_host, size_t t, float* dx_host) {
  if (!l || !x_host || !dy_host || !dx_host) return RT_ERR_BAD_ARG;
  rt_ctx* c = l->ctx;
  if (t == 0) return RT_OK;
  if (t > (1u << 24)) return c->fail(RT_ERR_BAD_SHAPE, "too many rows");
  RT_CUDA(c, cudaSetDevice(c->device));
  const size_t K = l->in_dim(), N = l->out_dim();
  float* xf = (float*)c->get_scratch(0, (t * (K > N ? K : N)) * sizeof(float));
  uint8_t* s1 = (uint8_t*)c->get_scratch(1, t * (K + N) * sizeof(__half) + t * sizeof(float) + 512);
  float* dxf = (float*)c->get_scratch(2, t * K * sizeof(float));
  if (!xf || !s1 || !dxf) return c->fail(RT_ERR_CUDA, "out of device memory");
  __half* xh = (__half*)s1;
  __half* dyh = (__half*)(s1 + (t * K * sizeof(__half) + 255) / 256 * 256);
  float* dsc = (float*)((uint8_t*)dyh + (t * N * sizeof(__half) + 255) / 256 * 256);
  RT_CUDA(c, cudaMemcpyAsync(xf, x_host, t * K * sizeof(float), cudaMemcpyHostToDevice, c->stream));
  launch_f32_to_16(xf, xh, t * K, true, c->stream);
  RT_CUDA(c, cudaMemcpyAsync(xf, dy_host, t * N * sizeof(float), cudaMemcpyHostToDevice, c->stream));
  launch_normalize_rows(xf, (int)t, (int)N, dyh, dsc, c->stream);
  rt_status st = linear_backward_dev(l, ctx_scratch(c), xh, dyh, dsc, (int)t, dxf, 0);
  if (st) return st;
  RT_CUDA(c, cudaMemcpyAsync(dx_host, dxf, t * K * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  return c->check_device_status("rt_linear_backward");
}

rt_status rt_lora_read(rt_linear* l, float* a, float* b, float* ga, float* gb) {
  if (!l) return RT_ERR_BAD_ARG;
  rt_ctx* c = l->ctx;
  if (!l->has_lora) return c->fail(RT_ERR_BAD_ARG, "linear has no adapter");
  RT_CUDA(c, cudaSetDevice(c->device));
  const size_t na = (size_t)l->lora.rank * l->in_dim() * sizeof(float), nb = (size_t)l->out_dim() * l->lora.rank * sizeof(float);
  if (a) RT_CUDA(c, cudaMemcpyAsync(a, l->lora.a, na, cudaMemcpyDeviceToHost, c->stream));
  if (b) RT_CUDA(c, cudaMemcpyAsync(b, l->lora.b, nb, cudaMemcpyDeviceToHost, c->stream));
  if (ga) RT_CUDA(c, cudaMemcpyAsync(ga, l->lora.ga, na, cudaMemcpyDeviceToHost, c->stream));
  if (gb) RT_CUDA(c, cudaMemcpyAsync(gb, l->lora.gb, nb, cudaMemcpyDeviceToHost, c->stream));
  return c->check_device_status("rt_lora_read");
}

rt_status rt_lora_write(rt_linear* l, const float* a, const float* b) {
  if (!l) return RT_ERR_BAD_ARG;
  rt_ctx* c = l->ctx;
  if (!l->has_lora) return c->fail(RT_ERR_BAD_ARG, "linear has no adapter");
  RT_CUDA(c, cudaSetDevice(c->device));
  const size_t na = (size_t)l->lora.rank * l->in_dim() * sizeof(float), nb = (size_t)l->out_dim() * l->lora.rank * sizeof(float);
  if (a) RT_CUDA(c, cudaMemcpyAsync(l->lora.a, a, na, cudaMemcpyHostToDevice, c->stream));
  if (b) RT_CUDA(c, cudaMemcpyAsync(l->lora.b, b, nb, cudaMemcpyHostToDevice, c->stream));
  RT_CUDA(c, cudaStreamSynchronize(c->stream));
  l->lora.stale = true;
  ++l->lora.version;
  return RT_OK;
}

rt_status rt_lora_zero_grad(rt_linear* l) {
  if (!l) return RT_ERR_BAD_ARG;
  rt_ctx* c = l->ctx;
  if (!l->has_lora) return RT_OK;
  RT_CUDA(c, cudaSetDevice(c->device));
  const size_t na = (size_t)l->lora.rank * l->in_dim() * sizeof(float), nb = (size_t)l->out_dim() * l->lora.rank * sizeof(float);
  RT_CUDA(c, cudaMemsetAsync(l->lora.ga, 0, na, c->stream));
  RT_CUDA(c, cudaMemsetAsync(l->lora.gb, 0, nb, c->stream));
  return RT_OK;
}

const char* rt_linear_name(const rt_linear* l) { return l ? l->name.c_str() : ""; }
size_t rt_linear_in_dim(const rt_linear* l) { return l ? (size_t)l->in_dim() : 0; }
size_t rt_linear_out_dim(const rt_linear* l) { return l ? (size_t)l->out_dim() : 0; }
int rt_linear_lora_rank(const rt_linear* l) { return (l && l->has_lora) ? l->lora.rank : 0; }

// ------------------------------------------------------------------ level 3
static const char* LIN_NAMES[7] = {"attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"};
static const char* HF_NAMES[7] = {"q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"};

rt_status rt_model_create(rt_ctx* c, const rt_model_config* cfg, rt_model** out) {
  if (!c || !cfg || !out) return RT_ERR_BAD_ARG;
  *out = nullptr;
  if (cfg->vocab <= 0 || cfg->hidden <= 0 || cfg->ff <= 0 || cfg->n_layers <= 0 || cfg->n_heads <= 0 ||
      cfg->n_kv_heads <= 0 || cfg->n_heads % cfg->n_kv_heads != 0)
    return c->fail(RT_ERR_BAD_SHAPE, "bad model dimensions");
  if (cfg->head_dim != 64 && cfg->head_dim != 128) return c->fail(RT_ERR_BAD_SHAPE, "head_dim must be 64 or 128");
  if (cfg->rot_dim <= 0 || cfg->rot_dim > cfg->head_dim || cfg->rot_dim % 2) return c->fail(RT_ERR_BAD_SHAPE, "bad rot_dim");
  rt_model* m = new rt_model();
  m->ctx = c;
  m->device = c->device;
  m->cfg = *cfg;
  if (m->cfg.head_rows <= 0) m->cfg.head_rows = 1024;
  m->blocks.resize(cfg->n_layers);
  *out = m;
  return RT_OK;
}

void rt_model_destroy(rt_model* m) {
  if (!m) return;
  cudaSetDevice(m->device);
  if (rt::ctx_alive(m->ctx)) cudaStreamSynchronize(m->ctx->stream);
  else cudaDeviceSynchronize();  // destroyed after its context: the stream is gone, the device is not
  for (auto& b : m->blocks) {
    for (int i = 0; i < 7; ++i)
      if (b.lin[i]) rt_linear_destroy(b.lin[i]);
    b.qkv.store.release(); b.qkv.lora_copies.release();
    b.gu.store.release(); b.gu.lora_copies.release();
  }
  if (m->lm_head && m->lm_head != m->embed) rt_frozen_destroy(m->lm_head);
  if (m->embed) rt_frozen_destroy(m->embed);
  for (void* p : m->owned) cudaFree(p);
  DevBuf* bufs[] = {&m->P, &m->G, &m->Mo, &m->Vo, &m->opt_scalars, &m->inv_freq, &m->rope_cos, &m->rope_sin,
                    &m->lsc.hs, &m->lsc.gs, &m->lsc.hs2, &m->lsc.gs2, &m->lsc.smax, &m->lsc.grad_ws, &m->tokens, &m->pos, &m->seq_start, &m->x, &m->ckpt, &m->h,
                    &m->n1, &m->n2, &m->q_raw, &m->k_raw, &m->v_raw, &m->q16, &m->k16, &m->v16, &m->o16, &m->lse,
                    &m->delta, &m->g16, &m->u16, &m->hm16, &m->dx, &m->dy16, &m->sc_y, &m->dhm, &m->dg16, &m->du16,
                    &m->sc_g, &m->sc_u, &m->dn, &m->d_o, &m->dO16, &m->amax, &m->dq, &m->dk, &m->dv, &m->dq16, &m->dk16,
                    &m->dv16, &m->sc_q, &m->sc_k, &m->sc_v, &m->tpos, &m->ttok, &m->tw, &m->logp, &m->hits, &m->xs,
                    &m->ns16, &m->logits, &m->dl16, &m->sc_l, &m->dns, &m->dxs};
  for (DevBuf* b : bufs) b->release();
  for (int i = 0; i < 7; ++i) m->hs_keep[i].release();
  m->gap.release();
  m->argmax.release();
  for (auto& ge : m->graphs) cudaGraphExecDestroy(ge.exec);
  delete m;
}

static rt_status upload_f32(rt_model* m, const void* data, size_t n, float** out) {
  rt_ctx* c = m->ctx;
  float* p = nullptr;
  RT_CUDA(c, cudaMalloc(&p, n * sizeof(float)));
  m->owned.push_back(p);
  RT_CUDA(c, cudaMemcpy(p, data, n * sizeof(float), cudaMemcpyHostToDevice));
  *out = p;
  return RT_OK;
}

rt_status rt_model_set_tensor(rt_model* m, const char* name, int ggml_type, size_t rows, size_t cols,
                              const void* data, size_t nbytes) {
  if (!m || !name || !data) return RT_ERR_BAD_ARG;
  rt_ctx* c = m->ctx;
  RT_CUDA(c, cudaSetDevice(c->device));
  const rt_model_config& g = m->cfg;
  const std::string n(name);
  const size_t d = g.hidden, qd = (size_t)g.n_heads * g.head_dim, kvd = (size_t)g.n_kv_heads * g.head_dim;
  auto want_f32 = [&](size_t len) -> rt_status {
    if (ggml_type != 0) return c->fail(RT_ERR_UNSUPPORTED_TYPE, n + ": expected an f32 tensor");
    if (rows * cols != len || nbytes != len * 4) return c->fail(RT_ERR_BAD_SHAPE, n + ": wrong length");
    return RT_OK;
  };
  rt_status st;
  if (n == "token_embd.weight" || n == "output.weight") {
    if (rows != (size_t)g.vocab || cols != d) return c->fail(RT_ERR_BAD_SHAPE, n + ": expected [vocab x hidden]");
    rt_frozen* f = nullptr;
    st = rt_frozen_create(c, ggml_type, rows, cols, data, nbytes, &f);
    if (st) return st;
    if (n == "token_embd.weight") {
      if (m->embed) rt_frozen_destroy(m->embed);
      m->embed = f;
    } else {
      if (g.tie_embeddings) {
        rt_frozen_destroy(f);
        return c->fail(RT_ERR_BAD_ARG, "output.weight given for a model with tied embeddings");
      }
      if (m->lm_head) rt_frozen_destroy(m->lm_head);
      m->lm_head = f;
    }
    return RT_OK;
  }
  if (n == "output_norm.weight") {
    if ((st = want_f32(d))) return st;
    return upload_f32(m, data, d, &m->final_norm);
  }
  if (n == "rope_freqs.weight") {
    if ((st = want_f32((size_t)g.rot_dim / 2))) return st;
    m->rope_factors.assign((const float*)data, (const float*)data + g.rot_dim / 2);
    m->rope_max_pos = 0;
    return RT_OK;
  }
  int li = -1, off = 0;
  if (sscanf(name, "blk.%d.%n", &li, &off) < 1 || off == 0 || li < 0 || li >= g.n_layers)
    return c->fail(RT_ERR_BAD_ARG, n + ": unknown tensor name");
  const std::string rest(name + off);
  BlockDev& b = m->blocks[li];
  if (rest == "attn_norm.weight") { if ((st = want_f32(d))) return st; return upload_f32(m, data, d, &b.input_norm); }
  if (rest == "ffn_norm.weight") { if ((st = want_f32(d))) return st; return upload_f32(m, data, d, &b.post_norm); }
  if (rest == "attn_q_norm.weight") { if ((st = want_f32(g.head_dim))) return st; return upload_f32(m, data, g.head_dim, &b.q_norm); }
  if (rest == "attn_k_norm.weight") { if ((st = want_f32(g.head_dim))) return st; return upload_f32(m, data, g.head_dim, &b.k_norm); }
  const size_t shapes[7][2] = {{qd, d}, {kvd, d}, {kvd, d}, {d, qd}, {(size_t)g.ff, d}, {(size_t)g.ff, d}, {d, (size_t)g.ff}};
  for (int i = 0; i < 7; ++i) {
    if (rest == std::string(LIN_NAMES[i]) + ".weight") {
      if (rows != shapes[i][0] || cols != shapes[i][1]) return c->fail(RT_ERR_BAD_SHAPE, n + ": wrong shape for this configuration");
      rt_frozen* f = nullptr;
      st = rt_frozen_create(c, ggml_type, rows, cols, data, nbytes, &f);
      if (st) return st;
      if (b.lin[i]) rt_linear_destroy(b.lin[i]);
      rt_linear* l = nullptr;
      char nm[64];
      snprintf(nm, sizeof nm, "blk.%d.%s", li, LIN_NAMES[i]);
      st = rt_linear_create(c, f, nullptr, nm, &l);
      if (st) { rt_frozen_destroy(f); return st; }
      l->owns_w = true;
      b.lin[i] = l;
      return RT_OK;
    }
    if (i < 3 && rest == std::string(LIN_NAMES[i]) + ".bias") {
      if (!b.lin[i]) return c->fail(RT_ERR_BAD_ARG, n + ": set the weight before its bias");
      if ((st = want_f32(shapes[i][0]))) return st;
      rt_linear* l = b.lin[i];  // the linear owns its bias
      if (!l->bias) RT_CUDA(c, cudaMalloc(&l->bias, shapes[i][0] * sizeof(float)));
      RT_CUDA(c, cudaMemcpy(l->bias, data, shapes[i][0] * sizeof(float), cudaMemcpyHostToDevice));
      return RT_OK;
    }
  }
  return c->fail(RT_ERR_BAD_ARG, n + ": unknown tensor name");
}


// Stack the packed weights of `n` linears along the output rows (see LinGroup).  The members keep
// working on their own: their handles point into the stacked buffer afterwards.
static rt_status build_group(rt_model* m, LinGroup& g, rt_linear** lin, int n) {
  rt_ctx* c = m->ctx;
  g = LinGroup();
  g.n = n;
  const QWeight& w0 = lin[0]->w->w;
  size_t bytes = 0;
  bool has_bias = false;
  for (int i = 0; i < n; ++i) {
    g.lin[i] = lin[i];
    const QWeight& w = lin[i]->w->w;
    if (w.fmt != w0.fmt || w.cols != w0.cols || w.rows % 128 != 0 || lin[i]->w->borrowed || w.f32) return RT_OK;  // stays unstacked
    g.row_off[i] = g.rows_total;
    g.rows_total += w.rows;
    bytes += w.dev_nbytes;
    has_bias |= lin[i]->bias != nullptr;
  }
  if (!g.store.reserve(bytes)) return c->fail(RT_ERR_CUDA, "out of device memory (stacked weights)");
  g.w = w0;
  g.w.rows = g.rows_total;
  g.w.dev_nbytes = bytes;
  g.w.ggml_nbytes = 0;
  const bool is16 = fmt_is_16bit(w0.fmt);
  if (is16) g.w.dense16 = g.store.p;
  else { g.w.bricks = (uint8_t*)g.store.p; g.w.nbr = g.rows_total / 64; }
  size_t off = 0;
  for (int i = 0; i < n; ++i) {
    QWeight& w = lin[i]->w->w;
    uint8_t* dst = (uint8_t*)g.store.p + off;
    RT_CUDA(c, cudaMemcpy(dst, is16 ? w.dense16 : (void*)w.bricks, w.dev_nbytes, cudaMemcpyDeviceToDevice));
    RT_CUDA(c, cudaFree(is16 ? w.dense16 : (void*)w.bricks));
    if (is16) w.dense16 = dst; else w.bricks = dst;
    lin[i]->w->borrowed = true;
    off += w.dev_nbytes;
  }
  if (has_bias) {
    RT_CUDA(c, cudaMalloc(&g.bias, (size_t)g.rows_total * sizeof(float)));
    m->owned.push_back(g.bias);
    RT_CUDA(c, cudaMemset(g.bias, 0, (size_t)g.rows_total * sizeof(float)));
    for (int i = 0; i < n; ++i)
      if (lin[i]->bias)
        RT_CUDA(c, cudaMemcpy(g.bias + g.row_off[i], lin[i]->bias, (size_t)lin[i]->out_dim() * sizeof(float), cudaMemcpyDeviceToDevice));
  }
  g.stacked = true;
  g.lora_ok = true;  // no adapters yet
  return RT_OK;
}

// After adapters are attached: lay the members' adapters out as one stacked low-rank chunk.
static rt_status build_group_lora(rt_model* m, LinGroup& g) {
  rt_ctx* c = m->ctx;
  if (!g.stacked) return RT_OK;
  g.rank_total = 0;
  g.lora_ok = true;
  for (int i = 0; i < g.n; ++i) {
    g.seen[i] = 0;
    g.rank_off[i] = g.rank_total;
    if (!g.lin[i]->has_lora) continue;
    const int r = g.lin[i]->lora.rank;
    if (r % 8 != 0) g.lora_ok = false;  // column offsets must stay 16-byte aligned
    g.rank_total += r;
  }
  if (g.rank_total > 64 || (g.rank_total & 1)) g.lora_ok = false;
  if (g.rank_total == 0 || !g.lora_ok) return RT_OK;
  const size_t K = (size_t)g.w.cols, NT = (size_t)g.rows_total, R = (size_t)g.rank_total;
  auto up = [](size_t n) { return (n * 2 + 255) / 256 * 256; };
  const size_t total = 2 * up(R * K) + up(NT * 64) + up(R * NT);
  if (!g.lora_copies.reserve(total)) return c->fail(RT_ERR_CUDA, "out of device memory (stacked adapter copies)");
  RT_CUDA(c, cudaMemset(g.lora_copies.p, 0, g.lora_copies.bytes));
  uint8_t* base = (uint8_t*)g.lora_copies.p;
  g.a_s = (__half*)base;
  g.a_h = (__half*)(base + up(R * K));
  g.bp = (__half*)(base + 2 * up(R * K));
  g.bt_s = (__half*)(base + 2 * up(R * K) + up(NT * 64));
  return RT_OK;
}

rt_status rt_model_finalize(rt_model* m) {
  if (!m) return RT_ERR_BAD_ARG;
  rt_ctx* c = m->ctx;
  if (!m->embed) return c->fail(RT_ERR_BAD_ARG, "token_embd.weight missing");
  if (m->cfg.tie_embeddings) m->lm_head = m->embed;
  if (!m->lm_head) return c->fail(RT_ERR_BAD_ARG, "output.weight missing (untied model)");
  if (!m->final_norm) return c->fail(RT_ERR_BAD_ARG, "output_norm.weight missing");
  for (int li = 0; li < m->cfg.n_layers; ++li) {
    BlockDev& b = m->blocks[li];
    char buf[96];
    if (!b.input_norm || !b.post_norm) { snprintf(buf, sizeof buf, "blk.%d: norm weights missing", li); return c->fail(RT_ERR_BAD_ARG, buf); }
    if (m->cfg.qk_norm && (!b.q_norm || !b.k_norm)) { snprintf(buf, sizeof buf, "blk.%d: q/k norm weights missing", li); return c->fail(RT_ERR_BAD_ARG, buf); }
    for (int i = 0; i < 7; ++i)
      if (!b.lin[i]) { snprintf(buf, sizeof buf, "blk.%d.%s.weight missing", li, LIN_NAMES[i]); return c->fail(RT_ERR_BAD_ARG, buf); }
  }
  // opt_scalars: [0,1024) f64 partials, [1024] f64 sum, then one f32 norm
  if (!m->opt_scalars.reserve(1025 * sizeof(double) + 16) || !m->amax.reserve(16)) return c->fail(RT_ERR_CUDA, "out of device memory");
  if (!m->finalized) {
    const char* e = getenv("RT_B200_NO_GROUPS");  // measurement aid: one matmul per projection
    if (!(e && e[0] == '1'))
      for (auto& b : m->blocks) {
        rt_status st = build_group(m, b.qkv, &b.lin[0], 3);
        if (!st) st = build_group(m, b.gu, &b.lin[4], 2);
        if (st) return st;
      }
  }
  m->finalized = true;
  return RT_OK;
}

rt_status rt_model_attach_lora(rt_model* m, int rank, float alpha, const char* targets, uint64_t seed, size_t* n_out) {
  if (!m) return RT_ERR_BAD_ARG;
  rt_ctx* c = m->ctx;
  if (!m->finalized) return c->fail(RT_ERR_BAD_ARG, "finalize the model first");
  if (rank <= 0 || rank > 64) return c->fail(RT_ERR_BAD_ARG, "LoRA rank must be in 1..64");
  RT_CUDA(c, cudaSetDevice(c->device));
  // a target is a projection type (GGUF or HF short name: every layer's) or one module by its full
  // GGUF name ("blk.3.attn_q"), which is how an adapter file names what it holds
  const int NL = m->cfg.n_layers;
  std::vector<char> sel((size_t)NL * 7, targets == nullptr ? 1 : 0);
  if (targets) {
    std::string t(targets);
    size_t p = 0;
    while (p <= t.size()) {
      size_t e = t.find(',', p);
      if (e == std::string::npos) e = t.size();
      std::string tok = t.substr(p, e - p);
      bool known = tok.empty();
      for (int i = 0; i < 7; ++i)
        if (tok == LIN_NAMES[i] || tok == HF_NAMES[i]) {
          for (int li = 0; li < NL; ++li) sel[(size_t)li * 7 + i] = 1;
          known = true;
        }
      int li = -1, off = 0;
      if (!known && sscanf(tok.c_str(), "blk.%d.%n", &li, &off) >= 1 && off > 0 && li >= 0 && li < NL)
        for (int i = 0; i < 7; ++i)
          if (tok.substr(off) == LIN_NAMES[i]) {
            sel[(size_t)li * 7 + i] = 1;
            known = true;
          }
      (void)known;  // a name that matches nothing is skipped, as Model::attach_lora does (its default list names DeltaNet projections too)
      p = e + 1;
    }
  }
  m->lora_order.clear();
  size_t total = 0;
  for (int li = 0; li < NL; ++li) {
    BlockDev& b = m->blocks[li];
    for (int i = 0; i < 7; ++i) {
      b.lin[i]->has_lora = false;
      b.lin[i]->lora_enabled = true;
      if (sel[(size_t)li * 7 + i]) {
        m->lora_order.push_back(b.lin[i]);
        total += (size_t)rank * (b.lin[i]->in_dim() + b.lin[i]->out_dim());
      }
    }
  }
  m->n_params = total;
  if (total == 0) {
    for (auto& b : m->blocks) { build_group_lora(m, b.qkv); build_group_lora(m, b.gu); }
    if (n_out) *n_out = 0;
    return RT_OK;
  }
  const size_t bytes = total * sizeof(float);
  if (!m->P.reserve(bytes) || !m->G.reserve(bytes) || !m->Mo.reserve(bytes) || !m->Vo.reserve(bytes))
    return c->fail(RT_ERR_CUDA, "out of device memory (adapter state)");
  std::vector<float> host(total, 0.f);
  SplitMix rng(seed);
  size_t off = 0;
  for (rt_linear* l : m->lora_order) {
    const size_t na = (size_t)rank * l->in_dim(), nb = (size_t)l->out_dim() * rank;
    const float bound = 1.0f / sqrtf((float)l->in_dim());
    for (size_t i = 0; i < na; ++i) host[off + i] = rng.uniform_sym(bound);
    float* base = m->P.as<float>();
    float* gbase = m->G.as<float>();
    rt_status st = attach_views(l, rank, alpha, base + off, base + off + na, gbase + off, gbase + off + na);
    if (st) return st;
    off += na + nb;
  }
  for (auto& b : m->blocks) {
    rt_status st = build_group_lora(m, b.qkv);
    if (!st) st = build_group_lora(m, b.gu);
    if (st) return st;
  }
  RT_CUDA(c, cudaMemcpy(m->P.p, host.data(), bytes, cudaMemcpyHostToDevice));
  RT_CUDA(c, cudaMemset(m->G.p, 0, bytes));
  RT_CUDA(c, cudaMemset(m->Mo.p, 0, bytes));
  RT_CUDA(c, cudaMemset(m->Vo.p, 0, bytes));
  m->opt_t = 0;
  for (int i = 0; i < 7; ++i)
    if (m->hs_keep[i].p) RT_CUDA(c, cudaMemset(m->hs_keep[i].p, 0, m->hs_keep[i].bytes));
  // the copies and clears above went through the legacy stream; the first pass launches on the
  // ctx's non-blocking stream, which nothing orders after them except this
  RT_CUDA(c, cudaDeviceSynchronize());
  if (n_out) *n_out = total;
  return RT_OK;
}

size_t rt_model_num_lora(const rt_model* m) { return m ? m->lora_order.size() : 0; }
rt_linear* rt_model_lora_linear(rt_model* m, size_t i) { return (m && i < m->lora_order.size()) ? m->lora_order[i] : nullptr; }

rt_status rt_model_set_lora_enabled(rt_model* m, int on) {
  if (!m) return RT_ERR_BAD_ARG;
  for (auto& b : m->blocks)
    for (int i = 0; i < 7; ++i)
      if (b.lin[i]) b.lin[i]->lora_enabled = on != 0;
  return RT_OK;
}

rt_status rt_model_zero_grad(rt_model* m) {
  if (!m) return RT_ERR_BAD_ARG;
  rt_ctx* c = m->ctx;
  if (m->n_params == 0) return RT_OK;
  RT_CUDA(c, cudaSetDevice(c->device));
  RT_CUDA(c, cudaMemsetAsync(m->G.p, 0, m->n_params * sizeof(float), c->stream));
  return RT_OK;
}

rt_status rt_model_set_checkpointing(rt_model* m, int32_t mode) {
  if (!m || mode < -1 || mode > 1) return RT_ERR_BAD_ARG;
  m->recompute_policy = mode < 0 ? 0 : (mode == 1 ? 1 : 2);
  m->cap_tokens = 0;  // the next batch decides again and sizes the buffers for its mode
  return RT_OK;
}

int32_t rt_model_checkpointing(const rt_model* m) { return (m && m->store_acts) ? 0 : 1; }

rt_status rt_model_grad_buffer(rt_model* m, void** p, size_t* n) {
  if (!m || !p || !n) return RT_ERR_BAD_ARG;
  *p = m->G.p;
  *n = m->n_params;
  return RT_OK;
}

// ---- workspace
static bool ensure_tokens(rt_model* m, int M) {
  if (M <= m->cap_tokens) return true;
  const rt_model_config& g = m->cfg;
  const size_t d = g.hidden, ff = g.ff, qd = (size_t)g.n_heads * g.head_dim, kvd = (size_t)g.n_kv_heads * g.head_dim;
  const size_t T = (size_t)M;
  // per-layer bytes of everything a block's backward reads from its forward
  const size_t per_layer = T * (d * 2 * 2 + (qd + 2 * kvd) * 4 + qd * 2 * 2 + kvd * 2 * 2 + (size_t)g.n_heads * 4 + d * 4 + ff * 2 * 3 + 7 * 64 * 2);
  if (m->recompute_policy < 0) {
    const char* e = getenv("RT_B200_RECOMPUTE");
    m->recompute_policy = (e && e[0] == '1') ? 1 : 0;
  }
  m->store_acts = m->recompute_policy == 2;
  if (m->recompute_policy == 0 && g.n_layers > 1) {
    size_t free_b = 0, total_b = 0;
    if (cudaMemGetInfo(&free_b, &total_b) == cudaSuccess) {
      const size_t held = m->n1.bytes + m->n2.bytes + m->q_raw.bytes + m->k_raw.bytes + m->q16.bytes + m->k16.bytes + m->v16.bytes +
                          m->o16.bytes + m->lse.bytes + m->h.bytes + m->g16.bytes + m->u16.bytes + m->hm16.bytes;
      const size_t need = per_layer * g.n_layers;
      m->store_acts = need <= held || (double)(need - held) <= 0.6 * (double)free_b;
    }
  }
  const size_t L = m->store_acts ? (size_t)g.n_layers : 1;
  bool ok = true;
  ok &= m->tokens.reserve(T * 4) && m->pos.reserve(T * 4) && m->seq_start.reserve(T * 4);
  ok &= m->x.reserve(T * d * 4) && m->ckpt.reserve(T * d * 4 * g.n_layers) && m->h.reserve(T * d * 4 * L);
  ok &= m->n1.reserve(T * d * 2 * L) && m->n2.reserve(T * d * 2 * L);
  ok &= m->q_raw.reserve(T * (qd + 2 * kvd) * 4 * L);  // q | k | v before RoPE
  ok &= m->q16.reserve(T * qd * 2 * L) && m->k16.reserve(T * kvd * 2 * L) && m->v16.reserve(T * kvd * 2 * L) && m->o16.reserve(T * qd * 2 * L);
  ok &= m->lse.reserve(T * g.n_heads * 4 * L) && m->delta.reserve(T * g.n_heads * 4);
  ok &= m->g16.reserve(T * ff * 2 * 2 * L) && m->hm16.reserve(T * ff * 2 * L);  // gate | up
  ok &= m->dx.reserve(T * d * 4) && m->dy16.reserve(T * d * 2) && m->sc_y.reserve(T * 4);
  ok &= m->dhm.reserve(T * ff * 2) && m->dg16.reserve(T * ff * 2 * 2);  // d(gate) | d(up)
  ok &= m->sc_g.reserve(T * 4) && m->sc_u.reserve(T * 4) && m->dn.reserve(T * d * 4);
  ok &= m->dO16.reserve(T * qd * 2) && m->amax.reserve(2 * T * 4 + 16);  // amax: per token, its sequence's largest factor, then its weight against it
  ok &= m->dq.reserve(T * qd * 4) && m->dk.reserve(T * kvd * 4) && m->dv.reserve(T * kvd * 4);
  ok &= m->dq16.reserve(T * (qd + 2 * kvd) * 2);  // d(q) | d(k) | d(v)
  ok &= m->sc_q.reserve(T * 4) && m->sc_k.reserve(T * 4) && m->sc_v.reserve(T * 4);
  // zero beyond the rank, kept that way; 256 bytes of slack for reads that start at a column offset
  // every layer keeps its own Hs (128 bytes per token, layer and linear) whether or not the other
  // caches are kept: a recomputed forward then reuses it instead of running the low-rank products again
  for (int i = 0; i < 7; ++i) ok &= m->hs_keep[i].reserve(T * 64 * 2 * (size_t)g.n_layers + 256, true);
  if (ok) m->cap_tokens = M;
  return ok;
}

// One layer's view of the forward state its backward reads.  When every layer's state is kept,
// layer li owns the li-th slice (of M tokens) of each buffer; otherwise all layers share slice 0.
struct BlockActs {
  __half *n1, *n2, *q16, *k16, *v16, *o16, *g16, *u16, *hm16, *hs[7];
  float *q_raw, *k_raw, *v_raw, *h, *lse;
  size_t qkv_pitch, gu_pitch;  // 0: separate matrices; else q|k|v (gate|up) are column slices of one matrix
  bool qkv_group, gu_group;
};
static BlockActs block_acts(rt_model* m, int li, int M, bool own_slice) {
  const rt_model_config& g = m->cfg;
  const size_t d = g.hidden, ff = g.ff, qd = (size_t)g.n_heads * g.head_dim, kvd = (size_t)g.n_kv_heads * g.head_dim;
  const size_t o = own_slice ? (size_t)li * (size_t)M : 0, T = (size_t)M;
  BlockDev& b = m->blocks[li];
  BlockActs a;
  a.qkv_group = group_usable(b.qkv) && qk_rope_takes_pitches(g.n_heads, g.n_kv_heads, g.head_dim, g.rot_dim, g.rope_neox);
  a.gu_group = group_usable(b.gu) && (ff % 8 == 0);
  a.n1 = m->n1.as<__half>() + o * d;
  a.n2 = m->n2.as<__half>() + o * d;
  a.q16 = m->q16.as<__half>() + o * qd;
  a.k16 = m->k16.as<__half>() + o * kvd;
  a.v16 = m->v16.as<__half>() + o * kvd;
  a.o16 = m->o16.as<__half>() + o * qd;
  a.hm16 = m->hm16.as<__half>() + o * ff;
  for (int i = 0; i < 7; ++i) a.hs[i] = m->hs_keep[i].as<__half>() + (size_t)li * T * 64;
  float* qkv = m->q_raw.as<float>() + o * (qd + 2 * kvd);
  a.q_raw = qkv;
  a.k_raw = a.qkv_group ? qkv + qd : qkv + T * qd;
  a.v_raw = a.qkv_group ? qkv + qd + kvd : qkv + T * (qd + kvd);
  a.qkv_pitch = a.qkv_group ? qd + 2 * kvd : 0;
  __half* gu = m->g16.as<__half>() + o * 2 * ff;
  a.g16 = gu;
  a.u16 = a.gu_group ? gu + ff : gu + T * ff;
  a.gu_pitch = a.gu_group ? 2 * ff : 0;
  a.h = m->h.as<float>() + o * d;
  a.lse = m->lse.as<float>() + o * g.n_heads;
  return a;
}

static bool ensure_targets(rt_model* m, int n, bool backward) {
  const rt_model_config& g = m->cfg;
  bool ok = true;
  if (n > m->cap_targets) {
    ok &= m->tpos.reserve((size_t)n * 4) && m->ttok.reserve((size_t)n * 4) && m->tw.reserve((size_t)n * 4) &&
          m->logp.reserve((size_t)n * 4) && m->hits.reserve(16);
    if (ok) m->cap_targets = n;
  }
  const int R = n < g.head_rows ? n : g.head_rows;
  const size_t d = g.hidden, V = g.vocab;
  if (R > m->cap_head_rows) {
    ok &= m->xs.reserve((size_t)R * d * 4) && m->ns16.reserve((size_t)R * d * 2) && m->logits.reserve((size_t)R * V * 4);
    ok &= m->sc_l.reserve((size_t)R * 4) && m->dns.reserve((size_t)R * d * 4) && m->dxs.reserve((size_t)R * d * 4);
    if (ok) m->cap_head_rows = R;
  }
  // the logit gradients exist only for backward passes and are sized on their own: a forward-only
  // call may have raised cap_head_rows past what an earlier backward pass allocated here
  if (backward) ok &= m->dl16.reserve((size_t)R * V * 2);
  return ok;
}

// ops.rs:118-131 inverse frequencies (host, f32 like the reference), tables on the device
static rt_status ensure_rope(rt_model* m, int max_pos) {
  rt_ctx* c = m->ctx;
  if (max_pos <= m->rope_max_pos) return RT_OK;
  const rt_model_config& g = m->cfg;
  const int half = g.rot_dim / 2;
  int cap = 256;
  while (cap < max_pos) cap *= 2;
  std::vector<float> inv(half);
  for (int i = 0; i < half; ++i) {
    float f = powf(g.rope_theta, -2.0f * (float)i / (float)g.rot_dim) * g.rope_freq_scale;
    if (i < (int)m->rope_factors.size() && m->rope_factors[i] != 0.0f) f /= m->rope_factors[i];
    inv[i] = f;
  }
  if (!m->inv_freq.reserve(half * 4) || !m->rope_cos.reserve((size_t)cap * half * 4) || !m->rope_sin.reserve((size_t)cap * half * 4))
    return c->fail(RT_ERR_CUDA, "out of device memory (rope tables)");
  RT_CUDA(c, cudaMemcpyAsync(m->inv_freq.p, inv.data(), half * 4, cudaMemcpyHostToDevice, c->stream));
  RT_CUDA(c, cudaStreamSynchronize(c->stream));
  launch_rope_table(m->inv_freq.as<float>(), half, cap, m->rope_cos.as<float>(), m->rope_sin.as<float>(), c->stream);
  m->rope_max_pos = cap;
  return RT_OK;
}



// Block::forward (src/model.rs:165-183).  x_in is read only; h receives x_in + attention;
// when x_out is non-null it receives the block output (h + mlp), and may alias h.  With `keep`
// the adapters' Hs = X.(sA)^T are left in A.hs for the block's backward.
// hs: 0 = the adapters' Hs go to scratch (forward-only passes), 1 = they are left in A.hs for the
// block's backward, 2 = A.hs already holds them (the block's second forward when its caches are rebuilt).
static rt_status block_forward(rt_model* m, int li, int M, const float* x_in, float* h, float* x_out, const BlockActs& A,
                               int hs) {
  const bool keep = hs != 0, hs_ready = hs == 2;
  rt_ctx* c = m->ctx;
  const rt_model_config& g = m->cfg;
  BlockDev& b = m->blocks[li];
  cudaStream_t st = c->stream;
  const int d = g.hidden;
  launch_rmsnorm_fwd(x_in, b.input_norm, M, d, g.rms_eps, A.n1, st);
  if (A.qkv_group) {
    RT_TRY(group_forward_dev(b.qkv, m->lsc, A.n1, M, A.q_raw, RT_DT_F32, keep ? A.hs[0] : nullptr, hs_ready));
  } else {
    RT_TRY(linear_forward_dev(b.lin[0], m->lsc, A.n1, M, A.q_raw, RT_DT_F32, 0, keep ? A.hs[0] : nullptr, hs_ready));
    RT_TRY(linear_forward_dev(b.lin[1], m->lsc, A.n1, M, A.k_raw, RT_DT_F32, 0, keep ? A.hs[1] : nullptr, hs_ready));
    RT_TRY(linear_forward_dev(b.lin[2], m->lsc, A.n1, M, A.v_raw, RT_DT_F32, 0, keep ? A.hs[2] : nullptr, hs_ready));
  }
  launch_qk_rope_fwd(A.q_raw, A.k_raw, A.v_raw, A.qkv_pitch, g.qk_norm ? b.q_norm : nullptr,
                     g.qk_norm ? b.k_norm : nullptr, m->pos.as<int>(), m->rope_cos.as<float>(), m->rope_sin.as<float>(), M,
                     g.n_heads, g.n_kv_heads, g.head_dim, g.rot_dim, g.rope_neox, g.rms_eps, A.q16, A.k16, A.v16, st);
  if (attn_forward(c, A.q16, A.k16, A.v16, m->seq_start.as<int>(), m->staged_gap ? m->gap.as<int>() : nullptr, M, g.n_heads,
                   g.n_kv_heads, g.head_dim, A.o16, A.lse))
    return c->fail(RT_ERR_CUDA, "attention forward launch failed");
  if (h != x_in) RT_CUDA(c, cudaMemcpyAsync(h, x_in, (size_t)M * d * 4, cudaMemcpyDeviceToDevice, st));
  RT_TRY(linear_forward_dev(b.lin[3], m->lsc, A.o16, M, h, RT_DT_F32, 1, keep ? A.hs[3] : nullptr, hs_ready));
  launch_rmsnorm_fwd(h, b.post_norm, M, d, g.rms_eps, A.n2, st);
  if (A.gu_group) {
    RT_TRY(group_forward_dev(b.gu, m->lsc, A.n2, M, A.g16, RT_DT_F16, keep ? A.hs[4] : nullptr, hs_ready));
  } else {
    RT_TRY(linear_forward_dev(b.lin[4], m->lsc, A.n2, M, A.g16, RT_DT_F16, 0, keep ? A.hs[4] : nullptr, hs_ready));
    RT_TRY(linear_forward_dev(b.lin[5], m->lsc, A.n2, M, A.u16, RT_DT_F16, 0, keep ? A.hs[5] : nullptr, hs_ready));
  }
  launch_swiglu_fwd(A.g16, A.u16, A.gu_pitch, M, g.ff, A.hm16, c->status_dev, st);
  if (x_out) {
    if (x_out != h) RT_CUDA(c, cudaMemcpyAsync(x_out, h, (size_t)M * d * 4, cudaMemcpyDeviceToDevice, st));
    RT_TRY(linear_forward_dev(b.lin[6], m->lsc, A.hm16, M, x_out, RT_DT_F32, 1, keep ? A.hs[6] : nullptr, hs_ready));
  } else if (keep && !hs_ready && b.lin[6]->lora_active()) {
    RT_TRY(linear_lora_h(b.lin[6], A.hm16, M, A.hs[6]));  // the backward needs it
  }
  return RT_OK;
}

// Block::backward (src/model.rs:185-197).  On entry dx holds the gradient of the block output
// and (dy16, sc_y) its row-normalised f16 copy; on exit both describe the block input's.
static rt_status block_backward(rt_model* m, int li, int M, const float* x_in, const BlockActs& A) {
  rt_ctx* c = m->ctx;
  const rt_model_config& g = m->cfg;
  BlockDev& b = m->blocks[li];
  cudaStream_t st = c->stream;
  const int d = g.hidden;
  float* dx = m->dx.as<float>();
  __half* dy16 = m->dy16.as<__half>();
  float* sc_y = m->sc_y.as<float>();
#define HS(i) (b.lin[i]->lora_active() ? A.hs[i] : nullptr)
  // Mlp::backward (src/model.rs:120-134)
  // d(hm) leaves the matmul as f16 rows still lacking sc_y: SwiGLU's backward folds the factor into its own scales
  RT_TRY(linear_backward_dev(b.lin[6], m->lsc, A.hm16, dy16, sc_y, M, m->dhm.p, 0, HS(6), true));
  const size_t T = (size_t)M, ff = g.ff;
  __half* dg16 = m->dg16.as<__half>();
  __half* du16 = A.gu_group ? dg16 + ff : dg16 + T * ff;
  launch_swiglu_bwd(m->dhm.p, 1, sc_y, A.g16, A.u16, A.gu_pitch, M, g.ff, dg16, du16, A.gu_pitch, m->sc_g.as<float>(),
                    m->sc_u.as<float>(), st);
  if (A.gu_group) {
    RT_TRY(group_backward_dev(b.gu, m->lsc, A.n2, dg16, m->sc_g.as<float>(), M, m->dn.as<float>(), 0, HS(4)));
  } else {
    RT_TRY(linear_backward_dev(b.lin[4], m->lsc, A.n2, dg16, m->sc_g.as<float>(), M, m->dn.as<float>(), 0, HS(4)));
    RT_TRY(linear_backward_dev(b.lin[5], m->lsc, A.n2, du16, m->sc_u.as<float>(), M, m->dn.as<float>(), 1, HS(5)));
  }
  // dh = dy + rmsnorm_backward(h, post_norm, dn2)
  launch_rmsnorm_bwd(A.h, b.post_norm, m->dn.as<float>(), dx, M, d, g.rms_eps, dx, dy16, sc_y, st);
  // Attention::backward (src/attention.rs:246-367)
  // d(attention output) leaves the matmul as f16 rows still lacking sc_y; the attention backward
  // takes the factors per query row (in amax, for every token, the largest one of its own sequence:
  // nothing a sequence's backward sees may depend on its batch mates)
  RT_TRY(linear_backward_dev(b.lin[3], m->lsc, A.o16, dy16, sc_y, M, m->dO16.p, 0, HS(3), true));
  launch_rowscale_seqmax(sc_y, m->seq_start.as<int>(), M, m->amax.as<float>(), st);
  if (attn_backward(c, A.q16, A.k16, A.v16, A.o16, m->dO16.as<__half>(),
                    m->amax.as<float>(), sc_y, A.lse, m->seq_start.as<int>(), m->staged_gap ? m->gap.as<int>() : nullptr, M,
                    g.n_heads, g.n_kv_heads, g.head_dim,
                    m->delta.as<float>(), m->dq.as<float>(), m->dk.as<float>(), m->dv.as<float>()))
    return c->fail(RT_ERR_CUDA, "attention backward launch failed");
  const size_t qd = (size_t)g.n_heads * g.head_dim, kvd = (size_t)g.n_kv_heads * g.head_dim;
  __half* dq16 = m->dq16.as<__half>();
  __half* dk16 = A.qkv_group ? dq16 + qd : dq16 + T * qd;
  __half* dv16 = A.qkv_group ? dq16 + qd + kvd : dq16 + T * (qd + kvd);
  launch_qk_rope_bwd(m->dq.as<float>(), m->dk.as<float>(), m->dv.as<float>(), A.q_raw, A.k_raw, A.qkv_pitch,
                     g.qk_norm ? b.q_norm : nullptr, g.qk_norm ? b.k_norm : nullptr, m->pos.as<int>(), m->rope_cos.as<float>(),
                     m->rope_sin.as<float>(), M, g.n_heads, g.n_kv_heads, g.head_dim, g.rot_dim, g.rope_neox, g.rms_eps,
                     dq16, dk16, dv16, A.qkv_pitch, m->sc_q.as<float>(), m->sc_k.as<float>(), m->sc_v.as<float>(), st);
  if (A.qkv_group) {
    RT_TRY(group_backward_dev(b.qkv, m->lsc, A.n1, dq16, m->sc_q.as<float>(), M, m->dn.as<float>(), 0, HS(0)));
  } else {
    RT_TRY(linear_backward_dev(b.lin[0], m->lsc, A.n1, dq16, m->sc_q.as<float>(), M, m->dn.as<float>(), 0, HS(0)));
    RT_TRY(linear_backward_dev(b.lin[1], m->lsc, A.n1, dk16, m->sc_k.as<float>(), M, m->dn.as<float>(), 1, HS(1)));
    RT_TRY(linear_backward_dev(b.lin[2], m->lsc, A.n1, dv16, m->sc_v.as<float>(), M, m->dn.as<float>(), 1, HS(2)));
  }
  // dx = dh + rmsnorm_backward(x, input_norm, dn1)
  launch_rmsnorm_bwd(x_in, b.input_norm, m->dn.as<float>(), dx, M, d, g.rms_eps, dx, dy16, sc_y, st);
#undef HS
  return RT_OK;
}

// Model::head (src/model.rs:561-609) in chunks of head_rows targets.
static rt_status model_head(rt_model* m, int M, int n_targets, bool backward, float* logits_out_host) {
  rt_ctx* c = m->ctx;
  const rt_model_config& g = m->cfg;
  cudaStream_t st = c->stream;
  const int d = g.hidden, V = g.vocab;
  (void)M;
  RT_CUDA(c, cudaMemsetAsync(m->hits.p, 0, 4, st));
  rt_linear head;  // a bias-free, adapter-free Linear over the lm_head weight
  head.ctx = c;
  head.w = m->lm_head;
  for (int c0 = 0; c0 < n_targets; c0 += g.head_rows) {
    const int R = n_targets - c0 < g.head_rows ? n_targets - c0 : g.head_rows;
    const int* tpos = m->tpos.as<int>() + c0;
    launch_gather_f32_rows(m->x.as<float>(), tpos, R, d, m->xs.as<float>(), st);
    launch_rmsnorm_fwd(m->xs.as<float>(), m->final_norm, R, d, g.rms_eps, m->ns16.as<__half>(), st);
    RT_TRY(linear_forward_dev(&head, m->lsc, m->ns16.as<__half>(), R, m->logits.p, RT_DT_F32, 0));
    if (logits_out_host)
      RT_CUDA(c, cudaMemcpyAsync(logits_out_host + (size_t)c0 * V, m->logits.p, (size_t)R * V * 4, cudaMemcpyDeviceToHost, st));
    launch_ce_rows(m->logits.as<float>(), R, V, m->ttok.as<int>() + c0, m->tw.as<float>() + c0, m->logp.as<float>() + c0,
                   m->hits.as<int>(), backward ? m->dl16.as<__half>() : nullptr, backward ? m->sc_l.as<float>() : nullptr,
                   m->want_argmax ? m->argmax.as<int>() + c0 : nullptr, c->status_dev, st);
    if (backward) {
      RT_TRY(linear_backward_dev(&head, m->lsc, m->ns16.as<__half>(), m->dl16.as<__half>(), m->sc_l.as<float>(), R, m->dns.as<float>(), 0));
      launch_rmsnorm_bwd(m->xs.as<float>(), m->final_norm, m->dns.as<float>(), nullptr, R, d, g.rms_eps, m->dxs.as<float>(), nullptr, nullptr, st);
      launch_scatter_add_rows(m->dxs.as<float>(), tpos, R, d, m->dx.as<float>(), st);
    }
  }
  return RT_OK;
}

// positions / segments (both or neither): the reference's Packed layout (src/model.rs:234-290) for
// every sequence of the batch: a shared prompt (segment 0) followed by the examples' own tokens
// (segment k+1 for example k), each token keeping its position within its own example.
static rt_status upload_batch(rt_model* m, const int32_t* tokens, const int32_t* seq_offsets, int n_seq,
                              const int32_t* tpos, const int32_t* ttok, const float* tw, int n_targets, bool backward,
                              int* M_out, const int32_t* positions = nullptr, const int32_t* segments = nullptr) {
  rt_ctx* c = m->ctx;
  if (!m->finalized) return c->fail(RT_ERR_BAD_ARG, "finalize the model first");
  if (!tokens || !seq_offsets || n_seq <= 0) return c->fail(RT_ERR_BAD_ARG, "empty batch");
  if (n_targets < 0 || (n_targets > 0 && (!tpos || !ttok))) return c->fail(RT_ERR_BAD_ARG, "bad targets");
  if (seq_offsets[0] != 0) return c->fail(RT_ERR_BAD_ARG, "seq_offsets must start at 0");
  const long long M = seq_offsets[n_seq];
  if (M <= 0 || M > (1 << 24)) return c->fail(RT_ERR_BAD_SHAPE, "token count out of range");
  if ((positions == nullptr) != (segments == nullptr)) return c->fail(RT_ERR_BAD_ARG, "positions and segments go together");
  m->h_pos.resize(M);
  m->h_seq_start.resize(M);
  if (positions) m->h_gap.assign((size_t)M * 2, 0);
  int max_len = 0;
  for (int s = 0; s < n_seq; ++s) {
    const int a = seq_offsets[s], e = seq_offsets[s + 1];
    if (e <= a) return c->fail(RT_ERR_BAD_SHAPE, "empty or unordered sequence");
    for (int i = a; i < e; ++i) { m->h_pos[i] = i - a; m->h_seq_start[i] = a; }
    if (e - a > max_len) max_len = e - a;
    if (positions) {
      // segments: zeros (the shared prompt), then runs of 1, 2, ...; a token of run k may not see the
      // other runs, i.e. the keys from the end of the prompt up to the start of its own run
      int shared = 0;
      while (a + shared < e && segments[a + shared] == 0) ++shared;
      int run_start = a + shared, prev = 0;
      for (int i = a; i < e; ++i) {
        const int sg = segments[i], ps = positions[i];
        if (ps < 0 || ps >= (1 << 20)) return c->fail(RT_ERR_BAD_INDEX, "position out of range");
        if (i >= a + shared) {
          if (sg <= 0 || sg < prev || sg > prev + 1) return c->fail(RT_ERR_BAD_ARG, "segments must be 0.., then 1, 2, ... in runs");
          if (sg != prev) run_start = i;
          prev = sg;
          m->h_gap[2 * (size_t)i] = a + shared;
          m->h_gap[2 * (size_t)i + 1] = run_start;
        }
        m->h_pos[i] = ps;
        if (ps + 1 > max_len) max_len = ps + 1;
      }
    }
  }
  for (long long i = 0; i < M; ++i)
    if (tokens[i] < 0 || tokens[i] >= m->cfg.vocab) return c->fail(RT_ERR_BAD_INDEX, "token id out of vocabulary");  // model.rs:450 asserts
  for (int i = 0; i < n_targets; ++i) {
    if (tpos[i] < 0 || tpos[i] >= M) return c->fail(RT_ERR_BAD_INDEX, "target position out of range");  // model.rs:573 asserts
    if (ttok[i] < 0 || ttok[i] >= m->cfg.vocab) return c->fail(RT_ERR_BAD_INDEX, "target token out of vocabulary");
  }
  RT_CUDA(c, cudaSetDevice(c->device));
  if (!ensure_tokens(m, (int)M) || !ensure_targets(m, n_targets > 0 ? n_targets : 1, backward))
    return c->fail(RT_ERR_CUDA, "out of device memory (activations)");
  RT_TRY(ensure_rope(m, max_len));
  cudaStream_t st = c->stream;
  RT_CUDA(c, cudaMemcpyAsync(m->tokens.p, tokens, M * 4, cudaMemcpyHostToDevice, st));
  RT_CUDA(c, cudaMemcpyAsync(m->pos.p, m->h_pos.data(), M * 4, cudaMemcpyHostToDevice, st));
  RT_CUDA(c, cudaMemcpyAsync(m->seq_start.p, m->h_seq_start.data(), M * 4, cudaMemcpyHostToDevice, st));
  m->staged_gap = positions != nullptr;
  if (positions) {
    if (!m->gap.reserve((size_t)M * 8)) return c->fail(RT_ERR_CUDA, "out of device memory (activations)");
    RT_CUDA(c, cudaMemcpyAsync(m->gap.p, m->h_gap.data(), (size_t)M * 8, cudaMemcpyHostToDevice, st));
  }
  if (n_targets > 0) {
    RT_CUDA(c, cudaMemcpyAsync(m->tpos.p, tpos, (size_t)n_targets * 4, cudaMemcpyHostToDevice, st));
    RT_CUDA(c, cudaMemcpyAsync(m->ttok.p, ttok, (size_t)n_targets * 4, cudaMemcpyHostToDevice, st));
    if (tw) RT_CUDA(c, cudaMemcpyAsync(m->tw.p, tw, (size_t)n_targets * 4, cudaMemcpyHostToDevice, st));
  }
  *M_out = (int)M;
  return RT_OK;
}

static rt_status run_staged_body(rt_model* m, bool backward, float* logits_out_host) {
  rt_ctx* c = m->ctx;
  const int M = m->staged_tokens, n_targets = m->staged_targets;
  if (M <= 0) return c->fail(RT_ERR_BAD_ARG, "no batch staged");
  RT_CUDA(c, cudaSetDevice(c->device));
  cudaStream_t st = c->stream;
  const rt_model_config& g = m->cfg;
  const size_t xd = (size_t)M * g.hidden;
  float* x = m->x.as<float>();
  launch_gather_rows(m->embed->w, m->tokens.as<int>(), M, x, c->status_dev, st);
  const bool store = backward && m->store_acts;
  for (int li = 0; li < g.n_layers; ++li) {
    if (backward) RT_CUDA(c, cudaMemcpyAsync(m->ckpt.as<float>() + (size_t)li * xd, x, xd * 4, cudaMemcpyDeviceToDevice, st));
    const BlockActs A = block_acts(m, li, M, store);
    if (store) RT_TRY(block_forward(m, li, M, m->ckpt.as<float>() + (size_t)li * xd, A.h, x, A, 1));  // keeps h and every Hs
    else RT_TRY(block_forward(m, li, M, x, x, x, A, backward ? 1 : 0));  // a training pass keeps every Hs for the second forward
  }
  if (backward) RT_CUDA(c, cudaMemsetAsync(m->dx.p, 0, xd * 4, st));
  if (n_targets > 0) RT_TRY(model_head(m, M, n_targets, backward, logits_out_host));
  else RT_CUDA(c, cudaMemsetAsync(m->hits.p, 0, 4, st));
  if (!backward) return RT_OK;
  launch_normalize_rows(m->dx.as<float>(), M, g.hidden, m->dy16.as<__half>(), m->sc_y.as<float>(), st);
  for (int li = g.n_layers - 1; li >= 0; --li) {
    const float* x_in = m->ckpt.as<float>() + (size_t)li * xd;
    const BlockActs A = block_acts(m, li, M, store);
    if (!store) RT_TRY(block_forward(m, li, M, x_in, A.h, nullptr, A, 2));  // rebuild the block's caches (Hs is still there)
    RT_TRY(block_backward(m, li, M, x_in, A));
  }
  return RT_OK;
}

// Everything the captured launches point at: if any buffer moved, the graph is stale.
static uint64_t buffer_signature(rt_model* m) {
  uint64_t h = 1469598103934665603ull;
  auto mix = [&](const void* p) { h = (h ^ (uint64_t)(uintptr_t)p) * 1099511628211ull; };
  DevBuf* bufs[] = {&m->P, &m->G, &m->rope_cos, &m->rope_sin, &m->lsc.hs, &m->lsc.gs, &m->lsc.hs2, &m->lsc.gs2, &m->lsc.smax, &m->lsc.grad_ws,
                    &m->tokens, &m->pos, &m->seq_start, &m->x, &m->ckpt, &m->h, &m->n1, &m->n2, &m->q_raw, &m->k_raw, &m->v_raw,
                    &m->q16, &m->k16, &m->v16, &m->o16, &m->lse, &m->delta, &m->g16, &m->u16, &m->hm16, &m->dx, &m->dy16,
                    &m->sc_y, &m->dhm, &m->dg16, &m->du16, &m->sc_g, &m->sc_u, &m->dn, &m->d_o, &m->dO16, &m->amax, &m->dq,
                    &m->dk, &m->dv, &m->dq16, &m->dk16, &m->dv16, &m->sc_q, &m->sc_k, &m->sc_v, &m->tpos, &m->ttok, &m->tw,
                    &m->logp, &m->hits, &m->xs, &m->ns16, &m->logits, &m->dl16, &m->sc_l, &m->dns, &m->dxs};
  for (DevBuf* b : bufs) mix(b->p);
  for (int i = 0; i < 7; ++i) mix(m->hs_keep[i].p);
  for (int i = 0; i < 4; ++i) mix(m->ctx->scratch[i]);
  mix((const void*)(uintptr_t)m->n_params);
  mix((const void*)(uintptr_t)(m->store_acts ? 1 : 0));
  mix(m->staged_gap ? m->gap.p : nullptr);
  for (auto& b : m->blocks)
    for (int i = 0; i < 7; ++i) mix((const void*)(uintptr_t)(b.lin[i]->lora_active() ? b.lin[i]->lora.rank : 0));
  return h;
}

// The staged step replays as ONE CUDA graph once the same shape has run eagerly (the eager run
// sizes every buffer and encodes every TMA descriptor; capture then records ~3000 launches
// with no host work between them).
static rt_status run_staged(rt_model* m, bool backward, float* logits_out_host) {
  rt_ctx* c = m->ctx;
  RT_CUDA(c, cudaSetDevice(c->device));
  RT_TRY(refresh_adapter_copies(m));  // outside the graph: only after a parameter update
  if (m->use_graphs < 0) {
    const char* e = getenv("RT_B200_NO_GRAPH");
    m->use_graphs = (e && e[0] == '1') ? 0 : 1;
  }
  if (!m->use_graphs || c->profiling || logits_out_host || m->want_argmax || c->stream == nullptr)
    return run_staged_body(m, backward, logits_out_host);
  RT_CUDA(c, cudaSetDevice(c->device));
  const int M = m->staged_tokens, nt = m->staged_targets, bw = backward ? 1 : 0;
  const uint64_t sig = buffer_signature(m);
  for (auto& ge : m->graphs)
    if (ge.M == M && ge.n_targets == nt && ge.backward == bw && ge.sig == sig) {
      RT_CUDA(c, cudaGraphLaunch(ge.exec, c->stream));
      RT_COUNT_LAUNCH(ge.kernels);
      return RT_OK;
    }
  if (m->eager_M == M && m->eager_targets == nt && m->eager_backward == bw && m->eager_sig == sig) {
    const unsigned long long before = g_launch_count.load();
    cudaGraph_t graph = nullptr;
    RT_CUDA(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    rt_status st = run_staged_body(m, backward, nullptr);
    cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
    const unsigned long long kernels = g_launch_count.load() - before;
    g_launch_count.fetch_sub(kernels);  // nothing ran yet; the replay below counts them
    cudaGraphExec_t exec = nullptr;
    if (st == RT_OK && e == cudaSuccess && graph && cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess) {
      cudaGraphDestroy(graph);
      if (m->graphs.size() >= 8) {
        cudaGraphExecDestroy(m->graphs.front().exec);
        m->graphs.erase(m->graphs.begin());
      }
      m->graphs.push_back({M, nt, bw, sig, exec, kernels});
      RT_CUDA(c, cudaGraphLaunch(exec, c->stream));
      RT_COUNT_LAUNCH(kernels);
      return RT_OK;
    }
    if (graph) cudaGraphDestroy(graph);
    cudaGetLastError();
    m->use_graphs = 0;  // capture is not possible here: stay eager
    return run_staged_body(m, backward, nullptr);
  }
  rt_status st = run_staged_body(m, backward, nullptr);
  m->eager_M = M;
  m->eager_targets = nt;
  m->eager_backward = bw;
  m->eager_sig = buffer_signature(m);
  return st;
}

rt_status rt_model_stage_batch(rt_model* m, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq,
                               const int32_t* tpos, const int32_t* ttok, const float* weights, int32_t n_targets) {
  if (!m) return RT_ERR_BAD_ARG;
  int M = 0;
  m->staged_tokens = 0;
  RT_TRY(upload_batch(m, tokens, seq_offsets, n_seq, tpos, ttok, weights, n_targets, weights != nullptr, &M));
  RT_CUDA(m->ctx, cudaStreamSynchronize(m->ctx->stream));
  m->staged_tokens = M;
  m->staged_targets = n_targets;
  m->staged_has_weights = weights != nullptr;
  return RT_OK;
}

rt_status rt_model_run_staged(rt_model* m, int backward) {
  if (!m) return RT_ERR_BAD_ARG;
  if (backward && !m->staged_has_weights) return m->ctx->fail(RT_ERR_BAD_ARG, "the staged batch has no weights");
  return run_staged(m, backward != 0, nullptr);
}

rt_status rt_model_read_results(rt_model* m, float* logp_out, int32_t n_targets, int32_t* hits_out) {
  if (!m) return RT_ERR_BAD_ARG;
  rt_ctx* c = m->ctx;
  if (n_targets > m->staged_targets) return c->fail(RT_ERR_BAD_ARG, "more results requested than targets staged");
  RT_CUDA(c, cudaSetDevice(c->device));
  cudaStream_t st = c->stream;
  if (n_targets > 0 && logp_out) RT_CUDA(c, cudaMemcpyAsync(logp_out, m->logp.p, (size_t)n_targets * 4, cudaMemcpyDeviceToHost, st));
  int hits = 0;
  RT_CUDA(c, cudaMemcpyAsync(&hits, m->hits.p, 4, cudaMemcpyDeviceToHost, st));
  rt_status s = c->check_device_status("rt_model_read_results");
  if (hits_out) *hits_out = hits;
  return s;
}

rt_status rt_model_forward_backward(rt_model* m, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq,
                                    const int32_t* tpos, const int32_t* ttok, const float* weights, int32_t n_targets,
                                    float* logp_out, int32_t* hits_out) {
  if (!m) return RT_ERR_BAD_ARG;
  rt_ctx* c = m->ctx;
  if (n_targets > 0 && !weights) return c->fail(RT_ERR_BAD_ARG, "weights missing");  // model.rs:652 asserts equal lengths
  int M = 0;
  m->staged_tokens = 0;
  RT_TRY(upload_batch(m, tokens, seq_offsets, n_seq, tpos, ttok, weights, n_targets, true, &M));
  m->staged_tokens = M;
  m->staged_targets = n_targets;
  m->staged_has_weights = true;
  RT_TRY(run_staged(m, true, nullptr));
  return rt_model_read_results(m, logp_out, n_targets, hits_out);
}

rt_status rt_model_score(rt_model* m, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq,
                         const int32_t* tpos, const int32_t* ttok, int32_t n_targets, float* logp_out,
                         int32_t* hits_out, float* logits_out) {
  if (!m) return RT_ERR_BAD_ARG;
  int M = 0;
  m->staged_tokens = 0;
  RT_TRY(upload_batch(m, tokens, seq_offsets, n_seq, tpos, ttok, nullptr, n_targets, false, &M));
  m->staged_tokens = M;
  m->staged_targets = n_targets;
  m->staged_has_weights = false;
  RT_TRY(run_staged(m, false, logits_out));
  return rt_model_read_results(m, logp_out, n_targets, hits_out);
}

rt_status rt_model_forward_backward_layout(rt_model* m, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq,
                                           const int32_t* positions, const int32_t* segments, const int32_t* tpos,
                                           const int32_t* ttok, const float* weights, int32_t n_targets, float* logp_out,
                                           int32_t* hits_out) {
  if (!m) return RT_ERR_BAD_ARG;
  rt_ctx* c = m->ctx;
  if (n_targets > 0 && !weights) return c->fail(RT_ERR_BAD_ARG, "weights missing");
  int M = 0;
  m->staged_tokens = 0;
  RT_TRY(upload_batch(m, tokens, seq_offsets, n_seq, tpos, ttok, weights, n_targets, true, &M, positions, segments));
  m->staged_tokens = M;
  m->staged_targets = n_targets;
  m->staged_has_weights = true;
  RT_TRY(run_staged(m, true, nullptr));
  return rt_model_read_results(m, logp_out, n_targets, hits_out);
}

rt_status rt_model_score_layout(rt_model* m, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq,
                                const int32_t* positions, const int32_t* segments, const int32_t* tpos, const int32_t* ttok,
                                int32_t n_targets, float* logp_out, int32_t* hits_out) {
  if (!m) return RT_ERR_BAD_ARG;
  int M = 0;
  m->staged_tokens = 0;
  RT_TRY(upload_batch(m, tokens, seq_offsets, n_seq, tpos, ttok, nullptr, n_targets, false, &M, positions, segments));
  m->staged_tokens = M;
  m->staged_targets = n_targets;
  m->staged_has_weights = false;
  RT_TRY(run_staged(m, false, nullptr));
  return rt_model_read_results(m, logp_out, n_targets, hits_out);
}

// The greedy token at each target position of a forward-only pass (src/eval.rs:156-221:
// greedy_prefix asks logits_at for whole rows and takes their argmax on the host; here only the
// argmax leaves the device).
rt_status rt_model_argmax_layout(rt_model* m, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq,
                                 const int32_t* positions, const int32_t* segments, const int32_t* tpos, int32_t n_targets,
                                 int32_t* argmax_out) {
  if (!m || !argmax_out) return RT_ERR_BAD_ARG;
  rt_ctx* c = m->ctx;
  if (n_targets <= 0) return RT_OK;
  std::vector<int32_t> ttok((size_t)n_targets, 0);  // the pass scores against a target token; any valid id does
  int M = 0;
  m->staged_tokens = 0;
  RT_TRY(upload_batch(m, tokens, seq_offsets, n_seq, tpos, ttok.data(), nullptr, n_targets, false, &M, positions, segments));
  if (!m->argmax.reserve((size_t)n_targets * 4)) return c->fail(RT_ERR_CUDA, "out of device memory (argmax)");
  m->staged_tokens = M;
  m->staged_targets = n_targets;
  m->staged_has_weights = false;
  m->want_argmax = true;
  rt_status st = run_staged(m, false, nullptr);
  m->want_argmax = false;
  if (st) return st;
  RT_CUDA(c, cudaMemcpyAsync(argmax_out, m->argmax.p, (size_t)n_targets * 4, cudaMemcpyDeviceToHost, c->stream));
  return c->check_device_status("rt_model_argmax_layout");
}

rt_status rt_optim_step(rt_model* m, float lr, float max_norm, float beta1, float beta2, float eps, float wd,
                        float* norm_out) {
  if (!m) return RT_ERR_BAD_ARG;
  rt_ctx* c = m->ctx;
  if (m->n_params == 0) return c->fail(RT_ERR_BAD_ARG, "no adapters attached");
  RT_CUDA(c, cudaSetDevice(c->device));
  cudaStream_t st = c->stream;
  double* part = m->opt_scalars.as<double>();
  double* sum = part + 1024;
  float* normd = (float*)(sum + 1);
  launch_sumsq(m->G.as<float>(), m->n_params, part, sum, st);
  m->opt_t += 1;
  const float bc1 = 1.0f - powf(beta1, (float)m->opt_t), bc2 = 1.0f - powf(beta2, (float)m->opt_t);
  launch_adamw(m->P.as<float>(), m->G.as<float>(), m->Mo.as<float>(), m->Vo.as<float>(), m->n_params, sum, max_norm, lr,
               beta1, beta2, eps, wd, bc1, bc2, normd, st);
  for (rt_linear* l : m->lora_order) { l->lora.stale = true; ++l->lora.version; }
  float nrm = 0.f;
  RT_CUDA(c, cudaMemcpyAsync(&nrm, normd, 4, cudaMemcpyDeviceToHost, st));
  rt_status s = c->check_device_status("rt_optim_step");
  if (norm_out) *norm_out = nrm;
  return s;
}

rt_status rt_optim_state_read(rt_model* m, uint64_t* t_out, float* mh, float* vh) {
  if (!m) return RT_ERR_BAD_ARG;
  rt_ctx* c = m->ctx;
  RT_CUDA(c, cudaSetDevice(c->device));
  if (t_out) *t_out = m->opt_t;
  if (mh && m->n_params) RT_CUDA(c, cudaMemcpyAsync(mh, m->Mo.p, m->n_params * 4, cudaMemcpyDeviceToHost, c->stream));
  if (vh && m->n_params) RT_CUDA(c, cudaMemcpyAsync(vh, m->Vo.p, m->n_params * 4, cudaMemcpyDeviceToHost, c->stream));
  return c->check_device_status("rt_optim_state_read");
}

rt_status rt_optim_state_write(rt_model* m, uint64_t t, const float* mh, const float* vh) {
  if (!m) return RT_ERR_BAD_ARG;
  rt_ctx* c = m->ctx;
  RT_CUDA(c, cudaSetDevice(c->device));
  m->opt_t = t;
  if (mh && m->n_params) RT_CUDA(c, cudaMemcpyAsync(m->Mo.p, mh, m->n_params * 4, cudaMemcpyHostToDevice, c->stream));
  if (vh && m->n_params) RT_CUDA(c, cudaMemcpyAsync(m->Vo.p, vh, m->n_params * 4, cudaMemcpyHostToDevice, c->stream));
  RT_CUDA(c, cudaStreamSynchronize(c->stream));
  return RT_OK;
}

}  // extern "C"
