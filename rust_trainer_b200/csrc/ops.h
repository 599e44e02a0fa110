// Launchers of the memory-bound device ops (ops.cu) and attention (attention.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>

struct rt_ctx;

namespace rt {

// hi = f16(w), lo = f16(w - hi): the two-term split of f32 frozen weights
void launch_split_f32_hi_lo(const float* w, size_t n, __half* hi, __half* lo, cudaStream_t st);
void launch_f32_to_16(const float* in, void* out, size_t n, bool to_f16, cudaStream_t st);
void launch_normalize_rows(const float* x, int rows, int d, __half* y16, float* scale, cudaStream_t st);
void launch_rmsnorm_fwd(const float* x, const float* w, int rows, int d, float eps, __half* y16, cudaStream_t st);
void launch_rmsnorm_bwd(const float* x, const float* w, const float* dn, const float* dres, int rows, int d, float eps,
                        float* out, __half* out16, float* scale, cudaStream_t st);
void launch_rope_table(const float* inv_freq, int half, int max_pos, float* cs, float* sn, cudaStream_t st);
// raw_pitch / out_pitch = 0: q, k, v are separate row-major matrices.  Otherwise they are column
// slices of ONE matrix with that row pitch (elements); with out_pitch the three f16 outputs also
// share one scale per token.  Pitches need the head shapes qk_rope_takes_pitches() accepts.
bool qk_rope_takes_pitches(int nh, int nkv, int hd, int rot, int neox);
void launch_qk_rope_fwd(const float* q_raw, const float* k_raw, const float* v_raw, size_t raw_pitch, const float* qw,
                        const float* kw, const int* pos, const float* cs, const float* sn, int M, int nh, int nkv, int hd,
                        int rot, int neox, float eps, __half* q16, __half* k16, __half* v16, cudaStream_t st);
void launch_qk_rope_bwd(const float* dq, const float* dk, const float* dv, const float* q_raw, const float* k_raw,
                        size_t raw_pitch, const float* qw, const float* kw, const int* pos, const float* cs, const float* sn,
                        int M, int nh, int nkv, int hd, int rot, int neox, float eps, __half* dq16, __half* dk16,
                        __half* dv16, size_t out_pitch, float* sq, float* sk, float* sv, cudaStream_t st);
// status (optional): set to RT_ERR_NONFINITE when a product leaves f16's range
void launch_swiglu_fwd(const __half* g, const __half* u, size_t in_pitch, int rows, int ff, __half* h, int* status,
                       cudaStream_t st);
// dh: f32 rows, or (dh_f16) f16 rows whose per-row factor in_scale[r] has not been applied yet
void launch_swiglu_bwd(const void* dh, int dh_f16, const float* in_scale, const __half* g, const __half* u, size_t in_pitch,
                       int rows, int ff, __half* dg16, __half* du16, size_t out_pitch, float* sg, float* su, cudaStream_t st);
void launch_gather_f32_rows(const float* x, const int* idx, int rows, int d, float* out, cudaStream_t st);
void launch_scatter_add_rows(const float* src, const int* idx, int rows, int d, float* dx, cudaStream_t st);
// argmax (optional): per row, the last index holding the row's maximum
void launch_ce_rows(const float* logits, int rows, int v, const int* target, const float* weight, float* logp, int* hits,
                    __half* d16, float* scale, int* argmax, int* status, cudaStream_t st);
void launch_lora_refresh_group(const float* a, const float* b, int r, int K, int N, float s, __half* a_s, __half* a_h,
                               __half* bp, __half* bt_s, size_t ldb, cudaStream_t st);
void launch_lora_refresh(const float* a, const float* b, int r, int K, int N, float s, __half* a_s, __half* a_h,
                         __half* bp, __half* bt_s, cudaStream_t st);
// One adapter's operand copies as a row of a device table: every stale adapter of a model is
// rebuilt by ONE launch.  pad64 = 1: bp is this adapter's own [N x 64] block, columns from r up
// are zeroed, bt_s has row pitch N; pad64 = 0: bp / bt_s point into stacked operands (bp row
// pitch 64, only columns < r are written; bt_s row pitch ldb).
struct LoraRefreshJob {
  const float *a, *b;
  __half *a_s, *a_h, *bp, *bt_s;
  unsigned long long ldb;
  int r, K, N, pad64;
  float s;
  unsigned first_block;  // of this job in the grid; jobs are in increasing order
};
inline unsigned lora_refresh_job_blocks(const LoraRefreshJob& j) {
  const size_t na = (size_t)j.r * j.K, nb = (size_t)j.N * (j.pad64 ? 64 : j.r);
  return (unsigned)(((na > nb ? na : nb) + 255) / 256);
}
void launch_lora_refresh_table(const LoraRefreshJob* jobs_dev, int n_jobs, unsigned total_blocks, cudaStream_t st);
size_t lora_grad_workspace_floats(int M, int C, int r);
void launch_lora_grad(const __half* P, const __half* Q, const float* pscale, const float* qscale, int M, int C, int r,
                      size_t so_i, size_t so_j, float* out, float* workspace, cudaStream_t st);
void launch_rowscale_max(const float* sc, int M, float* out, cudaStream_t st);
// out[m] = largest sc of m's sequence (power of two, 1 for an all-zero sequence), out[M + m] = sc[m] / out[m]
void launch_rowscale_seqmax(const float* sc, const int* seq_start, int M, float* out, cudaStream_t st);
void launch_scale_lowrank_rows(const __half* in, const float* sc, const float* smax, int M, __half* out, cudaStream_t st);
void launch_sumsq(const float* g, size_t n, double* part, double* out, cudaStream_t st);
void launch_adamw(float* p, float* g, float* m, float* v, size_t n, const double* sumsq, float max_norm, float lr,
                  float beta1, float beta2, float eps, float wd, float bc1, float bc2, float* norm_out,
                  cudaStream_t st);
void launch_global_normalize(const float* x, size_t n, float* amax_dev, __half* y16, cudaStream_t st);

// ---- lora_kernels.cu: skinny low-rank products (return 1 when the shape is not supported)
// ---- lowrank_tc.cu: out64[M x 64] (f16, zero from column r up) = X[M x K] . Wt[r x K]^T on tcgen05; 1 = shape not taken
int launch_lowrank_tc(rt_ctx* c, const __half* X, const __half* Wt, int M, int K, int r, __half* out64);
size_t tok_contract_workspace_floats(int M, int C, int r);
size_t lora_grads_workspace_floats(int M, int N, int K, int r);
// lora_grads_tc.cu: the product kernel on tcgen05 (partial sums per split of lora_grads_tc_tokens_per_split(M) tokens)
int lora_grads_tc_tokens_per_split(int M);
int launch_lora_grads_tc(rt_ctx* c, const __half* hs, const __half* dy16, int ld_dy, const __half* gs, const __half* x16,
                         const float* dscale, int M, int N, int K, int r, float* partB, float* partA);
int launch_lora_grads_group(rt_ctx* c, const __half* hs, const __half* dy16, const __half* gs, const __half* x16, const float* dscale,
                            int M, int NT, int K, int R, int n, float* const* gb, float* const* ga, const int* row_off,
                            const int* rows, const int* rank_off, const int* rank, float* workspace, cudaStream_t st);
int launch_lora_grads(rt_ctx* c, const __half* hs, const __half* dy16, int ld_dy, const __half* gs, const __half* x16, const float* dscale,
                      int M, int N, int K, int r, float* gb, float* ga, float* workspace, cudaStream_t st);
// pscale (optional): P's rows are multiplied by pscale[m] / alpha_dev[0] on the fly; alpha_dev[0] then scales the result
int launch_tok_contract(const __half* P, const __half* Q, const float* pscale, int M, int C, int r, size_t so_i, size_t so_j,
                        const float* alpha_dev, float* out, float* workspace, cudaStream_t st);

// ---- attention_tc.cu: causal GQA attention over a concatenation of independent sequences, on
// tcgen05 / TMEM / TMA (waits report through the ctx status word).
// q [M x nh x hd], k/v [M x nkv x hd] f16 (q unscaled; the kernels apply 1/sqrt(hd)).
// seq_start[m] = index of the first token of m's sequence; gap [M x 2] or null; lse is [nh x M].
// Backward: dO row i stands for do_scale[0] * dO16[i], or, with row_scale, for row_scale[i] *
// dO16[i] (then do_scale is the array [2 M] of launch_rowscale_seqmax: for each token a power of two >=
// the largest row_scale of its own sequence, then each row's weight against it); outputs are true-scale f32.
int launch_attn_bwd_tc(rt_ctx* c, const __half* q, const __half* k, const __half* v, const __half* o, const __half* dO16,
                       const float* do_scale, const float* row_scale, const float* lse, const int* seq_start, const int* gap,
                       int M, int nh, int nkv, int hd, float* delta, float* dq, float* dk, float* dv);
int launch_attn_fwd_tc(rt_ctx* c, const __half* q, const __half* k, const __half* v, const int* seq_start, const int* gap, int M,
                       int nh, int nkv, int hd, __half* o, float* lse);

}  // namespace rt
