/*
 * rt_b200.h -- C ABI of the B200-native frozen-quantised-linear LoRA training path.
 *
 * The entry points replace, one for one, the methods a Rust host binds for this path in
 * olapwriter-prog/Rust_Trainer.  Citations are file:line inside that project.
 *
 * Conventions
 *   - every function returns an rt_status (0 = ok); rt_last_error() gives the message;
 *     nothing aborts and nothing throws across the ABI (the reference panics on shape errors:
 *     src/frozen.rs:126,143-144, src/linear.rs:75,99; here they are RT_ERR_BAD_SHAPE)
 *   - all matrices are row-major; activations are [tokens x dim]; a weight is [out x in]
 *   - handles are opaque, created and destroyed explicitly; packed weight bytes are copied to
 *     the device at create time (the caller may unmap its file afterwards); every output
 *     buffer is caller-allocated
 *   - one rt_ctx per GPU; calls on one ctx are serialised by the caller
 *   - pointers named *_host are host memory, pointers named *_dev are device memory of the
 *     ctx's GPU
 */
#ifndef RT_B200_H
#define RT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t rt_status;
enum {
  RT_OK = 0,
  RT_ERR_BAD_SHAPE = 1,
  RT_ERR_UNSUPPORTED_TYPE = 2,
  RT_ERR_CUDA = 3,
  RT_ERR_NCCL = 4,
  RT_ERR_DEVICE_WAIT_TIMEOUT = 5,
  RT_ERR_BAD_INDEX = 6,
  RT_ERR_BAD_ARG = 7,
  RT_ERR_TOO_LARGE = 8,
  RT_ERR_NONFINITE = 9 /* a 16-bit activation overflowed: silu(gate) * up beyond 65504 (the reference holds it in f32) */
};

/* ggml tensor types accepted for frozen weights (numeric values are GGUF's). */
enum {
  RT_GGML_F32 = 0, /* FrozenWeight::F32 (src/frozen.rs:33-38); also what norms, biases and rope_freqs are */
  RT_GGML_F16 = 1,
  RT_GGML_Q4_0 = 2,
  RT_GGML_Q8_0 = 8,
  RT_GGML_Q4_K = 12,
  RT_GGML_Q6_K = 14,
  RT_GGML_BF16 = 30
};

/* Element types of device-resident activations. */
enum { RT_DT_F32 = 0, RT_DT_BF16 = 1, RT_DT_F16 = 2 };

typedef struct rt_ctx rt_ctx;
typedef struct rt_frozen rt_frozen;
typedef struct rt_linear rt_linear;
typedef struct rt_model rt_model;

/* ------------------------------------------------------------------ context */
/* One per GPU: device id, stream, workspace.  Replaces the engine thread pool that
 * src/rie.rs:182 builds with make_pool(). */
rt_status rt_ctx_create(int device, rt_ctx** out);
void rt_ctx_destroy(rt_ctx* ctx);
const char* rt_last_error(const rt_ctx* ctx);
rt_status rt_ctx_synchronize(rt_ctx* ctx);
/* The CUDA stream (cudaStream_t) every call on this ctx is issued on. */
void* rt_ctx_stream(rt_ctx* ctx);
/* Issue all later calls on `cuda_stream` (a cudaStream_t of the same device) instead of the
 * stream the ctx created, so a host that owns its streams can order and time the work. */
rt_status rt_ctx_set_stream(rt_ctx* ctx, void* cuda_stream);
/* Measurement aids.  launch_count: kernels this library has launched on the ctx so far.
 * With profiling on, every frozen-matmul launch is bracketed by CUDA events on the ctx stream;
 * profile_read waits for them and returns, for the launches since the last read, their number,
 * their summed device time and their summed algorithmic work 2*tokens*out*in (flops) and
 * packed-weight + activation + result bytes. */
uint64_t rt_ctx_launch_count(const rt_ctx* ctx);
/* Failure detection without a fault: launches one warp that waits, with the same bounded wait the
 * matmul kernel uses, on a barrier nothing arrives on.  After `limit_cycles` SM cycles (at most
 * 2e9, about a second) the wait gives up and the kernel returns; the call then reports
 * RT_ERR_DEVICE_WAIT_TIMEOUT (site 999) and the context stays usable.  No counterpart in the
 * reference (its CPU path has no device waits). */
rt_status rt_ctx_selftest_wait_timeout(rt_ctx* ctx, uint64_t limit_cycles);
rt_status rt_ctx_set_profiling(rt_ctx* ctx, int enabled);
rt_status rt_ctx_profile_read(rt_ctx* ctx, uint64_t* n_launches, double* total_ms, double* total_flops,
                              double* total_bytes);
/* Bytes of ggml block storage for a [rows x cols] tensor of `ggml_type`; 0 if unsupported. */
size_t rt_ggml_nbytes(int ggml_type, size_t rows, size_t cols);

/* ------------------------------------------------------------------ level 1: trait FrozenMatmul
 * src/frozen.rs:14-25, implemented for GGUF weights by RieFrozen (src/rie.rs:66-129). */

/* RieFrozen::new (src/rie.rs:57-61): `packed_host` is the tensor exactly as stored in the
 * GGUF file, rows of ggml blocks. */
rt_status rt_frozen_create(rt_ctx* ctx, int ggml_type, size_t rows, size_t cols, const void* packed_host,
                           size_t nbytes, rt_frozen** out);
/* FrozenWeight::Q8_0 (src/frozen.rs:39-73), the trainer's own 8-bit storage: one f32 scale per
 * 32 columns (scales_host, rows*cols/32 values, row-major) and signed bytes (qs_host, rows*cols).
 * Not ggml's Q8_0 block, whose scale is f16.  row() returns scale*q exactly as the reference's. */
rt_status rt_frozen_create_q8_0(rt_ctx* ctx, size_t rows, size_t cols, const float* scales_host,
                                const int8_t* qs_host, rt_frozen** out);
void rt_frozen_destroy(rt_frozen* w);
/* FrozenMatmul::out_dim / in_dim / nbytes (src/frozen.rs:15-16,24). nbytes is the ggml size. */
size_t rt_frozen_out_dim(const rt_frozen* w);
size_t rt_frozen_in_dim(const rt_frozen* w);
size_t rt_frozen_nbytes(const rt_frozen* w);
/* FrozenMatmul::forward (src/frozen.rs:18, src/rie.rs:74-82): y[t x out] = x[t x in] . W^T */
rt_status rt_frozen_forward(rt_frozen* w, const float* x_host, size_t t, float* y_host);
/* FrozenMatmul::backward_input (src/frozen.rs:20, src/rie.rs:84-120): dx[t x in] += dy[t x out] . W */
rt_status rt_frozen_backward_input(rt_frozen* w, const float* dy_host, size_t t, float* dx_host);
/* FrozenMatmul::row (src/frozen.rs:22, src/rie.rs:122-124): dequantise row r into out_host[in]. */
rt_status rt_frozen_row(rt_frozen* w, size_t r, float* out_host);


/* Device-resident forms of forward / backward_input.  Activations stay in HBM as 16-bit
 * [t x dim] (`in_dtype` RT_DT_F16 or RT_DT_BF16; the tensor-core instruction needs both operands
 * in ONE 16-bit type, so the packed weight is unpacked to that type on the fly: f16 keeps 11
 * significant bits and suits the forward, bf16 keeps f32's range and suits gradients).  The
 * result is written as `out_dtype` (f32, bf16 or f16); `accumulate` (f32 only) adds into the
 * output, which is what backward_input's `+=` and the residual adds of
 * src/model.rs:178,181 need.  Asynchronous on the ctx stream; a kernel-side failure is
 * reported by the next rt_ctx_synchronize. */
rt_status rt_frozen_forward_dev(rt_frozen* w, const void* x_dev, int in_dtype, size_t t, void* y_dev,
                                int out_dtype, int accumulate);
rt_status rt_frozen_backward_input_dev(rt_frozen* w, const void* dy_dev, int in_dtype, size_t t, void* dx_dev,
                                       int out_dtype, int accumulate);
/* The same operation as rt_frozen_backward_input_dev for callers that must not allocate device
 * memory while they run: a host inside a memory-budgeted serving or training process that has
 * handed every byte of HBM to its own pool, a real-time loop that cannot take the driver's
 * allocation lock, or code running where cudaMalloc is simply not permitted.  It has no
 * counterpart in the reference (the reference never leaves the CPU).  When the contraction is
 * accumulated in pieces (more than 16384 weight rows: one piece per 8192), the partial sums go
 * to a fixed 8 MiB array that is part of the library's
 * device image (every GPU that loads the library holds it until the process exits) instead of
 * grow-on-demand scratch; the call makes no cudaMalloc / cudaFree and keeps no descriptor
 * cache.  Limits and rules:
 *   - a call whose partial sums need more than 2 Mi floats (pieces x t x in_dim) is refused with
 *     RT_ERR_TOO_LARGE; use fewer rows per call;
 *   - the FIRST call on a device looks up the array's device address; make that call before
 *     any stream capture begins;
 *   - all calls share the one array and it keeps the previous call's contents (nothing in it
 *     needs to start at zero: every element read was written by the same call); two calls that
 *     overlap on the GPU (different streams) race on it, so keep them on one stream. */
rt_status rt_frozen_backward_input_dev_noalloc(rt_frozen* w, const void* dy_dev, int in_dtype, size_t t,
                                               void* dx_dev, int out_dtype, int accumulate);

/* ------------------------------------------------------------------ op level: src/ops.rs, src/attention.rs
 * The device kernels of the per-row operations and of the attention core, one operation per call
 * with HOST buffers (copy in, launch, copy out, synchronise).  The training step never calls
 * these: it chains the same kernels on the device.  They are for checking one operation against
 * the CPU path.  Activations that feed a matmul leave the kernels as f16 (gradients: f16 rows
 * times one f32 factor per row), which is what the f32 results returned here were rounded to. */

/* rmsnorm (src/ops.rs:8-35): y[rows x d] = x * inv_rms(x) * w. */
rt_status rt_op_rmsnorm(rt_ctx* ctx, const float* x_host, const float* w_host, size_t rows, size_t d, float eps,
                        float* y_host);
/* rmsnorm_backward (src/ops.rs:39-56): dx from dy; the weight has no gradient (frozen). */
rt_status rt_op_rmsnorm_backward(rt_ctx* ctx, const float* x_host, const float* w_host, const float* dy_host, size_t rows,
                                 size_t d, float eps, float* dx_host);
/* What Attention::forward does between the projections and the scores (src/attention.rs:170-185):
 * per-head RMSNorm of q and k with the fused-scale rounding order (weights NULL: none), RoPE at
 * `positions` (Rope::with / at_positions / apply, src/ops.rs:99-184; NEOX pairs (i, i+rot/2) or
 * interleaved pairs; `factors` = rope_freqs divisors or NULL), then rounding to f16, which is the
 * reference's f16 K/V view for k and v.  q [M x nh x hd], k, v [M x nkv x hd]. */
rt_status rt_op_qk_norm_rope(rt_ctx* ctx, const float* q_raw_host, const float* k_raw_host, const float* v_raw_host,
                             const int32_t* positions, size_t M, int nh, int nkv, int hd, int rot, int neox, float theta,
                             float freq_scale, const float* factors, int n_factors, const float* q_norm_w,
                             const float* k_norm_w, float eps, float* q_host, float* k_host, float* v_host);
/* Its backward (src/attention.rs:330-358): inverse rotation, then the norm's backward. */
rt_status rt_op_qk_norm_rope_backward(rt_ctx* ctx, const float* dq_host, const float* dk_host, const float* dv_host,
                                      const float* q_raw_host, const float* k_raw_host, const int32_t* positions,
                                      size_t M, int nh, int nkv, int hd, int rot, int neox, float theta, float freq_scale,
                                      const float* factors, int n_factors, const float* q_norm_w, const float* k_norm_w,
                                      float eps, float* dq_raw_host, float* dk_raw_host, float* dv_host_out);
/* The attention core (src/attention.rs:187-230): causal softmax(q.k^T / sqrt(hd)).v per head with
 * grouped KV heads, over a concatenation of sequences (row i sees keys seq_start[i] .. i).
 * lse_host (optional) is [nh x M]. */
rt_status rt_op_attention(rt_ctx* ctx, const float* q_host, const float* k_host, const float* v_host,
                          const int32_t* seq_start, size_t M, int nh, int nkv, int hd, float* o_host, float* lse_host);
/* Its backward (src/attention.rs:246-329): dq, dk, dv from d(o), the KV gradients summed over the
 * query heads of a group. */
rt_status rt_op_attention_backward(rt_ctx* ctx, const float* q_host, const float* k_host, const float* v_host,
                                   const float* do_host, const int32_t* seq_start, size_t M, int nh, int nkv, int hd,
                                   float* dq_host, float* dk_host, float* dv_host);
/* Mlp's activation (src/model.rs:113-134, src/tensor.rs:122-143): h = silu(gate) * up and its backward. */
rt_status rt_op_swiglu(rt_ctx* ctx, const float* gate_host, const float* up_host, size_t rows, size_t ff, float* h_host);
rt_status rt_op_swiglu_backward(rt_ctx* ctx, const float* gate_host, const float* up_host, const float* dh_host, size_t rows,
                                size_t ff, float* dgate_host, float* dup_host);
/* The head's per-row arithmetic (src/model.rs:579-596 over softmax_row, src/ops.rs:238-247): log-
 * probability of the target with an f64 normaliser, hit count (no logit above the target's),
 * optionally the argmax (last index on ties) and dlogits = w * (p - onehot). */
rt_status rt_op_cross_entropy(rt_ctx* ctx, const float* logits_host, size_t rows, size_t vocab, const int32_t* target,
                              const float* weight, float* logp_host, int32_t* hits_out, int32_t* argmax_host,
                              float* dlogits_host);

/* ------------------------------------------------------------------ level 2: struct Linear / struct Lora
 * src/linear.rs:9-122.  y = W.x + b + (alpha/r).B.A.x forward; dx = W^T.dy + (LoRA term) and
 * the adapter gradients dA, dB backward.  Device-resident: this is the performance boundary,
 * a Rust `Linear` holding device buffers calls these instead of crossing PCIe per layer. */

/* Linear::new (src/linear.rs:48-53).  `bias_host` has out_dim floats or is NULL.  The linear
 * borrows `w` (several linears may share one frozen weight, as embed/lm_head do when tied,
 * src/rie.rs:189); destroy the linear before the weight. */
rt_status rt_linear_create(rt_ctx* ctx, rt_frozen* w, const float* bias_host, const char* name, rt_linear** out);
void rt_linear_destroy(rt_linear* lin);
/* Linear::attach_lora (src/linear.rs:60-62) with explicit initial values: a_host is
 * [rank x in], b_host is [out x rank] (row-major f32).  rank <= 64.  Gradients start at zero. */
rt_status rt_linear_attach_lora(rt_linear* lin, int rank, float alpha, const float* a_host, const float* b_host);
/* Linear::lora_enabled (src/linear.rs:44-45,64-70): 0 bypasses the adapter. */
rt_status rt_linear_set_lora_enabled(rt_linear* lin, int enabled);
/* Linear::forward (src/linear.rs:73-93), device form: x_f16_dev is [t x in] f16; y_dev is
 * [t x out] of y_dtype (RT_DT_*); accumulate (f32 only) adds into y. */
rt_status rt_linear_forward_dev(rt_linear* lin, const void* x_f16_dev, size_t t, void* y_dev, int y_dtype,
                                int accumulate);
/* Linear::backward (src/linear.rs:97-121), device form.  dy is passed as f16 rows divided by a
 * per-row positive scale (dy[m,:] = dy_f16[m,:] * dy_row_scale[m]; NULL scale = 1), which keeps
 * 11 significant bits for gradients of any magnitude.  Writes (or, with accumulate, adds to)
 * dx_f32_dev [t x in] and adds dA, dB into the adapter's gradient buffers. */
rt_status rt_linear_backward_dev(rt_linear* lin, const void* x_f16_dev, const void* dy_f16_dev,
                                 const float* dy_row_scale_dev, size_t t, float* dx_f32_dev, int accumulate);
/* Host-buffer forms with the reference's exact signatures: Linear::forward(x, t) -> y and
 * Linear::backward(x, dy, t) -> dx (fresh; accumulates ga/gb). */
rt_status rt_linear_forward(rt_linear* lin, const float* x_host, size_t t, float* y_host);
rt_status rt_linear_backward(rt_linear* lin, const float* x_host, const float* dy_host, size_t t, float* dx_host);
/* Read / write the adapter (struct Lora fields a, b, ga, gb; any pointer may be NULL). */
rt_status rt_lora_read(rt_linear* lin, float* a_host, float* b_host, float* ga_host, float* gb_host);
rt_status rt_lora_write(rt_linear* lin, const float* a_host, const float* b_host);
/* Lora::zero_grad (src/linear.rs:29-32). */
rt_status rt_lora_zero_grad(rt_linear* lin);

/* ------------------------------------------------------------------ level 3: struct Model
 * src/model.rs:292-687 as built by load_gguf_from (src/rie.rs:164-260): dense llama / qwen2 /
 * qwen3 decoders, pre-norm blocks, GQA attention with optional QK-norm and q/k/v bias, SwiGLU,
 * f16-rounded K/V (kv_f16 = true, src/rie.rs:200), activation recomputation per block
 * (checkpointing = true, src/rie.rs:254). */
typedef struct rt_model_config {
  int32_t vocab, hidden, ff, n_layers;
  int32_t n_heads, n_kv_heads, head_dim, rot_dim;
  float rope_theta, rope_freq_scale, rms_eps;
  int32_t rope_neox;       /* 1: pairs (i, i+rot/2); 0: pairs (2i, 2i+1)            src/ops.rs:177 */
  int32_t qk_norm;         /* 1: per-head RMSNorm on q and k                        src/attention.rs:170-177 */
  int32_t tie_embeddings;  /* 1: lm_head shares token_embd                          src/rie.rs:186-189 */
  int32_t head_rows;       /* rows of logits held at once (the reference's logits_chunk is 64,
                              src/rie.rs:255; 0 picks 1024); results do not depend on it */
} rt_model_config;

rt_status rt_model_create(rt_ctx* ctx, const rt_model_config* cfg, rt_model** out);
void rt_model_destroy(rt_model* m);
/* One call per GGUF tensor, by its GGUF name: token_embd.weight, output.weight (untied only),
 * output_norm.weight, rope_freqs.weight (optional), blk.N.{attn_norm,ffn_norm,attn_q_norm,
 * attn_k_norm}.weight, blk.N.{attn_q,attn_k,attn_v,attn_output,ffn_gate,ffn_up,ffn_down}.weight
 * and blk.N.attn_{q,k,v}.bias.  ggml_type 0 means f32 (norms, biases, rope_freqs). */
rt_status rt_model_set_tensor(rt_model* m, const char* name, int ggml_type, size_t rows, size_t cols,
                              const void* data_host, size_t nbytes);
/* Checks that every tensor the configuration needs has arrived (load_gguf_from's refusals). */
rt_status rt_model_finalize(rt_model* m);
/* Model::attach_lora (src/model.rs:406-419): adapters on the listed modules (comma-separated
 * GGUF or HF short names, NULL = all seven projections), A ~ U(-1/sqrt(in), 1/sqrt(in)) from the
 * trainer's SplitMix64 stream seeded with `seed`, B = 0.  Returns the number of trainable
 * parameters through n_params_out. */
rt_status rt_model_attach_lora(rt_model* m, int rank, float alpha, const char* targets_csv, uint64_t seed,
                               size_t* n_params_out);
/* Model::lora_linears (src/model.rs:431-433), in parameter order (optim.rs:32-34). */
size_t rt_model_num_lora(const rt_model* m);
rt_linear* rt_model_lora_linear(rt_model* m, size_t index);
const char* rt_linear_name(const rt_linear* lin);
size_t rt_linear_in_dim(const rt_linear* lin);
size_t rt_linear_out_dim(const rt_linear* lin);
int rt_linear_lora_rank(const rt_linear* lin);
/* Model::set_lora_enabled (src/model.rs:421-427), Model::zero_grad (src/model.rs:435-439). */
rt_status rt_model_set_lora_enabled(rt_model* m, int enabled);
rt_status rt_model_zero_grad(rt_model* m);
/* Model::forward_backward (src/model.rs:613-687) over a batch of independent sequences laid
 * end to end: tokens[seq_offsets[s] .. seq_offsets[s+1]) is sequence s.  Target i is scored
 * from the hidden state at global position target_pos[i] against token target_tok[i] with
 * weight weights[i] (the trainer passes 1/batch_tokens, src/train.rs:263,275).  Adds into every
 * adapter's gradients; writes log-probabilities per target and the count of argmax hits. */
rt_status rt_model_forward_backward(rt_model* m, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq,
                                    const int32_t* target_pos, const int32_t* target_tok, const float* weights,
                                    int32_t n_targets, float* logp_out, int32_t* hits_out);
/* Model::score / logprobs / logits_at (src/model.rs:505-557): forward only.  logits_out is
 * NULL or [n_targets x vocab]. */
rt_status rt_model_score(rt_model* m, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq,
                         const int32_t* target_pos, const int32_t* target_tok, int32_t n_targets, float* logp_out,
                         int32_t* hits_out, float* logits_out);
/* Model::forward_backward_packed / the packed scoring of src/eval.rs:176-186: every sequence of
 * the batch is a Packed group (src/model.rs:234-290): a shared prompt (segments[i] = 0) followed
 * by the examples' own tokens (segments[i] = k + 1 for example k, in runs), positions[i] = the
 * token's position within its own example (RoPE).  A token attends to the prompt and to its own
 * example's earlier tokens only (Rope::allowed, src/ops.rs:156-164).  The result equals running
 * the examples separately, with the prompt computed once.  Target positions index the packed
 * token array (Packed::index). */
rt_status rt_model_forward_backward_layout(rt_model* m, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq,
                                           const int32_t* positions, const int32_t* segments,
                                           const int32_t* target_pos, const int32_t* target_tok, const float* weights,
                                           int32_t n_targets, float* logp_out, int32_t* hits_out);
rt_status rt_model_score_layout(rt_model* m, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq,
                                const int32_t* positions, const int32_t* segments, const int32_t* target_pos,
                                const int32_t* target_tok, int32_t n_targets, float* logp_out, int32_t* hits_out);
/* greedy_prefix / greedy_prefix_batch (src/eval.rs:156-221): the greedy token, i.e. the argmax of
 * the logits (the last index on ties, as the reference's max_by gives), at each target position
 * of one forward-only pass.  positions / segments are NULL for plain sequences or describe
 * Packed groups as in rt_model_score_layout.  The caller counts, per example, how many leading
 * answer positions reproduce the example's tokens. */
rt_status rt_model_argmax_layout(rt_model* m, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq,
                                 const int32_t* positions, const int32_t* segments, const int32_t* target_pos,
                                 int32_t n_targets, int32_t* argmax_out);
/* The same step split for hosts that keep the batch on the device: stage copies tokens,
 * targets and weights to HBM once; run_staged does the forward + backward (backward != 0) or
 * the forward alone on the staged batch without touching host memory; read_results copies the
 * per-target log-probabilities and the hit count back. */
rt_status rt_model_stage_batch(rt_model* m, const int32_t* tokens, const int32_t* seq_offsets, int32_t n_seq,
                               const int32_t* target_pos, const int32_t* target_tok, const float* weights,
                               int32_t n_targets);
rt_status rt_model_run_staged(rt_model* m, int backward);
rt_status rt_model_read_results(rt_model* m, float* logp_out, int32_t n_targets, int32_t* hits_out);
/* Model.checkpointing (src/model.rs:299, 663-684).  mode 1: keep only each block's input and
 * run the block's forward again before its backward (the reference's default); mode 0: keep
 * every block's caches from the forward; mode -1 (the default here): keep the caches when
 * they fit in 60 % of the free device memory, else recompute.  The same results either way.
 * rt_model_checkpointing reports the mode the last staged batch used (0 or 1). */
rt_status rt_model_set_checkpointing(rt_model* m, int32_t mode);
int32_t rt_model_checkpointing(const rt_model* m);
/* The flat f32 gradient buffer on the device, [A_0 | B_0 | A_1 | B_1 ...] in parameter order:
 * what a data-parallel host all-reduces (sum) across ranks before rt_optim_step. */
rt_status rt_model_grad_buffer(rt_model* m, void** grads_dev_out, size_t* n_floats_out);
/* ------------------------------------------------------------------ data parallelism
 * No counterpart in the reference (one process, one device; src/train.rs:339-351 accumulates a
 * batch's examples one after the other).  Ranks hold replicas and take the batch's sequences in
 * turn; each weights its targets with the GLOBAL 1/batch_tokens (src/train.rs:330), so the SUM of
 * the ranks' gradient buffers is the batch gradient.  One NCCL communicator per ctx:
 *   rank 0: rt_comm_unique_id(id) and hands the 128 bytes to the other ranks by any means;
 *   every rank: rt_comm_init_rank(ctx, nranks, rank, id)   (collective: all ranks call it);
 *   per step: forward_backward ... ; rt_model_allreduce_grads(m); rt_optim_step(m, ...).
 * The all-reduce runs on the ctx stream, in place, asynchronously.  Without a communicator (a
 * world of one) it does nothing.  Failures are RT_ERR_NCCL with the library's message. */
#define RT_COMM_ID_BYTES 128
rt_status rt_comm_unique_id(uint8_t* id_out, size_t id_bytes);
rt_status rt_comm_init_rank(rt_ctx* ctx, int nranks, int rank, const uint8_t* id, size_t id_bytes);
rt_status rt_comm_destroy(rt_ctx* ctx);
int rt_comm_size(const rt_ctx* ctx);
int rt_comm_rank(const rt_ctx* ctx);
/* Sum over ranks, in place, of n floats in device memory (the loss, a token count, ...). */
rt_status rt_comm_allreduce_f32(rt_ctx* ctx, float* buf_dev, size_t n);
/* Sum over ranks of the flat LoRA-gradient buffer (rt_model_grad_buffer). */
rt_status rt_model_allreduce_grads(rt_model* m);

/* clip_grad_norm (src/optim.rs:73-90) followed by AdamW::step (src/optim.rs:48-69) on the
 * device; returns the pre-clip gradient norm. */
rt_status rt_optim_step(rt_model* m, float lr, float max_norm, float beta1, float beta2, float eps,
                        float weight_decay, float* grad_norm_out);
/* Optimiser state for checkpoints (src/train.rs:389-406): step count and flat m, v. */
rt_status rt_optim_state_read(rt_model* m, uint64_t* t_out, float* m_host, float* v_host);
rt_status rt_optim_state_write(rt_model* m, uint64_t t, const float* m_host, const float* v_host);

#ifdef __cplusplus
}
#endif
#endif /* RT_B200_H */
