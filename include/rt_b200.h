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
  RT_ERR_TOO_LARGE = 8
};

/* ggml tensor types accepted for frozen weights (numeric values are GGUF's). */
enum {
  RT_GGML_F16 = 1,
  RT_GGML_Q4_0 = 2,
  RT_GGML_Q8_0 = 8,
  RT_GGML_Q4_K = 12,
  RT_GGML_Q6_K = 14,
  RT_GGML_BF16 = 30
};

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
/* Bytes of ggml block storage for a [rows x cols] tensor of `ggml_type`; 0 if unsupported. */
size_t rt_ggml_nbytes(int ggml_type, size_t rows, size_t cols);

/* ------------------------------------------------------------------ level 1: trait FrozenMatmul
 * src/frozen.rs:14-25, implemented for GGUF weights by RieFrozen (src/rie.rs:66-129). */

/* RieFrozen::new (src/rie.rs:57-61): `packed_host` is the tensor exactly as stored in the
 * GGUF file, rows of ggml blocks. */
rt_status rt_frozen_create(rt_ctx* ctx, int ggml_type, size_t rows, size_t cols, const void* packed_host,
                           size_t nbytes, rt_frozen** out);
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


/* Device-resident forms of forward / backward_input: activations stay in HBM as bf16
 * [t x dim]; the result is written as f32 or bf16; `accumulate` (f32 only) adds into the
 * output, which is what backward_input's `+=` and the residual adds of
 * src/model.rs:178,181 need.  Asynchronous on the ctx stream; a kernel-side failure is
 * reported by the next rt_ctx_synchronize. */
rt_status rt_frozen_forward_dev(rt_frozen* w, const void* x_bf16_dev, size_t t, void* y_dev, int y_is_bf16,
                                int accumulate);
rt_status rt_frozen_backward_input_dev(rt_frozen* w, const void* dy_bf16_dev, size_t t, void* dx_dev,
                                       int dx_is_bf16, int accumulate);

#ifdef __cplusplus
}
#endif
#endif /* RT_B200_H */
