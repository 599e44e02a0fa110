// C ABI, level 1: the FrozenMatmul trait (reference src/frozen.rs:14-25) over host buffers.
#include "ctx.h"
#include "../../include/rt_b200.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <map>
#include <string>
#include <vector>
#include <mutex>
#include <set>

void* rt_ctx::get_scratch(int slot, size_t bytes) {
  if (bytes <= scratch_bytes[slot]) return scratch[slot];
  if (scratch[slot]) cudaFree(scratch[slot]);
  scratch[slot] = nullptr;
  scratch_bytes[slot] = 0;
  size_t want = bytes + bytes / 4 + 256;
  if (cudaMalloc(&scratch[slot], want) != cudaSuccess) return nullptr;
  scratch_bytes[slot] = want;
  return scratch[slot];
}

rt_status rt_ctx::check_device_status(const char* where) {
  cudaError_t e = cudaMemcpyAsync(status_host, status_dev, sizeof(int), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return cuda_fail(e, where);
  int s = *status_host;
  if (s == 0) return RT_OK;
  cudaMemsetAsync(status_dev, 0, sizeof(int), stream);
  char buf[160];
  if (s == RT_ERR_BAD_INDEX) {
    snprintf(buf, sizeof buf, "%s: index out of range on device", where);
    err = buf;
    return RT_ERR_BAD_INDEX;
  }
  if (s == RT_ERR_NONFINITE) {
    snprintf(buf, sizeof buf, "%s: silu(gate) * up left the range of f16 (an activation beyond 65504)", where);
    err = buf;
    return RT_ERR_NONFINITE;
  }
  snprintf(buf, sizeof buf, "%s: device wait timed out at site %d", where, s);
  err = buf;
  return RT_ERR_DEVICE_WAIT_TIMEOUT;
}

namespace rt {
static std::mutex g_ctx_mutex;
static std::set<const rt_ctx*> g_live_ctx;
bool ctx_alive(const rt_ctx* c) {
  std::lock_guard<std::mutex> lock(g_ctx_mutex);
  return g_live_ctx.count(c) != 0;
}
static void ctx_register(const rt_ctx* c, bool live) {
  std::lock_guard<std::mutex> lock(g_ctx_mutex);
  if (live) g_live_ctx.insert(c);
  else g_live_ctx.erase(c);
}

int frozen_matmul_launch(rt_ctx* ctx, const QWeight& w, const QGemmArgs& a) {
  int rc = qgemm_launch(ctx, w, a);
  if (rc || !w.dense16_lo || a.out_dtype != OUT_F32 || a.tok_mode) return rc;
  QWeight lo = w;
  lo.dense16 = w.dense16_lo;
  lo.dense16_lo = nullptr;
  QGemmArgs b = a;  // the low term adds into the result; bias and the adapter chunk went in with the high term
  b.accumulate = 1;
  b.bias = nullptr;
  b.lora = LoraSide();
  return qgemm_launch(ctx, lo, b);
}
}  // namespace rt

extern "C" {

rt_status rt_ctx_create(int device, rt_ctx** out) {
  if (!out) return RT_ERR_BAD_ARG;
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) return RT_ERR_CUDA;
  rt_ctx* c = new rt_ctx();
  c->device = device;
  cudaError_t e = cudaSetDevice(device);
  cudaDeviceProp prop;
  if (e == cudaSuccess) e = cudaGetDeviceProperties(&prop, device);
  if (e == cudaSuccess && prop.major != 10) {
    fprintf(stderr, "rt_b200: device %d is sm_%d%d; this library is built for sm_100a only\n", device, prop.major,
            prop.minor);
    delete c;
    return RT_ERR_CUDA;
  }
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking);
  c->stream = c->own_stream;
  if (e == cudaSuccess) e = cudaMalloc(&c->status_dev, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(c->status_dev, 0, sizeof(int));
  if (e == cudaSuccess) e = cudaDeviceSynchronize();  // the clear ran on the legacy stream; own_stream does not wait for it
  if (e == cudaSuccess) e = cudaMallocHost(&c->status_host, sizeof(int));
  if (e != cudaSuccess || rt::qgemm_init() != RT_OK) {
    fprintf(stderr, "rt_b200: context creation failed: %s\n", cudaGetErrorString(e));
    delete c;
    return RT_ERR_CUDA;
  }
  c->num_sms = prop.multiProcessorCount;
  rt::ctx_register(c, true);
  *out = c;
  return RT_OK;
}

void rt_ctx_destroy(rt_ctx* c) {
  if (!c || !rt::ctx_alive(c)) return;
  rt::ctx_register(c, false);
  cudaSetDevice(c->device);
  if (c->stream) cudaStreamSynchronize(c->stream);
  rt_comm_destroy(c);
  for (cudaEvent_t e : c->prof_events) cudaEventDestroy(e);
  for (int i = 0; i < 4; ++i)
    if (c->scratch[i]) cudaFree(c->scratch[i]);
  if (c->status_dev) cudaFree(c->status_dev);
  if (c->status_host) cudaFreeHost(c->status_host);
  if (c->own_stream) cudaStreamDestroy(c->own_stream);
  delete c;
}

const char* rt_last_error(const rt_ctx* c) { return c ? c->err.c_str() : "null context"; }

rt_status rt_ctx_synchronize(rt_ctx* c) {
  if (!c) return RT_ERR_BAD_ARG;
  return c->check_device_status("rt_ctx_synchronize");
}

rt_status rt_ctx_set_stream(rt_ctx* c, void* s) {
  if (!c) return RT_ERR_BAD_ARG;
  c->stream = (cudaStream_t)s;  // NULL is the legacy default stream, a valid choice
  return RT_OK;
}

uint64_t rt_ctx_launch_count(const rt_ctx*) { return (uint64_t)rt::g_launch_count.load(); }

rt_status rt_ctx_set_profiling(rt_ctx* c, int on) {
  if (!c) return RT_ERR_BAD_ARG;
  c->profiling = on != 0;
  return RT_OK;
}

rt_status rt_ctx_profile_read(rt_ctx* c, uint64_t* n, double* ms, double* flops, double* bytes) {
  if (!c) return RT_ERR_BAD_ARG;
  RT_CUDA(c, cudaSetDevice(c->device));
  RT_CUDA(c, cudaStreamSynchronize(c->stream));
  double total = 0;
  const bool verbose = getenv("RT_B200_PROFILE_VERBOSE") != nullptr;
  std::map<std::string, std::pair<int, double>> table;
  for (size_t i = 0; i + 1 < c->prof_used; i += 2) {
    float t = 0;
    RT_CUDA(c, cudaEventElapsedTime(&t, c->prof_events[i], c->prof_events[i + 1]));
    total += t;
    if (verbose && i / 2 < c->prof_recs.size()) {
      const auto& r = c->prof_recs[i / 2];
      char key[96];
      snprintf(key, sizeof key, "cls%d M=%d rows=%d contract=%d", r.cls, r.M, r.rows, r.contract);
      auto& e = table[key];
      e.first += 1;
      e.second += t;
    }
  }
  if (verbose)
    for (auto& kv : table)
      fprintf(stderr, "[rt_b200 profile] %-48s n=%5d total=%9.3f ms avg=%8.1f us\n", kv.first.c_str(), kv.second.first,
              kv.second.second, 1e3 * kv.second.second / kv.second.first);
  c->prof_recs.clear();
  if (n) *n = c->prof_used / 2;
  if (ms) *ms = total;
  if (flops) *flops = c->prof_flops;
  if (bytes) *bytes = c->prof_bytes;
  c->prof_used = 0;
  c->prof_flops = 0;
  c->prof_bytes = 0;
  return RT_OK;
}

void* rt_ctx_stream(rt_ctx* c) { return c ? (void*)c->stream : nullptr; }

size_t rt_ggml_nbytes(int t, size_t rows, size_t cols) {
  if (t == RT_GGML_F32) return rows * cols * 4;
  int be = rt::fmt_block_elems(t), bb = rt::fmt_block_bytes(t);
  if (bb == 0 || cols % be != 0) return 0;
  return rows * (cols / be) * bb;
}

// FrozenWeight::F32 (src/frozen.rs:33-52): the f32 matrix stays on the device for row(), and its
// two-term f16 split feeds the tensor cores.
static rt_status frozen_create_f32(rt_ctx* c, size_t rows, size_t cols, const float* w_host, size_t nbytes, rt_frozen** out) {
  if (rows == 0 || cols == 0 || rows > (1u << 30) || cols > (1u << 30)) return c->fail(RT_ERR_BAD_SHAPE, "empty or oversized weight");
  if (cols % 8 != 0) return c->fail(RT_ERR_BAD_SHAPE, "f32 rows must be a multiple of 8 long");
  if (nbytes != rows * cols * 4) return c->fail(RT_ERR_BAD_SHAPE, "nbytes does not match type and shape");
  RT_CUDA(c, cudaSetDevice(c->device));
  rt_frozen* f = new rt_frozen();
  f->ctx = c;
  f->device = c->device;
  rt::QWeight& w = f->w;
  w.fmt = rt::GGML_F16;
  w.rows = (int)rows;
  w.cols = (int)cols;
  w.ggml_nbytes = nbytes;
  w.dev_nbytes = rows * cols * 2;
  float* w32 = nullptr;
  cudaError_t e = cudaMalloc(&w32, nbytes);
  w.f32 = w32;
  if (e == cudaSuccess) e = cudaMalloc(&w.dense16, rows * cols * 2);
  if (e == cudaSuccess) e = cudaMalloc(&w.dense16_lo, rows * cols * 2);
  if (e == cudaSuccess) e = cudaMemcpyAsync(w32, w_host, nbytes, cudaMemcpyHostToDevice, c->stream);
  if (e == cudaSuccess) {
    rt::launch_split_f32_hi_lo(w32, rows * cols, (__half*)w.dense16, (__half*)w.dense16_lo, c->stream);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
  if (e != cudaSuccess) {
    rt_frozen_destroy(f);
    return c->cuda_fail(e, "rt_frozen_create (f32)");
  }
  *out = f;
  return RT_OK;
}

rt_status rt_frozen_create(rt_ctx* c, int ggml_type, size_t rows, size_t cols, const void* packed_host,
                           size_t nbytes, rt_frozen** out) {
  if (!c || !out || !packed_host) return RT_ERR_BAD_ARG;
  *out = nullptr;
  if (ggml_type == RT_GGML_F32) return frozen_create_f32(c, rows, cols, (const float*)packed_host, nbytes, out);
  if (rt::fmt_block_bytes(ggml_type) == 0) return c->fail(RT_ERR_UNSUPPORTED_TYPE, "unsupported ggml tensor type");
  if (rows == 0 || cols == 0 || rows > (1u << 30) || cols > (1u << 30)) return c->fail(RT_ERR_BAD_SHAPE, "empty or oversized weight");
  const int be = rt::fmt_block_elems(ggml_type);
  if (cols % be != 0) return c->fail(RT_ERR_BAD_SHAPE, "row length is not a multiple of the block size");
  if (rt::fmt_is_16bit(ggml_type) && cols % 8 != 0) return c->fail(RT_ERR_BAD_SHAPE, "16-bit rows must be a multiple of 8 long");
  if (nbytes != rt_ggml_nbytes(ggml_type, rows, cols)) return c->fail(RT_ERR_BAD_SHAPE, "nbytes does not match type and shape");
  RT_CUDA(c, cudaSetDevice(c->device));
  rt_frozen* f = new rt_frozen();
  f->ctx = c;
  f->device = c->device;
  rt::QWeight& w = f->w;
  w.fmt = ggml_type;
  w.rows = (int)rows;
  w.cols = (int)cols;
  w.ggml_nbytes = nbytes;
  cudaError_t e;
  if (rt::fmt_is_16bit(ggml_type)) {
    e = cudaMalloc(&w.dense16, nbytes);
    if (e == cudaSuccess) e = cudaMemcpyAsync(w.dense16, packed_host, nbytes, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    w.dev_nbytes = nbytes;
  } else {
    w.nbr = (int)((rows + 127) / 128) * 2;
    w.nbk = (int)((cols + 127) / 128) * 2;
    w.dev_nbytes = (size_t)w.nbr * w.nbk * rt::fmt_brick_bytes(ggml_type);
    void* raw = nullptr;
    e = cudaMalloc(&w.bricks, w.dev_nbytes);
    if (e == cudaSuccess) e = cudaMalloc(&raw, nbytes);
    if (e == cudaSuccess) e = cudaMemcpyAsync(raw, packed_host, nbytes, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) {
      rt::launch_repack((const uint8_t*)raw, w, c->stream);
      e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (raw) cudaFree(raw);
  }
  if (e != cudaSuccess) {
    rt_frozen_destroy(f);
    return c->cuda_fail(e, "rt_frozen_create");
  }
  *out = f;
  return RT_OK;
}

// FrozenWeight::Q8_0 (src/frozen.rs:39-73): f32 scale per 32 columns + signed bytes.  The scale is
// f32, which ggml's Q8_0 block (f16 scale) cannot hold, so the values d*q go through the f32
// storage above: q is exact in f16 and d*q splits into two f16 terms like any f32 weight.
rt_status rt_frozen_create_q8_0(rt_ctx* c, size_t rows, size_t cols, const float* scales_host, const int8_t* qs_host,
                                rt_frozen** out) {
  if (!c || !out || !scales_host || !qs_host) return RT_ERR_BAD_ARG;
  *out = nullptr;
  if (rows == 0 || cols == 0 || cols % 32 != 0) return c->fail(RT_ERR_BAD_SHAPE, "Q8_0 rows must be a multiple of 32 long");
  std::vector<float> w(rows * cols);
  for (size_t i = 0; i < rows * cols; ++i) w[i] = scales_host[i / 32] * (float)qs_host[i];
  rt_status st = frozen_create_f32(c, rows, cols, w.data(), rows * cols * 4, out);
  if (st == RT_OK) (*out)->w.ggml_nbytes = rows * cols / 32 * 4 + rows * cols;  // FrozenWeight::nbytes, src/frozen.rs:181-186
  return st;
}

void rt_frozen_destroy(rt_frozen* f) {
  if (!f) return;
  cudaSetDevice(f->device);
  if (!rt::ctx_alive(f->ctx)) cudaDeviceSynchronize();  // the context's stream is gone: finish whatever still reads the weight
  if (!f->borrowed) {
    if (f->w.bricks) cudaFree(f->w.bricks);
    if (f->w.dense16) cudaFree(f->w.dense16);
  }
  if (f->w.dense16_lo) cudaFree(f->w.dense16_lo);
  if (f->w.f32) cudaFree((void*)f->w.f32);
  delete f;
}

size_t rt_frozen_out_dim(const rt_frozen* f) { return f ? (size_t)f->w.rows : 0; }
size_t rt_frozen_in_dim(const rt_frozen* f) { return f ? (size_t)f->w.cols : 0; }
size_t rt_frozen_nbytes(const rt_frozen* f) { return f ? f->w.ggml_nbytes : 0; }

static rt_status frozen_matmul_host(rt_frozen* f, int dir, const float* in_host, size_t t, float* out_host,
                                    bool accumulate) {
  if (!f || !in_host || !out_host) return RT_ERR_BAD_ARG;
  rt_ctx* c = f->ctx;
  if (t == 0) return RT_OK;
  if (t > (1u << 24)) return c->fail(RT_ERR_BAD_SHAPE, "too many rows");
  RT_CUDA(c, cudaSetDevice(c->device));
  const size_t in_dim = dir == rt::QG_FWD ? f->w.cols : f->w.rows;
  const size_t out_dim = dir == rt::QG_FWD ? f->w.rows : f->w.cols;
  float* in_f32 = (float*)c->get_scratch(0, t * in_dim * sizeof(float));
  // the 16-bit copy of the input and, behind it, one f32 factor per row
  const size_t in16_bytes = (t * in_dim * sizeof(__half) + 255) / 256 * 256;
  __nv_bfloat16* in_bf = (__nv_bfloat16*)c->get_scratch(1, in16_bytes + t * sizeof(float));
  float* out_f32 = (float*)c->get_scratch(2, t * out_dim * sizeof(float));
  if (!in_f32 || !in_bf || !out_f32) return c->fail(RT_ERR_CUDA, "out of device memory");
  RT_CUDA(c, cudaMemcpyAsync(in_f32, in_host, t * in_dim * sizeof(float), cudaMemcpyHostToDevice, c->stream));
  if (accumulate)
    RT_CUDA(c, cudaMemcpyAsync(out_f32, out_host, t * out_dim * sizeof(float), cudaMemcpyHostToDevice, c->stream));
  // forward activations go in as f16 (11 significant bits); gradients as f16 rows divided by their
  // largest magnitude, with that factor multiplied back onto the result row (f32's range, f16's bits)
  const bool fwd = dir == rt::QG_FWD;
  float* row_scale = nullptr;
  if (fwd) {
    rt::launch_f32_to_16(in_f32, in_bf, t * in_dim, true, c->stream);
  } else {
    row_scale = (float*)((uint8_t*)in_bf + in16_bytes);  // (scratch slot 3 holds the matmul's split-K partial sums)
    rt::launch_normalize_rows(in_f32, (int)t, (int)in_dim, (__half*)in_bf, row_scale, c->stream);
  }
  rt::QGemmArgs a;
  a.dir = dir;
  a.act = in_bf;
  a.act_f16 = 1;
  a.M = (int)t;
  a.out = out_f32;
  a.out_dtype = rt::OUT_F32;
  a.accumulate = accumulate ? 1 : 0;
  a.row_scale = row_scale;
  int rc = rt::frozen_matmul_launch(c, f->w, a);
  if (rc) return c->fail(rc, "qgemm launch failed");
  RT_CUDA(c, cudaMemcpyAsync(out_host, out_f32, t * out_dim * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  return c->check_device_status("rt_frozen matmul");
}

rt_status rt_frozen_forward(rt_frozen* f, const float* x_host, size_t t, float* y_host) {
  return frozen_matmul_host(f, rt::QG_FWD, x_host, t, y_host, false);
}

rt_status rt_frozen_backward_input(rt_frozen* f, const float* dy_host, size_t t, float* dx_host) {
  return frozen_matmul_host(f, rt::QG_BWD, dy_host, t, dx_host, true);
}

static rt_status frozen_matmul_dev(rt_frozen* f, int dir, const void* in_dev, int in_dtype, size_t t, void* out_dev,
                                   int out_dtype, int accumulate) {
  if (!f || !in_dev || !out_dev) return RT_ERR_BAD_ARG;
  rt_ctx* c = f->ctx;
  if (t == 0) return RT_OK;
  if (t > (1u << 24)) return c->fail(RT_ERR_BAD_SHAPE, "too many rows");
  if (in_dtype != RT_DT_F16 && in_dtype != RT_DT_BF16) return c->fail(RT_ERR_BAD_ARG, "activations must be f16 or bf16");
  if (out_dtype < 0 || out_dtype > 2) return c->fail(RT_ERR_BAD_ARG, "bad output dtype");
  if (accumulate && out_dtype != RT_DT_F32) return c->fail(RT_ERR_BAD_ARG, "accumulate needs an f32 output");
  RT_CUDA(c, cudaSetDevice(c->device));
  rt::QGemmArgs a;
  a.dir = dir;
  a.act = in_dev;
  a.act_f16 = in_dtype == RT_DT_F16;
  a.M = (int)t;
  a.out = out_dev;
  a.out_dtype = out_dtype;
  a.accumulate = accumulate ? 1 : 0;
  int rc = rt::frozen_matmul_launch(c, f->w, a);
  if (rc) return c->fail(rc, "qgemm launch failed");
  return RT_OK;
}

rt_status rt_frozen_forward_dev(rt_frozen* f, const void* x, int in_dt, size_t t, void* y, int out_dt, int acc) {
  return frozen_matmul_dev(f, rt::QG_FWD, x, in_dt, t, y, out_dt, acc);
}
rt_status rt_frozen_backward_input_dev(rt_frozen* f, const void* dy, int in_dt, size_t t, void* dx, int out_dt,
                                       int acc) {
  return frozen_matmul_dev(f, rt::QG_BWD, dy, in_dt, t, dx, out_dt, acc);
}

rt_status rt_frozen_row(rt_frozen* f, size_t r, float* out_host) {
  if (!f || !out_host) return RT_ERR_BAD_ARG;
  rt_ctx* c = f->ctx;
  if (r >= (size_t)f->w.rows) return c->fail(RT_ERR_BAD_INDEX, "row index out of range");
  RT_CUDA(c, cudaSetDevice(c->device));
  float* out = (float*)c->get_scratch(2, (size_t)f->w.cols * sizeof(float));
  int* id = (int*)c->get_scratch(3, sizeof(int));
  if (!out || !id) return c->fail(RT_ERR_CUDA, "out of device memory");
  int ri = (int)r;
  RT_CUDA(c, cudaMemcpyAsync(id, &ri, sizeof(int), cudaMemcpyHostToDevice, c->stream));
  rt::launch_gather_rows(f->w, id, 1, out, c->status_dev, c->stream);
  RT_CUDA(c, cudaMemcpyAsync(out_host, out, (size_t)f->w.cols * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  return c->check_device_status("rt_frozen_row");
}

}  // extern "C"
