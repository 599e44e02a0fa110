// C ABI, op level: the per-row operations of src/ops.rs and the attention core of
// src/attention.rs as single calls with HOST buffers, exactly the device kernels the model
// driver launches.  They exist so that a host (and the parity tests) can check one operation at
// a time against the CPU path; the training step itself never crosses the host between ops.
// Every call copies in, launches on the ctx stream, copies out and synchronises.
#include "model.h"
#include <math.h>
#include <vector>

namespace {

// device temporaries of one call, freed when the call returns
struct Temps {
  std::vector<void*> ptrs;
  ~Temps() {
    for (void* p : ptrs) cudaFree(p);
  }
  template <class T>
  T* get(size_t n) {
    void* p = nullptr;
    if (cudaMalloc(&p, (n ? n : 1) * sizeof(T)) != cudaSuccess) return nullptr;
    ptrs.push_back(p);
    return (T*)p;
  }
  template <class T>
  T* up(const T* host, size_t n, cudaStream_t st) {
    T* d = get<T>(n);
    if (d && host && cudaMemcpyAsync(d, host, n * sizeof(T), cudaMemcpyHostToDevice, st) != cudaSuccess) return nullptr;
    return d;
  }
};

__global__ void f16_to_f32_kernel(const __half* in, float* out, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __half2float(in[i]);
}
// out[r, :] = in16[r, :] * scale[r]
__global__ void f16_rows_to_f32_kernel(const __half* in, const float* scale, int d, float* out, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __half2float(in[i]) * (scale ? scale[i / d] : 1.0f);
}

rt_status down_f16(rt_ctx* c, const __half* d16, const float* scale, int d, size_t n, float* host, Temps& t) {
  float* f = t.get<float>(n);
  if (!f) return c->fail(RT_ERR_CUDA, "out of device memory");
  f16_rows_to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(d16, scale, d, f, n);
  RT_CUDA(c, cudaMemcpyAsync(host, f, n * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  return RT_OK;
}

// ops.rs:118-131 inverse frequencies in f32, as the model driver builds them
rt_status rope_tables(rt_ctx* c, Temps& t, const int32_t* pos_host, size_t M, int rot, float theta, float freq_scale,
                      const float* factors, int n_factors, float** cs, float** sn, int** pos_dev) {
  const int half = rot / 2;
  int max_pos = 0;
  for (size_t i = 0; i < M; ++i) {
    if (pos_host[i] < 0 || pos_host[i] >= (1 << 20)) return c->fail(RT_ERR_BAD_INDEX, "position out of range");
    if (pos_host[i] > max_pos) max_pos = pos_host[i];
  }
  std::vector<float> inv(half);
  for (int i = 0; i < half; ++i) {
    float f = powf(theta, -2.0f * (float)i / (float)rot) * freq_scale;
    if (factors && i < n_factors && factors[i] != 0.0f) f /= factors[i];
    inv[i] = f;
  }
  float* inv_d = t.up(inv.data(), (size_t)half, c->stream);
  *cs = t.get<float>((size_t)(max_pos + 1) * half);
  *sn = t.get<float>((size_t)(max_pos + 1) * half);
  *pos_dev = t.up((const int*)pos_host, M, c->stream);
  if (!inv_d || !*cs || !*sn || !*pos_dev) return c->fail(RT_ERR_CUDA, "out of device memory");
  RT_CUDA(c, cudaStreamSynchronize(c->stream));  // `inv` leaves scope with the call
  rt::launch_rope_table(inv_d, half, max_pos + 1, *cs, *sn, c->stream);
  return RT_OK;
}

bool bad_heads(int nh, int nkv, int hd, int rot) {
  return nh <= 0 || nkv <= 0 || nh % nkv != 0 || (hd != 64 && hd != 128) || rot <= 0 || rot > hd || (rot & 1);
}

}  // namespace

using namespace rt;

extern "C" {

rt_status rt_op_rmsnorm(rt_ctx* c, const float* x, const float* w, size_t rows, size_t d, float eps, float* y) {
  if (!c || !x || !w || !y) return RT_ERR_BAD_ARG;
  if (rows == 0) return RT_OK;
  if (d == 0 || rows > (1u << 24) || d > (1u << 20)) return c->fail(RT_ERR_BAD_SHAPE, "bad rmsnorm shape");
  RT_CUDA(c, cudaSetDevice(c->device));
  Temps t;
  float* xd = t.up(x, rows * d, c->stream);
  float* wd = t.up(w, d, c->stream);
  __half* y16 = t.get<__half>(rows * d);
  if (!xd || !wd || !y16) return c->fail(RT_ERR_CUDA, "out of device memory");
  launch_rmsnorm_fwd(xd, wd, (int)rows, (int)d, eps, y16, c->stream);
  rt_status s = down_f16(c, y16, nullptr, (int)d, rows * d, y, t);
  if (s) return s;
  return c->check_device_status("rt_op_rmsnorm");
}

rt_status rt_op_rmsnorm_backward(rt_ctx* c, const float* x, const float* w, const float* dy, size_t rows, size_t d,
                                 float eps, float* dx) {
  if (!c || !x || !w || !dy || !dx) return RT_ERR_BAD_ARG;
  if (rows == 0) return RT_OK;
  if (d == 0 || rows > (1u << 24) || d > (1u << 20)) return c->fail(RT_ERR_BAD_SHAPE, "bad rmsnorm shape");
  RT_CUDA(c, cudaSetDevice(c->device));
  Temps t;
  float* xd = t.up(x, rows * d, c->stream);
  float* wd = t.up(w, d, c->stream);
  float* dyd = t.up(dy, rows * d, c->stream);
  float* out = t.get<float>(rows * d);
  __half* o16 = t.get<__half>(rows * d);
  float* sc = t.get<float>(rows);
  if (!xd || !wd || !dyd || !out || !o16 || !sc) return c->fail(RT_ERR_CUDA, "out of device memory");
  launch_rmsnorm_bwd(xd, wd, dyd, nullptr, (int)rows, (int)d, eps, out, o16, sc, c->stream);
  RT_CUDA(c, cudaMemcpyAsync(dx, out, rows * d * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  return c->check_device_status("rt_op_rmsnorm_backward");
}

rt_status rt_op_qk_norm_rope(rt_ctx* c, const float* q_raw, const float* k_raw, const float* v_raw, const int32_t* positions,
                             size_t M, int nh, int nkv, int hd, int rot, int neox, float theta, float freq_scale,
                             const float* factors, int n_factors, const float* q_norm_w, const float* k_norm_w, float eps,
                             float* q, float* k, float* v) {
  if (!c || !q_raw || !k_raw || !v_raw || !positions || !q || !k || !v) return RT_ERR_BAD_ARG;
  if (M == 0) return RT_OK;
  if (bad_heads(nh, nkv, hd, rot) || M > (1u << 24)) return c->fail(RT_ERR_BAD_SHAPE, "bad head shapes");
  if ((q_norm_w == nullptr) != (k_norm_w == nullptr)) return c->fail(RT_ERR_BAD_ARG, "q and k norm weights go together");
  RT_CUDA(c, cudaSetDevice(c->device));
  Temps t;
  const size_t nq = M * nh * hd, nk = M * nkv * hd;
  float *cs, *sn;
  int* pos;
  rt_status s = rope_tables(c, t, positions, M, rot, theta, freq_scale, factors, n_factors, &cs, &sn, &pos);
  if (s) return s;
  float *qd = t.up(q_raw, nq, c->stream), *kd = t.up(k_raw, nk, c->stream), *vd = t.up(v_raw, nk, c->stream);
  float *qw = q_norm_w ? t.up(q_norm_w, (size_t)hd, c->stream) : nullptr, *kw = k_norm_w ? t.up(k_norm_w, (size_t)hd, c->stream) : nullptr;
  __half *q16 = t.get<__half>(nq), *k16 = t.get<__half>(nk), *v16 = t.get<__half>(nk);
  if (!qd || !kd || !vd || !q16 || !k16 || !v16 || (q_norm_w && (!qw || !kw))) return c->fail(RT_ERR_CUDA, "out of device memory");
  launch_qk_rope_fwd(qd, kd, vd, 0, qw, kw, pos, cs, sn, (int)M, nh, nkv, hd, rot, neox, eps, q16, k16, v16, c->stream);
  if ((s = down_f16(c, q16, nullptr, 1, nq, q, t)) || (s = down_f16(c, k16, nullptr, 1, nk, k, t)) ||
      (s = down_f16(c, v16, nullptr, 1, nk, v, t)))
    return s;
  return c->check_device_status("rt_op_qk_norm_rope");
}

rt_status rt_op_qk_norm_rope_backward(rt_ctx* c, const float* dq, const float* dk, const float* dv, const float* q_raw,
                                      const float* k_raw, const int32_t* positions, size_t M, int nh, int nkv, int hd,
                                      int rot, int neox, float theta, float freq_scale, const float* factors,
                                      int n_factors, const float* q_norm_w, const float* k_norm_w, float eps,
                                      float* dq_raw, float* dk_raw, float* dv_out) {
  if (!c || !dq || !dk || !dv || !q_raw || !k_raw || !positions || !dq_raw || !dk_raw || !dv_out) return RT_ERR_BAD_ARG;
  if (M == 0) return RT_OK;
  if (bad_heads(nh, nkv, hd, rot) || M > (1u << 24)) return c->fail(RT_ERR_BAD_SHAPE, "bad head shapes");
  if ((q_norm_w == nullptr) != (k_norm_w == nullptr)) return c->fail(RT_ERR_BAD_ARG, "q and k norm weights go together");
  RT_CUDA(c, cudaSetDevice(c->device));
  Temps t;
  const size_t nq = M * nh * hd, nk = M * nkv * hd;
  float *cs, *sn;
  int* pos;
  rt_status s = rope_tables(c, t, positions, M, rot, theta, freq_scale, factors, n_factors, &cs, &sn, &pos);
  if (s) return s;
  float *dqd = t.up(dq, nq, c->stream), *dkd = t.up(dk, nk, c->stream), *dvd = t.up(dv, nk, c->stream);
  float *qd = t.up(q_raw, nq, c->stream), *kd = t.up(k_raw, nk, c->stream);
  float *qw = q_norm_w ? t.up(q_norm_w, (size_t)hd, c->stream) : nullptr, *kw = k_norm_w ? t.up(k_norm_w, (size_t)hd, c->stream) : nullptr;
  __half *q16 = t.get<__half>(nq), *k16 = t.get<__half>(nk), *v16 = t.get<__half>(nk);
  float *sq = t.get<float>(M), *sk = t.get<float>(M), *sv = t.get<float>(M);
  if (!dqd || !dkd || !dvd || !qd || !kd || !q16 || !k16 || !v16 || !sq || !sk || !sv || (q_norm_w && (!qw || !kw)))
    return c->fail(RT_ERR_CUDA, "out of device memory");
  launch_qk_rope_bwd(dqd, dkd, dvd, qd, kd, 0, qw, kw, pos, cs, sn, (int)M, nh, nkv, hd, rot, neox, eps, q16, k16, v16, 0, sq,
                     sk, sv, c->stream);
  if ((s = down_f16(c, q16, sq, nh * hd, nq, dq_raw, t)) || (s = down_f16(c, k16, sk, nkv * hd, nk, dk_raw, t)) ||
      (s = down_f16(c, v16, sv, nkv * hd, nk, dv_out, t)))
    return s;
  return c->check_device_status("rt_op_qk_norm_rope_backward");
}

rt_status rt_op_attention(rt_ctx* c, const float* q, const float* k, const float* v, const int32_t* seq_start, size_t M,
                          int nh, int nkv, int hd, float* o, float* lse) {
  if (!c || !q || !k || !v || !seq_start || !o) return RT_ERR_BAD_ARG;
  if (M == 0) return RT_OK;
  if (bad_heads(nh, nkv, hd, hd) || M > (1u << 24)) return c->fail(RT_ERR_BAD_SHAPE, "bad head shapes");
  for (size_t i = 0; i < M; ++i)
    if (seq_start[i] < 0 || (size_t)seq_start[i] > i || (i > 0 && seq_start[i] < seq_start[i - 1]))
      return c->fail(RT_ERR_BAD_INDEX, "seq_start must be non-decreasing and at most the row index");
  RT_CUDA(c, cudaSetDevice(c->device));
  Temps t;
  const size_t nq = M * nh * hd, nk = M * nkv * hd;
  float *qd = t.up(q, nq, c->stream), *kd = t.up(k, nk, c->stream), *vd = t.up(v, nk, c->stream);
  int* ss = t.up((const int*)seq_start, M, c->stream);
  __half *q16 = t.get<__half>(nq), *k16 = t.get<__half>(nk), *v16 = t.get<__half>(nk), *o16 = t.get<__half>(nq);
  float* lsed = t.get<float>(M * nh);
  if (!qd || !kd || !vd || !ss || !q16 || !k16 || !v16 || !o16 || !lsed) return c->fail(RT_ERR_CUDA, "out of device memory");
  launch_f32_to_16(qd, q16, nq, true, c->stream);
  launch_f32_to_16(kd, k16, nk, true, c->stream);
  launch_f32_to_16(vd, v16, nk, true, c->stream);
  if (attn_forward(c, q16, k16, v16, ss, nullptr, (int)M, nh, nkv, hd, o16, lsed))
    return c->fail(RT_ERR_CUDA, "attention forward launch failed");
  rt_status s = down_f16(c, o16, nullptr, 1, nq, o, t);
  if (s) return s;
  if (lse) RT_CUDA(c, cudaMemcpyAsync(lse, lsed, M * nh * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  return c->check_device_status("rt_op_attention");
}

rt_status rt_op_attention_backward(rt_ctx* c, const float* q, const float* k, const float* v, const float* d_o,
                                   const int32_t* seq_start, size_t M, int nh, int nkv, int hd, float* dq, float* dk,
                                   float* dv) {
  if (!c || !q || !k || !v || !d_o || !seq_start || !dq || !dk || !dv) return RT_ERR_BAD_ARG;
  if (M == 0) return RT_OK;
  if (bad_heads(nh, nkv, hd, hd) || M > (1u << 24)) return c->fail(RT_ERR_BAD_SHAPE, "bad head shapes");
  for (size_t i = 0; i < M; ++i)
    if (seq_start[i] < 0 || (size_t)seq_start[i] > i || (i > 0 && seq_start[i] < seq_start[i - 1]))
      return c->fail(RT_ERR_BAD_INDEX, "seq_start must be non-decreasing and at most the row index");
  RT_CUDA(c, cudaSetDevice(c->device));
  Temps t;
  const size_t nq = M * nh * hd, nk = M * nkv * hd;
  float *qd = t.up(q, nq, c->stream), *kd = t.up(k, nk, c->stream), *vd = t.up(v, nk, c->stream), *dod = t.up(d_o, nq, c->stream);
  int* ss = t.up((const int*)seq_start, M, c->stream);
  __half *q16 = t.get<__half>(nq), *k16 = t.get<__half>(nk), *v16 = t.get<__half>(nk), *o16 = t.get<__half>(nq), *do16 = t.get<__half>(nq);
  float *lsed = t.get<float>(M * nh), *delta = t.get<float>(M * nh), *sc = t.get<float>(M), *amax = t.get<float>(2 * M + 4);
  float *dqd = t.get<float>(nq), *dkd = t.get<float>(nk), *dvd = t.get<float>(nk);
  if (!qd || !kd || !vd || !dod || !ss || !q16 || !k16 || !v16 || !o16 || !do16 || !lsed || !delta || !sc || !amax || !dqd || !dkd || !dvd)
    return c->fail(RT_ERR_CUDA, "out of device memory");
  launch_f32_to_16(qd, q16, nq, true, c->stream);
  launch_f32_to_16(kd, k16, nk, true, c->stream);
  launch_f32_to_16(vd, v16, nk, true, c->stream);
  if (attn_forward(c, q16, k16, v16, ss, nullptr, (int)M, nh, nkv, hd, o16, lsed))
    return c->fail(RT_ERR_CUDA, "attention forward launch failed");
  // dO as the model passes it: f16 rows divided by their largest magnitude, factors beside them
  launch_normalize_rows(dod, (int)M, nh * hd, do16, sc, c->stream);
  launch_rowscale_seqmax(sc, ss, (int)M, amax, c->stream);
  if (attn_backward(c, q16, k16, v16, o16, do16, amax, sc, lsed, ss, nullptr, (int)M, nh, nkv, hd, delta, dqd, dkd, dvd))
    return c->fail(RT_ERR_CUDA, "attention backward launch failed");
  RT_CUDA(c, cudaMemcpyAsync(dq, dqd, nq * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  RT_CUDA(c, cudaMemcpyAsync(dk, dkd, nk * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  RT_CUDA(c, cudaMemcpyAsync(dv, dvd, nk * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  return c->check_device_status("rt_op_attention_backward");
}

rt_status rt_op_swiglu(rt_ctx* c, const float* gate, const float* up, size_t rows, size_t ff, float* h) {
  if (!c || !gate || !up || !h) return RT_ERR_BAD_ARG;
  if (rows == 0) return RT_OK;
  if (ff == 0 || rows > (1u << 24) || ff > (1u << 20)) return c->fail(RT_ERR_BAD_SHAPE, "bad swiglu shape");
  RT_CUDA(c, cudaSetDevice(c->device));
  Temps t;
  const size_t n = rows * ff;
  float *gd = t.up(gate, n, c->stream), *ud = t.up(up, n, c->stream);
  __half *g16 = t.get<__half>(n), *u16 = t.get<__half>(n), *h16 = t.get<__half>(n);
  if (!gd || !ud || !g16 || !u16 || !h16) return c->fail(RT_ERR_CUDA, "out of device memory");
  launch_f32_to_16(gd, g16, n, true, c->stream);
  launch_f32_to_16(ud, u16, n, true, c->stream);
  launch_swiglu_fwd(g16, u16, 0, (int)rows, (int)ff, h16, c->status_dev, c->stream);
  rt_status s = down_f16(c, h16, nullptr, 1, n, h, t);
  if (s) return s;
  return c->check_device_status("rt_op_swiglu");
}

rt_status rt_op_swiglu_backward(rt_ctx* c, const float* gate, const float* up, const float* dh, size_t rows, size_t ff,
                                float* dgate, float* dup) {
  if (!c || !gate || !up || !dh || !dgate || !dup) return RT_ERR_BAD_ARG;
  if (rows == 0) return RT_OK;
  if (ff == 0 || rows > (1u << 24) || ff > (1u << 20)) return c->fail(RT_ERR_BAD_SHAPE, "bad swiglu shape");
  RT_CUDA(c, cudaSetDevice(c->device));
  Temps t;
  const size_t n = rows * ff;
  float *gd = t.up(gate, n, c->stream), *ud = t.up(up, n, c->stream), *dhd = t.up(dh, n, c->stream);
  __half *g16 = t.get<__half>(n), *u16 = t.get<__half>(n), *dg16 = t.get<__half>(n), *du16 = t.get<__half>(n);
  float *sg = t.get<float>(rows), *su = t.get<float>(rows);
  if (!gd || !ud || !dhd || !g16 || !u16 || !dg16 || !du16 || !sg || !su) return c->fail(RT_ERR_CUDA, "out of device memory");
  launch_f32_to_16(gd, g16, n, true, c->stream);
  launch_f32_to_16(ud, u16, n, true, c->stream);
  launch_swiglu_bwd(dhd, 0, nullptr, g16, u16, 0, (int)rows, (int)ff, dg16, du16, 0, sg, su, c->stream);
  rt_status s;
  if ((s = down_f16(c, dg16, sg, (int)ff, n, dgate, t)) || (s = down_f16(c, du16, su, (int)ff, n, dup, t))) return s;
  return c->check_device_status("rt_op_swiglu_backward");
}

rt_status rt_op_cross_entropy(rt_ctx* c, const float* logits, size_t rows, size_t vocab, const int32_t* target,
                              const float* weight, float* logp, int32_t* hits, int32_t* argmax, float* dlogits) {
  if (!c || !logits || !target || !logp) return RT_ERR_BAD_ARG;
  if (rows == 0) return RT_OK;
  if (vocab == 0 || rows > (1u << 24) || vocab > (1u << 24)) return c->fail(RT_ERR_BAD_SHAPE, "bad logits shape");
  if (dlogits && !weight) return c->fail(RT_ERR_BAD_ARG, "weights missing");
  RT_CUDA(c, cudaSetDevice(c->device));
  Temps t;
  const size_t n = rows * vocab;
  float* ld = t.up(logits, n, c->stream);
  int* td = t.up((const int*)target, rows, c->stream);
  float* wd = weight ? t.up(weight, rows, c->stream) : nullptr;
  float* lp = t.get<float>(rows);
  int* hd = t.get<int>(4);
  int* am = argmax ? t.get<int>(rows) : nullptr;
  __half* d16 = dlogits ? t.get<__half>(n) : nullptr;
  float* sc = dlogits ? t.get<float>(rows) : nullptr;
  if (!ld || !td || !lp || !hd || (weight && !wd) || (argmax && !am) || (dlogits && (!d16 || !sc)))
    return c->fail(RT_ERR_CUDA, "out of device memory");
  RT_CUDA(c, cudaMemsetAsync(hd, 0, 4, c->stream));
  launch_ce_rows(ld, (int)rows, (int)vocab, td, wd, lp, hd, d16, sc, am, c->status_dev, c->stream);
  RT_CUDA(c, cudaMemcpyAsync(logp, lp, rows * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  if (hits) RT_CUDA(c, cudaMemcpyAsync(hits, hd, 4, cudaMemcpyDeviceToHost, c->stream));
  if (argmax) RT_CUDA(c, cudaMemcpyAsync(argmax, am, rows * sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  if (dlogits) {
    rt_status s = down_f16(c, d16, sc, (int)vocab, n, dlogits, t);
    if (s) return s;
  }
  return c->check_device_status("rt_op_cross_entropy");
}

}  // extern "C"
