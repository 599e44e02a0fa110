/*
 * oracle.c -- CPU restatement of Rust_Trainer's frozen-quantised-linear LoRA training path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product (rust_trainer_b200/) may call this; it is
 * the checker for tests/, for __graft_entry__.smoke() and the timed CPU baseline of bench.py.
 *
 * Each function restates, in plain f32 C, the algorithm of the reference function it cites
 * (file:line inside olapwriter-prog/Rust_Trainer).  The quantised arithmetic itself lives in
 * the reference's un-vendored dependency rie-core 0.1.0 @ f3be365b (Cargo.lock:529-539), which
 * implements the public ggml block formats; the decoders below restate those published
 * formats and are pinned against the independent `gguf` Python package in tests/.
 *
 * Parity status: PINNED.  Block decode against gguf-py (bit exact); LR schedule, f16 rounding
 * and the adjoint identity against the reference's own known-answer tests; whole-model loss and
 * LoRA gradients against the reference's own float64 checker (tools/reference_check.py, run
 * unmodified on a file in the layout of examples/export_reference.rs that
 * tests/golden/make_reference_export.py writes from this oracle's numbers; its float64 outputs
 * are committed as tests/golden/reference_check_float64.npz).  The reference binary itself
 * cannot run here (no Rust toolchain).  What is restated is the "smooth" mode the reference's
 * backward and its checker assume (dequantised f32 weights, f32 activations, f16 K/V
 * rounding); orc_set_act_int8(1) adds the engine's per-block 8-bit rounding of forward
 * activations (src/rie.rs:77-80) as an informative second mode.
 *
 * Build: gcc -O3 -march=native -fopenmp -shared -fPIC oracle.c -o liboracle.so -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

enum { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q8_0 = 8, T_Q4_K = 12, T_Q6_K = 14, T_BF16 = 30 };

/* ------------------------------------------------------------------ scalar helpers */
static float f16_to_f32(uint16_t h) {
  uint32_t s = (uint32_t)(h & 0x8000) << 16, e = (h >> 10) & 31, m = h & 1023, u;
  if (e == 0) {
    if (m == 0) u = s;
    else {
      int sh = 0;
      while (!(m & 1024)) { m <<= 1; ++sh; }
      u = s | ((uint32_t)(113 - sh) << 23) | ((m & 1023) << 13);
    }
  } else if (e == 31) u = s | 0x7f800000u | (m << 13);
  else u = s | ((e + 112) << 23) | (m << 13);
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* attention.rs:34-51 round_f16: round an f32 to the nearest f16 value (ties to even), keep f32. */
float orc_round_f16(float x) {
  uint32_t b;
  memcpy(&b, &x, 4);
  uint32_t sign = b & 0x80000000u, ab = b & 0x7fffffffu;
  if (ab >= 0x7f800000u) return x;
  int e = (int)(ab >> 23) - 127;
  if (e > 15) {
    uint32_t r = sign | 0x7f800000u;
    float f;
    memcpy(&f, &r, 4);
    return f;
  }
  int q_exp = e < -14 ? -24 : e - 10;
  uint32_t qb = (uint32_t)(q_exp + 127) << 23;
  float q, v;
  memcpy(&q, &qb, 4);
  memcpy(&v, &ab, 4);
  float r = nearbyintf(v / q) * q; /* default rounding mode: ties to even */
  uint32_t rb;
  memcpy(&rb, &r, 4);
  rb |= sign;
  memcpy(&r, &rb, 4);
  return r;
}

/* tensor.rs:25-43 dot_portable: four partial sums, (s0+s1)+(s2+s3)+tail */
static float dotf(const float* a, const float* b, int n) {
  float s0 = 0, s1 = 0, s2 = 0, s3 = 0, tail = 0;
  int c = n / 4;
  for (int i = 0; i < c; ++i) {
    int j = i * 4;
    s0 += a[j] * b[j];
    s1 += a[j + 1] * b[j + 1];
    s2 += a[j + 2] * b[j + 2];
    s3 += a[j + 3] * b[j + 3];
  }
  for (int j = c * 4; j < n; ++j) tail += a[j] * b[j];
  return (s0 + s1) + (s2 + s3) + tail;
}
/* tensor.rs:46-51 axpy */
static void axpyf(float alpha, const float* x, float* y, int n) {
  for (int i = 0; i < n; ++i) y[i] += alpha * x[i];
}
/* tensor.rs:122-143 */
static float sigmoidf_(float x) {
  if (x >= 0) return 1.0f / (1.0f + expf(-x));
  float e = expf(x);
  return e / (1.0f + e);
}
static float siluf(float x) { return x / (1.0f + expf(-x)); }
static float silu_gradf(float x) {
  float s = sigmoidf_(x);
  return s * (1.0f + x * (1.0f - s));
}

/* Mlp's activation, model.rs:113-134 */
void orc_swiglu(const float* g, const float* u, size_t n, float* h) {
  for (size_t i = 0; i < n; ++i) h[i] = siluf(g[i]) * u[i];
}
void orc_swiglu_backward(const float* g, const float* u, const float* dh, size_t n, float* dg, float* du) {
  for (size_t i = 0; i < n; ++i) {
    dg[i] = dh[i] * u[i] * silu_gradf(g[i]);
    du[i] = dh[i] * siluf(g[i]);
  }
}

/* ------------------------------------------------------------------ ggml block decode
 * Weight::dequant_row at the call sites src/rie.rs:97,123. */
size_t orc_row_bytes(int type, int cols) {
  switch (type) {
    case T_F32: return (size_t)cols * 4;
    case T_F16: case T_BF16: return (size_t)cols * 2;
    case T_Q4_0: return (size_t)cols / 32 * 18;
    case T_Q8_0: return (size_t)cols / 32 * 34;
    case T_Q4_K: return (size_t)cols / 256 * 144;
    case T_Q6_K: return (size_t)cols / 256 * 210;
  }
  return 0;
}
static uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

void orc_dequant_row(int type, const uint8_t* row, int cols, float* out) {
  switch (type) {
    case T_F32: memcpy(out, row, (size_t)cols * 4); break;
    case T_F16: for (int i = 0; i < cols; ++i) out[i] = f16_to_f32(rd16(row + 2 * i)); break;
    case T_BF16: for (int i = 0; i < cols; ++i) out[i] = bf16_to_f32(rd16(row + 2 * i)); break;
    case T_Q8_0:
      for (int b = 0; b < cols / 32; ++b) {
        const uint8_t* p = row + b * 34;
        float d = f16_to_f32(rd16(p));
        for (int i = 0; i < 32; ++i) out[b * 32 + i] = (float)(int8_t)p[2 + i] * d;
      }
      break;
    case T_Q4_0:
      for (int b = 0; b < cols / 32; ++b) {
        const uint8_t* p = row + b * 18;
        float d = f16_to_f32(rd16(p));
        for (int i = 0; i < 16; ++i) {
          out[b * 32 + i] = (float)((p[2 + i] & 15) - 8) * d;
          out[b * 32 + i + 16] = (float)((p[2 + i] >> 4) - 8) * d;
        }
      }
      break;
    case T_Q4_K:
      for (int b = 0; b < cols / 256; ++b) {
        const uint8_t* p = row + b * 144;
        float d = f16_to_f32(rd16(p)), dmin = f16_to_f32(rd16(p + 2));
        const uint8_t* sc = p + 4;
        const uint8_t* q = p + 16;
        float* y = out + b * 256;
        for (int j = 0; j < 8; ++j) {
          int s, m;
          if (j < 4) { s = sc[j] & 63; m = sc[j + 4] & 63; }
          else { s = (sc[j + 4] & 15) | ((sc[j - 4] >> 6) << 4); m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
          float dl = d * (float)s, ml = dmin * (float)m;
          const uint8_t* qq = q + (j / 2) * 32;
          for (int l = 0; l < 32; ++l) {
            int c = (j & 1) ? (qq[l] >> 4) : (qq[l] & 15);
            y[j * 32 + l] = dl * (float)c - ml;
          }
        }
      }
      break;
    case T_Q6_K:
      for (int b = 0; b < cols / 256; ++b) {
        const uint8_t* p = row + b * 210;
        const uint8_t* ql = p;
        const uint8_t* qh = p + 128;
        const int8_t* sc = (const int8_t*)(p + 192);
        float d = f16_to_f32(rd16(p + 208));
        float* y = out + b * 256;
        for (int h = 0; h < 2; ++h) {
          for (int l = 0; l < 32; ++l) {
            int is = l / 16;
            int q1 = (int)((ql[l] & 15) | (((qh[l] >> 0) & 3) << 4)) - 32;
            int q2 = (int)((ql[l + 32] & 15) | (((qh[l] >> 2) & 3) << 4)) - 32;
            int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            y[l] = d * (float)sc[is] * (float)q1;
            y[l + 32] = d * (float)sc[is + 2] * (float)q2;
            y[l + 64] = d * (float)sc[is + 4] * (float)q3;
            y[l + 96] = d * (float)sc[is + 6] * (float)q4;
          }
          y += 128; ql += 64; qh += 32; sc += 8;
        }
      }
      break;
  }
}

/* ------------------------------------------------------------------ frozen weight (frozen.rs:14-25) */
typedef struct {
  int type, rows, cols;
  const uint8_t* data; /* ggml rows, borrowed */
  size_t row_bytes;
} orc_frozen;

/* rie.rs:122-124 */
void orc_frozen_row(const orc_frozen* w, int r, float* out) {
  orc_dequant_row(w->type, w->data + (size_t)r * w->row_bytes, w->cols, out);
}

/* Mode (ii), "engine-like": rie.rs:77-80 hands x to QuantActs::prepare before kernels::matmul, i.e.
 * the engine rounds the activations to 8 bits per block before every QUANTISED forward matmul
 * (the backward is straight-through f32).  Which activation format formats_for picks per weight
 * type is not in the tree (rie-core is absent); this switch applies the two ggml conventions:
 * blocks of 32 (Q8_0-style: d = amax/127, round to nearest) for Q8_0 / Q4_0 weights, blocks of 256
 * (Q8_K-style: d = amax/127) for the K-quants.  Informative only: it bounds how much of the GPU
 * path's distance from the reference that rounding can explain.  Off by default (mode (i)). */
static int g_act_int8 = 0;
void orc_set_act_int8(int on) { g_act_int8 = on; }
static void round_acts_int8(const float* x, int n, int block, float* out) {
  for (int b = 0; b < n; b += block) {
    int len = n - b < block ? n - b : block;
    float amax = 0;
    for (int i = 0; i < len; ++i) { float a = fabsf(x[b + i]); amax = a > amax ? a : amax; }
    float d = amax / 127.0f, id = d > 0 ? 1.0f / d : 0.0f;
    for (int i = 0; i < len; ++i) out[b + i] = nearbyintf(x[b + i] * id) * d;
  }
}

/* rie.rs:74-82 forward: y[t x rows] = x[t x cols] . W^T from dequantised rows.  Mode (i) "smooth"
 * (the default) leaves x in f32, as the reference's own backward assumes; mode (ii) rounds it. */
void orc_frozen_forward(const orc_frozen* w, const float* x, int t, float* y) {
  const int R = w->rows, K = w->cols;
  float* xq = NULL;
  if (g_act_int8 && (w->type == T_Q8_0 || w->type == T_Q4_0 || w->type == T_Q4_K || w->type == T_Q6_K)) {
    const int block = (w->type == T_Q4_K || w->type == T_Q6_K) ? 256 : 32;
    xq = (float*)malloc((size_t)t * K * sizeof(float));
    for (int ti = 0; ti < t; ++ti) round_acts_int8(x + (size_t)ti * K, K, block, xq + (size_t)ti * K);
    x = xq;
  }
#pragma omp parallel
  {
    float* buf = (float*)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
    for (int r = 0; r < R; ++r) {
      orc_frozen_row(w, r, buf);
      for (int ti = 0; ti < t; ++ti) y[(size_t)ti * R + r] = dotf(x + (size_t)ti * K, buf, K);
    }
    free(buf);
  }
  free(xq);
}

/* rie.rs:84-120 backward_input: dx[t x cols] += dy[t x rows] . W, 32 rows dequantised at a time
 * (BWD_ROWS, rie.rs:64), per-thread accumulators, then summed. */
void orc_frozen_backward_input(const orc_frozen* w, const float* dy, int t, float* dx) {
  const int R = w->rows, K = w->cols, CH = 32;
  const int n_chunks = (R + CH - 1) / CH;
#pragma omp parallel
  {
    float* acc = (float*)calloc((size_t)t * K, sizeof(float));
    float* buf = (float*)malloc((size_t)CH * K * sizeof(float));
#pragma omp for schedule(static)
    for (int c = 0; c < n_chunks; ++c) {
      int r0 = c * CH, r1 = r0 + CH < R ? r0 + CH : R;
      for (int r = r0; r < r1; ++r) orc_frozen_row(w, r, buf + (size_t)(r - r0) * K);
      for (int ti = 0; ti < t; ++ti) {
        float* dxr = acc + (size_t)ti * K;
        for (int r = r0; r < r1; ++r) {
          float g = dy[(size_t)ti * R + r];
          if (g != 0.0f) axpyf(g, buf + (size_t)(r - r0) * K, dxr, K);
        }
      }
    }
#pragma omp critical
    for (size_t i = 0; i < (size_t)t * K; ++i) dx[i] += acc[i];
    free(acc);
    free(buf);
  }
}

/* ------------------------------------------------------------------ dense helpers (tensor.rs:63-120) */
static void matmul_nt(const float* a, const float* b, int m, int k, int n, float* out) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) out[(size_t)i * n + j] = dotf(a + (size_t)i * k, b + (size_t)j * k, k);
}
static void matmul_nn(const float* a, const float* b, int m, int k, int n, float* out) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i) {
    float* o = out + (size_t)i * n;
    for (int j = 0; j < n; ++j) o[j] = 0;
    for (int p = 0; p < k; ++p) {
      float av = a[(size_t)i * k + p];
      if (av != 0.0f) axpyf(av, b + (size_t)p * n, o, n);
    }
  }
}
/* out[m x n] += a[k x m]^T . b[k x n] */
static void matmul_tn_acc(float* out, const float* a, const float* b, int k, int m, int n) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i) {
    float* o = out + (size_t)i * n;
    for (int p = 0; p < k; ++p) {
      float av = a[(size_t)p * m + i];
      if (av != 0.0f) axpyf(av, b + (size_t)p * n, o, n);
    }
  }
}

/* ------------------------------------------------------------------ Linear + LoRA (linear.rs) */
typedef struct {
  orc_frozen w;
  const float* bias; /* or NULL */
  int rank;          /* 0 = no adapter */
  float alpha;
  float *a, *b, *ga, *gb; /* a [r x in], b [out x r] */
  int lora_enabled;
} orc_linear;

/* linear.rs:73-93 */
void orc_linear_forward(const orc_linear* l, const float* x, int t, float* y) {
  const int in = l->w.cols, out = l->w.rows;
  orc_frozen_forward(&l->w, x, t, y);
  if (l->bias)
    for (int i = 0; i < t; ++i)
      for (int j = 0; j < out; ++j) y[(size_t)i * out + j] += l->bias[j];
  if (l->rank > 0 && l->lora_enabled) {
    const int r = l->rank;
    float* h = (float*)malloc((size_t)t * r * sizeof(float));
    float* d = (float*)malloc((size_t)t * out * sizeof(float));
    matmul_nt(x, l->a, t, in, r, h);
    matmul_nt(h, l->b, t, r, out, d);
    const float s = l->alpha / (float)r;
    for (size_t i = 0; i < (size_t)t * out; ++i) y[i] += s * d[i];
    free(h);
    free(d);
  }
}

/* linear.rs:97-121: dx (fresh) = dy.W + g.A; gb += (s dy)^T h; ga += g^T x */
void orc_linear_backward(orc_linear* l, const float* x, const float* dy, int t, float* dx) {
  const int in = l->w.cols, out = l->w.rows;
  memset(dx, 0, (size_t)t * in * sizeof(float));
  orc_frozen_backward_input(&l->w, dy, t, dx);
  if (l->rank > 0 && l->lora_enabled) {
    const int r = l->rank;
    const float s = l->alpha / (float)r;
    float* h = (float*)malloc((size_t)t * r * sizeof(float));
    float* sdy = (float*)malloc((size_t)t * out * sizeof(float));
    float* g = (float*)malloc((size_t)t * r * sizeof(float));
    float* gx = (float*)malloc((size_t)t * in * sizeof(float));
    matmul_nt(x, l->a, t, in, r, h);
    for (size_t i = 0; i < (size_t)t * out; ++i) sdy[i] = dy[i] * s;
    matmul_tn_acc(l->gb, sdy, h, t, out, r);
    matmul_nn(sdy, l->b, t, out, r, g);
    matmul_tn_acc(l->ga, g, x, t, r, in);
    matmul_nn(g, l->a, t, r, in, gx);
    for (size_t i = 0; i < (size_t)t * in; ++i) dx[i] += gx[i];
    free(h);
    free(sdy);
    free(g);
    free(gx);
  }
}

/* ------------------------------------------------------------------ ops.rs */
/* ops.rs:8-35 rmsnorm_ordered (offset 0 on the GGUF path, rie.rs:227,247) */
void orc_rmsnorm(const float* x, const float* w, int rows, int d, float eps, int fused_scale, float* y, float* inv) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (size_t)r * d;
    float ms = dotf(xr, xr, d) / (float)d;
    float ir = 1.0f / sqrtf(ms + eps);
    if (inv) inv[r] = ir;
    if (fused_scale) for (int i = 0; i < d; ++i) y[(size_t)r * d + i] = xr[i] * (ir * w[i]);
    else for (int i = 0; i < d; ++i) y[(size_t)r * d + i] = xr[i] * ir * w[i];
  }
}
/* ops.rs:39-56 */
void orc_rmsnorm_backward(const float* x, const float* w, const float* inv, const float* dy, int rows, int d, float* dx) {
#pragma omp parallel
  {
    float* g = (float*)malloc((size_t)d * sizeof(float));
#pragma omp for schedule(static)
    for (int r = 0; r < rows; ++r) {
      const float* xr = x + (size_t)r * d;
      const float* dyr = dy + (size_t)r * d;
      for (int i = 0; i < d; ++i) g[i] = dyr[i] * w[i];
      float ir = inv[r];
      float c = dotf(g, xr, d) * ir * ir * ir / (float)d;
      for (int i = 0; i < d; ++i) dx[(size_t)r * d + i] = g[i] * ir - xr[i] * c;
    }
    free(g);
  }
}

/* ops.rs:112-154 Rope::at_positions: tables [t x rot/2] */
typedef struct {
  int rot_dim, neox, t;
  float *cos, *sin;
} orc_rope;

void orc_rope_init(orc_rope* r, const int* positions, int t, int rot_dim, int neox, float base, float freq_scale,
                   const float* factors, int n_factors) {
  int half = rot_dim / 2;
  r->rot_dim = rot_dim; r->neox = neox; r->t = t;
  r->cos = (float*)malloc((size_t)t * half * sizeof(float));
  r->sin = (float*)malloc((size_t)t * half * sizeof(float));
  float* inv_freq = (float*)malloc((size_t)half * sizeof(float));
  for (int i = 0; i < half; ++i) {
    float f = powf(base, -2.0f * (float)i / (float)rot_dim) * freq_scale;
    if (factors && i < n_factors && factors[i] != 0.0f) f /= factors[i];
    inv_freq[i] = f;
  }
  for (int p = 0; p < t; ++p)
    for (int i = 0; i < half; ++i) {
      float a = (float)positions[p] * inv_freq[i];
      r->cos[(size_t)p * half + i] = cosf(a);
      r->sin[(size_t)p * half + i] = sinf(a);
    }
  free(inv_freq);
}
void orc_rope_free(orc_rope* r) { free(r->cos); free(r->sin); }

/* ops.rs:168-184 */
void orc_rope_apply(const orc_rope* r, float* x, int t, int heads, int head_dim, int inverse) {
  int half = r->rot_dim / 2;
  float sgn = inverse ? -1.0f : 1.0f;
#pragma omp parallel for schedule(static)
  for (int p = 0; p < t; ++p)
    for (int h = 0; h < heads; ++h) {
      size_t base = ((size_t)p * heads + h) * head_dim;
      for (int i = 0; i < half; ++i) {
        float c = r->cos[(size_t)p * half + i], s = sgn * r->sin[(size_t)p * half + i];
        size_t a = r->neox ? base + i : base + 2 * i, b = r->neox ? base + i + half : base + 2 * i + 1;
        float x1 = x[a], x2 = x[b];
        x[a] = x1 * c - x2 * s;
        x[b] = x2 * c + x1 * s;
      }
    }
}

/* ops.rs:238-247 softmax_row: max-subtracted exp in f32, sum in f64; returns lse, writes probs */
float orc_softmax_row(const float* logits, int n, float* p) {
  float m = -INFINITY;
  for (int i = 0; i < n; ++i) m = logits[i] > m ? logits[i] : m;
  double s = 0;
  for (int i = 0; i < n; ++i) { p[i] = expf(logits[i] - m); s += (double)p[i]; }
  float inv = (float)(1.0 / s);
  for (int i = 0; i < n; ++i) p[i] *= inv;
  return m + (float)log(s);
}

/* ------------------------------------------------------------------ attention.rs */
typedef struct {
  int n_heads, n_kv_heads, head_dim, rot_dim;
  float rope_theta, rope_freq_scale, eps;
  int qk_norm, rope_neox, kv_f16;
  orc_linear q, k, v, o;
  const float *q_norm, *k_norm;
} orc_attn;

typedef struct {
  float *x, *q_raw, *k_raw, *q_inv, *k_inv, *q, *k, *v, *probs, *o;
} orc_attn_cache;

static float* falloc(size_t n) { return (float*)calloc(n ? n : 1, sizeof(float)); }

/* attention.rs:187-230: the scores, softmax and P.V of every head.  q [t x nh x hd], k, v
 * [t x nkv x hd]; probs [nh x t x t] (zero where masked); o [t x nh x hd] must come in zeroed. */
void orc_attn_core_forward(const float* q, const float* k, const float* v, int t, int nh, int nkv, int hd,
                           const int* seg_start, float* probs, float* o) {
  const float scale = 1.0f / sqrtf((float)hd);
  const int group = nh / nkv;
#pragma omp parallel for schedule(dynamic)
  for (int h = 0; h < nh; ++h) {
    int g = h / group;
    float* qs = (float*)malloc((size_t)hd * sizeof(float));
    for (int i = 0; i < t; ++i) {
      const float* qi = q + ((size_t)i * nh + h) * hd;
      for (int d = 0; d < hd; ++d) qs[d] = qi[d] * scale;
      float* row = probs + ((size_t)h * t + i) * t;
      float m = -INFINITY;
      int j0 = seg_start ? seg_start[i] : 0;
      for (int j = j0; j <= i; ++j) {
        row[j] = dotf(qs, k + ((size_t)j * nkv + g) * hd, hd);
        m = row[j] > m ? row[j] : m;
      }
      float s = 0;
      for (int j = j0; j <= i; ++j) { row[j] = expf(row[j] - m); s += row[j]; }
      float inv = 1.0f / s;
      float* oi = o + ((size_t)i * nh + h) * hd;
      for (int j = j0; j <= i; ++j) {
        row[j] *= inv;
        axpyf(row[j], v + ((size_t)j * nkv + g) * hd, oi, hd);
      }
    }
    free(qs);
  }
}

/* attention.rs:246-329: dq [t x nh x hd], dk, dv [t x nkv x hd] (all zeroed on entry) from d_o and
 * the forward's probabilities; the KV gradients are summed over the query heads of a group. */
void orc_attn_core_backward(const float* q, const float* k, const float* v, const float* probs, const float* d_o, int t,
                            int nh, int nkv, int hd, const int* seg_start, float* dq, float* dk, float* dv) {
  const float scale = 1.0f / sqrtf((float)hd);
  const int group = nh / nkv;
  float* dkh = falloc((size_t)nh * t * hd);
  float* dvh = falloc((size_t)nh * t * hd);
#pragma omp parallel for schedule(dynamic)
  for (int h = 0; h < nh; ++h) {
    int g = h / group;
    const float* p = probs + (size_t)h * t * t;
    float* dp = (float*)malloc((size_t)t * sizeof(float));
    float* dkl = dkh + (size_t)h * t * hd;
    float* dvl = dvh + (size_t)h * t * hd;
    for (int i = 0; i < t; ++i) {
      const float* doi = d_o + ((size_t)i * nh + h) * hd;
      int j0 = seg_start ? seg_start[i] : 0;
      float sum = 0;
      for (int j = j0; j <= i; ++j) {
        dp[j] = dotf(doi, v + ((size_t)j * nkv + g) * hd, hd);
        float pij = p[(size_t)i * t + j];
        sum += pij * dp[j];
        for (int d = 0; d < hd; ++d) dvl[(size_t)j * hd + d] += pij * doi[d];
      }
      const float* qi = q + ((size_t)i * nh + h) * hd;
      float* dqi = dq + ((size_t)i * nh + h) * hd;
      for (int j = j0; j <= i; ++j) {
        float ds = p[(size_t)i * t + j] * (dp[j] - sum) * scale;
        if (ds == 0.0f) continue;
        const float* kj = k + ((size_t)j * nkv + g) * hd;
        for (int d = 0; d < hd; ++d) dqi[d] += ds * kj[d];
        for (int d = 0; d < hd; ++d) dkl[(size_t)j * hd + d] += ds * qi[d];
      }
    }
    free(dp);
  }
  for (int h = 0; h < nh; ++h) { /* GQA: sum over the group, attention.rs:320-328 */
    int g = h / group;
    for (int i = 0; i < t; ++i)
      for (int d = 0; d < hd; ++d) {
        dk[((size_t)i * nkv + g) * hd + d] += dkh[((size_t)h * t + i) * hd + d];
        dv[((size_t)i * nkv + g) * hd + d] += dvh[((size_t)h * t + i) * hd + d];
      }
  }
  free(dkh);
  free(dvh);
}

/* attention.rs:162-244.  seg_start[i] = first position of the sequence token i belongs to:
 * the reference runs one sequence per call; a batch here is a concatenation of independent
 * sequences, token i attends to j in [seg_start[i], i]. */
void orc_attn_forward(const orc_attn* a, const float* x, int t, const orc_rope* rope, const int* seg_start,
                      float* y, orc_attn_cache* c) {
  const int nh = a->n_heads, nkv = a->n_kv_heads, hd = a->head_dim, hidden = a->q.w.cols;
  c->x = falloc((size_t)t * hidden);
  memcpy(c->x, x, (size_t)t * hidden * sizeof(float));
  c->q_raw = falloc((size_t)t * nh * hd);
  c->k_raw = falloc((size_t)t * nkv * hd);
  c->v = falloc((size_t)t * nkv * hd);
  orc_linear_forward(&a->q, x, t, c->q_raw);
  orc_linear_forward(&a->k, x, t, c->k_raw);
  orc_linear_forward(&a->v, x, t, c->v);
  c->q = falloc((size_t)t * nh * hd);
  c->k = falloc((size_t)t * nkv * hd);
  c->q_inv = falloc((size_t)t * nh);
  c->k_inv = falloc((size_t)t * nkv);
  if (a->qk_norm) {
    orc_rmsnorm(c->q_raw, a->q_norm, t * nh, hd, a->eps, 1, c->q, c->q_inv);
    orc_rmsnorm(c->k_raw, a->k_norm, t * nkv, hd, a->eps, 1, c->k, c->k_inv);
  } else {
    memcpy(c->q, c->q_raw, (size_t)t * nh * hd * sizeof(float));
    memcpy(c->k, c->k_raw, (size_t)t * nkv * hd * sizeof(float));
  }
  orc_rope_apply(rope, c->q, t, nh, hd, 0);
  orc_rope_apply(rope, c->k, t, nkv, hd, 0);
  if (a->kv_f16) {
    for (size_t i = 0; i < (size_t)t * nkv * hd; ++i) { c->k[i] = orc_round_f16(c->k[i]); c->v[i] = orc_round_f16(c->v[i]); }
  }
  c->probs = falloc((size_t)nh * t * t);
  c->o = falloc((size_t)t * nh * hd);
  orc_attn_core_forward(c->q, c->k, c->v, t, nh, nkv, hd, seg_start, c->probs, c->o);
  orc_linear_forward(&a->o, c->o, t, y);
}

void orc_attn_cache_free(orc_attn_cache* c) {
  free(c->x); free(c->q_raw); free(c->k_raw); free(c->q_inv); free(c->k_inv);
  free(c->q); free(c->k); free(c->v); free(c->probs); free(c->o);
}

/* attention.rs:246-367 */
void orc_attn_backward(orc_attn* a, orc_attn_cache* c, const float* dy, int t, const orc_rope* rope,
                       const int* seg_start, float* dx) {
  const int nh = a->n_heads, nkv = a->n_kv_heads, hd = a->head_dim, hidden = a->q.w.cols;
  float* d_o = falloc((size_t)t * nh * hd);
  orc_linear_backward(&a->o, c->o, dy, t, d_o);
  float* dq = falloc((size_t)t * nh * hd);
  float* dk = falloc((size_t)t * nkv * hd);
  float* dv = falloc((size_t)t * nkv * hd);
  orc_attn_core_backward(c->q, c->k, c->v, c->probs, d_o, t, nh, nkv, hd, seg_start, dq, dk, dv);
  orc_rope_apply(rope, dq, t, nh, hd, 1);
  orc_rope_apply(rope, dk, t, nkv, hd, 1);
  float *dq_raw = dq, *dk_raw = dk;
  if (a->qk_norm) {
    dq_raw = falloc((size_t)t * nh * hd);
    dk_raw = falloc((size_t)t * nkv * hd);
    orc_rmsnorm_backward(c->q_raw, a->q_norm, c->q_inv, dq, t * nh, hd, dq_raw);
    orc_rmsnorm_backward(c->k_raw, a->k_norm, c->k_inv, dk, t * nkv, hd, dk_raw);
  }
  float* dxk = falloc((size_t)t * hidden);
  float* dxv = falloc((size_t)t * hidden);
  orc_linear_backward(&a->q, c->x, dq_raw, t, dx);
  orc_linear_backward(&a->k, c->x, dk_raw, t, dxk);
  orc_linear_backward(&a->v, c->x, dv, t, dxv);
  for (size_t i = 0; i < (size_t)t * hidden; ++i) dx[i] += dxk[i] + dxv[i];
  if (a->qk_norm) { free(dq_raw); free(dk_raw); }
  free(dq); free(dk); free(dv); free(dxk); free(dxv); free(d_o);
}

/* ------------------------------------------------------------------ model.rs: Mlp, Block, Model */
typedef struct {
  orc_linear gate, up, down;
} orc_mlp;

typedef struct {
  const float *input_norm, *post_norm;
  orc_attn attn;
  orc_mlp mlp;
} orc_block;

typedef struct {
  float *x, *inv1, *n1, *h, *inv2, *n2, *g, *u, *hm;
  orc_attn_cache ac;
} orc_block_cache;

typedef struct {
  int vocab, hidden, ff, n_layers;
  float rms_eps;
  orc_frozen embed, lm_head;
  const float* final_norm;
  const float* rope_factors;
  int n_rope_factors;
  int checkpointing, logits_chunk;
  orc_block* blocks;
} orc_model;

/* model.rs:165-183 Block::forward (+ Mlp::forward model.rs:113-119) */
static void block_forward(const orc_block* b, const float* x, int t, int d, int ff, const orc_rope* rope,
                          const int* seg_start, float eps, float* y, orc_block_cache* c) {
  c->x = falloc((size_t)t * d);
  memcpy(c->x, x, (size_t)t * d * sizeof(float));
  c->inv1 = falloc(t); c->n1 = falloc((size_t)t * d);
  orc_rmsnorm(x, b->input_norm, t, d, eps, 0, c->n1, c->inv1);
  float* m = falloc((size_t)t * d);
  orc_attn_forward(&b->attn, c->n1, t, rope, seg_start, m, &c->ac);
  c->h = falloc((size_t)t * d);
  for (size_t i = 0; i < (size_t)t * d; ++i) c->h[i] = x[i] + m[i];
  c->inv2 = falloc(t); c->n2 = falloc((size_t)t * d);
  orc_rmsnorm(c->h, b->post_norm, t, d, eps, 0, c->n2, c->inv2);
  c->g = falloc((size_t)t * ff); c->u = falloc((size_t)t * ff); c->hm = falloc((size_t)t * ff);
  orc_linear_forward(&b->mlp.gate, c->n2, t, c->g);
  orc_linear_forward(&b->mlp.up, c->n2, t, c->u);
  orc_swiglu(c->g, c->u, (size_t)t * ff, c->hm);
  orc_linear_forward(&b->mlp.down, c->hm, t, m);
  for (size_t i = 0; i < (size_t)t * d; ++i) y[i] = c->h[i] + m[i];
  free(m);
}
static void block_cache_free(orc_block_cache* c) {
  free(c->x); free(c->inv1); free(c->n1); free(c->h); free(c->inv2); free(c->n2); free(c->g); free(c->u); free(c->hm);
  orc_attn_cache_free(&c->ac);
}
/* model.rs:185-197 Block::backward (+ Mlp::backward model.rs:120-134); dx may alias dy */
static void block_backward(orc_block* b, orc_block_cache* c, const float* dy, int t, int d, int ff, const orc_rope* rope,
                           const int* seg_start, float* dx) {
  float* dhm = falloc((size_t)t * ff);
  orc_linear_backward(&b->mlp.down, c->hm, dy, t, dhm);
  float* dg = falloc((size_t)t * ff);
  float* du = falloc((size_t)t * ff);
  orc_swiglu_backward(c->g, c->u, dhm, (size_t)t * ff, dg, du);
  float* dn2 = falloc((size_t)t * d);
  float* dxu = falloc((size_t)t * d);
  orc_linear_backward(&b->mlp.gate, c->n2, dg, t, dn2);
  orc_linear_backward(&b->mlp.up, c->n2, du, t, dxu);
  for (size_t i = 0; i < (size_t)t * d; ++i) dn2[i] += dxu[i];
  float* dh = falloc((size_t)t * d);
  orc_rmsnorm_backward(c->h, b->post_norm, c->inv2, dn2, t, d, dh);
  for (size_t i = 0; i < (size_t)t * d; ++i) dh[i] += dy[i];
  float* dn1 = falloc((size_t)t * d);
  orc_attn_backward(&b->attn, &c->ac, dh, t, rope, seg_start, dn1);
  float* dxn = falloc((size_t)t * d);
  orc_rmsnorm_backward(c->x, b->input_norm, c->inv1, dn1, t, d, dxn);
  for (size_t i = 0; i < (size_t)t * d; ++i) dx[i] = dh[i] + dxn[i];
  free(dhm); free(dg); free(du); free(dn2); free(dxu); free(dh); free(dn1); free(dxn);
}

/* model.rs:446-454 */
static void embed_tokens(const orc_model* m, const int* tokens, int t, float* x) {
  for (int i = 0; i < t; ++i) orc_frozen_row(&m->embed, tokens[i], x + (size_t)i * m->hidden);
}

/* model.rs:561-609 head: logp per target, optional gradient into dx (weights != NULL), hit count */
static int model_head(const orc_model* m, const float* x, int t, const int* tpos, const int* ttok, int n_targets,
                      const float* weights, float* logp, float* dx, float* logits_out) {
  const int d = m->hidden, v = m->vocab;
  int chunk = m->logits_chunk > 0 ? m->logits_chunk : 1, hits = 0;
  (void)t;
  float* xs = falloc((size_t)chunk * d);
  float* ns = falloc((size_t)chunk * d);
  float* inv = falloc(chunk);
  float* logits = falloc((size_t)chunk * v);
  float* dlogits = weights ? falloc((size_t)chunk * v) : NULL;
  float* dns = falloc((size_t)chunk * d);
  float* dxs = falloc((size_t)chunk * d);
  float* p = falloc(v);
  for (int c0 = 0; c0 < n_targets; c0 += chunk) {
    int n = n_targets - c0 < chunk ? n_targets - c0 : chunk;
    for (int i = 0; i < n; ++i) memcpy(xs + (size_t)i * d, x + (size_t)tpos[c0 + i] * d, (size_t)d * sizeof(float));
    orc_rmsnorm(xs, m->final_norm, n, d, m->rms_eps, 0, ns, inv);
    orc_frozen_forward(&m->lm_head, ns, n, logits);
    if (logits_out) memcpy(logits_out + (size_t)c0 * v, logits, (size_t)n * v * sizeof(float));
    for (int i = 0; i < n; ++i) {
      const float* row = logits + (size_t)i * v;
      float lse = orc_softmax_row(row, v, p);
      float tl = row[ttok[c0 + i]];
      logp[c0 + i] = tl - lse;
      int hit = 1;
      for (int j = 0; j < v; ++j) if (row[j] > tl) { hit = 0; break; }
      hits += hit;
      if (weights) {
        float wi = weights[c0 + i];
        float* dl = dlogits + (size_t)i * v;
        for (int j = 0; j < v; ++j) dl[j] = wi * p[j];
        dl[ttok[c0 + i]] -= wi;
      }
    }
    if (weights) {
      memset(dns, 0, (size_t)n * d * sizeof(float));
      orc_frozen_backward_input(&m->lm_head, dlogits, n, dns);
      orc_rmsnorm_backward(xs, m->final_norm, inv, dns, n, d, dxs);
      for (int i = 0; i < n; ++i)
        for (int j = 0; j < d; ++j) dx[(size_t)tpos[c0 + i] * d + j] += dxs[(size_t)i * d + j];
    }
  }
  free(xs); free(ns); free(inv); free(logits); free(dlogits); free(dns); free(dxs); free(p);
  return hits;
}

static void make_rope(const orc_model* m, int t, const int* seg_start, orc_rope* rope) {
  const orc_attn* a = &m->blocks[0].attn;
  int* pos = (int*)malloc((size_t)t * sizeof(int));
  for (int i = 0; i < t; ++i) pos[i] = seg_start ? i - seg_start[i] : i;
  orc_rope_init(rope, pos, t, a->rot_dim, a->rope_neox, a->rope_theta, a->rope_freq_scale, m->rope_factors,
                m->n_rope_factors);
  free(pos);
}

/* model.rs:644-687 forward_backward_layout for a concatenation of independent sequences.
 * Accumulates ga/gb of every adapter; writes logp per target; returns the hit count. */
int orc_model_forward_backward(orc_model* m, const int* tokens, int t, const int* seg_start, const int* tpos,
                               const int* ttok, const float* weights, int n_targets, float* logp) {
  const int d = m->hidden, ff = m->ff, L = m->n_layers;
  orc_rope rope;
  make_rope(m, t, seg_start, &rope);
  float* x = falloc((size_t)t * d);
  embed_tokens(m, tokens, t, x);
  float** inputs = (float**)calloc(L, sizeof(float*));
  orc_block_cache* caches = (orc_block_cache*)calloc(L, sizeof(orc_block_cache));
  float* y = falloc((size_t)t * d);
  for (int li = 0; li < L; ++li) {
    if (m->checkpointing) {
      inputs[li] = falloc((size_t)t * d);
      memcpy(inputs[li], x, (size_t)t * d * sizeof(float));
      orc_block_cache tmp;
      block_forward(&m->blocks[li], x, t, d, ff, &rope, seg_start, m->rms_eps, y, &tmp);
      block_cache_free(&tmp);
    } else {
      block_forward(&m->blocks[li], x, t, d, ff, &rope, seg_start, m->rms_eps, y, &caches[li]);
    }
    float* s = x; x = y; y = s;
  }
  float* dx = falloc((size_t)t * d);
  int hits = model_head(m, x, t, tpos, ttok, n_targets, weights, logp, dx, NULL);
  for (int li = L - 1; li >= 0; --li) {
    if (m->checkpointing) {
      block_forward(&m->blocks[li], inputs[li], t, d, ff, &rope, seg_start, m->rms_eps, y, &caches[li]);
      free(inputs[li]);
    }
    block_backward(&m->blocks[li], &caches[li], dx, t, d, ff, &rope, seg_start, dx);
    block_cache_free(&caches[li]);
  }
  free(inputs); free(caches); free(x); free(y); free(dx);
  orc_rope_free(&rope);
  return hits;
}

/* model.rs:494-557 forward only: logp (score) and optionally the logits rows (logits_at) */
int orc_model_score(const orc_model* m, const int* tokens, int t, const int* seg_start, const int* tpos,
                    const int* ttok, int n_targets, float* logp, float* logits_out) {
  const int d = m->hidden, ff = m->ff;
  orc_rope rope;
  make_rope(m, t, seg_start, &rope);
  float* x = falloc((size_t)t * d);
  float* y = falloc((size_t)t * d);
  embed_tokens(m, tokens, t, x);
  for (int li = 0; li < m->n_layers; ++li) {
    orc_block_cache tmp;
    block_forward(&m->blocks[li], x, t, d, ff, &rope, seg_start, m->rms_eps, y, &tmp);
    block_cache_free(&tmp);
    float* s = x; x = y; y = s;
  }
  int hits = model_head(m, x, t, tpos, ttok, n_targets, NULL, logp, NULL, logits_out);
  free(x); free(y);
  orc_rope_free(&rope);
  return hits;
}

/* ------------------------------------------------------------------ optim.rs */
/* optim.rs:73-90: f64 sum of squares over all ga, gb; scale if above max_norm; returns the norm */
float orc_clip_grad_norm(float** grads, const size_t* sizes, int n, float max_norm) {
  double ss = 0;
  for (int k = 0; k < n; ++k)
    for (size_t i = 0; i < sizes[k]; ++i) ss += (double)grads[k][i] * (double)grads[k][i];
  float norm = (float)sqrt(ss);
  if (max_norm > 0 && norm > max_norm) {
    float s = max_norm / (norm + 1e-6f);
    for (int k = 0; k < n; ++k)
      for (size_t i = 0; i < sizes[k]; ++i) grads[k][i] *= s;
  }
  return norm;
}
/* optim.rs:48-69 AdamW::step for one tensor; t is the 1-based step count */
void orc_adamw_step(float* p, const float* g, float* m, float* v, size_t n, int t, float lr, float beta1,
                    float beta2, float eps, float wd) {
  float bc1 = 1.0f - powf(beta1, (float)t), bc2 = 1.0f - powf(beta2, (float)t);
  for (size_t i = 0; i < n; ++i) {
    m[i] = beta1 * m[i] + (1.0f - beta1) * g[i];
    v[i] = beta2 * v[i] + (1.0f - beta2) * g[i] * g[i];
    float mh = m[i] / bc1, vh = v[i] / bc2;
    p[i] -= lr * (mh / (sqrtf(vh) + eps) + wd * p[i]);
  }
}
/* optim.rs:102-111 Schedule::lr */
float orc_schedule_lr(float peak, uint64_t warmup, uint64_t total, float min_ratio, uint64_t step) {
  if (warmup > 0 && step < warmup) return peak * (float)(step + 1) / (float)warmup;
  uint64_t span = total > warmup ? total - warmup : 0;
  if (span < 1) span = 1;
  uint64_t w = warmup < step ? warmup : step;
  float p = (float)(step - w) / (float)span;
  if (p > 1.0f) p = 1.0f;
  float c = 0.5f * (1.0f + cosf(3.14159265358979323846f * p));
  return peak * (min_ratio + (1.0f - min_ratio) * c);
}

/* ------------------------------------------------------------------ tensor.rs:155-199 Rng (SplitMix64) */
static uint64_t rng_next(uint64_t* st) {
  *st += 0x9E3779B97F4A7C15ull;
  uint64_t z = *st;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
uint64_t orc_rng_new(uint64_t seed) { return seed ^ 0x9E3779B97F4A7C15ull; }
uint64_t orc_rng_next_u64(uint64_t* st) { return rng_next(st); }
float orc_rng_uniform(uint64_t* st) { return (float)(rng_next(st) >> 40) / (float)(1ull << 24); }
float orc_rng_normal(uint64_t* st) {
  float u1 = orc_rng_uniform(st);
  if (u1 < 1e-12f) u1 = 1e-12f;
  float u2 = orc_rng_uniform(st);
  return sqrtf(-2.0f * logf(u1)) * cosf(2.0f * 3.14159265358979323846f * u2);
}
void orc_rng_fill_normal(uint64_t* st, float* out, size_t n, float std) {
  for (size_t i = 0; i < n; ++i) out[i] = orc_rng_normal(st) * std;
}
void orc_rng_fill_uniform_sym(uint64_t* st, float* out, size_t n, float bound) {
  for (size_t i = 0; i < n; ++i) out[i] = (orc_rng_uniform(st) * 2.0f - 1.0f) * bound;
}

/* ------------------------------------------------------------------ construction helpers for the ctypes wrapper */
orc_model* orc_model_new(int vocab, int hidden, int ff, int n_layers, float rms_eps) {
  orc_model* m = (orc_model*)calloc(1, sizeof(orc_model));
  m->vocab = vocab; m->hidden = hidden; m->ff = ff; m->n_layers = n_layers; m->rms_eps = rms_eps;
  m->checkpointing = 1; m->logits_chunk = 64;
  m->blocks = (orc_block*)calloc(n_layers, sizeof(orc_block));
  return m;
}
void orc_model_free(orc_model* m) { free(m->blocks); free(m); }
void orc_model_set_flags(orc_model* m, int checkpointing, int logits_chunk) { m->checkpointing = checkpointing; m->logits_chunk = logits_chunk; }
static void set_frozen(orc_frozen* f, int type, int rows, int cols, const void* data) {
  f->type = type; f->rows = rows; f->cols = cols; f->data = (const uint8_t*)data; f->row_bytes = orc_row_bytes(type, cols);
}
void orc_model_set_embed(orc_model* m, int type, const void* data) { set_frozen(&m->embed, type, m->vocab, m->hidden, data); }
void orc_model_set_lm_head(orc_model* m, int type, const void* data) { set_frozen(&m->lm_head, type, m->vocab, m->hidden, data); }
void orc_model_set_final_norm(orc_model* m, const float* w) { m->final_norm = w; }
void orc_model_set_rope_factors(orc_model* m, const float* f, int n) { m->rope_factors = f; m->n_rope_factors = n; }
void orc_model_set_attn(orc_model* m, int layer, int n_heads, int n_kv_heads, int head_dim, int rot_dim, float theta,
                        float freq_scale, int qk_norm, int neox, int kv_f16, const float* q_norm, const float* k_norm,
                        const float* input_norm, const float* post_norm) {
  orc_block* b = &m->blocks[layer];
  orc_attn* a = &b->attn;
  a->n_heads = n_heads; a->n_kv_heads = n_kv_heads; a->head_dim = head_dim; a->rot_dim = rot_dim;
  a->rope_theta = theta; a->rope_freq_scale = freq_scale; a->eps = m->rms_eps;
  a->qk_norm = qk_norm; a->rope_neox = neox; a->kv_f16 = kv_f16; a->q_norm = q_norm; a->k_norm = k_norm;
  b->input_norm = input_norm; b->post_norm = post_norm;
}
/* which: 0 q, 1 k, 2 v, 3 o, 4 gate, 5 up, 6 down (the order of Block::linears, model.rs:199-218) */
static orc_linear* pick(orc_model* m, int layer, int which) {
  orc_block* b = &m->blocks[layer];
  switch (which) {
    case 0: return &b->attn.q; case 1: return &b->attn.k; case 2: return &b->attn.v; case 3: return &b->attn.o;
    case 4: return &b->mlp.gate; case 5: return &b->mlp.up; default: return &b->mlp.down;
  }
}
void orc_model_set_linear(orc_model* m, int layer, int which, int type, int rows, int cols, const void* data, const float* bias) {
  orc_linear* l = pick(m, layer, which);
  set_frozen(&l->w, type, rows, cols, data);
  l->bias = bias; l->rank = 0; l->lora_enabled = 1;
}
void orc_model_set_lora(orc_model* m, int layer, int which, int rank, float alpha, float* a, float* b, float* ga, float* gb) {
  orc_linear* l = pick(m, layer, which);
  l->rank = rank; l->alpha = alpha; l->a = a; l->b = b; l->ga = ga; l->gb = gb;
}
void orc_model_set_lora_enabled(orc_model* m, int on) {
  for (int li = 0; li < m->n_layers; ++li) for (int w = 0; w < 7; ++w) pick(m, li, w)->lora_enabled = on;
}
/* standalone entry points over raw buffers (used by the unit parity tests) */
void orc_frozen_forward_raw(int type, int rows, int cols, const void* data, const float* x, int t, float* y) {
  orc_frozen f; set_frozen(&f, type, rows, cols, data); orc_frozen_forward(&f, x, t, y);
}
void orc_frozen_backward_input_raw(int type, int rows, int cols, const void* data, const float* dy, int t, float* dx) {
  orc_frozen f; set_frozen(&f, type, rows, cols, data); orc_frozen_backward_input(&f, dy, t, dx);
}
void orc_linear_forward_raw(int type, int rows, int cols, const void* data, const float* bias, int rank, float alpha,
                            const float* a, const float* b, const float* x, int t, float* y) {
  orc_linear l; memset(&l, 0, sizeof l); set_frozen(&l.w, type, rows, cols, data);
  l.bias = bias; l.rank = rank; l.alpha = alpha; l.a = (float*)a; l.b = (float*)b; l.lora_enabled = 1;
  orc_linear_forward(&l, x, t, y);
}
void orc_linear_backward_raw(int type, int rows, int cols, const void* data, int rank, float alpha, const float* a,
                             const float* b, float* ga, float* gb, const float* x, const float* dy, int t, float* dx) {
  orc_linear l; memset(&l, 0, sizeof l); set_frozen(&l.w, type, rows, cols, data);
  l.rank = rank; l.alpha = alpha; l.a = (float*)a; l.b = (float*)b; l.ga = ga; l.gb = gb; l.lora_enabled = 1;
  orc_linear_backward(&l, x, dy, t, dx);
}
/* A launcher may have exported OMP_NUM_THREADS=1 (torchrun does); the timed CPU baseline asks for
 * the host's cores itself. */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
