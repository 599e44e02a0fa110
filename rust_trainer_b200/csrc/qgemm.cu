// Frozen quantised matmul on tcgen05 tensor cores (sm_100a).
//
//   forward  (reference src/rie.rs:74-82,  RieFrozen::forward)        Y[M x N]  = X[M x K] . W^T
//   backward (reference src/rie.rs:84-120, RieFrozen::backward_input) dX[M x K] = dY[M x N] . W
//
// both read the SAME packed weight bytes (64x64 bricks of ggml codes, see qformat.cuh); no
// dequantised copy of W exists in global memory.  The weight is the UMMA "A" operand (128
// weight rows or columns per tile), the activations are the "B" operand (up to 256 tokens per
// tile), so the TMEM accumulator is the transposed output tile [128 x tokens].
//
// One persistent CTA per SM, warp-specialised (15 warps; roles by warp id, see the kernel):
//   producer : one thread issues the TMA tiles of activations (and of 16-bit weights), 128B swizzle
//   bricks   : one thread issues the bulk copies of packed bricks, running ahead in its own ring
//   MMA      : one thread issues tcgen05.mma (kind::f16, fp32 accumulate in TMEM)
//   unpack   : eight warps turn packed bricks into the f16 tile in the UMMA shared-memory layout
//              (forward reads it K-major, backward reads the same bytes MN-major)
//   epilogue : four warps tcgen05.ld the accumulator (double buffered: 2 x 256 TMEM columns),
//              add bias / per-token factors, stage and TMA-store f32, bf16 or f16
// The LoRA low-rank term is one more contraction chunk fed through the same accumulator.
#include "pdl.cuh"
#include "ptx.cuh"
#include "qformat.cuh"
#include "ctx.h"
#include <stdio.h>

namespace rt {

constexpr int W_STAGE = 16384;        // 128 x 64 x 16-bit
constexpr int RAW_STAGE = 2 * 4352;   // largest brick pair (Q8_0)
constexpr int QG_THREADS = 480;       // producer, MMA, 8 unpack, 4 epilogue warps, packed-brick producer

// Shared-memory plan of one CTA.  A CTA of a pair stages half of the token tile, so its stages
// are a third smaller, so four of them leave room for the deeper unpack pipeline.
template <bool PAIR>
struct QCfg {
#ifndef RT_B200_PAIR_NS
#define RT_B200_PAIR_NS 4
#endif
  static constexpr int NS = PAIR ? RT_B200_PAIR_NS : 3;    // activation / unpacked-weight stages
#ifndef RT_B200_PAIR_NR
#define RT_B200_PAIR_NR 4
#endif
  static constexpr int NR = PAIR ? RT_B200_PAIR_NR : 4;    // packed brick-pair stages
  // The eight unpack warps work as UG groups on alternate contraction steps.  Waits are by phase
  // parity, which is only sound while a waiter cannot run two phases ahead of its barrier:
  // UG <= NS keeps a group from reaching a stage before the use two back has been released, and
  // NR a multiple of UG gives every slot of the brick ring to one group (bulk copies of different
  // slots may land out of order, so a group sharing a slot could otherwise see the landing of an
  // older copy as its own).
#ifndef RT_B200_PAIR_UG
#define RT_B200_PAIR_UG 4
#endif
  static constexpr int UG = PAIR ? RT_B200_PAIR_UG : 2;    // a power of two
  static constexpr int UTG = 256 / UG;                     // threads per group
  static_assert(UG <= NS && NR % UG == 0, "unpack groups would alias barrier phases");
  static constexpr int ACT_STAGE = PAIR ? 16384 : 32768;   // 128 or 256 tokens x 64 x 16-bit
  static constexpr int OFF_W = NS * ACT_STAGE;
  static constexpr int OFF_RAW = OFF_W + NS * W_STAGE;
  static constexpr int OFF_OUT = OFF_RAW + NR * RAW_STAGE;
  // Epilogue staging per warp: blocks of [32 tokens x 32 features], 2 KB (16-bit) or 4 KB (f32).
  // (A pair kernel built with five operand stages, a measurement variant, keeps half as many.)
  static constexpr int OUT_WARP = (PAIR && (NS > 4 || NR > 4)) ? 4096 : 8192;
  static constexpr int OUT_BUFS16 = OUT_WARP / 2048, OUT_BUFS32 = OUT_WARP / 4096;
  static constexpr int OFF_BAR = OFF_OUT + 4 * OUT_WARP;
  static constexpr int N_BARS = 3 * NS + 2 * NR + 4;
  static constexpr int SMEM_BYTES = OFF_BAR + N_BARS * 8 + 16 + 1024;
};
static_assert(QCfg<true>::SMEM_BYTES <= 232448 && QCfg<false>::SMEM_BYTES <= 232448, "shared memory plan exceeds one SM");

struct KParams {
  const uint8_t* bricks;
  int brick_bytes, nbk, fmt;
  int act_f16;   // activations (and therefore the unpacked weight tile) are f16, else bf16
  int conv16;    // 16-bit weight whose type differs from the activations': 1 = f16->bf16, 2 = bf16->f16
  int dir, out_rows, M, TN;
  int n_main, lora_mmas;
  int n_splits, steps_per_split;  // split-K: work item = (tile, split); partial results go to `part`
  int b_mn;                       // token-contraction mode: the B operand is MN-major (tile rows = contraction)
  float* part;                    // [n_splits][M][out_rows] f32 partials when n_splits > 1 or b_mn
  int n_row_tiles, n_tok_tiles;    // a row tile is 128 weight rows, 256 for a CTA pair
  void* out;
  int out_dtype, accumulate, ld_out;
  const float* row_scale;  // optional per-token factor applied to the result
  const float* bias;
  uint32_t idesc_main, idesc_lora;
  int* status;
  int tma_out;  // the epilogue stages [32 tokens x 128] tiles in shared memory and writes them with TMA
  long long* prof;  // measurement aid (RT_B200_QPROF): per-CTA cycle counts of each role's waits, else null
  int dbg;  // measurement aid, only in builds with -DRT_B200_QPROF (RT_B200_DBG bit mask; the default build compiles every test of it out): 1 = epilogue skips its stores, 2 = unpack warps skip the conversion,
            // 16 = no operand loads at all: the MMAs run on whatever shared memory holds (results are garbage),
            // 32 = no MMAs are issued, 64 = no activation tiles are loaded, 128 = half of the MMAs of a step,
            // 256 = half of the unpack work of a step, 512 = no helpers for the last tile's epilogue,
            // 1024 = staged blocks are not stored, 2048 = blocks are stored without being staged,
            // 4096 = 16-bit outputs take the scalar staging path, 32768 = unpack units one after the other.  (There is deliberately no switch that
            // removes the MMA thread's operand waits while the loads run: without that back-pressure the
            // producers overrun the ring and the barriers' byte counts, and the launch faults.)
};

// Knock-out switches exist only in measurement builds: in the default build every test is the
// constant 0 and the branches vanish from the roles' loops (the MMA-issuing thread's included).
#ifdef RT_B200_QPROF
#define QDBG(p, m) (((p).dbg & (m)) != 0)
#else
#define QDBG(p, m) false
#endif

// ------------------------------------------------------------------ unpackers
__device__ __forceinline__ void store_chunk(uint8_t* dst, int r, int c, uint32_t a, uint32_t b, uint32_t c2,
                                            uint32_t d) {
  *(uint4*)(dst + r * 128 + ((c ^ (r & 7)) << 4)) = make_uint4(a, b, c2, d);
}
template <bool WBF16>
__device__ __forceinline__ uint32_t fin(__half2 h) {
  if (WBF16) {
    __nv_bfloat162 b = __float22bfloat162_rn(__half22float2(h));
    return *(uint32_t*)&b;
  }
  return *(uint32_t*)&h;
}
__device__ __forceinline__ __half2 u32_as_h2(uint32_t x) { return *(__half2*)&x; }

template <bool WBF16>
__device__ __forceinline__ void unpack_q4_0(const uint8_t* brick, int t, uint8_t* dst) {
  const uint4 q = *(const uint4*)(brick + t * 16);
  const __half2 d2 = __half2half2(((const __half*)(brick + 2048))[t]);
  const __half2 off = __floats2half2_rn(1032.f, 1032.f);  // 1024 (magic) + 8 (code bias)
  const int r = t >> 1, cb = (t & 1) * 4;
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t o[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      uint32_t x = ((w[j] >> (4 * p)) & 0x000F000Fu) | 0x64006400u;
      o[p] = fin<WBF16>(__hmul2(__hsub2(u32_as_h2(x), off), d2));
    }
    store_chunk(dst, r, cb + j, o[0], o[1], o[2], o[3]);
  }
}

template <bool WBF16>
__device__ __forceinline__ void unpack_q8_0(const uint8_t* brick, int t, uint8_t* dst) {
  // units are 32 bytes apart: lanes 4-7 of every eight fetch their halves in the other order, so
  // each 128-bit load of a quarter-warp touches every bank once
  const int swp = (t >> 2) & 1;
  const uint4 q0 = *(const uint4*)(brick + t * 32 + swp * 16);
  const uint4 q1 = *(const uint4*)(brick + t * 32 + (swp ^ 1) * 16);
  const uint4 qa = swp ? q1 : q0;
  const uint4 qb = swp ? q0 : q1;
  const __half2 d2 = __half2half2(((const __half*)(brick + 4096))[t]);
  const __half2 off = __floats2half2_rn(1152.f, 1152.f);  // 1024 (magic) + 128 (stored offset)
  const int r = t >> 1, cb = (t & 1) * 4;
  const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t o[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      uint32_t x = __byte_perm(w[2 * j + (p >> 1)], 0x64646464u, (p & 1) ? 0x4342 : 0x4140);
      o[p] = fin<WBF16>(__hmul2(__hsub2(u32_as_h2(x), off), d2));
    }
    store_chunk(dst, r, cb + j, o[0], o[1], o[2], o[3]);
  }
}

template <bool WBF16>
__device__ __forceinline__ void unpack_q4_k(const uint8_t* brick, int t, uint8_t* dst) {
  const uint4 q = *(const uint4*)(brick + t * 16);
  const __half2 dd = ((const __half2*)(brick + 2048))[t >> 1];
  const uchar2 sm = ((const uchar2*)(brick + 2304))[t];
  const float2 ddf = __half22float2(dd);
  // value = (d*sc)*q - dmin*m is a difference of like-sized terms: each factor is carried as an
  // f16 pair (hi + lo) so the only rounding that matters is the final one, relative to the value
  const float dscf = ddf.x * (float)sm.x, ndmf = -ddf.y * (float)sm.y;
  const __half dsc_h = __float2half_rn(dscf), ndm_h = __float2half_rn(ndmf);
  const __half2 dsc = __half2half2(dsc_h), ndm = __half2half2(ndm_h);
  const __half2 dsc_lo = __half2half2(__float2half_rn(dscf - __half2float(dsc_h)));
  const __half2 ndm_lo = __half2half2(__float2half_rn(ndmf - __half2float(ndm_h)));
  const __half2 off = __floats2half2_rn(1024.f, 1024.f);
  const int r = t >> 1, cb = (t & 1) * 4;
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t o[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      uint32_t x = ((w[j] >> (4 * p)) & 0x000F000Fu) | 0x64006400u;
      const __half2 qv = __hsub2(u32_as_h2(x), off);
      o[p] = fin<WBF16>(__hadd2(__hfma2(qv, dsc, ndm), __hfma2(qv, dsc_lo, ndm_lo)));
    }
    store_chunk(dst, r, cb + j, o[0], o[1], o[2], o[3]);
  }
}

template <bool WBF16>
__device__ __forceinline__ void unpack_q6_k(const uint8_t* brick, int t, uint8_t* dst) {
  const uint4 lo = *(const uint4*)(brick + t * 16);
  const uint2 hi = *(const uint2*)(brick + 2048 + t * 8);
  const char2 sc = ((const char2*)(brick + 3072))[t];
  const float d = __half2float(((const __half*)(brick + 3328))[t >> 1]);
  const __half2 ds0 = __half2half2(__float2half_rn(d * (float)sc.x));
  const __half2 ds1 = __half2half2(__float2half_rn(d * (float)sc.y));
  const __half2 off = __floats2half2_rn(1056.f, 1056.f);  // 1024 (magic) + 32 (code bias)
  const int r = t >> 1, cb = (t & 1) * 4;
  const uint32_t w[4] = {lo.x, lo.y, lo.z, lo.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t hw = (j < 2) ? hi.x : hi.y;
    if (j & 1) hw = __funnelshift_r(hw, hw, 8);
    const __half2 ds = (j < 2) ? ds0 : ds1;
    uint32_t o[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      uint32_t x = ((w[j] >> (4 * p)) & 0x000F000Fu) | ((hw >> (2 * p)) & 0x00300030u) | 0x64006400u;
      o[p] = fin<WBF16>(__hmul2(__hsub2(u32_as_h2(x), off), ds));
    }
    store_chunk(dst, r, cb + j, o[0], o[1], o[2], o[3]);
  }
}

// one brick (64 x 64 codes) -> one 8 KB half of the 16-bit weight tile; t = unit 0..127
template <bool WBF16>
__device__ __forceinline__ void unpack_brick(int fmt, const uint8_t* raw, int t, uint8_t* dst) {
  switch (fmt) {
    case GGML_Q4_0: unpack_q4_0<WBF16>(raw, t, dst); break;
    case GGML_Q8_0: unpack_q8_0<WBF16>(raw, t, dst); break;
    case GGML_Q4_K: unpack_q4_k<WBF16>(raw, t, dst); break;
    case GGML_Q6_K: unpack_q6_k<WBF16>(raw, t, dst); break;
  }
}

// NU units of one thread (unit u = tg + k * UTG of the 256 in a brick pair) with the format switch
// outside the unrolled loop: the compiler can then issue every unit's loads before the first convert.
template <int NU, int UTG>
__device__ __forceinline__ void unpack_units_f16(int fmt, const uint8_t* raw, int brick_bytes, int tg, uint8_t* dst) {
#define QG_UNITS(fn)                                                               \
  _Pragma("unroll") for (int k = 0; k < NU; ++k) {                                 \
    const int u = tg + k * UTG;                                                    \
    fn<false>(raw + (u >> 7) * brick_bytes, u & 127, dst + (u >> 7) * 8192);       \
  }
  switch (fmt) {
    case GGML_Q4_0: QG_UNITS(unpack_q4_0) break;
    case GGML_Q4_K: QG_UNITS(unpack_q4_k) break;
  }
#undef QG_UNITS
}

// ------------------------------------------------------------------ kernel
// PAIR = false: one CTA per output tile of 128 weight rows x TN tokens.
// PAIR = true : a cluster of two CTAs shares a tile of 256 weight rows x TN tokens.  Each CTA
//   holds its own 128 weight rows (unpacked by its own warps) and HALF of the token tile; the
//   leader CTA (cluster rank 0) issues tcgen05.mma.cta_group::2, which reads both CTAs' shared
//   memory and writes 128 accumulator rows into each CTA's TMEM.  Per CTA and per MMA cycle this
//   halves the activation bytes that TMA writes and the tensor core reads, and its smaller stages
//   leave room for four of them and four unpack groups.  Barriers that gate the MMA (full, w_ready, acc_empty)
//   live in the leader and are arrived on from both CTAs; barriers the MMA releases
//   (stage_empty, acc_full) exist in both CTAs and are signalled by one multicast commit.
// Build with -DRT_B200_QPROF to count, per CTA and role, the cycles spent in each wait (measurement aid).
#ifdef RT_B200_QPROF
#define QG_TIMED(slot, expr)                  \
  do {                                        \
    const long long t_ = clock64();           \
    expr;                                     \
    prof_acc[slot] += clock64() - t_;         \
  } while (0)
#define QG_PROF_BEGIN() long long prof_acc[6] = {0, 0, 0, 0, 0, 0}; const long long prof_t0 = clock64(); const uint64_t prof_ns0 = globaltimer_ns()
#define QG_PROF_END(role)                                                                  \
  do {                                                                                     \
    if (p.prof) {                                                                          \
      prof_acc[3] = clock64() - prof_t0;                                                   \
      if ((role) == 3) prof_acc[2] = (long long)(globaltimer_ns() - prof_ns0);             \
      for (int q_ = 0; q_ < 6; ++q_) p.prof[((size_t)blockIdx.x * 4 + (role)) * 6 + q_] = prof_acc[q_]; \
    }                                                                                      \
  } while (0)
#else
#define QG_TIMED(slot, expr) do { expr; } while (0)
#define QG_PROF_BEGIN() do { } while (0)
#define QG_PROF_END(role) do { } while (0)
#endif
template <bool PAIR>
__global__ void __launch_bounds__(QG_THREADS, 1)
qgemm_kernel(const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ CUtensorMap tm_w16,
             const __grid_constant__ CUtensorMap tm_lact, const __grid_constant__ CUtensorMap tm_lw,
             const __grid_constant__ CUtensorMap tm_out, const KParams p) {
  using C = QCfg<PAIR>;
  constexpr int NS = C::NS;
  constexpr int NR = C::NR;
  constexpr int UG = C::UG;
  constexpr int UTG = C::UTG;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sAct = smem;
  uint8_t* sW = smem + C::OFF_W;
  uint8_t* sRaw = smem + C::OFF_RAW;
  uint8_t* sOut = smem + C::OFF_OUT;
  uint64_t* bars = (uint64_t*)(smem + C::OFF_BAR);
  uint64_t* full = bars;                   // [NS] activations (+ TMA'd weight tile) landed      (leader's is used)
  uint64_t* w_ready = bars + NS;           // [NS] unpack warps done with the weight tile         (leader's is used)
  uint64_t* stage_empty = bars + 2 * NS;   // [NS] MMAs reading the stage have completed          (every CTA)
  uint64_t* raw_full = bars + 3 * NS;      // [NR]                                                (every CTA)
  uint64_t* raw_empty = raw_full + NR;     // [NR]
  uint64_t* acc_full = raw_empty + NR;     // [2]                                                 (every CTA)
  uint64_t* acc_empty = acc_full + 2;      // [2]                                                 (leader's is used)
  uint32_t* tmem_slot = (uint32_t*)(bars + C::N_BARS);
  pdl_launch_dependents();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef RT_B200_QPROF
#define QG_STAMP(i) do { if (p.prof && blockIdx.x == 0) p.prof[512 * 24 + (i)] = (long long)globaltimer_ns(); } while (0)
#else
#define QG_STAMP(i) do { } while (0)
#endif
#ifdef RT_B200_QPROF
#define QG_STEPSTAMP(kind, itv) do { if (p.prof && blockIdx.x == 0 && (itv) >= 16 && (itv) < 32) p.prof[512 * 24 + 16 + (kind) * 16 + ((itv) - 16)] = (long long)globaltimer_ns(); } while (0)
#else
#define QG_STEPSTAMP(kind, itv) do { } while (0)
#endif
  if (threadIdx.x == 0) QG_STAMP(0);
  // Roles by warp.  A warp runs on scheduler (warp % 4).  The MMA-issuing thread's instruction
  // latency sets the pace of the whole pipeline (every tcgen05.mma and commit goes through it), so
  // its scheduler (1) hosts only the two single-thread producers and one epilogue warp beside
  // it (the epilogue needs one warp per residue: a warp reads TMEM lanes 32 * (warp % 4) ..), and
  // the eight unpack warps share schedulers 0, 2 and 3 with the other epilogue warps.
  //   warp 1 MMA | 5 activation producer | 9 packed-brick producer | 0, 2, 3, 13 epilogue | rest unpack
  constexpr int R_PROD = 0, R_MMA = 1, R_UNPACK = 2, R_EPI = 3, R_RAW = 4;
  int role = R_UNPACK, uidx = 0;  // uidx: 0..7 among the unpack warps, neighbours on different schedulers
  switch (warp) {
    case 1: role = R_MMA; break;
    case 5: role = R_PROD; break;
    case 9: role = R_RAW; break;
    case 0: case 2: case 3: case 13: role = R_EPI; break;
    case 4: uidx = 0; break;
    case 6: uidx = 1; break;
    case 7: uidx = 2; break;
    case 8: uidx = 3; break;
    case 10: uidx = 4; break;
    case 11: uidx = 5; break;
    case 12: uidx = 6; break;
    default: uidx = 7; break;  // warp 14
  }
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;  // 0 = leader
  const int n_cta = PAIR ? 2 : 1;
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int n_workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int tn_cta = PAIR ? p.TN >> 1 : p.TN;  // token rows of the tile this CTA loads
  const bool is16 = fmt_is_16bit(p.fmt);
  const int n_tiles = p.n_row_tiles * p.n_tok_tiles;
  const int n_items = n_tiles * p.n_splits;
// work item -> tile, its range of contraction steps, and whether the LoRA chunk is appended
#define QG_ITEM_DECODE(item)                                                                  \
  const int tile = (item) % n_tiles, split = (item) / n_tiles;                                \
  const int s_begin = split * p.steps_per_split;                                              \
  const int s_main = min(p.n_main, s_begin + p.steps_per_split) - s_begin;                    \
  const int n_steps = s_main + ((p.lora_mmas > 0 && split == p.n_splits - 1) ? 1 : 0);        \
  (void)split
// first weight row (output feature) of this CTA's half of the tile, first token of the tile
#define QG_TILE_ORIGIN()                                                                      \
  const int r0 = (tile % p.n_row_tiles) * (128 * n_cta) + (int)rank * 128;                    \
  const int m0 = (tile / p.n_row_tiles) * p.TN

  if (threadIdx.x == 0) {
    for (int i = 0; i < NS; ++i) {
      // One barrier gates a step's MMAs: the producer's expect-tx arrival (with the bytes TMA brings)
      // plus one arrival per warp of the unpack group that owns the step, from every CTA of the pair.
      // Only the in-place 16-bit conversion needs the landing and the conversion told apart: then
      // the warps wait on `full` themselves and report on `w_ready`.
      mbar_init(&full[i], p.conv16 ? 1 : 1 + (8 / UG) * n_cta);
      mbar_init(&w_ready[i], (8 / UG) * n_cta);
      mbar_init(&stage_empty[i], 1);
    }
    for (int i = 0; i < NR; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], UTG); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4 * n_cta); }  // per epilogue warp
    mbar_fence_init();
    prefetch_tmap(&tm_act);
    prefetch_tmap(&tm_w16);
    prefetch_tmap(&tm_lact);
    prefetch_tmap(&tm_lw);
    if (p.tma_out) prefetch_tmap(&tm_out);
  }
  if (warp == 1) {
    if (PAIR) { tmem_alloc_pair(tmem_slot, 512); tmem_relinquish_pair(); }
    else { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  }
  tc_fence_before();
  __syncwarp();
  if (PAIR) cluster_sync_all();  // both CTAs' barriers are initialised and both hold their TMEM columns
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *(volatile uint32_t*)tmem_slot;
  // barriers, TMEM and descriptors are set up; from here on the kernel reads what its predecessor wrote
  pdl_wait();
  if (threadIdx.x == 0) QG_STAMP(1);

  // One [32 tokens x 32 features] block of an accumulator -> staging -> TMA store / reduce-add.
  // Transposes through shared memory (lane = output feature, register j = token); `stage_base`
  // is 8 KB private to the calling warp: two f32 blocks or four 16-bit ones, a block is reused
  // only after the store issued (nbuf) chunks ago has read it.
  auto tma_chunk = [&](int acc, int wq, int c, int r0, int m0, float bias_v, uint8_t* stage_base, uint32_t& cnt) {
    const bool wide = p.out_dtype == OUT_F32;
    const int buf = wide ? (int)(cnt % C::OUT_BUFS32) : (int)(cnt % C::OUT_BUFS16);
    ++cnt;
    uint8_t* stage = stage_base + buf * (wide ? 4096 : 2048);
    const uint32_t tcol = tmem_base + acc * 256 + ((uint32_t)(wq * 32) << 16) + c * 32;
    if (!wide && !QDBG(p, 4096)) {
      // 16-bit output: the accumulator block arrives in mma-fragment layout (a thread holds two
      // neighbouring tokens of one feature), is rounded to pairs and written with transposing
      // matrix stores into a [32 tokens][32 features] block of 64-byte rows, 16-byte units
      // XOR-swizzled by (token / 2) % 4 as the output map's 64-byte swizzle expects.
      uint32_t v[2][16];
      tmem_ld_16x256b_x4(tcol, v[0]);
      tmem_ld_16x256b_x4(tcol + (16u << 16), v[1]);
      float2 rs[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int tok = m0 + c * 32 + 8 * k + 2 * (lane & 3);
        rs[k] = make_float2(1.f, 1.f);
        if (p.row_scale) {
          rs[k].x = tok < p.M ? p.row_scale[tok] : 0.f;
          rs[k].y = tok + 1 < p.M ? p.row_scale[tok + 1] : 0.f;
        }
      }
      float bv[4] = {0.f, 0.f, 0.f, 0.f};  // features 16h + lane/4 + 8e -> bv[2h + e]
      if (p.bias) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = r0 + wq * 32 + 8 * e + (lane >> 2);
          bv[e] = row < p.out_rows ? p.bias[row] : 0.f;
        }
      }
      if (lane == 0) bulk_wait_group_read<C::OUT_BUFS16 - 1>();
      tmem_ld_wait();
      __syncwarp();
      uint32_t pk[2][8];  // [h][2k + e]: tokens 8k.., features 16h + 8e..
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int k = 0; k < 4; ++k)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float lo = __uint_as_float(v[h][4 * k + 2 * e]) * rs[k].x + bv[2 * h + e];
            const float hi = __uint_as_float(v[h][4 * k + 2 * e + 1]) * rs[k].y + bv[2 * h + e];
            if (p.out_dtype == OUT_BF16) { __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi); pk[h][2 * k + e] = *(uint32_t*)&b; }
            else { __half2 b = __floats2half2_rn(lo, hi); pk[h][2 * k + e] = *(uint32_t*)&b; }
          }
      // matrix mi = lane / 8 of a store: tokens 8(2kp + mi/2).., feature unit 2h + (mi & 1); this lane addresses row lane % 8
      const uint32_t sbase = smem_u32(stage);
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int kp = 0; kp < 2; ++kp) {
          const int mi = lane >> 3;
          const int tok = 8 * (2 * kp + (mi >> 1)) + (lane & 7);
          const int unit = 2 * h + (mi & 1);
          const uint32_t addr = sbase + tok * 64 + ((unit ^ ((tok >> 1) & 3)) << 4);
          stmatrix_x4_trans(addr, pk[h][4 * kp], pk[h][4 * kp + 1], pk[h][4 * kp + 2], pk[h][4 * kp + 3]);
        }
    } else {
      uint32_t v[32];
      tmem_ld32(tcol, v);
      tmem_ld_wait();
      if (lane == 0) {
        if (wide) bulk_wait_group_read<C::OUT_BUFS32 - 1>();
        else bulk_wait_group_read<C::OUT_BUFS16 - 1>();
      }
      // this chunk's 32 per-token factors: one coalesced load, handed round by shuffles
      float rs_lane = 1.0f;
      if (p.row_scale) { const int tok = m0 + c * 32 + lane; rs_lane = tok < p.M ? p.row_scale[tok] : 0.f; }
      __syncwarp();
      if (!QDBG(p, 2048)) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float val = __uint_as_float(v[j]);
          if (p.row_scale) val *= __shfl_sync(0xffffffffu, rs_lane, j);
          val += bias_v;
          if (p.out_dtype == OUT_F32) ((float*)stage)[j * 32 + lane] = val;
          else if (p.out_dtype == OUT_BF16) ((__nv_bfloat16*)stage)[j * 32 + lane] = __float2bfloat16_rn(val);
          else ((__half*)stage)[j * 32 + lane] = __float2half_rn(val);
        }
      }
    }
    if (!QDBG(p, 8)) fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0 && !QDBG(p, 1024)) {
      if (p.accumulate) tma_reduce_add_2d(&tm_out, r0 + wq * 32, m0 + c * 32, stage);
      else tma_store_2d(&tm_out, r0 + wq * 32, m0 + c * 32, stage);
      bulk_commit_group();
    }
  };
  // The epilogue of a CTA's LAST tile has nothing to hide behind, so the warps whose own work
  // is over by then help: every warp with residue q (mod 4) may read TMEM lane quarter q.
  // Quarter q's blocks go round-robin over its epilogue warp (turn 0) and its helpers (turns
  // 1..): residues 0 and 2 have three unpack warps each, residue 3 two, residue 1 the two
  // producer warps.  Helpers stage in the operand stages, which are idle once the last
  // accumulator is complete.
  const int n_my = worker < n_items ? (n_items - worker + n_workers - 1) / n_workers : 0;
  const bool tail_help = p.tma_out && n_my > 0 && !QDBG(p, (1 | 512));
  const int q_res = warp & 3;
  const int q_turns = (q_res == 0 || q_res == 2) ? 4 : 3;  // epilogue warp + helpers of this residue
  auto tail_helper = [&](int turn, int hslot) {
    if (!tail_help) return;
    const int tc_last = n_my - 1, item = worker + tc_last * n_workers;
    QG_ITEM_DECODE(item);
    (void)s_begin; (void)n_steps; (void)s_main;
    QG_TILE_ORIGIN();
    const int acc = tc_last & 1;
    if (!mbar_wait(&acc_full[acc], (uint32_t)((tc_last >> 1) & 1), p.status, 402)) return;
    tc_fence_after();
    const int row = r0 + q_res * 32 + lane;
    const float bias_v = (p.bias != nullptr && row < p.out_rows) ? p.bias[row] : 0.f;
    uint32_t cnt = 0;
    for (int c = turn; c < p.TN / 32; c += q_turns) tma_chunk(acc, q_res, c, r0, m0, bias_v, smem + hslot * 8192, cnt);
    if (lane == 0) bulk_wait_group_read<0>();  // staging may go once read; the writes land by the end of the grid
  };

  if (role == R_PROD) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      QG_PROF_BEGIN();
      for (int item = worker; item < n_items && ok && !QDBG(p, 16); item += n_workers) {
        QG_ITEM_DECODE(item);
        QG_TILE_ORIGIN();
        const int m_cta = m0 + (int)rank * tn_cta;  // this CTA's half of the tokens
        for (int si = 0; si < n_steps && ok; ++si, ++it) {
          const int s = s_begin + si;
          const int st = it % NS;
          const uint32_t ph = (it / NS) & 1;
          { bool w_; QG_TIMED(0, w_ = mbar_wait(&stage_empty[st], ph ^ 1, p.status, 101)); if (!w_) { ok = false; break; } }
          const bool lora = si >= s_main;
          uint8_t* a_dst = sAct + st * C::ACT_STAGE;
          uint8_t* w_dst = sW + st * W_STAGE;
          // the leader's barrier counts the bytes both CTAs will bring
          if (rank == 0)
            mbar_expect_tx(&full[st], (QDBG(p, 64) ? 0u : (uint32_t)p.TN * 128u) + ((is16 || lora) ? (uint32_t)(W_STAGE * n_cta) : 0u));
          const uint32_t fbar = PAIR ? mapa_u32(smem_u32(&full[st]), 0) : 0u;
          auto load2d = [&](void* dst, const CUtensorMap* map, int x, int y) {
            if (PAIR) tma_load_2d_pair(dst, map, x, y, fbar);
            else tma_load_2d(dst, map, x, y, &full[st]);
          };
          if (!lora) {
            if (QDBG(p, 64)) {
            } else if (p.b_mn) load2d(a_dst, &tm_act, 0, s * 64);  // [64 contraction rows x 64]
            else load2d(a_dst, &tm_act, s * 64, m_cta);
            if (is16) {
              if (p.dir == QG_FWD) {
                load2d(w_dst, &tm_w16, s * 64, r0);
                load2d(w_dst + 8192, &tm_w16, s * 64, r0 + 64);
              } else {
                load2d(w_dst, &tm_w16, r0, s * 64);
                load2d(w_dst + 8192, &tm_w16, r0 + 64, s * 64);
              }
            }
          } else {
            load2d(a_dst, &tm_lact, 0, m_cta);
            if (p.dir == QG_FWD) {
              load2d(w_dst, &tm_lw, 0, r0);
              load2d(w_dst + 8192, &tm_lw, 0, r0 + 64);
            } else {
              load2d(w_dst, &tm_lw, r0, 0);
              load2d(w_dst + 8192, &tm_lw, r0 + 64, 0);
            }
          }
        }
      }
      QG_PROF_END(0);
    }
    __syncwarp();
    tail_helper(warp >> 2, warp - 4);
  } else if (role == R_MMA) {
    // ------------------------------------------------------------ MMA issue (the leader's thread only)
    if (lane == 0 && rank == 0) {
      uint32_t tcount = 0, itg = 0;
      bool it_first = true;
      int st = 0;        // stage ring position and its phase, advanced without divisions
      uint32_t ph = 0;
      bool ok = true;
      // Descriptors: the high words are fixed for the launch, the low words are address >> 4 plus
      // the leading-dimension field; a stage or a K step of 16 only adds a constant to them.
      const uint64_t a_d0 = (p.dir == QG_FWD) ? umma_desc_sw128(smem_u32(sW), 16, 1024) : umma_desc_sw128(smem_u32(sW), 8192, 1024);
      const uint64_t b_d0 = p.b_mn ? umma_desc_sw128(smem_u32(sAct), 8192, 1024) : umma_desc_sw128(smem_u32(sAct), 16, 1024);
      const uint32_t a_hi = (uint32_t)(a_d0 >> 32), b_hi = (uint32_t)(b_d0 >> 32);
      const uint32_t a_k = (p.dir == QG_FWD) ? (32u >> 4) : (2048u >> 4);  // low-word step per K = 16
      const uint32_t b_k = p.b_mn ? (2048u >> 4) : (32u >> 4);
      QG_PROF_BEGIN();
      for (int item = worker; item < n_items && ok; item += n_workers, ++tcount) {
        QG_ITEM_DECODE(item);
        (void)tile; (void)s_begin;
        const int acc = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        { bool w_; QG_TIMED(0, w_ = mbar_wait<false>(&acc_empty[acc], aph ^ 1, p.status, 301)); if (!w_) { ok = false; break; } }
        tc_fence_after();
#ifdef RT_B200_QPROF
        if (p.prof && blockIdx.x == 0 && tcount < 8) p.prof[512 * 24 + 8 + tcount] = (long long)globaltimer_ns();
#endif
        const uint32_t d_tmem = tmem_base + acc * 256;
        for (int s = 0; s < n_steps; ++s) {
          if (!QDBG(p, 16)) {
            { bool w_; QG_TIMED(1, w_ = mbar_wait<false>(&full[st], ph, p.status, 302)); if (!w_) { ok = false; break; } }
            QG_STEPSTAMP(5, itg);
            if (p.conv16) { bool w_; QG_TIMED(2, w_ = mbar_wait<false>(&w_ready[st], ph, p.status, 303)); if (!w_) { ok = false; break; } }
          }
          tc_fence_after();  // (measured free: the step time is the same without it)
          QG_STEPSTAMP(0, itg);
          const uint32_t a_lo = (uint32_t)a_d0 + (uint32_t)st * (W_STAGE >> 4);
          const uint32_t b_lo = (uint32_t)b_d0 + (uint32_t)st * (C::ACT_STAGE >> 4);
          if (it_first) { QG_STAMP(2); it_first = false; }
          if (QDBG(p, 32)) {
          } else if (s < s_main) {
            QG_TIMED(4, {
            umma_f16_split<PAIR>(d_tmem, a_lo, a_hi, b_lo, b_hi, p.idesc_main, (uint32_t)(s != 0));
            umma_f16_split<PAIR>(d_tmem, a_lo + a_k, a_hi, b_lo + b_k, b_hi, p.idesc_main, 1u);
            if (!QDBG(p, 128)) {
              umma_f16_split<PAIR>(d_tmem, a_lo + 2 * a_k, a_hi, b_lo + 2 * b_k, b_hi, p.idesc_main, 1u);
              umma_f16_split<PAIR>(d_tmem, a_lo + 3 * a_k, a_hi, b_lo + 3 * b_k, b_hi, p.idesc_main, 1u);
            }
            });
          } else {
            for (int kk = 0; kk < p.lora_mmas; ++kk)
              umma_f16_split<PAIR>(d_tmem, a_lo + kk * a_k, a_hi, b_lo + kk * b_k, b_hi, p.idesc_lora, (uint32_t)((s | kk) != 0));
          }
          QG_TIMED(5, {
          if (PAIR) umma_commit_pair(&stage_empty[st], 3);
          else umma_commit(&stage_empty[st]);
          });
          QG_STEPSTAMP(1, itg);
          ++itg;
          if (++st == NS) { st = 0; ph ^= 1; }
        }
        if (ok) {
          if (PAIR) umma_commit_pair(&acc_full[acc], 3);
          else umma_commit(&acc_full[acc]);
        }
      }
      QG_STAMP(3);
      QG_PROF_END(1);
    }
  } else if (role == R_UNPACK) {
    // ------------------------------------------------------------ unpack
    // One pass over a weight tile (load codes, convert, store, fence, arrive) is a chain of
    // dependent shared-memory operations: its latency, not its instruction count, sets the pace.
    // The eight warps therefore work as UG groups on alternate contraction steps, so UG passes
    // are in flight at a time.
    const int t = uidx * 32 + lane;
    const int grp = t / UTG, tg = t % UTG;
    uint32_t it = 0, rit = 0;
    bool ok = true;
    QG_PROF_BEGIN();
    for (int item = worker; item < n_items && ok && !QDBG(p, 16); item += n_workers) {
      QG_ITEM_DECODE(item);
      (void)tile; (void)s_begin;
      for (int s = 0; s < n_steps; ++s, ++it) {
        const bool packed_step = !is16 && s < s_main;
        if ((int)(it & (UG - 1)) != grp) {  // another group's step: only keep the ring positions in step
          if (packed_step) ++rit;
          continue;
        }
        const int st = it % NS;
        const uint32_t ph = (it / NS) & 1;
        { bool w_; QG_TIMED(0, w_ = mbar_wait(&stage_empty[st], ph ^ 1, p.status, 201)); if (!w_) { ok = false; break; } }
        if (tg == 0) QG_STEPSTAMP(2, it);
        if (!PAIR && is16 && p.conv16 && s < s_main) {
          // The TMA'd 16-bit weight tile has the other 16-bit type: convert it in place
          // (element-wise, so the swizzled placement is untouched).  Single-CTA kernel only.
          if (!mbar_wait(&full[st], ph, p.status, 203)) { ok = false; break; }
          uint4* tile = (uint4*)(sW + st * W_STAGE);
#pragma unroll
          for (int i = 0; i < 1024 / UTG; ++i) {
            uint4 v = tile[tg + i * UTG];
            uint32_t* w = (uint32_t*)&v;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (p.conv16 == 1) {
                __nv_bfloat162 b = __float22bfloat162_rn(__half22float2(*(__half2*)&w[j]));
                w[j] = *(uint32_t*)&b;
              } else {
                __half2 h = __float22half2_rn(__bfloat1622float2(*(__nv_bfloat162*)&w[j]));
                w[j] = *(uint32_t*)&h;
              }
            }
            tile[tg + i * UTG] = v;
          }
          fence_proxy_async_smem();
        } else if (packed_step) {
          const int rs = rit % NR;
          const uint32_t rph = (rit / NR) & 1;
          { bool w_; QG_TIMED(1, w_ = mbar_wait(&raw_full[rs], rph, p.status, 202)); if (!w_) { ok = false; break; } }
          if (tg == 0) QG_STEPSTAMP(3, it);
          const uint8_t* raw = sRaw + rs * RAW_STAGE;
          uint8_t* dst = sW + st * W_STAGE;
          QG_TIMED(2, {
            if (!QDBG(p, 2)) {
              // 256 units (two bricks of 128) per tile; unit u: brick u >> 7 fills the 8 KB half u >> 7
              if (QDBG(p, (256 | 32768)) || !p.act_f16 || (p.fmt != GGML_Q4_0 && p.fmt != GGML_Q4_K)) {
                for (int u = tg; u < (QDBG(p, 256) ? 128 : 256); u += UTG) {
                  if (p.act_f16) unpack_brick<false>(p.fmt, raw + (u >> 7) * p.brick_bytes, u & 127, dst + (u >> 7) * 8192);
                  else unpack_brick<true>(p.fmt, raw + (u >> 7) * p.brick_bytes, u & 127, dst + (u >> 7) * 8192);
                }
              } else {
                // f16 tiles of the 4-bit formats: the format switch outside a fully unrolled loop, so
                // the loads of a thread's 256 / UTG units are in flight together (measured: Q4_K
                // forward +9 %, Q4_0 +1 %; Q8_0 loses 4-10 % that way and Q6_K gains nothing, so
                // they keep the unit-by-unit loop)
                (unpack_units_f16<256 / UTG, UTG>(p.fmt, raw, p.brick_bytes, tg, dst));
              }
            }
            if (!QDBG(p, 4)) fence_proxy_async_smem();
          });
          mbar_arrive(&raw_empty[rs]);
          ++rit;
        }
        // one arrival per warp, after every lane's writes are fenced towards the tensor core's reads
        __syncwarp();
        if (lane == 0) {
          uint64_t* ready = p.conv16 ? &w_ready[st] : &full[st];
          if (PAIR) mbar_arrive_cluster(mapa_u32(smem_u32(ready), 0));
          else mbar_arrive(ready);
        }
        if (tg == 0) QG_STEPSTAMP(4, it);
      }
    }
    if (t == 0) QG_PROF_END(2);
    tail_helper(warp >> 2, warp - 4);
  } else if (role == R_RAW) {
    // ------------------------------------------------------------ packed-brick producer
    // Runs ahead of the stage ring: a brick pair is fetched as soon as its slot in the raw ring
    // is free, so its latency is not added to the time a weight stage is held.
    if (lane == 0 && !is16 && !QDBG(p, 16)) {
      uint32_t rit = 0;
      bool ok = true;
      QG_PROF_BEGIN();
      const uint32_t bb = (uint32_t)p.brick_bytes;
      for (int item = worker; item < n_items && ok; item += n_workers) {
        QG_ITEM_DECODE(item);
        (void)n_steps;
        QG_TILE_ORIGIN();
        (void)m0;
        const int tr2 = (r0 >> 6);
        for (int si = 0; si < s_main; ++si, ++rit) {
          const int s = s_begin + si;
          const int rs = rit % NR;
          const uint32_t rph = (rit / NR) & 1;
          { bool w_; QG_TIMED(1, w_ = mbar_wait(&raw_empty[rs], rph ^ 1, p.status, 102)); if (!w_) { ok = false; break; } }
          mbar_expect_tx(&raw_full[rs], 2 * bb);
          const uint8_t *b0, *b1;
          if (p.dir == QG_FWD) {
            b0 = p.bricks + ((size_t)tr2 * p.nbk + s) * bb;
            b1 = p.bricks + ((size_t)(tr2 + 1) * p.nbk + s) * bb;
          } else {
            b0 = p.bricks + ((size_t)s * p.nbk + tr2) * bb;
            b1 = b0 + bb;
          }
          bulk_load_1d(sRaw + rs * RAW_STAGE, b0, bb, &raw_full[rs]);
          bulk_load_1d(sRaw + rs * RAW_STAGE + bb, b1, bb, &raw_full[rs]);
        }
      }
    }
    __syncwarp();
    tail_helper(warp >> 2, warp - 4);
  } else {
    // ------------------------------------------------------------ epilogue
    const int wq = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t tcount = 0, out_chunk = 0;
    bool ok = true;
    QG_PROF_BEGIN();
    for (int item = worker; item < n_items && ok; item += n_workers, ++tcount) {
      QG_ITEM_DECODE(item);
      (void)s_begin; (void)n_steps; (void)s_main;
      QG_TILE_ORIGIN();
      const int acc = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      { bool w_; QG_TIMED(0, w_ = mbar_wait(&acc_full[acc], aph, p.status, 401)); if (!w_) { ok = false; break; } }
      tc_fence_after();
      const int row = r0 + wq * 32 + lane;
      const bool row_ok = row < p.out_rows;
      const float bias_v = (p.bias != nullptr && row_ok) ? p.bias[row] : 0.f;
      for (int c = 0; c < p.TN / 32; ++c) {
        if (p.tma_out && !QDBG(p, 1)) {
          if (tail_help && (int)tcount == n_my - 1 && (c % q_turns) != 0) continue;  // a helper's block
          tma_chunk(acc, wq, c, r0, m0, bias_v, sOut + wq * C::OUT_WARP, out_chunk);
          continue;
        }
        uint32_t v[32];
        tmem_ld32(tmem_base + acc * 256 + ((uint32_t)(wq * 32) << 16) + c * 32, v);
        tmem_ld_wait();
        if (row_ok && !QDBG(p, 1)) {
          if (p.part != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int tok = m0 + c * 32 + j;
              if (tok < p.M) p.part[((size_t)split * p.M + tok) * p.out_rows + row] = __uint_as_float(v[j]);
            }
          } else {
            const size_t base = (size_t)(m0 + c * 32) * p.ld_out + row;
            const int nvalid = min(32, p.M - (m0 + c * 32));
            float old[32];
            if (p.accumulate) {
              // all loads first: a load-add-store chain per element would serialise on memory latency
              const float* o = (const float*)p.out + base;
#pragma unroll
              for (int j = 0; j < 32; ++j) old[j] = j < nvalid ? o[(size_t)j * p.ld_out] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j < nvalid) {
                float val = __uint_as_float(v[j]);
                if (p.row_scale) val *= p.row_scale[m0 + c * 32 + j];
                val += bias_v;
                if (p.accumulate) val += old[j];
                const size_t idx = base + (size_t)j * p.ld_out;
                if (p.out_dtype == OUT_F32) ((float*)p.out)[idx] = val;
                else if (p.out_dtype == OUT_BF16) ((__nv_bfloat16*)p.out)[idx] = __float2bfloat16_rn(val);
                else ((__half*)p.out)[idx] = __float2half_rn(val);
              }
            }
          }
        }
      }
      // the accumulator buffer is free once every epilogue warp of every CTA has read its lanes
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(mapa_u32(smem_u32(&acc_empty[acc]), 0));
        else mbar_arrive(&acc_empty[acc]);
      }
    }
    if (p.tma_out && lane == 0) bulk_wait_group_read<0>();  // staging may go once read; the writes land by the end of the grid
    if (warp == 0 && lane == 0) { QG_STAMP(4); QG_PROF_END(3); }
  }

  // ---------------------------------------------------------------- teardown
  if (*(volatile int*)p.status != 0) {
    // A wait gave up somewhere: give copies already in flight time to land before smem goes away.
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncwarp();
  // a CTA of a pair must not leave while its partner may still signal its barriers or read its memory
  if (PAIR) cluster_sync_all();
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 32) QG_STAMP(5);
}

// Sums split-K partials in split order (deterministic) and applies the epilogue the fused path
// would have applied: per-token scale, scalar factor, bias, accumulate.  Output is f32 at
// out[tok * s_tok + row * s_row].
__global__ void splitk_reduce_kernel(const float* __restrict__ part, int splits, int M, int R, float* __restrict__ out,
                                     size_t s_tok, size_t s_row, const float* __restrict__ row_scale,
                                     const float* __restrict__ alpha_dev, const float* __restrict__ bias,
                                     int accumulate) {
  pdl_entry();
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t n = (size_t)M * R;
  if (e >= n) return;
  const int tok = (int)(e / R), row = (int)(e % R);
  float v = 0.f;
  for (int k = 0; k < splits; ++k) v += part[(size_t)k * n + e];
  if (row_scale) v *= row_scale[tok];
  if (alpha_dev) v *= alpha_dev[0];
  if (bias) v += bias[row];
  float* o = out + tok * s_tok + row * s_row;
  if (accumulate) v += *o;
  *o = v;
}

// ------------------------------------------------------------------ host side
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static PFN_encodeTiled g_encode = nullptr;

size_t qgemm_smem_bytes() { return QCfg<true>::SMEM_BYTES > QCfg<false>::SMEM_BYTES ? QCfg<true>::SMEM_BYTES : QCfg<false>::SMEM_BYTES; }

// how many CTA pairs the device runs at once (0: the pair kernel is not used)
static int g_pair_workers = -1;

int qgemm_init() {
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn)
      return RT_ERR_CUDA;
    g_encode = (PFN_encodeTiled)fn;
  }
  if (cudaFuncSetAttribute(qgemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, QCfg<false>::SMEM_BYTES) !=
          cudaSuccess ||
      cudaFuncSetAttribute(qgemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, QCfg<true>::SMEM_BYTES) !=
          cudaSuccess)
    return RT_ERR_CUDA;
  if (g_pair_workers < 0) {
    int dev = 0, sms = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3((unsigned)(sms & ~1));
    cfg.blockDim = dim3(QG_THREADS);
    cfg.dynamicSmemBytes = QCfg<true>::SMEM_BYTES;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&n, qgemm_kernel<true>, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    const char* e = getenv("RT_B200_NO_PAIR");
    g_pair_workers = (e && atoi(e)) ? 0 : n;
  }
  return RT_OK;
}

// 2-D row-major 16-bit matrix [rows x cols]; box = box_cols x box_rows, 128-byte swizzle.
static int encode_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols,
                      uint32_t box_rows, bool is_bf16, uint64_t ld = 0) {
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {(ld ? ld : cols) * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(m, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? RT_OK : RT_ERR_CUDA;
}

std::atomic<unsigned long long> g_launch_count{0};

static int make_map_cached(rt_ctx* ctx, CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols,
                           uint32_t box_rows, bool is_bf16, uint64_t ld = 0) {
  if (ld == cols) ld = 0;
  if (!ctx) return encode_map(m, base, rows, cols, box_cols, box_rows, is_bf16, ld);  // no cache: nothing is allocated
  auto key = std::make_tuple(base, rows, cols | (ld << 32), box_cols, box_rows, is_bf16);
  auto it = ctx->tmap_cache.find(key);
  if (it != ctx->tmap_cache.end()) {
    *m = it->second;
    return RT_OK;
  }
  int rc = encode_map(m, base, rows, cols, box_cols, box_rows, is_bf16, ld);
  if (rc) return rc;
  if (ctx->tmap_cache.size() > 8192) ctx->tmap_cache.clear();
  ctx->tmap_cache.emplace(key, *m);
  return RT_OK;
}
#define make_map(m, ...) make_map_cached(a.fixed_part ? nullptr : ctx, m, __VA_ARGS__)

int tensor_map_f16_2d(rt_ctx* ctx, CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols,
                      uint32_t box_rows) {
  if (!g_encode) {
    int rc = qgemm_init();
    if (rc) return rc;
  }
  return make_map_cached(ctx, m, base, rows, cols, box_cols, box_rows, false);
}

int tensor_map_f16_2d_ld(rt_ctx* ctx, CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                         uint32_t box_cols, uint32_t box_rows) {
  if (!g_encode) {
    int rc = qgemm_init();
    if (rc) return rc;
  }
  return make_map_cached(ctx, m, base, rows, cols, box_cols, box_rows, false, ld);
}

// Output matrix [rows x cols] of f32 / bf16 / f16 with a row pitch of `ld` elements; box = 32 columns x 32 rows
// (one epilogue warp's block), no swizzle (the epilogue writes the staging block row-major).
static int make_out_map(rt_ctx* ctx, CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, int dtype,
                        bool swizzle64) {
  auto key = std::make_tuple(base, rows, cols | (ld << 32), 32u, 32u | ((uint32_t)dtype << 8) | (swizzle64 ? 1u << 16 : 0u), true);
  if (ctx) {
    auto it = ctx->tmap_cache.find(key);
    if (it != ctx->tmap_cache.end()) {
      *m = it->second;
      return RT_OK;
    }
  }
  const uint64_t es = dtype == OUT_F32 ? 4 : 2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * es};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = dtype == OUT_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : dtype == OUT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = g_encode(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return RT_ERR_CUDA;
  if (!ctx) return RT_OK;
  if (ctx->tmap_cache.size() > 8192) ctx->tmap_cache.clear();
  ctx->tmap_cache.emplace(key, *m);
  return RT_OK;
}

int qgemm_launch(rt_ctx* ctx, const QWeight& w, const QGemmArgs& a) {
  int* status_dev = ctx->status_dev;
  const int num_sms = ctx->num_sms;
  cudaStream_t st = ctx->stream;
  if (!g_encode) {
    int rc = qgemm_init();
    if (rc) return rc;
  }
  if (a.M <= 0) return RT_OK;
  const bool is16 = fmt_is_16bit(w.fmt);
  const int contract = a.dir == QG_FWD ? w.cols : w.rows;
  const int out_rows = a.dir == QG_FWD ? w.rows : w.cols;
  if ((!a.tok_mode && contract % 8 != 0) || (is16 && w.cols % 8 != 0)) return RT_ERR_BAD_SHAPE;
  if (a.tok_mode && (!is16 || a.dir != QG_BWD || a.M > 64 || a.lora.rank > 0 || a.out_dtype != OUT_F32)) return RT_ERR_BAD_ARG;
  if (a.accumulate && a.out_dtype != OUT_F32) return RT_ERR_BAD_ARG;
  if (a.lora.rank > 64 || (a.lora.rank > 0 && (!a.lora.act || !a.lora.w))) return RT_ERR_BAD_ARG;

  KParams p;
  p.bricks = w.bricks;
  p.brick_bytes = fmt_brick_bytes(w.fmt);
  p.nbk = w.nbk;
  p.fmt = w.fmt;
  p.act_f16 = a.act_f16 ? 1 : 0;
  p.conv16 = (w.fmt == GGML_F16 && !a.act_f16) ? 1 : (w.fmt == GGML_BF16 && a.act_f16) ? 2 : 0;
  p.row_scale = a.row_scale;
  p.dir = a.dir;
  p.out_rows = out_rows;
  p.M = a.M;
  p.TN = a.M > 128 ? 256 : a.M > 64 ? 128 : a.M > 32 ? 64 : 32;
  // a single 128-row weight tile (the skinny LoRA products): narrow token tiles spread the work over more SMs
  if (out_rows <= 128 && a.M > 64) p.TN = 64;
  if (a.tok_mode) p.TN = 64;
  if (p.TN == 256 && !a.tok_mode) {
    // pick the token-tile width that wastes the least of the last wave of the persistent grid
    const int row_tiles = (out_rows + 127) / 128;
    long best_cost = -1;
    for (int tn = 256; tn >= 128; tn -= 32) {
      const long tiles = (long)row_tiles * ((a.M + tn - 1) / tn);
      const long rounds = (tiles + num_sms - 1) / num_sms;
      const long cost = rounds * (tn + 40);  // + a per-tile fixed cost, in token units
      if (best_cost < 0 || cost < best_cost) { best_cost = cost; p.TN = tn; }
    }
  }
#ifdef RT_B200_QPROF
  static int tn_force = -1;
  if (tn_force < 0) { const char* e = getenv("RT_B200_TN"); tn_force = e ? atoi(e) : 0; }
  if (tn_force > 0 && p.TN >= 128 && !a.tok_mode) p.TN = tn_force;
#endif
  p.n_main = (contract + 63) / 64;
  p.lora_mmas = a.lora.rank > 0 ? (a.lora.rank + 15) / 16 : 0;
  p.n_row_tiles = (out_rows + 127) / 128;
  p.n_tok_tiles = (a.M + p.TN - 1) / p.TN;
  p.out = a.out;
  p.out_dtype = a.out_dtype;
  p.accumulate = a.accumulate;
  p.ld_out = a.ld_out > 0 ? a.ld_out : out_rows;
  p.bias = a.dir == QG_FWD ? a.bias : nullptr;
  // tcgen05.mma kind::f16 needs A and B of ONE 16-bit type (f16 x bf16 is an illegal instruction).
  const int ab_fmt = a.act_f16 ? 0 : 1;
  p.idesc_main = umma_idesc(ab_fmt, ab_fmt, a.dir == QG_BWD ? 1 : 0, 0, 128, p.TN);
  p.idesc_lora = p.idesc_main;
  p.status = status_dev;
  p.prof = nullptr;
#ifdef RT_B200_QPROF
  static long long* prof_dev = nullptr;
  if (!prof_dev) cudaMalloc(&prof_dev, (512 * 24 + 16 + 96) * sizeof(long long));
  cudaMemsetAsync(prof_dev, 0, (512 * 24 + 16 + 96) * sizeof(long long), st);
  p.prof = prof_dev;
#endif
  p.dbg = 0;
#ifdef RT_B200_QPROF
  {
    static int dbg = -1;
    if (dbg < 0) { const char* e = getenv("RT_B200_DBG"); dbg = e ? atoi(e) : 0; }
    p.dbg = dbg;
  }
#endif

  if (a.tok_mode) p.idesc_main = p.idesc_lora = umma_idesc(ab_fmt, ab_fmt, 1, 1, 128, 64);
  CUtensorMap tm_act, tm_w16, tm_lact, tm_lw;
  int rc = a.tok_mode ? make_map(&tm_act, a.act, (uint64_t)contract, 64, 64, 64, !a.act_f16)
                      : make_map(&tm_act, a.act, (uint64_t)a.M, (uint64_t)contract, 64, (uint32_t)p.TN, !a.act_f16);
  if (rc) return rc;
  tm_w16 = tm_act;
  tm_lact = tm_act;
  tm_lw = tm_act;
  if (is16) {
    rc = make_map(&tm_w16, w.dense16, (uint64_t)w.rows, (uint64_t)w.cols, 64, 64, w.fmt == GGML_BF16);
    if (rc) return rc;
  }
  if (a.lora.rank > 0) {
    rc = make_map(&tm_lact, a.lora.act, (uint64_t)a.M, 64, 64, (uint32_t)p.TN, !a.act_f16);
    if (rc) return rc;
    if (a.dir == QG_FWD) rc = make_map(&tm_lw, a.lora.w, (uint64_t)w.rows, 64, 64, 64, !a.act_f16);
    else rc = make_map(&tm_lw, a.lora.w, (uint64_t)a.lora.rank, (uint64_t)w.cols, 64, 64, !a.act_f16);
    if (rc) return rc;
  }
  int n_tiles = p.n_row_tiles * p.n_tok_tiles;
  // How the contraction is cut into accumulation chains depends on the weight's shape ONLY, never
  // on the number of tokens: the tensor core's accumulator does not round to nearest, so two
  // partitions of one sum differ by a few 1e-6 relative, which the next 16-bit rounding of the
  // activations amplifies a hundredfold.  With a token-dependent split-K a sequence's result
  // depended on its batch mates (a shard of one or two sequences against the whole batch: 7e-4
  // on the gradients); with a fixed partition it is bit-identical in any batch.
  // A very long contraction (the head's backward runs over the whole vocabulary) is accumulated
  // in pieces of a FIXED 8192 elements whose f32 partial sums are added afterwards: the error of
  // one chain grows with its length (about 3e-4 relative over 150 000 elements).
  p.steps_per_split = p.n_main;
  if (!a.tok_mode && a.out_dtype == OUT_F32 && p.n_main > 256) p.steps_per_split = 128;
  if (a.tok_mode) {
    int splits = num_sms / (n_tiles > 0 ? n_tiles : 1);
    if (splits > p.n_main / 4) splits = p.n_main / 4;
    if (splits < 1) splits = 1;
    p.steps_per_split = (p.n_main + splits - 1) / splits;
  }
  p.n_splits = (p.n_main + p.steps_per_split - 1) / p.steps_per_split;
  p.b_mn = a.tok_mode ? 1 : 0;
  // CTA pairs: 256 weight rows per tile, each CTA stages half of the tokens.  Needs whole pairs of
  // row tiles; the other shapes keep the single-CTA kernel.
  const bool pair = g_pair_workers > 0 && !a.tok_mode && !p.conv16 && p.n_splits == 1 && a.M > 128 &&
                    out_rows % 256 == 0;
  if (pair) {
    p.n_row_tiles = out_rows / 256;
    long best_cost = -1;
    for (int tn = 256; tn >= 128; tn -= 32) {
      const long tiles = (long)p.n_row_tiles * ((a.M + tn - 1) / tn);
      const long rounds = (tiles + g_pair_workers - 1) / g_pair_workers;
      const long cost = rounds * (tn + 40);
      if (best_cost < 0 || cost < best_cost) { best_cost = cost; p.TN = tn; }
    }
#ifdef RT_B200_QPROF
    if (tn_force > 0) p.TN = tn_force;
#endif
    p.n_tok_tiles = (a.M + p.TN - 1) / p.TN;
    n_tiles = p.n_row_tiles * p.n_tok_tiles;
    p.idesc_main = p.idesc_lora = umma_idesc(ab_fmt, ab_fmt, a.dir == QG_BWD ? 1 : 0, 0, 256, p.TN);
    // each CTA fetches its half of the token tile
    rc = make_map(&tm_act, a.act, (uint64_t)a.M, (uint64_t)contract, 64, (uint32_t)(p.TN / 2), !a.act_f16);
    if (rc) return rc;
    if (!is16) tm_w16 = tm_act;
    if (a.lora.rank > 0) {
      rc = make_map(&tm_lact, a.lora.act, (uint64_t)a.M, 64, 64, (uint32_t)(p.TN / 2), !a.act_f16);
      if (rc) return rc;
    } else {
      tm_lact = tm_act;
      tm_lw = tm_act;
    }
  }
  p.part = nullptr;
  if (p.n_splits > 1 || a.tok_mode) {
    const size_t need = (size_t)p.n_splits * a.M * out_rows;
    if (a.fixed_part) {
      if (need > a.fixed_part_floats) return RT_ERR_TOO_LARGE;
      p.part = a.fixed_part;
    } else {
      p.part = (float*)ctx->get_scratch(3, need * sizeof(float));
      if (!p.part) return RT_ERR_CUDA;
    }
  }
  // TMA-store epilogue whenever the output is TMA-addressable (16-byte aligned base and row pitch)
  CUtensorMap tm_out = tm_act;
  p.tma_out = 0;
  {
    const uint64_t es = a.out_dtype == OUT_F32 ? 4 : 2;
    if (!p.part && ((uintptr_t)a.out % 16 == 0) && ((uint64_t)p.ld_out * es) % 16 == 0) {
      rc = make_out_map(a.fixed_part ? nullptr : ctx, &tm_out, a.out, (uint64_t)a.M, (uint64_t)out_rows, (uint64_t)p.ld_out, a.out_dtype,
                        a.out_dtype != OUT_F32 && !QDBG(p, 4096));
      if (rc) return rc;
      p.tma_out = 1;
    }
  }
  const int n_items = n_tiles * p.n_splits;
  int workers = pair ? g_pair_workers : num_sms;
#ifdef RT_B200_QPROF
  {
    static int lim = -1;
    if (lim < 0) { const char* e = getenv("RT_B200_WORKERS"); lim = e ? atoi(e) : 0; }
    if (lim > 0 && lim < workers) workers = lim;  // measurement aid: fewer CTAs (pairs) than the device holds
  }
#endif
  const int grid = (n_items < workers ? n_items : workers) * (pair ? 2 : 1);
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (ctx->profiling && !a.fixed_part) {
    if (ctx->prof_used + 2 > ctx->prof_events.size()) {
      for (int i = 0; i < 256; ++i) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess) return RT_ERR_CUDA;
        ctx->prof_events.push_back(e);
      }
    }
    e0 = ctx->prof_events[ctx->prof_used++];
    e1 = ctx->prof_events[ctx->prof_used++];
    cudaEventRecord(e0, st);
  }
  if (pair) {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(QG_THREADS);
    cfg.dynamicSmemBytes = QCfg<true>::SMEM_BYTES;
    cfg.stream = st;
    cfg.attrs = at;
    cfg.numAttrs = 2;
    if (cudaLaunchKernelEx(&cfg, qgemm_kernel<true>, tm_act, tm_w16, tm_lact, tm_lw, tm_out, p) != cudaSuccess)
      return RT_ERR_CUDA;
  } else {
    pdl(qgemm_kernel<false>, grid, QG_THREADS, QCfg<false>::SMEM_BYTES, st)(tm_act, tm_w16, tm_lact, tm_lw, tm_out, p);
  }
  RT_COUNT_LAUNCH(1);
#ifdef RT_B200_QPROF
  {
    static long long host[512 * 24 + 16 + 96];
    cudaMemcpyAsync(host, prof_dev, sizeof(host), cudaMemcpyDeviceToHost, st);
    cudaStreamSynchronize(st);
    {
      const long long* t = host + 512 * 24;
      fprintf(stderr, "qstamp CTA0 ns from entry: init %lld first_mma %lld last_mma_issue %lld epilogue_done %lld exit %lld\n",
              t[1] - t[0], t[2] - t[0], t[3] - t[0], t[4] - t[0], t[5] - t[0]);
      const long long* u = host + 512 * 24 + 16;
      for (int i = 4; i < 12; ++i)
        fprintf(stderr, "qstep %d: unpack wake %lld raw %lld done %lld | mma full %lld ready %lld commit %lld   (ns after commit of step %d: wake %lld, ready-done %lld)\n",
                16 + i, u[32 + i] - t[0], u[48 + i] - t[0], u[64 + i] - t[0], u[80 + i] - t[0], u[i] - t[0], u[16 + i] - t[0], 16 + i - 4,
                u[32 + i] - u[16 + i - 4], u[i] - u[64 + i]);
      fprintf(stderr, "qstamp tile starts:");
      for (int i = 0; i < 8; ++i) if (t[8 + i]) fprintf(stderr, " %lld", t[8 + i] - t[0]);
      fprintf(stderr, "\n");
    }
    double sum[24] = {0};
    for (int c = 0; c < grid; ++c)
      for (int q = 0; q < 24; ++q) sum[q] += (double)host[c * 24 + q] / ((q >= 6 && q < 12 && pair) ? grid / 2 : grid);
    fprintf(stderr, "qprof pair=%d dir=%d TN=%d grid=%d | prod: stage_empty %.0f total %.0f | mma: acc_empty %.0f full %.0f w_ready %.0f issue4 %.0f commit %.0f total %.0f | unpack: stage_empty %.0f raw_full %.0f work %.0f total %.0f | epi: acc_full %.0f total %.0f = %.0f ns -> %.0f MHz\n",
            (int)pair, a.dir, p.TN, grid, sum[0], sum[3], sum[6], sum[7], sum[8], sum[10], sum[11], sum[9], sum[12], sum[13], sum[14], sum[15], sum[18], sum[21], sum[20], sum[21] / sum[20] * 1e3);
  }
#endif
  if (p.part) {
    const size_t n = (size_t)a.M * out_rows;
    const size_t s_tok = a.tok_mode ? a.out_s_tok : (size_t)p.ld_out, s_row = a.tok_mode ? a.out_s_row : 1;
    pdl(splitk_reduce_kernel, (unsigned)((n + 255) / 256), 256, 0, st)(p.part, p.n_splits, a.M, out_rows, (float*)a.out, s_tok,
                                                                    s_row, a.row_scale, a.alpha_dev, p.bias, a.accumulate);
    RT_COUNT_LAUNCH(1);
  }
  if (e1) {
    cudaEventRecord(e1, st);
    const double out_bytes = a.out_dtype == OUT_F32 ? 4.0 : 2.0;
    ctx->prof_flops += 2.0 * (double)a.M * (double)w.rows * (double)w.cols;
    ctx->prof_recs.push_back({a.tok_mode ? 3 : (a.aux ? 2 : a.dir), a.M, out_rows, contract});
    ctx->prof_bytes += (double)w.dev_nbytes + 2.0 * (double)a.M * contract + out_bytes * (double)a.M * out_rows * (a.accumulate ? 2.0 : 1.0);
  }
  return cudaGetLastError() == cudaSuccess ? RT_OK : RT_ERR_CUDA;
}


// ------------------------------------------------------------------ the bounded wait, exercised on its own
// One warp waits on a barrier nobody arrives on, with a short limit: the wait gives up, records
// its site code and the kernel returns normally, which is what every wait of the matmul kernel
// does when a peer never shows up.  The context stays usable.
__global__ void wait_selftest_kernel(int* status, long long limit_cycles) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(&bar, 0, status, 999, limit_cycles);
}

// ------------------------------------------------------------------ allocation-free entry point
// The partial sums of a contraction that is accumulated in pieces (more than 16384 weight rows)
// live here for rt_frozen_backward_input_dev_noalloc instead of in memory from cudaMalloc.  Every GPU that loads the library holds these 8 MiB until the process exits.
constexpr size_t NOALLOC_SCRATCH_FLOATS = (size_t)2 << 20;
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_SCRATCH_FLOATS];
static float* g_noalloc_scratch_addr[64] = {nullptr};  // device address of the array, per device ordinal

// In host code `g_noalloc_scratch` is only a stand-in for the symbol, not a device address: the
// address a kernel can use comes from cudaGetSymbolAddress, asked once per device with that
// device current.
static int noalloc_scratch_for(int device, float** out) {
  if (device < 0 || device >= 64) return RT_ERR_BAD_ARG;
  if (!g_noalloc_scratch_addr[device]) {
    void* p = nullptr;
    if (cudaSetDevice(device) != cudaSuccess) return RT_ERR_CUDA;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) return RT_ERR_CUDA;
    g_noalloc_scratch_addr[device] = (float*)p;
  }
  *out = g_noalloc_scratch_addr[device];
  return RT_OK;
}

}  // namespace rt

extern "C" rt_status rt_ctx_selftest_wait_timeout(rt_ctx* c, uint64_t limit_cycles) {
  if (!c) return RT_ERR_BAD_ARG;
  if (limit_cycles == 0 || limit_cycles > 2000000000ull) return c->fail(RT_ERR_BAD_ARG, "limit must be 1..2e9 cycles");
  if (cudaSetDevice(c->device) != cudaSuccess) return RT_ERR_CUDA;
  rt::wait_selftest_kernel<<<1, 32, 0, c->stream>>>(c->status_dev, (long long)limit_cycles);
  if (cudaGetLastError() != cudaSuccess) return c->fail(RT_ERR_CUDA, "self-test launch failed");
  return c->check_device_status("rt_ctx_selftest_wait_timeout");  // expected: RT_ERR_DEVICE_WAIT_TIMEOUT, site 999
}

extern "C" rt_status rt_frozen_backward_input_dev_noalloc(rt_frozen* f, const void* dy_dev, int in_dtype, size_t t,
                                                          void* dx_dev, int out_dtype, int accumulate) {
  if (!f || !dy_dev || !dx_dev) return RT_ERR_BAD_ARG;
  rt_ctx* c = f->ctx;
  if (t == 0) return RT_OK;
  if (t > (1u << 24)) return RT_ERR_BAD_SHAPE;
  if (in_dtype != RT_DT_F16 && in_dtype != RT_DT_BF16) return RT_ERR_BAD_ARG;
  if (out_dtype < 0 || out_dtype > 2 || (accumulate && out_dtype != RT_DT_F32)) return RT_ERR_BAD_ARG;
  if (cudaSetDevice(c->device) != cudaSuccess) return RT_ERR_CUDA;
  float* scratch = nullptr;
  int rc = rt::noalloc_scratch_for(c->device, &scratch);  // first call on a device: looks the array up
  if (rc) return rc;
  rt::QGemmArgs a;
  a.dir = rt::QG_BWD;
  a.act = dy_dev;
  a.act_f16 = in_dtype == RT_DT_F16;
  a.M = (int)t;
  a.out = dx_dev;
  a.out_dtype = out_dtype;
  a.accumulate = accumulate ? 1 : 0;
  a.fixed_part = scratch;
  a.fixed_part_floats = rt::NOALLOC_SCRATCH_FLOATS;
  return rt::qgemm_launch(c, f->w, a);
}
