// wide_rows_kernel: rows whose softmax runs over the whole vocabulary (top-k off).
//
// One row at a time per persistent CTA. Warp w owns one contiguous span of the row (1/W_NW of it,
// rounded up to whole steps); in a step every lane handles eight logits (two 16-byte vectors
// of f32, one of bf16), loaded straight into registers one or two steps ahead of their use
// and asked from L2 two steps before that. Nothing is shared between threads inside a pass,
// so a pass contains no barrier; the loads carry L2 cache hints (keep in pass 1, evict first
// in pass 3), and the later passes find in L2 what has stayed there.
//
// This header has no include guard: it is included once per instance, with GS_W_NS naming the
// instance's namespace inside gs and GS_W_NT its threads per CTA.
//   256:  four CTAs per SM. With four rows per SM the load latency and the serial tail of one
//         row hide behind the arithmetic of the others: the instance for batches that fill the GPU.
//   1024: one CTA per SM. A row finishes about a quarter sooner: the instance for batches of at
//         most one row per SM.
//
//   sample                     the first step of every warp: an upper estimate (anchor) of the
//                              row's maximum and its range
//   pass 1 (HBM)               max, min, NaN; with an active top-p cut also the count histogram
//                              over 4096 linear buckets of s - anchor, whose width is the power
//                              of two that covers the estimated range
//   bracket                    count-based lower/upper mass bounds bracket the cut to a zone of
//                              buckets (a maximum above the anchor: pass 2 recounts exactly)
//   pass 3 (L2)                exponentials. Mass of d >= dA (certainly kept) per piece of
//                              four steps, zone logits (dB <= d < dA) into an exact list
//   tail                       weighted selection inside the zone, prefix over the pieces,
//                              rescan of the one piece that holds the drawn token
//
// Row semantics: model/generate.go:147-240 (mode A), model/qwen/generate.go:92-153 (mode B).
#include "sample_batch.cuh"   // includes row_stream.cuh

#ifndef GS_W_NS
#define GS_W_NS w256
#define GS_W_NT 256
#endif

namespace gs {
namespace GS_W_NS {

constexpr int W_NT = GS_W_NT;           // threads per CTA
constexpr int W_CTAS = 1024 / W_NT;     // CTAs per SM
constexpr int W_NSUB = W_NT;            // sub-buckets of one weighted-selection round
constexpr int W_NW = W_NT / 32;
constexpr int W_NB = 4096;              // histogram buckets
constexpr int W_ZCAP = 2048;            // exact zone list capacity
constexpr int W_D1 = 2;                 // steps of register prefetch in pass 1
constexpr int W_G = 4;                  // steps per piece (power of two)
constexpr int W_MAX_STEPS = (W_NT >= 512) ? 64 : 128;         // steps per warp and pass; longer rows go to the single-CTA kernel
constexpr int W_MAX_PPW = W_MAX_STEPS / W_G;
constexpr int W_MAX_PIECES = W_NW * W_MAX_PPW;                 // 512
constexpr int W_EB_REP = 16;            // copies of a table entry in the conflict-free layout
constexpr int W_EB_REP_ENTRIES = 128;   // entries of that layout: d > -(128-1)/32
constexpr int W_OFF_HIST = 0;
constexpr int W_OFF_ZONE = W_OFF_HIST + W_NB * 4;
constexpr int W_OFF_EB = W_OFF_ZONE + W_ZCAP * 8;              // 1024 entries, or 128 entries x 16 copies
constexpr int W_OFF_PART = W_OFF_EB + W_EB_REP * W_EB_REP_ENTRIES * 8;
constexpr int W_DYN_BYTES = W_OFF_PART + W_MAX_PIECES * 8;     // 52 KB
static_assert(W_EB_REP * W_EB_REP_ENTRIES >= NB1, "either layout fits");
static_assert(W_NT >= 256 && W_NT <= 1024 && W_MAX_PIECES <= W_NT && W_G * 64 <= W_NT && W_NSUB * 12 <= W_NB * 4,
              "one piece / one vector of a piece / one sub-bucket per thread");

// Histogram buckets of width 1/scale (scale a power of two): bucket = round(-d * scale),
// clamped to W_NB - 1. Multiplying by a power of two is exact, so the bucket edges are exact.
__device__ __forceinline__ int bucket_w(float d, float scale, float dclamp) {
  const float f = fmaf(fmaxf(d, dclamp), -scale, 8388608.0f);
  return __float_as_int(f) & 0x1fff;
}
// smallest d whose bucket is <= bmax (the edge is a tie that rounds to even)
__device__ __forceinline__ float bucket_floor_w(int bmax, float scale, float dclamp) {
  if (bmax >= W_NB - 1) return -INFINITY;
  if (bmax < 0) return INFINITY;
  const float t = -(static_cast<float>(2 * bmax + 1) * (0.5f / scale));
  return (bucket_w(t, scale, dclamp) <= bmax) ? t : __uint_as_float(__float_as_uint(t) - 1u);
}

__device__ __forceinline__ double lds_f64(uint32_t addr) {
  double v;
  asm("ld.shared.f64 %0, [%1];" : "=d"(v) : "r"(addr));
  return v;
}
// exp(d) for -31.9 < d <= 0 from the table E[b] = exp(-b/32) in shared memory: d = -b/32 + dl with
// |dl| <= 1/64 exactly (f32), exp = E[b] * (1 + w), w = dl + dl^2/2 + ... + dl^5/120 in f32. The one
// rounding of w (at most 2^-31 relative to the result, unbiased) is the error that matters.
// The bits of f are 0x4B000000 + b, so bits * eb_mul + eb_bias is the address of E[b] (mod 2^32)
// with eb_mul = 8 and eb_bias = table - 0x4B000000 * 8 for the plain table. In the conflict-free
// layout (rows whose d stay above -(W_EB_REP_ENTRIES-1)/32) entry b has sixteen copies 8 bytes
// apart and lane l reads copy l mod 16, its own pair of banks: eb_mul = 128, eb_bias = table +
// 8 (l mod 16) - 0x4B000000 * 128.
__device__ __forceinline__ double exp_fast_s(float d, uint32_t eb_mul, uint32_t eb_bias) {
  const float f = fmaf(d, -32.0f, 8388608.0f);
  const float dl = fmaf(f - 8388608.0f, 0.03125f, d);
  float t = fmaf(dl, 8.3333338e-3f, 4.1666668e-2f);
  t = fmaf(t, dl, 1.6666667e-1f);
  t = fmaf(t, dl, 0.5f);
  const float w = fmaf(t, dl * dl, dl);
  const double E = lds_f64(__float_as_uint(f) * eb_mul + eb_bias);
  return fma(E, static_cast<double>(w), E);
}
// Two-wide f32 arithmetic (one issue slot for two results on sm_100).
typedef unsigned long long f32x2_t;
__device__ __forceinline__ f32x2_t pk2(float a, float b) { f32x2_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ void upk2(f32x2_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2_t fma2(f32x2_t a, f32x2_t b, f32x2_t c) { f32x2_t d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ f32x2_t add2(f32x2_t a, f32x2_t b) { f32x2_t d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ f32x2_t mul2(f32x2_t a, f32x2_t b) { f32x2_t d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
// exp_fast_s for two arguments at once (D = the pair of d values)
__device__ __forceinline__ void exp_fast_s2(f32x2_t D, uint32_t eb_mul, uint32_t eb_bias, double& e0, double& e1) {
  const f32x2_t F = fma2(D, pk2(-32.0f, -32.0f), pk2(8388608.0f, 8388608.0f));
  const f32x2_t DL = fma2(add2(F, pk2(-8388608.0f, -8388608.0f)), pk2(0.03125f, 0.03125f), D);
  f32x2_t T = fma2(DL, pk2(8.3333338e-3f, 8.3333338e-3f), pk2(4.1666668e-2f, 4.1666668e-2f));
  T = fma2(T, DL, pk2(1.6666667e-1f, 1.6666667e-1f));
  T = fma2(T, DL, pk2(0.5f, 0.5f));
  const f32x2_t W = fma2(T, mul2(DL, DL), DL);
  float f0, f1, w0, w1;
  upk2(F, f0, f1); upk2(W, w0, w1);
  const double E0 = lds_f64(__float_as_uint(f0) * eb_mul + eb_bias);
  const double E1 = lds_f64(__float_as_uint(f1) * eb_mul + eb_bias);
  e0 = fma(E0, static_cast<double>(w0), E0);
  e1 = fma(E1, static_cast<double>(w1), E1);
}
constexpr double W_EXP_REL_ERR = 6e-10;   // bound of exp_fast_s against the exact exponential

// Steps [st0, st1) of one pass; qa/qb hold the vectors of steps st0 .. st0+D-1 on entry and of
// st1 .. st1+D-1 on exit (D steps of register prefetch). CLEAN runs hold no logit outside the
// row and skip all masking; the others (a warp's step that holds the row's first or last vector,
// or vectors past the end) give every logit outside the row the value -Inf and a clear bit in
// `valid`. body(x, valid, st, gv): eight logits of this lane, validity bits, step, the lane's
// first vector.
template <typename T, int D, bool CLEAN, typename F>
__device__ __forceinline__ void wide_steps(const WSpan& sp, const RowView<T>& rv, unsigned long long pol, int lane,
                                           int st0, int st1, uint4 (&qa)[D], uint4 (&qb)[D], F&& body) {
  constexpr int VEC = Elem<T>::VEC, EPI = 8 / VEC, SV = 32 * EPI;
#pragma unroll 1
  for (int st = st0; st < st1; st++) {
    uint4 na, nb;
    w_load<T>(sp, st + D, pol, na, nb);
    float x[8];
    if (EPI == 2) { Elem<T>::unpack(qa[0], x); Elem<T>::unpack(qb[0], x + 4 * (EPI - 1)); }
    else Elem<T>::unpack(qa[0], x);
#pragma unroll
    for (int k = 0; k + 1 < D; k++) { qa[k] = qa[k + 1]; qb[k] = qb[k + 1]; }
    qa[D - 1] = na; qb[D - 1] = nb;
    const int gv = sp.first + st * SV + lane;
    uint32_t valid = 0xffu;
    if (!CLEAN) {
      valid = 0u;
#pragma unroll
      for (int h = 0; h < EPI; h++) {
        const int g = gv + 32 * h;
        const int i0 = g * VEC - rv.shift;
#pragma unroll
        for (int c = 0; c < VEC; c++) {
          const int i = i0 + c;
          if (g < rv.nvec && i >= 0 && i < rv.V) valid |= 1u << (h * VEC + c);
          else x[h * VEC + c] = -INFINITY;
        }
      }
    }
    body(x, valid, st, gv);
  }
}
// One pass over the warp's span with D steps of prefetch: runs of clean and other steps, in order.
#define GS_WIDE_STREAM(T, D, sp, rv, pol, lane, BODY)                                           \
  do {                                                                                          \
    uint4 qa_[D], qb_[D];                                                                       \
    _Pragma("unroll") for (int s_ = 0; s_ < D; s_++) w_load<T>(sp, s_, pol, qa_[s_], qb_[s_]);  \
    if (sp.clean_lo > 0) wide_steps<T, D, false>(sp, rv, pol, lane, 0, sp.clean_lo, qa_, qb_, BODY(false)); \
    wide_steps<T, D, true>(sp, rv, pol, lane, sp.clean_lo, sp.clean_hi, qa_, qb_, BODY(true));  \
    if (sp.clean_hi < sp.nst) wide_steps<T, D, false>(sp, rv, pol, lane, sp.clean_hi, sp.nst, qa_, qb_, BODY(false)); \
  } while (0)

// pass 1: max, min, NaN flag over the row's logits. With HIST it also counts the logits into the
// histogram of q = s - anchor (an upper estimate of the row's maximum taken from a sample), so that
// rows whose maximum stays below the anchor need no second pass for their histogram.
template <typename T, bool HIST, bool TONE>
__device__ __noinline__ void wide_pass1(const WSpan& sp_in, const RowView<T>& rv_in, unsigned long long pol, int lane,
                                        uint32_t hist_bias, float anchor, float Tm, float scale, float dclamp,
                                        float& xmax, float& xmin, bool& nan_seen) {
  const WSpan sp = sp_in;                // registers, not memory, inside the loop
  const RowView<T> rv = rv_in;
  float vmax = -INFINITY, vmin = INFINITY;   // vmax with NaN-propagating maxima: NaN iff the span held one
#define GS_BODY1(CL) [&](const float* x, uint32_t valid, int, int) {                             \
    if (CL) {                                                                                    \
      vmax = max3nan(vmax, x[0], x[1]); vmax = max3nan(vmax, x[2], x[3]);                        \
      vmax = max3nan(vmax, x[4], x[5]); vmax = max3nan(vmax, x[6], x[7]);                        \
      vmin = min3f(vmin, x[0], x[1]); vmin = min3f(vmin, x[2], x[3]);                            \
      vmin = min3f(vmin, x[4], x[5]); vmin = min3f(vmin, x[6], x[7]);                            \
    }                                                                                            \
    _Pragma("unroll") for (int c = 0; c < 8; c++) {                                              \
      if (!CL) {                                                                                 \
        vmax = maxnan(vmax, x[c]);                           /* masked logits read as -Inf */    \
        vmin = fminf(vmin, ((valid >> c) & 1u) ? x[c] : INFINITY);                               \
      }                                                                                          \
      if (HIST) {                                                                                \
        const float s = TONE ? x[c] : __fdiv_rn(x[c], Tm);                                       \
        /* NaN and anything above the anchor land in bucket 0 or W_NB-1: such rows are redone */ \
        const float f = fmaf(fminf(fmaxf(s - anchor, dclamp), 0.0f), -scale, 8388608.0f);        \
        const uint32_t a = __float_as_uint(f) * 4u + hist_bias;                                  \
        if (CL || ((valid >> c) & 1u)) asm volatile("red.shared.add.u32 [%0], 1;" :: "r"(a) : "memory"); \
      }                                                                                          \
    } }
  GS_WIDE_STREAM(T, W_D1, sp, rv, pol, lane, GS_BODY1);
#undef GS_BODY1
  xmax = vmax; xmin = vmin; nan_seen = (vmax != vmax);
}

// pass 2: count histogram of d (logits outside the row are not counted).
// hist_bias = shared address of the histogram - 0x4B000000 * 4 (mod 2^32): see exp_fast_s.
template <typename T, bool TONE>
__device__ __noinline__ void wide_pass2(const WSpan& sp_in, const RowView<T>& rv_in, unsigned long long pol, int lane,
                                        uint32_t hist_bias, float m, float Tm, float scale, float dclamp) {
  const WSpan sp = sp_in;
  const RowView<T> rv = rv_in;
#define GS_BODY2(CL) [&](const float* x, uint32_t valid, int, int) {                             \
    _Pragma("unroll") for (int c = 0; c < 8; c++) {                                              \
      const float s = TONE ? x[c] : __fdiv_rn(x[c], Tm);                                         \
      const float f = fmaf(fmaxf(s - m, dclamp), -scale, 8388608.0f);                            \
      const uint32_t a = __float_as_uint(f) * 4u + hist_bias;                                    \
      if (CL || ((valid >> c) & 1u)) asm volatile("red.shared.add.u32 [%0], 1;" :: "r"(a) : "memory"); \
    } }
  GS_WIDE_STREAM(T, 1, sp, rv, pol, lane, GS_BODY2);
#undef GS_BODY2
}

// pass 3: exponentials. part[warp * ppw + piece] receives the certainly-kept mass (d >= dA) of
// each piece of W_G steps; zone logits (dB <= d < dA) go to the list zl. The lane-private sum of
// all mass comes back in Ssum, the kept mass of the warp's pieces in lane 0's Ksum.
// FAST: every logit of the row has d > -31.9 (bucket-table exponential, no range check);
// TONE: temperature 1; CUT: a top-p cut is active.
template <typename T, bool FAST, bool TONE, bool CUT>
__device__ __noinline__ void wide_pass3(const WSpan& sp_in, const RowView<T>& rv_in, unsigned long long pol, int lane, int warp,
                                        float m, float Tm, float dA, float dB, uint32_t eb_mul, uint32_t eb_bias, const double* s_tab,
                                        double* part, int ppw, uint2* zl, int* zcnt, double& Ssum, double& Ksum) {
  constexpr int VEC = Elem<T>::VEC;
  const WSpan sp = sp_in;
  const RowView<T> rv = rv_in;
  // |d - dmid| <= dhalf is a superset of the zone dB <= d < dA (infinite ends are clamped)
  const float dAc = fminf(dA, 3.0e38f), dBc = fmaxf(dB, -3.0e38f);
  const float dmid = 0.5f * dAc + 0.5f * dBc;
  const float dhalf = (0.5f * dAc - 0.5f * dBc) * 1.000001f + 1e-30f;
  const bool none_kept = CUT && (dA == INFINITY);
  const float dfloor = (eb_mul == 8u) ? -31.9f : -(W_EB_REP_ENTRIES - 1.5f) / 32.0f;   // keeps masked logits inside the table
  double t0 = 0.0, t1 = 0.0, sub = 0.0;
  double stot = 0.0, ksum = 0.0;
#define GS_BODY3(CL) [&](const float* x, uint32_t valid, int st, int gv) {                       \
    float nearest = INFINITY;                                                                    \
    _Pragma("unroll") for (int c = 0; c < 8; c += 2) {                                           \
      const float s0 = TONE ? x[c] : __fdiv_rn(x[c], Tm);                                        \
      const float s1 = TONE ? x[c + 1] : __fdiv_rn(x[c + 1], Tm);                                \
      const float d0 = s0 - m, d1 = s1 - m;                                                      \
      double e0, e1;                                                                             \
      if (FAST) {                                                                                \
        if (CL) exp_fast_s2(pk2(d0, d1), eb_mul, eb_bias, e0, e1);                               \
        else exp_fast_s2(pk2(fmaxf(d0, dfloor), fmaxf(d1, dfloor)), eb_mul, eb_bias, e0, e1);    \
        if (!CL) {                                                                               \
          const bool v0 = (valid >> c) & 1u, v1 = (valid >> (c + 1)) & 1u;                       \
          e0 = __hiloint2double(v0 ? __double2hiint(e0) : 0, v0 ? __double2loint(e0) : 0);       \
          e1 = __hiloint2double(v1 ? __double2hiint(e1) : 0, v1 ? __double2loint(e1) : 0);       \
        }                                                                                        \
      } else {                                                                                   \
        e0 = exp_safe(d0, s_tab);                            /* exp_safe(-Inf) is exactly 0 */   \
        e1 = exp_safe(d1, s_tab);                                                                \
      }                                                                                          \
      t0 += e0; t1 += e1;                                                                        \
      if (CUT) {                                                                                 \
        sub = fma(e0, __hiloint2double((d0 < dA) ? 0x3ff00000 : 0, 0), sub);                     \
        sub = fma(e1, __hiloint2double((d1 < dA) ? 0x3ff00000 : 0, 0), sub);                     \
        nearest = fminf(nearest, fminf(fabsf(d0 - dmid), fabsf(d1 - dmid)));                     \
      }                                                                                          \
    }                                                                                            \
    if (CUT && nearest <= dhalf) {                           /* rare: a logit of this lane near the zone */ \
      _Pragma("unroll") for (int c = 0; c < 8; c++) {                                            \
        const float s = TONE ? x[c] : __fdiv_rn(x[c], Tm);                                       \
        const float d = s - m;                                                                   \
        if ((CL || ((valid >> c) & 1u)) && d < dA && d >= dB) {                                  \
          const int i = (gv + 32 * (c / VEC)) * VEC - rv.shift + (c % VEC);                      \
          const int slot = atomicAdd(zcnt, 1);                                                   \
          if (slot < W_ZCAP) zl[slot] = make_uint2(__float_as_uint(d), static_cast<uint32_t>(i)); \
        }                                                                                        \
      }                                                                                          \
    }                                                                                            \
    if ((st & (W_G - 1)) == W_G - 1 || st == sp.nst - 1) {   /* end of a piece */                \
      const double tot = t0 + t1;                                                                \
      /* With dA = +Inf nothing is certainly kept (exactly 0); otherwise the subtraction's */    \
      /* rounding is far below the row maximum's own mass. */                                    \
      double kw = none_kept ? 0.0 : tot - sub;                                                   \
      kw = warp_sum_d(kw);                                                                       \
      stot += tot;                                                                               \
      if (lane == 0) { part[warp * ppw + (st / W_G)] = kw; ksum += kw; }                         \
      t0 = t1 = 0.0; sub = 0.0;                                                                  \
    } }
  GS_WIDE_STREAM(T, 1, sp, rv, pol, lane, GS_BODY3);
#undef GS_BODY3
  Ssum = stot; Ksum = ksum;
}

// fn(key, d) for every logit of the warp's span that lies in the zone dB <= d < dA, streamed from
// global memory. Only rows whose zone outgrew the shared list come here (long runs of equal
// logits around the cut), so every step takes the masked form.
template <typename T, typename F>
__device__ __forceinline__ void wide_for_zone(const WSpan& sp, const RowView<T>& rv, unsigned long long pol, int lane,
                                              float m, float Tm, float dA, float dB, int mode, F&& fn) {
  constexpr int VEC = Elem<T>::VEC;
  uint4 qa[1], qb[1];
  w_load<T>(sp, 0, pol, qa[0], qb[0]);
  wide_steps<T, 1, false>(sp, rv, pol, lane, 0, sp.nst, qa, qb, [&](const float* x, uint32_t valid, int, int gv) {
#pragma unroll
    for (int c = 0; c < 8; c++) {
      if ((valid >> c) & 1u) {
        const float s = (Tm == 1.0f) ? x[c] : __fdiv_rn(x[c], Tm);
        const float d = s - m;
        if (d < dA && d >= dB) {
          const int i = (gv + 32 * (c / VEC)) * VEC - rv.shift + (c % VEC);
          fn(zone_key(d, i, mode), d);
        }
      }
    }
  });
}

struct WideShared {
  bu::Scratch sc;
  double tab[256];
  double bcd[4];
  int bc[4];
  int cnt;
  int row;
};

// The exact cut for a zone that outgrew the shared list (long runs of equal logits around the
// cut): the weighted selection of wide_row, with the row itself as the source of the zone's keys,
// one more pass per round. Adds the kept zone mass to part[]; false: the bracket did not hold.
template <typename T>
__device__ __noinline__ bool wide_big_zone(const WSpan& sp_in, const RowView<T>& rv_in, unsigned long long pol, WideShared& sh,
                                           uint32_t* hist, double* part, const double* s_tab, float m, float Tm, float dA,
                                           float dB, float dlow, int mode, double plim, double S, double Ktot, bool fast_ok,
                                           int span, int ppw, unsigned long long& cut_key_out, int& cut_incl_out, uint32_t& flags) {
  const WSpan sp = sp_in;
  const RowView<T> rv = rv_in;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int PV = W_G * 32 * (8 / Elem<T>::VEC);
  bu::Scratch& sc = sh.sc;
  unsigned long long cut_key = 0ull;
  int cut_incl = 0;
  bool bad = false;
  {
    // every zone key with its d: from the list, or from the row when the list overflowed
    auto each_zone = [&](auto&& fn) { wide_for_zone<T>(sp, rv, pol, lane, m, Tm, dA, dB, mode, fn); };
    // G(c) = Ktot + mass{key <= c} rises along the zone order. Both flavours need the first key c*
    // where G crosses: mode B (first G/S >= p) keeps through c*, mode A (first G/S > 1.5p) keeps
    // everything before it. Narrow [lo, hi] around c* with linear sub-buckets until at most 32
    // keys remain, then one warp finishes.
    auto crossed = [&](double g) -> bool { return mode == 0 ? (g / S > plim) : (g / S >= plim); };
    if (Ktot > 0.0 && crossed(Ktot)) bad = true;             // the bracket was wrong
    double* sm = reinterpret_cast<double*>(hist);            // [W_NSUB] mass per sub-bucket
    int* scn = reinterpret_cast<int*>(hist) + 2 * W_NSUB;    // [W_NSUB] count per sub-bucket
    unsigned long long lo = ~0ull, hi = 0ull;
    int nz_loc = 0;
    each_zone([&](unsigned long long k, float) { lo = k < lo ? k : lo; hi = k > hi ? k : hi; nz_loc++; });
    lo = bu::min_u64<W_NW>(lo, sc, tid);
    hi = bu::max_u64<W_NW>(hi, sc, tid);
    double gbase = Ktot;                                     // Ktot + mass of keys below lo; never crossed
    int inrange = bu::sum_i<W_NW>(nz_loc, sc, tid);
    bool all_in = false;
    for (int iter = 0; iter < 10 && inrange > 32 && !bad && !all_in; iter++) {
      const unsigned long long spn = hi - lo;
      int shf = 0;
      while (shf < 63 && (spn >> shf) >= static_cast<unsigned long long>(W_NSUB)) shf++;
      __syncthreads();
      sm[tid] = 0.0; scn[tid] = 0;                           // W_NT == W_NSUB
      __syncthreads();
      each_zone([&](unsigned long long k, float d) {
        if (k >= lo && k <= hi) {
          const int sb = static_cast<int>((k - lo) >> shf);
          atomicAdd(&sm[sb], exp_safe(d, s_tab));
          atomicAdd(&scn[sb], 1);
        }
      });
      __syncthreads();
      const double mine = sm[tid];
      double totm;
      const double exm = bu::scan_excl_d<W_NW>(mine, totm, sc, tid);
      const int first = (scn[tid] > 0 && crossed(gbase + exm + mine)) ? tid : W_NSUB;
      const int sbx = bu::min_i<W_NW>(first, sc, tid);
      if (sbx == W_NSUB) { all_in = true; break; }
      if (tid == sbx) { sh.bcd[0] = gbase + exm; sh.bc[0] = scn[tid]; }
      __syncthreads();
      gbase = sh.bcd[0];
      inrange = sh.bc[0];
      const unsigned long long nlo = lo + (static_cast<unsigned long long>(sbx) << shf);
      unsigned long long nhi = nlo + ((1ull << shf) - 1ull);
      if (nhi < nlo || nhi > hi) nhi = hi;
      lo = nlo; hi = nhi;
    }
    if (inrange > 32 && !all_in) bad = true;
    double g_at = gbase, g_before = gbase;
    if (!bad && !all_in) {
      unsigned long long* few = reinterpret_cast<unsigned long long*>(hist);   // [32]
      __syncthreads();
      if (tid == 0) sh.cnt = 0;
      __syncthreads();
      each_zone([&](unsigned long long k, float) {
        if (k >= lo && k <= hi) { const int slot = atomicAdd(&sh.cnt, 1); if (slot < 32) few[slot] = k; }
      });
      __syncthreads();
      const int nf = min(32, sh.cnt);
      if (warp == 0) {
        const unsigned long long k = (lane < nf) ? few[lane] : ~0ull;
        const double e = (lane < nf) ? exp_safe(zone_key_d(k), s_tab) : 0.0;
        double g = gbase;                                    // G(k) = gbase + masses of the keys <= k
        for (int l = 0; l < nf; l++) {
          const unsigned long long kl = __shfl_sync(FULL, k, l);
          const double el = __shfl_sync(FULL, e, l);
          if (kl <= k) g += el;
        }
        const bool cr = (lane < nf) && crossed(g);
        unsigned long long candk = cr ? k : ~0ull;           // first crossed key = smallest crossed key
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const unsigned long long tt = __shfl_xor_sync(FULL, candk, o);
          candk = tt < candk ? tt : candk;
        }
        const unsigned who = __ballot_sync(FULL, cr && k == candk);
        if (lane == 0) { sc.u[0] = candk; sh.bc[1] = who ? 1 : 0; }
        if (who && lane == __ffs(who) - 1) { sh.bcd[1] = g; sh.bcd[2] = g - e; }
      }
      __syncthreads();
      if (sh.bc[1]) {
        cut_key = sc.u[0];
        g_at = sh.bcd[1];
        g_before = sh.bcd[2];
        cut_incl = (mode == 0) ? 0 : 1;
      } else {
        all_in = true;                                       // rounding: nothing in the last group crossed
      }
      __syncthreads();
    }
    if (!bad && all_in) {
      cut_key = ~0ull; cut_incl = 1;
      if (mode == 1 && dlow < dB) bad = true;                // logits below the zone exist: the bracket promised a crossing
    }
    if (!bad && !all_in) {
      // the sums carry exp_fast_s's error; in G/S >= p it enters as 2 p (1-p) times that bound
      const double etol = 1e-12 + (fast_ok ? 2.0 * plim * fabs(1.0 - plim) * W_EXP_REL_ERR : 0.0);
      if (fabs(g_at / S - plim) <= etol || fabs(g_before / S - plim) <= etol) flags |= FLAG_TOPP_EDGE;
      if (mode == 1) {
        // a later key with the same d as c*: the cut separates equal probabilities
        int tie = 0;
        each_zone([&](unsigned long long k, float) { tie |= (k > cut_key && (k >> 32) == (cut_key >> 32)) ? 1 : 0; });
        if (bu::max_i<W_NW>(tie, sc, tid)) flags |= FLAG_TIE_CUT;
      }
    }
    if (bad) return false;
    // kept zone entries add their mass to the piece they sit in
    __syncthreads();
    each_zone([&](unsigned long long k, float d) {
      if (k < cut_key || (cut_incl && k == cut_key)) {
        const int v = rv.vec_of(zone_key_index(k, mode));
        const int w = v / span;
        atomicAdd(&part[w * ppw + (v - w * span) / PV], exp_safe(d, s_tab));
      }
    });
    __syncthreads();
  }
  cut_key_out = cut_key; cut_incl_out = cut_incl;
  return true;
}

// ---------------------------------------------------------------------------------------------
// One-pass front end. Where a sample of the row (every eighth step of every warp) places the
// top-p cut inside a narrow window of logit values, one pass over the row is enough: it sums the
// mass of everything (S) and of what lies above the window (certainly kept, per piece) with the fast
// exponential, relative to an anchor near the row maximum, and notes which lane-steps hold a logit
// inside the window; those few vectors are read again (from L2) into the exact zone list, and the
// tail decides the cut inside the window as it does after two passes. The sample only chooses the
// window: whether the cut really lies inside it is checked on the sums of the whole row, and a row
// whose window failed (or that the sample cannot place: a few heavy tokens, NaN, a wide window) takes
// the two-pass front end. Rows without a cut need no window at all.
//
// Error budget of the fast sums against exp(d) in f64, d = x/T - max rounded to f32 as upstream:
// ex2.approx 2.4e-7, three f32 additions per step before the f64 accumulators 1.8e-7, and per unit
// of |x/T - anchor| the roundings of that difference, of d itself, of the product with log2(e) and
// of the constant, 2e-7 together: W1_EPS_FIXED + W1_EPS_PER_D * (largest |d| that carries mass).
// ---------------------------------------------------------------------------------------------
constexpr int W1_STRIDE = 8;             // the sample: every eighth step
#ifndef GS_W1_PF
#define GS_W1_PF 10
#endif
constexpr int W1_PF = GS_W1_PF;          // steps ahead that the pass asks L2 for its lines (0: never)
constexpr int W_ZCAP1 = 2 * W_ZCAP;      // zone list of the one-pass front end (zone + table areas)
constexpr double W1_EPS_FIXED = 4.5e-7;
constexpr double W1_EPS_PER_D = 2.0e-7;
constexpr float W1_MAGIC = 2097152.0f;   // 2^21: floats in [2^21, 2^22) have an ulp of 1/4
constexpr float W1_FCLAMP = 2097152.0f + 4095.75f;
static_assert(W_OFF_EB == W_OFF_ZONE + W_ZCAP * 8 && W_EB_REP * W_EB_REP_ENTRIES * 8 >= W_ZCAP * 8, "the long zone list spans both areas");

__device__ __forceinline__ void l2_prefetch(const void* p) { asm volatile("prefetch.global.L2 [%0];" :: "l"(p)); }
__device__ __forceinline__ float ex2_approx(float t) { float e; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t)); return e; }
__device__ __forceinline__ float set_ge(float a, float b) { float r; asm("set.ge.f32.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r; }   // 1.0f or 0.0f
__device__ __forceinline__ float min3abs(float a, float b, float c) { float d; asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(fabsf(b)), "f"(fabsf(c))); return d; }

// Histogram bucket of a raw logit: y = (anchor' - x) * hs, f = RN(hc - x * hs) rounds the exact
// y + 2^21 to a multiple of 1/4 (one rounding, by fma); bits 2..13 of f are the bucket: y in
// [b - 1/8, b + 7/8]. f is clamped from above (everything below the range, -Inf and NaN land in the
// last bucket); a logit above the anchor leaves the binade and lands anywhere inside the array:
// the caller checks the maximum it saw against the anchor.
__device__ __forceinline__ uint32_t bucket_off1(float x, float nhs, float hc) {
  return __float_as_uint(fminf(fmaf(x, nhs, hc), W1_FCLAMP)) & 0x3ffcu;
}
// Smallest float whose bucket is <= bmax (the buckets fall as x rises). +Inf: none; -Inf: every float.
__device__ __forceinline__ float bucket_floor1(int bmax, float nhs, float hc, bool& ok) {
  if (bmax >= W_NB - 1) return -INFINITY;
  if (bmax < 0) return INFINITY;
  float x = ((hc - W1_MAGIC) - (static_cast<float>(bmax) + 0.875f)) / (-nhs);
  const uint32_t lim = static_cast<uint32_t>(bmax) * 4u + 3u;
  int it = 0;
  while (bucket_off1(x, nhs, hc) > lim && it < 24) { x = nextafterf(x, INFINITY); it++; }
  while (it < 24) {
    const float below = nextafterf(x, -INFINITY);
    if (bucket_off1(below, nhs, hc) > lim) break;
    x = below; it++;
  }
  if (it >= 24) ok = false;
  return x;
}
// x / T in IEEE f32 round-to-nearest by q0 = x y, r = fma(-q0, T, x), q = fma(r, y, q0) with y = RN(1/T):
// the correctly rounded quotient whenever T's significand is not all ones and nothing over- or underflows
// (the caller takes this form for 2^-20 <= T <= 2^20 only and clamps x at -1e30: whatever lies below has
// mass 0 either way).
__device__ __forceinline__ f32x2_t div2_fast(f32x2_t X, float T, float y) {
  const f32x2_t Y = pk2(y, y);
  const f32x2_t Q0 = mul2(X, Y);
  const f32x2_t R = fma2(Q0, pk2(-T, -T), X);
  return fma2(R, Y, Q0);
}

struct OnePassOut {
  float m;                 // row maximum of x / T
  double S, Ktot;          // all mass; mass above the window (both relative to exp(m))
  int nz;                  // zone entries in the list
  float xA, xB;            // above the window: x >= xA; the window: xB <= x < xA
  double eps;              // relative error bound of S and Ktot
};
struct P1Consts {
  float as, Tm, yT;        // anchor in units of x / T; temperature and its rounded reciprocal
  float xA, xB;            // above the window: x >= xA; the window: xB <= x < xA
  float xmid, xhalf;       // |x - xmid| <= xhalf is a superset of the window
  uint32_t zl_s, zcnt_s;   // shared-memory addresses of the window list (W_ZCAP1 entries of (logit bits, index)) and its counter
};
struct P1Acc {
  double tot;              // running piece without a cut: all its mass; with a cut: all mass so far
  double kep;              // with a cut: mass above the window of the running piece
  double stot;             // without a cut: all mass of the pieces done
  float vmax;              // NaN-propagating running maximum
};

// The window's logits of one lane-step go to the list. Only lanes that saw a logit near the window
// come here; CHECK: the step may hold logits outside the row (index tested against V).
template <int VEC, bool CHECK>
__device__ __forceinline__ void p1_append(const float* x, int i_first, int V, const P1Consts& k) {
#pragma unroll
  for (int c = 0; c < 8; c++) {
    if (x[c] < k.xA && x[c] >= k.xB) {                         // (masked logits are -Inf: never at or above a finite xB)
      const int i = i_first + (c / VEC) * 32 * VEC + (c % VEC);
      if (!CHECK || (i >= 0 && i < V)) {
        uint32_t slot;
        asm volatile("atom.shared.add.u32 %0, [%1], 1;" : "=r"(slot) : "r"(k.zcnt_s) : "memory");
        if (slot < static_cast<uint32_t>(W_ZCAP1)) {
          asm volatile("st.shared.v2.u32 [%0], {%1, %2};" :: "r"(k.zl_s + slot * 8u), "r"(__float_as_uint(x[c])), "r"(static_cast<uint32_t>(i)) : "memory");
        }
      }
    }
  }
}

// Eight logits of a lane: exp(x/T - anchor) = 2^((x/T - anchor) log2 e); masked logits are -Inf and
// add 2^-Inf = 0. Three f32 additions per sum, then f64. Returns whether a logit lies near the window.
template <bool TONE, bool CUT>
__device__ __forceinline__ bool p1_body(const float* x, const P1Consts& k, P1Acc& a) {
  const float LOG2E = 1.4426950408889634f;
  const f32x2_t NA = pk2(-k.as, -k.as), LL = pk2(LOG2E, LOG2E);
  a.vmax = max3nan(a.vmax, x[0], x[1]); a.vmax = max3nan(a.vmax, x[2], x[3]);
  a.vmax = max3nan(a.vmax, x[4], x[5]); a.vmax = max3nan(a.vmax, x[6], x[7]);
  float nearest = INFINITY;
  f32x2_t E[4], KK[2];
#pragma unroll
  for (int c = 0; c < 4; c++) {
    const f32x2_t X = pk2(x[2 * c], x[2 * c + 1]);
    f32x2_t S_;
    if (TONE) S_ = X;
    else S_ = div2_fast(pk2(fmaxf(x[2 * c], -1e30f), fmaxf(x[2 * c + 1], -1e30f)), k.Tm, k.yT);
    float t0, t1;
    upk2(mul2(add2(S_, NA), LL), t0, t1);
    E[c] = pk2(ex2_approx(t0), ex2_approx(t1));
    if (CUT) {
      const f32x2_t M = pk2(set_ge(x[2 * c], k.xA), set_ge(x[2 * c + 1], k.xA));
      if ((c & 1) == 0) KK[c >> 1] = mul2(E[c], M); else KK[c >> 1] = fma2(E[c], M, KK[c >> 1]);
      float z0, z1;
      upk2(add2(X, pk2(-k.xmid, -k.xmid)), z0, z1);
      nearest = min3abs(nearest, z0, z1);
    }
  }
  { float p, q; upk2(add2(add2(E[0], E[1]), add2(E[2], E[3])), p, q); a.tot += static_cast<double>(p + q); }
  if (CUT) {
    float p, q;
    upk2(add2(KK[0], KK[1]), p, q);
    a.kep += static_cast<double>(p + q);
  }
  return CUT && nearest <= k.xhalf;
}
template <bool CUT>
__device__ __forceinline__ void p1_piece_end(int st, int nst, int lane, double* part_w, P1Acc& a) {
  if ((st & (W_G - 1)) == W_G - 1 || st == nst - 1) {
    const double kw = warp_sum_d(CUT ? a.kep : a.tot);
    if (lane == 0) part_w[st / W_G] = kw;
    if (CUT) { a.kep = 0.0; } else { a.stot += a.tot; a.tot = 0.0; }
  }
}
// A step that holds the row's first or last vector, or vectors past the end: loaded on the spot and masked.
template <typename T, bool TONE, bool CUT>
__device__ __noinline__ void p1_edge_step(const WSpan& sp, const RowView<T>& rv, int lane, int st,
                                          const P1Consts& k, double* part_w, P1Acc& a) {
  constexpr int VEC = Elem<T>::VEC, EPI = 8 / VEC, SV = 32 * EPI;
  const int gv = sp.first + st * SV + lane;
  float x[8];
#pragma unroll
  for (int h = 0; h < EPI; h++) {
    const int g = gv + 32 * h;
    float xv[VEC];
    Elem<T>::unpack(__ldg(rv.vbase + min(g, rv.nvec - 1)), xv);
    const int i0 = g * VEC - rv.shift;
#pragma unroll
    for (int c = 0; c < VEC; c++) {
      const int i = i0 + c;
      x[h * VEC + c] = (g < rv.nvec && i >= 0 && i < rv.V) ? xv[c] : -INFINITY;
    }
  }
  if (p1_body<TONE, CUT>(x, k, a)) p1_append<VEC, true>(x, gv * VEC - rv.shift, rv.V, k);
  p1_piece_end<CUT>(st, sp.nst, lane, part_w, a);
}
// The pass: part_w[piece] (this warp's pieces) receives the mass of each piece (of all its logits
// without a cut, of those above the window with one); the lane-private sum of all mass comes back
// in Ssum, the lane's running maximum in vmax.
template <typename T, bool TONE, bool CUT>
__device__ __noinline__ void wide_onepass_stream(const WSpan& sp, const RowView<T>& rv, int lane, const P1Consts& k_in,
                                                 double* part_w, double& Ssum, float& vmax) {
  constexpr int VEC = Elem<T>::VEC, EPI = 8 / VEC, SV = 32 * EPI;
  const P1Consts k = k_in;
  P1Acc a;
  a.tot = 0.0; a.kep = 0.0; a.stot = 0.0; a.vmax = -INFINITY;
  const int nst = sp.nst, clean_lo = sp.clean_lo, clean_hi = sp.clean_hi;
  int st = 0;
  for (; st < clean_lo; st++) p1_edge_step<T, TONE, CUT>(sp, rv, lane, st, k, part_w, a);
  // Clean steps: every vector exists and none is the row's first or last. Two register buffers used
  // in turn (no copies between them): a step's vectors are asked for two steps ahead, and L2 is asked
  // for the lines W1_PF steps ahead. The steady loop runs while both refills stay inside the clean
  // range; what is left is loaded on the spot. (Four steps in flight, two of them in a cp.async ring
  // in shared memory, were measured and changed nothing: the pass is bound by instruction issue.)
  auto unpack8 = [&](const uint4& q0, const uint4& q1, float* x) {
    if (EPI == 2) { Elem<T>::unpack(q0, x); Elem<T>::unpack(q1, x + 4 * (EPI - 1)); }
    else Elem<T>::unpack(q0, x);
  };
  if (clean_hi - clean_lo >= 4) {
    const uint4* p = sp.lane_src + clean_lo * SV;
    int i_first = (sp.first + clean_lo * SV + lane) * VEC - rv.shift;
    const int st_end = clean_lo + ((clean_hi - clean_lo - 2) & ~1);   // steps [clean_lo, st_end) in pairs, refills < clean_hi
    uint4 a0 = __ldg(p), a1 = a0, b0, b1;
    if (EPI == 2) a1 = __ldg(p + 32);
    b0 = __ldg(p + SV); b1 = b0;
    if (EPI == 2) b1 = __ldg(p + SV + 32);
    const int pf_end = clean_hi - W1_PF;                      // last step that may still ask for step + W1_PF
    float x[8];
#pragma unroll 1
    for (; st < st_end; st += 2) {
      unpack8(a0, a1, x);
      a0 = __ldg(p + 2 * SV); if (EPI == 2) a1 = __ldg(p + 2 * SV + 32);
      if (W1_PF > 0 && st + 1 < pf_end) {
        l2_prefetch(p + W1_PF * SV); l2_prefetch(p + (W1_PF + 1) * SV);
        if (EPI == 2) { l2_prefetch(p + W1_PF * SV + 32); l2_prefetch(p + (W1_PF + 1) * SV + 32); }
      }
      if (p1_body<TONE, CUT>(x, k, a)) p1_append<VEC, false>(x, i_first, 0, k);
      p1_piece_end<CUT>(st, nst, lane, part_w, a);
      unpack8(b0, b1, x);
      b0 = __ldg(p + 3 * SV); if (EPI == 2) b1 = __ldg(p + 3 * SV + 32);
      if (p1_body<TONE, CUT>(x, k, a)) p1_append<VEC, false>(x, i_first + SV * VEC, 0, k);
      p1_piece_end<CUT>(st + 1, nst, lane, part_w, a);
      p += 2 * SV;
      i_first += 2 * SV * VEC;
    }
    unpack8(a0, a1, x);
    if (p1_body<TONE, CUT>(x, k, a)) p1_append<VEC, false>(x, i_first, 0, k);
    p1_piece_end<CUT>(st, nst, lane, part_w, a);
    unpack8(b0, b1, x);
    if (p1_body<TONE, CUT>(x, k, a)) p1_append<VEC, false>(x, i_first + SV * VEC, 0, k);
    p1_piece_end<CUT>(st + 1, nst, lane, part_w, a);
    st += 2;
  }
  for (; st < nst; st++) p1_edge_step<T, TONE, CUT>(sp, rv, lane, st, k, part_w, a);
  Ssum = CUT ? a.tot : a.stot;
  vmax = a.vmax;
}

// false: the row takes the two-pass front end (nothing of the row has been decided or written).
template <typename T>
__device__ __noinline__ bool wide_front_onepass(const BatchArgs& BA, const int64_t row_id, const RowView<T>& rv, const WSpan& sp,
                                                unsigned char* dyn, WideShared& sh, const RowCfg cfg, const bool cut_on,
                                                const int span, const int ppw, const int npiece, OnePassOut& out, uint32_t* clk) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  long long tprev = clock64();
  auto stamp = [&](int slot) { const long long now = clock64(); clk[slot] = static_cast<uint32_t>(now - tprev); tprev = now; };
  auto fail = [&](int why) -> bool { out.nz = why; return false; };   // why the row takes two passes (diagnostics)
  constexpr int VEC = Elem<T>::VEC, EPI = 8 / VEC, SV = 32 * EPI;
  bu::Scratch& sc = sh.sc;
  const double* s_tab = sh.tab;
  uint32_t* hist = reinterpret_cast<uint32_t*>(dyn + W_OFF_HIST);
  uint2* zl = reinterpret_cast<uint2*>(dyn + W_OFF_ZONE);                 // W_ZCAP1 entries
  double* part = reinterpret_cast<double*>(dyn + W_OFF_PART);
  const float Tm = cfg.temperature;
  const int mode = cfg.topp_mode;
  const double plim = (mode == 0) ? static_cast<double>(cfg.top_p) * 1.5 : static_cast<double>(cfg.top_p);
  const bool t_is_one = (Tm == 1.0f);
  const uint32_t tb = __float_as_uint(Tm);
  if (!t_is_one && !(Tm >= 9.5367431640625e-7f && Tm <= 1048576.0f && (tb & 0x7fffffu) != 0x7fffffu)) return fail(1);
  if (rv.nvec < W_NW * SV * 8) return fail(2);                              // short rows: nothing to gain

  // ask L2 for the sample's lines now: the sweep below then finds them there
  if (cut_on) {
    for (int st = 0; st < sp.nst; st += W1_STRIDE) {
#pragma unroll
      for (int h = 0; h < EPI; h++) {
        const int g = sp.first + st * SV + lane + 32 * h;
        if (g < rv.nvec) asm volatile("prefetch.global.L2::evict_last [%0];" :: "l"(rv.vbase + g));
      }
    }
  }
  // ---- a first look: every warp's first step gives a value near the row maximum and the range
  float smax = -INFINITY, smin = INFINITY;
  bool snan = false;
#pragma unroll
  for (int h = 0; h < EPI; h++) {
    const int g = sp.first + 32 * h + lane;
    if (sp.nst > 0 && g < rv.nvec) rv.visit(g, [&](float xv, int) { smax = fmaxf(smax, xv); smin = fminf(smin, xv); snan |= (xv != xv); });
  }
  if (bu::max_i<W_NW>(snan ? 1 : 0, sc, tid)) return fail(3);
  smax = okey_to_float(static_cast<uint32_t>(bu::max_u64<W_NW>(static_cast<unsigned long long>(okey(smax)), sc, tid)));
  smin = okey_to_float(static_cast<uint32_t>(bu::min_u64<W_NW>(static_cast<unsigned long long>(okey(smin)), sc, tid)));
  const float r0 = smax - smin;
  if (!(r0 >= 0.0f && r0 < 1e30f && fabsf(smax) < 1e30f)) return fail(3);
  // the anchor of the fast exponentials: where the row maximum is expected (for bell-shaped rows the
  // maximum of the whole row lies about an eighth of the first look's range above its maximum)
  const float as = scale_t(smax + 0.125f * r0, Tm);
  if (!(fabsf(as) < 1e30f)) return fail(3);

  stamp(0);
  P1Consts k;
  k.as = as; k.Tm = Tm; k.yT = t_is_one ? 1.0f : __frcp_rn(Tm);
  k.xA = -INFINITY; k.xmid = 0.0f; k.xhalf = -1.0f;
  k.xB = -INFINITY; k.zl_s = smem_addr(zl); k.zcnt_s = smem_addr(&sh.cnt);
  float xA = -INFINITY, xB = -INFINITY;
  double eps = W1_EPS_FIXED + W1_EPS_PER_D * 9.7;
  if (cut_on) {
    // ---- the sample: count histogram over 4096 buckets of (anchor - x), anchor half of the first
    // look's range above its maximum, bucket width so that the range and as much again below fit
    const float margin = fmaxf(0.5f * r0, 1e-3f * fmaxf(1.0f, fabsf(smax)));
    const float hs = 4094.0f / fmaxf(2.25f * r0 + margin, 1e-30f);
    const float Tc = Tm;
    // bucket width in units of x / T between 2^-16 and 2^-7
    const float hs_c = fminf(fmaxf(hs, 128.0f / Tc), 65536.0f / Tc);
    if (!(hs_c > 1e-30f && hs_c < 1e30f)) return fail(4);
    const float nhs = -hs_c;
    const float hc = fmaf(smax + margin, hs_c, W1_MAGIC);
    if (!(fabsf(hc) < 1e30f)) return fail(4);
    for (int j = tid; j < W_NB; j += W_NT) hist[j] = 0;
    __syncthreads();
    float svmax = -INFINITY;
    const uint32_t hb = smem_addr(hist);
    // four sampled steps at a time: their loads are in flight together
    for (int st0 = 0; st0 < sp.nst; st0 += 4 * W1_STRIDE) {
      uint4 q[4 * EPI];
#pragma unroll
      for (int u = 0; u < 4; u++) {
#pragma unroll
        for (int h = 0; h < EPI; h++) {
          const int g = sp.first + (st0 + u * W1_STRIDE) * SV + lane + 32 * h;
          q[u * EPI + h] = __ldg(rv.vbase + min(g, rv.nvec - 1));
        }
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        if (st0 + u * W1_STRIDE < sp.nst) {
#pragma unroll
          for (int h = 0; h < EPI; h++) {
            const int g = sp.first + (st0 + u * W1_STRIDE) * SV + lane + 32 * h;
            if (g < rv.nvec) {
              rv.visit_raw(q[u * EPI + h], g, [&](float xv, int, int) {
                svmax = maxnan(svmax, xv);
                asm volatile("red.shared.add.u32 [%0], 1;" :: "r"(bucket_off1(xv, nhs, hc) + hb) : "memory");
              });
            }
          }
        }
      }
    }
    const int bad_s = bu::max_i<W_NW>((svmax != svmax) ? 1 : 0, sc, tid);  // also orders the histogram
    stamp(1);
    svmax = okey_to_float(static_cast<uint32_t>(bu::max_u64<W_NW>(static_cast<unsigned long long>(okey(svmax)), sc, tid)));
    if (bad_s || !(fmaf(svmax, nhs, hc) >= W1_MAGIC)) return fail(6);       // NaN, or a sampled logit above the anchor
    // ---- the window from the sample's histogram: bucket b holds y = (anchor' - x) hs in
    // [b - 1/8, b + 7/8], a width of w = 1 / (hs T) in units of x / T; masses relative to
    // exp(anchor' / T) lie between exp(-(b + 7/8) w) and exp(-(b - 1/8) w). The bracket is the one of
    // the two-pass front end, widened by the sampling error of a mass fraction estimated from n logits.
    // Placing the window is a matter of speed, not of correctness (the pass checks it on the whole
    // row): f32 and the fast exponential do.
    constexpr int PER = W_NB / W_NT;
    const double wd = 1.0 / (static_cast<double>(hs_c) * static_cast<double>(Tm));
    const float wl2 = static_cast<float>(wd * 1.4426950408889634);        // bucket width in units of log2
    const float ratio = ex2_approx(-wl2);
    const float edge0 = ex2_approx(-(static_cast<float>(tid * PER) - 0.125f) * wl2);
    float slo = 0.0f, shi = 0.0f;
    int cnt_loc = 0, lowest = -1, top = W_NB;
    uint32_t cnt[PER];                                                    // this thread's buckets, read once
    {
      const uint4* mine = reinterpret_cast<const uint4*>(hist) + tid * (PER / 4);
#pragma unroll
      for (int q = 0; q < PER / 4; q++) { const uint4 v = mine[q]; cnt[4 * q] = v.x; cnt[4 * q + 1] = v.y; cnt[4 * q + 2] = v.z; cnt[4 * q + 3] = v.w; }
    }
    {
      float edge = edge0;
#pragma unroll
      for (int j = 0; j < PER; j++) {
        const int b = tid * PER + j;
        const int ci = static_cast<int>(cnt[j]);
        const float c = static_cast<float>(ci);
        const float ehi = edge;
        edge *= ratio;
        const float elo = (b == W_NB - 1) ? 0.0f : edge;
        slo = fmaf(c, elo, slo); shi = fmaf(c, ehi, shi);
        cnt_loc += ci;
        if (ci) { lowest = b; top = min(top, b); }
      }
    }
    double ex_lo, ex_hi, tot_lo, tot_hi;
    bu::scan_excl_d2<W_NW>(static_cast<double>(slo), static_cast<double>(shi), ex_lo, ex_hi, tot_lo, tot_hi, sc, tid);
    const int nsamp = bu::sum_i<W_NW>(cnt_loc, sc, tid);
    int nlow = -lowest;                                                   // the lowest populated bucket as a minimum of negatives
    bu::min_i2<W_NW>(top, nlow, sc, tid);
    lowest = -nlow;
    if (nsamp < 4096 || !(tot_lo > 0.0)) return fail(7);
    // a few heavy tokens: the sample cannot place the cut (one token above a thousandth of the mass)
    const double heavy = static_cast<double>(ex2_approx(-(static_cast<float>(top) - 0.125f) * wl2));
    if (heavy > 1e-3 * tot_lo) return fail(8);
    // five standard errors of a mass fraction estimated from nsamp logits
    const double delta = 5.0 * sqrt(plim * fabs(1.0 - plim) / static_cast<double>(nsamp)) + 4.0 / static_cast<double>(nsamp);
    const float p_lo = static_cast<float>(plim - delta), p_hi = static_cast<float>(plim + delta);
    if (!(p_lo > 0.0f)) return fail(9);
    int b1 = W_NB - 1, b2 = W_NB - 1, wcount = 0;
    {
      float edge = edge0, a_lo = static_cast<float>(ex_lo), a_hi = static_cast<float>(ex_hi);
      const float t_lo = static_cast<float>(tot_lo), t_hi = static_cast<float>(tot_hi);
#pragma unroll
      for (int j = 0; j < PER; j++) {
        const int b = tid * PER + j;
        const float c = static_cast<float>(cnt[j]);
        const float ehi = edge;
        edge *= ratio;
        const float elo = (b == W_NB - 1) ? 0.0f : edge;
        a_lo = fmaf(c, elo, a_lo); a_hi = fmaf(c, ehi, a_hi);
        const float den_hi = a_hi + (t_lo - a_lo), den_lo = a_lo + (t_hi - a_hi);
        const bool c1 = a_hi >= p_lo * den_hi, c2 = a_lo >= p_hi * den_lo;
        if (c1 && a_hi > 0.0f) b1 = min(b1, b);
        if (c2 && a_lo > 0.0f) b2 = min(b2, b);
      }
    }
    bu::min_i2<W_NW>(b1, b2, sc, tid);
    if (b2 < b1) b2 = b1;
    if (b1 > 0) b1--;                                                     // one bucket of slack for the f32 sums
    if (b2 < W_NB - 1) b2++;
#pragma unroll
    for (int j = 0; j < PER; j++) { const int b = tid * PER + j; if (b >= b1 && b <= b2) wcount += static_cast<int>(cnt[j]); }
    wcount = bu::sum_i<W_NW>(wcount, sc, tid);
    // the window must stay small: its logits go through the exact list
    if (static_cast<long long>(wcount) * W1_STRIDE > (W_ZCAP1 * 13) / 16) return fail(10);
    bool ok = true;
    xA = bucket_floor1(b1 - 1, nhs, hc, ok);
    xB = bucket_floor1(b2, nhs, hc, ok);
    if (!ok) return fail(11);
    k.xA = xA; k.xB = xB;
    const float xAc = fminf(xA, 3.0e38f), xBc = fmaxf(xB, -3.0e38f);
    k.xmid = 0.5f * xAc + 0.5f * xBc;
    k.xhalf = (0.5f * xAc - 0.5f * xBc) * 1.000001f + 1e-30f;
    if (lowest >= 0 && lowest < W_NB - 1) {
      const double dmax = (static_cast<double>(lowest) + 1.0) * wd + 1e-3;   // from the histogram's anchor down
      eps = W1_EPS_FIXED + W1_EPS_PER_D * fmin(9.7, dmax);
    }
    __syncthreads();                                                      // the histogram area becomes the record list
  }

  stamp(2);
  // ---- the pass
  if (tid < npiece) part[tid] = 0.0;                                      // pieces past the row's end stay empty
  if (tid == 0) sh.cnt = 0;
  __syncthreads();
  double Ssum = 0.0;
  float vmax = -INFINITY;
  double* part_w = part + warp * ppw;
  if (cut_on) {
    if (t_is_one) wide_onepass_stream<T, true, true>(sp, rv, lane, k, part_w, Ssum, vmax);
    else wide_onepass_stream<T, false, true>(sp, rv, lane, k, part_w, Ssum, vmax);
  } else {
    if (t_is_one) wide_onepass_stream<T, true, false>(sp, rv, lane, k, part_w, Ssum, vmax);
    else wide_onepass_stream<T, false, false>(sp, rv, lane, k, part_w, Ssum, vmax);
  }
  __syncthreads();
  stamp(6);
  const int anynan = bu::max_i<W_NW>((vmax != vmax) ? 1 : 0, sc, tid);
  const float xmax = okey_to_float(static_cast<uint32_t>(bu::max_u64<W_NW>(static_cast<unsigned long long>(okey(vmax)), sc, tid)));
  const float m = scale_t(xmax, Tm);
  if (anynan || !(fabsf(m) < INFINITY)) return fail(12);                     // the two-pass front end reports such rows
  // the fast sums round x/T - anchor where upstream rounds x/T - max: the two must be close for the
  // heavy logits to keep the error budget (2e-7 per unit of distance)
  if (!(fabsf(m - as) <= 2.0f)) return fail(13);
  int nz = 0;
  double S = bu::sum_d<W_NW>(Ssum, sc, tid);
  nz = sh.cnt;
  if (!(S > 0.0) || !(S < 1e300)) return fail(14);
  // everything so far is relative to exp(anchor); the tail works relative to exp(max)
  const double cf = exp(static_cast<double>(as) - static_cast<double>(m));
  S *= cf;
  if (tid < npiece) part[tid] *= cf;
  __syncthreads();
  double Ktot = 0.0;
  if (cut_on) {
    Ktot = bu::sum_d<W_NW>((tid < npiece) ? part[tid] : 0.0, sc, tid);
    // ---- the window's logits: x -> d = x / T - max, in place, and their mass
    if (nz > W_ZCAP1 || nz == 0) return fail(5);
    double zmass = 0.0;
    for (int j = tid; j < nz; j += W_NT) {
      const uint2 e = zl[j];
      const float d = scale_t(__uint_as_float(e.x), Tm) - m;
      zl[j] = make_uint2(__float_as_uint(d), e.y);
      zmass += exp_safe(d, s_tab);
    }
    zmass = bu::sum_d<W_NW>(zmass, sc, tid);
    // the cut must lie inside the window by more than the error of the sums
    const double etol = 1e-12 + 2.0 * plim * fabs(1.0 - plim) * eps + 1e-9;
    if (!(Ktot / S < plim - etol) || !((Ktot + zmass) / S > plim + etol)) {
      if (!(xB == -INFINITY && Ktot / S < plim - etol)) return fail(15);     // a window open at the bottom holds whatever is left
    }
  }
  stamp(7);
  out.m = m; out.S = S; out.Ktot = Ktot; out.nz = nz; out.xA = xA; out.xB = xB; out.eps = eps;
  return true;
}

template <typename T>
__device__ void wide_row(const BatchArgs& BA, const int64_t row_id, unsigned char* dyn, WideShared& sh,
                         unsigned long long pol_keep, unsigned long long pol_drop) {
  const KernelArgs& A = BA.k;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int V = A.V;
  constexpr int VEC = Elem<T>::VEC;
  constexpr int SV = 32 * (8 / VEC);                         // vectors of one warp-step
  constexpr int PV = W_G * SV;                               // vectors of one piece
  const T* row = static_cast<const T*>(A.logits) + row_id * A.row_stride;
  RowView<T> rv;
  rv.init(row, V);
  bu::Scratch& sc = sh.sc;
  const double* s_tab = sh.tab;
  uint32_t* hist = reinterpret_cast<uint32_t*>(dyn + W_OFF_HIST);
  uint2* zl = reinterpret_cast<uint2*>(dyn + W_OFF_ZONE);
  unsigned long long* zk = reinterpret_cast<unsigned long long*>(dyn + W_OFF_ZONE);
  double* ebs = reinterpret_cast<double*>(dyn + W_OFF_EB);
  double* part = reinterpret_cast<double*>(dyn + W_OFF_PART);   // [warp][piece] kept mass, row order
  const double QNAN = __longlong_as_double(0x7ff8000000000000ll);

  const RowCfg cfg = A.cfgs[row_id];
  const float Tm = cfg.temperature;
  const bool topp_on = (cfg.top_p > 0.0f && cfg.top_p < 1.0f);
  const int mode = cfg.topp_mode;
  const double u = A.uniforms[row_id];
  const double plim = (mode == 0) ? static_cast<double>(cfg.top_p) * 1.5 : static_cast<double>(cfg.top_p);
  // mode A prunes only while the mass exceeds 1.5p; the mass starts at 1 up to ~1e-11 of rounding
  // and 1.5*float(p) is never that close to 1
  const bool cut_on = topp_on && !(mode == 0 && plim >= 1.0);
  const bool t_is_one = (Tm == 1.0f);
  uint32_t flags = FLAG_GENERAL_PATH;
  RowDebug dbg;
  dbg.sum_exp = 0; dbg.resum = 1.0; dbg.edge_lo = 0; dbg.edge_hi = 0; dbg.kept = 0;
  dbg.max_scaled = 0; dbg.threshold = __int_as_float(0x7fc00000); dbg.path = 2;
  for (int q = 0; q < 8; q++) dbg.reserved[q] = 0;
  long long tprev = clock64();
  auto stamp = [&](int slot) { const long long now = clock64(); dbg.reserved[slot] = static_cast<uint32_t>(now - tprev); tprev = now; };
  auto write_row = [&](int id, uint32_t fl) {
    if (tid == 0) {
      A.out_ids[row_id] = id;
      if (A.out_flags) A.out_flags[row_id] = fl;
      if (A.out_debug) A.out_debug[row_id] = dbg;
    }
  };
  auto fill_probs_row = [&](double v) {
    if (A.out_probs) {
      double* pr = A.out_probs + row_id * static_cast<int64_t>(V);
      for (int i = tid; i < V; i += W_NT) pr[i] = v;
    }
  };

  // the warp's span: 1/W_NW of the row, rounded up to whole steps
  const int span = (((rv.nvec + W_NW - 1) / W_NW + SV - 1) / SV) * SV;
  const int steps_max = span / SV;
  if (steps_max > W_MAX_STEPS) {
    if (tid == 0) hand_to_single(BA, row_id);
    return;
  }
  const int ppw = (steps_max + W_G - 1) / W_G;               // pieces per warp
  const int npiece = W_NW * ppw;
  const WSpan sp = make_span<T>(rv, warp * span, span, lane);

  // What the tail needs of the row, from either front end.
  float m = 0.0f, dlow = -INFINITY;
  float dA = -INFINITY, dB = -INFINITY;    // certainly kept: d >= dA; zone: dB <= d < dA; dropped: d < dB
  bool fast_ok = false;
  double S = 0.0, Ktot = 0.0;
  int nz = 0;
  // one-pass front end: thresholds on the raw logits (xs), its own error bound and list capacity
  bool xs = false;
  int onepass_why = 0;
  float xA = -INFINITY, xB = -INFINITY;
  double eps_rel = W_EXP_REL_ERR;
  int zcap = W_ZCAP;
  {
    OnePassOut fo;
    fo.nz = 0;
    if (wide_front_onepass<T>(BA, row_id, rv, sp, dyn, sh, cfg, cut_on, span, ppw, npiece, fo, dbg.reserved)) {
      xs = true;
      m = fo.m; S = fo.S; Ktot = fo.Ktot; nz = fo.nz; xA = fo.xA; xB = fo.xB; eps_rel = fo.eps; zcap = W_ZCAP1;
      fast_ok = true;
      dlow = -INFINITY;
      dB = (xB == -INFINITY) ? -INFINITY : 0.0f;             // "logits below the zone may exist"
      dbg.max_scaled = m;
      dbg.path = 3;
    } else {
      onepass_why = fo.nz;
    }
  }
  if (!xs) {
  // ---- a sample of the row (every warp's first step) gives an upper estimate of the maximum
  // and the bucket width, so that pass 1 can already count the histogram the cut needs
  bool anchored = false;
  float anchor = 0.0f, scale = 128.0f, width = 0.0078125f, dclamp = -31.99f;
  auto set_scale = [&](float range) {      // power of two (1/128 .. 1/65536) at which `range` just fits
    int jexp = 7;
    const float q = 4094.0f / range;                         // +Inf for range 0, 0 for an infinite range
    if (q >= 65536.0f) jexp = 16; else if (q >= 128.0f) jexp = ilogbf(q);
    scale = __int_as_float((127 + jexp) << 23);
    width = 1.0f / scale;
    dclamp = -4095.4f * width;
  };
  if (cut_on) {
    for (int j = tid; j < W_NB; j += W_NT) hist[j] = 0;
    float smax = -INFINITY, smin = INFINITY;
    bool snan = false;
#pragma unroll
    for (int h = 0; h < 8 / VEC; h++) {
      const int g = sp.first + 32 * h + lane;
      if (sp.nst > 0 && g < rv.nvec) rv.visit(g, [&](float xv, int) { smax = fmaxf(smax, xv); smin = fminf(smin, xv); snan |= (xv != xv); });
    }
    const int bad_sample = bu::max_i<W_NW>(snan ? 1 : 0, sc, tid);
    smax = okey_to_float(static_cast<uint32_t>(bu::max_u64<W_NW>(static_cast<unsigned long long>(okey(smax)), sc, tid)));
    smin = okey_to_float(static_cast<uint32_t>(bu::min_u64<W_NW>(static_cast<unsigned long long>(okey(smin)), sc, tid)));
    const float s_hi = scale_t(smax, Tm), s_lo = scale_t(smin, Tm);
    const float r0 = s_hi - s_lo;
    if (!bad_sample && r0 >= 0.0f && r0 < 1e30f && fabsf(s_hi) < 1e30f) {
      // half the sample's range above its maximum (a maximum beyond that costs an extra pass),
      // a quarter below its minimum (what lies lower shares the last bucket)
      const float margin = fmaxf(0.5f * r0, 1e-3f * fmaxf(1.0f, fabsf(s_hi)));
      anchor = s_hi + margin;
      set_scale(r0 + 1.5f * margin);
      anchored = true;
    }
  }

  // ---- pass 1: max, min, NaN (from HBM; L2 is asked to keep the row)
  float xmax = -INFINITY, xmin = INFINITY;
  bool nan_seen = false;
  {
    const uint32_t hb = smem_addr(hist) - 0x4B000000u * 4u;
    if (!anchored) wide_pass1<T, false, true>(sp, rv, pol_keep, lane, hb, anchor, Tm, scale, dclamp, xmax, xmin, nan_seen);
    else if (t_is_one) wide_pass1<T, true, true>(sp, rv, pol_keep, lane, hb, anchor, Tm, scale, dclamp, xmax, xmin, nan_seen);
    else wide_pass1<T, true, false>(sp, rv, pol_keep, lane, hb, anchor, Tm, scale, dclamp, xmax, xmin, nan_seen);
  }
  __syncthreads();
  const int anynan = bu::max_i<W_NW>(nan_seen ? 1 : 0, sc, tid);
  xmax = okey_to_float(static_cast<uint32_t>(bu::max_u64<W_NW>(static_cast<unsigned long long>(okey(xmax)), sc, tid)));
  xmin = okey_to_float(static_cast<uint32_t>(bu::min_u64<W_NW>(static_cast<unsigned long long>(okey(xmin)), sc, tid)));
  m = scale_t(xmax, Tm);
  dbg.max_scaled = m;
  stamp(0);
  // A NaN anywhere, or an infinite maximum, makes the softmax sum NaN upstream
  // (generate.go:173-181): every comparison of the walk fails, result n-1 (:239).
  if (anynan || !(fabsf(m) < INFINITY)) {
    fill_probs_row(QNAN);
    dbg.sum_exp = QNAN;
    write_row(V - 1, flags | FLAG_NONFINITE | FLAG_FALLBACK);
    return;
  }
  dlow = scale_t(xmin, Tm) - m;                  // smallest d of the row (-Inf with a -Inf logit)
  fast_ok = (dlow > -31.9f);                      // every d inside the bucket table's range

  // ---- bracket of the cut from the count histogram
  if (cut_on) {
    // The histogram of pass 1 counts q = s - anchor; it stands when no logit lies above the anchor.
    // Mass bounds relative to exp(anchor) serve as well as bounds relative to exp(max): only their
    // ratios are used. q and d are each rounded once, so a logit's true mass can differ from
    // exp(q) exp(anchor - max) by the factor exp(+-2^-24 * 64): `slack` covers it.
    double slack = 1e-5;
    if (!(anchored && m <= anchor)) {
      anchored = false;
      slack = 1e-7;
      set_scale(-dlow);
      __syncthreads();
      for (int j = tid; j < W_NB; j += W_NT) hist[j] = 0;
      __syncthreads();
      if (t_is_one) wide_pass2<T, true>(sp, rv, pol_keep, lane, smem_addr(hist) - 0x4B000000u * 4u, m, Tm, scale, dclamp);
      else wide_pass2<T, false>(sp, rv, pol_keep, lane, smem_addr(hist) - 0x4B000000u * 4u, m, Tm, scale, dclamp);
    }
    __syncthreads();
    constexpr int PER = W_NB / W_NT;                         // buckets per thread
    // bucket b holds q (or d) in [-(b+.5) width, -(b-.5) width], the last one everything below.
    // Its members' masses lie between edge(b+1) and edge(b), edge(k) = exp(-(k-.5) width): one
    // exponential per thread, the next edges by the common ratio (rounding far inside `slack`).
    // The walk over the thread's buckets is done twice (sums, then the tests against the scanned
    // sums) rather than kept in registers.
    const double ratio = exp_safe(-width, s_tab);
    const double edge0 = exp_safe(-(tid * PER - 0.5f) * width, s_tab);
    double slo = 0.0, shi = 0.0;
    {
      double edge = edge0;
#pragma unroll 4
      for (int j = 0; j < PER; j++) {
        const int b = tid * PER + j;
        const double c = static_cast<double>(hist[b]);
        const double ehi = fmin(edge, 1.0) * (1.0 + slack);
        edge *= ratio;
        const double elo = (b == W_NB - 1) ? 0.0 : edge * (1.0 - slack);
        slo += c * elo; shi += c * ehi;
      }
    }
    double ex_lo, ex_hi, tot_lo, tot_hi;
    bu::scan_excl_d2<W_NW>(slo, shi, ex_lo, ex_hi, tot_lo, tot_hi, sc, tid);
    int b1 = W_NB - 1, b2 = W_NB - 1;
    const double p_lo = plim * (1.0 - 1e-9), p_hi = plim * (1.0 + 1e-9);
    {
      double edge = edge0, a_lo = ex_lo, a_hi = ex_hi;
#pragma unroll 4
      for (int j = 0; j < PER; j++) {
        const int b = tid * PER + j;
        const double c = static_cast<double>(hist[b]);
        const double ehi = fmin(edge, 1.0) * (1.0 + slack);
        edge *= ratio;
        const double elo = (b == W_NB - 1) ? 0.0 : edge * (1.0 - slack);
        a_lo += c * elo; a_hi += c * ehi;
        // largest / smallest possible mass fraction through bucket b against the limit, as products
        const double den_hi = a_hi + (tot_lo - a_lo), den_lo = a_lo + (tot_hi - a_hi);
        bool c1, c2;
        if (mode == 0) { c1 = a_hi > p_lo * den_hi; c2 = a_lo > p_hi * den_lo; }
        else           { c1 = a_hi >= p_lo * den_hi; c2 = a_lo >= p_hi * den_lo; }
        if (c1 && a_hi > 0.0) b1 = min(b1, b);
        if (c2 && a_lo > 0.0) b2 = min(b2, b);
      }
    }
    bu::min_i2<W_NW>(b1, b2, sc, tid);
    if (b2 < b1) b2 = b1;
    const float qA = bucket_floor_w(b1 - 1, scale, dclamp);  // certainly kept: q >= qA
    const float qB = bucket_floor_w(b2, scale, dclamp);      // certainly dropped: q < qB
    if (!anchored) {
      dA = qA; dB = qB;
    } else {
      // Thresholds on d = rn(s - max) that are at least as cautious as those on q = rn(s - anchor):
      // d >= dA must imply q >= qA, and q >= qB must imply d >= dB. Both roundings are monotone:
      // s - anchor >= qA implies q >= qA, and q >= qB implies s - anchor >= pred(qB).
      if (qA == INFINITY) dA = INFINITY;
      else dA = nextafterf(__double2float_ru(static_cast<double>(anchor) + static_cast<double>(qA) - static_cast<double>(m)), INFINITY);
      if (qB == -INFINITY) dB = -INFINITY;
      else dB = nextafterf(__double2float_rd(static_cast<double>(anchor) + static_cast<double>(nextafterf(qB, -INFINITY)) - static_cast<double>(m)), -INFINITY);
      if (dA > 0.0f) dA = INFINITY;                          // no d reaches it: nothing is certainly kept
    }
  }
  stamp(1);

  // ---- pass 3: exponentials (last use of the row: evict-first)
  // exponential table: sixteen conflict-free copies of the first 128 entries when the row's range
  // allows it, else the plain 1024 entries
  const bool eb_rep = fast_ok && (dlow > -(W_EB_REP_ENTRIES - 2.0f) / 32.0f);
  if (eb_rep) {
    for (int j = tid; j < W_EB_REP * W_EB_REP_ENTRIES; j += W_NT) ebs[j] = __ldg(BA.eb_table + j / W_EB_REP);
  } else if (fast_ok) {
    for (int j = tid; j < NB1; j += W_NT) ebs[j] = __ldg(BA.eb_table + j);
  }
  if (tid < npiece) part[tid] = 0.0;                         // pieces past the row's end stay empty
  if (tid == 0) sh.cnt = 0;
  __syncthreads();
  double Ssum = 0.0, Ksum = 0.0;
  const uint32_t eb_mul = eb_rep ? 8u * W_EB_REP : 8u;
  const uint32_t eb_bias = smem_addr(ebs) + (eb_rep ? 8u * (lane & (W_EB_REP - 1)) : 0u) - 0x4B000000u * eb_mul;
#define GS_P3(F, O, C) wide_pass3<T, F, O, C>(sp, rv, pol_drop, lane, warp, m, Tm, dA, dB, eb_mul, eb_bias, s_tab, part, ppw, zl, &sh.cnt, Ssum, Ksum)
  if (cut_on) {
    if (fast_ok) { if (t_is_one) GS_P3(true, true, true); else GS_P3(true, false, true); }
    else         { if (t_is_one) GS_P3(false, true, true); else GS_P3(false, false, true); }
  } else {
    if (fast_ok) { if (t_is_one) GS_P3(true, true, false); else GS_P3(true, false, false); }
    else         { if (t_is_one) GS_P3(false, true, false); else GS_P3(false, false, false); }
  }
#undef GS_P3
  __syncthreads();
  if (lane != 0) Ksum = 0.0;                                 // kept mass is already warp-reduced into lane 0
  double unused = 0.0;
  S = Ssum; Ktot = Ksum;
  bu::sum_d3<W_NW>(S, Ktot, unused, sc, tid);
  nz = sh.cnt;
  stamp(2);
  dbg.reserved[6] = static_cast<uint32_t>(onepass_why);     // why the row took two passes
  }  // two-pass front end
  // A zone that outgrew the list (long runs of equal logits around the cut): the same selection
  // runs over the row itself, one more pass per round.
  const bool big = cut_on && nz > zcap;
  dbg.sum_exp = S;

  // ---- exact cut inside the zone by weighted selection
  unsigned long long cut_key = 0ull;       // zone entries are kept when key < cut_key, or == with cut_incl
  int cut_incl = 0;
  bool bad = false;
  if (big && xs) {
    if (tid == 0) hand_to_single(BA, row_id);
    return;
  } else if (big) {
    if (!wide_big_zone<T>(sp, rv, pol_keep, sh, hist, part, s_tab, m, Tm, dA, dB, dlow, mode, plim, S, Ktot, fast_ok,
                          span, ppw, cut_key, cut_incl, flags)) {
      if (tid == 0) hand_to_single(BA, row_id);
      return;
    }
  } else if (cut_on && nz > 0) {
    for (int j = tid; j < nz; j += W_NT) {                   // entries -> keys, in place
      const uint2 e = zl[j];
      zk[j] = zone_key(__uint_as_float(e.x), static_cast<int>(e.y), mode);
    }
    __syncthreads();
    // G(c) = Ktot + mass{key <= c} rises along the zone order. Both flavours need the first key c*
    // where G crosses: mode B (first G/S >= p) keeps through c*, mode A (first G/S > 1.5p) keeps
    // everything before it. Narrow [lo, hi] around c* with linear sub-buckets until at most 32
    // keys remain, then one warp finishes.
    auto crossed = [&](double g) -> bool { return mode == 0 ? (g / S > plim) : (g / S >= plim); };
    if (Ktot > 0.0 && crossed(Ktot)) bad = true;             // the bracket was wrong
    double* sm = reinterpret_cast<double*>(hist);            // [W_NSUB] mass per sub-bucket
    int* scn = reinterpret_cast<int*>(hist) + 2 * W_NSUB;    // [W_NSUB] count per sub-bucket
    unsigned long long lo = ~0ull, hi = 0ull;
    for (int j = tid; j < nz; j += W_NT) { const unsigned long long k = zk[j]; lo = k < lo ? k : lo; hi = k > hi ? k : hi; }
    lo = bu::min_u64<W_NW>(lo, sc, tid);
    hi = bu::max_u64<W_NW>(hi, sc, tid);
    double gbase = Ktot;                                     // Ktot + mass of keys below lo; never crossed
    int inrange = nz;
    bool all_in = false;
    for (int iter = 0; iter < 8 && inrange > 32 && !bad && !all_in; iter++) {
      const unsigned long long spn = hi - lo;
      int shf = 0;
      while (shf < 63 && (spn >> shf) >= static_cast<unsigned long long>(W_NSUB)) shf++;
      __syncthreads();
      sm[tid] = 0.0; scn[tid] = 0;                           // W_NT == W_NSUB
      __syncthreads();
      for (int j = tid; j < nz; j += W_NT) {
        const unsigned long long k = zk[j];
        if (k >= lo && k <= hi) {
          const int sb = static_cast<int>((k - lo) >> shf);
          atomicAdd(&sm[sb], exp_safe(zone_key_d(k), s_tab));
          atomicAdd(&scn[sb], 1);
        }
      }
      __syncthreads();
      const double mine = sm[tid];
      double totm;
      const double exm = bu::scan_excl_d<W_NW>(mine, totm, sc, tid);
      const int first = (scn[tid] > 0 && crossed(gbase + exm + mine)) ? tid : W_NSUB;
      const int sbx = bu::min_i<W_NW>(first, sc, tid);
      if (sbx == W_NSUB) { all_in = true; break; }
      if (tid == sbx) { sh.bcd[0] = gbase + exm; sh.bc[0] = scn[tid]; }
      __syncthreads();
      gbase = sh.bcd[0];
      inrange = sh.bc[0];
      const unsigned long long nlo = lo + (static_cast<unsigned long long>(sbx) << shf);
      unsigned long long nhi = nlo + ((1ull << shf) - 1ull);
      if (nhi < nlo || nhi > hi) nhi = hi;
      lo = nlo; hi = nhi;
    }
    if (inrange > 32 && !all_in) bad = true;
    double g_at = gbase, g_before = gbase;
    if (!bad && !all_in) {
      unsigned long long* few = reinterpret_cast<unsigned long long*>(hist);   // [32]
      __syncthreads();
      if (tid == 0) sh.cnt = 0;
      __syncthreads();
      for (int j = tid; j < nz; j += W_NT) {
        const unsigned long long k = zk[j];
        if (k >= lo && k <= hi) { const int slot = atomicAdd(&sh.cnt, 1); if (slot < 32) few[slot] = k; }
      }
      __syncthreads();
      const int nf = min(32, sh.cnt);
      if (warp == 0) {
        const unsigned long long k = (lane < nf) ? few[lane] : ~0ull;
        const double e = (lane < nf) ? exp_safe(zone_key_d(k), s_tab) : 0.0;
        double g = gbase;                                    // G(k) = gbase + masses of the keys <= k
        for (int l = 0; l < nf; l++) {
          const unsigned long long kl = __shfl_sync(FULL, k, l);
          const double el = __shfl_sync(FULL, e, l);
          if (kl <= k) g += el;
        }
        const bool cr = (lane < nf) && crossed(g);
        unsigned long long candk = cr ? k : ~0ull;           // first crossed key = smallest crossed key
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const unsigned long long tt = __shfl_xor_sync(FULL, candk, o);
          candk = tt < candk ? tt : candk;
        }
        const unsigned who = __ballot_sync(FULL, cr && k == candk);
        if (lane == 0) { sc.u[0] = candk; sh.bc[1] = who ? 1 : 0; }
        if (who && lane == __ffs(who) - 1) { sh.bcd[1] = g; sh.bcd[2] = g - e; }
      }
      __syncthreads();
      if (sh.bc[1]) {
        cut_key = sc.u[0];
        g_at = sh.bcd[1];
        g_before = sh.bcd[2];
        cut_incl = (mode == 0) ? 0 : 1;
      } else {
        all_in = true;                                       // rounding: nothing in the last group crossed
      }
      __syncthreads();
    }
    if (!bad && all_in) {
      cut_key = ~0ull; cut_incl = 1;
      if (mode == 1 && dlow < dB) bad = true;                // logits below the zone exist: the bracket promised a crossing
    }
    if (!bad && !all_in) {
      // the sums carry exp_fast_s's error; in G/S >= p it enters as 2 p (1-p) times that bound
      const double etol = 1e-12 + (fast_ok ? 2.0 * plim * fabs(1.0 - plim) * eps_rel : 0.0);
      if (fabs(g_at / S - plim) <= etol || fabs(g_before / S - plim) <= etol) flags |= FLAG_TOPP_EDGE;
      if (xs) {
        // Several logits can share one d, and the order among equal d is by index: a cut whose d is also
        // the d of a logit outside the window (at its upper or lower edge) is decided on the whole row.
        const float dc = zone_key_d(cut_key);
        if (xA < INFINITY && dc == scale_t(xA, Tm) - m) bad = true;
        if (xB > -INFINITY && dc == scale_t(nextafterf(xB, -INFINITY), Tm) - m) bad = true;
      }
      if (mode == 1) {
        // a later key with the same d as c*: the cut separates equal probabilities
        int tie = 0;
        for (int j = tid; j < nz; j += W_NT) { const unsigned long long k = zk[j]; tie |= (k > cut_key && (k >> 32) == (cut_key >> 32)) ? 1 : 0; }
        if (bu::max_i<W_NW>(tie, sc, tid)) flags |= FLAG_TIE_CUT;
      }
    }
    if (bad) {
      if (tid == 0) hand_to_single(BA, row_id);
      return;
    }
    // kept zone entries add their mass to the piece they sit in
    __syncthreads();
    for (int j = tid; j < nz; j += W_NT) {
      const unsigned long long k = zk[j];
      if (k < cut_key || (cut_incl && k == cut_key)) {
        const int v = rv.vec_of(zone_key_index(k, mode));
        const int w = v / span;
        atomicAdd(&part[w * ppw + (v - w * span) / PV], exp_safe(zone_key_d(k), s_tab));
      }
    }
    __syncthreads();
  }
  // ---- kept mass and the piece that holds the drawn token: prefix over the pieces in row order
  const double pm = (tid < npiece) ? part[tid] : 0.0;
  double Re;
  const double pex = bu::scan_excl_d<W_NW>(pm, Re, sc, tid);
  dbg.resum = Re / S;
  stamp(3);
  if (!(S == S) || !(S > 0.0) || !(Re > 0.0)) {
    // mode A removed every token (generate.go:221-227 divides by zero): the walk falls through
    fill_probs_row(QNAN);
    if (S == S && S > 0.0) dbg.resum = 0.0; else dbg.sum_exp = QNAN;
    write_row(V - 1, flags | FLAG_NONFINITE | FLAG_FALLBACK);
    return;
  }
  // final rule for one logit: its kept mass (0 when cut away)
  auto kept_mass = [&](float xv, int i) -> double {
    if (i < 0 || i >= V) return 0.0;
    const float s = t_is_one ? xv : __fdiv_rn(xv, Tm);
    const float d = s - m;
    if (xs ? (cut_on && !(xv >= xA)) : (d < dA)) {
      if (xs ? !(xv >= xB) : !(d >= dB)) return 0.0;
      const unsigned long long k = zone_key(d, i, mode);
      if (!(k < cut_key || (cut_incl && k == cut_key))) return 0.0;
    }
    return exp_safe(d, s_tab);
  };
  if (A.out_probs || A.out_debug) {                          // parity runs only
    double* pr = A.out_probs ? A.out_probs + row_id * static_cast<int64_t>(V) : nullptr;
    const double rq = Re / S;
    int kept_loc = 0;
    for (int v = tid; v < rv.nvec; v += W_NT) {
      float x[VEC];
      Elem<T>::unpack(__ldg(rv.vbase + v), x);
      const int i0 = v * VEC - rv.shift;
#pragma unroll
      for (int c = 0; c < VEC; c++) {
        const int i = i0 + c;
        if (i >= 0 && i < V) {
          const double f = (kept_mass(x[c], i) / S) / rq;
          kept_loc += (f > 0) ? 1 : 0;
          if (pr) pr[i] = f;
        }
      }
    }
    dbg.kept = bu::sum_i<W_NW>(kept_loc, sc, tid);
  }
  stamp(4);
  // ---- draw (generate.go:231-239): u < prefix/Re is tested as u*Re < prefix
  const double tgt = u * Re;
  int psel = (tid < npiece && tgt < pex + pm) ? tid : 0x7fffffff;
  psel = bu::min_i<W_NW>(psel, sc, tid);
  if (tid == psel) sh.bcd[0] = pex;
  __syncthreads();
  int id = -1;
  double edge_lo = 0.0, edge_hi = 0.0;
  double run_end = (psel != 0x7fffffff) ? sh.bcd[0] : Re;
  if (psel != 0x7fffffff) {
    // walk pieces from the selected one (rounding can push the crossing into the next piece)
    for (int pi = psel; pi < npiece && id < 0; pi++) {       // uniform; normally one trip
      const int w = pi / ppw;
      const int vb = w * span + (pi - w * ppw) * PV;
      const int vend = min(min(vb + PV, w * span + span), rv.nvec);
      const int j = vb + tid;
      double em[VEC];
      double tsum = 0.0;
#pragma unroll
      for (int c = 0; c < VEC; c++) em[c] = 0.0;
      int i0 = 0;
      if (j < vend) {
        float x[VEC];
        Elem<T>::unpack(__ldg(rv.vbase + j), x);
        i0 = j * VEC - rv.shift;
#pragma unroll
        for (int c = 0; c < VEC; c++) { em[c] = kept_mass(x[c], i0 + c); tsum += em[c]; }
      }
      double totc;
      const double ex = bu::scan_excl_d<W_NW>(tsum, totc, sc, tid);
      int pick_loc = 0x7fffffff;
      double run = run_end + ex, lo = 0.0, hi = 0.0;
#pragma unroll
      for (int c = 0; c < VEC; c++) {
        const double before = run;
        run += em[c];
        if (em[c] > 0.0 && tgt < run && pick_loc == 0x7fffffff) { pick_loc = i0 + c; lo = before; hi = run; }
      }
      const int pick = bu::min_i<W_NW>(pick_loc, sc, tid);
      if (pick != 0x7fffffff) {
        if (pick_loc == pick) { sh.bcd[1] = lo; sh.bcd[2] = hi; }
        __syncthreads();
        id = pick;
        edge_lo = sh.bcd[1] / Re;
        edge_hi = sh.bcd[2] / Re;
      }
      run_end += totc;
    }
  }
  if (id >= 0) {
    dbg.edge_lo = edge_lo; dbg.edge_hi = edge_hi;
    if ((edge_lo > 0.0 && u - edge_lo <= 1e-6) || edge_hi - u <= 1e-6) flags |= FLAG_BOUNDARY;
  } else {
    id = V - 1;                                              // generate.go:239
    flags |= FLAG_FALLBACK;
    dbg.edge_lo = dbg.edge_hi = run_end / Re;
    if (u - run_end / Re <= 1e-6) flags |= FLAG_BOUNDARY;
  }
  stamp(5);
  write_row(id, flags);
}

template <typename T>
__global__ void __launch_bounds__(W_NT, W_CTAS) wide_rows_kernel(BatchArgs BA) {
  extern __shared__ __align__(16) unsigned char dyn[];
  __shared__ WideShared sh;
  if (threadIdx.x < 256) sh.tab[threadIdx.x] = BA.k.exp_table[threadIdx.x];
  unsigned long long pol_keep, pol_drop;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol_keep));
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol_drop));
  for (;;) {
    __syncthreads();
    if (threadIdx.x == 0) {
      int w;                                                 // next row of this kernel's kind
      for (;;) {
        w = atomicAdd(&BA.hdr[3], 1);
        if (w >= BA.B) { w = -1; break; }
        if (row_kind(BA.k, w) == 1) break;
      }
      sh.row = w;
    }
    __syncthreads();
    const int row = sh.row;
    if (row < 0) break;
    wide_row<T>(BA, row, dyn, sh, pol_keep, pol_drop);
  }
}

}  // namespace GS_W_NS
}  // namespace gs

#undef GS_W_NS
#undef GS_W_NT
