// Shared device helpers for the sampling kernels (sm_100a).
//
// Everything here restates arithmetic of the reference's scalar Go routines
// (model/generate.go:134-260, model/qwen/generate.go:77-181) in a form that
// many threads can evaluate; the comments name the line each rule comes from.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace gs {

constexpr unsigned FULL = 0xffffffffu;

// out_flags bits (kept in step with include/gorch_cuda_shim.h).
constexpr uint32_t FLAG_BOUNDARY = 1u << 0;
constexpr uint32_t FLAG_FALLBACK = 1u << 1;
constexpr uint32_t FLAG_NONFINITE = 1u << 2;
constexpr uint32_t FLAG_TIE_CUT = 1u << 3;
constexpr uint32_t FLAG_TOPP_EDGE = 1u << 5;
constexpr uint32_t FLAG_GENERAL_PATH = 1u << 6;
constexpr uint32_t FLAG_INTERNAL = 1u << 7;
constexpr uint32_t FLAG_BAD_CFG = 1u << 8;

struct RowCfg {  // 16 bytes, the sampling fields of GenerateConfig (model/generate.go:13-20)
  float temperature;
  int32_t top_k;
  float top_p;
  int32_t topp_mode;
};

struct RowDebug {  // optional per-row record for the parity tests
  double sum_exp;   // softmax denominator over the kept set
  double resum;     // top-p renormaliser in probability units (1 when inactive)
  double edge_lo;   // cumulative before the chosen token
  double edge_hi;   // cumulative through the chosen token
  int32_t kept;     // tokens with non-zero final probability
  float max_scaled; // max of logits/T
  float threshold;  // top-k threshold in logits/T units (NaN when inactive)
  int32_t path;     // 0 greedy, 1 small-set path, 2 full-row path
  uint32_t reserved[8]; // scratch of the kernels (phase clocks, list sizes); no meaning is promised
};

// ---------------------------------------------------------------------------
// Order-preserving key for IEEE floats under Go's '>' (generate.go:138,249):
// -0 and +0 are equal, NaN is never greater than anything (key 0, the lowest).
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t okey(float x) {
  uint32_t b = __float_as_uint(x);
  if ((b & 0x7fffffffu) > 0x7f800000u) return 0u;  // NaN
  if (b == 0x80000000u) b = 0u;                    // -0 -> +0
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float okey_to_float(uint32_t k) {
  uint32_t b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(b);
}

// logits[i] / temperature in IEEE f32 round-to-nearest (generate.go:152).
__device__ __forceinline__ float scale_t(float x, float T) {
  return (T == 1.0f) ? x : __fdiv_rn(x, T);
}

// ---------------------------------------------------------------------------
// exp for d <= 0 in f64 (generate.go:176: math.Exp(float64(v - maxVal))).
// Table-driven: d = (k/256) ln2 + r, |r| <= ln2/512, exp = 2^(k>>8) * T[k&255]
// * (1 + r + r^2/2 + r^3/6 + r^4/24); truncation 4e-17, total about 1 ulp.
// The table holds 2^(j/256), j = 0..255, and is staged in shared memory.
// ---------------------------------------------------------------------------
__device__ __forceinline__ double exp_neg_f64(float d, const double* __restrict__ tab) {
  if (!(d >= -700.0f)) {  // deep underflow range, -Inf, NaN: exact library path
    return exp(static_cast<double>(d));
  }
  const double x = static_cast<double>(d);
  const double INV = 369.3299304675746;           // 256/ln2
  const double MAGIC = 6755399441055744.0;        // 1.5 * 2^52
  const double L_HI = 0x1.62e42fee00000p-9;       // ln2/256 to 32 bits: k*L_HI is exact
  const double L_LO = 0x1.a39ef35793c76p-41;      // ln2/256 - L_HI
  double t = fma(x, INV, MAGIC);
  int ki = __double2loint(t);
  double kd = t - MAGIC;
  double r = fma(kd, -L_HI, x);
  r = fma(kd, -L_LO, r);
  double q = fma(r, 4.1666666666666664e-02, 1.6666666666666666e-01);
  q = fma(q, r, 0.5);
  q = fma(q, r, 1.0);
  double tj = tab[ki & 255];
  double res = fma(tj, q * r, tj);
  int hi = __double2hiint(res) + ((ki >> 8) << 20);
  return __hiloint2double(hi, __double2loint(res));
}

// ---------------------------------------------------------------------------
// Warp / block primitives (NT threads, NT/32 warps).
// ---------------------------------------------------------------------------
__device__ __forceinline__ double shfl_down_d(double v, int off) {
  return __shfl_down_sync(FULL, v, off);
}
__device__ __forceinline__ double shfl_up_d(double v, int off) {
  return __shfl_up_sync(FULL, v, off);
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
  return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
  return __reduce_add_sync(FULL, v);
}
__device__ __forceinline__ double warp_scan_incl_d(double v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    double t = __shfl_up_sync(FULL, v, o);
    if (lane >= o) v += t;
  }
  return v;
}

__device__ __forceinline__ uint32_t dkey_of(float d) {   // d <= 0 (or NaN): ascending = falling probability
  return (d != d) ? 0x7fffffffu : (__float_as_uint(-d) & 0x7fffffffu);
}
// Zone order: falling probability, equal d by ascending index in mode B; mode A
// removes the lowest index of a tie first (generate.go:208-212), so its survivors
// are the highest indices and the index is complemented.
__device__ __forceinline__ unsigned long long zone_key(float d, int idx, int mode) {
  const uint32_t ix = (mode == 0) ? ~static_cast<uint32_t>(idx) : static_cast<uint32_t>(idx);
  return (static_cast<unsigned long long>(dkey_of(d)) << 32) | ix;
}
__device__ __forceinline__ int zone_key_index(unsigned long long k, int mode) {
  const uint32_t ix = static_cast<uint32_t>(k);
  return static_cast<int>(mode == 0 ? ~ix : ix);
}
__device__ __forceinline__ float zone_key_d(unsigned long long k) {
  return -__uint_as_float(static_cast<uint32_t>(k >> 32));
}


}  // namespace gs
