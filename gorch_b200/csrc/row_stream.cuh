// Streaming a row by warps: warp w owns a contiguous span of the row's 16-byte vectors; in a step
// every lane takes VPL vectors (by default eight logits: two vectors of f32, one of bf16) that it
// loads straight into registers ahead of their use and asks from L2 a few steps before that.
#pragma once

#include "sample_kernel.cuh"

namespace gs {

#ifndef GS_W_PF
#define GS_W_PF 2
#endif
constexpr int W_PF = GS_W_PF;           // L2 prefetch distance in steps (passes that may find the row in L2)
#ifndef GS_N_PF
#define GS_N_PF 8
#endif
constexpr int N_PF = GS_N_PF;           // the same for single passes from HBM (Multinomial)
__device__ __forceinline__ uint4 ldg_hint(const uint4* p, unsigned long long pol) {
  uint4 v;
  asm volatile("ld.global.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(pol));
  return v;
}

// max / min of three at once (sm_100), and maxima that return NaN as soon as an operand is NaN:
// a running maximum kept with them says at the end whether the row held a NaN.
__device__ __forceinline__ float max3nan(float a, float b, float c) { float d; asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }
__device__ __forceinline__ float maxnan(float a, float b) { float d; asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b)); return d; }
__device__ __forceinline__ float min3f(float a, float b, float c) { float d; asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }
__device__ __forceinline__ uint32_t maxnan_bf16x2(uint32_t a, uint32_t b) { uint32_t d; asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
// NaN-propagating maximum of the eight logits a lane holds in one step
template <typename T> __device__ __forceinline__ float step_max_nan(const uint4& a, const uint4& b);
template <> __device__ __forceinline__ float step_max_nan<float>(const uint4& a, const uint4& b) {
  float m = max3nan(__uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z));
  m = max3nan(m, __uint_as_float(a.w), __uint_as_float(b.x));
  m = max3nan(m, __uint_as_float(b.y), __uint_as_float(b.z));
  return maxnan(m, __uint_as_float(b.w));
}
template <> __device__ __forceinline__ float step_max_nan<uint16_t>(const uint4& a, const uint4&) {
  const uint32_t p = maxnan_bf16x2(maxnan_bf16x2(a.x, a.y), maxnan_bf16x2(a.z, a.w));
  return maxnan(__uint_as_float(p << 16), __uint_as_float(p & 0xffff0000u));
}

// What one thread needs to stream its warp's span of a row.
struct WSpan {
  const uint4* lane_src;   // this lane's first vector: row vector (first + lane)
  int first;               // first vector of the warp's span
  int rel;                 // vectors from lane_src to the row's end (<= 0: none)
  int nst;                 // steps this warp runs
  int omax;                // largest valid vector offset from lane_src
  int clean_lo, clean_hi;  // steps [clean_lo, clean_hi) hold no logit outside the row (warp-uniform)
};

// The lane's vectors of step st. A vector past the row's end is replaced by the lane's last one
// (or the row's first when the lane has none): always a valid address, and such vectors are
// masked by the caller from their true index.
template <typename T, int PF = W_PF, int VPL = 8 / Elem<T>::VEC>
__device__ __forceinline__ void w_load(const WSpan& sp, int st, unsigned long long pol, uint4& ra, uint4& rb) {
  constexpr int EPI = VPL, SV = 32 * EPI;
  const int o = st * SV;
  ra = ldg_hint(sp.lane_src + min(o, sp.omax), pol);
  if (EPI == 2) rb = ldg_hint(sp.lane_src + min(o + 32, sp.omax), pol);
  else rb = ra;
  // ask L2 for the step PF steps further on: costs no register, and the load above then finds
  // its line in L2 whether the row came from HBM or was evicted since the last pass
  if (PF > 0) {
    const int o2 = o + PF * SV;
    asm volatile("prefetch.global.L2 [%0];" :: "l"(sp.lane_src + min(o2, sp.omax)));
    if (EPI == 2) asm volatile("prefetch.global.L2 [%0];" :: "l"(sp.lane_src + min(o2 + 32, sp.omax)));
  }
}

// Fills in a span for the vectors [first, first + span) of the row (span a multiple of the step
// size), cut at the row's end.
template <typename T, int VPL = 8 / Elem<T>::VEC>
__device__ __forceinline__ WSpan make_span(const RowView<T>& rv, int first, int span, int lane) {
  constexpr int SV = 32 * VPL;
  WSpan sp;
  sp.first = first;
  const int end = min(rv.nvec, first + span);
  sp.nst = (end > first) ? (end - first + SV - 1) / SV : 0;
  sp.rel = rv.nvec - first - lane;
  sp.lane_src = rv.vbase + (sp.rel > 0 ? first + lane : 0);
  sp.omax = max(sp.rel - 1, 0);
  // a step is clean when all its SV vectors exist and none is the row's first or last
  sp.clean_lo = (first == 0) ? min(1, sp.nst) : 0;
  sp.clean_hi = max(sp.clean_lo, min(sp.nst, (rv.nvec - 1 - first) / SV));
  return sp;
}

}  // namespace gs
