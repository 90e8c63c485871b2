// Block-wide reductions and scans for CTAs of NWARPS warps (sm_100a).
#pragma once

#include "sample_common.cuh"

namespace gs {
namespace bu {

// Scratch shared by the helpers below; one instance per CTA.
struct Scratch {
  double d0[32];
  double d1[32];
  unsigned long long u[32];
  int i0[32];
  int i1[32];
};

template <int NWARPS>
__device__ __forceinline__ double sum_d(double v, Scratch& s, int tid) {
  v = warp_sum_d(v);
  __syncthreads();
  if ((tid & 31) == 0) s.d0[tid >> 5] = v;
  __syncthreads();
  double t = 0.0;
#pragma unroll
  for (int w = 0; w < NWARPS; w++) t += s.d0[w];
  return t;
}

// Three sums with one pair of barriers.
template <int NWARPS>
__device__ __forceinline__ void sum_d3(double& a, double& b, double& c, Scratch& s, int tid) {
  a = warp_sum_d(a); b = warp_sum_d(b); c = warp_sum_d(c);
  __syncthreads();
  if ((tid & 31) == 0) { s.d0[tid >> 5] = a; s.d1[tid >> 5] = b; s.u[tid >> 5] = static_cast<unsigned long long>(__double_as_longlong(c)); }
  __syncthreads();
  double ta = 0.0, tb = 0.0, tc = 0.0;
#pragma unroll
  for (int w = 0; w < NWARPS; w++) { ta += s.d0[w]; tb += s.d1[w]; tc += __longlong_as_double(static_cast<long long>(s.u[w])); }
  a = ta; b = tb; c = tc;
}

template <int NWARPS>
__device__ __forceinline__ int sum_i(int v, Scratch& s, int tid) {
  v = __reduce_add_sync(FULL, v);
  __syncthreads();
  if ((tid & 31) == 0) s.i0[tid >> 5] = v;
  __syncthreads();
  int t = 0;
#pragma unroll
  for (int w = 0; w < NWARPS; w++) t += s.i0[w];
  return t;
}

template <int NWARPS>
__device__ __forceinline__ int min_i(int v, Scratch& s, int tid) {
  v = __reduce_min_sync(FULL, v);
  __syncthreads();
  if ((tid & 31) == 0) s.i0[tid >> 5] = v;
  __syncthreads();
  int t = s.i0[0];
#pragma unroll
  for (int w = 1; w < NWARPS; w++) t = min(t, s.i0[w]);
  return t;
}

template <int NWARPS>
__device__ __forceinline__ int max_i(int v, Scratch& s, int tid) {
  v = __reduce_max_sync(FULL, v);
  __syncthreads();
  if ((tid & 31) == 0) s.i0[tid >> 5] = v;
  __syncthreads();
  int t = s.i0[0];
#pragma unroll
  for (int w = 1; w < NWARPS; w++) t = max(t, s.i0[w]);
  return t;
}

// Two minima with one pair of barriers.
template <int NWARPS>
__device__ __forceinline__ void min_i2(int& a, int& b, Scratch& s, int tid) {
  a = __reduce_min_sync(FULL, a);
  b = __reduce_min_sync(FULL, b);
  __syncthreads();
  if ((tid & 31) == 0) { s.i0[tid >> 5] = a; s.i1[tid >> 5] = b; }
  __syncthreads();
  int ta = s.i0[0], tb = s.i1[0];
#pragma unroll
  for (int w = 1; w < NWARPS; w++) { ta = min(ta, s.i0[w]); tb = min(tb, s.i1[w]); }
  a = ta; b = tb;
}

template <int NWARPS>
__device__ __forceinline__ unsigned long long max_u64(unsigned long long v, Scratch& s, int tid) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long t = __shfl_xor_sync(FULL, v, o);
    v = t > v ? t : v;
  }
  __syncthreads();
  if ((tid & 31) == 0) s.u[tid >> 5] = v;
  __syncthreads();
  unsigned long long t = s.u[0];
#pragma unroll
  for (int w = 1; w < NWARPS; w++) t = s.u[w] > t ? s.u[w] : t;
  return t;
}
template <int NWARPS>
__device__ __forceinline__ unsigned long long min_u64(unsigned long long v, Scratch& s, int tid) {
  return ~max_u64<NWARPS>(~v, s, tid);
}

// Exclusive prefix in thread order; `total` receives the block sum.
template <int NWARPS>
__device__ __forceinline__ double scan_excl_d(double v, double& total, Scratch& s, int tid) {
  const int lane = tid & 31, w = tid >> 5;
  const double incl = warp_scan_incl_d(v, lane);
  __syncthreads();
  if (lane == 31) s.d0[w] = incl;
  __syncthreads();
  double base = 0.0, tot = 0.0;
#pragma unroll
  for (int j = 0; j < NWARPS; j++) {
    const double x = s.d0[j];
    if (j < w) base += x;
    tot += x;
  }
  total = tot;
  return base + incl - v;
}

// Exclusive prefixes of two values at once.
template <int NWARPS>
__device__ __forceinline__ void scan_excl_d2(double a, double b, double& ea, double& eb, double& ta, double& tb,
                                             Scratch& s, int tid) {
  const int lane = tid & 31, w = tid >> 5;
  const double ia = warp_scan_incl_d(a, lane), ib = warp_scan_incl_d(b, lane);
  __syncthreads();
  if (lane == 31) { s.d0[w] = ia; s.d1[w] = ib; }
  __syncthreads();
  double ba = 0, bb = 0, sa = 0, sb = 0;
#pragma unroll
  for (int j = 0; j < NWARPS; j++) {
    const double va = s.d0[j], vb = s.d1[j];
    if (j < w) { ba += va; bb += vb; }
    sa += va; sb += vb;
  }
  ea = ba + ia - a; eb = bb + ib - b; ta = sa; tb = sb;
}

// k-th largest (with multiplicity) of the float bit patterns list[j].x, j < n, by
// MSB-first radix select on order keys. hist: 256 uint32 of scratch; bc: 2 ints.
template <int NTHREADS>
__device__ uint32_t select_kth(const uint2* list, int n, int k, uint32_t* hist, int* bc, int tid) {
  uint32_t prefix = 0, mask = 0;
  int need = k;
  for (int round = 0; round < 4; round++) {
    const int sh = 24 - 8 * round;
    __syncthreads();
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (int j = tid; j < n; j += NTHREADS) {
      const uint32_t key = okey(__uint_as_float(list[j].x));
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> sh) & 255u], 1u);
    }
    __syncthreads();
    if (tid < 32) {
      int loc[8];
      int s = 0;
#pragma unroll
      for (int j = 7; j >= 0; j--) { s += static_cast<int>(hist[tid * 8 + j]); loc[j] = s; }
      int run = s;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_down_sync(FULL, run, o);
        if (tid + o < 32) run += t;
      }
      const int above = run - s;
      if (above < need && above + s >= need) {
#pragma unroll
        for (int j = 7; j >= 0; j--) {
          if (above + loc[j] >= need) {
            bc[0] = tid * 8 + j;
            bc[1] = need - (above + loc[j] - static_cast<int>(hist[tid * 8 + j]));
            break;
          }
        }
      }
    }
    __syncthreads();
    prefix |= static_cast<uint32_t>(bc[0]) << sh;
    mask |= 255u << sh;
    need = bc[1];
  }
  return prefix;
}

// In-place inclusive scan of a shared array a[0..n), n <= PER * 32 * NWARPS, in index order.
template <int NWARPS, int PER>
__device__ __forceinline__ void smem_scan_incl(double* a, int n, Scratch& s, int tid) {
  double loc[PER];
  double acc = 0.0;
  const int base = tid * PER;
#pragma unroll
  for (int j = 0; j < PER; j++) {
    const double v = (base + j < n) ? a[base + j] : 0.0;
    acc += v;
    loc[j] = acc;
  }
  double tot;
  const double ex = scan_excl_d<NWARPS>(acc, tot, s, tid);
#pragma unroll
  for (int j = 0; j < PER; j++) {
    if (base + j < n) a[base + j] = ex + loc[j];
  }
  __syncthreads();
}

}  // namespace bu
}  // namespace gs
