// Block-wide reductions and scans for CTAs of NWARPS <= 32 warps (sm_100a).
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

// Second level of every reduction below: each warp reads the NWARPS per-warp partials (one per
// lane) and reduces them with shuffles, so a reduction costs one shared load per thread and
// every thread ends with the same bits.
template <int NWARPS>
__device__ __forceinline__ double sum_d(double v, Scratch& s, int tid) {
  v = warp_sum_d(v);
  __syncthreads();
  if ((tid & 31) == 0) s.d0[tid >> 5] = v;
  __syncthreads();
  return warp_sum_d(((tid & 31) < NWARPS) ? s.d0[tid & 31] : 0.0);
}

// Three sums with one pair of barriers.
template <int NWARPS>
__device__ __forceinline__ void sum_d3(double& a, double& b, double& c, Scratch& s, int tid) {
  a = warp_sum_d(a); b = warp_sum_d(b); c = warp_sum_d(c);
  __syncthreads();
  if ((tid & 31) == 0) { s.d0[tid >> 5] = a; s.d1[tid >> 5] = b; s.u[tid >> 5] = static_cast<unsigned long long>(__double_as_longlong(c)); }
  __syncthreads();
  const int l = tid & 31;
  a = warp_sum_d((l < NWARPS) ? s.d0[l] : 0.0);
  b = warp_sum_d((l < NWARPS) ? s.d1[l] : 0.0);
  c = warp_sum_d((l < NWARPS) ? __longlong_as_double(static_cast<long long>(s.u[l])) : 0.0);
}

template <int NWARPS>
__device__ __forceinline__ int sum_i(int v, Scratch& s, int tid) {
  v = __reduce_add_sync(FULL, v);
  __syncthreads();
  if ((tid & 31) == 0) s.i0[tid >> 5] = v;
  __syncthreads();
  return __reduce_add_sync(FULL, ((tid & 31) < NWARPS) ? s.i0[tid & 31] : 0);
}

template <int NWARPS>
__device__ __forceinline__ int min_i(int v, Scratch& s, int tid) {
  v = __reduce_min_sync(FULL, v);
  __syncthreads();
  if ((tid & 31) == 0) s.i0[tid >> 5] = v;
  __syncthreads();
  return __reduce_min_sync(FULL, s.i0[(tid & 31) < NWARPS ? (tid & 31) : 0]);
}

template <int NWARPS>
__device__ __forceinline__ int max_i(int v, Scratch& s, int tid) {
  v = __reduce_max_sync(FULL, v);
  __syncthreads();
  if ((tid & 31) == 0) s.i0[tid >> 5] = v;
  __syncthreads();
  return __reduce_max_sync(FULL, s.i0[(tid & 31) < NWARPS ? (tid & 31) : 0]);
}

// Two minima with one pair of barriers.
template <int NWARPS>
__device__ __forceinline__ void min_i2(int& a, int& b, Scratch& s, int tid) {
  a = __reduce_min_sync(FULL, a);
  b = __reduce_min_sync(FULL, b);
  __syncthreads();
  if ((tid & 31) == 0) { s.i0[tid >> 5] = a; s.i1[tid >> 5] = b; }
  __syncthreads();
  const int l = (tid & 31) < NWARPS ? (tid & 31) : 0;
  a = __reduce_min_sync(FULL, s.i0[l]);
  b = __reduce_min_sync(FULL, s.i1[l]);
}

__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long t = __shfl_xor_sync(FULL, v, o);
    v = t > v ? t : v;
  }
  return v;
}
template <int NWARPS>
__device__ __forceinline__ unsigned long long max_u64(unsigned long long v, Scratch& s, int tid) {
  v = warp_max_u64(v);
  __syncthreads();
  if ((tid & 31) == 0) s.u[tid >> 5] = v;
  __syncthreads();
  return warp_max_u64(s.u[(tid & 31) < NWARPS ? (tid & 31) : 0]);
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
  const double wv = (lane < NWARPS) ? s.d0[lane] : 0.0;
  const double wi = warp_scan_incl_d(wv, lane);
  total = __shfl_sync(FULL, wi, NWARPS - 1);
  const double base = __shfl_sync(FULL, wi - wv, w);
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
  const double wa = (lane < NWARPS) ? s.d0[lane] : 0.0, wb = (lane < NWARPS) ? s.d1[lane] : 0.0;
  const double sa = warp_scan_incl_d(wa, lane), sb = warp_scan_incl_d(wb, lane);
  ta = __shfl_sync(FULL, sa, NWARPS - 1); tb = __shfl_sync(FULL, sb, NWARPS - 1);
  ea = __shfl_sync(FULL, sa - wa, w) + ia - a;
  eb = __shfl_sync(FULL, sb - wb, w) + ib - b;
}

// k-th largest (with multiplicity) of the order keys that the threads of the block enumerate:
// for_each_key(f) calls f(key) for every key of the calling thread (the same keys on every call).
// MSB-first radix select. Every key lies in [lo, hi] (0 and 0xffffffff when nothing is known): the
// bits that lo and hi share are shared by all keys, so the first digit starts at the highest bit
// in which they differ. Keys that are close together (logits above a threshold) then spread over
// the bins of the first round instead of meeting in one or two, and need a round less.
// hist: 256 uint32 of scratch; bc: 2 ints.
template <int NTHREADS, typename F>
__device__ __forceinline__ uint32_t select_kth_of(F&& for_each_key, int k, uint32_t lo, uint32_t hi,
                                                   uint32_t* hist, int* bc, int tid) {
  if (lo == hi) return lo;
  const int top = 31 - __clz(lo ^ hi);                        // highest differing bit
  uint32_t mask = (top == 31) ? 0u : ~((2u << top) - 1u);
  uint32_t prefix = hi & mask;
  int need = k;
  for (int sh = max(top - 7, 0);; sh = max(sh - 8, 0)) {
    __syncthreads();
    for (int j = tid; j < 256; j += NTHREADS) hist[j] = 0;
    __syncthreads();
    for_each_key([&](uint32_t key) {
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> sh) & 255u], 1u);
    });
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
    // a digit that reaches above bit `top` (fewer than eight bits differ) or into the previous
    // digit repeats bits that are fixed already: the same in every key that is still counted
    prefix = (prefix & ~(255u << sh)) | (static_cast<uint32_t>(bc[0]) << sh);
    mask |= 255u << sh;
    need = bc[1];
    if (sh == 0) break;
  }
  return prefix;
}

// The same over the float bit patterns list[j].x, j < n.
template <int NTHREADS>
__device__ uint32_t select_kth(const uint2* list, int n, int k, uint32_t* hist, int* bc, int tid,
                               uint32_t lo = 0u, uint32_t hi = 0xffffffffu) {
  return select_kth_of<NTHREADS>([&](auto&& f) {
    for (int j = tid; j < n; j += NTHREADS) f(okey(__uint_as_float(list[j].x)));
  }, k, lo, hi, hist, bc, tid);
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
