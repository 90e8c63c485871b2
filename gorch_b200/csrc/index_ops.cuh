// Tensor-level index ops of the reference as batched device ops.
//
//   Multinomial (index_ops.go:203-227): per row, the first index j with u < sum_{i<=j} probs[i]
//   (f32 probabilities, f64 running sum), else V-1. multinomial_rows_kernel: 256 threads, rows
//   pulled by a grid-stride loop; every warp sums its span of the row step by step (one f64 sum
//   per warp-step of 256 probabilities), a block scan over the steps finds the step the uniform
//   falls into, and one warp rescans that step in index order. The running sum is formed in a
//   different order than the reference's sequential loop: a row whose uniform lies within 1e-6 of
//   an edge of the chosen interval is flagged FLAG_BOUNDARY.
//   TopK (index_ops.go:153-190) is the narrow kernel of sample_batch.cuh with KernelArgs::tk_k set
//   for k <= 256 (one pass over the row), and topk_large_kernel below for 256 < k <= 16384: an
//   exact radix select of the k-th largest value over the row (four passes, the row coming from L2
//   after the first), a gather of everything above it plus the lowest-index ties, and a bitonic
//   sort of the k results in shared memory.
#pragma once

#include "sample_batch.cuh"

namespace gs {

constexpr int MN_NT = 256;
constexpr int MN_NW = MN_NT / 32;
constexpr int MN_MAX_STEPS = 256;                          // steps per warp: rows up to 8 * 256 * 256 = 524288 probabilities
constexpr int MN_NQ = 3;                                   // steps of the row in flight per thread
constexpr int MN_RING_OFF = MN_NW * MN_MAX_STEPS * 8;      // after the 16 KB of step sums
constexpr int MN_DYN_BYTES = MN_RING_OFF + MN_NQ * 2 * MN_NT * 16;   // + 24 KB of ring

struct MultinomialArgs {
  const float* probs;      // [B, row_stride]
  int64_t row_stride;
  int32_t V;
  const double* uniforms;  // [B]
  int32_t* out_ids;        // [B]
  uint32_t* out_flags;     // [B] or null
  int64_t B;
};

__global__ void __launch_bounds__(MN_NT, 4) multinomial_rows_kernel(MultinomialArgs M) {
  extern __shared__ __align__(16) unsigned char dyn[];
  __shared__ bu::Scratch sc;
  __shared__ double s_bcd[4];
  __shared__ int s_bc[2];
  double* stepsum = reinterpret_cast<double*>(dyn);        // [warp][step], row order
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int SV = 64;                                   // vectors per warp-step (two per lane)
  unsigned long long pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  for (int64_t row = blockIdx.x; row < M.B; row += gridDim.x) {
    __syncthreads();
    RowView<float> rv;
    rv.init(M.probs + row * M.row_stride, M.V);
    const double u = M.uniforms[row];
    const int span = (((rv.nvec + MN_NW - 1) / MN_NW + SV - 1) / SV) * SV;
    const int steps = span / SV;
    int id = -1;
    uint32_t fl = 0u;
    if (steps > MN_MAX_STEPS) {                            // beyond the step table: not supported
      if (tid == 0) { M.out_ids[row] = -1; if (M.out_flags) M.out_flags[row] = FLAG_INTERNAL; }
      continue;
    }
    const WSpan sp = make_span<float>(rv, warp * span, span, lane);
    for (int j = tid; j < MN_NW * steps; j += MN_NT) stepsum[j] = 0.0;
    __syncthreads();
    // masked value of element c of this lane's vectors in step st (0 outside the row)
    auto vals = [&](int st, const uint4& a, const uint4& b, double* v) {
      float x[8];
      Elem<float>::unpack(a, x); Elem<float>::unpack(b, x + 4);
      const int gv = sp.first + st * SV + lane;
#pragma unroll
      for (int c = 0; c < 8; c++) {
        const int g = gv + 32 * (c / 4);
        const int i = g * 4 - rv.shift + (c % 4);
        v[c] = (g < rv.nvec && i >= 0 && i < rv.V) ? static_cast<double>(x[c]) : 0.0;
      }
    };
    {
      // The row is staged through a ring in shared memory by asynchronous 16-byte copies, MN_NQ
      // steps ahead (a thread copies what it consumes itself and waits only for its own groups):
      // loads into registers in a rolled loop share one scoreboard and do not run ahead.
      const uint32_t ring_addr = static_cast<uint32_t>(__cvta_generic_to_shared(dyn + MN_RING_OFF)) + static_cast<uint32_t>(tid * 16);
      const uint4* ring = reinterpret_cast<const uint4*>(dyn + MN_RING_OFF) + tid;
      auto issue = [&](int q) {
        if (q < sp.nst) {
          const uint32_t dst = ring_addr + static_cast<uint32_t>((q % MN_NQ) * 2 * MN_NT * 16);
          const int o = q * SV;
          asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;"
                       :: "r"(dst), "l"(sp.lane_src + min(o, sp.omax)), "l"(pol) : "memory");
          asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;"
                       :: "r"(dst + MN_NT * 16), "l"(sp.lane_src + min(o + 32, sp.omax)), "l"(pol) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
      };
#pragma unroll
      for (int q = 0; q < MN_NQ; q++) issue(q);
#pragma unroll 1
      for (int st = 0; st < sp.nst; st++) {
        asm volatile("cp.async.wait_group %0;" :: "n"(MN_NQ - 1) : "memory");
        const uint4 ca = ring[(st % MN_NQ) * 2 * MN_NT];
        const uint4 cb = ring[(st % MN_NQ) * 2 * MN_NT + MN_NT];
        double v[8];
        vals(st, ca, cb, v);
        issue(st + MN_NQ);                                 // into the slot just read
        double s = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
        s = warp_sum_d(s);
        if (lane == 0) stepsum[warp * steps + st] = s;
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    // prefix over the warp-steps in row order: thread t owns steps [t*PER, t*PER+PER)
    constexpr int PER = (MN_NW * MN_MAX_STEPS) / MN_NT;    // 8
    const int nsteps = MN_NW * steps;
    double loc[PER], acc = 0.0;
#pragma unroll
    for (int q = 0; q < PER; q++) { const int j = tid * PER + q; acc += (j < nsteps) ? stepsum[j] : 0.0; loc[q] = acc; }
    double total;
    const double ex = bu::scan_excl_d<MN_NW>(acc, total, sc, tid);
    int mine = 0x7fffffff;
#pragma unroll
    for (int q = PER - 1; q >= 0; q--) { const int j = tid * PER + q; if (j < nsteps && u < ex + loc[q]) mine = j; }
    const int jsel = bu::min_i<MN_NW>(mine, sc, tid);
    if (jsel != 0x7fffffff && tid == jsel / PER) s_bcd[0] = ex + ((jsel % PER) ? loc[jsel % PER - 1] : 0.0);
    if (tid == 0) s_bc[0] = -1;
    __syncthreads();
    if (jsel != 0x7fffffff && warp == 0) {
      // rescan the chosen warp-step in index order: first vectors of lanes 0..31, then the second
      const int w = jsel / steps, st = jsel % steps;
      const WSpan sw = make_span<float>(rv, w * span, span, lane);
      uint4 a, b;
      w_load<float, 0>(sw, st, pol, a, b);
      double v[8];
      {
        float x[8];
        Elem<float>::unpack(a, x); Elem<float>::unpack(b, x + 4);
        const int gv = sw.first + st * SV + lane;
#pragma unroll
        for (int c = 0; c < 8; c++) {
          const int g = gv + 32 * (c / 4);
          const int i = g * 4 - rv.shift + (c % 4);
          v[c] = (g < rv.nvec && i >= 0 && i < rv.V) ? static_cast<double>(x[c]) : 0.0;
        }
      }
      const double s0 = (v[0] + v[1]) + (v[2] + v[3]), s1 = (v[4] + v[5]) + (v[6] + v[7]);
      const double i0 = warp_scan_incl_d(s0, lane), i1 = warp_scan_incl_d(s1, lane);
      const double tot0 = __shfl_sync(FULL, i0, 31);
      const double base = s_bcd[0];
      double run = base + (i0 - s0);
      int pick = 0x7fffffff;
      double lo = 0.0, hi = 0.0;
      const int gv = sw.first + st * SV + lane;
#pragma unroll
      for (int c = 0; c < 8; c++) {
        if (c == 4) run = base + tot0 + (i1 - s1);
        const double before = run;
        run += v[c];
        const int i = (gv + 32 * (c / 4)) * 4 - rv.shift + (c % 4);
        if (pick == 0x7fffffff && u < run && i >= 0 && i < rv.V) { pick = i; lo = before; hi = run; }
      }
      const int best = __reduce_min_sync(FULL, pick);
      if (best != 0x7fffffff && pick == best) { s_bc[0] = best; s_bcd[1] = lo; s_bcd[2] = hi; }
      if (best == 0x7fffffff) {
        // the block scan put u inside this step, this rescan (another order of additions) just past
        // its end: u sits on the step's last edge to within rounding. Take the step's last index.
        int last = -1;
#pragma unroll
        for (int c = 0; c < 8; c++) {
          const int i = (gv + 32 * (c / 4)) * 4 - rv.shift + (c % 4);
          if (i >= 0 && i < rv.V && (gv + 32 * (c / 4)) < rv.nvec) last = max(last, i);
        }
        last = __reduce_max_sync(FULL, last);
        if (lane == 0) { s_bc[0] = last; s_bcd[1] = u; s_bcd[2] = u; }
      }
    }
    __syncthreads();
    if (jsel != 0x7fffffff && s_bc[0] >= 0) {
      id = s_bc[0];
      if ((s_bcd[1] > 0.0 && u - s_bcd[1] <= 1e-6) || s_bcd[2] - u <= 1e-6) fl |= FLAG_BOUNDARY;
    } else {
      id = M.V - 1;                                        // index_ops.go: falls through to the last index
      fl |= FLAG_FALLBACK;
      if (u - total <= 1e-6) fl |= FLAG_BOUNDARY;
    }
    if (tid == 0) { M.out_ids[row] = id; if (M.out_flags) M.out_flags[row] = fl; }
  }
}

// ---------------------------------------------------------------------------
// TopK for 256 < k <= TKL_MAX_K. One CTA of 512 threads per row at a time.
// Order: value descending, equal values by ascending index; NaNs last (the reference's comparator
// leaves them unspecified), -0 and +0 equal. The values written are the row's own bits.
// ---------------------------------------------------------------------------
constexpr int TKL_NT = 512;
constexpr int TKL_MAX_K = 16384;
constexpr int TKL_DYN_BYTES = TKL_MAX_K * 8;               // the k results as 64-bit sort keys

struct TopKLargeArgs {
  const void* x;           // [B, row_stride]
  int64_t row_stride;
  int32_t V;
  int32_t k;
  float* out_values;       // [B, k]
  int32_t* out_indices;    // [B, k]
  uint32_t* out_flags;     // [B] or null
  int64_t B;
};

template <typename T>
__global__ void __launch_bounds__(TKL_NT, 1) topk_large_kernel(TopKLargeArgs A) {
  extern __shared__ __align__(16) unsigned char dyn[];
  __shared__ bu::Scratch sc;
  __shared__ uint32_t hist[256];
  __shared__ int bc[4];
  __shared__ int s_cnt;
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(dyn);
  const int tid = threadIdx.x;
  const int V = A.V, k = A.k;
  int P = 1;
  while (P < k) P <<= 1;                                     // sort size
  for (int64_t row = blockIdx.x; row < A.B; row += gridDim.x) {
    const T* xr = static_cast<const T*>(A.x) + row * A.row_stride;
    RowView<T> rv;
    rv.init(xr, V);
    // smallest and largest order key of the row: the select starts at the highest bit in which they
    // differ, so that the keys spread over its bins (the top byte of a float is the same for nearly
    // all logits of a row, and 150,000 shared atomics on one counter would take a millisecond)
    uint32_t kmin = 0xffffffffu, kmax = 0u;
    for (int v = tid; v < rv.nvec; v += TKL_NT)
      rv.visit(v, [&](float x, int) { const uint32_t key = okey(x); kmin = min(kmin, key); kmax = max(kmax, key); });
    kmax = static_cast<uint32_t>(bu::max_u64<TKL_NT / 32>(kmax, sc, tid));
    kmin = ~static_cast<uint32_t>(bu::max_u64<TKL_NT / 32>(~kmin, sc, tid));
    // the k-th largest value (as an order key) ...
    const uint32_t kkey = bu::select_kth_of<TKL_NT>([&](auto&& f) {
      for (int v = tid; v < rv.nvec; v += TKL_NT) rv.visit(v, [&](float x, int) { f(okey(x)); });
    }, k, kmin, kmax, hist, bc, tid);
    // ... how many logits lie above it, and how many equal it
    int above = 0, ties = 0;
    for (int v = tid; v < rv.nvec; v += TKL_NT)
      rv.visit(v, [&](float x, int) { const uint32_t key = okey(x); above += (key > kkey) ? 1 : 0; ties += (key == kkey) ? 1 : 0; });
    above = bu::sum_i<TKL_NT / 32>(above, sc, tid);
    ties = bu::sum_i<TKL_NT / 32>(ties, sc, tid);
    const int need = k - above;                              // 1 <= need <= ties
    // among equals the lowest indices win: the need-th smallest index of them, when not all are wanted
    uint32_t last_index = 0xffffffffu;
    if (need < ties) {                                       // uniform
      const uint32_t inv = bu::select_kth_of<TKL_NT>([&](auto&& f) {
        for (int v = tid; v < rv.nvec; v += TKL_NT)
          rv.visit(v, [&](float x, int i) { if (okey(x) == kkey) f(~static_cast<uint32_t>(i)); });
      }, need, ~static_cast<uint32_t>(V - 1), 0xffffffffu, hist, bc, tid);
      last_index = ~inv;
    }
    __syncthreads();
    if (tid == 0) s_cnt = 0;
    for (int j = tid; j < P; j += TKL_NT) keys[j] = 0ull;    // padding sorts last
    __syncthreads();
    for (int v = tid; v < rv.nvec; v += TKL_NT) {
      rv.visit(v, [&](float x, int i) {
        const uint32_t key = okey(x);
        if (key > kkey || (key == kkey && static_cast<uint32_t>(i) <= last_index)) {
          const int slot = atomicAdd(&s_cnt, 1);
          if (slot < k) keys[slot] = (static_cast<unsigned long long>(key) << 32) | static_cast<uint32_t>(~static_cast<uint32_t>(i));
        }
      });
    }
    __syncthreads();
    const bool ok = (s_cnt == k);                            // an invariant of the two selects
    // bitonic sort, descending (a larger key first: larger value, then lower index)
    for (int size = 2; size <= P; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int t = tid; t < (P >> 1); t += TKL_NT) {
          const int lo = 2 * t - (t & (stride - 1));
          const int hi = lo + stride;
          const bool desc = ((lo & size) == 0);
          const unsigned long long a = keys[lo], b = keys[hi];
          if ((a < b) == desc) { keys[lo] = b; keys[hi] = a; }
        }
        __syncthreads();
      }
    }
    float* ov = A.out_values + row * static_cast<int64_t>(k);
    int32_t* oi = A.out_indices + row * static_cast<int64_t>(k);
    for (int j = tid; j < k; j += TKL_NT) {
      if (ok) {
        const int i = static_cast<int>(~static_cast<uint32_t>(keys[j] & 0xffffffffull));
        float xv = 0.f;
        rv.visit(rv.vec_of(i), [&](float x, int ii) { if (ii == i) xv = x; });
        ov[j] = xv; oi[j] = i;
      } else {
        ov[j] = __int_as_float(0x7fc00000); oi[j] = -1;
      }
    }
    if (tid == 0 && A.out_flags) A.out_flags[row] = ok ? 0u : FLAG_INTERNAL;
    __syncthreads();
  }
}

}  // namespace gs
