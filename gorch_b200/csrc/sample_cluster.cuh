// Cluster kernel: one thread-block cluster (1, 2, 4 or 8 CTAs) per logits row.
//
// Each CTA owns a contiguous slice of the row's 16-byte vectors and keeps it in
// shared memory, so HBM is read exactly once per logit; later passes read shared
// memory. Cross-CTA reductions go through distributed shared memory: a peer
// stores into the consumer's shared memory, then a cluster barrier publishes it.
// Every CTA loads its own slice with plain vector loads.
//
// Row semantics: model/generate.go:134-260 (mode A), model/qwen/generate.go:
// 77-181 (mode B). Per row:
//   greedy         slice argmax -> rank 0 picks (max value, lowest index).
//   top-k <= 256   pass A: slice -> smem, row max, one running max per thread.
//                  The k-th largest of those 512 per-thread maxima bounds the
//                  k-th largest logit from below, so pass B (shared memory)
//                  collects a few hundred candidates at most; rank 0 merges the
//                  CTAs' lists and finishes in shared memory.
//   top-k off      L: slice -> smem, max and min.  P2 (only with an active
//                  top-p cut): count histogram over 1024 linear buckets of
//                  d = s - max; rank 0 brackets the cut from count-based mass
//                  bounds.  P3: exponentials; certainly-kept / dropped mass goes
//                  to running sums, the bracketed zone to an exact list that
//                  rank 0 cuts by weighted selection.  The CTA whose slice holds
//                  the drawn token rescans one warp's run.
// Rows this kernel does not serve (top-k above 256, a zone or a candidate list
// that outgrows its buffer) are appended to a work list that the single-CTA
// kernel processes right after.
//
// Control flow is uniform across a cluster: every CTA passes the same cluster
// barriers, and nobody touches a peer's shared memory after the last one.
#pragma once

#include <cooperative_groups.h>

#include <type_traits>

#include "sample_kernel.cuh"

namespace gs {
namespace cg = cooperative_groups;

constexpr int CL_MAX = 8;            // largest cluster
constexpr int NB1 = 1024;            // buckets of width 1/32 over d in [-32, 0]
constexpr int ZCAP = 2048;           // exact zone list capacity on rank 0 (entries of 8 B)
constexpr int ZLOC = 1024;           // per-CTA zone list capacity
constexpr int UCAP = 2048;           // merged top-k candidate capacity on rank 0
constexpr int KFAST = 256;           // largest top_k served here
constexpr int KEEP_MAX = 512;        // largest kept set finished here
constexpr int NSUB = 1024;           // sub-buckets of one weighted-selection round
constexpr int REGION_A = 16384;      // bytes: zone keys / merged candidates / histogram staging
constexpr int REGION_B = 16384;      // bytes: local lists, bucket table, selection scratch
constexpr int MIN_SLICE_BYTES = 32768;

struct ClusterArgs {
  KernelArgs k;
  int32_t slice_bytes;      // shared bytes reserved for the slice region
  const double* eb_table;   // 1024 doubles: exp(-b/32)
  int32_t* worklist;        // [0] = count, [1..] = rows left to the single-CTA kernel
};

// Written by peers through distributed shared memory. Every slot has exactly one
// writer, so nothing here needs to be initialised.
struct Xchg {
  unsigned long long u64[CL_MAX];   // packed (key << 32 | payload) per rank
  float mn[CL_MAX];                 // slice minimum per rank
  double K[CL_MAX], D[CL_MAX], Z[CL_MAX];
  int cnt[CL_MAX];
  int giveup[CL_MAX];
  // pushed by rank 0
  float dA, dB;
  int zone_total;
  int verdict;            // 0 owner resolves, 1 poisoned, 2 handed to the work list, 3 id written by rank 0
  int owner;
  unsigned long long cut_key;   // zone entries are kept when key < cut_key, or == cut_key with cut_incl
  int cut_incl;
  double local_target, base_mass, Re, S;
};

// 1024 buckets of width 1/32: round(-32 d) clamped to 1023. Non-decreasing as d falls.
__device__ __forceinline__ int bucket1(float d) {
  float f = fmaf(fmaxf(d, -31.97f), -32.0f, 8388608.0f);
  return __float_as_int(f) & 0x7ff;
}

// Smallest d (d <= 0) whose bucket is <= bmax. round(-32 d) <= bmax holds down to
// -(bmax + 1/2)/32, a tie that rounds to even.
__device__ __forceinline__ float bucket_floor(int bmax) {
  if (bmax >= NB1 - 1) return -INFINITY;
  if (bmax < 0) return INFINITY;
  float t = -(static_cast<float>(2 * bmax + 1) * 0.015625f);
  return (bucket1(t) <= bmax) ? t : __uint_as_float(__float_as_uint(t) - 1u);
}

// exp(d), d <= 0, via the 256-entry 2^(j/256) table entirely in f64 (about 1 ulp);
// falls back to the library below -700 and for -Inf / NaN.
__device__ __forceinline__ double exp_safe(float d, const double* __restrict__ tab) {
  if (!(d >= -700.0f)) return exp(static_cast<double>(d));
  const double x = static_cast<double>(d);
  double t = fma(x, 369.3299304675746, 6755399441055744.0);
  int ki = __double2loint(t);
  double kd = t - 6755399441055744.0;
  double r = fma(kd, -0x1.62e42fee00000p-9, x);
  r = fma(kd, -0x1.a39ef35793c76p-41, r);
  double q = fma(r, 4.1666666666666664e-02, 1.6666666666666666e-01);
  q = fma(q, r, 0.5);
  q = fma(q, r, 1.0);
  double tj = tab[ki & 255];
  double res = fma(tj, q * r, tj);
  int hi = __double2hiint(res) + ((ki >> 8) << 20);
  return __hiloint2double(hi, __double2loint(res));
}

// exp(d) for -31.9 < d <= 0: d = -b/32 + dl with |dl| <= 1/64 exactly (f32),
// exp = E[b] * (1 + dl + tail(dl)); the tail dl^2/2 + ... + dl^5/120 is below
// 1.3e-4 and is evaluated in f32, which leaves a relative error near 2e-11.
__device__ __forceinline__ double exp_fast(float d, const double* __restrict__ eb) {
  float f = fmaf(d, -32.0f, 8388608.0f);
  int b = __float_as_int(f) & 0x7ff;
  float dl = fmaf(f - 8388608.0f, 0.03125f, d);
  float t = fmaf(dl, 8.3333338e-3f, 4.1666668e-2f);
  t = fmaf(t, dl, 1.6666667e-1f);
  t = fmaf(t, dl, 0.5f);
  float tail = t * (dl * dl);
  double w = static_cast<double>(dl) + static_cast<double>(tail);
  double E = eb[b];
  return fma(E, w, E);
}

template <typename T> struct Neutral;
template <> struct Neutral<float> { static constexpr uint32_t word = 0xff800000u; };      // -Inf
template <> struct Neutral<uint16_t> { static constexpr uint32_t word = 0xff80ff80u; };   // two bf16 -Inf

// Load vector v of the row; lanes outside [0, V) become -Inf. Max, min and the NaN
// flag cover the valid lanes only.
template <typename T>
__device__ __forceinline__ uint4 mask_and_stats(const RowView<T>& rv, int v, uint4 raw, float& vmax, float& vmin, bool& nan_seen) {
  constexpr int VEC = Elem<T>::VEC;
  float x[VEC];
  Elem<T>::unpack(raw, x);
  if (v > 0 && v < rv.nvec - 1) {
#pragma unroll
    for (int c = 0; c < VEC; c++) {
      vmax = fmaxf(vmax, x[c]);
      vmin = fminf(vmin, x[c]);
      nan_seen |= (x[c] != x[c]);
    }
    return raw;
  }
  uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  const int i0 = v * VEC - rv.shift;
#pragma unroll
  for (int c = 0; c < VEC; c++) {
    int i = i0 + c;
    if (i < 0 || i >= rv.V) {
      if (sizeof(T) == 4) w[c] = 0xff800000u;
      else if (c & 1) w[c >> 1] = (w[c >> 1] & 0x0000ffffu) | 0xff800000u;
      else w[c >> 1] = (w[c >> 1] & 0xffff0000u) | 0x0000ff80u;
    } else {
      vmax = fmaxf(vmax, x[c]);
      vmin = fminf(vmin, x[c]);
      nan_seen |= (x[c] != x[c]);
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <typename T>
__device__ __forceinline__ uint4 load_masked(const RowView<T>& rv, int v, float& vmax, float& vmin, bool& nan_seen) {
  return mask_and_stats(rv, v, __ldg(rv.vbase + v), vmax, vmin, nan_seen);
}

__device__ __forceinline__ void block_min_i2(int& a_min, int& b_min, Ctl& c, int tid) {
  a_min = __reduce_min_sync(FULL, a_min);
  b_min = __reduce_min_sync(FULL, b_min);
  __syncthreads();
  if ((tid & 31) == 0) { c.red_i[tid >> 5] = a_min; c.red_u64[tid >> 5] = static_cast<unsigned long long>(static_cast<uint32_t>(b_min)); }
  __syncthreads();
  int a = c.red_i[0], b = static_cast<int>(c.red_u64[0]);
#pragma unroll
  for (int w = 1; w < NW; w++) { a = min(a, c.red_i[w]); b = min(b, static_cast<int>(c.red_u64[w])); }
  a_min = a; b_min = b;
}
__device__ __forceinline__ unsigned long long block_min_u64(unsigned long long v, Ctl& c, int tid) {
  return ~block_max_u64(~v, c, tid);
}

// Exclusive prefix over two doubles per thread at once.
__device__ __forceinline__ void block_scan_excl_d2(double a, double b, double& ea, double& eb_, double& ta, double& tb, Ctl& c, int tid) {
  int lane = tid & 31, w = tid >> 5;
  double ia = warp_scan_incl_d(a, lane), ib = warp_scan_incl_d(b, lane);
  __syncthreads();
  if (lane == 31) { c.red_d[w] = ia; c.red_d2[w] = ib; }
  __syncthreads();
  double ba = 0, bb = 0, sa = 0, sb = 0;
#pragma unroll
  for (int j = 0; j < NW; j++) {
    double va = c.red_d[j], vb = c.red_d2[j];
    if (j < w) { ba += va; bb += vb; }
    sa += va; sb += vb;
  }
  ea = ba + ia - a; eb_ = bb + ib - b; ta = sa; tb = sb;
}

template <typename T>
__global__ void __launch_bounds__(NT, 2) sample_cluster_kernel(ClusterArgs CA) {
  extern __shared__ __align__(16) unsigned char dyn[];
  __shared__ Ctl ctl;
  __shared__ Xchg X;
  __shared__ double s_tab[256];
  __shared__ double s_kseg[NW];
  __shared__ double s_zk[CL_MAX];
  __shared__ uint32_t s_sel[256];

  cg::cluster_group cluster = cg::this_cluster();
  // a row whose sequence has ended (model/generate.go:82-84) is skipped by its whole cluster, before any barrier
  if (CA.k.row_done && CA.k.row_done[CA.k.row_offset + blockIdx.x / cluster.num_blocks()] != 0) return;
  cluster.barrier_arrive();          // matched by the wait before the first remote store
  const int C = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  const KernelArgs& A = CA.k;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t row_id = A.row_offset + blockIdx.x / C;
  const int V = A.V;
  constexpr int VEC = Elem<T>::VEC;
  const T* row = static_cast<const T*>(A.logits) + row_id * A.row_stride;
  RowView<T> rv;
  rv.init(row, V);
  const int SV = (rv.nvec + C - 1) / C;                 // vectors per slice
  const int v0 = min(rv.nvec, rank * SV), v1 = min(rv.nvec, v0 + SV);
  const int nv = v1 - v0;

  uint4* slice = reinterpret_cast<uint4*>(dyn);
  unsigned char* regA = dyn + CA.slice_bytes;
  unsigned char* regB = regA + REGION_A;

  RowCfg cfg;
  if (A.force_greedy) { cfg.temperature = 0.f; cfg.top_k = 0; cfg.top_p = 0.f; cfg.topp_mode = 0; }
  else cfg = A.cfgs[row_id];
  const float Tm = cfg.temperature;

  if (tid < 256) s_tab[tid] = A.exp_table[tid];
  if (tid < CL_MAX) s_zk[tid] = 0.0;
  if (tid == 0) { ctl.cand_count = 0; ctl.overflow = 0; }
  __syncthreads();

  Xchg* X0 = cluster.map_shared_rank(&X, 0);
  const double QNAN = __longlong_as_double(0x7ff8000000000000ll);
  auto finish = [&](int id, uint32_t flags, const RowDebug& dbg) {
    if (tid == 0) {
      A.out_ids[row_id] = id;
      if (A.out_flags) A.out_flags[row_id] = flags;
      if (A.out_debug) A.out_debug[row_id] = dbg;
    }
  };
  auto fill_probs_slice = [&](double v) {   // this CTA's share of the dense probability row
    if (A.out_probs) {
      double* pr = A.out_probs + row_id * static_cast<int64_t>(V);
      int i_lo = max(0, v0 * VEC - rv.shift), i_hi = min(V, v1 * VEC - rv.shift);
      for (int i = i_lo + tid; i < i_hi; i += NT) pr[i] = v;
    }
  };
  auto fill_probs_row = [&](double v) {
    if (A.out_probs) {
      double* pr = A.out_probs + row_id * static_cast<int64_t>(V);
      for (int i = tid; i < V; i += NT) pr[i] = v;
    }
  };
  auto to_worklist = [&]() {                // rank 0 hands the row to the single-CTA kernel
    if (tid == 0) {
      int slot = atomicAdd(&CA.worklist[0], 1);
      CA.worklist[1 + slot] = static_cast<int32_t>(row_id);
    }
  };

  RowDebug dbg;
  dbg.sum_exp = 0; dbg.resum = 1.0; dbg.edge_lo = 0; dbg.edge_hi = 0; dbg.kept = 0;
  dbg.max_scaled = 0; dbg.threshold = __int_as_float(0x7fc00000); dbg.path = 0;
  for (int q = 0; q < 8; q++) dbg.reserved[q] = 0;
  long long tprev = clock64();
  auto stamp = [&](int slot) { long long now = clock64(); dbg.reserved[slot] = static_cast<uint32_t>(now - tprev); tprev = now; };

  // ================================================================ greedy
  if (Tm == 0.0f) {
    unsigned long long best = 0ull;
    for (int v = v0 + tid; v < v1; v += NT) {
      uint4 raw = __ldg(rv.vbase + v);
      rv.visit_raw(raw, v, [&](float x, int i, int) {
        unsigned long long p = (static_cast<unsigned long long>(okey(x)) << 32) |
                               static_cast<uint32_t>(~static_cast<uint32_t>(i));
        best = p > best ? p : best;
      });
    }
    best = block_max_u64(best, ctl, tid);
    fill_probs_slice(0.0);
    cluster.barrier_wait();
    if (tid == 0) X0->u64[rank] = best;
    cluster.sync();
    if (rank == 0) {
      unsigned long long b = 0;
      for (int r = 0; r < C; r++) b = X.u64[r] > b ? X.u64[r] : b;
      int id = static_cast<int>(~static_cast<uint32_t>(b & 0xffffffffull));
      float x0 = 0.f;
      rv.visit(0, [&](float x, int i) { if (i == 0) x0 = x; });
      if (x0 != x0) id = 0;     // generate.go:136: maxVal starts as NaN, nothing is greater
      if (A.out_probs && tid == 0) A.out_probs[row_id * static_cast<int64_t>(V) + id] = 1.0;
      dbg.kept = 1;
      finish(id, 0u, dbg);
    }
    return;
  }
  if (!(Tm > 0.0f) || !(Tm < INFINITY)) {
    fill_probs_slice(QNAN);
    if (rank == 0) finish(-1, FLAG_BAD_CFG, dbg);
    cluster.barrier_wait();
    return;
  }

  const int topk = (cfg.top_k > 0 && cfg.top_k < V) ? cfg.top_k : 0;
  const bool topp_on = (cfg.top_p > 0.0f && cfg.top_p < 1.0f);
  const int mode = cfg.topp_mode;
  const double u = A.uniforms[row_id];
  const double plim = (mode == 0) ? static_cast<double>(cfg.top_p) * 1.5 : static_cast<double>(cfg.top_p);
  const bool cut_on = topp_on && !(mode == 0 && plim >= 1.0);
  const bool t_is_one = (Tm == 1.0f);
  uint32_t flags = 0;

  if (topk > KFAST || (topk > 0 && topk * C > UCAP / 2)) {
    // large top-k: the single-CTA kernel's counting select serves it
    if (rank == 0) to_worklist();
    cluster.barrier_wait();
    return;
  }

  // ---- L / pass A: slice -> shared memory; max, min, NaN, one running max per thread
  float xmax = -INFINITY, xmin = INFINITY;
  bool nan_seen = false;
  // four vectors per thread in flight at a time: a slice of 50 KB is two trips to HBM, not seven
  for (int vb = v0 + tid; vb < v1; vb += 4 * NT) {
    uint4 r4[4];
#pragma unroll
    for (int q = 0; q < 4; q++) r4[q] = __ldg(rv.vbase + min(vb + q * NT, v1 - 1));
#pragma unroll
    for (int q = 0; q < 4; q++) {
      const int v = vb + q * NT;
      if (v < v1) slice[v - v0] = mask_and_stats(rv, v, r4[q], xmax, xmin, nan_seen);
    }
  }
  const float tmax = xmax;                                  // this thread's group maximum
  const int anynan_loc = block_max_i(nan_seen ? 1 : 0, ctl, tid);
  const unsigned long long pmax = block_max_u64(static_cast<unsigned long long>(okey(xmax)) << 32, ctl, tid);
  const float slice_min = okey_to_float(static_cast<uint32_t>(block_min_u64(static_cast<unsigned long long>(okey(xmin)), ctl, tid)));
  stamp(0);

  // ======================================================= top-k, k <= 256
  if (topk > 0) {
    // thr0: a lower bound of the k-th largest logit = lower edge of the 16-bit key
    // bin that holds the k-th largest of the 512 per-thread maxima.
    uint32_t prefix = 0, mask = 0;
    int need = topk;
    const uint32_t mykey = okey(tmax);
    bool have_thr = true;
    for (int round = 0; round < 2; round++) {
      const int sh = 24 - 8 * round;
      __syncthreads();
      if (tid < 256) s_sel[tid] = 0;
      if (tid == 0) ctl.bcast_i[0] = -1;
      __syncthreads();
      if ((mykey & mask) == prefix) atomicAdd(&s_sel[(mykey >> sh) & 255u], 1u);
      __syncthreads();
      if (tid < 32) {
        int loc[8];
        int s = 0;
#pragma unroll
        for (int j = 7; j >= 0; j--) { s += static_cast<int>(s_sel[tid * 8 + j]); loc[j] = s; }
        int run = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          int t = __shfl_down_sync(FULL, run, o);
          if (tid + o < 32) run += t;
        }
        const int above = run - s;
        if (above < need && above + s >= need) {
#pragma unroll
          for (int j = 7; j >= 0; j--) {
            if (above + loc[j] >= need) {
              ctl.bcast_i[0] = tid * 8 + j;
              ctl.bcast_i[1] = need - (above + loc[j] - static_cast<int>(s_sel[tid * 8 + j]));
              break;
            }
          }
        }
      }
      __syncthreads();
      if (ctl.bcast_i[0] < 0) { have_thr = false; break; }   // fewer than k groups: keep everything
      prefix |= static_cast<uint32_t>(ctl.bcast_i[0]) << sh;
      mask |= 255u << sh;
      need = ctl.bcast_i[1];
    }
    float thr0 = -INFINITY;
    if (prefix <= 0x007fffffu) have_thr = false;             // bound at or below -Inf: keep everything
    if (have_thr) {
      __syncthreads();
      if (tid == 0) ctl.thr = quotient_class_floor(okey_to_float(prefix), Tm);
      __syncthreads();
      thr0 = ctl.thr;
    }
    // pass B: candidates >= thr0 from shared memory
    uint2* lc = reinterpret_cast<uint2*>(regB);              // up to 2048 entries
    const int cap_r = UCAP / C;
    for (int j = tid; j < nv; j += NT) {
      float x[VEC];
      Elem<T>::unpack(slice[j], x);
      bool any = false;
#pragma unroll
      for (int c = 0; c < VEC; c++) any |= (x[c] >= thr0);
      if (any) {
        const int i0 = (v0 + j) * VEC - rv.shift;
#pragma unroll
        for (int c = 0; c < VEC; c++) {
          int i = i0 + c;
          if (x[c] >= thr0 && i >= 0 && i < V) {
            int slot = atomicAdd(&ctl.cand_count, 1);
            if (slot < cap_r) lc[slot] = make_uint2(__float_as_uint(x[c]), static_cast<uint32_t>(i));
          }
        }
      }
    }
    __syncthreads();
    const int n_loc = ctl.cand_count;
    const bool giveup = n_loc > cap_r;
    stamp(1);
    cluster.barrier_wait();
    if (tid == 0) {
      X0->u64[rank] = pmax | static_cast<unsigned long long>(anynan_loc);
      X0->cnt[rank] = giveup ? 0 : n_loc;
      X0->giveup[rank] = giveup ? 1 : 0;
    }
    if (!giveup) {
      uint2* dst = cluster.map_shared_rank(reinterpret_cast<uint2*>(regA), 0) + rank * cap_r;
      for (int j = tid; j < n_loc; j += NT) dst[j] = lc[j];
    }
    cluster.sync();                                          // B1: the only barrier of this path
    if (rank != 0) return;
    stamp(2);
    // ---------------- rank 0: merge and finish in shared memory
    dbg.path = 1;
    unsigned long long mx = 0;
    int anynan = 0, bad = 0, n = 0;
    for (int r = 0; r < C; r++) {
      mx = X.u64[r] > mx ? X.u64[r] : mx;
      anynan |= static_cast<int>(X.u64[r] & 1ull);
      bad |= X.giveup[r];
      n += X.cnt[r];
    }
    if (bad) { to_worklist(); return; }
    xmax = okey_to_float(static_cast<uint32_t>(mx >> 32));
    const float m = scale_t(xmax, Tm);
    dbg.max_scaled = m;
    auto poison_exit = [&](bool nan_sum) {
      fill_probs_row(QNAN);
      if (nan_sum) dbg.sum_exp = QNAN;
      finish(V - 1, flags | FLAG_NONFINITE | FLAG_FALLBACK, dbg);
    };
    if (anynan || !(fabsf(m) < INFINITY)) { poison_exit(true); return; }
    // compact the per-rank sub-ranges of region A into region B
    uint2* uc = reinterpret_cast<uint2*>(regB);
    {
      const uint2* src = reinterpret_cast<const uint2*>(regA);
      int off = 0;
      for (int r = 0; r < C; r++) {
        const int cr = X.cnt[r];
        for (int j = tid; j < cr; j += NT) uc[off + j] = src[r * cap_r + j];
        off += cr;
      }
    }
    __syncthreads();
    float keep_lo = -INFINITY;
    if (n > topk) {
      uint32_t kkey = block_select_kth(uc, n, topk, s_sel, ctl, tid);
      if (tid == 0) ctl.thr = quotient_class_floor(okey_to_float(kkey), Tm);
      __syncthreads();
      keep_lo = ctl.thr;
    }
    // kept entries -> region A; order by index with a counting rank
    uint2* kp = reinterpret_cast<uint2*>(regA);
    __syncthreads();
    if (tid == 0) ctl.cand_count = 0;
    __syncthreads();
    for (int j = tid; j < n; j += NT) {
      uint2 e = uc[j];
      if (__uint_as_float(e.x) >= keep_lo) {
        int slot = atomicAdd(&ctl.cand_count, 1);
        if (slot < KEEP_MAX) kp[slot] = e;
      }
    }
    __syncthreads();
    const int nk = ctl.cand_count;
    if (nk > KEEP_MAX) { to_worklist(); return; }            // long run of ties at the threshold
    // work arrays over the slice region (free now)
    unsigned char* wr = dyn;
    float* sx = reinterpret_cast<float*>(wr);                // [512] scaled value, index order
    int* sidx = reinterpret_cast<int*>(wr + 2048);           // [512]
    double* se = reinterpret_cast<double*>(wr + 4096);       // [512]
    double* sf = reinterpret_cast<double*>(wr + 8192);       // [512]
    int* rnk = reinterpret_cast<int*>(wr + 12288);           // [512]
    int* ord = reinterpret_cast<int*>(wr + 14336);           // [512]
    float thr_s = INFINITY;
    if (tid < nk) {
      const uint32_t myi = kp[tid].y;
      int r = 0;
      for (int l = 0; l < nk; l++) r += (kp[l].y < myi) ? 1 : 0;
      float s = scale_t(__uint_as_float(kp[tid].x), Tm);
      sx[r] = s;
      sidx[r] = static_cast<int>(myi);
      thr_s = s;
    }
    dbg.threshold = okey_to_float(static_cast<uint32_t>(block_min_u64(static_cast<unsigned long long>(okey(thr_s)), ctl, tid)));
    __syncthreads();
    double e_me = 0.0;
    if (tid < nk) e_me = exp(static_cast<double>(sx[tid] - m));   // f32 subtract, f64 exp (generate.go:176)
    double S;
    (void)block_scan_excl_d(e_me, S, ctl, tid);
    dbg.sum_exp = S;
    const double q_me = e_me / S;                                 // generate.go:179-181
    if (tid < nk) se[tid] = q_me;
    __syncthreads();
    double f_me = q_me;
    if (topp_on) {
      // order by probability; equal probabilities by index, ascending in both flavours
      // (mode A removes the lowest index first, mode B keeps it first)
      if (tid < nk) {
        int r = 0;
        if (mode == 0) { for (int l = 0; l < nk; l++) { double ql = se[l]; r += (ql < q_me || (ql == q_me && l < tid)) ? 1 : 0; } }
        else           { for (int l = 0; l < nk; l++) { double ql = se[l]; r += (ql > q_me || (ql == q_me && l < tid)) ? 1 : 0; } }
        ord[r] = tid;
        rnk[tid] = r;
      }
      __syncthreads();
      if (mode == 0) {
        // generate.go:184-228: the mass left after removing the r smallest is a suffix sum.
        // Scan from the largest down: position t holds rank nk-1-t.
        const double v = (tid < nk) ? se[ord[nk - 1 - tid]] : 0.0;
        double tot;
        const double exs = block_scan_excl_d(v, tot, ctl, tid);
        if (tid < nk) sf[nk - 1 - tid] = exs + v;                   // sf[r] = left after removing r smallest
        __syncthreads();
        int rs = nk;
        if (tid < nk && sf[tid] <= plim) rs = tid;
        const int rstar = block_min_i(rs, ctl, tid);
        if (rstar == nk) { dbg.resum = 0.0; poison_exit(false); return; }   // everything removed: 0/0
        const double resum = sf[rstar];
        if (fabs(resum - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
        if (rstar > 0 && fabs(sf[rstar - 1] - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
        dbg.resum = resum;
        f_me = (tid < nk && rnk[tid] >= rstar) ? q_me / resum : 0.0;
      } else {
        // qwen/generate.go:123-153: shortest descending prefix with mass >= p
        const double v = (tid < nk) ? se[ord[tid]] : 0.0;
        double tot;
        const double exs = block_scan_excl_d(v, tot, ctl, tid);
        if (tid < nk) sf[tid] = exs + v;
        __syncthreads();
        int cl = nk;
        if (tid < nk && sf[tid] >= plim) cl = tid + 1;
        const int cutn = block_min_i(cl, ctl, tid);
        const double resum = sf[cutn - 1];
        if (fabs(resum - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
        if (cutn >= 2 && fabs(sf[cutn - 2] - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
        if (cutn < nk && se[ord[cutn]] == se[ord[cutn - 1]]) flags |= FLAG_TIE_CUT;
        dbg.resum = resum;
        f_me = (tid < nk && rnk[tid] < cutn) ? q_me / resum : 0.0;
      }
    }
    dbg.kept = block_sum_i((tid < nk && f_me > 0) ? 1 : 0, ctl, tid);
    if (A.out_probs) {
      fill_probs_row(0.0);
      __syncthreads();
      if (tid < nk) A.out_probs[row_id * static_cast<int64_t>(V) + sidx[tid]] = f_me;
    }
    // draw (generate.go:231-239): first index with u < cumulative
    double tot;
    const double cexcl = block_scan_excl_d(f_me, tot, ctl, tid);
    const double c_me = cexcl + f_me;
    int pl = nk;
    if (tid < nk && u < c_me) pl = tid;
    const int pick = block_min_i(pl, ctl, tid);
    if (pick < nk && tid == pick) { ctl.bcast_d[0] = cexcl; ctl.bcast_d[1] = c_me; }
    __syncthreads();
    int id;
    if (pick < nk) {
      id = sidx[pick];
      const double lo = ctl.bcast_d[0], hi = ctl.bcast_d[1];
      dbg.edge_lo = lo; dbg.edge_hi = hi;
      if ((pick > 0 && u - lo <= 1e-6) || hi - u <= 1e-6) flags |= FLAG_BOUNDARY;
    } else {
      id = V - 1;
      flags |= FLAG_FALLBACK;
      dbg.edge_lo = dbg.edge_hi = tot;
      if (u - tot <= 1e-6) flags |= FLAG_BOUNDARY;
    }
    stamp(3);
    finish(id, flags, dbg);
    return;
  }

  // ============================================================ full row (top-k off)
  dbg.path = 2;
  flags |= FLAG_GENERAL_PATH;
  cluster.barrier_wait();
  if (tid == 0) {
    const unsigned long long p = pmax | static_cast<unsigned long long>(anynan_loc);
    for (int r = 0; r < C; r++) {
      Xchg* xr = cluster.map_shared_rank(&X, r);
      xr->u64[rank] = p;
      xr->mn[rank] = slice_min;
    }
  }
  cluster.sync();                                            // G1
  stamp(1);
  float row_min = INFINITY;
  int anynan = 0;
  {
    unsigned long long mx = 0;
    for (int r = 0; r < C; r++) {
      mx = X.u64[r] > mx ? X.u64[r] : mx;
      anynan |= static_cast<int>(X.u64[r] & 1ull);
      row_min = fminf(row_min, X.mn[r]);
    }
    xmax = okey_to_float(static_cast<uint32_t>(mx >> 32));
  }
  const float m = scale_t(xmax, Tm);
  dbg.max_scaled = m;
  const bool poisoned_early = anynan || !(fabsf(m) < INFINITY);
  // every element has d > -31.9: the bucket-table exponential applies
  const bool fast_ok = !poisoned_early && (scale_t(row_min, Tm) - m > -31.9f);

  // ---- P2: count histogram + bracket of the top-p cut
  float dA = -INFINITY, dB = -INFINITY;    // certainly kept: d >= dA; zone: dB <= d < dA; dropped: d < dB
  int nzone = 0;
  if (cut_on) {
    uint32_t* hist = (rank == 0) ? reinterpret_cast<uint32_t*>(regA) : reinterpret_cast<uint32_t*>(regB);
    for (int j = tid; j < NB1; j += NT) hist[j] = 0;
    __syncthreads();
    for (int j = tid; j < nv; j += NT) {
      float x[VEC];
      Elem<T>::unpack(slice[j], x);
      if (t_is_one) {
#pragma unroll
        for (int c = 0; c < VEC; c++) atomicAdd(&hist[bucket1(x[c] - m)], 1u);
      } else {
#pragma unroll
        for (int c = 0; c < VEC; c++) atomicAdd(&hist[bucket1(__fdiv_rn(x[c], Tm) - m)], 1u);
      }
    }
    __syncthreads();
    if (rank != 0) {
      // rank 0 stages [C][1024] counters across its regions A and B (32 KB at C = 8)
      uint32_t* dst = cluster.map_shared_rank(reinterpret_cast<uint32_t*>(regA), 0) + rank * NB1;
      for (int j = tid; j < NB1; j += NT) dst[j] = hist[j];
    }
    stamp(2);
    cluster.sync();                                          // G2
    if (rank == 0) {
      const uint32_t* all = reinterpret_cast<const uint32_t*>(regA);
      constexpr int PER = NB1 / NT;                          // 2 buckets per thread
      double lo_inc[PER], hi_inc[PER];
      int cb[PER];
      double slo = 0.0, shi = 0.0;
#pragma unroll
      for (int j = 0; j < PER; j++) {
        const int b = tid * PER + j;
        uint32_t cnt = 0;
        for (int r = 0; r < C; r++) cnt += all[r * NB1 + b];
        cb[j] = static_cast<int>(cnt);
        const double c = static_cast<double>(cnt);
        // bucket b holds d in [-(b+.5)/32, -(b-.5)/32]; the last one everything below.
        // Masked lanes (-Inf) are counted there too; their mass bound starts at 0.
        const double eb = __ldg(CA.eb_table + b);
        const double elo = (b == NB1 - 1) ? 0.0 : eb * 0.98449643700540845 * (1.0 - 1e-7);   // exp(-1/64)
        const double ehi = fmin(1.0, eb * 1.0157477085866857 * (1.0 + 1e-7));                 // exp(+1/64)
        slo += c * elo; shi += c * ehi;
        lo_inc[j] = slo; hi_inc[j] = shi;
      }
      double ex_lo, ex_hi, tot_lo, tot_hi;
      block_scan_excl_d2(slo, shi, ex_lo, ex_hi, tot_lo, tot_hi, ctl, tid);
      int b1 = NB1 - 1, b2 = NB1 - 1;
#pragma unroll
      for (int j = 0; j < PER; j++) {
        const int b = tid * PER + j;
        const double a_lo = ex_lo + lo_inc[j], a_hi = ex_hi + hi_inc[j];
        const double r_hi = a_hi / (a_hi + (tot_lo - a_lo));   // largest possible mass fraction through bucket b
        const double r_lo = a_lo / (a_lo + (tot_hi - a_hi));   // smallest possible
        bool c1, c2;
        if (mode == 0) { c1 = r_hi > plim * (1.0 - 1e-9); c2 = r_lo > plim * (1.0 + 1e-9); }
        else           { c1 = r_hi >= plim * (1.0 - 1e-9); c2 = r_lo >= plim * (1.0 + 1e-9); }
        if (c1) b1 = min(b1, b);
        if (c2) b2 = min(b2, b);
      }
      block_min_i2(b1, b2, ctl, tid);
      if (b2 < b1) b2 = b1;
      int nz_part = 0;
#pragma unroll
      for (int j = 0; j < PER; j++) {
        const int b = tid * PER + j;
        if (b >= b1 && b <= b2) nz_part += cb[j];
      }
      const int nz = block_sum_i(nz_part, ctl, tid);
      if (tid == 0) {
        const float tA = bucket_floor(b1 - 1), tB = bucket_floor(b2);
        for (int r = 0; r < C; r++) {
          Xchg* xr = cluster.map_shared_rank(&X, r);
          xr->dA = tA; xr->dB = tB; xr->zone_total = nz;
        }
      }
    }
    stamp(3);
    cluster.sync();                                          // G3
    dA = X.dA; dB = X.dB; nzone = X.zone_total;
  }
  // the zone count includes masked lanes when the zone reaches the last bucket; they are never listed
  const bool zone_ok = nzone <= ZCAP + 2 * VEC;

  // ---- P3: exponentials. Each warp owns a contiguous run of the slice; eight elements in flight.
  double* ebs = reinterpret_cast<double*>(regB + 8192);     // bucket table exp(-b/32), 8 KB
  uint2* lz = reinterpret_cast<uint2*>(regB);               // local zone list (d bits, idx), 1024 entries
  __syncthreads();
  if (fast_ok) for (int j = tid; j < NB1; j += NT) ebs[j] = __ldg(CA.eb_table + j);
  if (tid == 0) ctl.cand_count = 0;
  __syncthreads();
  const int wv = (nv + NW - 1) / NW;                        // vectors per warp run
  const int w0 = min(nv, warp * wv), w1 = min(nv, w0 + wv);
  double t0 = 0.0, t1 = 0.0, t2 = 0.0, t3 = 0.0, dsum = 0.0, zsum = 0.0;
  if (zone_ok) {
    auto body = [&](auto fast_tag, auto tone_tag) {
      constexpr bool FAST = decltype(fast_tag)::value;
      constexpr bool TONE = decltype(tone_tag)::value;
      constexpr int U = (VEC == 4) ? 2 : 1;                  // vectors per iteration: 8 elements
      for (int j = w0 + lane; j < w1; j += 32 * U) {
        float x[8];
        uint4 ra = slice[j];
        if (U == 2) {
          uint4 rb = (j + 32 < w1) ? slice[j + 32]
                                   : make_uint4(Neutral<T>::word, Neutral<T>::word, Neutral<T>::word, Neutral<T>::word);
          float xa[VEC], xb[VEC];
          Elem<T>::unpack(ra, xa);
          Elem<T>::unpack(rb, xb);
#pragma unroll
          for (int c = 0; c < 4; c++) { x[c] = xa[c]; x[4 + c] = xb[c]; }
        } else {
          float xa[VEC];
          Elem<T>::unpack(ra, xa);
#pragma unroll
          for (int c = 0; c < 8; c++) x[c] = xa[c % VEC];
        }
        double e[8];
        float d[8];
        float dmin = 0.0f;
#pragma unroll
        for (int c = 0; c < 8; c++) {
          const float s = TONE ? x[c] : __fdiv_rn(x[c], Tm);
          d[c] = s - m;
          if (FAST) e[c] = (d[c] > -31.9f) ? exp_fast(d[c], ebs) : 0.0;   // only masked lanes (-Inf) are below
          else      e[c] = exp_safe(d[c], s_tab);
          dmin = fminf(dmin, d[c]);
        }
        t0 += e[0] + e[4]; t1 += e[1] + e[5]; t2 += e[2] + e[6]; t3 += e[3] + e[7];
        if (dmin < dA) {
#pragma unroll
          for (int c = 0; c < 8; c++) {
            if (d[c] < dA) {
              if (d[c] >= dB) {
                const int jj = (U == 2 && c >= 4) ? j + 32 : j;
                const int i = (v0 + jj) * VEC - rv.shift + ((U == 2) ? (c & 3) : c);
                if (jj < w1 && i >= 0 && i < V) {
                  const int slot = atomicAdd(&ctl.cand_count, 1);
                  if (slot < ZLOC) lz[slot] = make_uint2(__float_as_uint(d[c]), static_cast<uint32_t>(i));
                  zsum += e[c];
                }
              } else {
                dsum += e[c];
              }
            }
          }
        }
      }
    };
    if (fast_ok) { if (t_is_one) body(std::true_type{}, std::true_type{}); else body(std::true_type{}, std::false_type{}); }
    else         { if (t_is_one) body(std::false_type{}, std::true_type{}); else body(std::false_type{}, std::false_type{}); }
  }
  const double tot_w = warp_sum_d((t0 + t1) + (t2 + t3));
  dsum = warp_sum_d(dsum); zsum = warp_sum_d(zsum);
  // certainly-kept mass of this warp's run. With dA = +Inf nothing is certainly kept (exactly 0);
  // otherwise the row maximum is, and the subtraction's rounding is far below that mass.
  const double kw = (dA == INFINITY) ? 0.0 : tot_w - dsum - zsum;
  if (lane == 0) s_kseg[warp] = kw;
  const double Kr = block_sum_d(lane == 0 ? kw : 0.0, ctl, tid);
  const double Dr = block_sum_d(lane == 0 ? dsum : 0.0, ctl, tid);
  const double Zr = block_sum_d(lane == 0 ? zsum : 0.0, ctl, tid);
  const int nz_cta = ctl.cand_count;
  // Rank r owns the sub-range [r*ZCAP/C, (r+1)*ZCAP/C) of rank 0's region A.
  const int zcap_r = ZCAP / C;
  const int zlog = 31 - __clz(zcap_r);
  const bool z_over = nz_cta > min(ZLOC, zcap_r);
  const int nz_loc = z_over ? 0 : nz_cta;
  if (tid == 0) {
    X0->K[rank] = Kr; X0->D[rank] = Dr; X0->Z[rank] = Zr;
    X0->cnt[rank] = nz_loc;
    X0->giveup[rank] = (z_over || !zone_ok) ? 1 : 0;
  }
  {
    unsigned long long* dst = cluster.map_shared_rank(reinterpret_cast<unsigned long long*>(regA), 0) + rank * zcap_r;
    for (int j = tid; j < nz_loc; j += NT) {
      const uint2 e = lz[j];
      dst[j] = zone_key(__uint_as_float(e.x), static_cast<int>(e.y), mode);
    }
  }
  stamp(4);
  cluster.sync();                                            // G4
  stamp(5);

  // ---- rank 0: exact cut inside the zone by weighted selection, then the owner of the draw
  if (rank == 0) {
    double Ktot = 0, Dtot = 0, Ztot = 0;
    int bad = 0, nz = 0;
    for (int r = 0; r < C; r++) { Ktot += X.K[r]; Dtot += X.D[r]; Ztot += X.Z[r]; bad |= X.giveup[r]; nz += X.cnt[r]; }
    const double S = Ktot + Ztot + Dtot;
    dbg.sum_exp = S;
    const bool poisoned = poisoned_early || !(S == S) || !(S > 0.0);
    const unsigned long long* zk = reinterpret_cast<const unsigned long long*>(regA);
    // zone entry t of the staged list is live when it lies inside its rank's filled part
    auto zlive = [&](int t) -> bool { return (t & (zcap_r - 1)) < X.cnt[t >> zlog]; };
    unsigned long long cut_key = 0ull;     // nothing of the zone kept
    int cut_incl = 0;
    if (cut_on && !poisoned && !bad && nz > 0) {
      // G(c) = Ktot + mass{key <= c} rises along the zone order. Both flavours need the first
      // key c* where G "crosses": mode B (first G/S >= p) keeps through c*, mode A (first
      // G/S > 1.5p) keeps everything before it. Narrow [lo, hi] around c* with linear
      // sub-buckets until at most 32 keys remain, then one warp finishes.
      auto crossed = [&](double g) -> bool { return mode == 0 ? (g / S > plim) : (g / S >= plim); };
      if (Ktot > 0.0 && crossed(Ktot)) bad = 1;              // the bracket was wrong
      double* sm = reinterpret_cast<double*>(regB);           // [NSUB] mass per sub-bucket
      int* sc = reinterpret_cast<int*>(regB + 8192);          // [NSUB] count per sub-bucket
      unsigned long long lo = ~0ull, hi = 0ull;
      for (int t = tid; t < ZCAP; t += NT) {
        if (zlive(t)) { const unsigned long long k = zk[t]; lo = k < lo ? k : lo; hi = k > hi ? k : hi; }
      }
      lo = block_min_u64(lo, ctl, tid);
      hi = block_max_u64(hi, ctl, tid);
      double gbase = Ktot;                                     // Ktot + mass of keys below lo; never crossed
      int inrange = nz;
      bool all_in = false;
      for (int iter = 0; iter < 8 && inrange > 32 && !bad && !all_in; iter++) {
        const unsigned long long span = hi - lo;
        int sh = 0;
        while (sh < 63 && (span >> sh) >= static_cast<unsigned long long>(NSUB)) sh++;
        __syncthreads();
        for (int j = tid; j < NSUB; j += NT) { sm[j] = 0.0; sc[j] = 0; }
        __syncthreads();
        for (int t = tid; t < ZCAP; t += NT) {
          if (zlive(t)) {
            const unsigned long long k = zk[t];
            if (k >= lo && k <= hi) {
              const int sb = static_cast<int>((k - lo) >> sh);
              atomicAdd(&sm[sb], exp_safe(zone_key_d(k), s_tab));
              atomicAdd(&sc[sb], 1);
            }
          }
        }
        __syncthreads();
        constexpr int PER = NSUB / NT;
        double inc[PER];
        double s = 0.0;
#pragma unroll
        for (int j = 0; j < PER; j++) { s += sm[tid * PER + j]; inc[j] = s; }
        double totm;
        const double exm = block_scan_excl_d(s, totm, ctl, tid);
        int first = NSUB;
#pragma unroll
        for (int j = 0; j < PER; j++) {
          if (first == NSUB && sc[tid * PER + j] > 0 && crossed(gbase + exm + inc[j])) first = tid * PER + j;
        }
        const int sbx = block_min_i(first, ctl, tid);
        if (sbx == NSUB) { all_in = true; break; }
        if (tid == sbx / PER) {
          const int j = sbx % PER;
          ctl.bcast_d[0] = gbase + exm + (j > 0 ? inc[j - 1] : 0.0);
          ctl.bcast_i[0] = sc[sbx];
        }
        __syncthreads();
        gbase = ctl.bcast_d[0];
        inrange = ctl.bcast_i[0];
        const unsigned long long nlo = lo + (static_cast<unsigned long long>(sbx) << sh);
        unsigned long long nhi = nlo + ((1ull << sh) - 1ull);
        if (nhi < nlo || nhi > hi) nhi = hi;
        lo = nlo; hi = nhi;
      }
      if (inrange > 32 && !all_in) bad = 1;
      double g_at = gbase;                                     // G(c*) and G just before c*
      double g_before = gbase;
      if (!bad && !all_in) {
        unsigned long long* few = reinterpret_cast<unsigned long long*>(regB);   // [32]
        __syncthreads();
        if (tid == 0) ctl.cand_count = 0;
        __syncthreads();
        for (int t = tid; t < ZCAP; t += NT) {
          if (zlive(t)) {
            const unsigned long long k = zk[t];
            if (k >= lo && k <= hi) { const int slot = atomicAdd(&ctl.cand_count, 1); if (slot < 32) few[slot] = k; }
          }
        }
        __syncthreads();
        const int nf = min(32, ctl.cand_count);
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
          unsigned long long cand = cr ? k : ~0ull;            // first crossed key = smallest crossed key
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long t = __shfl_xor_sync(FULL, cand, o);
            cand = t < cand ? t : cand;
          }
          const unsigned who = __ballot_sync(FULL, cr && k == cand);
          if (lane == 0) { ctl.red_u64[0] = cand; ctl.bcast_i[1] = who ? 1 : 0; }
          if (who && lane == __ffs(who) - 1) { ctl.bcast_d[1] = g; ctl.bcast_d[2] = g - e; }
        }
        __syncthreads();
        if (ctl.bcast_i[1]) {
          const unsigned long long cstar = ctl.red_u64[0];
          g_at = ctl.bcast_d[1];
          g_before = ctl.bcast_d[2];
          cut_key = cstar;
          cut_incl = (mode == 0) ? 0 : 1;
        } else {
          all_in = true;                                       // rounding: nothing in the last group crossed
        }
      }
      if (!bad && all_in) {
        cut_key = ~0ull; cut_incl = 1;
        g_at = g_before = Ktot + Ztot;
        if (mode == 1 && Dtot > 0.0) bad = 1;                  // the bracket promised a crossing
      }
      if (!bad && !all_in) {
        if (fabs(g_at / S - plim) <= 1e-12 || fabs(g_before / S - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
        if (mode == 1) {
          // a later key with the same d as c*: the cut separates equal probabilities
          int tie = 0;
          for (int t = tid; t < ZCAP; t += NT) {
            if (zlive(t)) { const unsigned long long k = zk[t]; tie |= (k > cut_key && (k >> 32) == (cut_key >> 32)) ? 1 : 0; }
          }
          if (block_max_i(tie, ctl, tid)) flags |= FLAG_TIE_CUT;
        }
      }
      // kept zone mass per owning rank
      __syncthreads();
      if (!bad) {
        for (int t = tid; t < ZCAP; t += NT) {
          if (zlive(t)) {
            const unsigned long long k = zk[t];
            if (k < cut_key || (cut_incl && k == cut_key)) {
              const int idx = zone_key_index(k, mode);
              atomicAdd(&s_zk[min(C - 1, rv.vec_of(idx) / SV)], exp_safe(zone_key_d(k), s_tab));
            }
          }
        }
      }
      __syncthreads();
    }
    double Zk = 0.0;
    for (int r = 0; r < C; r++) Zk += s_zk[r];
    const double Re = Ktot + Zk;
    dbg.resum = Re / S;
    int owner = -1;
    int code;                                                // see Xchg::verdict
    if (bad) {
      to_worklist();
      code = 2;
    } else if (poisoned || !(Re > 0.0)) {
      // NaN/Inf in the row, or mode A removed every token (generate.go:221-227): the walk falls through
      flags |= FLAG_NONFINITE | FLAG_FALLBACK;
      dbg.sum_exp = poisoned ? QNAN : S;
      if (!poisoned) dbg.resum = 0.0;
      finish(V - 1, flags, dbg);
      code = 1;
    } else {
      const double tgt = u * Re;
      double acc = 0.0, base = 0.0;
      for (int r = 0; r < C; r++) {
        const double nxt = acc + X.K[r] + s_zk[r];
        if (tgt < nxt) { owner = r; base = acc; break; }
        acc = nxt;
      }
      code = 0;
      if (owner < 0) {
        flags |= FLAG_FALLBACK;                              // generate.go:239
        dbg.edge_lo = dbg.edge_hi = acc / Re;
        if (u - acc / Re <= 1e-6) flags |= FLAG_BOUNDARY;
        finish(V - 1, flags, dbg);
        code = 3;
      }
      if (tid == 0) {
        for (int r = 0; r < C; r++) {
          Xchg* xr = cluster.map_shared_rank(&X, r);
          xr->local_target = tgt - base;
          xr->base_mass = base;
        }
      }
    }
    stamp(6);
    if (tid == 0) {
      for (int r = 0; r < C; r++) {
        Xchg* xr = cluster.map_shared_rank(&X, r);
        xr->owner = owner;
        xr->cut_key = cut_key; xr->cut_incl = cut_incl;
        xr->Re = Re; xr->S = S;
        xr->verdict = code;
      }
      if (code == 0) {                                       // the owner adds the id, the edges and the boundary flag
        if (A.out_flags) A.out_flags[row_id] = flags;
        if (A.out_debug) A.out_debug[row_id] = dbg;
      }
    }
  }
  cluster.sync();                                            // G5: last barrier

  const int verdict = X.verdict;
  if (verdict == 2) return;                                  // the work list owns this row now
  if (verdict == 1) { fill_probs_slice(QNAN); return; }
  const double Re = X.Re, S = X.S;
  const unsigned long long ckey = X.cut_key;
  const int cincl = X.cut_incl;
  // final rule for one element: its kept mass (0 when cut away)
  auto kept_mass = [&](float xv, int i) -> double {
    if (i < 0 || i >= V) return 0.0;
    const float s = t_is_one ? xv : __fdiv_rn(xv, Tm);
    const float d = s - m;
    if (d < dA) {
      if (!(d >= dB)) return 0.0;
      const unsigned long long k = zone_key(d, i, mode);
      if (!(k < ckey || (cincl && k == ckey))) return 0.0;
    }
    return exp_safe(d, s_tab);
  };

  if (A.out_probs || A.out_debug) {                          // parity runs only
    double* pr = A.out_probs ? A.out_probs + row_id * static_cast<int64_t>(V) : nullptr;
    const double rq = Re / S;
    int kept_loc = 0;
    for (int j = tid; j < nv; j += NT) {
      float x[VEC];
      Elem<T>::unpack(slice[j], x);
      const int i0 = (v0 + j) * VEC - rv.shift;
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
    const int kept_cta = block_sum_i(kept_loc, ctl, tid);
    if (A.out_debug && tid == 0) atomicAdd(&A.out_debug[row_id].kept, kept_cta);
  }
  if (verdict == 3 || rank != X.owner) return;

  // ---- owner: kept mass per warp run = certain mass + kept zone entries, then one run is rescanned
  __syncthreads();
  if (cut_on) {
    if (rank == 0) {
      // rank 0's region B was reused by the selection: it filters the staged list instead
      const unsigned long long* zk = reinterpret_cast<const unsigned long long*>(regA);
      for (int t = tid; t < ZCAP; t += NT) {
        if ((t & (zcap_r - 1)) < X.cnt[t >> zlog]) {
          const unsigned long long k = zk[t];
          const int jj = rv.vec_of(zone_key_index(k, mode)) - v0;
          if ((k < ckey || (cincl && k == ckey)) && jj >= 0 && jj < nv) {
            atomicAdd(&s_kseg[min(NW - 1, jj / max(wv, 1))], exp_safe(zone_key_d(k), s_tab));
          }
        }
      }
    } else {
      for (int j = tid; j < nz_loc; j += NT) {
        const uint2 e = lz[j];
        const float d = __uint_as_float(e.x);
        const int i = static_cast<int>(e.y);
        const unsigned long long k = zone_key(d, i, mode);
        if (k < ckey || (cincl && k == ckey)) {
          atomicAdd(&s_kseg[min(NW - 1, (rv.vec_of(i) - v0) / max(wv, 1))], exp_safe(d, s_tab));
        }
      }
    }
  }
  __syncthreads();
  const double ltgt = X.local_target;
  const double base_mass = X.base_mass;
  int wsel = NW - 1;
  double wbase = 0.0;
  {
    double acc = 0.0;
    bool found = false;
    for (int w = 0; w < NW; w++) {
      const double nxt = acc + s_kseg[w];
      if (!found && ltgt < nxt) { wsel = w; wbase = acc; found = true; }
      acc = nxt;
    }
    if (!found) wbase = acc - s_kseg[NW - 1];
  }
  int id = -1;
  int last_kept = -1;
  double edge_lo = 0.0, edge_hi = 0.0, run_end = wbase;
  for (int w = wsel; w < NW && id < 0; w++) {               // uniform; normally one trip
    const int a0 = min(nv, w * wv), a1 = min(nv, a0 + wv);
    for (int jb = a0; jb < a1 && id < 0; jb += NT) {
      const int j = jb + tid;
      double em[VEC];
      double tsum = 0.0;
#pragma unroll
      for (int c = 0; c < VEC; c++) em[c] = 0.0;
      int i0 = 0;
      if (j < a1) {
        float x[VEC];
        Elem<T>::unpack(slice[j], x);
        i0 = (v0 + j) * VEC - rv.shift;
#pragma unroll
        for (int c = 0; c < VEC; c++) { em[c] = kept_mass(x[c], i0 + c); tsum += em[c]; }
      }
      double totc;
      const double ex = block_scan_excl_d(tsum, totc, ctl, tid);
      int pick_loc = 0x7fffffff;
      int lk = -1;
      double run = run_end + ex, lo = 0.0, hi = 0.0;
#pragma unroll
      for (int c = 0; c < VEC; c++) {
        const double before = run;
        run += em[c];
        if (em[c] > 0.0) {
          lk = i0 + c;
          if (ltgt < run && pick_loc == 0x7fffffff) { pick_loc = i0 + c; lo = before; hi = run; }
        }
      }
      const int pick = block_min_i(pick_loc, ctl, tid);
      last_kept = max(last_kept, block_max_i(lk, ctl, tid));
      if (pick != 0x7fffffff) {
        if (pick_loc == pick) { ctl.bcast_d[1] = lo; ctl.bcast_d[2] = hi; }
        __syncthreads();
        id = pick;
        edge_lo = (base_mass + ctl.bcast_d[1]) / Re;
        edge_hi = (base_mass + ctl.bcast_d[2]) / Re;
      }
      run_end += totc;
    }
  }
  uint32_t oflags = 0;
  if (id < 0) {
    // rounding pushed the crossing past this slice's end: take its last kept token
    id = last_kept >= 0 ? last_kept : V - 1;
    oflags |= FLAG_BOUNDARY;
    edge_lo = edge_hi = (base_mass + run_end) / Re;
  } else if ((edge_lo > 0.0 && u - edge_lo <= 1e-6) || edge_hi - u <= 1e-6) {
    oflags |= FLAG_BOUNDARY;
  }
  if (tid == 0) {
    A.out_ids[row_id] = id;
    if (A.out_flags && oflags) atomicOr(&A.out_flags[row_id], oflags);
    if (A.out_debug) { A.out_debug[row_id].edge_lo = edge_lo; A.out_debug[row_id].edge_hi = edge_hi; }
  }
}

}  // namespace gs
