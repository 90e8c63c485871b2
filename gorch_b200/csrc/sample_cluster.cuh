// Cluster kernel: one thread-block cluster (1, 2, 4 or 8 CTAs) per logits row.
//
// Each CTA owns a contiguous slice of the row's 16-byte vectors. Rows that
// need more than one pass (top-k off: softmax over the whole vocabulary, with
// or without a top-p cut) keep their slice in shared memory, so HBM is read
// once; the cross-CTA reductions go through distributed shared memory
// (peers store into the consumer's shared memory, then a cluster barrier).
// Nothing in this file loads with multicast.
//
// Row semantics: model/generate.go:134-260 (mode A), model/qwen/generate.go:
// 77-181 (mode B). Per row:
//   greedy            slice argmax -> rank 0 picks (max value, lowest index).
//   top-k (small k)   every CTA streams its slice once with an adaptive
//                     threshold, prunes to its local top-k (+ties), pushes the
//                     survivors to rank 0, which finishes in shared memory.
//   full row          L: slice -> smem + max.  P2 (only with an active top-p
//                     cut): count histogram over 1024 linear buckets of
//                     d = s - max; rank 0 brackets the cut from count-based
//                     mass bounds.  P3: f64 exponentials; elements certainly
//                     kept / dropped go to running sums, the bracketed zone to
//                     an exact list that rank 0 sorts and cuts.  The CTA whose
//                     slice holds the drawn token rescans one warp segment.
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
constexpr int ZCAP = 2048;           // exact zone list capacity (entries of 8 B)
constexpr int UCAP = 2048;           // merged top-k candidate capacity on rank 0
constexpr int LCAP = 6144;           // local streaming candidate capacity
constexpr int LKEEP = 1536;          // a local prune must get below this
constexpr int REGION_A = 16384;      // bytes: zone keys / merged candidates
constexpr int REGION_B = 16384;      // bytes: local zone list / histogram staging tail
constexpr int MIN_SLICE_BYTES = 65536;

struct ClusterArgs {
  KernelArgs k;
  int32_t slice_bytes;   // shared bytes reserved for the slice region (>= MIN_SLICE_BYTES)
  int32_t resident_ok;   // slice of a full row fits in slice_bytes
};

// Written by peers through distributed shared memory.
struct Xchg {
  unsigned long long u64[CL_MAX];
  double K[CL_MAX], D[CL_MAX], Z[CL_MAX];
  int cnt[CL_MAX];
  int giveup[CL_MAX];
  int cand_total;
  int overflow;
  // verdicts pushed by rank 0
  int verdict;           // top-k: 0 proceed on rank 0, 1 everybody takes the full-row path
  float dA, dB;          // zone thresholds on d
  int deep;              // some element lies below the last bucket edge / cut inactive
  int zone_total;
  int owner;             // rank that resolves the draw, -1: rank 0 already wrote the id
  int cut_idx;           // index of the last kept zone entry
  uint32_t cut_dkey;     // its key; 0xffffffff: no zone entry kept... see keep_zone()
  int cut_any;           // 0: no zone entry kept
  double local_target;   // u*Re minus the kept mass of lower ranks
  double base_mass;      // kept mass of lower ranks
  double Re, S;
  uint32_t sel_prefix;   // exact top-k select: digit broadcast
  int sel_need;
  float flt_lo;
};

__device__ __forceinline__ uint32_t dkey_of(float d) {   // d <= 0 (or NaN): ascending = falling probability
  return __float_as_uint(-d) & 0x7fffffffu | (d != d ? 0x7fffffffu : 0u);
}

// 1024 buckets of width 1/32: round(-32 d) clamped to 1023 (everything at or
// below -31.97 shares the last bucket). Non-decreasing as d falls.
__device__ __forceinline__ int bucket1(float d) {
  float f = fmaf(fmaxf(d, -31.97f), -32.0f, 8388608.0f);
  return __float_as_int(f) & 0x7ff;
}

// Smallest d (as a float, d <= 0) whose bucket is <= bmax; -Inf when bmax is the last bucket.
__device__ float bucket_floor(int bmax) {
  if (bmax >= NB1 - 1) return -INFINITY;
  if (bmax < 0) return INFINITY;
  uint32_t lo = 0x007fffffu, hi = 0x80000000u;   // keys of -Inf and +0; pred(hi) holds
  while (lo < hi) {
    uint32_t mid = lo + ((hi - lo) >> 1);
    if (bucket1(okey_to_float(mid)) <= bmax) hi = mid; else lo = mid + 1;
  }
  return okey_to_float(hi);
}

template <bool CHECK>
__device__ __forceinline__ double exp_neg(float d, const double* __restrict__ tab) {
  if (CHECK) {
    if (!(d >= -700.0f)) return exp(static_cast<double>(d));
  }
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

// Ascending in-place bitonic sort of keys[0..n2), n2 a power of two.
__device__ void block_bitonic_u64(unsigned long long* keys, int n2, int tid) {
  for (int k = 2; k <= n2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      __syncthreads();
      for (int i = tid; i < (n2 >> 1); i += NT) {
        int a = ((i & ~(j - 1)) << 1) | (i & (j - 1));
        int b = a | j;
        bool up = ((a & k) == 0);
        unsigned long long x = keys[a], y = keys[b];
        if ((x > y) == up) { keys[a] = y; keys[b] = x; }
      }
    }
  }
  __syncthreads();
}
__device__ __forceinline__ int pow2_at_least(int n) {
  int p = 2;
  while (p < n) p <<= 1;
  return p;
}

template <typename T> struct Neutral;
template <> struct Neutral<float> { static constexpr uint32_t word = 0xff800000u; };      // -Inf
template <> struct Neutral<uint16_t> { static constexpr uint32_t word = 0xff80ff80u; };   // two bf16 -Inf

// Load vector v of the row; lanes outside [0, V) become -Inf.
template <typename T>
__device__ __forceinline__ uint4 load_masked(const RowView<T>& rv, int v) {
  constexpr int VEC = Elem<T>::VEC;
  uint4 raw = __ldg(rv.vbase + v);
  if (v == 0 || v == rv.nvec - 1) {
    uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    int i0 = v * VEC - rv.shift;
    if (sizeof(T) == 4) {
#pragma unroll
      for (int c = 0; c < 4; c++) {
        int i = i0 + c;
        if (i < 0 || i >= rv.V) w[c] = 0xff800000u;
      }
    } else {
#pragma unroll
      for (int c = 0; c < 8; c++) {
        int i = i0 + c;
        if (i < 0 || i >= rv.V) {
          if (c & 1) w[c >> 1] = (w[c >> 1] & 0x0000ffffu) | 0xff800000u;
          else w[c >> 1] = (w[c >> 1] & 0xffff0000u) | 0x0000ff80u;
        }
      }
    }
    raw = make_uint4(w[0], w[1], w[2], w[3]);
  }
  return raw;
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

  unsigned char* slice_b = dyn;
  uint4* slice = reinterpret_cast<uint4*>(dyn);
  unsigned char* regA = dyn + CA.slice_bytes;
  unsigned char* regB = regA + REGION_A;

  RowCfg cfg;
  if (A.force_greedy) { cfg.temperature = 0.f; cfg.top_k = 0; cfg.top_p = 0.f; cfg.topp_mode = 0; }
  else cfg = A.cfgs[row_id];
  const float Tm = cfg.temperature;

  if (tid < 256) s_tab[tid] = A.exp_table[tid];
  if (tid == 0) {
    ctl.cand_count = 0; ctl.overflow = 0; ctl.thr = -INFINITY; ctl.flags = 0;
    X.cand_total = 0; X.overflow = 0; X.verdict = 0; X.zone_total = 0; X.owner = -1;
  }
  if (tid < CL_MAX) { X.giveup[tid] = 0; X.cnt[tid] = 0; X.u64[tid] = 0; X.K[tid] = 0; X.D[tid] = 0; X.Z[tid] = 0; s_zk[tid] = 0; }
  // peers may store into X after this barrier only
  cluster.sync();

  Xchg* X0 = cluster.map_shared_rank(&X, 0);
  auto finish = [&](int id, uint32_t flags, const RowDebug& dbg) {
    if (tid == 0) {
      if (id != -2) A.out_ids[row_id] = id;
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
  const double QNAN = __longlong_as_double(0x7ff8000000000000ll);

  RowDebug dbg;
  dbg.sum_exp = 0; dbg.resum = 1.0; dbg.edge_lo = 0; dbg.edge_hi = 0; dbg.kept = 0;
  dbg.max_scaled = 0; dbg.threshold = __int_as_float(0x7fc00000); dbg.path = 0;

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
    if (tid == 0) X0->u64[rank] = best;
    fill_probs_slice(0.0);
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
  bool general = !(topk > 0 && topk * C <= LKEEP);
  float xmax = -INFINITY;
  bool nan_seen = false;

  // ======================================================= top-k, small k
  if (!general) {
    uint2* lc = reinterpret_cast<uint2*>(slice_b);          // local candidates, LCAP entries
    const int tile_elems = NT * VEC;
    float thr = -INFINITY;
    bool giveup = false;
    auto prune = [&](int cnt) -> int {                      // block-wide; returns the new count
      if (cnt <= topk) return cnt;
      uint32_t kkey = block_select_kth(lc, cnt, topk, s_sel, ctl, tid);
      if (tid == 0) ctl.thr = quotient_class_floor(okey_to_float(kkey), Tm);
      __syncthreads();
      thr = ctl.thr;
      constexpr int PER = LCAP / NT;
      uint2 mine[PER];
#pragma unroll
      for (int j = 0; j < PER; j++) {
        int e = tid + j * NT;
        mine[j] = (e < cnt) ? lc[e] : make_uint2(0xffc00000u, 0u);
      }
      __syncthreads();
      if (tid == 0) ctl.cand_count = 0;
      __syncthreads();
#pragma unroll
      for (int j = 0; j < PER; j++) {
        if (__uint_as_float(mine[j].x) >= thr) lc[atomicAdd(&ctl.cand_count, 1)] = mine[j];
      }
      __syncthreads();
      return ctl.cand_count;
    };
    uint4 raw_next = make_uint4(Neutral<T>::word, Neutral<T>::word, Neutral<T>::word, Neutral<T>::word);
    if (v0 + tid < v1) raw_next = load_masked(rv, v0 + tid);
    // The decision to prune is taken from the atomic counter's return values: the
    // thread that made the last append of a tile knows the exact count, and the
    // barrier that ends the tile ORs the verdicts, so every thread sees the same.
    int do_prune = 0;
    for (int base = v0; base < v1; base += NT) {            // uniform loop
      uint4 raw = raw_next;
      const int v = base + tid;
      raw_next = make_uint4(Neutral<T>::word, Neutral<T>::word, Neutral<T>::word, Neutral<T>::word);
      if (v + NT < v1) raw_next = load_masked(rv, v + NT);
      if (do_prune) {
        int cnt = prune(ctl.cand_count);
        if (cnt > LKEEP) { giveup = true; break; }          // ties at the threshold fill the buffer
      }
      float x[VEC];
      Elem<T>::unpack(raw, x);
      bool any = false;
#pragma unroll
      for (int c = 0; c < VEC; c++) {
        xmax = fmaxf(xmax, x[c]);
        nan_seen |= (x[c] != x[c]);
        any |= (x[c] >= thr);
      }
      bool want = false;
      if (any && v < v1) {
        const int i0 = v * VEC - rv.shift;
#pragma unroll
        for (int c = 0; c < VEC; c++) {
          int i = i0 + c;
          if (x[c] >= thr && i >= 0 && i < V) {
            int slot = atomicAdd(&ctl.cand_count, 1);
            lc[slot] = make_uint2(__float_as_uint(x[c]), static_cast<uint32_t>(i));
            want |= (slot + 1 + tile_elems > LCAP);
          }
        }
      }
      do_prune = __syncthreads_or(want ? 1 : 0);
    }
    int n_loc = 0;
    if (!giveup) {
      n_loc = prune(ctl.cand_count);
      if (n_loc > LKEEP) giveup = true;
    }
    // push survivors, max and NaN flag to rank 0
    __syncthreads();
    if (tid == 0) {
      int base = giveup ? 0 : atomicAdd(&X0->cand_total, n_loc);
      ctl.bcast_i[3] = base;
      if (giveup) X0->giveup[rank] = 1;
      else if (base + n_loc > UCAP) X0->overflow = 1;
    }
    {
      int anynan = block_max_i(nan_seen ? 1 : 0, ctl, tid);
      unsigned long long p = block_max_u64(static_cast<unsigned long long>(okey(xmax)) << 32, ctl, tid);
      if (tid == 0) X0->u64[rank] = p | static_cast<unsigned long long>(anynan);
    }
    __syncthreads();
    {
      int base = ctl.bcast_i[3];
      if (!giveup && base + n_loc <= UCAP) {
        uint2* dst = cluster.map_shared_rank(reinterpret_cast<uint2*>(regA), 0);
        for (int j = tid; j < n_loc; j += NT) dst[base + j] = lc[j];
      }
    }
    cluster.sync();                                          // B1
    if (rank == 0 && tid == 0) {
      int bad = X.overflow;
      for (int r = 0; r < C; r++) bad |= X.giveup[r];
      for (int r = 0; r < C; r++) cluster.map_shared_rank(&X, r)->verdict = bad;
    }
    cluster.sync();                                          // B2
    general = X.verdict != 0;
    if (!general) {
      if (rank != 0) return;
      // ---------------- rank 0: finish in shared memory
      dbg.path = 1;
      unsigned long long mx = 0;
      int anynan = 0;
      for (int r = 0; r < C; r++) { mx = X.u64[r] > mx ? X.u64[r] : mx; anynan |= static_cast<int>(X.u64[r] & 1ull); }
      xmax = okey_to_float(static_cast<uint32_t>(mx >> 32));
      const float m = scale_t(xmax, Tm);
      dbg.max_scaled = m;
      auto poison_exit = [&](bool nan_sum) {
        if (A.out_probs) {
          double* pr = A.out_probs + row_id * static_cast<int64_t>(V);
          for (int i = tid; i < V; i += NT) pr[i] = QNAN;
        }
        if (nan_sum) dbg.sum_exp = QNAN;
        finish(V - 1, flags | FLAG_NONFINITE | FLAG_FALLBACK, dbg);
      };
      if (anynan || !(fabsf(m) < INFINITY)) {
        poison_exit(true);
        return;
      }
      uint2* uc = reinterpret_cast<uint2*>(regA);           // merged candidates (regA+regB)
      int n = X.cand_total;
      // global threshold: k-th largest of the union, then its quotient-class floor
      float keep_lo = -INFINITY;
      if (n > topk) {
        uint32_t kkey = block_select_kth(uc, n, topk, s_sel, ctl, tid);
        if (tid == 0) ctl.thr = quotient_class_floor(okey_to_float(kkey), Tm);
        __syncthreads();
        keep_lo = ctl.thr;
      }
      // kept set sorted by index: keys (idx << 32 | xbits), padded with ~0
      unsigned long long* keys = reinterpret_cast<unsigned long long*>(slice_b);        // 16 KB
      double* se = reinterpret_cast<double*>(slice_b + 16384);                          // 16 KB
      double* sf = reinterpret_cast<double*>(slice_b + 32768);                          // 16 KB
      unsigned long long* ok = reinterpret_cast<unsigned long long*>(slice_b + 49152);  // 16 KB
      __syncthreads();
      if (tid == 0) ctl.cand_count = 0;
      __syncthreads();
      for (int j = tid; j < n; j += NT) {
        uint2 e = uc[j];
        if (__uint_as_float(e.x) >= keep_lo) {
          int slot = atomicAdd(&ctl.cand_count, 1);
          keys[slot] = (static_cast<unsigned long long>(e.y) << 32) | e.x;
        }
      }
      __syncthreads();
      const int nk = ctl.cand_count;
      const int n2 = pow2_at_least(nk);
      for (int j = nk + tid; j < n2; j += NT) keys[j] = ~0ull;
      block_bitonic_u64(keys, n2, tid);
      // softmax over the kept set (generate.go:167-181)
      float thr_s = INFINITY;
      for (int j = tid; j < nk; j += NT) {
        float s = scale_t(__uint_as_float(static_cast<uint32_t>(keys[j])), Tm);
        thr_s = fminf(thr_s, s);
        float d = s - m;
        double e = exp(static_cast<double>(d));
        se[j] = e;
        sf[j] = e;
        // order key for top-p: falling probability = rising dkey; ties by position (= index order)
        uint32_t dk = dkey_of(d);
        ok[j] = (static_cast<unsigned long long>(mode == 0 ? ~dk : dk) << 32) | static_cast<uint32_t>(j);
      }
      {
        unsigned long long pk = block_max_u64(~static_cast<unsigned long long>(okey(thr_s)), ctl, tid);
        dbg.threshold = okey_to_float(static_cast<uint32_t>(~pk));
      }
      __syncthreads();
      smem_scan_incl<4>(sf, nk, ctl, tid);
      const double S = sf[nk - 1];
      dbg.sum_exp = S;
      __syncthreads();
      for (int j = tid; j < nk; j += NT) se[j] = se[j] / S;        // q
      __syncthreads();
      bool all_removed = false;
      if (topp_on) {
        for (int j = nk + tid; j < n2; j += NT) ok[j] = ~0ull;
        block_bitonic_u64(ok, n2, tid);
        // sf[r] = q in sorted order, inclusive scan
        for (int r = tid; r < nk; r += NT) sf[r] = se[static_cast<uint32_t>(ok[r])];
        __syncthreads();
        if (mode == 0) {
          // removal order is ascending probability (generate.go:206-219): sorted order r = 0 is removed first.
          // remaining(r) = total - prefix(r-1); computed as a suffix sum for accuracy: reverse, scan.
          for (int r = tid; r < nk / 2; r += NT) { double a = sf[r]; sf[r] = sf[nk - 1 - r]; sf[nk - 1 - r] = a; }
          __syncthreads();
          smem_scan_incl<4>(sf, nk, ctl, tid);                     // sf[t] = mass of the t+1 largest
          // remaining after removing r smallest = sf[nk-1-r]
          int rstar_loc = nk;
          for (int r = tid; r < nk; r += NT) if (sf[nk - 1 - r] <= plim) rstar_loc = min(rstar_loc, r);
          int rstar = block_min_i(rstar_loc, ctl, tid);
          double resum = 0.0;
          if (rstar == nk) {
            all_removed = true;
          } else {
            resum = sf[nk - 1 - rstar];
            if (fabs(resum - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
            if (rstar > 0 && fabs(sf[nk - rstar] - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
          }
          dbg.resum = resum;
          __syncthreads();
          // final probabilities back in index order
          for (int r = tid; r < nk; r += NT) {
            int j = static_cast<int>(static_cast<uint32_t>(ok[r]));
            double q = se[j];
            sf[j] = all_removed ? QNAN : ((r < rstar) ? 0.0 : q / resum);
          }
        } else {
          smem_scan_incl<4>(sf, nk, ctl, tid);
          int cut_loc = nk;
          for (int r = tid; r < nk; r += NT) if (sf[r] >= plim) cut_loc = min(cut_loc, r + 1);
          int cutn = block_min_i(cut_loc, ctl, tid);
          double resum = sf[cutn - 1];
          if (fabs(resum - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
          if (cutn >= 2 && fabs(sf[cutn - 2] - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
          if (cutn < nk && (ok[cutn] >> 32) == (ok[cutn - 1] >> 32)) flags |= FLAG_TIE_CUT;
          dbg.resum = resum;
          __syncthreads();
          for (int r = tid; r < nk; r += NT) {
            int j = static_cast<int>(static_cast<uint32_t>(ok[r]));
            sf[j] = (r < cutn) ? se[j] / resum : 0.0;
          }
        }
      } else {
        for (int j = tid; j < nk; j += NT) sf[j] = se[j];
      }
      __syncthreads();
      if (all_removed) { dbg.resum = 0.0; poison_exit(false); return; }
      int kept_loc = 0;
      for (int j = tid; j < nk; j += NT) kept_loc += (sf[j] > 0) ? 1 : 0;
      dbg.kept = block_sum_i(kept_loc, ctl, tid);
      if (A.out_probs) {
        double* pr = A.out_probs + row_id * static_cast<int64_t>(V);
        for (int i = tid; i < V; i += NT) pr[i] = 0.0;
        __syncthreads();
        for (int j = tid; j < nk; j += NT) pr[static_cast<uint32_t>(keys[j] >> 32)] = sf[j];
      }
      for (int j = tid; j < nk; j += NT) se[j] = sf[j];
      __syncthreads();
      smem_scan_incl<4>(se, nk, ctl, tid);
      int pick_loc = nk;
      for (int j = tid; j < nk; j += NT) if (u < se[j]) pick_loc = min(pick_loc, j);
      int pick = block_min_i(pick_loc, ctl, tid);
      int id;
      if (pick < nk) {
        id = static_cast<int>(static_cast<uint32_t>(keys[pick] >> 32));
        double hi = se[pick], lo = pick > 0 ? se[pick - 1] : 0.0;
        dbg.edge_lo = lo; dbg.edge_hi = hi;
        if ((pick > 0 && u - lo <= 1e-6) || hi - u <= 1e-6) flags |= FLAG_BOUNDARY;
      } else {
        id = V - 1;
        flags |= FLAG_FALLBACK;
        dbg.edge_lo = dbg.edge_hi = se[nk - 1];
        if (u - se[nk - 1] <= 1e-6) flags |= FLAG_BOUNDARY;
      }
      finish(id, flags, dbg);
      return;
    }
    // verdict: fall through to the full-row path (all CTAs)
    xmax = -INFINITY;
    nan_seen = false;
    __syncthreads();
    if (tid == 0) { ctl.cand_count = 0; X.cand_total = 0; X.overflow = 0; }
    __syncthreads();
  }

  // ============================================================ full-row path
  dbg.path = 2;
  flags |= FLAG_GENERAL_PATH;
  const bool resident = CA.resident_ok != 0;
  const bool filt = topk > 0;

  // ---- L: slice -> shared memory, local max (NaN check only when a filter could hide it)
  for (int v = v0 + tid; v < v1; v += NT) {
    uint4 raw = load_masked(rv, v);
    if (resident) slice[v - v0] = raw;
    float x[VEC];
    Elem<T>::unpack(raw, x);
#pragma unroll
    for (int c = 0; c < VEC; c++) {
      xmax = fmaxf(xmax, x[c]);
      if (filt) nan_seen |= (x[c] != x[c]);
    }
  }
  {
    int anynan = block_max_i(nan_seen ? 1 : 0, ctl, tid);
    unsigned long long p = block_max_u64(static_cast<unsigned long long>(okey(xmax)) << 32, ctl, tid);
    if (tid == 0) {
      p |= static_cast<unsigned long long>(anynan);
      for (int r = 0; r < C; r++) cluster.map_shared_rank(&X, r)->u64[rank] = p;
    }
  }
  cluster.sync();                                            // G1
  int anynan = 0;
  {
    unsigned long long mx = 0;
    for (int r = 0; r < C; r++) { mx = X.u64[r] > mx ? X.u64[r] : mx; anynan |= static_cast<int>(X.u64[r] & 1ull); }
    xmax = okey_to_float(static_cast<uint32_t>(mx >> 32));
  }
  const float m = scale_t(xmax, Tm);
  dbg.max_scaled = m;
  const bool poisoned_early = anynan || !(fabsf(m) < INFINITY);
  // (poisoned rows still walk the barriers below; they are resolved by rank 0 at the end)

  // element access for the later passes: vector j of this slice
  auto slice_vec = [&](int j) -> uint4 {
    return resident ? slice[j] : load_masked(rv, v0 + j);
  };

  // ---- exact top-k threshold by distributed counting (only when the streaming path gave up)
  float flt_lo = -INFINITY;
  if (filt) {
    uint32_t* hist = reinterpret_cast<uint32_t*>(regB);      // 256 bins
    uint32_t prefix = 0, mask = 0;
    int need = topk;
    for (int round = 0; round < 4; round++) {
      const int sh = 24 - 8 * round;
      __syncthreads();
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      for (int j = tid; j < nv; j += NT) {
        float x[VEC];
        Elem<T>::unpack(slice_vec(j), x);
        const int i0 = (v0 + j) * VEC - rv.shift;
#pragma unroll
        for (int c = 0; c < VEC; c++) {
          uint32_t key = okey(x[c]);
          int i = i0 + c;
          if ((key & mask) == prefix && i >= 0 && i < V) atomicAdd(&hist[(key >> sh) & 255u], 1u);
        }
      }
      __syncthreads();
      {
        uint32_t* dst = cluster.map_shared_rank(reinterpret_cast<uint32_t*>(regA), 0);   // [C][256]
        if (tid < 256) dst[rank * 256 + tid] = hist[tid];
      }
      cluster.sync();
      if (rank == 0) {
        uint32_t* all = reinterpret_cast<uint32_t*>(regA);
        if (tid < 256) {
          uint32_t s = 0;
          for (int r = 0; r < C; r++) s += all[r * 256 + tid];
          hist[tid] = s;
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
            int t = __shfl_down_sync(FULL, run, o);
            if (tid + o < 32) run += t;
          }
          int above = run - s;
          if (above < need && above + s >= need) {
#pragma unroll
            for (int j = 7; j >= 0; j--) {
              if (above + loc[j] >= need) {
                int digit = tid * 8 + j;
                int nn = need - (above + loc[j] - static_cast<int>(hist[tid * 8 + j]));
                for (int r = 0; r < C; r++) {
                  Xchg* xr = cluster.map_shared_rank(&X, r);
                  xr->sel_prefix = prefix | (static_cast<uint32_t>(digit) << sh);
                  xr->sel_need = nn;
                }
                break;
              }
            }
          }
        }
      }
      cluster.sync();
      prefix = X.sel_prefix;
      mask |= 255u << sh;
      need = X.sel_need;
    }
    flt_lo = quotient_class_floor(okey_to_float(prefix), Tm);
    dbg.threshold = scale_t(okey_to_float(prefix), Tm);
  }

  // ---- P2: count histogram + bracket of the top-p cut
  float dA = -INFINITY, dB = -INFINITY;    // def-kept: d >= dA; zone: dB <= d < dA; dropped: d < dB
  bool deep = true;
  if (cut_on) {
    uint32_t* hist = (rank == 0) ? reinterpret_cast<uint32_t*>(regA) : reinterpret_cast<uint32_t*>(regB);
    __syncthreads();
    for (int j = tid; j < NB1; j += NT) hist[j] = 0;
    __syncthreads();
    for (int j = tid; j < nv; j += NT) {
      float x[VEC];
      Elem<T>::unpack(slice_vec(j), x);
#pragma unroll
      for (int c = 0; c < VEC; c++) {
        if (!filt || x[c] >= flt_lo) {
          float s = t_is_one ? x[c] : __fdiv_rn(x[c], Tm);
          atomicAdd(&hist[bucket1(s - m)], 1u);
        }
      }
    }
    __syncthreads();
    if (rank != 0) {
      // rank 0 stages [C][1024] counters across its regions A and B (32 KB at C = 8)
      uint32_t* dst = cluster.map_shared_rank(reinterpret_cast<uint32_t*>(regA), 0) + rank * NB1;
      for (int j = tid; j < NB1; j += NT) dst[j] = hist[j];
    }
    cluster.sync();                                          // G2
    if (rank == 0) {
      uint32_t* all = reinterpret_cast<uint32_t*>(regA);
      constexpr int PER = NB1 / NT;                          // 2 buckets per thread
      double lo_inc[PER], hi_inc[PER];
      int cb[PER];
      double slo = 0.0, shi = 0.0;
#pragma unroll
      for (int j = 0; j < PER; j++) {
        int b = tid * PER + j;
        uint32_t cnt = 0;
        for (int r = 0; r < C; r++) cnt += all[r * NB1 + b];
        cb[j] = static_cast<int>(cnt);
        double c = static_cast<double>(cnt);
        // bucket b holds d in [-(b+.5)/32, -(b-.5)/32]; the last one everything below
        double elo = (b == NB1 - 1) ? 0.0 : exp(-(b + 0.5) / 32.0) * (1.0 - 1e-7);
        double ehi = fmin(1.0, exp(-(b - 0.5) / 32.0) * (1.0 + 1e-7));
        slo += c * elo; shi += c * ehi;
        lo_inc[j] = slo; hi_inc[j] = shi;
      }
      double tot_lo, tot_hi;
      double ex_lo = block_scan_excl_d(slo, tot_lo, ctl, tid);
      double ex_hi = block_scan_excl_d(shi, tot_hi, ctl, tid);
      int b1_loc = NB1 - 1, b2_loc = NB1 - 1;
#pragma unroll
      for (int j = 0; j < PER; j++) {
        int b = tid * PER + j;
        double a_lo = ex_lo + lo_inc[j], a_hi = ex_hi + hi_inc[j];
        double r_hi = a_hi / (a_hi + (tot_lo - a_lo));
        double r_lo = a_lo / (a_lo + (tot_hi - a_hi));
        bool c1, c2;
        if (mode == 0) { c1 = r_hi > plim * (1.0 - 1e-9); c2 = r_lo > plim * (1.0 + 1e-9); }
        else           { c1 = r_hi >= plim * (1.0 - 1e-9); c2 = r_lo >= plim * (1.0 + 1e-9); }
        if (c1) b1_loc = min(b1_loc, b);
        if (c2) b2_loc = min(b2_loc, b);
      }
      int b1 = block_min_i(b1_loc, ctl, tid);
      int b2 = block_min_i(b2_loc, ctl, tid);
      if (b2 < b1) b2 = b1;
      int nz_loc = 0;
#pragma unroll
      for (int j = 0; j < PER; j++) {
        int b = tid * PER + j;
        if (b >= b1 && b <= b2) nz_loc += cb[j];
      }
      int nz = block_sum_i(nz_loc, ctl, tid);
      int last = 0;
      if (tid == NT - 1) last = cb[PER - 1];
      last = block_max_i(last, ctl, tid);
      if (tid == 0) { ctl.bcast_d[0] = 0; }
      float tA = 0.f, tB = 0.f;
      if (tid == 0) tA = bucket_floor(b1 - 1);
      if (tid == 32) tB = bucket_floor(b2);
      if (tid == 0) *reinterpret_cast<float*>(&ctl.bcast_i[4]) = tA;
      if (tid == 32) *reinterpret_cast<float*>(&ctl.bcast_i[5]) = tB;
      __syncthreads();
      if (tid == 0) {
        for (int r = 0; r < C; r++) {
          Xchg* xr = cluster.map_shared_rank(&X, r);
          xr->dA = *reinterpret_cast<float*>(&ctl.bcast_i[4]);
          xr->dB = *reinterpret_cast<float*>(&ctl.bcast_i[5]);
          xr->deep = (last > 0) ? 1 : 0;
          xr->zone_total = nz;
        }
      }
    }
    cluster.sync();                                          // G3
    dA = X.dA; dB = X.dB; deep = X.deep != 0;
  }
  const int nzone = cut_on ? X.zone_total : 0;
  const bool zone_ok = nzone <= ZCAP;

  // ---- P3: exponentials. Each warp owns a contiguous run of the slice.
  uint2* lz = reinterpret_cast<uint2*>(regB);               // local zone list (dbits, idx)
  __syncthreads();
  if (tid == 0) ctl.cand_count = 0;
  __syncthreads();
  const int wv = (nv + NW - 1) / NW;                        // vectors per warp segment
  const int w0 = min(nv, warp * wv), w1 = min(nv, w0 + wv);
  double tot = 0.0, dsum = 0.0, zsum = 0.0;
  if (zone_ok) {
    auto body = [&](auto check_tag, auto tone_tag) {
      constexpr bool CHK = decltype(check_tag)::value;
      constexpr bool TONE = decltype(tone_tag)::value;
      for (int j = w0 + lane; j < w1; j += 32) {
        float x[VEC];
        Elem<T>::unpack(slice_vec(j), x);
#pragma unroll
        for (int c = 0; c < VEC; c++) {
          if (filt && !(x[c] >= flt_lo)) continue;
          float s = TONE ? x[c] : __fdiv_rn(x[c], Tm);
          float d = s - m;
          double e = exp_neg<CHK>(d, s_tab);
          tot += e;
          if (d < dA) {
            if (d >= dB) {
              int i = (v0 + j) * VEC - rv.shift + c;
              if (i >= 0 && i < V) {
                int slot = atomicAdd(&ctl.cand_count, 1);
                if (slot < ZCAP) lz[slot] = make_uint2(__float_as_uint(d), static_cast<uint32_t>(i));
                zsum += e;
              }
            } else {
              dsum += e;
            }
          }
        }
      }
    };
    if (deep) { if (t_is_one) body(std::true_type{}, std::true_type{}); else body(std::true_type{}, std::false_type{}); }
    else      { if (t_is_one) body(std::false_type{}, std::true_type{}); else body(std::false_type{}, std::false_type{}); }
  }
  tot = warp_sum_d(tot); dsum = warp_sum_d(dsum); zsum = warp_sum_d(zsum);
  if (lane == 0) s_kseg[warp] = tot - dsum - zsum;          // certainly-kept mass of this warp's run
  double Kr = block_sum_d(lane == 0 ? tot - dsum - zsum : 0.0, ctl, tid);
  double Dr = block_sum_d(lane == 0 ? dsum : 0.0, ctl, tid);
  double Zr = block_sum_d(lane == 0 ? zsum : 0.0, ctl, tid);
  __syncthreads();
  const int nz_loc = min(ctl.cand_count, ZCAP);
  if (tid == 0) {
    X0->K[rank] = Kr; X0->D[rank] = Dr; X0->Z[rank] = Zr;
    int base = atomicAdd(&X0->cand_total, nz_loc);
    ctl.bcast_i[3] = base;
    if (base + nz_loc > ZCAP) X0->overflow = 1;
  }
  __syncthreads();
  {
    // zone keys on rank 0: (dkey << 32) | index (mode B: ascending index among equal d;
    // mode A keeps the HIGHEST indices of a tie, generate.go:208-212, so ~index)
    int base = ctl.bcast_i[3];
    if (base + nz_loc <= ZCAP) {
      unsigned long long* dst = cluster.map_shared_rank(reinterpret_cast<unsigned long long*>(regA), 0);
      for (int j = tid; j < nz_loc; j += NT) {
        uint2 e = lz[j];
        uint32_t dk = dkey_of(__uint_as_float(e.x));
        uint32_t ix = (mode == 0) ? ~e.y : e.y;
        dst[base + j] = (static_cast<unsigned long long>(dk) << 32) | ix;
      }
    }
  }
  cluster.sync();                                            // G4

  // ---- rank 0: exact cut inside the zone, owner of the draw
  if (rank == 0) {
    double Ktot = 0, Dtot = 0, Ztot = 0;
    for (int r = 0; r < C; r++) { Ktot += X.K[r]; Dtot += X.D[r]; Ztot += X.Z[r]; }
    const double S = Ktot + Ztot + Dtot;
    dbg.sum_exp = S;
    uint32_t bad = 0;
    if (!zone_ok || X.overflow) bad = FLAG_INTERNAL;         // zone larger than the exact list: not served
    const bool poisoned = poisoned_early || !(S == S) || !(S > 0.0);
    int kept_zone = 0;
    const int nz = min(X.cand_total, ZCAP);
    unsigned long long* zk = reinterpret_cast<unsigned long long*>(regA);
    double Zk = 0.0;
    if (cut_on && !poisoned && !bad) {
      const int n2 = pow2_at_least(nz);
      for (int j = nz + tid; j < n2; j += NT) zk[j] = ~0ull;
      block_bitonic_u64(zk, n2, tid);
      // masses in sorted order, 4 consecutive entries per thread, block scan
      double e4[4];
      double loc = 0.0;
#pragma unroll
      for (int q = 0; q < 4; q++) {
        int r = tid * 4 + q;
        e4[q] = 0.0;
        if (r < nz) e4[q] = exp_neg<true>(-__uint_as_float(static_cast<uint32_t>(zk[r] >> 32)), s_tab);
        loc += e4[q];
      }
      double ztot_sorted;
      double ex = block_scan_excl_d(loc, ztot_sorted, ctl, tid);
      int cnt_loc = (mode == 0) ? 0 : nz + 1;
      double run = ex;
      double zk_at[4];
#pragma unroll
      for (int q = 0; q < 4; q++) {
        int r = tid * 4 + q;
        run += e4[q];
        zk_at[q] = run;
        if (r < nz) {
          double ratio = (Ktot + run) / S;
          if (mode == 0) { if (ratio <= plim) cnt_loc = max(cnt_loc, r + 1); }
          else { if (ratio >= plim) cnt_loc = min(cnt_loc, r + 1); }
          if (fabs(ratio - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
        }
      }
      if (mode == 0) {
        kept_zone = block_max_i(cnt_loc, ctl, tid);
        if (Ktot > 0.0 && Ktot / S > plim) bad |= FLAG_INTERNAL;
      } else {
        kept_zone = block_min_i(cnt_loc, ctl, tid);
        if (Ktot > 0.0 && Ktot / S >= plim) bad |= FLAG_INTERNAL;
        if (kept_zone == nz + 1) { if (!(Dtot == 0.0)) bad |= FLAG_INTERNAL; kept_zone = nz; }
      }
      flags = static_cast<uint32_t>(block_max_i(static_cast<int>(flags & FLAG_TOPP_EDGE), ctl, tid)) | (flags & ~FLAG_TOPP_EDGE);
      // mass of the kept part of the zone, per owning rank
      __syncthreads();
#pragma unroll
      for (int q = 0; q < 4; q++) {
        int r = tid * 4 + q;
        if (r < kept_zone) {
          uint32_t ix = static_cast<uint32_t>(zk[r]);
          int idx = static_cast<int>(mode == 0 ? ~ix : ix);
          int owner_rank = min(C - 1, rv.vec_of(idx) / SV);
          atomicAdd(&s_zk[owner_rank], e4[q]);
          if (r == kept_zone - 1) ctl.bcast_d[3] = zk_at[q];
        }
      }
      __syncthreads();
      Zk = kept_zone > 0 ? ctl.bcast_d[3] : 0.0;
      if (kept_zone > 0 && kept_zone < nz && (zk[kept_zone] >> 32) == (zk[kept_zone - 1] >> 32)) flags |= FLAG_TIE_CUT;
    }
    const double Re = Ktot + Zk;
    dbg.resum = Re / S;
    int owner = -1;
    int id_now = -2;                                         // -2: the owner writes the id
    if (bad) {
      flags |= bad;
      id_now = -1;
    } else if (poisoned || !(Re > 0.0)) {
      // NaN/Inf in the row, or mode A removed every token (generate.go:221-227): walk falls through
      flags |= FLAG_NONFINITE | FLAG_FALLBACK;
      dbg.sum_exp = poisoned ? QNAN : S;
      if (!poisoned) dbg.resum = 0.0;
      id_now = V - 1;
    } else {
      const double tgt = u * Re;
      double acc = 0.0, base = 0.0;
      for (int r = 0; r < C; r++) {
        double nxt = acc + X.K[r] + s_zk[r];
        if (tgt < nxt) { owner = r; base = acc; break; }
        acc = nxt;
      }
      if (owner < 0) {
        id_now = -3;                                         // generate.go:239: walk falls through
        flags |= FLAG_FALLBACK;
        dbg.edge_lo = dbg.edge_hi = acc / Re;
        if (u - acc / Re <= 1e-6) flags |= FLAG_BOUNDARY;
      }
      if (tid == 0) {
        for (int r = 0; r < C; r++) {
          Xchg* xr = cluster.map_shared_rank(&X, r);
          xr->local_target = tgt - base;
          xr->base_mass = base;
        }
      }
    }
    if (tid == 0) {
      uint32_t cdk = 0; int cix = -1; int cany = 0;
      if (kept_zone > 0) {
        unsigned long long last = zk[kept_zone - 1];
        cdk = static_cast<uint32_t>(last >> 32);
        uint32_t ix = static_cast<uint32_t>(last);
        cix = static_cast<int>(mode == 0 ? ~ix : ix);
        cany = 1;
      }
      for (int r = 0; r < C; r++) {
        Xchg* xr = cluster.map_shared_rank(&X, r);
        xr->owner = owner;
        xr->cut_dkey = cdk; xr->cut_idx = cix; xr->cut_any = cany;
        xr->Re = Re; xr->S = S;
        // 0 owner resolves, 1 poisoned (NaN probabilities), 2 internal, 3 id = V-1 already written
        xr->verdict = (id_now == -2) ? 0 : (id_now == -1 ? 2 : (id_now == -3 ? 3 : 1));
      }
    }
    // rank 0 publishes flags/debug now; the owner adds the id, the edges and the boundary flag
    if (id_now != -2) finish(id_now == -3 ? V - 1 : id_now, flags, dbg);
    else if (tid == 0) {
      if (A.out_flags) A.out_flags[row_id] = flags;
      if (A.out_debug) A.out_debug[row_id] = dbg;
    }
  }
  cluster.sync();                                            // G5: last barrier

  const int verdict = X.verdict;
  if (verdict == 1 || verdict == 2) {
    fill_probs_slice(QNAN);
    return;
  }
  const double Re = X.Re, S = X.S;
  const uint32_t cdk = X.cut_dkey;
  const int cix = X.cut_idx;
  const bool cany = X.cut_any != 0;
  // final rule for one element: its kept mass (0 when filtered or cut away)
  auto kept_mass = [&](float xv, int i) -> double {
    if (i < 0 || i >= V) return 0.0;
    if (filt && !(xv >= flt_lo)) return 0.0;
    float s = t_is_one ? xv : __fdiv_rn(xv, Tm);
    float d = s - m;
    if (d < dA) {
      if (!(d >= dB)) return 0.0;
      if (!cany) return 0.0;
      uint32_t dk = dkey_of(d);
      bool keep = (dk < cdk) || (dk == cdk && (mode == 0 ? i >= cix : i <= cix));
      if (!keep) return 0.0;
    }
    return exp_neg<true>(d, s_tab);
  };

  if (A.out_probs || A.out_debug) {                          // parity runs only
    double* pr = A.out_probs ? A.out_probs + row_id * static_cast<int64_t>(V) : nullptr;
    const double rq = Re / S;
    int kept_loc = 0;
    for (int j = tid; j < nv; j += NT) {
      float x[VEC];
      Elem<T>::unpack(slice_vec(j), x);
      const int i0 = (v0 + j) * VEC - rv.shift;
#pragma unroll
      for (int c = 0; c < VEC; c++) {
        int i = i0 + c;
        if (i >= 0 && i < V) {
          double f = (kept_mass(x[c], i) / S) / rq;
          kept_loc += (f > 0) ? 1 : 0;
          if (pr) pr[i] = f;
        }
      }
    }
    int kept_cta = block_sum_i(kept_loc, ctl, tid);
    if (A.out_debug && tid == 0) atomicAdd(&A.out_debug[row_id].kept, kept_cta);
  }
  if (verdict == 3 || rank != X.owner) return;

  // ---- owner: kept mass per warp run = certain mass + kept zone entries, then one run is rescanned
  __syncthreads();
  for (int j = tid; j < nz_loc; j += NT) {
    uint2 e = lz[j];
    float d = __uint_as_float(e.x);
    int i = static_cast<int>(e.y);
    uint32_t dk = dkey_of(d);
    bool keep = cany && ((dk < cdk) || (dk == cdk && (mode == 0 ? i >= cix : i <= cix)));
    if (keep) {
      int jj = rv.vec_of(i) - v0;
      atomicAdd(&s_kseg[min(NW - 1, jj / wv)], exp_neg<true>(d, s_tab));
    }
  }
  __syncthreads();
  const double ltgt = X.local_target;
  const double base_mass = X.base_mass;
  int wsel = NW;
  double wbase = 0.0;
  {
    double acc = 0.0;
    for (int w = 0; w < NW; w++) {
      double nxt = acc + s_kseg[w];
      if (ltgt < nxt) { wsel = w; wbase = acc; break; }
      acc = nxt;
    }
    if (wsel == NW) { wsel = NW - 1; wbase = acc - s_kseg[NW - 1]; }
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
        Elem<T>::unpack(slice_vec(j), x);
        i0 = (v0 + j) * VEC - rv.shift;
#pragma unroll
        for (int c = 0; c < VEC; c++) { em[c] = kept_mass(x[c], i0 + c); tsum += em[c]; }
      }
      double totc;
      double ex = block_scan_excl_d(tsum, totc, ctl, tid);
      int pick_loc = 0x7fffffff;
      int lk = -1;
      double run = run_end + ex, lo = 0.0, hi = 0.0;
#pragma unroll
      for (int c = 0; c < VEC; c++) {
        double before = run;
        run += em[c];
        if (em[c] > 0.0) {
          lk = i0 + c;
          if (ltgt < run && pick_loc == 0x7fffffff) { pick_loc = i0 + c; lo = before; hi = run; }
        }
      }
      int pick = block_min_i(pick_loc, ctl, tid);
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
