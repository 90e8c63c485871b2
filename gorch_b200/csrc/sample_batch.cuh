// Large-batch kernels: rows are first sorted by what they need, then two
// persistent kernels pull rows from work lists.
//
//   classify_rows_kernel   one thread per row: greedy / top-k rows go to the
//                          "narrow" list, top-k-off rows to the "wide" list,
//                          top-k above 256 to the single-CTA kernel's list.
//   narrow_rows_kernel     256 threads, four CTAs per SM. One streaming pass per
//                          row: the first 4096 logits give a threshold (k-th
//                          largest of the 256 per-thread maxima, a lower bound
//                          of the k-th largest logit), later tiles append the
//                          few logits above it; the list is pruned to the exact
//                          k-th largest when it fills. Everything after the pass
//                          happens on a few hundred candidates in shared memory.
//   wide_rows_kernel       (sample_wide.cuh) rows whose softmax runs over the
//                          whole vocabulary.
//
// Row semantics: model/generate.go:134-260 (mode A), model/qwen/generate.go:
// 77-181 (mode B). Rows a kernel cannot finish (candidate or zone lists that
// outgrow their buffers) are appended to the single-CTA kernel's list.
#pragma once

#include "block_util.cuh"
#include "sample_cluster.cuh"

namespace gs {

constexpr int N_NT = 256;               // narrow kernel threads
constexpr int N_NW = N_NT / 32;
constexpr int N_CAP = 4096;             // candidate capacity (entries of 8 B)
constexpr int N_KEEP = 1536;            // a prune must get below this
constexpr int N_WARM_ELEMS = 4096;      // logits of the warm-up chunk
constexpr int N_DYN_BYTES = 16384 + N_CAP * 8;


struct BatchArgs {
  KernelArgs k;
  const double* eb_table;   // 1024 doubles: exp(-b/32)
  int32_t* hdr;             // [0] narrow count, [1] wide count, [2] narrow cursor, [3] wide cursor
  int32_t* list_narrow;     // [B]
  int32_t* list_wide;       // [B]
  int32_t* list_single;     // [0] = count, [1..] rows for the single-CTA kernel
  int64_t B;
};

__global__ void classify_rows_kernel(BatchArgs BA) {
  const int64_t b = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (b >= BA.B) return;
  const KernelArgs& A = BA.k;
  int kind = 0;   // 0 narrow, 1 wide, 2 single-CTA
  if (!A.force_greedy) {
    const RowCfg c = A.cfgs[b];
    const float T = c.temperature;
    if (T == 0.0f || !(T > 0.0f) || !(T < INFINITY)) {
      kind = 0;   // greedy, or a bad temperature (reported by the narrow kernel)
    } else {
      const int topk = (c.top_k > 0 && c.top_k < A.V) ? c.top_k : 0;
      kind = (topk == 0) ? 1 : (topk <= KFAST ? 0 : 2);
    }
  }
  if (kind == 0) BA.list_narrow[atomicAdd(&BA.hdr[0], 1)] = static_cast<int32_t>(b);
  else if (kind == 1) BA.list_wide[atomicAdd(&BA.hdr[1], 1)] = static_cast<int32_t>(b);
  else BA.list_single[1 + atomicAdd(&BA.list_single[0], 1)] = static_cast<int32_t>(b);
}

__device__ __forceinline__ void hand_to_single(const BatchArgs& BA, int64_t row_id) {
  BA.list_single[1 + atomicAdd(&BA.list_single[0], 1)] = static_cast<int32_t>(row_id);
}

// ---------------------------------------------------------------------------
// Finish a row whose kept set (nk <= 512 entries of (logit bits, index)) sits in
// shared memory: softmax over the kept set, top-p, draw. Work arrays: 16 KB.
// ---------------------------------------------------------------------------
template <int NTHREADS>
__device__ void finish_small_set(const KernelArgs& A, int64_t row_id, const uint2* kp, int nk, float m, float Tm,
                                 bool topp_on, int mode, double plim, double u, unsigned char* work,
                                 bu::Scratch& sc, double* bc_d, RowDebug& dbg, uint32_t flags) {
  constexpr int NWARPS = NTHREADS / 32;
  constexpr int PER = (KEEP_MAX + NTHREADS - 1) / NTHREADS;
  const int tid = threadIdx.x;
  const int V = A.V;
  const double QNAN = __longlong_as_double(0x7ff8000000000000ll);
  float* sx = reinterpret_cast<float*>(work);                 // [512] scaled value, index order
  int* sidx = reinterpret_cast<int*>(work + 2048);            // [512]
  double* se = reinterpret_cast<double*>(work + 4096);        // [512] probability
  double* sf = reinterpret_cast<double*>(work + 8192);        // [512] scratch / final probability
  int* rnk = reinterpret_cast<int*>(work + 12288);            // [512]
  int* ord = reinterpret_cast<int*>(work + 14336);            // [512]
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
      for (int i = tid; i < V; i += NTHREADS) pr[i] = v;
    }
  };
  __syncthreads();
  float thr_s = INFINITY;
  for (int j = tid; j < nk; j += NTHREADS) {
    const uint32_t myi = kp[j].y;
    int r = 0;
    for (int l = 0; l < nk; l++) r += (kp[l].y < myi) ? 1 : 0;
    const float s = scale_t(__uint_as_float(kp[j].x), Tm);
    sx[r] = s;
    sidx[r] = static_cast<int>(myi);
    thr_s = fminf(thr_s, s);
  }
  dbg.threshold = okey_to_float(static_cast<uint32_t>(bu::min_u64<NWARPS>(static_cast<unsigned long long>(okey(thr_s)), sc, tid)));
  __syncthreads();
  double e_loc = 0.0;
  for (int j = tid; j < nk; j += NTHREADS) {
    const double e = exp(static_cast<double>(sx[j] - m));     // f32 subtract, f64 exp (generate.go:176)
    se[j] = e;
    e_loc += e;
  }
  const double S = bu::sum_d<NWARPS>(e_loc, sc, tid);
  dbg.sum_exp = S;
  for (int j = tid; j < nk; j += NTHREADS) { const double q = se[j] / S; se[j] = q; sf[j] = q; }   // generate.go:179-181
  __syncthreads();
  if (topp_on) {
    // order by probability; equal probabilities by index, ascending in both flavours
    // (mode A removes the lowest index first, mode B keeps it first)
    for (int j = tid; j < nk; j += NTHREADS) {
      const double qj = se[j];
      int r = 0;
      if (mode == 0) { for (int l = 0; l < nk; l++) { const double ql = se[l]; r += (ql < qj || (ql == qj && l < j)) ? 1 : 0; } }
      else           { for (int l = 0; l < nk; l++) { const double ql = se[l]; r += (ql > qj || (ql == qj && l < j)) ? 1 : 0; } }
      ord[r] = j;
      rnk[j] = r;
    }
    __syncthreads();
    if (mode == 0) {
      // generate.go:184-228: the mass left after removing the r smallest is a suffix sum.
      // sf[t] = probability of rank nk-1-t, scanned: sf[t] = mass of the t+1 largest.
      for (int t = tid; t < nk; t += NTHREADS) sf[t] = se[ord[nk - 1 - t]];
      __syncthreads();
      bu::smem_scan_incl<NWARPS, PER>(sf, nk, sc, tid);
      // left after removing r smallest = sf[nk-1-r]
      int rs = nk;
      for (int r = tid; r < nk; r += NTHREADS) if (sf[nk - 1 - r] <= plim) rs = min(rs, r);
      const int rstar = bu::min_i<NWARPS>(rs, sc, tid);
      if (rstar == nk) {                                      // everything removed: 0/0 (generate.go:221-227)
        dbg.resum = 0.0;
        fill_probs_row(QNAN);
        write_row(V - 1, flags | FLAG_NONFINITE | FLAG_FALLBACK);
        return;
      }
      const double resum = sf[nk - 1 - rstar];
      if (fabs(resum - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
      if (rstar > 0 && fabs(sf[nk - rstar] - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
      dbg.resum = resum;
      __syncthreads();
      for (int j = tid; j < nk; j += NTHREADS) sf[j] = (rnk[j] >= rstar) ? se[j] / resum : 0.0;
    } else {
      // qwen/generate.go:123-153: shortest descending prefix with mass >= p
      for (int t = tid; t < nk; t += NTHREADS) sf[t] = se[ord[t]];
      __syncthreads();
      bu::smem_scan_incl<NWARPS, PER>(sf, nk, sc, tid);
      int cl = nk;
      for (int r = tid; r < nk; r += NTHREADS) if (sf[r] >= plim) cl = min(cl, r + 1);
      const int cutn = bu::min_i<NWARPS>(cl, sc, tid);
      const double resum = sf[cutn - 1];
      if (fabs(resum - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
      if (cutn >= 2 && fabs(sf[cutn - 2] - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
      if (cutn < nk && se[ord[cutn]] == se[ord[cutn - 1]]) flags |= FLAG_TIE_CUT;
      dbg.resum = resum;
      __syncthreads();
      for (int j = tid; j < nk; j += NTHREADS) sf[j] = (rnk[j] < cutn) ? se[j] / resum : 0.0;
    }
    __syncthreads();
  }
  int kept_loc = 0;
  for (int j = tid; j < nk; j += NTHREADS) kept_loc += (sf[j] > 0) ? 1 : 0;
  dbg.kept = bu::sum_i<NWARPS>(kept_loc, sc, tid);
  if (A.out_probs) {
    fill_probs_row(0.0);
    __syncthreads();
    double* pr = A.out_probs + row_id * static_cast<int64_t>(V);
    for (int j = tid; j < nk; j += NTHREADS) pr[sidx[j]] = sf[j];
  }
  // draw (generate.go:231-239): first index with u < cumulative
  for (int j = tid; j < nk; j += NTHREADS) se[j] = sf[j];
  __syncthreads();
  bu::smem_scan_incl<NWARPS, PER>(se, nk, sc, tid);
  int pl = nk;
  for (int j = tid; j < nk; j += NTHREADS) if (u < se[j]) pl = min(pl, j);
  const int pick = bu::min_i<NWARPS>(pl, sc, tid);
  int id;
  if (pick < nk) {
    id = sidx[pick];
    const double hi = se[pick], lo = pick > 0 ? se[pick - 1] : 0.0;
    dbg.edge_lo = lo; dbg.edge_hi = hi;
    if ((pick > 0 && u - lo <= 1e-6) || hi - u <= 1e-6) flags |= FLAG_BOUNDARY;
  } else {
    id = V - 1;
    flags |= FLAG_FALLBACK;
    const double tot = se[nk - 1];
    dbg.edge_lo = dbg.edge_hi = tot;
    if (u - tot <= 1e-6) flags |= FLAG_BOUNDARY;
  }
  (void)bc_d;
  write_row(id, flags);
}

template <typename T>
__device__ __forceinline__ uint4 mask_edges(const RowView<T>& rv, int v, uint4 raw);

// ---------------------------------------------------------------------------
// narrow: greedy and top-k <= 256 rows, one streaming pass each
// ---------------------------------------------------------------------------
template <typename T>
__device__ void narrow_row(const BatchArgs& BA, const int64_t row_id, unsigned char* dyn, bu::Scratch& sc,
                           uint32_t* s_sel, int* s_bc, double* s_bcd, int* s_cnt, float* s_thr) {
  const KernelArgs& A = BA.k;
  const int tid = threadIdx.x;
  const int V = A.V;
  constexpr int VEC = Elem<T>::VEC;
  constexpr int WARM_VECS = N_WARM_ELEMS / VEC;
  constexpr int TILE_ELEMS = N_NT * VEC;
  const T* row = static_cast<const T*>(A.logits) + row_id * A.row_stride;
  RowView<T> rv;
  rv.init(row, V);
  uint4* chunk = reinterpret_cast<uint4*>(dyn);              // warm-up vectors, 16 KB; later work arrays
  uint2* cand = reinterpret_cast<uint2*>(dyn + 16384);       // N_CAP entries
  const double QNAN = __longlong_as_double(0x7ff8000000000000ll);

  RowCfg cfg;
  if (A.force_greedy) { cfg.temperature = 0.f; cfg.top_k = 0; cfg.top_p = 0.f; cfg.topp_mode = 0; }
  else cfg = A.cfgs[row_id];
  const float Tm = cfg.temperature;
  RowDebug dbg;
  dbg.sum_exp = 0; dbg.resum = 1.0; dbg.edge_lo = 0; dbg.edge_hi = 0; dbg.kept = 0;
  dbg.max_scaled = 0; dbg.threshold = __int_as_float(0x7fc00000); dbg.path = 0;
  for (int q = 0; q < 8; q++) dbg.cycles[q] = 0;
  long long tprev = clock64();
  auto stamp = [&](int slot) { const long long now = clock64(); dbg.cycles[slot] = static_cast<uint32_t>(now - tprev); tprev = now; };
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
      for (int i = tid; i < V; i += N_NT) pr[i] = v;
    }
  };

  // ---- greedy (generate.go:75-76, 134-144): strict '>' from index 0, lowest index wins ties
  if (Tm == 0.0f) {
    unsigned long long best = 0ull;
    for (int v = tid; v < rv.nvec; v += N_NT) {
      const uint4 raw = __ldg(rv.vbase + v);
      rv.visit_raw(raw, v, [&](float x, int i, int) {
        const unsigned long long p = (static_cast<unsigned long long>(okey(x)) << 32) |
                                     static_cast<uint32_t>(~static_cast<uint32_t>(i));
        best = p > best ? p : best;
      });
    }
    best = bu::max_u64<N_NW>(best, sc, tid);
    int id = static_cast<int>(~static_cast<uint32_t>(best & 0xffffffffull));
    float x0 = 0.f;
    rv.visit(0, [&](float x, int i) { if (i == 0) x0 = x; });
    if (x0 != x0) id = 0;                                    // a NaN at index 0 is never beaten
    fill_probs_row(0.0);
    __syncthreads();
    if (A.out_probs && tid == 0) A.out_probs[row_id * static_cast<int64_t>(V) + id] = 1.0;
    dbg.kept = 1;
    write_row(id, 0u);
    return;
  }
  if (!(Tm > 0.0f) || !(Tm < INFINITY)) {
    fill_probs_row(QNAN);
    write_row(-1, FLAG_BAD_CFG);
    return;
  }
  const int topk = cfg.top_k;                                // 0 < top_k <= KFAST, < V (classified)
  const bool topp_on = (cfg.top_p > 0.0f && cfg.top_p < 1.0f);
  const int mode = cfg.topp_mode;
  const double plim = (mode == 0) ? static_cast<double>(cfg.top_p) * 1.5 : static_cast<double>(cfg.top_p);
  dbg.path = 1;

  // ---- warm-up chunk: park it, one running maximum per thread
  float xmax = -INFINITY, xmin = INFINITY;
  bool nan_seen = false;
  if (tid == 0) *s_cnt = 0;
  const int warm = min(rv.nvec, WARM_VECS);
  {
    constexpr int G = WARM_VECS / N_NT;
    uint4 r[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
      const int v = g * N_NT + tid;
      if (v < warm) { r[g] = load_masked(rv, v, xmax, xmin, nan_seen); chunk[v] = r[g]; }
    }
  }
  // thr: lower edge of the 16-bit key bin holding the k-th largest per-thread maximum
  float thr = -INFINITY;
  {
    uint32_t prefix = 0, mask = 0;
    int need = topk;
    const uint32_t mykey = okey(xmax);
    bool have_thr = true;
    for (int round = 0; round < 2; round++) {
      const int sh = 24 - 8 * round;
      __syncthreads();
      s_sel[tid] = 0;
      if (tid == 0) s_bc[0] = -1;
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
          const int t = __shfl_down_sync(FULL, run, o);
          if (tid + o < 32) run += t;
        }
        const int above = run - s;
        if (above < need && above + s >= need) {
#pragma unroll
          for (int j = 7; j >= 0; j--) {
            if (above + loc[j] >= need) {
              s_bc[0] = tid * 8 + j;
              s_bc[1] = need - (above + loc[j] - static_cast<int>(s_sel[tid * 8 + j]));
              break;
            }
          }
        }
      }
      __syncthreads();
      if (s_bc[0] < 0) { have_thr = false; break; }
      prefix |= static_cast<uint32_t>(s_bc[0]) << sh;
      mask |= 255u << sh;
      need = s_bc[1];
    }
    if (prefix <= 0x007fffffu) have_thr = false;             // bound at or below -Inf: keep everything
    __syncthreads();
    if (have_thr) {
      if (tid == 0) *s_thr = quotient_class_floor(okey_to_float(prefix), Tm);
      __syncthreads();
      thr = *s_thr;
    }
  }
  // candidates of the warm-up chunk
  for (int v = tid; v < warm; v += N_NT) {
    float x[VEC];
    Elem<T>::unpack(chunk[v], x);
    const int i0 = v * VEC - rv.shift;
#pragma unroll
    for (int c = 0; c < VEC; c++) {
      const int i = i0 + c;
      if (x[c] >= thr && i >= 0 && i < V) {
        const int slot = atomicAdd(s_cnt, 1);
        cand[slot] = make_uint2(__float_as_uint(x[c]), static_cast<uint32_t>(i));
      }
    }
  }
  __syncthreads();
  stamp(0);
  bool giveup = false;
  // exact k-th largest of the list -> threshold; keepers move through the chunk buffer
  auto prune = [&](int cnt) -> int {
    if (cnt <= topk) return cnt;
    const uint32_t kkey = bu::select_kth<N_NT>(cand, cnt, topk, s_sel, s_bc, tid);
    if (tid == 0) { *s_thr = quotient_class_floor(okey_to_float(kkey), Tm); *s_cnt = 0; }
    __syncthreads();
    thr = *s_thr;
    uint2* tmp = reinterpret_cast<uint2*>(chunk);            // 2048 entries
    for (int j = tid; j < cnt; j += N_NT) {
      const uint2 e = cand[j];
      if (__uint_as_float(e.x) >= thr) { const int slot = atomicAdd(s_cnt, 1); if (slot < 2048) tmp[slot] = e; }
    }
    __syncthreads();
    const int kept = *s_cnt;
    if (kept <= 2048) for (int j = tid; j < kept; j += N_NT) cand[j] = tmp[j];
    __syncthreads();
    return kept;
  };
  int do_prune = (*s_cnt + TILE_ELEMS > N_CAP) ? 1 : 0;
  __syncthreads();                                           // everybody has read the count before anyone appends again
  // ---- stream the rest. Raw vectors are fetched two tiles ahead and only looked at when
  // their tile comes up, so two loads per thread stay in flight.
  const uint4 NEUT = make_uint4(Neutral<T>::word, Neutral<T>::word, Neutral<T>::word, Neutral<T>::word);
  constexpr int PF = 4;                                      // tiles in flight per thread
  uint4 nxt[PF];
#pragma unroll
  for (int q = 0; q < PF; q++) {
    nxt[q] = NEUT;
    if (warm + q * N_NT + tid < rv.nvec) nxt[q] = __ldg(rv.vbase + warm + q * N_NT + tid);
  }
  for (int base = warm; base < rv.nvec; base += N_NT) {      // uniform loop
    uint4 raw = nxt[0];
#pragma unroll
    for (int q = 0; q + 1 < PF; q++) nxt[q] = nxt[q + 1];
    nxt[PF - 1] = NEUT;
    const int v = base + tid;
    if (v + PF * N_NT < rv.nvec) nxt[PF - 1] = __ldg(rv.vbase + v + PF * N_NT);
    if (do_prune) {
      const int cnt = prune(*s_cnt);
      if (cnt > N_KEEP) { giveup = true; break; }            // ties at the threshold fill the buffer
    }
    if (v == rv.nvec - 1) raw = mask_edges(rv, v, raw);      // lanes past the row's end become -Inf
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
    if (any) {                                               // threads past the row hold -Inf: thr > -Inf here or i is checked
      const int i0 = v * VEC - rv.shift;
#pragma unroll
      for (int c = 0; c < VEC; c++) {
        const int i = i0 + c;
        if (x[c] >= thr && i >= 0 && i < V) {
          const int slot = atomicAdd(s_cnt, 1);
          cand[slot] = make_uint2(__float_as_uint(x[c]), static_cast<uint32_t>(i));
          want |= (slot + 1 + TILE_ELEMS > N_CAP);
        }
      }
    }
    do_prune = __syncthreads_or(want ? 1 : 0);
  }
  stamp(1);
  dbg.cycles[5] = static_cast<uint32_t>(*s_cnt);
  int nk = 0;
  if (!giveup) {
    nk = prune(*s_cnt);
    if (nk > KEEP_MAX) giveup = true;                        // long run of ties at the threshold
  }
  const int anynan = bu::max_i<N_NW>(nan_seen ? 1 : 0, sc, tid);
  xmax = okey_to_float(static_cast<uint32_t>(bu::max_u64<N_NW>(static_cast<unsigned long long>(okey(xmax)), sc, tid)));
  const float m = scale_t(xmax, Tm);
  dbg.max_scaled = m;
  // A NaN anywhere, or an infinite maximum, makes the softmax sum NaN upstream
  // (generate.go:173-181): every comparison of the walk fails, result n-1 (:239).
  if (anynan || !(fabsf(m) < INFINITY)) {
    fill_probs_row(QNAN);
    dbg.sum_exp = QNAN;
    write_row(V - 1, FLAG_NONFINITE | FLAG_FALLBACK);
    return;
  }
  if (giveup) {
    if (tid == 0) hand_to_single(BA, row_id);
    return;
  }
  stamp(2);
  finish_small_set<N_NT>(A, row_id, cand, nk, m, Tm, topp_on, mode, plim, A.uniforms[row_id],
                         reinterpret_cast<unsigned char*>(chunk), sc, s_bcd, dbg, 0u);
}

template <typename T>
__global__ void __launch_bounds__(N_NT, 4) narrow_rows_kernel(BatchArgs BA) {
  extern __shared__ __align__(16) unsigned char dyn[];
  __shared__ bu::Scratch sc;
  __shared__ uint32_t s_sel[256];
  __shared__ int s_bc[4];
  __shared__ double s_bcd[4];
  __shared__ int s_cnt;
  __shared__ float s_thr;
  __shared__ int s_row;
  const int n = BA.hdr[0];
  for (;;) {
    __syncthreads();
    if (threadIdx.x == 0) {
      const int w = atomicAdd(&BA.hdr[2], 1);
      s_row = (w < n) ? BA.list_narrow[w] : -1;
    }
    __syncthreads();
    const int row = s_row;
    if (row < 0) break;
    narrow_row<T>(BA, row, dyn, sc, s_sel, s_bc, s_bcd, &s_cnt, &s_thr);
  }
}


template <typename T>
__device__ __forceinline__ uint4 mask_edges(const RowView<T>& rv, int v, uint4 raw) {
  if (v > 0 && v < rv.nvec - 1) return raw;
  constexpr int VEC = Elem<T>::VEC;
  uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  const int i0 = v * VEC - rv.shift;
#pragma unroll
  for (int c = 0; c < VEC; c++) {
    const int i = i0 + c;
    if (i < 0 || i >= rv.V) {
      if (sizeof(T) == 4) w[c] = 0xff800000u;
      else if (c & 1) w[c >> 1] = (w[c >> 1] & 0x0000ffffu) | 0xff800000u;
      else w[c >> 1] = (w[c >> 1] & 0xffff0000u) | 0x0000ff80u;
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

}  // namespace gs
