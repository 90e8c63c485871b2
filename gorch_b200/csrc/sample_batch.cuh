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
//   wide_rows_kernel       1024 threads, one CTA per SM, for rows whose softmax
//                          runs over the whole vocabulary. Pass 1 (max) streams
//                          the row from HBM, parks its head in shared memory
//                          and asks L2 to keep the rest (evict-last); pass 2
//                          (count histogram, only with an active top-p cut) and
//                          pass 3 (exponentials) re-read shared memory and L2.
//                          The cut is bracketed from count-based mass bounds,
//                          the bracketed zone is listed and cut exactly.
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

constexpr int W_NT = 1024;              // wide kernel threads
constexpr int W_NW = W_NT / 32;
constexpr int W_CACHE_VECS = 11264;     // 16-byte vectors of a row parked in shared memory (176 KB)
constexpr int W_NB = 4096;              // histogram buckets of width 1/128 over d in [-32, 0]
constexpr int W_ZCAP = 2048;            // exact zone list capacity
constexpr int W_OFF_HIST = W_CACHE_VECS * 16;
constexpr int W_OFF_ZONE = W_OFF_HIST + W_NB * 4;
constexpr int W_OFF_EB = W_OFF_ZONE + W_ZCAP * 8;
constexpr int W_DYN_BYTES = W_OFF_EB + NB1 * 8;   // (layout of the earlier register-fetch variant; the ring layout follows below)

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

// ---------------------------------------------------------------------------
// wide: rows whose softmax runs over the whole vocabulary
// ---------------------------------------------------------------------------
__device__ __forceinline__ int bucket_w(float d) {           // 4096 buckets of width 1/128
  const float f = fmaf(fmaxf(d, -31.992f), -128.0f, 8388608.0f);
  return __float_as_int(f) & 0x1fff;
}
__device__ __forceinline__ float bucket_floor_w(int bmax) {   // smallest d whose bucket is <= bmax
  if (bmax >= W_NB - 1) return -INFINITY;
  if (bmax < 0) return INFINITY;
  const float t = -(static_cast<float>(2 * bmax + 1) * 0.00390625f);
  return (bucket_w(t) <= bmax) ? t : __uint_as_float(__float_as_uint(t) - 1u);
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

#ifndef GS_W_TILE_VECS
#define GS_W_TILE_VECS 2048
#define GS_W_NST 4
#endif
constexpr int W_TILE_VECS = GS_W_TILE_VECS;   // 32 KB tiles
constexpr int W_NST = GS_W_NST;                // ring stages
constexpr int W_MAX_TILES = 64;         // rows above 64 tiles (131072 vectors) go to the single-CTA kernel
constexpr int W2_OFF_HIST = W_NST * W_TILE_VECS * 16;        // 128 KB ring
constexpr int W2_OFF_ZONE = W2_OFF_HIST + W_NB * 4;
constexpr int W2_OFF_EB = W2_OFF_ZONE + W_ZCAP * 8;
constexpr int W2_OFF_PART = W2_OFF_EB + NB1 * 8;
constexpr int W2_DYN_BYTES = W2_OFF_PART + W_MAX_TILES * W_NW * 8;

// Thread-private asynchronous prefetch through shared memory. A tile is W_TILE_VECS vectors; warp w
// owns vectors [64w, 64w+64) of every tile and lane l of it the two vectors 64w+l and 64w+32+l. Each
// thread copies exactly the vectors it will read (cp.async, 16 bytes each, through L2 like an
// ordinary load) W_NST-1 tiles ahead into its own slots of a W_NST-deep ring and waits for its own
// copy groups: no barrier of any kind inside a pass, and the row is re-read from L2 by later passes.
struct WRing {
  uint4* base;
  const uint4* src;        // vector 0 of the row
  int nvec, ntiles;
  unsigned long long pol;
};
__device__ __forceinline__ void cp_async16(uint32_t dst_s, const void* src, unsigned long long pol) {
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" :: "r"(dst_s), "l"(src), "l"(pol) : "memory");
}
__device__ __forceinline__ void wring_issue(const WRing& r, int t, int warp, int lane) {
  if (t < r.ntiles) {
    const int j = warp * (W_TILE_VECS / W_NW) + lane;
    const int g = t * W_TILE_VECS + j;
    const uint32_t d = smem_addr(r.base + (t % W_NST) * W_TILE_VECS + j);
    if (g < r.nvec) cp_async16(d, r.src + g, r.pol);
    if (g + 32 < r.nvec) cp_async16(d + 512u, r.src + g + 32, r.pol);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");   // one group per tile, empty or not
}
__device__ __forceinline__ void wring_begin(const WRing& r, int tid) {
#pragma unroll
  for (int t = 0; t < W_NST - 1; t++) wring_issue(r, t, tid >> 5, tid & 31);
}
// Issues tile t+W_NST-1 into the slot read one iteration ago and returns tile t once this
// thread's copies of it have landed.
__device__ __forceinline__ const uint4* wring_acquire(const WRing& r, int t, int warp, int lane) {
  wring_issue(r, t + W_NST - 1, warp, lane);
  asm volatile("cp.async.wait_group %0;" :: "n"(W_NST - 1) : "memory");
  return r.base + (t % W_NST) * W_TILE_VECS;
}
__device__ __forceinline__ void wring_release(const WRing&, int, int) {}
__device__ __forceinline__ void wring_end(const WRing&, int) {
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}
// Shared-memory loads by 32-bit shared address (the pointers below travel through structs and
// function arguments, where the compiler would otherwise fall back to generic loads).
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
  uint4 v;
  asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ double lds_f64(uint32_t addr) {
  double v;
  asm("ld.shared.f64 %0, [%1];" : "=d"(v) : "r"(addr));
  return v;
}
// exp_fast with the bucket table addressed in the shared window
__device__ __forceinline__ double exp_fast_s(float d, uint32_t eb_s) {
  const float f = fmaf(d, -32.0f, 8388608.0f);
  const uint32_t b8 = (__float_as_uint(f) & 0x7ffu) << 3;
  const float dl = fmaf(f - 8388608.0f, 0.03125f, d);
  float t = fmaf(dl, 8.3333338e-3f, 4.1666668e-2f);
  t = fmaf(t, dl, 1.6666667e-1f);
  t = fmaf(t, dl, 0.5f);
  const float tail = t * (dl * dl);
  const double w = static_cast<double>(dl) + static_cast<double>(tail);
  const double E = lds_f64(eb_s + b8);
  return fma(E, w, E);
}

// A warp's piece of a tile is "clean" when all of its 64 vectors exist and none of them is the
// row's first or last vector (the only ones that can hold lanes outside the row). Clean pieces
// take the unchecked loops below; the others (two or three per row) check every lane.
__device__ __forceinline__ bool piece_clean(int t, int warp, int nvt, int nvec) {
  constexpr int PIECE = W_TILE_VECS / W_NW;
  const int pb = warp * PIECE, g0 = t * W_TILE_VECS + pb;
  return (pb + PIECE <= nvt) && g0 > 0 && (g0 + PIECE - 1 < nvec - 1);
}
// Eight logits of a lane for step `step`: vectors j0 and j0+32 (f32) or vector j0 (bf16).
template <typename T>
__device__ __forceinline__ void load8(const uint4* tile, int warp, int lane, int step, float* x, int& j0) {
  constexpr int VEC = Elem<T>::VEC;
  constexpr int PIECE = W_TILE_VECS / W_NW;
  constexpr int EPI = 8 / VEC;
  j0 = warp * PIECE + step * 32 * EPI + lane;
  const uint32_t a = smem_addr(tile) + static_cast<uint32_t>(j0) * 16u;
  if (EPI == 2) {
    float xa[4], xb[4];
    Elem<T>::unpack(lds_v4(a), xa);
    Elem<T>::unpack(lds_v4(a + 512u), xb);
#pragma unroll
    for (int c = 0; c < 4; c++) { x[c] = xa[c]; x[4 + c] = xb[c]; }
  } else {
    Elem<T>::unpack(lds_v4(a), x);
  }
}
// Same for a piece that is not clean: `valid` gets one bit per logit that lies inside the tile
// and inside the row; the others read as -Inf.
template <typename T>
__device__ __forceinline__ void load8_checked(const uint4* tile, int nvt, int t, const RowView<T>& rv, int warp, int lane,
                                              int step, float* x, int& j0, uint32_t& valid) {
  constexpr int VEC = Elem<T>::VEC;
  constexpr int PIECE = W_TILE_VECS / W_NW;
  constexpr int EPI = 8 / VEC;
  j0 = warp * PIECE + step * 32 * EPI + lane;
  valid = 0u;
#pragma unroll
  for (int h = 0; h < EPI; h++) {
    const int j = j0 + 32 * h;
    float xv[VEC];
#pragma unroll
    for (int c = 0; c < VEC; c++) xv[c] = -INFINITY;
    if (j < nvt) {
      Elem<T>::unpack(tile[j], xv);
      const int i0 = (t * W_TILE_VECS + j) * VEC - rv.shift;
#pragma unroll
      for (int c = 0; c < VEC; c++) {
        const int i = i0 + c;
        if (i >= 0 && i < rv.V) valid |= 1u << (h * VEC + c); else xv[c] = -INFINITY;
      }
    }
#pragma unroll
    for (int c = 0; c < VEC; c++) x[h * VEC + c] = xv[c];
  }
}

// pass 1: max, min, NaN flag over the row's logits
template <typename T>
__device__ __noinline__ void wide_pass1(const WRing& r_io, const RowView<T>& rv_in, int tid, float& xmax, float& xmin, bool& nan_seen) {
  constexpr int VEC = Elem<T>::VEC;
  constexpr int STEPS = (W_TILE_VECS / W_NW) / (32 * (8 / VEC));
  const int warp = tid >> 5, lane = tid & 31;
  const WRing r = r_io;                // registers, not memory, inside the loop
  const RowView<T> rv = rv_in;
  float vmax = -INFINITY, vmin = INFINITY;
  bool nan = false;
  wring_begin(r, tid);
  for (int t = 0; t < r.ntiles; t++) {
    const uint4* tile = wring_acquire(r, t, warp, lane);
    const int nvt = min(W_TILE_VECS, r.nvec - t * W_TILE_VECS);
    if (piece_clean(t, warp, nvt, r.nvec)) {
#pragma unroll
      for (int step = 0; step < STEPS; step++) {
        float x[8];
        int j0;
        load8<T>(tile, warp, lane, step, x, j0);
#pragma unroll
        for (int c = 0; c < 8; c++) { vmax = fmaxf(vmax, x[c]); vmin = fminf(vmin, x[c]); nan |= (x[c] != x[c]); }
      }
    } else {
#pragma unroll
      for (int step = 0; step < STEPS; step++) {
        float x[8];
        int j0;
        uint32_t valid;
        load8_checked<T>(tile, nvt, t, rv, warp, lane, step, x, j0, valid);
#pragma unroll
        for (int c = 0; c < 8; c++) {
          if ((valid >> c) & 1u) { vmax = fmaxf(vmax, x[c]); vmin = fminf(vmin, x[c]); nan |= (x[c] != x[c]); }
        }
      }
    }
    wring_release(r, t, lane);
  }
  wring_end(r, warp);
  xmax = vmax; xmin = vmin; nan_seen = nan;
}

// pass 2: count histogram over the 1/128 buckets of d (logits outside the row are not counted)
template <typename T>
__device__ __noinline__ void wide_pass2(const WRing& r_io, const RowView<T>& rv_in, int tid, uint32_t* hist, float m, float Tm) {
  constexpr int VEC = Elem<T>::VEC;
  constexpr int STEPS = (W_TILE_VECS / W_NW) / (32 * (8 / VEC));
  const int warp = tid >> 5, lane = tid & 31;
  const bool t_is_one = (Tm == 1.0f);
  const WRing r = r_io;
  const RowView<T> rv = rv_in;
  wring_begin(r, tid);
  for (int t = 0; t < r.ntiles; t++) {
    const uint4* tile = wring_acquire(r, t, warp, lane);
    const int nvt = min(W_TILE_VECS, r.nvec - t * W_TILE_VECS);
    if (piece_clean(t, warp, nvt, r.nvec)) {
#pragma unroll
      for (int step = 0; step < STEPS; step++) {
        float x[8];
        int j0;
        load8<T>(tile, warp, lane, step, x, j0);
        if (t_is_one) {
#pragma unroll
          for (int c = 0; c < 8; c++) atomicAdd(&hist[bucket_w(x[c] - m)], 1u);
        } else {
#pragma unroll
          for (int c = 0; c < 8; c++) atomicAdd(&hist[bucket_w(__fdiv_rn(x[c], Tm) - m)], 1u);
        }
      }
    } else {
#pragma unroll
      for (int step = 0; step < STEPS; step++) {
        float x[8];
        int j0;
        uint32_t valid;
        load8_checked<T>(tile, nvt, t, rv, warp, lane, step, x, j0, valid);
#pragma unroll
        for (int c = 0; c < 8; c++) {
          if ((valid >> c) & 1u) atomicAdd(&hist[bucket_w(scale_t(x[c], Tm) - m)], 1u);
        }
      }
    }
    wring_release(r, t, lane);
  }
  wring_end(r, warp);
}

// pass 3: exponentials. part[t*W_NW + warp] receives the certainly-kept mass of the warp's
// piece of tile t; the lane-private sums of dropped and zone mass come back by reference.
// FAST: every logit of the row has d > -31.9 (bucket-table exponential, no range check);
// TONE: temperature 1; CUT: a top-p cut is active (dA/dB classify the logits).
template <typename T, bool FAST, bool TONE, bool CUT>
__device__ __noinline__ void wide_pass3(const WRing& r_io, const RowView<T>& rv_in, int tid, float m, float Tm, float dA, float dB,
                                        const double* ebs, const double* s_tab, double* part, uint2* zl, int* zcnt,
                                        double& Ksum, double& Dsum, double& Zsum) {
  constexpr int VEC = Elem<T>::VEC;
  constexpr int EPI = 8 / VEC;
  constexpr int STEPS = (W_TILE_VECS / W_NW) / (32 * EPI);
  const int warp = tid >> 5, lane = tid & 31;
  const WRing r = r_io;
  const RowView<T> rv = rv_in;
  const uint32_t eb_s = smem_addr(ebs);
  double dsum = 0.0, zsum = 0.0, ksum = 0.0;
  wring_begin(r, tid);
  for (int t = 0; t < r.ntiles; t++) {
    const uint4* tile = wring_acquire(r, t, warp, lane);
    const int nvt = min(W_TILE_VECS, r.nvec - t * W_TILE_VECS);
    double t0 = 0.0, t1 = 0.0, t2 = 0.0, t3 = 0.0, sub = 0.0;   // sub: zone + dropped mass of this tile
#ifdef GS_EXPERIMENT_CLEAN
    const bool clean = true;
#else
    const bool clean = piece_clean(t, warp, nvt, r.nvec);
#endif
#pragma unroll
    for (int step = 0; step < STEPS; step++) {
      float x[8];
      int j0;
      uint32_t valid = 0xffu;
      if (clean) load8<T>(tile, warp, lane, step, x, j0);
      else load8_checked<T>(tile, nvt, t, rv, warp, lane, step, x, j0, valid);
      double e[8];
      float d[8];
      float dmin = 0.0f;
#pragma unroll
      for (int c = 0; c < 8; c++) {
        const float s = TONE ? x[c] : __fdiv_rn(x[c], Tm);
        d[c] = s - m;
        if (FAST) {
          if (clean) e[c] = exp_fast_s(d[c], eb_s);
          else e[c] = ((valid >> c) & 1u) ? exp_fast_s(d[c], eb_s) : 0.0;
        } else {
          e[c] = exp_safe(d[c], s_tab);                      // -Inf gives exactly 0
        }
        if (CUT) dmin = fminf(dmin, d[c]);
      }
      t0 += e[0] + e[4]; t1 += e[1] + e[5]; t2 += e[2] + e[6]; t3 += e[3] + e[7];
      if (CUT && dmin < dA) {
#pragma unroll
        for (int c = 0; c < 8; c++) {
          if (d[c] < dA && ((valid >> c) & 1u)) {
            sub += e[c];
            if (d[c] >= dB) {
              const int jj = (EPI == 2 && c >= 4) ? j0 + 32 : j0;
              const int i = (t * W_TILE_VECS + jj) * VEC - rv.shift + ((EPI == 2) ? (c & 3) : c);
              const int slot = atomicAdd(zcnt, 1);
              if (slot < W_ZCAP) zl[slot] = make_uint2(__float_as_uint(d[c]), static_cast<uint32_t>(i));
              zsum += e[c];
            } else {
              dsum += e[c];
            }
          }
        }
      }
    }
    wring_release(r, t, lane);
    // certainly-kept mass of this piece. With dA = +Inf nothing is certainly kept (exactly 0);
    // otherwise the subtraction's rounding is far below the row maximum's own mass.
    double kw = (CUT && dA == INFINITY) ? 0.0 : ((t0 + t1) + (t2 + t3)) - sub;
    kw = warp_sum_d(kw);
    if (lane == 0) { part[t * W_NW + warp] = kw; ksum += kw; }
  }
  wring_end(r, warp);
  Ksum = ksum; Dsum = dsum; Zsum = zsum;
}

struct WideShared {
  bu::Scratch sc;
  double tab[256];
  double bcd[4];
  int bc[4];
  int cnt;
  int row;
};

template <typename T>
__device__ void wide_row(const BatchArgs& BA, const int64_t row_id, unsigned char* dyn, WideShared& sh,
                         unsigned long long pol_keep, unsigned long long pol_drop) {
  const KernelArgs& A = BA.k;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int V = A.V;
  constexpr int VEC = Elem<T>::VEC;
  const T* row = static_cast<const T*>(A.logits) + row_id * A.row_stride;
  RowView<T> rv;
  rv.init(row, V);
  bu::Scratch& sc = sh.sc;
  const double* s_tab = sh.tab;
  uint4* ring = reinterpret_cast<uint4*>(dyn);
  uint32_t* hist = reinterpret_cast<uint32_t*>(dyn + W2_OFF_HIST);
  uint2* zl = reinterpret_cast<uint2*>(dyn + W2_OFF_ZONE);
  unsigned long long* zk = reinterpret_cast<unsigned long long*>(dyn + W2_OFF_ZONE);
  double* ebs = reinterpret_cast<double*>(dyn + W2_OFF_EB);
  double* part = reinterpret_cast<double*>(dyn + W2_OFF_PART);   // [tile][warp] kept mass
  const double QNAN = __longlong_as_double(0x7ff8000000000000ll);
  const int ntiles = (rv.nvec + W_TILE_VECS - 1) / W_TILE_VECS;

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
      for (int i = tid; i < V; i += W_NT) pr[i] = v;
    }
  };
  if (ntiles > W_MAX_TILES) {
    if (tid == 0) hand_to_single(BA, row_id);
    return;
  }

  WRing ring_;
  ring_.base = ring; ring_.src = rv.vbase; ring_.nvec = rv.nvec; ring_.ntiles = ntiles;

  // ---- pass 1: max, min, NaN (from HBM; L2 is asked to keep the row)
  float xmax = -INFINITY, xmin = INFINITY;
  bool nan_seen = false;
  ring_.pol = pol_keep;
  wide_pass1<T>(ring_, rv, tid, xmax, xmin, nan_seen);
  __syncthreads();
  const int anynan = bu::max_i<W_NW>(nan_seen ? 1 : 0, sc, tid);
  xmax = okey_to_float(static_cast<uint32_t>(bu::max_u64<W_NW>(static_cast<unsigned long long>(okey(xmax)), sc, tid)));
  xmin = okey_to_float(static_cast<uint32_t>(bu::min_u64<W_NW>(static_cast<unsigned long long>(okey(xmin)), sc, tid)));
  const float m = scale_t(xmax, Tm);
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
  // every logit of the row has d inside the bucket table's range (a -Inf logit makes this false)
  const bool fast_ok = (scale_t(xmin, Tm) - m > -31.9f);

  // ---- pass 2: count histogram (from L2), bracket of the cut
  float dA = -INFINITY, dB = -INFINITY;    // certainly kept: d >= dA; zone: dB <= d < dA; dropped: d < dB
  if (cut_on) {
    for (int j = tid; j < W_NB; j += W_NT) hist[j] = 0;
    __syncthreads();
    ring_.pol = pol_keep;
    wide_pass2<T>(ring_, rv, tid, hist, m, Tm);
    __syncthreads();
    constexpr int PER = W_NB / W_NT;                         // 4 buckets per thread
    double lo_inc[PER], hi_inc[PER];
    int cb[PER];
    double slo = 0.0, shi = 0.0;
#pragma unroll
    for (int j = 0; j < PER; j++) {
      const int b = tid * PER + j;
      cb[j] = static_cast<int>(hist[b]);
      const double c = static_cast<double>(cb[j]);
      // bucket b holds d in [-(b+.5)/128, -(b-.5)/128]; the last one everything below
      // (masked lanes land there too: their mass bound starts at 0)
      const double elo = (b == W_NB - 1) ? 0.0 : exp_safe(-(b + 0.5f) * 0.0078125f, s_tab) * (1.0 - 1e-7);
      const double ehi = (b == 0) ? 1.0 : fmin(1.0, exp_safe(-(b - 0.5f) * 0.0078125f, s_tab) * (1.0 + 1e-7));
      slo += c * elo; shi += c * ehi;
      lo_inc[j] = slo; hi_inc[j] = shi;
    }
    double ex_lo, ex_hi, tot_lo, tot_hi;
    bu::scan_excl_d2<W_NW>(slo, shi, ex_lo, ex_hi, tot_lo, tot_hi, sc, tid);
    int b1 = W_NB - 1, b2 = W_NB - 1;
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
    bu::min_i2<W_NW>(b1, b2, sc, tid);
    if (b2 < b1) b2 = b1;
    int nz_part = 0;
#pragma unroll
    for (int j = 0; j < PER; j++) {
      const int b = tid * PER + j;
      if (b >= b1 && b <= b2) nz_part += cb[j];
    }
    const int nzone = bu::sum_i<W_NW>(nz_part, sc, tid);
    if (nzone > W_ZCAP + 2 * VEC) {                          // zone larger than the exact list
      if (tid == 0) hand_to_single(BA, row_id);
      return;
    }
    dA = bucket_floor_w(b1 - 1);
    dB = bucket_floor_w(b2);
  }
  stamp(1);

  // ---- pass 3: exponentials (last use of the row: evict-first). Inside a tile each warp owns a
  // contiguous piece; eight logits are in flight per lane.
  if (fast_ok) ebs[tid] = __ldg(BA.eb_table + tid);          // W_NT == NB1
  if (tid == 0) sh.cnt = 0;
  __syncthreads();
  constexpr int PIECE = W_TILE_VECS / W_NW;                  // 64 vectors per warp and tile
  double Ksum = 0.0, Dsum = 0.0, Zsum = 0.0;                 // lane 0 of each warp: its pieces; others: partial
  ring_.pol = pol_drop;
#define GS_P3(F, O, C) wide_pass3<T, F, O, C>(ring_, rv, tid, m, Tm, dA, dB, ebs, s_tab, part, zl, &sh.cnt, Ksum, Dsum, Zsum)
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
  double Ktot = Ksum, Dtot = Dsum, Ztot = Zsum;
  bu::sum_d3<W_NW>(Ktot, Dtot, Ztot, sc, tid);
  const int nz = sh.cnt;
  stamp(2);
  if (nz > W_ZCAP) {
    if (tid == 0) hand_to_single(BA, row_id);
    return;
  }
  const double S = Ktot + Ztot + Dtot;
  dbg.sum_exp = S;
  const int npiece = ntiles * W_NW;

  // ---- exact cut inside the zone by weighted selection
  unsigned long long cut_key = 0ull;       // zone entries are kept when key < cut_key, or == with cut_incl
  int cut_incl = 0;
  bool bad = false;
  if (cut_on && nz > 0) {
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
    double* sm = reinterpret_cast<double*>(hist);            // [NSUB] mass per sub-bucket
    int* scn = reinterpret_cast<int*>(hist) + 2 * NSUB;      // [NSUB] count per sub-bucket
    unsigned long long lo = ~0ull, hi = 0ull;
    for (int j = tid; j < nz; j += W_NT) { const unsigned long long k = zk[j]; lo = k < lo ? k : lo; hi = k > hi ? k : hi; }
    lo = bu::min_u64<W_NW>(lo, sc, tid);
    hi = bu::max_u64<W_NW>(hi, sc, tid);
    double gbase = Ktot;                                     // Ktot + mass of keys below lo; never crossed
    int inrange = nz;
    bool all_in = false;
    for (int iter = 0; iter < 8 && inrange > 32 && !bad && !all_in; iter++) {
      const unsigned long long span = hi - lo;
      int shf = 0;
      while (shf < 63 && (span >> shf) >= static_cast<unsigned long long>(NSUB)) shf++;
      __syncthreads();
      sm[tid] = 0.0; scn[tid] = 0;                           // W_NT == NSUB
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
      const int first = (scn[tid] > 0 && crossed(gbase + exm + mine)) ? tid : NSUB;
      const int sbx = bu::min_i<W_NW>(first, sc, tid);
      if (sbx == NSUB) { all_in = true; break; }
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
      if (mode == 1 && Dtot > 0.0) bad = true;               // the bracket promised a crossing
    }
    if (!bad && !all_in) {
      if (fabs(g_at / S - plim) <= 1e-12 || fabs(g_before / S - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
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
        atomicAdd(&part[(v / W_TILE_VECS) * W_NW + (v % W_TILE_VECS) / PIECE], exp_safe(zone_key_d(k), s_tab));
      }
    }
    __syncthreads();
  }
  // ---- kept mass and the piece that holds the drawn token: prefix over the pieces in row order
  constexpr int PPER = (W_MAX_TILES * W_NW) / W_NT;          // 2 pieces per thread
  double pm[PPER];
  double psum = 0.0;
#pragma unroll
  for (int q = 0; q < PPER; q++) { const int pi = tid * PPER + q; pm[q] = (pi < npiece) ? part[pi] : 0.0; psum += pm[q]; }
  double Re;
  const double pex = bu::scan_excl_d<W_NW>(psum, Re, sc, tid);
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
    if (d < dA) {
      if (!(d >= dB)) return 0.0;
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
  // ---- draw (generate.go:231-239): u < prefix/Re is tested as u*Re < prefix
  const double tgt = u * Re;
  int psel = 0x7fffffff;
  {
    double run = pex;
#pragma unroll
    for (int q = 0; q < PPER; q++) {
      run += pm[q];
      if (psel == 0x7fffffff && tid * PPER + q < npiece && tgt < run) psel = tid * PPER + q;
    }
  }
  psel = bu::min_i<W_NW>(psel, sc, tid);
  if (psel != 0x7fffffff && tid == psel / PPER) {
    double b = pex;
    for (int q = 0; q < psel % PPER; q++) b += pm[q];
    sh.bcd[0] = b;
  }
  __syncthreads();
  int id = -1;
  double edge_lo = 0.0, edge_hi = 0.0;
  double run_end = (psel != 0x7fffffff) ? sh.bcd[0] : Re;
  if (psel != 0x7fffffff) {
    // walk pieces from the selected one (rounding can push the crossing into the next piece)
    for (int pi = psel; pi < npiece && id < 0; pi++) {       // uniform; normally one trip
      const int vbase_p = (pi / W_NW) * W_TILE_VECS + (pi % W_NW) * PIECE;
      const int j = vbase_p + tid;
      double em[VEC];
      double tsum = 0.0;
#pragma unroll
      for (int c = 0; c < VEC; c++) em[c] = 0.0;
      int i0 = 0;
      if (tid < PIECE && j < rv.nvec) {
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
  stamp(4);
  write_row(id, flags);
}

template <typename T>
__global__ void __launch_bounds__(W_NT, 1) wide_rows_kernel(BatchArgs BA) {
  extern __shared__ __align__(16) unsigned char dyn[];
  __shared__ WideShared sh;
  if (threadIdx.x < 256) sh.tab[threadIdx.x] = BA.k.exp_table[threadIdx.x];
  unsigned long long pol_keep, pol_drop;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol_keep));
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol_drop));
  const int n = BA.hdr[1];
  for (;;) {
    __syncthreads();
    if (threadIdx.x == 0) {
      const int w = atomicAdd(&BA.hdr[3], 1);
      sh.row = (w < n) ? BA.list_wide[w] : -1;
    }
    __syncthreads();
    const int row = sh.row;
    if (row < 0) break;
    wide_row<T>(BA, row, dyn, sh, pol_keep, pol_drop);
  }
}

}  // namespace gs
