// Large-batch kernels: rows are first sorted by what they need, then two
// persistent kernels pull rows from work lists.
//
//   row_kind               what a row needs, from its config alone: greedy and
//                          top-k <= 256 rows are "narrow", top-k-off rows "wide",
//                          top-k above 256 goes to the single-CTA kernel. Each
//                          persistent kernel walks ALL rows with its own atomic
//                          cursor and takes the rows of its kind, so no separate
//                          classification launch and no per-kind lists exist.
//   narrow_rows_kernel     256 threads, four CTAs per SM. One streaming pass per
//                          row: the first 4096 logits give a threshold (k-th
//                          largest of the 256 per-thread maxima, a lower bound
//                          of the k-th largest logit); then every warp walks
//                          its own span of the rest (row_stream.cuh) and appends
//                          the few logits above the threshold, with no barrier
//                          per step; the list is pruned to the exact k-th
//                          largest when a warp sees it half full. Everything
//                          after the pass happens on a few hundred candidates
//                          in shared memory.
//   wide_rows_kernel       (sample_wide.cuh) rows whose softmax runs over the
//                          whole vocabulary.
//
// Row semantics: model/generate.go:134-260 (mode A), model/qwen/generate.go:
// 77-181 (mode B). Rows a kernel cannot finish (candidate or zone lists that
// outgrow their buffers) are appended to the single-CTA kernel's list.
#pragma once

#include "block_util.cuh"
#include "row_stream.cuh"
#include "sample_cluster.cuh"

namespace gs {

constexpr int N_NT = 256;               // narrow kernel threads
constexpr int N_NW = N_NT / 32;
constexpr int N_CTAS_PER_SM = 5;        // 5 x 256 threads of at most 48 registers; 5 x 45 KB of shared memory
constexpr int N_CAP = 1536;             // candidate capacity (entries of 8 B)
constexpr int N_KEEP = 768;             // a prune must get below this
constexpr int N_WARM_ELEMS = 4096;      // logits of the warm-up chunk
constexpr int N_HITS = 1536;            // hit list: positions of lane-steps that hold a candidate (4 B each)
// Dynamic shared memory of the narrow kernel, 42 KB: [0, 24 KB) the ring the stream is staged
// through; its upper 16 KB double as the work arrays of the phases that run while no copy is in
// flight (prune, finish); then the candidate list and the hit list.
constexpr int N_RING_BYTES = 24576;
constexpr int N_WORK_OFF = 8192;
constexpr int N_CAND_OFF = N_RING_BYTES;
constexpr int N_HITS_OFF = N_CAND_OFF + N_CAP * 8;
constexpr int N_DYN_BYTES = N_HITS_OFF + N_HITS * 4;
static_assert(N_WORK_OFF + 16384 <= N_CAND_OFF, "work arrays end where the candidate list starts");


// Vocab-sharded sampling: what one rank knows about one row of its column slice. cand holds every
// local logit at or above the local k-th largest (global indices); the global kept set is a
// subset of the union of the ranks' lists, because the global k-th largest is at least every
// local one.
constexpr int VS_CAND = 128;
constexpr uint32_t VS_NONFINITE = 1u, VS_BAD_CFG = 2u, VS_OVERFLOW = 4u, VS_UNSUPPORTED = 8u, VS_NAN_AT_0 = 16u;
struct VsRecord {
  float xmax;              // largest local logit (not yet divided by the temperature)
  int32_t n;               // entries in cand
  uint32_t flags;          // VS_*
  int32_t pad;
  uint2 cand[VS_CAND];     // (logit bits, global index)
};
static_assert(sizeof(VsRecord) == 16 + 8 * VS_CAND, "record layout is part of the C ABI");
// Record `row` of an array whose records hold `cand` candidates each (16 + 8 * cand bytes apart).
__device__ __forceinline__ VsRecord& vs_record(void* base, int64_t row, int cand) {
  return *reinterpret_cast<VsRecord*>(static_cast<unsigned char*>(base) + row * (16 + 8 * static_cast<int64_t>(cand)));
}
__device__ __forceinline__ const VsRecord& vs_record(const void* base, int64_t row, int cand) {
  return *reinterpret_cast<const VsRecord*>(static_cast<const unsigned char*>(base) + row * (16 + 8 * static_cast<int64_t>(cand)));
}

struct BatchArgs {
  KernelArgs k;
  const double* eb_table;   // 1024 doubles: exp(-b/32)
  int32_t* hdr;             // [2] narrow kernel's row cursor, [3] wide kernel's row cursor
  int32_t* list_single;     // [0] = count, [1..] rows for the single-CTA kernel
  int64_t B;
};

// 0: narrow kernel, 1: wide kernel, 2: single-CTA kernel, 3: nobody (the row's sequence has ended)
__device__ __forceinline__ int row_kind(const KernelArgs& A, int64_t b) {
  if (A.row_done && A.row_done[b] != 0) return 3;
  if (A.force_greedy || A.vs_records || A.tk_k > 0) return 0;
  const RowCfg c = A.cfgs[b];
  const float T = c.temperature;
  if (T == 0.0f || !(T > 0.0f) || !(T < INFINITY)) return 0;   // greedy, or a bad temperature (reported by the narrow kernel)
  const int topk = (c.top_k > 0 && c.top_k < A.V) ? c.top_k : 0;
  return (topk == 0) ? 1 : (topk <= KFAST ? 0 : 2);
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
  dbg.reserved[4] = static_cast<uint32_t>(clock64());       // with reserved[3]: the row's whole time on its CTA
  write_row(id, flags);
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

template <typename T>
__device__ __forceinline__ uint4 mask_edges(const RowView<T>& rv, int v, uint4 raw);

// ---------------------------------------------------------------------------
// narrow: greedy and top-k <= 256 rows, one streaming pass each
// ---------------------------------------------------------------------------
template <typename T>
__device__ void narrow_row(const BatchArgs& BA, const int64_t row_id, unsigned char* dyn, bu::Scratch& sc,
                           uint32_t* s_sel, int* s_bc, double* s_bcd, int* s_cnt, int* s_hcnt, float* s_thr, int* s_flag,
                           const bool allow_tight, bool& redo) {
  const KernelArgs& A = BA.k;
  redo = false;
  const int tid = threadIdx.x;
  const int V = A.V;
  constexpr int VEC = Elem<T>::VEC;
  constexpr int WARM_VECS = N_WARM_ELEMS / VEC;
  const T* row = static_cast<const T*>(A.logits) + row_id * A.row_stride;
  RowView<T> rv;
  rv.init(row, V);
  unsigned char* work = dyn + N_WORK_OFF;                    // 16 KB of work arrays (prune, finish)
  uint2* cand = reinterpret_cast<uint2*>(dyn + N_CAND_OFF);  // N_CAP entries
  int* hits = reinterpret_cast<int*>(dyn + N_HITS_OFF);      // N_HITS entries
  const double QNAN = __longlong_as_double(0x7ff8000000000000ll);

  RowCfg cfg;
  if (A.force_greedy) { cfg.temperature = 0.f; cfg.top_k = 0; cfg.top_p = 0.f; cfg.topp_mode = 0; }
  else if (A.tk_k > 0) { cfg.temperature = 1.f; cfg.top_k = A.tk_k; cfg.top_p = 0.f; cfg.topp_mode = 0; }
  else cfg = A.cfgs[row_id];
  const float Tm = cfg.temperature;
  RowDebug dbg;
  dbg.sum_exp = 0; dbg.resum = 1.0; dbg.edge_lo = 0; dbg.edge_hi = 0; dbg.kept = 0;
  dbg.max_scaled = 0; dbg.threshold = __int_as_float(0x7fc00000); dbg.path = 0;
  for (int q = 0; q < 8; q++) dbg.reserved[q] = 0;
  long long tprev = clock64();
  dbg.reserved[3] = static_cast<uint32_t>(tprev);
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
    // a NaN at index 0 is never beaten (index 0 of the whole row: a later slice has no such column)
    if (x0 != x0 && (!A.vs_records || A.vs_col_offset == 0)) id = 0;
    if (A.vs_records) {                                      // vocab-sharded: this slice's champion
      if (tid == 0) {
        VsRecord& rec = vs_record(A.vs_records, row_id, A.vs_cand);
        float xid = 0.f;
        rv.visit(rv.vec_of(id), [&](float x, int i) { if (i == id) xid = x; });
        rec.xmax = xid; rec.n = 1; rec.pad = 0;
        rec.flags = (x0 != x0 && A.vs_col_offset == 0) ? VS_NAN_AT_0 : 0u;
        rec.cand[0] = make_uint2(__float_as_uint(xid), static_cast<uint32_t>(id + A.vs_col_offset));
      }
      return;
    }
    fill_probs_row(0.0);
    __syncthreads();
    if (A.out_probs && tid == 0) A.out_probs[row_id * static_cast<int64_t>(V) + id] = 1.0;
    dbg.kept = 1;
    write_row(id, 0u);
    return;
  }
  auto vs_flag_only = [&](uint32_t fl) {
    if (tid == 0) {
      VsRecord& rec = vs_record(A.vs_records, row_id, A.vs_cand);
      rec.xmax = 0.f; rec.n = 0; rec.flags = fl; rec.pad = 0;
    }
  };
  if (!(Tm > 0.0f) || !(Tm < INFINITY)) {
    if (A.vs_records) { vs_flag_only(VS_BAD_CFG); return; }
    fill_probs_row(QNAN);
    write_row(-1, FLAG_BAD_CFG);
    return;
  }
  if (A.vs_records && !(cfg.top_k > 0 && cfg.top_k <= A.vs_cand)) {   // the merge needs a top-k to bound the lists
    vs_flag_only(VS_UNSUPPORTED);
    return;
  }
  const int topk = cfg.top_k;                                // 0 < top_k <= KFAST, < V (classified)
  const bool topp_on = (cfg.top_p > 0.0f && cfg.top_p < 1.0f);
  const int mode = cfg.topp_mode;
  const double plim = (mode == 0) ? static_cast<double>(cfg.top_p) * 1.5 : static_cast<double>(cfg.top_p);
  dbg.path = 1;

  // ---- warm-up chunk: 16 logits per thread, kept in registers; one running maximum per thread
  float xmax = -INFINITY, xmin = INFINITY;
  bool nan_seen = false;
  if (tid == 0) { *s_cnt = 0; *s_hcnt = 0; *s_flag = 0; }
  const int warm = min(rv.nvec, WARM_VECS);
  constexpr int G = WARM_VECS / N_NT;
  uint4 wr[G];                                               // logits outside the row come back as -Inf
  constexpr uint32_t NEG_INF_BITS = (sizeof(T) == 4) ? 0xff800000u : 0xff80ff80u;
#pragma unroll
  for (int g = 0; g < G; g++) {
    const int v = g * N_NT + tid;
    wr[g] = make_uint4(NEG_INF_BITS, NEG_INF_BITS, NEG_INF_BITS, NEG_INF_BITS);
    if (v < warm) wr[g] = load_masked(rv, v, xmax, xmin, nan_seen);
  }
  // ---- the rest of the row is streamed by warps, every warp over its own span, eight logits per
  // lane and step (two 16-byte vectors of f32, one of bf16). The vectors are staged through a ring
  // in shared memory by asynchronous 16-byte copies: a thread copies what it will consume itself
  // (no barrier: it only waits for its own copy groups), NQ steps ahead. Loads into registers
  // cannot run that far ahead: in a rolled loop they share one scoreboard, so waiting for the
  // oldest waits for the newest too. The first copies go out now and fly during the selection.
  constexpr int EPI = 8 / VEC, SV = 32 * EPI;
  constexpr int NQ = N_RING_BYTES / (EPI * N_NT * 16);       // stages: 6 of bf16, 3 of f32
  const int lane = tid & 31, warp = tid >> 5;
  const int rest = max(rv.nvec - warm, 0);
  const int span = (((rest + N_NW - 1) / N_NW + SV - 1) / SV) * SV;
  const WSpan sp = make_span<T>(rv, warm + warp * span, span, lane);
  unsigned long long pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  const uint32_t ring_addr = smem_addr(dyn) + static_cast<uint32_t>(tid * 16);
  const uint4* ring = reinterpret_cast<const uint4*>(dyn) + tid;
  // the copies of step q (none past the warp's last step: an empty group keeps the count right)
  auto ring_issue = [&](int q) {
    if (q < sp.nst) {
      const uint32_t dst = ring_addr + static_cast<uint32_t>((q % NQ) * EPI * N_NT * 16);
      const int o = q * SV;
#pragma unroll
      for (int h = 0; h < EPI; h++)
        asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;"
                     :: "r"(dst + h * N_NT * 16), "l"(sp.lane_src + min(o + 32 * h, sp.omax)), "l"(pol) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
#pragma unroll
  for (int q = 0; q < NQ; q++) ring_issue(q);
  // Threshold from the 256 per-thread maxima of the chunk: every warp sorts its 32 maxima with
  // shuffles, and every thread then finds the place of its own among all 256 by a binary search
  // in each of the other warps' sorted lists (two barriers; a radix select over so few keys costs
  // several rounds of barriers and of shared atomics that all hit the same few bins, and counting
  // all 256 against each other three times the instructions).
  //  * The top_k-th largest maximum is a BOUND: top_k threads each hold a logit at or above it, so
  //    the top_k-th largest logit of the row is at or above it.
  //  * The r-th largest maximum with r < top_k, r chosen so that about four times top_k logits of
  //    the whole row are expected above it, is an ESTIMATE (`tight`). If the row ends with at
  //    least top_k candidates, its top_k-th largest is among them and nothing was lost; if not
  //    (the chunk was not typical of the row), the row is redone: by the single-CTA kernel when it
  //    is a sampling row, by this kernel without the estimate (`redo`) when it is a TopK row or a
  //    vocab-sharded slice, which that kernel does not serve.
  // Either way the threshold is lowered to the edge of its class of equal quotients x / T (what
  // ties with the k-th largest after the division is then collected too), and it is never -Inf:
  // a -Inf logit has probability 0 whether or not top-k keeps it, so it is never a candidate (a
  // masked vocabulary would otherwise flood the list with ties at -Inf); a row with fewer than
  // top_k finite logits simply ends with fewer candidates.
  constexpr float LOWEST = -3.402823466e+38f;
  float thr = LOWEST;
  bool tight = false;
  {
    int rank = topk;
    if (allow_tight && rv.nvec > warm) {
      const long long welems = static_cast<long long>(warm) * VEC;
      const int r = static_cast<int>((4ll * topk * welems + V - 1) / V) + 4;
      if (r < topk) { rank = r; tight = true; }
    }
    uint32_t key = okey(xmax);
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {                      // bitonic network, descending by lane
#pragma unroll
      for (int j = k >> 1; j > 0; j >>= 1) {
        const uint32_t other = __shfl_xor_sync(FULL, key, j);
        const bool take_max = ((lane & j) == 0) == ((lane & k) == 0);
        key = take_max ? max(key, other) : min(key, other);
      }
    }
    s_sel[tid] = key;                                        // list of warp w: s_sel[32 w .. 32 w + 31]
    if (tid == 0) *s_thr = LOWEST;
    __syncthreads();
    // place of (key, warp, lane) in the order "larger key first, then lower warp, then lower lane"
    int before = lane;
#pragma unroll
    for (int w = 0; w < N_NW; w++) {
      if (w == warp) continue;
      const uint32_t* L = s_sel + 32 * w;
      const bool ties_first = w < warp;                      // equal keys of a lower warp order before mine
      int c = 0;
#pragma unroll
      for (int step = 16; step >= 1; step >>= 1) {
        const uint32_t v = L[c + step - 1];
        if (v > key || (ties_first && v == key)) c += step;
      }
      const uint32_t v = L[c];
      if (v > key || (ties_first && v == key)) c++;
      before += c;
    }
    if (before == rank - 1 && key > 0x007fffffu)             // at or below -Inf: keep everything
      *s_thr = fmaxf(quotient_class_floor(okey_to_float(key), Tm), LOWEST);
    __syncthreads();
    thr = *s_thr;
    if (thr == LOWEST) tight = false;
  }
  // candidates of the warm-up chunk (a logit outside the row is -Inf there: below every threshold)
  auto warm_candidates = [&]() {
#pragma unroll
    for (int g = 0; g < G; g++) {
      float x[VEC];
      Elem<T>::unpack(wr[g], x);
      const int i0 = (g * N_NT + tid) * VEC - rv.shift;
#pragma unroll
      for (int c = 0; c < VEC; c++) {
        if (x[c] >= thr) {
          const int slot = atomicAdd(s_cnt, 1);
          if (slot < N_CAP) cand[slot] = make_uint2(__float_as_uint(x[c]), static_cast<uint32_t>(i0 + c));
        }
      }
    }
  };
  warm_candidates();
  __syncthreads();
  if (*s_cnt > N_CAP) {                                      // uniform
    // A large top_k makes the bound from the maxima a weak one (the top_k-th largest of 256
    // maxima is near the smallest of them), and more of the chunk passed it than the list holds.
    // The exact top_k-th largest of the chunk is a bound too; more than top_k pass it only by ties.
    const uint32_t kkey = bu::select_kth_of<N_NT>([&](auto&& f) {
#pragma unroll
      for (int g = 0; g < G; g++) {
        float x[VEC];
        Elem<T>::unpack(wr[g], x);
#pragma unroll
        for (int c = 0; c < VEC; c++) f(okey(x[c]));
      }
    }, topk, 0u, 0xffffffffu, s_sel, s_bc, tid);
    if (tid == 0) { *s_thr = fmaxf(quotient_class_floor(okey_to_float(kkey), Tm), LOWEST); *s_cnt = 0; }
    __syncthreads();
    thr = fmaxf(thr, *s_thr);
    warm_candidates();                                       // a list that ties overflow again ends the row below
  }
  stamp(0);
  bool giveup = false;
  // exact k-th largest of the list -> threshold; keepers move through the chunk buffer
  // (every entry is at or above thr; hi_key: a key no entry exceeds)
  auto prune = [&](int cnt, uint32_t hi_key) -> int {
    if (cnt <= topk) return cnt;
    const uint32_t kkey = bu::select_kth<N_NT>(cand, cnt, topk, s_sel, s_bc, tid, okey(thr), hi_key);
    if (tid == 0) { *s_thr = quotient_class_floor(okey_to_float(kkey), Tm); *s_cnt = 0; }
    __syncthreads();
    thr = *s_thr;                                            // finite: the list holds finite logits only
    uint2* tmp = reinterpret_cast<uint2*>(work);             // 2048 entries
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
  // ---- the stream. No barrier per step. A lane whose eight logits hold one at or above the
  // threshold only notes WHERE (its vector index, 4 bytes in the hit list): unpacking and
  // appending on the spot would cost the whole warp some hundred instructions on nearly every
  // other step. The noted vectors are read again (from L2, or HBM at worst) by all threads at once
  // after the stream, or when the hit list fills: a warp that sees it past H_TRIGGER raises
  // *s_flag; every warp looks at the flag before each step and comes to the barrier below, where
  // the hits are resolved into the candidate list and that is pruned to the exact k-th largest;
  // then the warps walk on. Between the flag going up and a warp seeing it, each of its lanes
  // notes at most one more hit: the room above H_TRIGGER. Steps that hold the row's edges (at
  // most two per warp) append their logits directly, masked by index.
  constexpr int H_TRIGGER = N_HITS - N_NT;
  volatile int* vflag = s_flag;
  float run = xmax;                                          // NaN-propagating running maximum of this thread
  int st = 0;
  // hits -> candidates: every thread re-reads the vectors of its share of the noted lane-steps
  auto resolve_hits = [&](int first_hit, int nh) {
    for (int j = first_hit + tid; j < first_hit + nh; j += N_NT) {
      const int gv = hits[j];
#pragma unroll
      for (int h = 0; h < 8 / VEC; h++) {
        const int g = gv + 32 * h;
        float x[VEC];
        Elem<T>::unpack(__ldg(rv.vbase + g), x);
        const int i0 = g * VEC - rv.shift;
#pragma unroll
        for (int c = 0; c < VEC; c++) {
          if (x[c] >= thr) {                                 // clean steps only: every index is inside the row
            const int slot = atomicAdd(s_cnt, 1);
            if (slot < N_CAP) cand[slot] = make_uint2(__float_as_uint(x[c]), static_cast<uint32_t>(i0 + c));
          }
        }
      }
    }
  };
  __syncthreads();
  for (;;) {                                                 // uniform: one trip per prune, plus one
    {
      // The steady part: steps whose own vectors and whose refill (step st + NQ) are clean, so
      // that no address needs a clamp and no logit a mask. The ring slot, the global source and
      // the vector index advance by additions (the general loop below pays a division by NQ, two
      // multiplications and two clamps per step, about as many instructions as the step's work).
      constexpr uint32_t STAGE = EPI * N_NT * 16;
      const int steady_end = sp.clean_hi - NQ;
      uint32_t slot_off = static_cast<uint32_t>(st % NQ) * STAGE;
      const uint4* gsrc = sp.lane_src + static_cast<int64_t>(st + NQ) * SV;
      int gv = sp.first + st * SV + lane;
#pragma unroll 1
      while (st < steady_end && *vflag == 0) {
        asm volatile("cp.async.wait_group %0;" :: "n"(NQ - 1) : "memory");   // the copies of step st have landed
        const uint4* rd = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(ring) + slot_off);
        const uint4 ca = rd[0];
        const uint4 cb = (EPI == 2) ? rd[N_NT] : ca;
        const float hi8 = step_max_nan<T>(ca, cb);
        run = maxnan(run, hi8);
        if (hi8 >= thr) {
          const int slot = atomicAdd(s_hcnt, 1);
          hits[min(slot, N_HITS - 1)] = gv;
          if (slot >= H_TRIGGER) *vflag = 1;
        }
#pragma unroll
        for (int h = 0; h < EPI; h++)
          asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;"
                       :: "r"(ring_addr + slot_off + h * N_NT * 16), "l"(gsrc + 32 * h), "l"(pol) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
        slot_off = (slot_off + STAGE == NQ * STAGE) ? 0u : slot_off + STAGE;
        gsrc += SV;
        gv += SV;
        st++;
      }
    }
#pragma unroll 1
    while (st < sp.nst && *vflag == 0) {
      asm volatile("cp.async.wait_group %0;" :: "n"(NQ - 1) : "memory");   // the copies of step st have landed
      const uint4 ca = ring[(st % NQ) * EPI * N_NT];
      const uint4 cb = (EPI == 2) ? ring[(st % NQ) * EPI * N_NT + N_NT] : ca;
      if (st < sp.clean_hi) {                                // no logit outside the row in this step
        const float hi8 = step_max_nan<T>(ca, cb);
        run = maxnan(run, hi8);
        if (hi8 >= thr) {
          const int slot = atomicAdd(s_hcnt, 1);
          hits[min(slot, N_HITS - 1)] = sp.first + st * SV + lane;   // never past H_TRIGGER + N_NT: see above
          if (slot >= H_TRIGGER) *vflag = 1;
        }
      } else {                                               // the row's last vector, or past the end
        float x[8];
        if (VEC == 4) { Elem<T>::unpack(ca, x); Elem<T>::unpack(cb, x + 4 * (8 / VEC - 1)); }
        else Elem<T>::unpack(ca, x);
        const int gv = sp.first + st * SV + lane;
#pragma unroll
        for (int c = 0; c < 8; c++) {
          const int g = gv + 32 * (c / VEC);
          const int i = g * VEC - rv.shift + (c % VEC);
          if (g < rv.nvec && i < V) {
            run = maxnan(run, x[c]);
            if (x[c] >= thr) {
              const int slot = atomicAdd(s_cnt, 1);
              if (slot < N_CAP) cand[slot] = make_uint2(__float_as_uint(x[c]), static_cast<uint32_t>(i));
            }
          }
        }
      }
      ring_issue(st + NQ);                                   // into the slot just read
      st++;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");     // the ring's memory is about to serve as work arrays
    const int more = __syncthreads_or((st < sp.nst) ? 1 : 0);
    const int full = __syncthreads_or(*vflag);               // every thread reads it before anyone can raise it again
    if (full || !more) {
      const int nh = min(*s_hcnt, N_HITS);                   // never above N_HITS: the trigger's room
      __syncthreads();
      if (tid == 0) { *s_flag = 0; *s_hcnt = 0; }
      // A hit stands for up to eight candidates, so the hits are resolved in portions that fit the
      // candidate list, with a prune (which raises the threshold) between them. Ordinarily one
      // portion takes them all; a row whose threshold is far too low (a start well below the rest
      // of the row) notes a hit in every lane-step and needs a few.
      int done = 0;
      bool careful = false;
      for (;;) {                                             // uniform
        const int c0 = *s_cnt;
        __syncthreads();
        if (c0 > N_CAP) { giveup = true; break; }            // entries were dropped
        // first all at once, if they fit at one candidate per hit (nearly always so); taken back
        // when the list overflowed, and then in portions that fit at eight per hit
        const int take = min(nh - done, (N_CAP - c0) / (careful ? 8 : 1));
        resolve_hits(done, take);
        __syncthreads();
        if (!careful && *s_cnt > N_CAP) {
          __syncthreads();
          if (tid == 0) *s_cnt = c0;
          careful = true;
          __syncthreads();
          continue;
        }
        done += take;
        if (done >= nh && !full) break;
        const int cnt = prune(*s_cnt, 0xffffffffu);
        if (cnt > N_KEEP) { giveup = true; break; }          // ties at the threshold fill the buffer
        if (done >= nh) break;
      }
      if (giveup) break;
    }
    if (!more) break;
    __syncthreads();                                         // the work arrays are done with: refill the ring
#pragma unroll
    for (int q = 0; q < NQ; q++) ring_issue(st + q);
  }
  nan_seen |= (run != run);
  xmax = run;
  stamp(1);
  dbg.reserved[5] = static_cast<uint32_t>(*s_cnt);
  int nk = 0;
  if (!giveup && *s_cnt > N_CAP) giveup = true;
  if (!giveup && tight && *s_cnt < topk) {                   // the estimated threshold was too tight for this row
    if (A.vs_records || A.tk_k > 0) { redo = true; return; } // uniform: *s_cnt is read after the loop's last barrier
    giveup = true;
  }
  const int anynan = bu::max_i<N_NW>(nan_seen ? 1 : 0, sc, tid);
  xmax = okey_to_float(static_cast<uint32_t>(bu::max_u64<N_NW>(static_cast<unsigned long long>(okey(xmax)), sc, tid)));
  if (!giveup) {
    // the row's maximum bounds the list from above, unless a thread's maximum was lost to a NaN
    nk = prune(*s_cnt, anynan ? 0xffffffffu : okey(xmax));
    if (nk > KEEP_MAX) giveup = true;                        // long run of ties at the threshold
  }
  const float m = scale_t(xmax, Tm);
  dbg.max_scaled = m;
  // A NaN anywhere, or an infinite maximum, makes the softmax sum NaN upstream
  // (generate.go:173-181): every comparison of the walk fails, result n-1 (:239).
  if (A.tk_k > 0) {
    // TopK op (index_ops.go:153-190): the k largest, descending, equal values by ascending index.
    // NaNs order last here (the reference's comparator leaves them unspecified).
    float* ov = A.tk_values + row_id * static_cast<int64_t>(topk);
    int32_t* oi = A.tk_indices + row_id * static_cast<int64_t>(topk);
    if (giveup || nk < topk) {                               // more than 512 logits tie at the k-th value, or it is -Inf
      for (int j = tid; j < topk; j += N_NT) { ov[j] = __int_as_float(0x7fc00000); oi[j] = -1; }
      if (tid == 0 && A.out_flags) A.out_flags[row_id] = FLAG_INTERNAL;
      return;
    }
    for (int j = tid; j < nk; j += N_NT) {
      const uint32_t kj = okey(__uint_as_float(cand[j].x)), ij = cand[j].y;
      int r = 0;
      for (int l = 0; l < nk; l++) {
        const uint32_t kl = okey(__uint_as_float(cand[l].x));
        r += (kl > kj || (kl == kj && cand[l].y < ij)) ? 1 : 0;
      }
      if (r < topk) { ov[r] = __uint_as_float(cand[j].x); oi[r] = static_cast<int32_t>(ij); }
    }
    if (tid == 0 && A.out_flags) A.out_flags[row_id] = 0u;
    return;
  }
  if (A.vs_records) {                                        // vocab-sharded: hand the list over instead of drawing
    VsRecord& rec = vs_record(A.vs_records, row_id, A.vs_cand);
    uint32_t fl = 0u;
    // a slice of -Inf only (a masked part of the vocabulary) is no verdict on the row: the merge
    // decides that from all slices; a slice given up early was not read to its end
    if (!giveup && (anynan || m == INFINITY || m != m)) fl |= VS_NONFINITE;
    if (giveup || nk > A.vs_cand) fl |= VS_OVERFLOW;
    const int nout = (fl == 0u) ? nk : 0;
    if (tid == 0) { rec.xmax = xmax; rec.n = nout; rec.flags = fl; rec.pad = 0; }
    for (int j = tid; j < nout; j += N_NT) rec.cand[j] = make_uint2(cand[j].x, cand[j].y + static_cast<uint32_t>(A.vs_col_offset));
    return;
  }
  if (giveup) {                                              // before any verdict on the row: it may not have been read to its end
    if (tid == 0) hand_to_single(BA, row_id);
    return;
  }
  if (anynan || !(fabsf(m) < INFINITY)) {
    fill_probs_row(QNAN);
    dbg.sum_exp = QNAN;
    write_row(V - 1, FLAG_NONFINITE | FLAG_FALLBACK);
    return;
  }
  stamp(2);
  finish_small_set<N_NT>(A, row_id, cand, nk, m, Tm, topp_on, mode, plim, A.uniforms[row_id],
                         work, sc, s_bcd, dbg, 0u);
}

template <typename T>
__global__ void __launch_bounds__(N_NT, N_CTAS_PER_SM) narrow_rows_kernel(BatchArgs BA) {
  extern __shared__ __align__(16) unsigned char dyn[];
  __shared__ bu::Scratch sc;
  __shared__ uint32_t s_sel[256];
  __shared__ int s_bc[4];
  __shared__ double s_bcd[4];
  __shared__ int s_cnt;
  __shared__ int s_hcnt;
  __shared__ float s_thr;
  __shared__ int s_flag;
  __shared__ int s_row;
  for (;;) {
    __syncthreads();
    if (threadIdx.x == 0) {
      // next row of this kernel's kind; rows for the single-CTA kernel are handed over here.
      // (Drawing the ticket ahead - at the start of the current row, or when its stream has ended,
      // with an L2 prefetch of the next row's start - was measured: the first binds the rows of a
      // last, partial wave to CTAs before it is known which are free first and costs a third of
      // the step; the second gains nothing.)
      int w;
      for (;;) {
        w = atomicAdd(&BA.hdr[2], 1);
        if (w >= BA.B) { w = -1; break; }
        const int kind = row_kind(BA.k, w);
        if (kind == 0) break;
        if (kind == 2) hand_to_single(BA, w);
      }
      s_row = w;
    }
    __syncthreads();
    const int row = s_row;
    if (row < 0) break;
    bool redo, allow_tight = true;
    for (;;) {                                               // at most twice: the second time without the estimate
      narrow_row<T>(BA, row, dyn, sc, s_sel, s_bc, s_bcd, &s_cnt, &s_hcnt, &s_thr, &s_flag, allow_tight, redo);
      if (!redo) break;
      allow_tight = false;
      __syncthreads();
    }
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


}  // namespace gs
