// Large-batch kernels: rows are first sorted by what they need, then two
// persistent kernels pull rows from work lists.
//
//   row_kind               what a row needs, from its config alone: greedy and
//                          top-k <= 256 rows are "narrow", top-k-off rows "wide",
//                          top-k above 256 goes to the single-CTA kernel. Each
//                          persistent kernel walks ALL rows with its own atomic
//                          cursor and takes the rows of its kind, so no separate
//                          classification launch and no per-kind lists exist.
//   narrow_rows_kernel     (sample_narrow.cuh, two instances: 256 threads x five CTAs per SM,
//                          128 threads x eight). One streaming pass per row: the first
//                          16 logits per thread give a threshold (from the per-thread
//                          maxima: a lower bound of the k-th largest logit, or a tighter
//                          estimate that is checked at the row's end); then every warp
//                          walks its own span of the rest, staged through a ring of
//                          asynchronous copies in shared memory, and only notes where
//                          a logit reaches the threshold; the noted vectors are read
//                          again after the stream, and everything from there on happens
//                          on a few hundred candidates in shared memory.
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

// Vocab-sharded sampling: what one rank knows about one row of its column slice. cand holds every
// local logit at or above the local k-th largest (global indices); the global kept set is a
// subset of the union of the ranks' lists, because the global k-th largest is at least every
// local one.
constexpr int VS_CAND = 128;
constexpr uint32_t VS_NONFINITE = 1u, VS_BAD_CFG = 2u, VS_OVERFLOW = 4u, VS_UNSUPPORTED = 8u, VS_NAN_AT_0 = 16u,
                   VS_SUMEXP = 32u;   // a row without top-k: cand[0] holds the slice's sum of exponentials (f64 bits)
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

// A row's top-p setting cuts nothing: off, or the mode A rule with 1.5 p >= 1 (generate.go:184-228).
__device__ __forceinline__ bool vs_cut_inert(const RowCfg& c) {
  const bool on = c.top_p > 0.0f && c.top_p < 1.0f;
  return !on || (c.topp_mode == 0 && static_cast<double>(c.top_p) * 1.5 >= 1.0);
}
// exp(d), d <= 0, as f64: the table form (2e-11) where it applies, the all-f64 routine elsewhere.
// The local pass and the owner's draw use the same function, so that their sums agree term by term.
__device__ __forceinline__ double vs_exp(float d, const double* __restrict__ eb, const double* __restrict__ tab) {
  return (d > -31.9f) ? exp_fast(d, eb) : exp_safe(d, tab);
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

// The narrow kernel, compiled twice from one source (sample_narrow.cuh): n256 with 256 threads and
// five CTAs per SM for batches of at most one row per CTA slot (a row is then streamed by eight
// warps), n128 with 128 threads and eight CTAs per SM beyond that (1184 rows in flight: the phases
// before and after a row's stream then run once per slot instead of twice).
#define GS_N_NS n256
#define GS_N_NT 256
#include "sample_narrow.cuh"
#undef GS_N_NS
#undef GS_N_NT
#define GS_N_NS n128
#define GS_N_NT 128
#include "sample_narrow.cuh"
#undef GS_N_NS
#undef GS_N_NT

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
