// Vocab-sharded sampling: each rank holds a contiguous column slice of every row.
//
//   step 1 (every rank)   narrow_rows_kernel with KernelArgs::vs_records set: one pass over the
//                         rank's slice per row, leaving a VsRecord (local maximum, every local
//                         logit at or above the local k-th largest, with global indices)
//   exchange              one all-gather of the records, rank order (done by the caller: NCCL)
//   step 2 (every rank)   vocab_merge_kernel: joins the ranks' lists of a row, takes the global
//                         k-th largest (ties kept, generate.go:157-164), and finishes the row
//                         (softmax over the kept set, top-p, draw) exactly like the one-GPU path.
//                         Every rank computes every id: the result needs no second exchange.
//
// The reference has no multi-device path; the row semantics are model/generate.go:147-240 and
// model/qwen/generate.go:92-153 applied to the whole row.
#pragma once

#include "sample_batch.cuh"

namespace gs {

constexpr int VM_NT = 128;                                  // eight CTAs per SM: 1184 rows in flight
constexpr int VM_MAX_RANKS = 16;
constexpr int VM_LIST = VM_MAX_RANKS * VS_CAND;             // 2048 entries
constexpr int VM_DYN_BYTES = VM_LIST * 8 + 16384 + KEEP_MAX * 8;   // the most a launch asks for
// dynamic shared memory of a launch: the joined list sized by its ranks and candidates
__host__ __device__ constexpr int vm_list_entries(int nranks, int cand) { return ((nranks * cand + 15) / 16) * 16; }
__host__ __device__ constexpr int vm_dyn_bytes(int nranks, int cand) { return vm_list_entries(nranks, cand) * 8 + 16384 + KEEP_MAX * 8; }

struct MergeArgs {
  KernelArgs k;             // V = whole vocabulary; logits unused
  const void* records;      // [nranks][B] records of 16 + 8 * cand bytes
  int32_t nranks;
  int32_t cand;             // candidates per record
  int64_t B;
  int32_t my_rank;          // rows without top-k: which rank this is (-1: such rows are not served)
  double* draw_req;         // [B][3] or null: for rows without top-k that this rank owns, what vocab_draw_kernel needs
};

// Rows without top-k (records carry VS_SUMEXP): the merge adds the slices' sums, rescaled to the
// row's maximum, in rank order (= index order: the slices are contiguous); the rank in whose slice
// u * S falls owns the row and finds the token by a pass over its slice (vocab_draw_kernel); the
// other ranks write -1, and an all-reduce (max) of the ids hands the token to everyone.
// draw_req[row] = {target in units of the owner's own sum, S in those units, the owner's scaled
// maximum}; a row this rank does not own gets a NaN target.
constexpr int VD_NT = 256;

__global__ void __launch_bounds__(VM_NT, 8) vocab_merge_kernel(MergeArgs M) {
  extern __shared__ __align__(16) unsigned char dyn[];
  __shared__ bu::Scratch sc;
  __shared__ uint32_t s_sel[256];
  __shared__ int s_bc[4];
  __shared__ double s_bcd[4];
  __shared__ int s_cnt;
  uint2* list = reinterpret_cast<uint2*>(dyn);                                   // joined candidates
  const int list_bytes = vm_list_entries(M.nranks, M.cand) * 8;
  unsigned char* work = dyn + list_bytes;                                         // 16 KB for finish_small_set
  uint2* kept = reinterpret_cast<uint2*>(dyn + list_bytes + 16384);              // KEEP_MAX entries
  const KernelArgs& A = M.k;
  const int tid = threadIdx.x;
  constexpr int NW = VM_NT / 32;
  for (int64_t row = blockIdx.x; row < M.B; row += gridDim.x) {
    __syncthreads();
    const RowCfg cfg = A.cfgs[row];
    const float Tm = cfg.temperature;
    RowDebug dbg;
    dbg.sum_exp = 0; dbg.resum = 1.0; dbg.edge_lo = 0; dbg.edge_hi = 0; dbg.kept = 0;
    dbg.max_scaled = 0; dbg.threshold = __int_as_float(0x7fc00000); dbg.path = 3;
    for (int q = 0; q < 8; q++) dbg.reserved[q] = 0;
    auto write_row = [&](int id, uint32_t fl) {
      if (tid == 0) {
        A.out_ids[row] = id;
        if (A.out_flags) A.out_flags[row] = fl;
        if (A.out_debug) A.out_debug[row] = dbg;
      }
    };
    // a row that no draw follows (every row with a top-k, greedy rows, refused rows) says so
    if (tid == 0 && M.draw_req) M.draw_req[row * 3] = __longlong_as_double(0x7ff8000000000000ll);
    // ---- join the ranks' records
    if (tid == 0) s_cnt = 0;
    __syncthreads();
    uint32_t fl_loc = 0u;
    unsigned long long mx = 0ull;
    for (int r = 0; r < M.nranks; r++) {
      const VsRecord& rec = vs_record(M.records, static_cast<int64_t>(r) * M.B + row, M.cand);
      const int n = min(max(rec.n, 0), M.cand);
      fl_loc |= rec.flags;
      if (n > 0) { const unsigned long long k = okey(rec.xmax); mx = k > mx ? k : mx; }
      int base = 0;
      if (tid == 0) { base = s_cnt; s_cnt = base + n; }
      __syncthreads();
      base = s_cnt - n;
      for (int j = tid; j < n; j += VM_NT) list[base + j] = rec.cand[j];
      __syncthreads();
    }
    const int cnt = s_cnt;
    const uint32_t vfl = fl_loc;                             // uniform: every thread read every record header
    if (vfl & VS_BAD_CFG) { write_row(-1, FLAG_BAD_CFG); continue; }
    if (vfl & (VS_OVERFLOW | VS_UNSUPPORTED)) { write_row(-1, FLAG_INTERNAL); continue; }
    if (vfl & VS_SUMEXP) {
      if (!M.draw_req || M.my_rank < 0) { write_row(-1, FLAG_INTERNAL); continue; }
      if (tid == 0) {
        double* req = M.draw_req + row * 3;
        float mrow = -INFINITY;
        for (int r = 0; r < M.nranks; r++)
          mrow = fmaxf(mrow, scale_t(vs_record(M.records, static_cast<int64_t>(r) * M.B + row, M.cand).xmax, Tm));
        double w[VM_MAX_RANKS], S = 0.0;
        for (int r = 0; r < M.nranks; r++) {
          const VsRecord& rec = vs_record(M.records, static_cast<int64_t>(r) * M.B + row, M.cand);
          const double Sr = __longlong_as_double(static_cast<long long>((static_cast<unsigned long long>(rec.cand[0].y) << 32) | rec.cand[0].x));
          const float sr = scale_t(rec.xmax, Tm);
          w[r] = (sr == -INFINITY) ? 0.0 : Sr * exp(static_cast<double>(sr) - static_cast<double>(mrow));
          S += w[r];
        }
        dbg.max_scaled = mrow; dbg.sum_exp = S;
        int id = -1;
        uint32_t fl = 0u;
        if ((vfl & VS_NONFINITE) || !(fabsf(mrow) < INFINITY) || !(S > 0.0) || !(S == S)) {
          id = A.V - 1; fl = FLAG_NONFINITE | FLAG_FALLBACK;   // generate.go:173-181, 239
        } else {
          const double target = A.uniforms[row] * S;          // first index with u < cumulative / S
          double cum = 0.0;
          int owner = -1;
          for (int r = 0; r < M.nranks; r++) {
            if (target < cum + w[r]) { owner = r; break; }
            cum += w[r];
          }
          if (owner < 0) {
            id = A.V - 1; fl = FLAG_FALLBACK | ((target - S <= 1e-6 * S) ? FLAG_BOUNDARY : 0u);
          } else if (owner == M.my_rank) {
            const VsRecord& rec = vs_record(M.records, static_cast<int64_t>(owner) * M.B + row, M.cand);
            const float sr = scale_t(rec.xmax, Tm);
            const double f = exp(static_cast<double>(sr) - static_cast<double>(mrow));
            req[0] = (target - cum) / f;
            req[1] = S / f;
            req[2] = static_cast<double>(sr);
          }
        }
        A.out_ids[row] = id;
        if (A.out_flags) A.out_flags[row] = fl;
        if (A.out_debug) A.out_debug[row] = dbg;
      }
      continue;
    }
    // ---- greedy (generate.go:134-144): largest logit, lowest index; a NaN at index 0 is never beaten
    if (Tm == 0.0f) {
      unsigned long long best = 0ull;
      for (int j = tid; j < cnt; j += VM_NT) {
        const unsigned long long p = (static_cast<unsigned long long>(okey(__uint_as_float(list[j].x))) << 32) |
                                     static_cast<uint32_t>(~list[j].y);
        best = p > best ? p : best;
      }
      best = bu::max_u64<NW>(best, sc, tid);
      int id = static_cast<int>(~static_cast<uint32_t>(best & 0xffffffffull));
      if ((vfl & VS_NAN_AT_0) || cnt == 0) id = 0;           // no champion anywhere: index 0 is never beaten
      dbg.kept = 1;
      write_row(id, 0u);
      continue;
    }
    const float xmax = okey_to_float(static_cast<uint32_t>(mx));
    const float m = scale_t(xmax, Tm);
    dbg.max_scaled = m;
    // A NaN anywhere, or an infinite maximum: the walk of generate.go:231-239 falls through
    // (no candidate in any slice: the row holds no finite logit at all)
    if ((vfl & VS_NONFINITE) || cnt == 0 || !(fabsf(m) < INFINITY)) {
      dbg.sum_exp = __longlong_as_double(0x7ff8000000000000ll);
      write_row(A.V - 1, FLAG_NONFINITE | FLAG_FALLBACK);
      continue;
    }
    // ---- global k-th largest with ties (generate.go:157-164), then the kept set
    const int topk = cfg.top_k;                              // 0 < top_k <= VS_CAND (checked by the local pass)
    float thr = -INFINITY;
    if (cnt > topk) {
      const uint32_t kkey = bu::select_kth<VM_NT>(list, cnt, topk, s_sel, s_bc, tid, 0u, static_cast<uint32_t>(mx));
      thr = quotient_class_floor(okey_to_float(kkey), Tm);
    }
    __syncthreads();
    if (tid == 0) s_cnt = 0;
    __syncthreads();
    for (int j = tid; j < cnt; j += VM_NT) {
      const uint2 e = list[j];
      if (__uint_as_float(e.x) >= thr) { const int slot = atomicAdd(&s_cnt, 1); if (slot < KEEP_MAX) kept[slot] = e; }
    }
    __syncthreads();
    const int nk = s_cnt;
    if (nk > KEEP_MAX) { write_row(-1, FLAG_INTERNAL); continue; }
    const bool topp_on = (cfg.top_p > 0.0f && cfg.top_p < 1.0f);
    const int mode = cfg.topp_mode;
    const double plim = (mode == 0) ? static_cast<double>(cfg.top_p) * 1.5 : static_cast<double>(cfg.top_p);
    finish_small_set<VM_NT>(A, row, kept, nk, m, Tm, topp_on, mode, plim, A.uniforms[row], work, sc, s_bcd, dbg, 0u);
  }
}

// The local pass of a vocab-sharded row without top-k and without an effective top-p cut (plain
// softmax sampling): what the merge needs from a slice is its maximum and its sum of exponentials
// relative to that maximum (generate.go:167-181 on the slice). Two passes over the slice, the
// second from L2. A kernel of its own, beside the narrow kernel's launch, so that the narrow kernel
// (whose registers are spoken for) stays as it is for every other caller.
template <typename T>
__global__ void __launch_bounds__(VD_NT, 4) vocab_sumexp_kernel(KernelArgs A, const double* eb_table, int64_t B) {
  __shared__ bu::Scratch sc;
  const int tid = threadIdx.x;
  constexpr int NW = VD_NT / 32;
  for (int64_t row = blockIdx.x; row < B; row += gridDim.x) {
    const RowCfg cfg = A.cfgs[row];
    const float Tm = cfg.temperature;
    if (!(Tm > 0.0f) || !(Tm < INFINITY) || cfg.top_k != 0 || !vs_cut_inert(cfg)) continue;   // the narrow kernel's rows
    RowView<T> rv;
    rv.init(static_cast<const T*>(A.logits) + row * A.row_stride, A.V);
    float vmax = -INFINITY;
    bool nan_loc = false;
    for (int v = tid; v < rv.nvec; v += VD_NT)
      rv.visit(v, [&](float x, int) { vmax = fmaxf(vmax, x); nan_loc |= (x != x); });
    const int slice_nan = bu::max_i<NW>(nan_loc ? 1 : 0, sc, tid);
    const float smax_x = okey_to_float(static_cast<uint32_t>(bu::max_u64<NW>(static_cast<unsigned long long>(okey(vmax)), sc, tid)));
    const float sm = scale_t(smax_x, Tm);
    double acc = 0.0;
    if (!slice_nan && fabsf(sm) < INFINITY) {
      for (int v = tid; v < rv.nvec; v += VD_NT)
        rv.visit(v, [&](float x, int) { acc += vs_exp(scale_t(x, Tm) - sm, eb_table, A.exp_table); });
    }
    const double Sr = bu::sum_d<NW>(acc, sc, tid);
    if (tid == 0) {
      VsRecord& rec = vs_record(A.vs_records, row, A.vs_cand);
      rec.xmax = smax_x; rec.n = 0; rec.pad = 0;
      // a slice of -Inf only (a masked part of the vocabulary) carries no mass and no verdict
      rec.flags = VS_SUMEXP | ((slice_nan || sm == INFINITY || sm != sm) ? VS_NONFINITE : 0u);
      const unsigned long long bits = static_cast<unsigned long long>(__double_as_longlong((sm == -INFINITY) ? 0.0 : Sr));
      rec.cand[0] = make_uint2(static_cast<uint32_t>(bits), static_cast<uint32_t>(bits >> 32));
    }
    __syncthreads();
  }
}

struct DrawArgs {
  const void* logits;       // this rank's slice [B, row_stride]
  int64_t row_stride;
  int32_t V;                // slice length
  int32_t col_offset;       // global index of the slice's first column
  const RowCfg* cfgs;
  const double* draw_req;   // [B][3] from the merge
  const double* eb_table;
  const double* exp_table;
  int32_t* out_ids;
  uint32_t* out_flags;
  int64_t B;
};

// The owner's pass over its slice: first index whose running sum of exp(x/T - own maximum), in
// index order, exceeds the target. Tiles of VD_NT x 4 logits, one block scan per tile.
template <typename T>
__global__ void __launch_bounds__(VD_NT, 4) vocab_draw_kernel(DrawArgs D) {
  __shared__ bu::Scratch sc;
  __shared__ int s_hit[2];
  const int tid = threadIdx.x;
  constexpr int NW = VD_NT / 32, PER = 4;
  for (int64_t row = blockIdx.x; row < D.B; row += gridDim.x) {
    const double target = D.draw_req[row * 3];
    if (!(target == target)) continue;                       // not this rank's row (uniform: all threads read it)
    const double S = D.draw_req[row * 3 + 1];
    const float sr = static_cast<float>(D.draw_req[row * 3 + 2]);
    const float Tm = D.cfgs[row].temperature;
    const T* xr = static_cast<const T*>(D.logits) + row * D.row_stride;
    double base = 0.0;
    int found = -1, lastpos = -1;                           // lastpos: this thread's last logit with mass
    double lo = 0.0, hi = 0.0;
    for (int i0 = 0; i0 < D.V && found < 0; i0 += VD_NT * PER) {   // uniform
      double e[PER], mine = 0.0;
#pragma unroll
      for (int c = 0; c < PER; c++) {
        const int i = i0 + tid * PER + c;
        e[c] = 0.0;
        if (i < D.V) {
          const float x = Elem<T>::to_float(xr[i]);
          e[c] = vs_exp(scale_t(x, Tm) - sr, D.eb_table, D.exp_table);
          if (e[c] > 0.0) lastpos = i;
        }
        mine += e[c];
      }
      double tot;
      const double ex = bu::scan_excl_d<NW>(mine, tot, sc, tid);
      const int first = (target < base + ex + mine) ? tid : VD_NT;
      const int who = bu::min_i<NW>(first, sc, tid);
      if (who < VD_NT) {
        if (tid == who) {
          double run = base + ex;
          int pick = -1;
#pragma unroll
          for (int c = 0; c < PER; c++) {
            if (pick < 0 && target < run + e[c]) { pick = i0 + tid * PER + c; lo = run; hi = run + e[c]; }
            if (pick < 0) run += e[c];
          }
          s_hit[0] = pick;
          uint32_t fl = 0u;
          if ((target - lo) <= 1e-6 * S || (hi - target) <= 1e-6 * S) fl |= FLAG_BOUNDARY;
          s_hit[1] = static_cast<int>(fl);
        }
        __syncthreads();
        found = s_hit[0];
        if (tid == 0) {
          D.out_ids[row] = found + D.col_offset;
          if (D.out_flags) D.out_flags[row] = static_cast<uint32_t>(s_hit[1]);
        }
        __syncthreads();
      }
      base += tot;
    }
    if (found < 0) {                                         // uniform
      // the slice's running sum, formed in another order than the local pass's, fell short of the
      // target by rounding: the slice's last logit with mass is the nearest answer
      const int last = bu::max_i<NW>(lastpos, sc, tid);
      if (tid == 0) {
        D.out_ids[row] = max(last, 0) + D.col_offset;
        if (D.out_flags) D.out_flags[row] = FLAG_BOUNDARY;
      }
    }
  }
}

// done[b] = 0 for the rows that the gathered-rows path samples: sampling rows without top-k whose
// top-p cut is active, and with owner_draw off every sampling row without top-k; 1 for all others
// (they have their token from the records).
__global__ void vocab_gather_mask_kernel(const RowCfg* cfgs, int32_t V, int64_t B, bool owner_draw, int32_t* done) {
  const int64_t b = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (b >= B) return;
  const RowCfg c = cfgs[b];
  const float T = c.temperature;
  const bool sampling = T > 0.0f && T < INFINITY;
  const bool topk_off = !(c.top_k > 0 && c.top_k < V);
  done[b] = (sampling && topk_off && !(owner_draw && vs_cut_inert(c))) ? 0 : 1;
}

}  // namespace gs
