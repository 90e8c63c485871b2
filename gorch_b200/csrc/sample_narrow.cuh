// The narrow kernel of the sorted-batch path (greedy and top-k <= 256 rows, one streaming pass
// each), written once and compiled for two CTA sizes: the including file defines GS_N_NS (the
// instance's namespace inside gs) and GS_N_NT (threads per CTA: 256 or 128). No include guard.
// Row semantics: model/generate.go:134-260 (mode A), model/qwen/generate.go:77-181 (mode B).

// (included inside namespace gs)
namespace GS_N_NS {

constexpr int N_NT = GS_N_NT;           // threads per CTA
constexpr int N_NW = N_NT / 32;
constexpr int N_WARM_ELEMS = 16 * N_NT; // logits of the warm-up chunk: 16 per thread, kept in registers
// 256 threads: five CTAs per SM (48 registers, 42 KB of dynamic shared memory: [0, 24 KB) the ring
// the stream is staged through, whose upper 16 KB double as the work arrays of the phases that
// run while no copy is in flight (prune, finish); then the candidate list and the hit list).
// 128 threads: eight CTAs per SM (64 registers, 20 KB: candidate list, ring, hit list; the
// prune's buffer is the ring, the finish's work arrays lie over the upper half of the candidate
// list, the ring and the hit list, all of them dead by then).
constexpr int N_CTAS_PER_SM = (N_NT == 256) ? 5 : 8;
constexpr int N_CAP = (N_NT == 256) ? 1536 : 1024;   // candidate capacity (entries of 8 B)
constexpr int N_KEEP = 768;                           // a prune must get below this
constexpr int N_HITS = (N_NT == 256) ? 1536 : 1024;  // hit list: positions of lane-steps that hold a candidate (4 B each)
constexpr int N_RING_BYTES = (N_NT == 256) ? 24576 : 8192;
constexpr int N_RING_OFF = (N_NT == 256) ? 0 : 8192;
constexpr int N_CAND_OFF = (N_NT == 256) ? 24576 : 0;
constexpr int N_HITS_OFF = (N_NT == 256) ? N_CAND_OFF + N_CAP * 8 : 16384;
constexpr int N_WORK_OFF = (N_NT == 256) ? 8192 : 4096;   // 16 KB of work arrays for the finish
constexpr int N_TMP_OFF = (N_NT == 256) ? 8192 : 8192;    // the prune's buffer ...
constexpr int N_TMP_CAP = (N_NT == 256) ? 2048 : 1024;    // ... and its entries
constexpr int N_DYN_BYTES = N_HITS_OFF + N_HITS * 4;
static_assert(N_WORK_OFF + 16384 <= N_DYN_BYTES &&
              (N_WORK_OFF >= N_CAND_OFF + KEEP_MAX * 8 || N_WORK_OFF + 16384 <= N_CAND_OFF),
              "the finish's work arrays leave the kept set alone");
static_assert(N_TMP_OFF >= N_RING_OFF && N_TMP_OFF + N_TMP_CAP * 8 <= N_RING_OFF + N_RING_BYTES, "the prune's buffer lies in the ring");
static_assert(N_TMP_CAP >= N_KEEP && N_KEEP + 8 <= N_CAP, "a pruned list fits its buffer and leaves room for a portion of hits");

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
  unsigned char* work = dyn + N_WORK_OFF;                    // 16 KB of work arrays (finish)
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
  // a vocab-sharded row without top-k: vocab_sumexp_kernel fills its record, when the caller asked for that
  if (A.vs_records && A.vs_sumexp && cfg.top_k == 0 && vs_cut_inert(cfg)) return;
  if (A.vs_records && !(cfg.top_k > 0 && cfg.top_k <= A.vs_cand)) {   // the merge needs a top-k to bound the lists
    vs_flag_only(VS_UNSUPPORTED);
    return;
  }
  const int topk = cfg.top_k;                                // 0 < top_k <= KFAST, < V (classified)
  const bool topp_on = (cfg.top_p > 0.0f && cfg.top_p < 1.0f);
  const int mode = cfg.topp_mode;
  const double plim = (mode == 0) ? static_cast<double>(cfg.top_p) * 1.5 : static_cast<double>(cfg.top_p);
  dbg.path = 1;

  // ---- warm-up chunk: the row's first 16 logits per thread, kept in registers; one running maximum per thread
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
  constexpr int NQ = N_RING_BYTES / (EPI * N_NT * 16);       // stages: 6 of bf16, 3 of f32 (128 threads: 4 and 2)
  const int lane = tid & 31, warp = tid >> 5;
  const int rest = max(rv.nvec - warm, 0);
  const int span = (((rest + N_NW - 1) / N_NW + SV - 1) / SV) * SV;
  const WSpan sp = make_span<T>(rv, warm + warp * span, span, lane);
  unsigned long long pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  const uint32_t ring_addr = smem_addr(dyn + N_RING_OFF) + static_cast<uint32_t>(tid * 16);
  const uint4* ring = reinterpret_cast<const uint4*>(dyn + N_RING_OFF) + tid;
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
  // Threshold from the N_NT per-thread maxima of the chunk: every warp sorts its 32 maxima with
  // shuffles, and every thread then finds the place of its own among all of them by a binary search
  // in each of the other warps' sorted lists (two barriers; a radix select over so few keys costs
  // several rounds of barriers and of shared atomics that all hit the same few bins, and counting
  // all maxima against each other three times the instructions). A rank beyond N_NT (top_k above
  // 128 on a short row, 128-thread instance) finds no thread: the threshold stays open and the
  // overflow path below takes the exact top_k-th largest of the chunk instead.
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
    uint2* tmp = reinterpret_cast<uint2*>(dyn + N_TMP_OFF);  // N_TMP_CAP entries
    for (int j = tid; j < cnt; j += N_NT) {
      const uint2 e = cand[j];
      if (__uint_as_float(e.x) >= thr) { const int slot = atomicAdd(s_cnt, 1); if (slot < N_TMP_CAP) tmp[slot] = e; }
    }
    __syncthreads();
    const int kept = *s_cnt;
    if (kept <= N_TMP_CAP) for (int j = tid; j < kept; j += N_NT) cand[j] = tmp[j];
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

}  // namespace GS_N_NS
