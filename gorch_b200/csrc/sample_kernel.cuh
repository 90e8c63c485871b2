// One CTA per logits row: greedy argmax, temperature, top-k (ties kept),
// top-p (both reference flavours) and the inverse-CDF draw.
//
// Row semantics follow model/generate.go:134-260 ("mode A") and
// model/qwen/generate.go:77-181 ("mode B"); see the rule comments below.
//
// Structure per row
//   greedy (T == 0)      one pass, (value, lowest index) reduction.
//   small-set path       rows whose kept set fits in shared memory
//                        (top_k <= KFAST_MAX, or V <= KEPT_CAP): one streaming
//                        pass with an adaptive threshold collects the
//                        candidates, everything else happens in shared memory.
//   full-row path        everything else (top_k off or huge): pass 1 row max,
//                        pass 2 a count histogram over linear buckets of
//                        d = s - max that brackets the top-p cut, pass 3 the
//                        f64 exponentials with per-segment sums, then an exact
//                        resolution of the bracketed zone and a rescan of the
//                        one segment that holds the drawn token.
#pragma once

#include "sample_common.cuh"

namespace gs {

constexpr int NT = 512;            // threads per CTA
constexpr int NW = NT / 32;        // warps per CTA
constexpr int CAND_CAP = 2048;     // candidate / zone list capacity (entries of 8 B)
constexpr int KFAST_MAX = 1024;    // largest top_k served by the streaming small-set path
constexpr int KEPT_CAP = 1024;     // largest kept set finished in shared memory
constexpr int NBUCKET = 4096;      // level-0 buckets of width 1/128 over d in [-32, 0]
constexpr int MAXSEG = 256;        // contiguous row segments with their own mass sums
constexpr int SEG_VECS_MIN = 256;  // 16-byte vectors per segment (lower bound)

// Shared-memory pool carved by hand (bytes).
constexpr int POOL_HIST = 0;                       // 16 KB: uint32[4096] histogram
constexpr int POOL_CAND = 16384;                   // 16 KB: uint2[2048] candidates / zone list
constexpr int POOL_X = 32768;                      // 16 KB: scratch for sorted values
constexpr int POOL_Y = 49152;                      // 8 KB: order / rank scratch
constexpr int POOL_BYTES = 57344;

struct KernelArgs {
  const void* logits;      // [B, row_stride] f32 or bf16
  int64_t row_stride;      // elements between rows
  int32_t V;
  int32_t force_greedy;    // argmax entry point: ignore cfgs
  const RowCfg* cfgs;      // [B]
  const double* uniforms;  // [B]
  int32_t* out_ids;        // [B]
  uint32_t* out_flags;     // [B] (may be null)
  double* out_probs;       // [B, V] dense final probabilities (may be null)
  RowDebug* out_debug;     // [B] (may be null)
  const double* exp_table; // 256 doubles: 2^(j/256)
  int64_t row_offset;      // first row handled by this launch (for chunked launches)
  const int32_t* worklist; // single-CTA kernel only: [0] = count, [1..] = rows to process (null: every row)
  void* vs_records;        // vocab-sharded local pass (narrow kernel only): [B] VsRecord to fill instead of drawing
  int32_t vs_col_offset;   // global index of this slice's first column
  int32_t vs_cand;         // candidates per record (records are 16 + 8 * vs_cand bytes apart), at most VS_CAND
  int32_t vs_sumexp;       // rows without top-k are served (their records come from vocab_sumexp_kernel)
  float* tk_values;        // TopK op (narrow kernel only): [B, tk_k] values, descending; null otherwise
  int32_t* tk_indices;     // [B, tk_k] indices (ties: ascending index)
  int32_t tk_k;            // 0: not a TopK launch
  const int32_t* row_done; // generate loops: rows whose entry is non-zero have ended and are skipped (null: none)
};

template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int VEC = 4;
  __device__ static __forceinline__ void unpack(const uint4& r, float* x) {
    x[0] = __uint_as_float(r.x); x[1] = __uint_as_float(r.y);
    x[2] = __uint_as_float(r.z); x[3] = __uint_as_float(r.w);
  }
  __device__ static __forceinline__ float to_float(float v) { return v; }
};
template <> struct Elem<uint16_t> {  // bf16 bit patterns; upcast = bits << 16 (tensor.go:96-99)
  static constexpr int VEC = 8;
  __device__ static __forceinline__ void unpack(const uint4& r, float* x) {
    x[0] = __uint_as_float(r.x << 16); x[1] = __uint_as_float(r.x & 0xffff0000u);
    x[2] = __uint_as_float(r.y << 16); x[3] = __uint_as_float(r.y & 0xffff0000u);
    x[4] = __uint_as_float(r.z << 16); x[5] = __uint_as_float(r.z & 0xffff0000u);
    x[6] = __uint_as_float(r.w << 16); x[7] = __uint_as_float(r.w & 0xffff0000u);
  }
  __device__ static __forceinline__ float to_float(uint16_t v) { return __uint_as_float(static_cast<uint32_t>(v) << 16); }
};

// A row seen as 16-byte vectors. Rows need not start on a 16-byte boundary
// (V = 50257 floats does not): vector 0 starts at the boundary at or below the
// row's first byte, and `shift` elements of it belong to whatever precedes the
// row. A 16-byte aligned load that holds at least one valid byte never leaves
// the allocation's page, so the edge vectors are loaded whole and masked.
template <typename T>
struct RowView {
  const uint4* vbase;
  int V;
  int shift;
  int nvec;
  __device__ __forceinline__ void init(const T* row, int V_) {
    constexpr int VEC = Elem<T>::VEC;
    uintptr_t a = reinterpret_cast<uintptr_t>(row);
    shift = static_cast<int>((a & 15u) / sizeof(T));
    vbase = reinterpret_cast<const uint4*>(a & ~static_cast<uintptr_t>(15));
    V = V_;
    nvec = (V_ + shift + VEC - 1) / VEC;
  }
  // f(x, i) for every valid element of vector v.
  template <typename F>
  __device__ __forceinline__ void visit(int v, F&& f) const {
    constexpr int VEC = Elem<T>::VEC;
    uint4 raw = __ldg(vbase + v);
    float x[VEC];
    Elem<T>::unpack(raw, x);
    int i0 = v * VEC - shift;
    if (v > 0 && v < nvec - 1) {
#pragma unroll
      for (int c = 0; c < VEC; c++) f(x[c], i0 + c);
    } else {
#pragma unroll
      for (int c = 0; c < VEC; c++) {
        int i = i0 + c;
        if (i >= 0 && i < V) f(x[c], i);
      }
    }
  }
  template <typename F>
  __device__ __forceinline__ void visit_raw(const uint4& raw, int v, F&& f) const {
    constexpr int VEC = Elem<T>::VEC;
    float x[VEC];
    Elem<T>::unpack(raw, x);
    int i0 = v * VEC - shift;
    if (v > 0 && v < nvec - 1) {
#pragma unroll
      for (int c = 0; c < VEC; c++) f(x[c], i0 + c, c);
    } else {
#pragma unroll
      for (int c = 0; c < VEC; c++) {
        int i = i0 + c;
        if (i >= 0 && i < V) f(x[c], i, c);
      }
    }
  }
  __device__ __forceinline__ int vec_of(int i) const { return (i + shift) / Elem<T>::VEC; }
};

// Small block-wide state.
struct Ctl {
  double red_d[NW];
  double red_d2[NW];
  double bcast_d[4];
  unsigned long long red_u64[NW];
  int red_i[NW];
  int bcast_i[8];
  int cand_count;
  int overflow;
  float thr;       // current streaming threshold in logit units
  uint32_t flags;
};

struct Cut {       // how the top-p cut applies to a full-row element
  int active;      // 0: every live element is kept
  int b1, b2;      // zone buckets; b < b1 kept, b > b2 dropped
  int mode;
  int idx_c;       // index of the zone element at the cut
  double e_c;      // its mass; +Inf when no zone element is kept, -1 when all are
  int incl;        // 1: the element at the cut is itself kept
};

__device__ __forceinline__ double block_sum_d(double v, Ctl& c, int tid) {
  v = warp_sum_d(v);
  __syncthreads();
  if ((tid & 31) == 0) c.red_d[tid >> 5] = v;
  __syncthreads();
  double t = 0.0;
#pragma unroll
  for (int w = 0; w < NW; w++) t += c.red_d[w];
  return t;
}
__device__ __forceinline__ int block_sum_i(int v, Ctl& c, int tid) {
  v = warp_sum_i(v);
  __syncthreads();
  if ((tid & 31) == 0) c.red_i[tid >> 5] = v;
  __syncthreads();
  int t = 0;
#pragma unroll
  for (int w = 0; w < NW; w++) t += c.red_i[w];
  return t;
}
__device__ __forceinline__ int block_min_i(int v, Ctl& c, int tid) {
  v = __reduce_min_sync(FULL, v);
  __syncthreads();
  if ((tid & 31) == 0) c.red_i[tid >> 5] = v;
  __syncthreads();
  int t = c.red_i[0];
#pragma unroll
  for (int w = 1; w < NW; w++) t = min(t, c.red_i[w]);
  return t;
}
__device__ __forceinline__ int block_max_i(int v, Ctl& c, int tid) {
  v = __reduce_max_sync(FULL, v);
  __syncthreads();
  if ((tid & 31) == 0) c.red_i[tid >> 5] = v;
  __syncthreads();
  int t = c.red_i[0];
#pragma unroll
  for (int w = 1; w < NW; w++) t = max(t, c.red_i[w]);
  return t;
}
// max over (key, lowest index): packed as key<<32 | ~idx so that u64 max does both.
__device__ __forceinline__ unsigned long long block_max_u64(unsigned long long v, Ctl& c, int tid) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long t = __shfl_xor_sync(FULL, v, o);
    v = t > v ? t : v;
  }
  __syncthreads();
  if ((tid & 31) == 0) c.red_u64[tid >> 5] = v;
  __syncthreads();
  unsigned long long t = c.red_u64[0];
#pragma unroll
  for (int w = 1; w < NW; w++) t = c.red_u64[w] > t ? c.red_u64[w] : t;
  return t;
}

// Exclusive prefix over one double per thread (thread order); returns the
// exclusive prefix and writes the block total.
__device__ __forceinline__ double block_scan_excl_d(double v, double& total, Ctl& c, int tid) {
  int lane = tid & 31, w = tid >> 5;
  double incl = warp_scan_incl_d(v, lane);
  __syncthreads();
  if (lane == 31) c.red_d2[w] = incl;
  __syncthreads();
  double base = 0.0, tot = 0.0;
#pragma unroll
  for (int j = 0; j < NW; j++) {
    double s = c.red_d2[j];
    if (j < w) base += s;
    tot += s;
  }
  total = tot;
  return base + incl - v;
}

// In-place inclusive scan of a shared array a[0..n), n <= PER*NT, in index order.
template <int PER>
__device__ __forceinline__ void smem_scan_incl(double* a, int n, Ctl& c, int tid) {
  double loc[PER];
  double s = 0.0;
  int base = tid * PER;
#pragma unroll
  for (int j = 0; j < PER; j++) {
    double v = (base + j < n) ? a[base + j] : 0.0;
    s += v;
    loc[j] = s;
  }
  double tot;
  double ex = block_scan_excl_d(s, tot, c, tid);
#pragma unroll
  for (int j = 0; j < PER; j++) {
    if (base + j < n) a[base + j] = ex + loc[j];
  }
  __syncthreads();
}

// Smallest logit x' whose scaled value x'/T is still >= x/T: the k-th largest
// is defined on scaled values (generate.go:158-163), and f32 division can map
// neighbouring logits to one quotient, so the logit-space threshold is the
// bottom of that quotient class.
__device__ float quotient_class_floor(float x, float T) {
  if (T == 1.0f) return x;
  float q = __fdiv_rn(x, T);
  uint32_t hi = okey(x);
  uint32_t k = hi;
  for (int s = 0; s < 16; s++) {
    if (k <= 0x007fffffu) return okey_to_float(k);  // reached -Inf
    float nx = okey_to_float(k - 1);
    if (__fdiv_rn(nx, T) >= q) k = k - 1; else return okey_to_float(k);
  }
  uint32_t lo = 0x007fffffu;  // key of -Inf
  // invariant: pred(hi) true; find the least key in [lo, hi] with pred true
  while (lo < hi) {
    uint32_t mid = lo + ((hi - lo) >> 1);
    if (__fdiv_rn(okey_to_float(mid), T) >= q) hi = mid; else lo = mid + 1;
  }
  return okey_to_float(hi);
}

// k-th largest (with multiplicity) of the float bit patterns list[j].x,
// j < n, by MSB-first radix select on order keys. hist: 256 uint32 of scratch.
__device__ uint32_t block_select_kth(const uint2* list, int n, int k, uint32_t* hist, Ctl& c, int tid) {
  uint32_t prefix = 0, mask = 0;
  int need = k;
  for (int round = 0; round < 4; round++) {
    int sh = 24 - 8 * round;
    __syncthreads();
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (int j = tid; j < n; j += NT) {
      uint32_t key = okey(__uint_as_float(list[j].x));
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> sh) & 255u], 1u);
    }
    __syncthreads();
    if (tid < 32) {
      // lane l owns bins [8l, 8l+8); scan from the top bin downwards
      int loc[8];
      int s = 0;
#pragma unroll
      for (int j = 7; j >= 0; j--) { s += static_cast<int>(hist[tid * 8 + j]); loc[j] = s; }
      int above = 0;  // total of higher lanes
      int run = s;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_down_sync(FULL, run, o);
        if (tid + o < 32) run += t;
      }
      above = run - s;
      if (above < need && above + s >= need) {
        int digit = 0, before = above;
#pragma unroll
        for (int j = 7; j >= 0; j--) {
          if (above + loc[j] >= need) { digit = j; before = above + loc[j] - static_cast<int>(hist[tid * 8 + j]); break; }
        }
        c.bcast_i[0] = tid * 8 + digit;
        c.bcast_i[1] = need - before;
      }
    }
    __syncthreads();
    prefix |= static_cast<uint32_t>(c.bcast_i[0]) << sh;
    mask |= 255u << sh;
    need = c.bcast_i[1];
  }
  return prefix;
}

// Level-0 bucket of d = s - max (d <= 0): round(-128 d) clamped to 4095.
// Non-decreasing as d falls, so "bucket order" is "descending probability".
__device__ __forceinline__ int bucket0(float d) {
  float f = fmaf(fmaxf(d, -31.992f), -128.0f, 8388608.0f);
  return __float_as_int(f) & 0x1fff;
}

template <typename T>
__device__ void single_cta_row(const KernelArgs& A, const int64_t row_id, unsigned char* pool) {
  __shared__ Ctl ctl;
  __shared__ Cut cut;
  __shared__ double s_tab[256];
  __shared__ double s_kseg[MAXSEG];

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int V = A.V;
  const T* row = static_cast<const T*>(A.logits) + row_id * A.row_stride;
  RowView<T> rv;
  rv.init(row, V);
  constexpr int VEC = Elem<T>::VEC;

  uint32_t* hist = reinterpret_cast<uint32_t*>(pool + POOL_HIST);
  uint2* cand = reinterpret_cast<uint2*>(pool + POOL_CAND);

  RowCfg cfg;
  if (A.force_greedy) { cfg.temperature = 0.f; cfg.top_k = 0; cfg.top_p = 0.f; cfg.topp_mode = 0; }
  else cfg = A.cfgs[row_id];
  const float Tm = cfg.temperature;

  if (tid < 256) s_tab[tid] = A.exp_table[tid];
  if (tid == 0) { ctl.cand_count = 0; ctl.overflow = 0; ctl.thr = -INFINITY; ctl.flags = 0; }
  __syncthreads();

  auto finish = [&](int id, uint32_t flags, const RowDebug& dbg) {
    if (tid == 0) {
      A.out_ids[row_id] = id;
      if (A.out_flags) A.out_flags[row_id] = flags;
      if (A.out_debug) A.out_debug[row_id] = dbg;
    }
  };
  auto fill_probs = [&](double v) {
    if (A.out_probs) {
      double* pr = A.out_probs + row_id * static_cast<int64_t>(V);
      for (int i = tid; i < V; i += NT) pr[i] = v;
    }
  };

  RowDebug dbg;
  dbg.sum_exp = 0; dbg.resum = 1.0; dbg.edge_lo = 0; dbg.edge_hi = 0; dbg.kept = 0;
  dbg.max_scaled = 0; dbg.threshold = __int_as_float(0x7fc00000); dbg.path = 0;
  for (int q = 0; q < 8; q++) dbg.reserved[q] = 0;

  // ------------------------------------------------------------------ greedy
  // generate.go:75-76 + 134-144: strict '>' from index 0. Lowest index wins
  // ties; a NaN is never selected unless it sits at index 0.
  if (Tm == 0.0f) {
    unsigned long long best = 0ull;
    for (int v = tid; v < rv.nvec; v += NT) {
      rv.visit(v, [&](float x, int i) {
        unsigned long long p = (static_cast<unsigned long long>(okey(x)) << 32) |
                               static_cast<uint32_t>(~static_cast<uint32_t>(i));
        best = p > best ? p : best;
      });
    }
    best = block_max_u64(best, ctl, tid);
    int id = static_cast<int>(~static_cast<uint32_t>(best & 0xffffffffull));
    float x0 = 0.f;
    rv.visit(0, [&](float x, int i) { if (i == 0) x0 = x; });
    if (x0 != x0) id = 0;
    fill_probs(0.0);
    __syncthreads();
    if (A.out_probs && tid == 0) A.out_probs[row_id * static_cast<int64_t>(V) + id] = 1.0;
    dbg.kept = 1;
    finish(id, 0u, dbg);
    return;
  }
  if (!(Tm > 0.0f) || !(Tm < INFINITY)) {  // negative, NaN or infinite temperature
    fill_probs(__longlong_as_double(0x7ff8000000000000ll));
    finish(-1, FLAG_BAD_CFG, dbg);
    return;
  }

  const int topk = (cfg.top_k > 0 && cfg.top_k < V) ? cfg.top_k : 0;     // generate.go:157
  const bool topp_on = (cfg.top_p > 0.0f && cfg.top_p < 1.0f);           // generate.go:184
  const int mode = cfg.topp_mode;
  const double u = A.uniforms[row_id];
  // Mode A prunes only while the mass exceeds 1.5*p; the mass starts at 1 up to
  // a few 1e-11 of rounding and 1.5*float(p) is never that close to 1.
  const double plim = (mode == 0) ? static_cast<double>(cfg.top_p) * 1.5 : static_cast<double>(cfg.top_p);
  const bool cut_on = topp_on && !(mode == 0 && plim >= 1.0);

  const bool small_path = (topk > 0 && topk <= KFAST_MAX) || (V <= KEPT_CAP);
  uint32_t flags = 0;
  float xmax = -INFINITY;
  bool nan_seen = false;
  bool need_general = !small_path;
  float flt_lo = -INFINITY;   // full-row path: live elements are x >= flt_lo
  int nk = 0;

  // ------------------------------------------------ pass 1 (small-set path)
  if (small_path) {
    const int kk = topk > 0 ? topk : V;   // no top-k: keep everything (V <= KEPT_CAP)
    float thr = -INFINITY;
    // Tiles of NT*U vectors; the first tile is one vector per thread so the
    // buffer cannot overflow before a threshold exists.
    int vbeg = 0;
    bool first = true;
    while (vbeg < rv.nvec) {   // uniform loop
      const int U = first ? 1 : 2;
      const int tile_vecs = first ? (CAND_CAP / VEC) : 2 * NT;
      const int tstride = first ? (CAND_CAP / VEC) : NT;
      const bool tactive = tid < tstride;
      bool settled = false;
      uint4 raw[2];
      uint32_t pend[2] = {0u, 0u};  // per-vector bitmask of elements still to append
#pragma unroll
      for (int j = 0; j < 2; j++) {
        int v = vbeg + j * tstride + tid;
        if (j < U && tactive && v < rv.nvec) {
          raw[j] = __ldg(rv.vbase + v);
          rv.visit_raw(raw[j], v, [&](float x, int i, int cix) {
            xmax = fmaxf(xmax, x);
            nan_seen |= (x != x);
            if (x >= thr) pend[j] |= (1u << cix);
          });
        }
      }
      // append with overflow / redo
      for (int attempt = 0; attempt < 16; attempt++) {   // uniform loop
#pragma unroll
        for (int j = 0; j < 2; j++) {
          int v = vbeg + j * tstride + tid;
          if (pend[j]) {
            rv.visit_raw(raw[j], v, [&](float x, int i, int cix) {
              if ((pend[j] >> cix) & 1u) {
                if (x >= thr) {
                  int slot = atomicAdd(&ctl.cand_count, 1);
                  if (slot < CAND_CAP) {
                    cand[slot] = make_uint2(__float_as_uint(x), static_cast<uint32_t>(i));
                    pend[j] &= ~(1u << cix);
                  } else {
                    ctl.overflow = 1;
                  }
                } else {
                  pend[j] &= ~(1u << cix);
                }
              }
            });
          }
        }
        __syncthreads();
        int ovf = ctl.overflow;
        int cnt = min(ctl.cand_count, CAND_CAP);
        __syncthreads();   // everybody has read the counters before anyone appends again
        bool last_tile = (vbeg + tile_vecs >= rv.nvec);
        bool do_prune = ovf || (cnt > CAND_CAP / 2) || (last_tile && !ovf);
        if (!do_prune) { settled = true; break; }
        __syncthreads();
        if (tid == 0) { ctl.cand_count = cnt; ctl.overflow = 0; }
        if (cnt > kk) {
          uint32_t kkey = block_select_kth(cand, cnt, kk, hist, ctl, tid);
          if (tid == 0) ctl.thr = quotient_class_floor(okey_to_float(kkey), Tm);
          __syncthreads();
          thr = ctl.thr;
          // compact: keep entries >= thr
          uint2 mine[CAND_CAP / NT];
#pragma unroll
          for (int j = 0; j < CAND_CAP / NT; j++) {
            int e = tid + j * NT;
            mine[j] = (e < cnt) ? cand[e] : make_uint2(0xffc00000u, 0u);  // NaN: dropped
          }
          __syncthreads();
          if (tid == 0) ctl.cand_count = 0;
          __syncthreads();
#pragma unroll
          for (int j = 0; j < CAND_CAP / NT; j++) {
            if (__uint_as_float(mine[j].x) >= thr) {
              int slot = atomicAdd(&ctl.cand_count, 1);
              cand[slot] = mine[j];
            }
          }
          __syncthreads();
          cnt = ctl.cand_count;
        } else {
          __syncthreads();
        }
        if (cnt > (CAND_CAP * 3) / 4) {   // ties at the threshold fill the buffer
          need_general = true;
          break;
        }
        if (!ovf) { settled = true; break; }
      }
      if (!settled) need_general = true;
      if (need_general) break;
      vbeg += tile_vecs;
      first = false;
    }
    if (!need_general) {
      nk = ctl.cand_count;
      if (nk > KEPT_CAP) need_general = true;
    }
    if (need_general) {
      // the streaming pass stopped early: redo the max over the whole row below
      xmax = -INFINITY;
      nan_seen = false;
    }
  }

  // ------------------------------------------------ pass 1 (full-row path)
  if (need_general) {
    for (int v = tid; v < rv.nvec; v += NT) {
      rv.visit(v, [&](float x, int i) {
        xmax = fmaxf(xmax, x);
        nan_seen |= (x != x);
      });
    }
  }
  {
    int anynan = block_max_i(nan_seen ? 1 : 0, ctl, tid);
    unsigned long long p = block_max_u64(static_cast<unsigned long long>(okey(xmax)) << 32, ctl, tid);
    xmax = okey_to_float(static_cast<uint32_t>(p >> 32));
    nan_seen = anynan != 0;
  }
  const float m = scale_t(xmax, Tm);   // max of scaled == scaled max: division by T > 0 is monotone
  dbg.max_scaled = m;
  // A NaN anywhere, or an infinite maximum, makes the softmax sum NaN in the
  // reference (generate.go:173-181); every comparison in the walk then fails
  // and it returns n-1 (generate.go:239).
  if (nan_seen || !(fabsf(m) < INFINITY)) {
    fill_probs(__longlong_as_double(0x7ff8000000000000ll));
    dbg.sum_exp = __longlong_as_double(0x7ff8000000000000ll);
    finish(V - 1, FLAG_NONFINITE | FLAG_FALLBACK, dbg);
    return;
  }

  // ================================================== small-set finale
  if (!need_general) {
    dbg.path = 1;
    float* sx = reinterpret_cast<float*>(pool + POOL_HIST);             // [1024] scaled, index order
    int* sidx = reinterpret_cast<int*>(pool + POOL_HIST + 4096);        // [1024]
    double* se = reinterpret_cast<double*>(pool + POOL_HIST + 8192);    // [1024] e, then q
    double* sf = reinterpret_cast<double*>(pool + POOL_X);              // [1024] scan scratch / final
    int* ord = reinterpret_cast<int*>(pool + POOL_Y);                   // [1024]
    int* rnk = reinterpret_cast<int*>(pool + POOL_Y + 4096);            // [1024]
    __syncthreads();
    // order by index
    for (int j = tid; j < nk; j += NT) {
      uint32_t myi = cand[j].y;
      int r = 0;
      for (int l = 0; l < nk; l++) r += (cand[l].y < myi) ? 1 : 0;
      float s = scale_t(__uint_as_float(cand[j].x), Tm);
      sx[r] = s;
      sidx[r] = static_cast<int>(myi);
    }
    __syncthreads();
    float thr_s = INFINITY;
    for (int j = tid; j < nk; j += NT) {
      float s = sx[j];
      thr_s = fminf(thr_s, s);
      float d = s - m;                                  // f32 subtract (generate.go:176)
      se[j] = exp(static_cast<double>(d));
      sf[j] = se[j];
    }
    if (topk > 0) {   // smallest kept scaled value = the top-k threshold (generate.go:158)
      unsigned long long pk = block_max_u64(~static_cast<unsigned long long>(okey(thr_s)), ctl, tid);
      dbg.threshold = okey_to_float(static_cast<uint32_t>(~pk));
    }
    __syncthreads();
    smem_scan_incl<2>(sf, nk, ctl, tid);
    const double S = sf[nk - 1];
    dbg.sum_exp = S;
    __syncthreads();
    for (int j = tid; j < nk; j += NT) se[j] = se[j] / S;     // generate.go:179-181
    __syncthreads();
    double resum = 1.0;
    bool all_removed = false;
    if (topp_on && mode == 0) {
      // generate.go:184-228. Removal order: ascending (prob, index) over positives.
      int np_loc = 0;
      for (int j = tid; j < nk; j += NT) {
        double qj = se[j];
        int r = -1;
        if (qj > 0) {
          r = 0;
          for (int l = 0; l < nk; l++) {
            double ql = se[l];
            r += (ql > 0 && (ql < qj || (ql == qj && l < j))) ? 1 : 0;
          }
          np_loc++;
        }
        rnk[j] = r;
      }
      int np = block_sum_i(np_loc, ctl, tid);
      // suffix sums in removal order: sf[t] = q of rank (np-1-t), scanned
      for (int j = tid; j < nk; j += NT) if (rnk[j] >= 0) sf[np - 1 - rnk[j]] = se[j];
      __syncthreads();
      smem_scan_incl<2>(sf, np, ctl, tid);
      // remaining mass after removing r smallest = sf[np-1-r] (r < np), 0 for r = np
      int rstar_loc = np;
      for (int r = tid; r < np; r += NT) {
        if (sf[np - 1 - r] <= plim) { rstar_loc = min(rstar_loc, r); }
      }
      int rstar = block_min_i(rstar_loc, ctl, tid);
      if (rstar == np) {
        all_removed = true;     // every token zeroed: resum = 0, probs 0/0 (generate.go:221-227)
      } else {
        resum = sf[np - 1 - rstar];
        double at = sf[np - 1 - rstar];
        if (fabs(at - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
        if (rstar > 0 && fabs(sf[np - rstar] - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
      }
      __syncthreads();
      for (int j = tid; j < nk; j += NT) {
        double qj = se[j];
        if (rnk[j] >= 0 && rnk[j] < rstar) qj = 0.0;
        sf[j] = all_removed ? __longlong_as_double(0x7ff8000000000000ll) : qj / resum;
      }
      dbg.resum = all_removed ? 0.0 : resum;
    } else if (topp_on) {
      // qwen/generate.go:123-153. Descending prob, equal probs by ascending index.
      for (int j = tid; j < nk; j += NT) {
        double qj = se[j];
        int r = 0;
        for (int l = 0; l < nk; l++) {
          double ql = se[l];
          r += (ql > qj || (ql == qj && l < j)) ? 1 : 0;
        }
        rnk[j] = r;
        ord[r] = j;
      }
      __syncthreads();
      for (int r = tid; r < nk; r += NT) sf[r] = se[ord[r]];
      __syncthreads();
      smem_scan_incl<2>(sf, nk, ctl, tid);
      int cut_loc = nk;
      for (int r = tid; r < nk; r += NT) if (sf[r] >= plim) cut_loc = min(cut_loc, r + 1);
      int cutn = block_min_i(cut_loc, ctl, tid);
      resum = sf[cutn - 1];
      if (fabs(resum - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
      if (cutn >= 2 && fabs(sf[cutn - 2] - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
      if (cutn < nk && se[ord[cutn]] == se[ord[cutn - 1]]) flags |= FLAG_TIE_CUT;
      __syncthreads();
      for (int j = tid; j < nk; j += NT) sf[j] = (rnk[j] < cutn) ? se[j] / resum : 0.0;
      dbg.resum = resum;
    } else {
      for (int j = tid; j < nk; j += NT) sf[j] = se[j];
    }
    __syncthreads();
    if (all_removed) {
      fill_probs(__longlong_as_double(0x7ff8000000000000ll));
      finish(V - 1, flags | FLAG_NONFINITE | FLAG_FALLBACK, dbg);
      return;
    }
    // final probabilities are in sf (index order); write them out if asked
    int kept_loc = 0;
    for (int j = tid; j < nk; j += NT) kept_loc += (sf[j] > 0) ? 1 : 0;
    dbg.kept = block_sum_i(kept_loc, ctl, tid);
    if (A.out_probs) {
      fill_probs(0.0);
      __syncthreads();
      double* pr = A.out_probs + row_id * static_cast<int64_t>(V);
      for (int j = tid; j < nk; j += NT) pr[sidx[j]] = sf[j];
    }
    // draw (generate.go:231-239): first index with u < cumulative
    for (int j = tid; j < nk; j += NT) se[j] = sf[j];
    __syncthreads();
    smem_scan_incl<2>(se, nk, ctl, tid);
    int pick_loc = nk;
    for (int j = tid; j < nk; j += NT) if (u < se[j]) pick_loc = min(pick_loc, j);
    int pick = block_min_i(pick_loc, ctl, tid);
    int id;
    if (pick < nk) {
      id = sidx[pick];
      double hi = se[pick], lo = hi - sf[pick];
      if (pick > 0) lo = se[pick - 1];
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

  // ================================================== full-row path
  dbg.path = 2;
  flags |= FLAG_GENERAL_PATH;
  const bool t_is_one = (Tm == 1.0f);

  // ---- exact top-k threshold by counting (only when the streaming path could not serve)
  if (topk > 0) {
    uint32_t prefix = 0, mask = 0;
    int need = topk;
    const int shifts[3] = {21, 10, 0};
    const int widths[3] = {11, 11, 10};
    for (int round = 0; round < 3; round++) {
      const int sh = shifts[round];
      const int nb = 1 << widths[round];
      __syncthreads();
      for (int j = tid; j < nb; j += NT) hist[j] = 0;
      __syncthreads();
      for (int v = tid; v < rv.nvec; v += NT) {
        rv.visit(v, [&](float x, int i) {
          uint32_t key = okey(x);
          if ((key & mask) == prefix) atomicAdd(&hist[(key >> sh) & (nb - 1)], 1u);
        });
      }
      __syncthreads();
      // find the bin (from the top) where the running count reaches `need`
      {
        constexpr int PER = 2048 / NT;
        int loc[PER];
        int s = 0;
        // thread t owns bins descending: top-first order position p = t*PER + j <-> bin nb-1-p
#pragma unroll
        for (int j = 0; j < PER; j++) {
          int p = tid * PER + j;
          int c = (p < nb) ? static_cast<int>(hist[nb - 1 - p]) : 0;
          s += c;
          loc[j] = s;
        }
        // exclusive scan of s over threads (int): reuse double scan for simplicity of code
        double tot;
        double ex = block_scan_excl_d(static_cast<double>(s), tot, ctl, tid);
        int before = static_cast<int>(ex);
        if (before < need && before + s >= need) {
#pragma unroll
          for (int j = 0; j < PER; j++) {
            if (before + loc[j] >= need) {
              int p = tid * PER + j;
              int c = static_cast<int>(hist[nb - 1 - p]);
              ctl.bcast_i[0] = nb - 1 - p;
              ctl.bcast_i[1] = need - (before + loc[j] - c);
              break;
            }
          }
        }
      }
      __syncthreads();
      prefix |= static_cast<uint32_t>(ctl.bcast_i[0]) << sh;
      mask |= static_cast<uint32_t>(nb - 1) << sh;
      need = ctl.bcast_i[1];
    }
    if (tid == 0) ctl.thr = quotient_class_floor(okey_to_float(prefix), Tm);
    __syncthreads();
    flt_lo = ctl.thr;
    dbg.threshold = scale_t(okey_to_float(prefix), Tm);
  }
  const bool filt = topk > 0;

  // segments
  int seg_vecs = SEG_VECS_MIN;
  {
    int need_sv = (rv.nvec + MAXSEG - 1) / MAXSEG;
    if (need_sv > seg_vecs) seg_vecs = ((need_sv + 31) / 32) * 32;
  }
  const int nseg = (rv.nvec + seg_vecs - 1) / seg_vecs;

  // ---- pass 2: count histogram over level-0 buckets, zone bracket
  if (tid == 0) { cut.active = 0; cut.b1 = 0; cut.b2 = NBUCKET - 1; cut.mode = mode; cut.idx_c = -1; cut.e_c = INFINITY; cut.incl = 1; }
  int nzone = 0;
  __syncthreads();
  if (cut_on) {
    for (int j = tid; j < NBUCKET; j += NT) hist[j] = 0;
    __syncthreads();
    for (int v = tid; v < rv.nvec; v += NT) {
      rv.visit(v, [&](float x, int i) {
        if (!filt || x >= flt_lo) {
          float s = t_is_one ? x : __fdiv_rn(x, Tm);
          atomicAdd(&hist[bucket0(s - m)], 1u);
        }
      });
    }
    __syncthreads();
    // bounds on bucket masses: bucket b holds d in [-(b+.5)/128, -(b-.5)/128];
    // the last bucket holds everything at or below -31.99 (mass down to 0).
    constexpr int PER = NBUCKET / NT;
    double lo_inc[PER], hi_inc[PER];
    double slo = 0.0, shi = 0.0;
#pragma unroll
    for (int j = 0; j < PER; j++) {
      int b = tid * PER + j;
      double c = static_cast<double>(hist[b]);
      double elo = (b == NBUCKET - 1) ? 0.0 : exp(-(b + 0.5) / 128.0) * (1.0 - 1e-7);
      double ehi = fmin(1.0, exp(-(b - 0.5) / 128.0) * (1.0 + 1e-7));
      slo += c * elo; shi += c * ehi;
      lo_inc[j] = slo; hi_inc[j] = shi;
    }
    double tot_lo, tot_hi;
    double ex_lo = block_scan_excl_d(slo, tot_lo, ctl, tid);
    double ex_hi = block_scan_excl_d(shi, tot_hi, ctl, tid);
    int b1_loc = NBUCKET - 1, b2_loc = NBUCKET - 1;
#pragma unroll
    for (int j = 0; j < PER; j++) {
      int b = tid * PER + j;
      double a_lo = ex_lo + lo_inc[j], a_hi = ex_hi + hi_inc[j];
      double r_hi = a_hi / (a_hi + (tot_lo - a_lo));   // largest possible mass fraction through bucket b
      double r_lo = a_lo / (a_lo + (tot_hi - a_hi));   // smallest possible
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
      if (b >= b1 && b <= b2) nz_loc += static_cast<int>(hist[b]);
    }
    nzone = block_sum_i(nz_loc, ctl, tid);
    if (tid == 0) { cut.active = 1; cut.b1 = b1; cut.b2 = b2; }
    __syncthreads();
  }
  const int zb1 = cut.b1, zb2 = cut.b2;
  const bool cut_active = cut.active != 0;

  // ---- pass 3: exponentials, per-segment kept mass, zone list
  __syncthreads();
  if (tid == 0) ctl.cand_count = 0;
  for (int j = tid; j < MAXSEG; j += NT) s_kseg[j] = 0.0;
  __syncthreads();
  double Ktot_l = 0.0, Dtot_l = 0.0;
  for (int sg = warp; sg < nseg; sg += NW) {
    int v0 = sg * seg_vecs, v1 = min(rv.nvec, v0 + seg_vecs);
    double kacc = 0.0;
    for (int v = v0 + lane; v < v1; v += 32) {
      rv.visit(v, [&](float x, int i) {
        if (!filt || x >= flt_lo) {
          float s = t_is_one ? x : __fdiv_rn(x, Tm);
          float d = s - m;
          if (cut_active) {
            int b = bucket0(d);
            if (b < zb1) {
              kacc += exp_neg_f64(d, s_tab);
            } else if (b > zb2) {
              Dtot_l += exp_neg_f64(d, s_tab);
            } else {
              int slot = atomicAdd(&ctl.cand_count, 1);
              if (slot < CAND_CAP) cand[slot] = make_uint2(__float_as_uint(d), static_cast<uint32_t>(i));
            }
          } else {
            kacc += exp_neg_f64(d, s_tab);
          }
        }
      });
    }
    kacc = warp_sum_d(kacc);
    if (lane == 0) s_kseg[sg] = kacc;
    Ktot_l += (lane == 0) ? kacc : 0.0;
  }
  double Ktot = block_sum_d(Ktot_l, ctl, tid);
  double Dtot = block_sum_d(Dtot_l, ctl, tid);
  __syncthreads();
  double S = Ktot + Dtot;     // + zone mass below
  double Re = Ktot;           // kept mass in exp units
  int kept_zone = 0;

  // A zone that outgrew the list (long runs of equal logits around the cut) is cut by the same
  // rule applied to the row itself: weighted selection on the keys (d, index), one pass per round.
  const bool big_zone = cut_active && ctl.cand_count > CAND_CAP;
  if (big_zone) {
    auto each_zone = [&](auto&& fn) {
      for (int v = tid; v < rv.nvec; v += NT) {
        rv.visit(v, [&](float x, int i) {
          if (!filt || x >= flt_lo) {
            const float s = t_is_one ? x : __fdiv_rn(x, Tm);
            const float d = s - m;
            const int b = bucket0(d);
            if (b >= zb1 && b <= zb2) fn(zone_key(d, i, mode), d);
          }
        });
      }
    };
    auto crossed = [&](double g) -> bool { return mode == 0 ? (g / S > plim) : (g / S >= plim); };
    double* sm = reinterpret_cast<double*>(pool + POOL_HIST);          // [NT] mass per sub-bucket
    int* scn = reinterpret_cast<int*>(pool + POOL_HIST + NT * 8);      // [NT] count per sub-bucket
    unsigned long long* few = reinterpret_cast<unsigned long long*>(pool + POOL_X);   // [32]
    unsigned long long lo = ~0ull, hi = 0ull;
    double z_loc = 0.0;
    int n_loc = 0;
    each_zone([&](unsigned long long k, float d) { lo = k < lo ? k : lo; hi = k > hi ? k : hi; z_loc += exp_neg_f64(d, s_tab); n_loc++; });
    const double Z = block_sum_d(z_loc, ctl, tid);
    int inrange = block_sum_i(n_loc, ctl, tid);
    lo = ~block_max_u64(~lo, ctl, tid);
    hi = block_max_u64(hi, ctl, tid);
    S = Ktot + Z + Dtot;
    bool bad = (Ktot > 0.0 && crossed(Ktot));                  // bracket violated
    double gbase = Ktot;
    bool all_in = false;
    for (int iter = 0; iter < 10 && inrange > 32 && !bad && !all_in; iter++) {
      const unsigned long long spn = hi - lo;
      int shf = 0;
      while (shf < 63 && (spn >> shf) >= static_cast<unsigned long long>(NT)) shf++;
      __syncthreads();
      sm[tid] = 0.0; scn[tid] = 0;
      __syncthreads();
      each_zone([&](unsigned long long k, float d) {
        if (k >= lo && k <= hi) {
          const int sb = static_cast<int>((k - lo) >> shf);
          atomicAdd(&sm[sb], exp_neg_f64(d, s_tab));
          atomicAdd(&scn[sb], 1);
        }
      });
      __syncthreads();
      const double mine = sm[tid];
      double totm;
      const double exm = block_scan_excl_d(mine, totm, ctl, tid);
      const int first = (scn[tid] > 0 && crossed(gbase + exm + mine)) ? tid : NT;
      const int sbx = block_min_i(first, ctl, tid);
      if (sbx == NT) { all_in = true; break; }
      if (tid == sbx) { ctl.bcast_d[0] = gbase + exm; ctl.bcast_i[0] = scn[tid]; }
      __syncthreads();
      gbase = ctl.bcast_d[0];
      inrange = ctl.bcast_i[0];
      const unsigned long long nlo = lo + (static_cast<unsigned long long>(sbx) << shf);
      unsigned long long nhi = nlo + ((1ull << shf) - 1ull);
      if (nhi < nlo || nhi > hi) nhi = hi;
      lo = nlo; hi = nhi;
    }
    if (inrange > 32 && !all_in) bad = true;
    unsigned long long cut_key = ~0ull;
    int cut_incl = 1;
    double g_at = gbase, g_before = gbase;
    if (!bad && !all_in) {
      __syncthreads();
      if (tid == 0) ctl.cand_count = 0;
      __syncthreads();
      each_zone([&](unsigned long long k, float) {
        if (k >= lo && k <= hi) { const int slot = atomicAdd(&ctl.cand_count, 1); if (slot < 32) few[slot] = k; }
      });
      __syncthreads();
      const int nf = min(32, ctl.cand_count);
      if (warp == 0) {
        const unsigned long long k = (lane < nf) ? few[lane] : ~0ull;
        const double e = (lane < nf) ? exp_neg_f64(zone_key_d(k), s_tab) : 0.0;
        double g = gbase;
        for (int l = 0; l < nf; l++) {
          const unsigned long long kl = __shfl_sync(FULL, k, l);
          const double el = __shfl_sync(FULL, e, l);
          if (kl <= k) g += el;
        }
        const bool cr = (lane < nf) && crossed(g);
        unsigned long long candk = cr ? k : ~0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const unsigned long long tt = __shfl_xor_sync(FULL, candk, o);
          candk = tt < candk ? tt : candk;
        }
        const unsigned who = __ballot_sync(FULL, cr && k == candk);
        if (lane == 0) { ctl.red_u64[0] = candk; ctl.bcast_i[1] = who ? 1 : 0; }
        if (who && lane == __ffs(who) - 1) { ctl.bcast_d[1] = g; ctl.bcast_d[2] = g - e; }
      }
      __syncthreads();
      if (ctl.bcast_i[1]) {
        cut_key = ctl.red_u64[0];
        g_at = ctl.bcast_d[1];
        g_before = ctl.bcast_d[2];
        cut_incl = (mode == 0) ? 0 : 1;
      } else {
        all_in = true;
      }
      __syncthreads();
    }
    if (!bad && all_in) {
      cut_key = ~0ull; cut_incl = 1;
      if (mode == 1 && !(Dtot == 0.0)) bad = true;             // the bracket promised the cut inside the zone
    }
    if (bad) {
      fill_probs(__longlong_as_double(0x7ff8000000000000ll));
      finish(-1, flags | FLAG_INTERNAL, dbg);
      return;
    }
    if (!all_in) {
      if (fabs(g_at / S - plim) <= 1e-12 || fabs(g_before / S - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
      if (mode == 1) {
        int tie = 0;
        each_zone([&](unsigned long long k, float) { tie |= (k > cut_key && (k >> 32) == (cut_key >> 32)) ? 1 : 0; });
        if (block_max_i(tie, ctl, tid)) flags |= FLAG_TIE_CUT;
      }
    }
    Re = all_in ? Ktot + Z : ((mode == 0) ? g_before : g_at);
    __syncthreads();
    each_zone([&](unsigned long long k, float d) {
      if (k < cut_key || (cut_incl && k == cut_key)) {
        atomicAdd(&s_kseg[rv.vec_of(zone_key_index(k, mode)) / seg_vecs], exp_neg_f64(d, s_tab));
      }
    });
    if (tid == 0) {
      if (all_in) { cut.e_c = -1.0; cut.idx_c = -1; cut.incl = 1; }
      else { cut.e_c = exp_neg_f64(zone_key_d(cut_key), s_tab); cut.idx_c = zone_key_index(cut_key, mode); cut.incl = cut_incl; }
    }
    __syncthreads();
  } else if (cut_active) {
    const int nz = min(ctl.cand_count, CAND_CAP);
    double* ze = reinterpret_cast<double*>(pool + POOL_HIST);   // [2048] mass per zone entry
    double* zs = reinterpret_cast<double*>(pool + POOL_X);      // [2048] masses in cut order, scanned
    uint16_t* zrank = reinterpret_cast<uint16_t*>(pool + POOL_Y);          // [2048]
    uint16_t* zord = reinterpret_cast<uint16_t*>(pool + POOL_Y + 4096);    // [2048]
    for (int j = tid; j < nz; j += NT) ze[j] = exp_neg_f64(__uint_as_float(cand[j].x), s_tab);
    __syncthreads();
    // cut order: descending mass; equal masses by ascending index (mode B) or
    // descending index (mode A removes the lowest index first, generate.go:208-212)
    for (int j = tid; j < nz; j += NT) {
      double ej = ze[j];
      uint32_t ij = cand[j].y;
      int r = 0;
      for (int l = 0; l < nz; l++) {
        double el = ze[l];
        uint32_t il = cand[l].y;
        bool before = (el > ej) || (el == ej && (mode == 0 ? il > ij : il < ij));
        r += before ? 1 : 0;
      }
      zrank[j] = static_cast<uint16_t>(r);
      zord[r] = static_cast<uint16_t>(j);
      zs[r] = ej;
    }
    __syncthreads();
    smem_scan_incl<4>(zs, nz, ctl, tid);
    const double Z = nz > 0 ? zs[nz - 1] : 0.0;
    S = Ktot + Z + Dtot;
    // number of zone entries kept
    int cnt_loc;
    if (mode == 0) {
      // kept prefix: remaining mass (K + prefix)/S <= 1.5p, largest such prefix
      cnt_loc = 0;
      for (int r = tid; r < nz; r += NT) if ((Ktot + zs[r]) / S <= plim) cnt_loc = max(cnt_loc, r + 1);
      kept_zone = block_max_i(cnt_loc, ctl, tid);
      if (Ktot > 0.0 && Ktot / S > plim) flags |= FLAG_INTERNAL;   // bracket violated
    } else {
      cnt_loc = nz + 1;
      for (int r = tid; r < nz; r += NT) if ((Ktot + zs[r]) / S >= plim) cnt_loc = min(cnt_loc, r + 1);
      kept_zone = block_min_i(cnt_loc, ctl, tid);
      if (Ktot > 0.0 && Ktot / S >= plim) flags |= FLAG_INTERNAL;  // bracket violated
      if (kept_zone == nz + 1) {
        // the bracket promised the cut inside the zone
        if (!(Dtot == 0.0)) flags |= FLAG_INTERNAL;
        kept_zone = nz;
      }
    }
    const double Zk = kept_zone > 0 ? zs[kept_zone - 1] : 0.0;
    Re = Ktot + Zk;
    {
      double at = (Ktot + Zk) / S;
      if (fabs(at - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
      if (kept_zone < nz && fabs((Ktot + zs[kept_zone]) / S - plim) <= 1e-12) flags |= FLAG_TOPP_EDGE;
      if (kept_zone > 0 && kept_zone < nz && ze[zord[kept_zone]] == ze[zord[kept_zone - 1]]) flags |= FLAG_TIE_CUT;
    }
    __syncthreads();
    for (int j = tid; j < nz; j += NT) {
      if (zrank[j] < kept_zone) atomicAdd(&s_kseg[rv.vec_of(static_cast<int>(cand[j].y)) / seg_vecs], ze[j]);
    }
    if (tid == 0) {
      if (kept_zone > 0) { int j = zord[kept_zone - 1]; cut.e_c = ze[j]; cut.idx_c = static_cast<int>(cand[j].y); }
      else { cut.e_c = INFINITY; cut.idx_c = -1; }
    }
    __syncthreads();
  }
  dbg.sum_exp = S;
  dbg.resum = Re / S;
  if (!(Re > 0.0)) {
    // mode A removed every token (generate.go:221-227 divides by zero)
    fill_probs(__longlong_as_double(0x7ff8000000000000ll));
    dbg.resum = 0.0;
    finish(V - 1, flags | FLAG_NONFINITE | FLAG_FALLBACK, dbg);
    return;
  }
  const double ec = cut.e_c;
  const int idxc = cut.idx_c;
  const bool cincl = cut.incl != 0;
  // kept mass of one element (0 when filtered or cut away)
  auto kept_mass = [&](float x, int i) -> double {
    if (filt && !(x >= flt_lo)) return 0.0;
    float s = t_is_one ? x : __fdiv_rn(x, Tm);
    float d = s - m;
    double e = exp_neg_f64(d, s_tab);
    if (cut_active) {
      int b = bucket0(d);
      if (b > zb2) return 0.0;
      if (b >= zb1) {
        bool keep = (e > ec) || (e == ec && (mode == 0 ? (cincl ? i >= idxc : i > idxc) : (cincl ? i <= idxc : i < idxc)));
        if (!keep) return 0.0;
      }
    }
    return e;
  };

  // ---- optional dense probabilities and kept count (parity runs only)
  if (A.out_probs || A.out_debug) {
    double* pr = A.out_probs ? A.out_probs + row_id * static_cast<int64_t>(V) : nullptr;
    const double rq = Re / S;
    int kept_loc = 0;
    for (int v = tid; v < rv.nvec; v += NT) {
      rv.visit(v, [&](float x, int i) {
        double e = kept_mass(x, i);
        double f = (e / S) / rq;
        kept_loc += (f > 0) ? 1 : 0;
        if (pr) pr[i] = f;
      });
    }
    dbg.kept = block_sum_i(kept_loc, ctl, tid);
  }

  // ---- locate the segment where u is crossed, then rescan segments from there
  // cumulative through element i is prefix_mass(i) / Re
  // (u < prefix/Re is tested as u*Re < prefix: one rounding instead of a division per element)
  const double tgt = u * Re;
  double segbase = 0.0;
  int sg0 = nseg;
  if (tid == 0) {
    double acc = 0.0;
    int found = nseg;
    double base_found = 0.0;
    for (int sgi = 0; sgi < nseg; sgi++) {
      double nxt = acc + s_kseg[sgi];
      if (tgt < nxt) { found = sgi; base_found = acc; break; }
      acc = nxt;
    }
    if (found == nseg) base_found = acc;
    ctl.bcast_i[2] = found;
    ctl.bcast_d[0] = base_found;
  }
  __syncthreads();
  sg0 = ctl.bcast_i[2];
  segbase = ctl.bcast_d[0];
  int id = -1;
  double edge_lo = 0.0, edge_hi = 0.0;
  for (int sg = sg0; sg < nseg; sg++) {     // uniform loop; normally one trip
    int v0 = sg * seg_vecs, v1 = min(rv.nvec, v0 + seg_vecs);
    // chunks of NT vectors, each thread one vector, in index order
    for (int vb = v0; vb < v1; vb += NT) {
      int v = vb + tid;
      double em[VEC];
      double tsum = 0.0;
#pragma unroll
      for (int c = 0; c < VEC; c++) em[c] = 0.0;
      if (v < v1) {
        uint4 raw = __ldg(rv.vbase + v);
        rv.visit_raw(raw, v, [&](float x, int i, int cix) {
          double e = kept_mass(x, i);
          em[cix] = e;
        });
#pragma unroll
        for (int c = 0; c < VEC; c++) tsum += em[c];
      }
      double tot;
      double ex = block_scan_excl_d(tsum, tot, ctl, tid);
      int pick_loc = 0x7fffffff;
      double run = segbase + ex;
      if (v < v1) {
#pragma unroll
        for (int c = 0; c < VEC; c++) {
          double before = run;
          run += em[c];
          if (em[c] > 0.0 && tgt < run && pick_loc == 0x7fffffff) {
            pick_loc = v * VEC - rv.shift + c;
            edge_lo = before / Re; edge_hi = run / Re;
          }
        }
      }
      int pick = block_min_i(pick_loc, ctl, tid);
      if (pick != 0x7fffffff) {
        if (pick_loc == pick) { ctl.bcast_d[1] = edge_lo; ctl.bcast_d[2] = edge_hi; }
        __syncthreads();
        id = pick;
        edge_lo = ctl.bcast_d[1]; edge_hi = ctl.bcast_d[2];
        break;
      }
      segbase += tot;
    }
    if (id >= 0) break;
  }
  if (id >= 0) {
    dbg.edge_lo = edge_lo; dbg.edge_hi = edge_hi;
    if ((edge_lo > 0.0 && u - edge_lo <= 1e-6) || edge_hi - u <= 1e-6) flags |= FLAG_BOUNDARY;
  } else {
    id = V - 1;
    flags |= FLAG_FALLBACK;
    dbg.edge_lo = dbg.edge_hi = segbase / Re;
    if (u - segbase / Re <= 1e-6) flags |= FLAG_BOUNDARY;
  }
  finish(id, flags, dbg);
}

// One CTA per row; with a work list, a fixed grid walks the listed rows.
template <typename T>
__global__ void __launch_bounds__(NT, 2) sample_rows_kernel(KernelArgs A) {
  extern __shared__ __align__(16) unsigned char pool[];
  if (A.worklist) {
    const int n = A.worklist[0];
    for (int w = blockIdx.x; w < n; w += gridDim.x) {
      single_cta_row<T>(A, A.worklist[1 + w], pool);
      __syncthreads();
    }
  } else {
    const int64_t row = A.row_offset + blockIdx.x;
    if (A.row_done && A.row_done[row] != 0) return;        // the sequence has ended (model/generate.go:82-84)
    single_cta_row<T>(A, row, pool);
  }
}

}  // namespace gs
