// Row softmax, log-softmax and cross-entropy over [B, V] logits at vocabulary scale
// (ops.go:527-563 Softmax, :566-603 LogSoftmax; loss.go:55-124 CrossEntropyLoss forward,
// :128-141 its backward; the Metal kernels they replace: metal/kernels.go:348-432).
//
// One 1024-thread CTA per SM; a row at a time per CTA, or per pair of CTAs (a cluster of two) when
// rows are long. The rows being worked on stay in L2 between the two passes of the ops that write
// [B, V], so HBM sees each logit once and each output once.
//   pass 1   one read of the row: every thread keeps a running maximum m and the sum s of
//            exp(x - m) over its own elements (rescaled when m grows), then the block combines
//            them: M = max m, S = sum s * exp(m - M) in f64.
//   pass 2   softmax: exp(x - M) / S; log-softmax: (x - M) - log S; cross-entropy backward:
//            exp(x - lse) * scale, minus scale at the target. Written with streaming stores.
// Cross-entropy forward needs pass 1 only: lse = M + log S, loss = lse - x[target].
//
// Values follow the reference's expressions with its f32 roundings (x - M in f32, the result of
// exp rounded to f32, lse = M + f32(log(f64(S)))); the sum itself is formed in a different order
// and in higher precision than the reference's sequential f32 loop. NaN and infinities come out
// as upstream: a NaN anywhere, a +Inf, or a row of -Inf only makes the whole row NaN.
#pragma once

#include <cooperative_groups.h>

#include <cstdint>

#include "block_util.cuh"
#include "sample_common.cuh"
#include "sample_kernel.cuh"   // Elem, RowView

namespace gs {

constexpr int RS_NT = 1024;
constexpr int RS_NW = RS_NT / 32;
constexpr int RS_UNROLL = 4;      // 16-byte loads per thread and loop iteration
constexpr int RS_STAGES = 3;      // pass 1: iterations staged in shared memory (two in flight while one is consumed)
constexpr int RS_DYN_BYTES = RS_STAGES * RS_UNROLL * RS_NT * 16;   // 192 KB

constexpr int RS_SOFTMAX = 0;
constexpr int RS_LOG_SOFTMAX = 1;
constexpr int RS_CE_FWD = 2;
constexpr int RS_CE_BWD = 3;

struct RowSoftmaxArgs {
  const void* x;            // [B, row_stride] f32 or bf16
  int64_t row_stride;
  int32_t V;
  int64_t B;
  int32_t mode;
  void* out;                // softmax / log-softmax: [B, out_stride] in x's type; CE backward: f32 dx
  int64_t out_stride;
  const int32_t* targets;   // CE: [B]
  float* row_loss;          // CE forward: [B]
  float* row_lse;           // CE forward: [B] written; CE backward: [B] read
  float scale;              // CE backward: grad / batch
};

// f32 -> bf16 bits, round to nearest even, NaN kept quiet (tensor.go:85-94)
__device__ __forceinline__ uint32_t bf16_bits_rne(float v) {
  const uint32_t b = __float_as_uint(v);
  if (((b >> 23) & 0xffu) == 0xffu && (b & 0x7fffffu) != 0u) return (b >> 16) | 0x40u;
  return (b + 0x7fffu + ((b >> 16) & 1u)) >> 16;
}

// Two f32 in one 64-bit register for the packed FMA pipe (half the issue slots per element).
typedef unsigned long long rs_f2;
__device__ __forceinline__ rs_f2 rs_pk(float a, float b) { rs_f2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ void rs_upk(rs_f2 v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ rs_f2 rs_fma2(rs_f2 a, rs_f2 b, rs_f2 c) { rs_f2 d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ rs_f2 rs_add2(rs_f2 a, rs_f2 b) { rs_f2 d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ rs_f2 rs_mul2(rs_f2 a, rs_f2 b) { rs_f2 d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ float rs_maxnan(float a, float b) { float d; asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b)); return d; }
__device__ __forceinline__ float rs_ex2(float t) { float e; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t)); return e; }

// exp of two f32 arguments, each result within about 3e-7 relative of the correctly rounded one
// (the reference rounds a double exp to f32). exp(d) = 2^t (1 + r ln 2) with t = rn(d log2 e) and
// r = d log2 e - t recovered exactly by an FMA plus the low part of log2 e; 2^t from the special
// function unit (2 ulp). Arguments below -200 give 0 like everything below -104 does in f32 (the
// clamp keeps -Inf from turning into Inf - Inf); a NaN stays a NaN.
__device__ __forceinline__ rs_f2 rs_exp2(float d0, float d1) {
  constexpr float L2E = 1.44269502162933349609375f, L2E_LO = 1.925963033500011e-8f, LN2 = 0.693147182464599609375f;
  const rs_f2 D = rs_pk(rs_maxnan(d0, -200.0f), rs_maxnan(d1, -200.0f));
  const rs_f2 NT = rs_mul2(D, rs_pk(-L2E, -L2E));                       // -t, exactly
  rs_f2 R = rs_fma2(D, rs_pk(L2E, L2E), NT);
  R = rs_fma2(D, rs_pk(L2E_LO, L2E_LO), R);
  float n0, n1;
  rs_upk(NT, n0, n1);
  const rs_f2 P = rs_pk(rs_ex2(-n0), rs_ex2(-n1));
  return rs_fma2(P, rs_mul2(R, rs_pk(LN2, LN2)), P);
}
__device__ __forceinline__ float rs_exp1(float d) {
  float a, b;
  rs_upk(rs_exp2(d, d), a, b);
  return a;
}

// the elements of vector v of the row; those outside the row read -Inf
template <typename T>
__device__ __forceinline__ void rs_unpack(const RowView<T>& rv, int v, const uint4& raw, float* x) {
  constexpr int VEC = Elem<T>::VEC;
  Elem<T>::unpack(raw, x);
  if (v == 0 || v >= rv.nvec - 1) {
    const int i0 = v * VEC - rv.shift;
#pragma unroll
    for (int c = 0; c < VEC; c++) if (i0 + c < 0 || i0 + c >= rv.V) x[c] = -INFINITY;
  }
}

// Pass 1 over the vectors [v0, v1) of the row. Returns their maximum M (NaNs ignored; -Inf when
// there is none) and S = sum exp(x - M) (0 when M is -Inf, NaN when a NaN was seen) to every thread.
template <typename T>
__device__ __forceinline__ void rs_max_sum(const RowView<T>& rv, int v0, int v1, bool primed, const RowView<T>* nrv, int nv0, int nv1,
                                           const uint4* ring, bu::Scratch& sc, int tid, float& M, double& S) {
  constexpr int VEC = Elem<T>::VEC;
  const uint32_t ring_addr = static_cast<uint32_t>(__cvta_generic_to_shared(ring));
  float m = -INFINITY;
  rs_f2 s2 = rs_pk(0.0f, 0.0f);                                // two running sums (even and odd elements)
  // The terms of the sum need no compensated exponential: a term's error from rounding t = d log2 e
  // grows with |t| while the term shrinks as 2^t, and the errors of different terms are independent,
  // so the sum stays within about 1e-7 relative. exp(-Inf) is 0 and a NaN stays NaN without a clamp.
  auto accumulate = [&](const float* x) {
    if (m > -INFINITY) {
      const rs_f2 NM = rs_pk(-m, -m), L = rs_pk(1.44269502162933349609375f, 1.44269502162933349609375f);
#pragma unroll
      for (int c = 0; c < VEC; c += 2) {
        float t0, t1;
        rs_upk(rs_mul2(rs_add2(rs_pk(x[c], x[c + 1]), NM), L), t0, t1);
        s2 = rs_add2(s2, rs_pk(rs_ex2(t0), rs_ex2(t1)));       // a NaN logit turns the sum NaN
      }
    } else {
      // only -Inf and NaN so far: exp(-Inf - -Inf) must not poison the sum, a NaN logit must
      float t = x[0];
#pragma unroll
      for (int c = 1; c < VEC; c++) t += x[c];
      if (t != t) s2 = rs_pk(t, t);
    }
  };
  auto take = [&](int v, const uint4& raw, bool interior) {
    float x[VEC];
    if (interior) Elem<T>::unpack(raw, x);
    else rs_unpack<T>(rv, v, raw, x);
    float vm = x[0];
#pragma unroll
    for (int c = 1; c < VEC; c++) vm = fmaxf(vm, x[c]);
    if (vm > m) {                                              // m = -Inf before: the sums are 0 (or NaN) and stay so
      // the accurate exponential here: in a row that keeps growing (sorted logits) the sums are
      // rescaled at every vector, and the error of a cheaper one would add up over those steps
      const float f = expf(m - vm);
      s2 = rs_mul2(s2, rs_pk(f, f));
      m = vm;
    }
    accumulate(x);
  };
  // Registers could hold 64 KB of loads in flight per SM, which at HBM latency is about half of
  // an SM's share of the bandwidth. So the row is staged through shared memory by asynchronous
  // 16-byte copies: a thread copies the vectors it will consume itself (no barrier, it only waits
  // for its own copy groups), RS_STAGES - 1 iterations (128 KB per SM) ahead of their use.
  // `primed`: the first RS_STAGES - 1 iterations of this range were issued already, at the end of
  // the previous row's pass 1 (they arrived while that row's reduction and second pass ran). At the
  // end of this pass the same is done for the range [nv0, nv1) of the CTA's next row, if any.
  auto issue = [&](const RowView<T>& r, int a0, int a1, int it) {
    const int base = a0 + it * RS_UNROLL * RS_NT + tid;
    const uint32_t dst = ring_addr + static_cast<uint32_t>(((it % RS_STAGES) * RS_UNROLL * RS_NT + tid) * 16);
#pragma unroll
    for (int q = 0; q < RS_UNROLL; q++) {
      if (base + q * RS_NT < a1)                               // also false for every iteration past the range
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst + q * RS_NT * 16), "l"(r.vbase + base + q * RS_NT) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int n_it = (v1 - v0 + RS_UNROLL * RS_NT - 1) / (RS_UNROLL * RS_NT);
  if (!primed) {
#pragma unroll
    for (int st = 0; st < RS_STAGES - 1; st++) issue(rv, v0, v1, st);
  }
  for (int it = 0; it < n_it; it++) {
    issue(rv, v0, v1, it + RS_STAGES - 1);
    asm volatile("cp.async.wait_group %0;" :: "n"(RS_STAGES - 1) : "memory");
    const int first = v0 + it * RS_UNROLL * RS_NT;
    const int base = first + tid;
    const uint4* src = ring + (it % RS_STAGES) * RS_UNROLL * RS_NT + tid;
    if (first > 0 && first + RS_UNROLL * RS_NT < min(v1, rv.nvec - 1)) {
      // every vector of the iteration exists and is neither the row's first nor its last one
#pragma unroll
      for (int q = 0; q < RS_UNROLL; q++) take(base + q * RS_NT, src[q * RS_NT], true);
    } else {
#pragma unroll
      for (int q = 0; q < RS_UNROLL; q++) {
        if (base + q * RS_NT < v1) take(base + q * RS_NT, src[q * RS_NT], false);
      }
    }
  }
  // every copy of this row has been waited for (the groups still pending are empty); this thread
  // has consumed its part of every stage, so the next row's first stages can start now
  if (nrv != nullptr) {
#pragma unroll
    for (int st = 0; st < RS_STAGES - 1; st++) issue(*nrv, nv0, nv1, st);
  }
  M = okey_to_float(static_cast<uint32_t>(bu::max_u64<RS_NW>(static_cast<unsigned long long>(okey(m)), sc, tid)));
  // s NaN: NaN * anything stays NaN; m = -Inf with s = 0: the thread adds nothing
  float sa, sb;
  rs_upk(s2, sa, sb);
  const float s = sa + sb;
  const double part = (m > -INFINITY || s != s) ? static_cast<double>(s) * static_cast<double>(expf(m - M)) : 0.0;
  S = bu::sum_d<RS_NW>(part, sc, tid);
}

// The N results of one input vector (elements i0 .. i0+N-1 of the row) into the output row:
// 16-byte streaming stores where the output is aligned like the input (vec_ok) and the vector
// lies inside the row, element by element otherwise.
template <typename TO, int N>
__device__ __forceinline__ void rs_store(TO* orow, bool vec_ok, int V, int i0, const float* y) {
  static_assert((sizeof(TO) == 4 && (N == 4 || N == 8)) || (sizeof(TO) == 2 && N == 8), "f32 out of f32/bf16 in, bf16 out of bf16 in");
  if (vec_ok && i0 >= 0 && i0 + N <= V) {
    if (sizeof(TO) == 4) {
#pragma unroll
      for (int h = 0; h < N / 4; h++) {
        uint4 o;
        o.x = __float_as_uint(y[4 * h]); o.y = __float_as_uint(y[4 * h + 1]);
        o.z = __float_as_uint(y[4 * h + 2]); o.w = __float_as_uint(y[4 * h + 3]);
        __stcs(reinterpret_cast<uint4*>(orow + i0) + h, o);
      }
    } else {
      uint4 o;
      o.x = bf16_bits_rne(y[0]) | (bf16_bits_rne(y[1]) << 16);
      o.y = bf16_bits_rne(y[2]) | (bf16_bits_rne(y[3]) << 16);
      o.z = bf16_bits_rne(y[N - 4]) | (bf16_bits_rne(y[N - 3]) << 16);
      o.w = bf16_bits_rne(y[N - 2]) | (bf16_bits_rne(y[N - 1]) << 16);
      __stcs(reinterpret_cast<uint4*>(orow + i0), o);
    }
  } else {
#pragma unroll
    for (int c = 0; c < N; c++) {
      const int i = i0 + c;
      if (i >= 0 && i < V) {
        if (sizeof(TO) == 4) reinterpret_cast<float*>(orow)[i] = y[c];
        else reinterpret_cast<uint16_t*>(orow)[i] = static_cast<uint16_t>(bf16_bits_rne(y[c]));
      }
    }
  }
}

// Pass 2: f(xa, xb, i, ya, yb) maps elements i and i+1 of the row; the results go to orow.
template <typename T, typename TO, typename F>
__device__ __forceinline__ void rs_map(const RowView<T>& rv, int v0, int v1, TO* orow, int tid, F&& f) {
  constexpr int VEC = Elem<T>::VEC;
  // orow + (v * VEC - shift) is 16-byte aligned for every v, or for none
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(orow) - static_cast<uintptr_t>(rv.shift) * sizeof(TO)) & 15u) == 0;
  auto put = [&](int v, const uint4& raw) {
    float x[VEC], y[VEC];
    Elem<T>::unpack(raw, x);
    const int i0 = v * VEC - rv.shift;
#pragma unroll
    for (int c = 0; c < VEC; c += 2) f(x[c], x[c + 1], i0 + c, y[c], y[c + 1]);
    rs_store<TO, VEC>(orow, vec_ok, rv.V, i0, y);
  };
  int v = v0 + tid;
  for (; v + (RS_UNROLL - 1) * RS_NT < v1; v += RS_UNROLL * RS_NT) {
    uint4 r[RS_UNROLL];
#pragma unroll
    for (int q = 0; q < RS_UNROLL; q++) r[q] = __ldg(rv.vbase + v + q * RS_NT);
#pragma unroll
    for (int q = 0; q < RS_UNROLL; q++) put(v + q * RS_NT, r[q]);
  }
  for (; v < v1; v += RS_NT) put(v, __ldg(rv.vbase + v));
}

// What one CTA of a pair tells the other about its half of a row.
struct RsHalf {
  float m;
  double s;
};

// Launched as clusters of C = 1 or 2 CTAs; cluster c takes rows c, c + #clusters, ... With two
// CTAs each handles half of the row's vectors and the two exchange (M, S) of their halves through
// distributed shared memory, one cluster barrier per row. Two CTAs per row halve the rows in
// flight (74 x 608 KB: what the second pass re-reads fits in the part of L2 an SM reads at full
// speed), halve a row's latency and even out the last round (512 rows: 6.9 per pair instead of
// 3.5 per SM).
template <typename T>
__global__ void __launch_bounds__(RS_NT, 1) row_softmax_kernel(const RowSoftmaxArgs A) {
  namespace cg = cooperative_groups;
  extern __shared__ __align__(16) unsigned char rs_dyn[];
  __shared__ bu::Scratch sc;
  __shared__ RsHalf xch[2];                                  // by row parity: one barrier per row is enough
  const uint4* ring = reinterpret_cast<const uint4*>(rs_dyn);
  const int tid = threadIdx.x;
  const T* x = static_cast<const T*>(A.x);
  cg::cluster_group cluster = cg::this_cluster();
  const int C = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  const int64_t ncl = gridDim.x / C;
  int k = 0;
  bool primed = false;
  // this CTA's vectors of a row: halves cut at a 128-byte line
  auto range = [&](const RowView<T>& r, int& a0, int& a1) {
    const int per = (C == 1) ? r.nvec : (((r.nvec + 1) / 2 + 7) & ~7);
    a0 = min(rank * per, r.nvec);
    a1 = min(a0 + per, r.nvec);
  };
  for (int64_t row = blockIdx.x / C; row < A.B; row += ncl, k++) {
    RowView<T> rv, nx;
    rv.init(x + row * A.row_stride, A.V);
    int v0, v1, nv0 = 0, nv1 = 0;
    range(rv, v0, v1);
    // only the one-pass op runs its copies on into the next row: behind a second pass the early
    // copies competed with that pass's L2 reads and stores and cost more than they saved (measured)
    const bool has_next = A.mode == RS_CE_FWD && row + ncl < A.B;
    if (has_next) {
      nx.init(x + (row + ncl) * A.row_stride, A.V);
      range(nx, nv0, nv1);
    }
    if (A.mode == RS_CE_BWD) {
      // loss.go:128-141: dx = exp(x - lse) * scale, minus scale at the target
      const float lse = A.row_lse[row], scale = A.scale;
      const int t = A.targets[row];
      rs_map<T, float>(rv, v0, v1, static_cast<float*>(A.out) + row * A.out_stride, tid,
                       [&](float xa, float xb, int i, float& ya, float& yb) {
        rs_upk(rs_mul2(rs_exp2(xa - lse, xb - lse), rs_pk(scale, scale)), ya, yb);
        if (i == t) ya -= scale;
        if (i + 1 == t) yb -= scale;
      });
      continue;
    }
    float M;
    double S;
    rs_max_sum<T>(rv, v0, v1, primed, has_next ? &nx : nullptr, nv0, nv1, ring, sc, tid, M, S);
    primed = has_next;
    if (C > 1) {
      if (tid == 0) { xch[k & 1].m = M; xch[k & 1].s = S; }
      cluster.sync();                                        // both halves published (release / acquire)
      const RsHalf* peer = cluster.map_shared_rank(&xch[k & 1], rank ^ 1);
      const float Mp = peer->m;
      const double Sp = peer->s;
      const float Mt = fmaxf(M, Mp);
      // the same expression on both CTAs, halves in rank order: both get the same bits
      const double own = (M > -INFINITY || S != S) ? S * static_cast<double>(expf(M - Mt)) : 0.0;
      const double oth = (Mp > -INFINITY || Sp != Sp) ? Sp * static_cast<double>(expf(Mp - Mt)) : 0.0;
      S = (rank == 0) ? own + oth : oth + own;
      M = Mt;
    }
    if (!(M > -INFINITY)) S = __longlong_as_double(0x7ff8000000000000ll);   // a row of -Inf only: upstream's -Inf - -Inf
    const float Sf = static_cast<float>(S);                  // the reference's f32 sum
    if (A.mode == RS_CE_FWD) {
      if (tid == 0 && rank == 0) {
        // loss.go:118-120: l = rowMax + f32(log(f64(sumExp))); loss = l - row[target]
        const float lse = M + static_cast<float>(log(static_cast<double>(Sf)));
        const int t = A.targets[row];
        float xt = __int_as_float(0x7fc00000);               // a target outside the row: upstream panics; NaN here
        if (t >= 0 && t < A.V) {
          if (sizeof(T) == 4) xt = reinterpret_cast<const float*>(x)[row * A.row_stride + t];
          else xt = __uint_as_float(static_cast<uint32_t>(reinterpret_cast<const uint16_t*>(x)[row * A.row_stride + t]) << 16);
        }
        A.row_lse[row] = lse;
        A.row_loss[row] = lse - xt;
      }
    } else if (A.mode == RS_SOFTMAX) {
      // ops.go:544-550: f32(exp(f64(x - max))) / sum; the quotient as a product with 1 / sum (within 1 ulp of it)
      const float inv = 1.0f / Sf;
      rs_map<T, T>(rv, v0, v1, static_cast<T*>(A.out) + row * A.out_stride, tid,
                   [&](float xa, float xb, int, float& ya, float& yb) {
        rs_upk(rs_mul2(rs_exp2(xa - M, xb - M), rs_pk(inv, inv)), ya, yb);
      });
    } else {
      // ops.go:589-592: x - max - f32(log(f64(sumExp)))
      const float logS = static_cast<float>(log(static_cast<double>(Sf)));
      rs_map<T, T>(rv, v0, v1, static_cast<T*>(A.out) + row * A.out_stride, tid,
                   [&](float xa, float xb, int, float& ya, float& yb) {
        ya = xa - M - logS;
        yb = xb - M - logS;
      });
    }
  }
  // the other CTA may still be reading this one's last (M, S): no CTA leaves before both are done
  if (C > 1 && A.mode != RS_CE_BWD) cluster.sync();
}

// Mean of the row losses in row order (loss.go:83: total / batch), one warp-sized CTA.
__global__ void __launch_bounds__(256) mean_loss_kernel(const float* row_loss, int64_t B, float* out) {
  __shared__ bu::Scratch sc;
  double acc = 0.0;
  for (int64_t i = threadIdx.x; i < B; i += 256) acc += static_cast<double>(row_loss[i]);
  acc = bu::sum_d<8>(acc, sc, threadIdx.x);
  if (threadIdx.x == 0) *out = static_cast<float>(acc / static_cast<double>(B));
}

}  // namespace gs
