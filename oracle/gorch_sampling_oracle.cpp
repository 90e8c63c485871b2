// CPU oracle for gorch's decode-time token-sampling step.
//
// TEST INFRASTRUCTURE ONLY. This file is the checker for the CUDA path: it is
// used by the tests, by the smoke check and by the benchmark's CPU-baseline
// leg. The product (libgorchcuda.so and the gorch_b200 package) never links,
// imports or calls it.
//
// What it is: a loop-for-loop C++ restatement of the reference's pure-Go
// routines, so that results are comparable value for value:
//   argmax        model/generate.go:134-144   (qwen: model/qwen/generate.go:77-87)
//   sample        model/generate.go:147-240   (top-p "mode A", the 1.5*p tail trim)
//   sampleLogits  model/qwen/generate.go:92-164 (top-p "mode B", true nucleus)
//   kthLargest    model/generate.go:243-260   (qwen: model/qwen/generate.go:168-181)
//   bf16ToF32     tensor.go:96-99
//   TopK          index_ops.go:153-190
//   Multinomial   index_ops.go:203-227
//
// The reference is Go and darwin-only; no Go toolchain exists where this is
// built, so the reference itself cannot be run. Pinning: every known-answer
// vector the reference's own tests hold for this path (model/generate_test.go
// :11-38, index_ops_test.go:157-208) is checked against this file by
// tests/test_oracle_golden.py. The reference has NO test vector for top-p
// (either mode), for ties at the top-k threshold, or for the n-1 fallback:
// for those behaviours parity is pinned by the source text only ("parity
// unpinned" beyond the listed vectors).
//
// Two deliberate differences from the Go text, both outside what Go defines:
//   * the uniform is an argument (the reference draws it from math/rand,
//     generate.go:231 / qwen/generate.go:155);
//   * mode B orders equal probabilities by ascending index (Go's sort.Slice
//     is unstable, so the reference's order among equals is unspecified);
//     `cut_in_tie` reports when that choice matters.
//
// Build: see oracle/Makefile (-O2 -ffp-contract=off, no -ffast-math).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <thread>
#include <unordered_map>
#include <vector>

extern "C" {

// Per-row sampling configuration; the same 16-byte layout the CUDA ABI uses.
// Mirrors the sampling fields of GenerateConfig (model/generate.go:13-20).
struct OracleCfg {
  float temperature;  // 0 => greedy (generate.go:75)
  int32_t top_k;      // 0 => off
  float top_p;        // 0 => off; active only when 0 < p < 1 (generate.go:184)
  int32_t topp_mode;  // 0 = mode A (model/generate.go), 1 = mode B (model/qwen/generate.go)
};

// Extra facts about one sampled row, used by the parity tests.
struct OracleInfo {
  int64_t kept;        // tokens with non-zero final probability
  double sum_exp;      // softmax denominator (generate.go:173-178)
  double resum;        // top-p renormaliser (1.0 when top-p inactive)
  double edge_lo;      // cumulative before the chosen token
  double edge_hi;      // cumulative through the chosen token
  int32_t fallback;    // 1 when the walk fell through to n-1 (generate.go:239)
  int32_t cut_in_tie;  // mode B: the cut separates equal probabilities
  double cut_cum;      // mode A: remaining mass at stop; mode B: cumulative at cut
  float max_scaled;    // max of logits/T (generate.go:167-172)
  float threshold;     // top-k threshold (generate.go:158), NaN when inactive
};

}  // extern "C"

namespace {

inline float bf16_to_f32(uint16_t v) {  // tensor.go:96-99
  uint32_t bits = static_cast<uint32_t>(v) << 16;
  float f;
  std::memcpy(&f, &bits, sizeof f);
  return f;
}

// model/generate.go:134-144: strict '>' so the lowest index wins ties.
int64_t argmax_impl(const float* logits, int64_t n) {
  int64_t max_idx = 0;
  float max_val = logits[0];
  for (int64_t i = 1; i < n; i++) {
    if (logits[i] > max_val) {
      max_val = logits[i];
      max_idx = i;
    }
  }
  return max_idx;
}

// model/generate.go:243-260: k rounds of selection sort on a copy.
float kth_largest_impl(const float* data, int64_t n, int64_t k) {
  std::vector<float> sorted(data, data + n);
  for (int64_t i = 0; i < k; i++) {
    int64_t max_idx = i;
    for (int64_t j = i + 1; j < n; j++) {
      if (sorted[j] > sorted[max_idx]) max_idx = j;
    }
    std::swap(sorted[i], sorted[max_idx]);
  }
  return sorted[k - 1];
}

// Same value as kth_largest_impl for NaN-free input, in O(n): used only where
// a test needs the oracle at a size the O(k*n) loop cannot finish in time.
float kth_largest_fast(const float* data, int64_t n, int64_t k) {
  std::vector<float> tmp(data, data + n);
  std::nth_element(tmp.begin(), tmp.begin() + (k - 1), tmp.end(),
                   [](float a, float b) { return a > b; });
  return tmp[k - 1];
}

// sample (mode A, generate.go:147-240) and sampleLogits (mode B,
// qwen/generate.go:92-164). `probs_out` (n doubles) receives the final
// distribution when non-null. `fast_kth` swaps in kth_largest_fast.
int64_t sample_impl(const float* logits, int64_t n, float temperature,
                    int64_t top_k, float top_p, int mode, double r,
                    double* probs_out, OracleInfo* info, bool fast_kth) {
  OracleInfo local;
  OracleInfo& I = info ? *info : local;
  I = OracleInfo{};
  I.resum = 1.0;
  I.threshold = std::numeric_limits<float>::quiet_NaN();

  // generate.go:150-154
  std::vector<float> scaled(n);
  for (int64_t i = 0; i < n; i++) scaled[i] = logits[i] / temperature;

  // generate.go:157-164: everything >= the k-th largest survives (ties kept).
  if (top_k > 0 && top_k < n) {
    float threshold = fast_kth ? kth_largest_fast(scaled.data(), n, top_k)
                               : kth_largest_impl(scaled.data(), n, top_k);
    I.threshold = threshold;
    for (int64_t i = 0; i < n; i++) {
      if (scaled[i] < threshold) scaled[i] = -std::numeric_limits<float>::infinity();
    }
  }

  // generate.go:167-181: f32 max, f32 subtract, f64 exp, f64 sum in index order.
  float max_val = scaled[0];
  for (int64_t i = 1; i < n; i++) {
    if (scaled[i] > max_val) max_val = scaled[i];
  }
  I.max_scaled = max_val;
  double sum = 0.0;
  std::vector<double> probs(n);
  for (int64_t i = 0; i < n; i++) {
    float d = scaled[i] - max_val;
    probs[i] = std::exp(static_cast<double>(d));
    sum += probs[i];
  }
  I.sum_exp = sum;
  for (int64_t i = 0; i < n; i++) probs[i] /= sum;

  if (top_p > 0 && top_p < 1) {
    if (mode == 0) {
      // generate.go:184-228: zero the smallest positive prob until the
      // remaining mass is <= 1.5*p, then renormalise.
      for (;;) {
        double cum = 0.0;
        for (int64_t i = 0; i < n; i++) {
          if (probs[i] > 0) cum += probs[i];
        }
        I.cut_cum = cum;
        if (cum <= static_cast<double>(top_p) * 1.5) break;
        double min_p = std::numeric_limits<double>::max();
        int64_t min_i = -1;
        for (int64_t i = 0; i < n; i++) {
          if (probs[i] > 0 && probs[i] < min_p) {
            min_p = probs[i];
            min_i = i;
          }
        }
        if (min_i >= 0) {
          probs[min_i] = 0;
        } else {
          break;
        }
      }
      double resum = 0.0;
      for (int64_t i = 0; i < n; i++) resum += probs[i];
      I.resum = resum;
      for (int64_t i = 0; i < n; i++) probs[i] /= resum;
    } else {
      // qwen/generate.go:123-153: descending order, shortest prefix with
      // cumulative mass >= p, renormalise the prefix, zero the rest.
      std::vector<int64_t> idx(n);
      for (int64_t i = 0; i < n; i++) idx[i] = i;
      std::stable_sort(idx.begin(), idx.end(),
                       [&](int64_t a, int64_t b) { return probs[a] > probs[b]; });
      double cum = 0.0;
      int64_t cut = n;
      for (int64_t rnk = 0; rnk < n; rnk++) {
        cum += probs[idx[rnk]];
        if (cum >= static_cast<double>(top_p)) {
          cut = rnk + 1;
          break;
        }
      }
      I.cut_cum = cum;
      I.cut_in_tie = (cut < n && probs[idx[cut]] == probs[idx[cut - 1]]) ? 1 : 0;
      double resum = 0.0;
      std::unordered_map<int64_t, bool> kept;
      kept.reserve(static_cast<size_t>(cut));
      for (int64_t rnk = 0; rnk < cut; rnk++) {
        kept[idx[rnk]] = true;
        resum += probs[idx[rnk]];
      }
      I.resum = resum;
      for (int64_t i = 0; i < n; i++) {
        if (kept.find(i) == kept.end()) {
          probs[i] = 0;
        } else {
          probs[i] /= resum;
        }
      }
    }
  }

  int64_t kept_count = 0;
  for (int64_t i = 0; i < n; i++) kept_count += (probs[i] > 0) ? 1 : 0;
  I.kept = kept_count;
  if (probs_out) std::memcpy(probs_out, probs.data(), sizeof(double) * n);

  // generate.go:231-239
  double cumulative = 0.0;
  for (int64_t i = 0; i < n; i++) {
    double before = cumulative;
    cumulative += probs[i];
    if (r < cumulative) {
      I.edge_lo = before;
      I.edge_hi = cumulative;
      return i;
    }
  }
  I.fallback = 1;
  I.edge_lo = cumulative;
  I.edge_hi = cumulative;
  return n - 1;
}

// The branch at the call sites: generate.go:75-79, qwen/generate.go:49-53.
int64_t step_impl(const float* row, int64_t n, const OracleCfg& c, double u,
                  double* probs_out, OracleInfo* info, bool fast_kth) {
  if (c.temperature == 0) {
    if (info) *info = OracleInfo{};
    int64_t id = argmax_impl(row, n);
    if (probs_out) {
      for (int64_t i = 0; i < n; i++) probs_out[i] = 0.0;
      probs_out[id] = 1.0;
    }
    if (info) info->kept = 1;
    return id;
  }
  return sample_impl(row, n, c.temperature, c.top_k, c.top_p, c.topp_mode, u,
                     probs_out, info, fast_kth);
}

}  // namespace

extern "C" {

int64_t gorch_oracle_argmax_f32(const float* logits, int64_t n) {
  return argmax_impl(logits, n);
}

float gorch_oracle_kth_largest_f32(const float* data, int64_t n, int64_t k) {
  return kth_largest_impl(data, n, k);
}

// One row, f32 logits. flags bit0: use the O(n) k-th-largest.
int64_t gorch_oracle_sample_f32(const float* logits, int64_t n, float temperature,
                                int64_t top_k, float top_p, int32_t mode, double u,
                                double* probs_out, OracleInfo* info, int32_t flags) {
  return sample_impl(logits, n, temperature, top_k, top_p, mode, u, probs_out, info,
                     (flags & 1) != 0);
}

// A [B,V] batch with per-row configs and uniforms; dtype 0 = f32, 1 = bf16
// (upcast per tensor.go:96-99, then the f32 routine). Rows are spread over
// `threads` host threads (<=1: the reference's single-goroutine model).
// probs_out: null or B*V doubles. infos: null or B records.
void gorch_oracle_sample_batch(const void* logits, int32_t dtype, int64_t B, int64_t V,
                               int64_t row_stride, const OracleCfg* cfgs,
                               const double* uniforms, int64_t* out_ids,
                               double* probs_out, OracleInfo* infos, int32_t flags,
                               int32_t threads) {
  auto work = [&](int64_t b0, int64_t b1) {
    std::vector<float> up;
    for (int64_t b = b0; b < b1; b++) {
      const float* row;
      if (dtype == 1) {
        const uint16_t* src = static_cast<const uint16_t*>(logits) + b * row_stride;
        up.resize(V);
        for (int64_t i = 0; i < V; i++) up[i] = bf16_to_f32(src[i]);
        row = up.data();
      } else {
        row = static_cast<const float*>(logits) + b * row_stride;
      }
      out_ids[b] = step_impl(row, V, cfgs[b], uniforms[b],
                             probs_out ? probs_out + b * V : nullptr,
                             infos ? infos + b : nullptr, (flags & 1) != 0);
    }
  };
  if (threads <= 1 || B <= 1) {
    work(0, B);
    return;
  }
  int64_t nt = std::min<int64_t>(threads, B);
  std::vector<std::thread> pool;
  for (int64_t t = 0; t < nt; t++) {
    // interleaved blocks keep mixed-cost rows balanced
    pool.emplace_back([&, t]() {
      for (int64_t b = t; b < B; b += nt) work(b, b + 1);
    });
  }
  for (auto& th : pool) th.join();
}

// index_ops.go:153-190. Returns 0, or 1 when k is out of [1,V] (the reference
// panics there). Order among equal values is unspecified in the reference
// (unstable sort); here ascending index.
int32_t gorch_oracle_topk_f32(const float* x, int64_t B, int64_t V, int64_t k,
                              float* values, int64_t* indices) {
  if (k <= 0 || k > V) return 1;
  std::vector<std::pair<float, int64_t>> pairs(V);
  for (int64_t b = 0; b < B; b++) {
    const float* row = x + b * V;
    for (int64_t i = 0; i < V; i++) pairs[i] = {row[i], i};
    std::stable_sort(pairs.begin(), pairs.end(),
                     [](const std::pair<float, int64_t>& a,
                        const std::pair<float, int64_t>& c) { return a.first > c.first; });
    for (int64_t i = 0; i < k; i++) {
      values[b * k + i] = pairs[i].first;
      indices[b * k + i] = pairs[i].second;
    }
  }
  return 0;
}

// index_ops.go:203-227: inverse-CDF walk over f32 probs with an f64 running sum.
void gorch_oracle_multinomial_f32(const float* probs, int64_t B, int64_t V,
                                  const double* uniforms, int64_t* out) {
  for (int64_t b = 0; b < B; b++) {
    double r = uniforms[b];
    double cum = 0.0;
    const float* row = probs + b * V;
    int64_t picked = V - 1;
    for (int64_t j = 0; j < V; j++) {
      cum += static_cast<double>(row[j]);
      if (r < cum) {
        picked = j;
        break;
      }
    }
    out[b] = picked;
  }
}

// The control flow of the reference's three generate loops, with the sampler's answers scripted:
// script[i] is what argmax / sample returns in iteration i, so the loop's own rules (prompt
// truncation, the stop test before the append, the MaxSeq test after it, the iteration limit)
// are all that is exercised.
//   loop 0: GenerateWithConfig, uncached (model/generate.go:57-88); one stop token, off when < 0
//   loop 1: generateCached (model/generate.go:93-131)
//   loop 2: qwen.Generate (model/qwen/generate.go:35-62); a list of stop tokens (isStop, :64-71)
// out_tokens holds n_prompt + max_new entries; returns the result's length. reason: 1 the stop
// token came, 2 the iteration limit, 3 the cache reached MaxSeq. sampler_calls: iterations that
// asked the sampler (= uniforms drawn when temperature != 0). fed: for loops 1 and 2 the tokens
// given to the incremental forward, in order (up to max_new entries); n_fed their count. For
// loop 0, fed[i] is the start of the input window of iteration i (len(result) - MaxSeq, or 0).
int64_t gorch_oracle_generate_scripted(int32_t loop, const int64_t* prompt, int64_t n_prompt,
                                       const int64_t* script, int64_t max_new, int64_t max_seq,
                                       const int64_t* stops, int64_t n_stops,
                                       int64_t* out_tokens, int32_t* reason,
                                       int64_t* sampler_calls, int64_t* fed, int64_t* n_fed) {
  std::vector<int64_t> result(prompt, prompt + n_prompt);
  int64_t calls = 0, nf = 0;
  int32_t why = 2;
  auto is_stop = [&](int64_t tok) {
    if (loop == 2) {
      for (int64_t i = 0; i < n_stops; i++) if (tok == stops[i]) return true;
      return false;
    }
    return n_stops > 0 && stops[0] >= 0 && tok == stops[0];
  };
  if (loop == 0) {
    for (int64_t i = 0; i < max_new; i++) {
      int64_t start = 0;
      if (static_cast<int64_t>(result.size()) > max_seq) start = static_cast<int64_t>(result.size()) - max_seq;
      fed[nf++] = start;
      const int64_t next = script[calls++];
      if (is_stop(next)) { why = 1; break; }
      result.push_back(next);
    }
  } else {
    if (loop == 1 && static_cast<int64_t>(result.size()) > max_seq) {
      result.erase(result.begin(), result.end() - max_seq);     // generate.go:101-103
    }
    int64_t cache_len = static_cast<int64_t>(result.size());    // prefill of the whole prompt
    for (int64_t i = 0; i < max_new; i++) {
      const int64_t next = script[calls++];
      if (is_stop(next)) { why = 1; break; }
      result.push_back(next);
      if (cache_len >= max_seq) { why = 3; break; }
      fed[nf++] = next;
      cache_len++;
    }
  }
  for (size_t i = 0; i < result.size(); i++) out_tokens[i] = result[i];
  *reason = why;
  *sampler_calls = calls;
  *n_fed = nf;
  return static_cast<int64_t>(result.size());
}

// ops.go:527-551: Softmax forward over a (batch, classes) f32 tensor, loop for loop: the row
// maximum by strict `>` from element 0, f32(exp(f64(x - max))) summed sequentially in f32, then
// an f32 division.
void gorch_oracle_softmax_f32(const float* x, int64_t B, int64_t V, float* out) {
  for (int64_t i = 0; i < B; i++) {
    const float* row = x + i * V;
    float* o = out + i * V;
    float row_max = row[0];
    for (int64_t j = 1; j < V; j++) if (row[j] > row_max) row_max = row[j];
    float sum = 0.0f;
    for (int64_t j = 0; j < V; j++) {
      o[j] = static_cast<float>(std::exp(static_cast<double>(row[j] - row_max)));
      sum += o[j];
    }
    for (int64_t j = 0; j < V; j++) o[j] /= sum;
  }
}

// ops.go:566-593: LogSoftmax forward: x - max - f32(log(f64(sumExp))), two f32 subtractions.
void gorch_oracle_log_softmax_f32(const float* x, int64_t B, int64_t V, float* out) {
  for (int64_t i = 0; i < B; i++) {
    const float* row = x + i * V;
    float* o = out + i * V;
    float row_max = row[0];
    for (int64_t j = 1; j < V; j++) if (row[j] > row_max) row_max = row[j];
    float sum_exp = 0.0f;
    for (int64_t j = 0; j < V; j++) sum_exp += static_cast<float>(std::exp(static_cast<double>(row[j] - row_max)));
    const float log_sum_exp = static_cast<float>(std::log(static_cast<double>(sum_exp)));
    for (int64_t j = 0; j < V; j++) o[j] = row[j] - row_max - log_sum_exp;
  }
}

// loss.go:108-124 (ceForwardCPU) and :83: per-row logsumexp and the mean loss. Upstream's row
// passes go through Accelerate (vDSP/vForce, not part of the reference's tree): maximum, x - max,
// elementwise f32 exp, f32 sum; they are restated here as scalar f32 loops.
float gorch_oracle_cross_entropy_fwd_f32(const float* x, const int32_t* targets, int64_t B, int64_t V,
                                         float* row_loss, float* row_lse) {
  float total = 0.0f;
  for (int64_t i = 0; i < B; i++) {
    const float* row = x + i * V;
    float row_max = row[0];
    for (int64_t j = 1; j < V; j++) if (row[j] > row_max) row_max = row[j];
    float sum_exp = 0.0f;
    for (int64_t j = 0; j < V; j++) sum_exp += static_cast<float>(std::exp(static_cast<double>(row[j] - row_max)));
    const float l = row_max + static_cast<float>(std::log(static_cast<double>(sum_exp)));
    row_lse[i] = l;
    row_loss[i] = l - row[targets[i]];
    total += row_loss[i];
  }
  return total / static_cast<float>(B);
}

// loss.go:128-141 (ceBackwardCPU): dx = exp(x - lse) * scale, then dx[target] -= scale.
void gorch_oracle_cross_entropy_bwd_f32(const float* x, const int32_t* targets, const float* row_lse,
                                        int64_t B, int64_t V, float scale, float* dx) {
  for (int64_t i = 0; i < B; i++) {
    const float* row = x + i * V;
    float* d = dx + i * V;
    for (int64_t j = 0; j < V; j++) d[j] = static_cast<float>(std::exp(static_cast<double>(row[j] - row_lse[i]))) * scale;
    d[targets[i]] -= scale;
  }
}

float gorch_oracle_bf16_to_f32(uint16_t v) { return bf16_to_f32(v); }

// tensor.go:85-94: round-to-nearest-even, quiet NaN preserved.
uint16_t gorch_oracle_f32_to_bf16(float v) {
  uint32_t bits;
  std::memcpy(&bits, &v, sizeof bits);
  if (((bits >> 23) & 0xff) == 0xff && (bits & 0x7fffff) != 0) {
    return static_cast<uint16_t>((bits >> 16) | 0x40);
  }
  uint32_t rounding = 0x7fffu + ((bits >> 16) & 1u);
  return static_cast<uint16_t>((bits + rounding) >> 16);
}

int32_t gorch_oracle_hw_threads(void) {
  unsigned n = std::thread::hardware_concurrency();
  return n ? static_cast<int32_t>(n) : 1;
}

}  // extern "C"
