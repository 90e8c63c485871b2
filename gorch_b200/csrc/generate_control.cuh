// generate_control_kernel: the bookkeeping of the reference's generate loops for a batch of
// sequences, on the device, so that a decode step needs no host round trip: after the sampling
// kernels have written one token id per row, this kernel applies the loop's rules to every row
// that is still live and leaves what the model's next forward needs in device memory.
//
// Rules (one iteration of the loops of model/generate.go:60-88 (uncached), :107-129 (cached) and
// model/qwen/generate.go:47-61), in the reference's order:
//   1. the iteration limit `i < MaxNewTokens` is tested before anything else;
//   2. a stop token ends the sequence and is NOT appended (generate.go:82-84; qwen isStop :54-56);
//   3. the token is appended to the result;
//   4. cached loops: if the cache already holds MaxSeq positions the sequence ends (the token
//      stays appended, no forward follows; generate.go:121-123, qwen :58-60); otherwise the token
//      is the next forward's input and the cache grows by one;
//      uncached loop: the next forward's input is the last MaxSeq tokens of the result
//      (generate.go:62-65): its start is written to window_start.
// A row that appends its MaxNewTokens-th token is marked finished at once (the reference runs one
// more forward whose logits it never reads).
//
// One CTA walks all rows (a few words of traffic per row), counts the live ones and writes the
// count for a host that wants to poll it now and then instead of every step.
#pragma once

#include <cstdint>

#include "block_util.cuh"

namespace gs {

constexpr int GC_NT = 256;
constexpr int GC_MAX_STOPS = 16;

// done[] codes
constexpr int GC_LIVE = 0;
constexpr int GC_STOP = 1;       // a stop token was sampled
constexpr int GC_MAX_NEW = 2;    // MaxNewTokens tokens appended
constexpr int GC_MAX_SEQ = 3;    // cached loops: the cache reached MaxSeq
constexpr int GC_ERROR = 4;      // the sampler reported an unusable id, or the token buffer is full

struct GenControlArgs {
  const int32_t* ids;        // [B] this step's sampled ids
  const uint32_t* flags;     // [B] the sampler's row flags, or null
  int32_t* tokens;           // [B, capacity] prompt + appended tokens
  long long capacity;
  int32_t* lengths;          // [B] tokens held per row
  int32_t* n_new;            // [B] tokens appended so far
  int32_t* cache_len;        // [B] positions in the KV cache (cached loops)
  int32_t* done;             // [B] GC_* code
  int32_t* next_input;       // [B] token of the next forward (cached), last token (uncached)
  int32_t* window_start;     // [B] uncached loop: start of the next input window; may be null
  int32_t* live_count;       // [1]
  int32_t stops[GC_MAX_STOPS];
  int n_stop;
  int max_new;
  int max_seq;
  int cached;
  uint32_t bad_flags;        // sampler flags that make an id unusable
  int B;
};

__global__ void __launch_bounds__(GC_NT) generate_control_kernel(const GenControlArgs A) {
  __shared__ bu::Scratch sc;
  const int tid = threadIdx.x;
  int live = 0;
  for (int b = tid; b < A.B; b += GC_NT) {
    if (A.done[b] != GC_LIVE) continue;
    int n = A.n_new[b];
    if (n >= A.max_new) { A.done[b] = GC_MAX_NEW; continue; }
    const int id = A.ids[b];
    if (id < 0 || (A.flags != nullptr && (A.flags[b] & A.bad_flags) != 0u)) { A.done[b] = GC_ERROR; continue; }
    bool stop = false;
    for (int s = 0; s < A.n_stop; s++) stop |= (id == A.stops[s]);
    if (stop) { A.done[b] = GC_STOP; continue; }
    const int len = A.lengths[b];
    if (len >= A.capacity) { A.done[b] = GC_ERROR; continue; }
    A.tokens[static_cast<long long>(b) * A.capacity + len] = id;
    A.lengths[b] = len + 1;
    A.n_new[b] = ++n;
    if (A.cached) {
      const int cl = A.cache_len[b];
      if (cl >= A.max_seq) { A.done[b] = GC_MAX_SEQ; continue; }
      A.cache_len[b] = cl + 1;
    } else if (A.window_start != nullptr) {
      A.window_start[b] = (len + 1 > A.max_seq) ? len + 1 - A.max_seq : 0;
    }
    A.next_input[b] = id;
    if (n >= A.max_new) { A.done[b] = GC_MAX_NEW; continue; }
    live++;
  }
  live = bu::sum_i<GC_NT / 32>(live, sc, tid);
  if (tid == 0) *A.live_count = live;
}

}  // namespace gs
