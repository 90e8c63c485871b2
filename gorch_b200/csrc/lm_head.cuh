// LM-head projection with the sampling step's first pass in its epilogue.
//
// logits[b, v] = sum_k x[b, k] * w[v, k]: the last matmul of a decode step, MatMulTransB(last, Embed.Weight)
// in model/qwen/qwen.go:80-85 (nn/gpt.go:119-120 for GPT-2; nn/extembed.go:152-195 is its CPU loop), with
// x [B, K] and w [V, K] in bf16 and f32 accumulation. It is the one dense contraction next to the
// sampling path, and it produces the [B, V] logits that the sampling kernels otherwise read back from
// HBM: here the rows of a batch tile stay in tensor memory until the epilogue has taken what sampling
// needs from them.
//
// One CTA per SM, persistent over vocabulary tiles of 128 columns; a batch tile is 128 rows (rows
// beyond B are zero-filled by TMA and ignored). Per tile, K is walked in chunks of 64:
//   warp 0      producer: two TMA loads per chunk (x tile and w tile, 128 x 64 bf16 each, 128-byte
//               swizzle) into a ring of shared-memory stages, completion on the stage's mbarrier
//   warp 1      issuer: one elected thread issues tcgen05.mma (M = 128 batch rows, N = 128 vocabulary
//               columns, K = 16; both operands K-major from shared memory) into one of two accumulator
//               buffers in tensor memory; tcgen05.commit frees the stage / publishes the accumulator
//   warps 2-5   epilogue: thread = batch row (a TMEM lane), its 128 logits of the tile by tcgen05.ld;
//               optional store of the logits, row maximum and NaN flag, and (fused sampling) the logits
//               at or above the row's threshold appended to the row's candidate list
// Every CTA fetches its own tiles (plain TMA loads), and every tensor map covers this GPU's own memory.
//
// Every wait on an mbarrier is bounded: a wait that runs out sets an abort flag that the other roles
// see in their own waits, the kernel reports LMH_ERR_TIMEOUT in its status word, frees its tensor
// memory and returns.
#pragma once

#include <cuda.h>

#include "sample_batch.cuh"

namespace gs {

constexpr int LMH_BM = 128;              // batch rows per tile (UMMA M)
constexpr int LMH_BN = 128;              // vocabulary columns per tile (UMMA N)
constexpr int LMH_BK = 64;               // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int LMH_STAGES = 5;
constexpr int LMH_NT = 192;              // warp 0 producer, warp 1 issuer, warps 2-5 epilogue
constexpr int LMH_STAGE_BYTES = (LMH_BM + LMH_BN) * LMH_BK * 2;     // 32 KB
constexpr int LMH_ROWS_S = 4096;         // rows whose running maximum, NaN bits and candidate count a CTA keeps in shared memory
constexpr int LMH_DYN_BYTES = LMH_STAGES * LMH_STAGE_BYTES + 1024 + LMH_ROWS_S * 12;  // ring (+ room to align it to 1024 bytes) + the per-row words
constexpr int LMH_TMEM_COLS = 256;       // two accumulators of 128 f32 columns
constexpr uint32_t LMH_WAIT_LIMIT = 4000000u;
constexpr int LMH_CAND_CAP = 2048;       // candidates per row that the finish kernel takes (entries of 8 bytes)
constexpr int LMH_SEG = 32;              // candidates per row and CTA: every CTA of the projection has its own segment of a row's list

constexpr uint32_t LMH_ERR_TIMEOUT = 1u;

// tcgen05 instruction descriptor (kind::f16): D = F32 (bits 4-5 = 1), A = B = BF16 (bits 7-9, 10-12 = 1),
// both K-major (bits 15, 16 = 0), N / 8 at bits 17-22, M / 16 at bits 24-28.
constexpr uint32_t LMH_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(LMH_BN >> 3) << 17) |
                               (static_cast<uint32_t>(LMH_BM >> 4) << 24);

struct LmHeadArgs {
  CUtensorMap map_x;       // x [B, K] bf16, box 64 x 128, 128-byte swizzle
  CUtensorMap map_w;       // w [V, K] bf16, box 64 x 128, 128-byte swizzle
  int32_t B, V, K;
  int32_t tile0, tile_step, ntile;   // vocabulary tiles tile0 + i * tile_step, i < ntile
  float* out_logits;       // [B, ld_out] f32, or null
  int64_t ld_out;
  int32_t out_col0;        // column of out_logits that vocabulary tile i starts at: i * LMH_BN when compact, else its own
  int32_t compact;         // 1: tile i goes to columns [i * 128, ...) of out_logits (the sample of tiles)
  // fused sampling (all null when unused)
  const float* thr;        // [B] candidate threshold per row (raw logit units)
  uint2* cand;             // [B, gridDim.x, LMH_SEG] (logit bits, index); needs B <= LMH_ROWS_S
  int32_t* cand_cnt;       // [B, gridDim.x], written by every CTA for every row
  uint32_t* rowmax_key;    // [B] order key of the row maximum (atomicMax)
  int32_t* row_nan;        // [B] a NaN was seen
  uint32_t* status;        // [1] LMH_ERR_* bits
};

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
// Bounded wait for the phase with parity `parity` to complete; false when it ran out or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t it = 0; it < LMH_WAIT_LIMIT; it++) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((it & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               :: "r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// Shared-memory matrix descriptor of a K-major tile of 128-byte rows with the 128-byte swizzle: start
// address / 16, leading byte offset 1 (unused for swizzled K-major), stride byte offset 1024 / 16 (eight
// rows), descriptor version 1 at bit 46, layout type 2 (128-byte swizzle) at bits 61-63.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr_bytes) {
  return static_cast<uint64_t>((smem_addr_bytes & 0x3ffffu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}

__global__ void __launch_bounds__(LMH_NT, 1) lm_head_kernel(const __grid_constant__ LmHeadArgs A) {
  extern __shared__ __align__(16) unsigned char lmh_dyn[];
  __shared__ __align__(8) unsigned long long full_bar[LMH_STAGES], empty_bar[LMH_STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t ring = (smem_addr(lmh_dyn) + 1023u) & ~1023u;          // the swizzled tiles need 1024-byte alignment
  // per-row running maximum and NaN bits of this CTA's tiles (a row always belongs to the same epilogue
  // thread, so no atomics here); flushed to global memory once at the end
  float* rowmax_s = reinterpret_cast<float*>(lmh_dyn + LMH_STAGES * LMH_STAGE_BYTES + 1024);
  int* rownan_s = reinterpret_cast<int*>(rowmax_s + LMH_ROWS_S);
  int* rowcnt_s = rownan_s + LMH_ROWS_S;
  const bool rows_in_smem = A.rowmax_key != nullptr && A.B <= LMH_ROWS_S;
  if (rows_in_smem) for (int r = tid; r < A.B; r += LMH_NT) { rowmax_s[r] = -INFINITY; rownan_s[r] = 0; rowcnt_s[r] = 0; }
  volatile int* abort_flag = &abort_s;
  const int nkc = A.K / LMH_BK;                                        // K chunks per tile
  const int nbt = (A.B + LMH_BM - 1) / LMH_BM;                         // batch tiles
  // this CTA's work items: (vocabulary tile, batch tile) pairs, vocabulary-major
  const int my_first = blockIdx.x, my_step = gridDim.x;

  if (tid == 0) {
    for (int s = 0; s < LMH_STAGES; s++) { mbar_init(smem_addr(&full_bar[s]), 1); mbar_init(smem_addr(&empty_bar[s]), 1); }
    for (int b = 0; b < 2; b++) { mbar_init(smem_addr(&acc_full[b]), 1); mbar_init(smem_addr(&acc_empty[b]), 4); }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {                                                      // the issuer's warp owns the tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_addr(&tmem_base_s)), "r"(LMH_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // ---- producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int t = my_first; t < A.ntile && ok; t += my_step) {
        const int vt = A.tile0 + t * A.tile_step;
        for (int bt = 0; bt < nbt && ok; bt++) {
          for (int kc = 0; kc < nkc; kc++) {
            if (!mbar_wait(smem_addr(&empty_bar[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
            const uint32_t bar = smem_addr(&full_bar[stage]);
            const uint32_t sa = ring + stage * LMH_STAGE_BYTES, sb = sa + LMH_BM * LMH_BK * 2;
            mbar_expect_tx(bar, LMH_STAGE_BYTES);
            tma_load_2d(sa, &A.map_x, bar, kc * LMH_BK, bt * LMH_BM);
            tma_load_2d(sb, &A.map_w, bar, kc * LMH_BK, vt * LMH_BN);
            if (++stage == LMH_STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- issuer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int t = my_first; t < A.ntile && ok; t += my_step) {
        for (int bt = 0; bt < nbt && ok; bt++) {
          if (!mbar_wait(smem_addr(&acc_empty[acc]), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t d_tmem = tmem_base + acc * LMH_BN;
          for (int kc = 0; kc < nkc; kc++) {
            if (!mbar_wait(smem_addr(&full_bar[stage]), phase, abort_flag)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t sa = ring + stage * LMH_STAGE_BYTES, sb = sa + LMH_BM * LMH_BK * 2;
#pragma unroll
            for (int k = 0; k < LMH_BK / 16; k++) {
              umma_f16(d_tmem, umma_desc(sa + k * 32), umma_desc(sb + k * 32), LMH_IDESC, (kc > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(smem_addr(&empty_bar[stage]));                  // the stage is free once these MMAs have read it
            if (++stage == LMH_STAGES) { stage = 0; phase ^= 1u; }
          }
          if (ok) umma_commit(smem_addr(&acc_full[acc]));               // the accumulator is complete
          if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
      }
    }
  } else {
    // ---- epilogue: warp w reads TMEM lanes 32 * (w % 4) .. + 31; thread = batch row
    const int q = warp & 3;
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (int t = my_first; t < A.ntile && ok; t += my_step) {
      const int vt = A.tile0 + t * A.tile_step;
      const int v0 = vt * LMH_BN;
      const int oc0 = A.compact ? t * LMH_BN : v0;
      for (int bt = 0; bt < nbt && ok; bt++) {
        if (!mbar_wait(smem_addr(&acc_full[acc]), acc_phase, abort_flag)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int row = bt * LMH_BM + q * 32 + lane;
        const bool live = row < A.B;
        const float thr = (A.thr && live) ? A.thr[row] : INFINITY;
        float vmax = -INFINITY;
        int nan_bits = 0;                                             // 1: a NaN in the row; 2: at index 0
#pragma unroll 1
        for (int c = 0; c < LMH_BN; c += 32) {
          uint32_t r[32];
          tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * LMH_BN + c, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (live) {
            const int nvalid = min(32, A.V - (v0 + c));                 // columns past the vocabulary hold zeros
            if (A.out_logits) {
              float* dst = A.out_logits + static_cast<int64_t>(row) * A.ld_out + oc0 + c;
              if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) *reinterpret_cast<uint4*>(dst + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; j++) if (j < nvalid) dst[j] = __uint_as_float(r[j]);
              }
            }
            if (A.rowmax_key) {
              // the chunk's maximum first (NaN-propagating): only a chunk that holds a candidate, a NaN
              // or columns past the vocabulary is looked at logit by logit
              float cm = max3nan(__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]));
#pragma unroll
              for (int j = 3; j + 1 < 32; j += 2) cm = max3nan(cm, __uint_as_float(r[j]), __uint_as_float(r[j + 1]));
              cm = maxnan(cm, __uint_as_float(r[31]));
              if (nvalid == 32 && cm < thr) {                          // (false for a NaN maximum)
                vmax = fmaxf(vmax, cm);
              } else {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                  const float x = __uint_as_float(r[j]);
                  if (j >= nvalid) continue;
                  if (x != x) nan_bits |= (v0 + c + j == 0) ? 3 : 1;
                  vmax = fmaxf(vmax, x);
                  if (x >= thr && rows_in_smem) {
                    // this CTA's own segment of the row's list, and a count that only this thread
                    // touches: nothing to wait for (an atomic on a count shared by all CTAs made
                    // every warp wait in nearly every chunk, a quarter more time for the kernel)
                    const int slot = rowcnt_s[row]++;
                    if (slot < LMH_SEG) A.cand[(static_cast<int64_t>(row) * gridDim.x + blockIdx.x) * LMH_SEG + slot] = make_uint2(r[j], static_cast<uint32_t>(v0 + c + j));
                  }
                }
              }
            }
          }
        }
        // the accumulator is free again: one arrival per epilogue warp
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_addr(&acc_empty[acc]));
        if (A.rowmax_key && live) {
          if (rows_in_smem) {
            rowmax_s[row] = fmaxf(rowmax_s[row], vmax);
            rownan_s[row] |= nan_bits;
          } else {
            atomicMax(&A.rowmax_key[row], okey(vmax));
            if (nan_bits) atomicOr(&A.row_nan[row], nan_bits);
          }
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  }
  // ---- teardown
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (rows_in_smem) {
    for (int r = tid; r < A.B; r += LMH_NT) {
      const float v = rowmax_s[r];
      if (v > -INFINITY) atomicMax(&A.rowmax_key[r], okey(v));
      if (rownan_s[r]) atomicOr(&A.row_nan[r], rownan_s[r]);
      if (A.cand_cnt) A.cand_cnt[static_cast<int64_t>(r) * gridDim.x + blockIdx.x] = rowcnt_s[r];
    }
  }
  if (abort_s) {
    // a wait ran out: give the copies and MMAs still in flight time to land before the shared and
    // tensor memory they target is given back (bounded: about a millisecond)
    for (int it = 0; it < 1000; it++) __nanosleep(1000);
    if (tid == 0 && A.status) atomicOr(A.status, LMH_ERR_TIMEOUT);
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(LMH_TMEM_COLS) : "memory");
  }
}


// ---- fused sampling on top of the projection (greedy and top-k rows) --------------------------------
//
//   1. the projection over a sample of vocabulary tiles (1/32 of them, 8 to 32 tiles spread over the
//      vocabulary) gives each row 1024 to 4096 of its logits;
//   2. lmh_threshold_kernel: the r-th largest of that sample, r chosen so that eight times top_k
//      logits of the whole row (at least 256, at most a third of the list) are expected above it: an
//      estimate, not a bound;
//   3. the projection over all tiles: the epilogue appends every logit at or above the row's
//      threshold to this CTA's segment of the row's candidate list (no [B, V] logits are written);
//   4. lmh_finish_kernel: the exact top_k-th largest of the candidates with ties kept
//      (model/generate.go:157-164), then softmax / top-p / draw on the kept set exactly as the
//      one-GPU narrow kernel does. A row whose estimate failed (fewer than top_k candidates, or more
//      than a segment or the list holds) or whose config the fused path does not serve is counted in nfail; the
//      host then recomputes the batch through the unfused path.
constexpr int LMH_SAMPLE_TILES_MIN = 8, LMH_SAMPLE_TILES_MAX = 32;   // the sample: 1/32 of the tiles, within these bounds
constexpr int LMH_F_NT = 256;
constexpr int LMH_F_DYN_BYTES = LMH_CAND_CAP * 8 + 16384 + KEEP_MAX * 8;

struct LmhSampleArgs {
  KernelArgs k;             // V, cfgs, uniforms, out_ids, out_flags, exp_table (logits unused)
  const float* sample;      // [B, nsample] logits of the sampled tiles
  int32_t nsample;
  int32_t fuse_top_k;       // rows with 0 < top_k <= fuse_top_k (or temperature 0) are served
  float* thr;               // [B]
  const uint2* cand;        // [B, nseg, LMH_SEG]
  const int32_t* cand_cnt;  // [B, nseg]
  int32_t nseg;             // CTAs of the projection that filled the lists
  const uint32_t* rowmax_key;
  const int32_t* row_nan;
  int32_t* nfail;           // [1]
  int64_t B;
};

__device__ __forceinline__ bool lmh_row_served(const RowCfg& c, int V, int fuse_top_k) {
  const float T = c.temperature;
  if (T == 0.0f) return true;
  if (!(T > 0.0f) || !(T < INFINITY)) return true;            // reported as a bad config by the finish kernel
  const int topk = (c.top_k > 0 && c.top_k < V) ? c.top_k : 0;
  return topk > 0 && topk <= fuse_top_k;
}

__global__ void __launch_bounds__(LMH_F_NT) lmh_threshold_kernel(LmhSampleArgs M) {
  __shared__ uint2 list[LMH_SAMPLE_TILES_MAX * LMH_BN];
  __shared__ uint32_t s_sel[256];
  __shared__ int s_bc[4];
  const int tid = threadIdx.x;
  for (int64_t row = blockIdx.x; row < M.B; row += gridDim.x) {
    __syncthreads();
    const RowCfg cfg = M.k.cfgs[row];
    if (!lmh_row_served(cfg, M.k.V, M.fuse_top_k)) { if (tid == 0) M.thr[row] = INFINITY; continue; }
    const int keff = (cfg.temperature == 0.0f || !(cfg.temperature > 0.0f) || !(cfg.temperature < INFINITY)) ? 1 : cfg.top_k;
    const int n = M.nsample;
    for (int j = tid; j < n; j += LMH_F_NT) list[j] = make_uint2(__float_as_uint(M.sample[row * n + j]), static_cast<uint32_t>(j));
    // expected logits of the whole row above the threshold: eight times top_k, at least 256, at most a
    // third of the list; the r-th largest of the sample stands for the (r V / n)-th largest of the row
    const long long want = min(max(8ll * keff, 256ll), static_cast<long long>(LMH_CAND_CAP / 3));
    const int r = max(2, static_cast<int>((want * n + M.k.V / 2) / M.k.V));
    float thr = -INFINITY;                                    // a sample too small to say: everything is a candidate
    if (r < n) {
      const uint32_t key = bu::select_kth<LMH_F_NT>(list, n, r, s_sel, s_bc, tid);
      thr = okey_to_float(key);
      if (!(thr == thr)) thr = -INFINITY;                     // NaNs order lowest: a NaN threshold would collect nothing
    }
    if (tid == 0) M.thr[row] = thr;
  }
}

__global__ void __launch_bounds__(LMH_F_NT, 4) lmh_finish_kernel(LmhSampleArgs M) {
  extern __shared__ __align__(16) unsigned char dyn[];
  __shared__ bu::Scratch sc;
  __shared__ uint32_t s_sel[256];
  __shared__ int s_bc[4];
  __shared__ double s_bcd[4];
  __shared__ int s_cnt;
  uint2* list = reinterpret_cast<uint2*>(dyn);                                       // the row's candidates
  unsigned char* work = dyn + LMH_CAND_CAP * 8;                                       // 16 KB for finish_small_set
  uint2* kept = reinterpret_cast<uint2*>(dyn + LMH_CAND_CAP * 8 + 16384);            // KEEP_MAX entries
  const KernelArgs& A = M.k;
  const int tid = threadIdx.x;
  constexpr int NW = LMH_F_NT / 32;
  for (int64_t row = blockIdx.x; row < M.B; row += gridDim.x) {
    __syncthreads();
    const RowCfg cfg = A.cfgs[row];
    const float Tm = cfg.temperature;
    RowDebug dbg;
    dbg.sum_exp = 0; dbg.resum = 1.0; dbg.edge_lo = 0; dbg.edge_hi = 0; dbg.kept = 0;
    dbg.max_scaled = 0; dbg.threshold = __int_as_float(0x7fc00000); dbg.path = 4;
    for (int q = 0; q < 8; q++) dbg.reserved[q] = 0;
    auto write_row = [&](int id, uint32_t fl) {
      if (tid == 0) {
        A.out_ids[row] = id;
        if (A.out_flags) A.out_flags[row] = fl;
      }
    };
    auto give_up = [&]() { if (tid == 0) atomicAdd(M.nfail, 1); write_row(-1, FLAG_INTERNAL); };
    if (!lmh_row_served(cfg, A.V, M.fuse_top_k)) { give_up(); continue; }
    if (Tm != 0.0f && (!(Tm > 0.0f) || !(Tm < INFINITY))) { write_row(-1, FLAG_BAD_CFG); continue; }
    // the row's candidates: one segment per CTA of the projection
    if (tid == 0) s_cnt = 0;
    __syncthreads();
    int over = 0;
    for (int c = tid; c < M.nseg; c += LMH_F_NT) {
      const int n = M.cand_cnt[row * M.nseg + c];
      if (n > LMH_SEG) over = 1;
      const int take = min(n, LMH_SEG);
      const int base = atomicAdd(&s_cnt, take);
      if (base + take <= LMH_CAND_CAP) {
        const uint2* seg = M.cand + (row * M.nseg + c) * LMH_SEG;
        for (int j = 0; j < take; j++) list[base + j] = seg[j];
      }
    }
    over = __syncthreads_or(over);
    const int cnt = s_cnt;
    const int nanb = M.row_nan[row];
    const int keff = (Tm == 0.0f) ? 1 : cfg.top_k;
    if (over || cnt > LMH_CAND_CAP || (cnt < keff && !(nanb & 1))) { give_up(); continue; }   // the estimate failed for this row
    // ---- greedy (generate.go:134-144): largest logit, lowest index; a NaN at index 0 is never beaten
    if (Tm == 0.0f) {
      unsigned long long best = 0ull;
      for (int j = tid; j < cnt; j += LMH_F_NT) {
        const unsigned long long p = (static_cast<unsigned long long>(okey(__uint_as_float(list[j].x))) << 32) |
                                     static_cast<uint32_t>(~list[j].y);
        best = p > best ? p : best;
      }
      best = bu::max_u64<NW>(best, sc, tid);
      int id = static_cast<int>(~static_cast<uint32_t>(best & 0xffffffffull));
      if ((nanb & 2) || cnt == 0) id = 0;
      write_row(id, 0u);
      continue;
    }
    const float xmax = okey_to_float(M.rowmax_key[row]);
    const float m = scale_t(xmax, Tm);
    // A NaN anywhere, or an infinite maximum: the walk of generate.go:231-239 falls through
    if ((nanb & 1) || !(fabsf(m) < INFINITY)) { write_row(A.V - 1, FLAG_NONFINITE | FLAG_FALLBACK); continue; }
    // ---- top_k-th largest with ties (generate.go:157-164), then the kept set
    const int topk = cfg.top_k;
    float thr = -INFINITY;
    if (cnt > topk) {
      const uint32_t kkey = bu::select_kth<LMH_F_NT>(list, cnt, topk, s_sel, s_bc, tid);
      thr = quotient_class_floor(okey_to_float(kkey), Tm);
    }
    __syncthreads();
    if (tid == 0) s_cnt = 0;
    __syncthreads();
    for (int j = tid; j < cnt; j += LMH_F_NT) {
      const uint2 e = list[j];
      if (__uint_as_float(e.x) >= thr) { const int slot = atomicAdd(&s_cnt, 1); if (slot < KEEP_MAX) kept[slot] = e; }
    }
    __syncthreads();
    const int nk = s_cnt;
    // Everything at or above the exact threshold must be on the list: that holds when the exact
    // threshold (the floor of the k-th value's class of equal quotients) is not below the list's own.
    if (nk > KEEP_MAX || cnt <= topk || !(thr >= M.thr[row])) { give_up(); continue; }
    const bool topp_on = (cfg.top_p > 0.0f && cfg.top_p < 1.0f);
    const int mode = cfg.topp_mode;
    const double plim = (mode == 0) ? static_cast<double>(cfg.top_p) * 1.5 : static_cast<double>(cfg.top_p);
    finish_small_set<LMH_F_NT>(A, row, kept, nk, m, Tm, topp_on, mode, plim, A.uniforms[row], work, sc, s_bcd, dbg, 0u);
  }
}

}  // namespace gs
