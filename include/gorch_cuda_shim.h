/* gorch CUDA shim: the C ABI of libgorchcuda.so.
 *
 * A third backend package next to the reference's metal/ and accelerate/
 * shims, for ONE path: the decode-time sampling step that
 * model.GenerateWithConfig / generateCached (model/generate.go:71-79,
 * :105-113) and qwen.Generate (model/qwen/generate.go:47-53) apply to LM-head
 * logits. Conventions follow metal/shim.h: opaque void* handles
 * (metal/shim.h:8-13), create/release pairs (:16-17, :230-231), NULL or a
 * non-zero int on failure with a strdup'd message through char** errOut
 * (:30-35) that the caller frees (:233-234), a blocking default with an
 * explicit sync for the asynchronous forms (:209-228). Plain C, no C++ types.
 *
 * Threading: one stream per context; calls on one context are not
 * concurrent (metal/shim.h:223-224). Contexts on different devices are
 * independent.
 */
#ifndef GORCH_CUDA_SHIM_H
#define GORCH_CUDA_SHIM_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* GorchCudaCtxRef;    /* device + stream + scratch; cf. MTLDeviceRef/MTLCommandQueueRef */
typedef void* GorchCudaBufferRef; /* device allocation; cf. MTLBufferRef */

/* Return codes (0 = success, like metal/shim.h:118-126). */
#define GORCH_CUDA_OK 0
#define GORCH_CUDA_ERR_BAD_ARG 1
#define GORCH_CUDA_ERR_CUDA 2
#define GORCH_CUDA_ERR_NCCL 3
#define GORCH_CUDA_ERR_LIMIT 5

/* Element types of a logits tensor. bf16 rows are upcast in-kernel by
 * bits << 16, the reference's bf16ToF32 (tensor.go:96-99). */
#define GORCH_CUDA_F32 0
#define GORCH_CUDA_BF16 1

/* Which of the reference's two top-p routines a row follows. */
#define GORCH_TOPP_MODE_A 0 /* model/generate.go:184-228 */
#define GORCH_TOPP_MODE_B 1 /* model/qwen/generate.go:123-153 */

/* Per-row flags written to out_flags. */
#define GORCH_FLAG_BOUNDARY 0x001u     /* uniform within 1e-6 of an edge of the chosen CDF interval */
#define GORCH_FLAG_FALLBACK 0x002u     /* walk fell through: id = V-1 (model/generate.go:239) */
#define GORCH_FLAG_NONFINITE 0x004u    /* NaN/Inf poisoned the softmax; id = V-1 as upstream */
#define GORCH_FLAG_TIE_CUT 0x008u      /* mode B cut separates equal probabilities */
#define GORCH_FLAG_TOPP_EDGE 0x020u    /* top-p stop test decided within 1e-12 of its threshold */
#define GORCH_FLAG_GENERAL_PATH 0x040u /* informational: row took the full-row path */
#define GORCH_FLAG_INTERNAL 0x080u     /* an internal invariant failed; id = -1 or unreliable */
#define GORCH_FLAG_BAD_CFG 0x100u      /* temperature negative, NaN or infinite; id = -1 */

/* The sampling fields of GenerateConfig (model/generate.go:13-20; qwen:
 * model/qwen/generate.go:13-20), one record per row. temperature 0 => greedy
 * (generate.go:75); top_k <= 0 or >= V => off (:157); top_p <= 0 or >= 1 =>
 * off (:184). */
typedef struct {
  float temperature;
  int32_t top_k;
  float top_p;
  int32_t topp_mode;
} GorchSampleCfg;

/* Optional per-row diagnostics for parity checks. */
typedef struct {
  double sum_exp;   /* softmax denominator (generate.go:173-178) */
  double resum;     /* top-p renormaliser (generate.go:221-227), 1 when inactive */
  double edge_lo;   /* cumulative before the chosen token */
  double edge_hi;   /* cumulative through the chosen token */
  int32_t kept;     /* tokens with non-zero final probability */
  float max_scaled; /* max of logits/T (generate.go:167-172) */
  float threshold;  /* top-k threshold (generate.go:158); NaN when inactive */
  int32_t path;     /* 0 greedy, 1 small-set path, 2 full-row path */
  uint32_t reserved[8]; /* unspecified */
} GorchSampleDebug;

typedef struct {
  uint64_t sample_launches; /* sampling calls dispatched, cf. MetalDispatchCounts (ops.go:17-78) */
  uint64_t kernel_launches; /* CUDA kernels launched by those calls */
  uint64_t argmax_launches;
  uint64_t rows;
  uint64_t h2d_bytes;       /* cf. metal.go:64-101 byte counters */
  uint64_t d2h_bytes;
  float last_kernel_ms;     /* device time of the last timed call (0 when timing is off) */
  float vs_local_ms;        /* phases of the last timed gorch_cuda_sample_vocab_sharded_dev: local pass, */
  float vs_gather_ms;       /* all-gather, */
  float vs_merge_ms;        /* merge */
  uint64_t lm_head_refused_rows; /* rows gorch_cuda_lm_head_sample_dev's fused form handed back (the batch was then redone unfused) */
} GorchCudaCounters;

/* ---- lifecycle: replaces metal_create_device / metal_create_command_queue /
 * metal_release / metal_free_string (metal/shim.h:16-17, 230-234) ---- */
int gorch_cuda_device_count(int* count, char** errOut);
GorchCudaCtxRef gorch_cuda_create_ctx(int device, char** errOut);
void gorch_cuda_release(GorchCudaCtxRef ctx);
void gorch_cuda_free_string(char* s);
/* Block until all work queued on the context is done; cf. metal_sync_queue
 * (metal/shim.h:228). */
int gorch_cuda_sync(GorchCudaCtxRef ctx, char** errOut);
/* external != 0: run the context's work on the caller-owned CUDA stream
 * `stream` (a cudaStream_t as void*; NULL is the legacy default stream).
 * external == 0: go back to the context's own stream. */
int gorch_cuda_set_stream(GorchCudaCtxRef ctx, void* stream, int external, char** errOut);
/* Record device time of each call into counters.last_kernel_ms (adds a sync). */
int gorch_cuda_set_timing(GorchCudaCtxRef ctx, int on);
int gorch_cuda_get_counters(GorchCudaCtxRef ctx, GorchCudaCounters* out);
/* Test hook, not part of the drop-in surface: which kernels serve the sampling calls, so that the
 * parity tests can run every kernel on every case. variant 0 (default): by batch size (large
 * batches: the narrow and wide kernels, each taking the rows of its kind; small ones: one
 * thread-block cluster per row with the row held in shared memory); 1: one CTA per row re-reading
 * global memory (an independent second implementation); 2: force the large-batch kernels; 3: force
 * the shared-memory cluster kernel; 4 / 5: as 2, with the wide kernel's 256-thread (four CTAs per
 * SM) / 1024-thread (one CTA per SM) instance forced instead of chosen by batch size; 6 / 7: as 2,
 * with the narrow kernel's 128-thread (eight CTAs per SM) / 256-thread (five CTAs per SM) instance
 * forced. cluster_size
 * 0 picks the cluster size of variant 3 from the shape; 1, 2, 4, 8 force it. */
int gorch_cuda_set_kernel_variant(GorchCudaCtxRef ctx, int variant, int cluster_size, char** errOut);

/* ---- device buffers: replaces metal_create_shared_buffer /
 * metal_buffer_contents / metal_release_buffer (metal/shim.h:21-28). CUDA
 * memory is not host-visible, so contents move by upload/download. ---- */
GorchCudaBufferRef gorch_cuda_buffer_alloc(GorchCudaCtxRef ctx, uint64_t bytes, char** errOut);
void gorch_cuda_buffer_free(GorchCudaBufferRef buf);
uint64_t gorch_cuda_buffer_length(GorchCudaBufferRef buf);
void* gorch_cuda_buffer_device_ptr(GorchCudaBufferRef buf);
int gorch_cuda_buffer_upload(GorchCudaBufferRef buf, uint64_t offset, const void* host,
                             uint64_t bytes, char** errOut);
int gorch_cuda_buffer_download(GorchCudaBufferRef buf, uint64_t offset, void* host,
                               uint64_t bytes, char** errOut);

/* ---- the sampling step ----
 * Replaces the branch `if cfg.Temperature == 0 { argmax } else { sample }` at
 * model/generate.go:75-79 and :109-113 (qwen: model/qwen/generate.go:49-53),
 * i.e. argmax (generate.go:134-144), sample (:147-240), kthLargest (:243-260)
 * and sampleLogits (qwen/generate.go:92-164), over a [B,V] batch of rows.
 *
 * logits      [B, row_stride] elements of `dtype`, row b at b*row_stride
 * cfgs        [B] per-row configuration
 * uniforms    [B] doubles in [0,1): the value the reference takes from
 *             rand.Float64() (generate.go:231 / qwen/generate.go:155)
 * out_ids     [B] sampled token ids
 * out_flags   [B] GORCH_FLAG_* bits, or NULL
 *
 * Host form: all pointers are host memory; copies in and out happen inside
 * the call, which blocks until the ids are written. */
int gorch_cuda_sample_host(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                           int64_t V, int64_t row_stride, const GorchSampleCfg* cfgs,
                           const double* uniforms, int32_t* out_ids, uint32_t* out_flags,
                           char** errOut);
/* Device form: all pointers are device memory on the context's device; the
 * launch is asynchronous on the context's stream (gorch_cuda_sync to wait).
 * out_probs ([B,V] doubles: the filtered, renormalised distribution of
 * generate.go:181/:227) and out_debug ([B]) may be NULL. */
int gorch_cuda_sample_dev(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                          int64_t V, int64_t row_stride, const GorchSampleCfg* cfgs,
                          const double* uniforms, int32_t* out_ids, uint32_t* out_flags,
                          double* out_probs, GorchSampleDebug* out_debug, char** errOut);

/* No counterpart in the reference. Same work, same dispatch and same results as
 * gorch_cuda_sample_dev (without the optional probability / diagnostic outputs), for callers that
 * must not trigger a device allocation: a decode loop that is being recorded into a CUDA stream
 * capture, where cudaMalloc is not permitted, or a serving process whose memory budget is fixed up
 * front and that treats any later cudaMalloc (which also synchronises the device) as a fault. The
 * row work lists that the other entry point keeps in a grow-only cudaMalloc'd buffer live here in
 * a fixed array inside the library image: about 16 KB of device memory on every GPU that loads the
 * library, held until the process exits.
 *   - at most 4096 rows per call; more is refused with GORCH_CUDA_ERR_LIMIT;
 *   - the array's device address is looked up (cudaGetSymbolAddress) when a context is created
 *     on the device, not inside this call;
 *   - all calls on a device share the one array: two calls whose kernels overlap on the GPU
 *     (different streams or contexts) race on it. Calls on one stream are safe: the cursors and
 *     counts are cleared at the start of every call;
 *   - neither this function nor anything it calls uses cudaMalloc or cudaFree. */
int gorch_cuda_sample_dev_static(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                                 int64_t V, int64_t row_stride, const GorchSampleCfg* cfgs,
                                 const double* uniforms, int32_t* out_ids, uint32_t* out_flags,
                                 char** errOut);

/* Vocab-sharded sampling (no counterpart in the reference, which runs on one device): every
 * rank holds the same B rows but only the columns [col_offset, col_offset + Vslice) of the
 * vocabulary. Rows must have 0 < top_k <= GORCH_VS_CAND (the top-k bounds what has to cross the
 * link) or temperature 0; rows with top_k == 0 and no effective top-p cut (top_p off, or the
 * model/generate.go rule with 1.5 top_p >= 1) are served by the calls that name a row's owner
 * (gorch_cuda_vocab_merge_owner_dev, gorch_cuda_sample_vocab_sharded_ex_dev); all other rows come
 * back with id -1 and GORCH_FLAG_INTERNAL.
 *   1. every rank: gorch_cuda_vocab_local_dev fills B records of GORCH_VS_RECORD_BYTES (local
 *      maximum, and every local logit at or above the local top_k-th largest with its global
 *      index: 16 header bytes + GORCH_VS_CAND pairs of (f32 bits, u32 index));
 *   2. the caller all-gathers the records in rank order (NCCL; nranks * B records);
 *   3. every rank: gorch_cuda_vocab_merge_dev joins the lists, keeps everything at or above the
 *      global top_k-th largest (ties kept, model/generate.go:157-164) and finishes the row as
 *      gorch_cuda_sample_dev does. Every rank computes all B ids, so no second exchange is needed.
 * Device pointers, asynchronous on the context's stream. */
#define GORCH_VS_CAND 128
#define GORCH_VS_RECORD_BYTES (16 + 8 * GORCH_VS_CAND)
int gorch_cuda_vocab_local_dev(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                               int64_t Vslice, int64_t row_stride, int64_t col_offset,
                               const GorchSampleCfg* cfgs, void* records, char** errOut);
int gorch_cuda_vocab_merge_dev(GorchCudaCtxRef ctx, const void* all_records, int nranks, int64_t B,
                               int64_t V, const GorchSampleCfg* cfgs, const double* uniforms,
                               int32_t* out_ids, uint32_t* out_flags, char** errOut);
/* Rows without top-k (plain softmax sampling over the whole vocabulary): a slice's record holds its
 * maximum and its sum of exponentials relative to that maximum (generate.go:167-181 on the slice).
 * gorch_cuda_vocab_merge_owner_dev is gorch_cuda_vocab_merge_dev that also serves such rows: it adds
 * the slices' sums, rescaled to the row's maximum, in rank order, and names the rank in whose
 * slice uniform * sum falls the row's owner; rank my_rank's draw_req [B][3] doubles then tells
 * gorch_cuda_vocab_draw_dev, which runs on every rank over its own slice, which rows it owns and
 * where in its slice's running sum the token lies; it writes the token into out_ids / out_flags of
 * the rows it owns. The other ranks hold -1 and 0 there: a max-reduction of out_ids and out_flags
 * over the ranks gives every rank every token (rows with a top-k already agree). The sums are
 * formed per slice, so such a row's token can differ from the one-device result when the uniform
 * lies within 1e-6 of an edge of the chosen interval (GORCH_FLAG_BOUNDARY). */
int gorch_cuda_vocab_merge_owner_dev(GorchCudaCtxRef ctx, const void* all_records, int nranks, int my_rank,
                                     int64_t B, int64_t V, const GorchSampleCfg* cfgs, const double* uniforms,
                                     int32_t* out_ids, uint32_t* out_flags, double* draw_req, char** errOut);
int gorch_cuda_vocab_draw_dev(GorchCudaCtxRef ctx, const void* logits_slice, int dtype, int64_t B,
                              int64_t Vslice, int64_t row_stride, int64_t col_offset,
                              const GorchSampleCfg* cfgs, const double* draw_req, int32_t* out_ids,
                              uint32_t* out_flags, char** errOut);

/* The three steps above as ONE call, with the collective inside the library (no counterpart in the
 * reference): local pass -> ncclAllGather of the records on the context's stream -> merge. Every
 * rank calls it with its own column slice of the same B rows and gets all B ids. The records that
 * cross the link hold max_top_k plus a quarter (room for ties at the local threshold) candidates
 * instead of GORCH_VS_CAND: max_top_k is the largest top_k among the batch's rows (0 or above
 * GORCH_VS_CAND: full records). A failing NCCL call returns GORCH_CUDA_ERR_NCCL with its message.
 *
 * gorch_cuda_comm_unique_id: rank 0 makes the 128-byte id (ncclGetUniqueId) and hands it to the
 * other ranks by whatever channel the host program has; gorch_cuda_comm_init (collective: every
 * rank calls it) binds a communicator of `nranks` ranks to the context (ncclCommInitRank on the
 * context's device); gorch_cuda_comm_release destroys it (gorch_cuda_release does too). libnccl.so.2
 * is loaded at the first of these calls; a process that never calls them does not need it. */
#define GORCH_CUDA_UNIQUE_ID_BYTES 128
int gorch_cuda_comm_unique_id(void* id_bytes, char** errOut);
int gorch_cuda_comm_init(GorchCudaCtxRef ctx, int rank, int nranks, const void* unique_id_bytes, char** errOut);
int gorch_cuda_comm_release(GorchCudaCtxRef ctx, char** errOut);
int gorch_cuda_sample_vocab_sharded_dev(GorchCudaCtxRef ctx, const void* logits_slice, int dtype, int64_t B,
                                        int64_t Vslice, int64_t row_stride, int64_t col_offset, int64_t V,
                                        int max_top_k, const GorchSampleCfg* cfgs, const double* uniforms,
                                        int32_t* out_ids, uint32_t* out_flags, char** errOut);
/* The same for batches that hold rows with top_k == 0; rows_without_top_k is a set of bits, 0 being
 * the call above. Bit 0: rows whose top-p cut removes nothing (off, or generate.go's rule with
 * 1.5 p >= 1) are served from the slices' sums: after the merge the owners draw from their slices
 * and two small ncclAllReduce (max) calls, over out_ids and out_flags, hand the tokens to every
 * rank. Bit 1: the rows with top_k == 0 that are left (an active cut over the whole vocabulary:
 * qwen/generate.go:123-153; with bit 0 clear every sampling row with top_k == 0) are sampled from
 * whole rows: every rank's slice goes into a [B, V] scratch buffer, one ncclAllReduce (sum) fills
 * in the others', and gorch_cuda_sample_dev's kernels take those rows on every rank. That is
 * correct and not fast (B * V elements cross the links), and it needs scratch memory for B whole
 * rows. out_flags is required with either bit. */
int gorch_cuda_sample_vocab_sharded_ex_dev(GorchCudaCtxRef ctx, const void* logits_slice, int dtype, int64_t B,
                                           int64_t Vslice, int64_t row_stride, int64_t col_offset, int64_t V,
                                           int max_top_k, int rows_without_top_k, const GorchSampleCfg* cfgs,
                                           const double* uniforms, int32_t* out_ids, uint32_t* out_flags,
                                           char** errOut);

/* The reference's tensor-level index ops as batched device ops (device pointers, asynchronous on
 * the context's stream).
 * TopK (index_ops.go:153-190): the k largest of each row of x [B,V] (f32, or bf16 upcast), values
 * [B,k] descending and their indices [B,k]; equal values by ascending index (upstream's sort is
 * unstable, so that order is unspecified there); NaNs order last. 1 <= k <= min(V, 16384), else
 * GORCH_CUDA_ERR_LIMIT. k <= 256 is served in one pass over the row; there a row with more than 512
 * logits tied at its k-th value (which includes a row with fewer than k logits above -Inf) gets
 * indices -1 and GORCH_FLAG_INTERNAL in out_flags (may be NULL). k > 256 takes a radix select over
 * the row (several passes, the row coming from L2 after the first) and has no such limit on ties.
 * Multinomial (index_ops.go:203-227): out_ids[b] = first j with uniforms[b] < sum_{i<=j} probs[b,i]
 * (f64 running sum over f32 probabilities), else V-1 (GORCH_FLAG_FALLBACK). The sum is formed in a
 * different order than upstream's loop; rows whose uniform lies within 1e-6 of an edge of the
 * chosen interval carry GORCH_FLAG_BOUNDARY. Rows up to 524 224 probabilities. */
int gorch_cuda_topk_dev(GorchCudaCtxRef ctx, const void* x, int dtype, int64_t B, int64_t V,
                        int64_t row_stride, int64_t k, float* out_values, int32_t* out_indices,
                        uint32_t* out_flags, char** errOut);
int gorch_cuda_multinomial_dev(GorchCudaCtxRef ctx, const float* probs, int64_t B, int64_t V,
                               int64_t row_stride, const double* uniforms, int32_t* out_ids,
                               uint32_t* out_flags, char** errOut);

/* The bookkeeping of the reference's generate loops for a batch of sequences, on the device: the
 * token ids stay in device memory between decode steps and the host no longer has to read each
 * step's id back to decide whether to go on (model/generate.go:60-88 uncached, :107-129 cached;
 * model/qwen/generate.go:47-61). All pointers are device pointers owned by the caller.
 *
 * For every row with done[b] == GORCH_GEN_LIVE, one loop iteration in the reference's order:
 * the iteration limit (n_new[b] >= max_new => GORCH_GEN_MAX_NEW); the stop test, the stop token
 * NOT appended (=> GORCH_GEN_STOP; stop_tokens entries < 0 never match, which is StopToken = -1 of
 * generate.go:82); the append to tokens[b, lengths[b]]; then, cached != 0: cache_len[b] >= max_seq
 * => GORCH_GEN_MAX_SEQ (generate.go:121-123), else next_input[b] = id and cache_len[b]++;
 * cached == 0: next_input[b] = id and window_start[b] (may be NULL) = start of the last max_seq
 * tokens of the row (generate.go:62-65). A row whose max_new-th token was just appended becomes
 * GORCH_GEN_MAX_NEW at once. An id < 0, a sampler flag in GORCH_FLAG_INTERNAL | GORCH_FLAG_BAD_CFG
 * (flags may be NULL) or a full token buffer => GORCH_GEN_ERROR, nothing appended.
 * live_count[0] = rows still live after the step.
 *
 * Before the first step the caller fills tokens/lengths with the prompts (cached loops of
 * generate.go: truncated to their last max_seq tokens, :101-103), n_new = 0, done = 0 and
 * cache_len = prompt length after the prefill. */
#define GORCH_GEN_LIVE 0
#define GORCH_GEN_STOP 1
#define GORCH_GEN_MAX_NEW 2
#define GORCH_GEN_MAX_SEQ 3
#define GORCH_GEN_ERROR 4
#define GORCH_GEN_MAX_STOPS 16
typedef struct {
  int32_t* tokens;       /* [B, capacity] */
  int64_t capacity;      /* >= prompt length + max_new */
  int32_t* lengths;      /* [B] */
  int32_t* n_new;        /* [B] */
  int32_t* cache_len;    /* [B]; read and written only when cached != 0 */
  int32_t* done;         /* [B] GORCH_GEN_* */
  int32_t* next_input;   /* [B] */
  int32_t* window_start; /* [B] or NULL; written only when cached == 0 */
  int32_t* live_count;   /* [1] */
  int32_t stop_tokens[GORCH_GEN_MAX_STOPS];
  int32_t n_stop;        /* 0..GORCH_GEN_MAX_STOPS */
  int32_t max_new;       /* MaxNewTokens */
  int32_t max_seq;       /* MaxSeq */
  int32_t cached;        /* 0: GenerateWithConfig without KV cache; else the cached loops */
} GorchGenControl;
/* The control step alone, over ids (and flags, may be NULL) that a sampling call on the same
 * context has written. One launch, asynchronous on the context's stream. */
int gorch_cuda_generate_control_dev(GorchCudaCtxRef ctx, const int32_t* ids, const uint32_t* flags,
                                    const GorchGenControl* gc, int64_t B, char** errOut);
/* gorch_cuda_sample_dev followed by the control step in one call: out_ids / out_flags receive the
 * sampled ids of the live rows; rows that have ended (done[b] != GORCH_GEN_LIVE) are skipped by the
 * sampling kernels, as the reference leaves its loop (model/generate.go:82-84), and their entries
 * of out_ids / out_flags keep what they held. */
int gorch_cuda_generate_step_dev(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                                 int64_t V, int64_t row_stride, const GorchSampleCfg* cfgs,
                                 const double* uniforms, int32_t* out_ids, uint32_t* out_flags,
                                 const GorchGenControl* gc, char** errOut);

/* Row softmax, log-softmax and cross-entropy over x [B,V] (f32, or bf16 upcast) at vocabulary
 * scale, as device ops (device pointers, asynchronous on the context's stream).
 * gorch_cuda_softmax_dev: log_softmax == 0: gorch.Softmax (ops.go:527-563), out = exp(x - max) /
 * sum; else gorch.LogSoftmax (ops.go:566-603), out = x - max - log(sum). out [B,out_stride] has
 * x's type (bf16: rounded to nearest even, as downcastToBF16). out may not overlap x.
 * gorch_cuda_cross_entropy_fwd_dev (loss.go:55-124): row_lse[b] = max + log(sum exp(x - max)),
 * row_loss[b] = row_lse[b] - x[b, targets[b]], mean_loss[0] = sum(row_loss) / B (may be NULL). A
 * target outside [0,V) makes that row's loss NaN (upstream panics).
 * gorch_cuda_cross_entropy_bwd_dev (loss.go:128-141): dx[b,j] = exp(x[b,j] - row_lse[b]) * scale,
 * minus scale at j = targets[b]; dx is f32 [B,dx_stride]; scale = upstream grad / batch.
 * The row sum is formed in another order and a higher precision than upstream's sequential f32
 * loop; everything else keeps upstream's f32 roundings. */
int gorch_cuda_softmax_dev(GorchCudaCtxRef ctx, const void* x, int dtype, int64_t B, int64_t V,
                           int64_t row_stride, void* out, int64_t out_stride, int log_softmax,
                           char** errOut);
int gorch_cuda_cross_entropy_fwd_dev(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                                     int64_t V, int64_t row_stride, const int32_t* targets,
                                     float* row_loss, float* row_lse, float* mean_loss,
                                     char** errOut);
int gorch_cuda_cross_entropy_bwd_dev(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                                     int64_t V, int64_t row_stride, const int32_t* targets,
                                     const float* row_lse, float scale, float* dx,
                                     int64_t dx_stride, char** errOut);

/* The LM-head projection that produces the logits: logits[b, v] = sum_k x[b, k] * w[v, k], i.e.
 * MatMulTransB(last, m.Embed.Weight) of model/qwen/qwen.go:80-85 (GPT-2: nn/gpt.go:119-120; the CPU
 * loop is nn/extembed.go:152-195), for x [B, K] and w [V, K] in bf16 (bit patterns, row pitches ldx /
 * ldw in elements) with f32 accumulation on the tensor cores. K must be a multiple of 64; pointers and
 * row pitches multiples of 16 bytes. Device pointers, asynchronous on the context's stream.
 * gorch_cuda_lm_head_status (blocking) reads the status word of the last LM-head call: 0, or bit 0 when
 * a bounded device-side wait ran out (the output is then incomplete). */
int gorch_cuda_lm_head_logits_dev(GorchCudaCtxRef ctx, const void* x, int64_t ldx, const void* w, int64_t ldw,
                                  int64_t B, int64_t V, int64_t K, float* out_logits, int64_t ld_out,
                                  char** errOut);
int gorch_cuda_lm_head_status(GorchCudaCtxRef ctx, uint32_t* status, char** errOut);
/* The projection and the sampling step in one call: out_ids[b] = the token sampled from row b of
 * x @ w^T under cfgs[b] with uniforms[b], as gorch_cuda_sample_dev would return on the materialised
 * logits. fuse_top_k in 1..256: the batch's largest top_k; rows with temperature 0 or 0 < top_k <=
 * fuse_top_k (DefaultGenerateConfig: T = 0.8, k = 40) are finished from candidate lists that the
 * projection's epilogue fills, and the [B, V] logits are never written; the call then blocks until
 * the ids are there, and if a row could not be finished that way (top_k off or above fuse_top_k, or
 * a row whose largest logits a sample of the vocabulary misjudged) the whole batch is redone through
 * the unfused form. fuse_top_k == 0 (or a vocabulary below 4096 columns, or more than 4096 rows): the
 * unfused form at once:
 * logits into scratch memory of the context, then the kernels of gorch_cuda_sample_dev
 * (asynchronous). */
int gorch_cuda_lm_head_sample_dev(GorchCudaCtxRef ctx, const void* x, int64_t ldx, const void* w, int64_t ldw,
                                  int64_t B, int64_t V, int64_t K, int fuse_top_k, const GorchSampleCfg* cfgs,
                                  const double* uniforms, int32_t* out_ids, uint32_t* out_flags, char** errOut);

/* One row, the exact shape of the reference's calls: sample(logits,
 * temperature, topK, topP) (generate.go:147) with the uniform passed in, and
 * argmax when temperature == 0. Returns the token id, or -1 with *errOut set. */
int64_t gorch_cuda_sample_row(GorchCudaCtxRef ctx, const float* logits, int64_t n,
                              float temperature, int64_t top_k, float top_p, int topp_mode,
                              double uniform, uint32_t* out_flag, char** errOut);

/* Greedy fast path: argmax (generate.go:134-144; argmaxF32 qwen/generate.go:77-87;
 * the inline loops at model/gpt2_loader.go:266-273 and model/qwen/voice.go:175)
 * over every row; lowest index wins ties. */
int gorch_cuda_argmax_host(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                           int64_t V, int64_t row_stride, int32_t* out_ids, char** errOut);
int gorch_cuda_argmax_dev(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                          int64_t V, int64_t row_stride, int32_t* out_ids, char** errOut);

#ifdef __cplusplus
}
#endif

#endif /* GORCH_CUDA_SHIM_H */
