// libgorchcuda.so: implementation of include/gorch_cuda_shim.h.
//
// Host-side conventions mirror the reference's Metal shim (metal/shim.m):
// opaque handles, strdup'd error strings, int return codes, a blocking default.
// There is no CPU fallback anywhere in this file: every entry point either
// runs the CUDA kernels or returns an error.

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>     // types and prototypes only: the library is loaded at run time, on first use

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <new>

#include "../../include/gorch_cuda_shim.h"
#define GS_W_NS w256
#define GS_W_NT 256
#include "sample_wide.cuh"      // gs::w256: 256 threads, four CTAs per SM (throughput)
#define GS_W_NS w1024
#define GS_W_NT 1024
#include "sample_wide.cuh"      // gs::w1024: 1024 threads, one CTA per SM (latency)
#include "sample_vocab.cuh"
#include "index_ops.cuh"
#include "generate_control.cuh"
#include "row_softmax.cuh"
#include "lm_head.cuh"

namespace {

// Largest slice kept in shared memory: 109 KB of dynamic shared memory per CTA
// (two CTAs per SM) minus the two 16 KB work regions.
constexpr int64_t kSliceCap = 109 * 1024 - gs::REGION_A - gs::REGION_B;

// Batches of at least this many rows are sorted by kind and served by the narrow / wide
// kernels; smaller ones use one cluster per row so that every SM still has work.
// Batches go to the sorted-batch kernels (one CTA per row) from this many rows on; smaller ones to
// the cluster kernel (several CTAs per row), whose latency is lower while the GPU is not full.
// Measured crossovers on B200: 40 rows of 608 KB, ~120 rows of 200 KB.
constexpr int64_t kBatchModeRows = 384;
constexpr int64_t kBatchModeBytes = 24ll << 20;
inline bool use_batch_mode(int64_t B, int64_t row_bytes) {
  if (B >= kBatchModeRows) return true;
  return B >= 32 && B * row_bytes >= kBatchModeBytes;
}

struct Buffer {
  int device;
  void* ptr;
  uint64_t bytes;
};

struct Scratch {  // grow-only device allocation
  void* ptr = nullptr;
  size_t cap = 0;
};

struct Ctx {
  int device = 0;
  int sm_count = 148;
  int64_t l2_bytes = 126ll << 20;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  cudaStream_t side_stream = nullptr;     // the wide kernel of a mixed batch runs here, beside the narrow one
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  double* exp_table = nullptr;
  double* eb_table = nullptr;
  Scratch worklist;        // int32[1 + rows]: rows the cluster kernel leaves to the single-CTA kernel
  Scratch st_logits, st_cfgs, st_uniforms, st_ids, st_flags;
  Scratch lmh_scratch;       // status word, thresholds, candidate lists, sample logits of the LM-head path
  Scratch lmh_logits;        // [B, V] f32 when rows need the unfused samplers
  Scratch vs_local, vs_all;  // records of the vocab-sharded call: this rank's, and every rank's after the all-gather
  Scratch vs_req;            // [B][3] doubles: what the owner's draw of a row without top-k needs
  Scratch vs_rows, vs_done;  // whole rows [B][V padded] and the mask of rows that do not need them (vocab-sharded rows without top-k that are gathered)
  ncclComm_t comm = nullptr; // set by gorch_cuda_comm_init
  int comm_rank = 0, comm_nranks = 0;
  cudaEvent_t ev_vs[4] = {nullptr, nullptr, nullptr, nullptr};
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  int timing = 0;
  int variant = 0;        // 0: by batch size, 1: single-CTA kernel, 2: narrow/wide kernels, 3: cluster kernel,
                          // 4 / 5: as 2 with the wide kernel's 256- / 1024-thread instance forced,
                          // 6 / 7: as 2 with the narrow kernel's 128- / 256-thread instance forced
  int force_cluster = 0;  // 0: choose from the shape
  GorchCudaCounters counters{};
};

// Work lists for gorch_cuda_sample_dev_static: fixed storage inside the loaded module, so the
// entry point never allocates. Every GPU that loads the library holds one copy (about 16 KB)
// until the process exits. In host code this name is only a handle for cudaGetSymbolAddress;
// the device address is looked up once per device (static_lists_ptr, called by gorch_cuda_create_ctx with
// that device current) and passed to the kernels.
constexpr int64_t kStaticMaxRows = 4096;
static __device__ __align__(256) int32_t g_static_worklists[16 + kStaticMaxRows + 1];
constexpr int kMaxDevices = 64;
int32_t* g_static_ptr[kMaxDevices] = {};

// Device address of g_static_worklists on the CURRENT device (looked up once per device).
int static_lists_ptr(int device, int32_t** out, char** errOut);

void set_err(char** errOut, const char* fmt, ...) {
  if (!errOut) return;
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  *errOut = strdup(buf);
}

#define CUDA_TRY(expr, errOut)                                                   \
  do {                                                                           \
    cudaError_t e__ = (expr);                                                    \
    if (e__ != cudaSuccess) {                                                    \
      set_err(errOut, "%s failed: %s", #expr, cudaGetErrorString(e__));          \
      return GORCH_CUDA_ERR_CUDA;                                                \
    }                                                                            \
  } while (0)

// NCCL, loaded on first use (a process that never shards the vocabulary does not need it). Inside a
// process that already holds a libnccl.so.2 (PyTorch's), the loader hands back that same copy.
struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};
NcclApi g_nccl;

int load_nccl(char** errOut) {
  if (g_nccl.handle) return GORCH_CUDA_OK;
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) {
    set_err(errOut, "gorch_cuda: cannot load libnccl.so.2: %s", dlerror());
    return GORCH_CUDA_ERR_NCCL;
  }
  NcclApi a;
  a.handle = h;
  a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
  a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
  a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
  a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(h, "ncclAllGather"));
  a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(h, "ncclAllReduce"));
  a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
  if (!a.GetUniqueId || !a.CommInitRank || !a.CommDestroy || !a.AllGather || !a.AllReduce || !a.GetErrorString) {
    set_err(errOut, "gorch_cuda: libnccl.so.2 lacks a symbol this library needs");
    return GORCH_CUDA_ERR_NCCL;
  }
  g_nccl = a;
  return GORCH_CUDA_OK;
}

#define NCCL_TRY(expr, errOut)                                                   \
  do {                                                                           \
    ncclResult_t r__ = (expr);                                                   \
    if (r__ != ncclSuccess) {                                                    \
      set_err(errOut, "%s failed: %s", #expr, g_nccl.GetErrorString(r__));       \
      return GORCH_CUDA_ERR_NCCL;                                                \
    }                                                                            \
  } while (0)

int static_lists_ptr(int device, int32_t** out, char** errOut) {
  if (device < 0 || device >= kMaxDevices) {
    set_err(errOut, "gorch_cuda: device index %d beyond the static table", device);
    return GORCH_CUDA_ERR_LIMIT;
  }
  if (!g_static_ptr[device]) {
    void* p = nullptr;
    CUDA_TRY(cudaGetSymbolAddress(&p, g_static_worklists), errOut);
    g_static_ptr[device] = static_cast<int32_t*>(p);
  }
  *out = g_static_ptr[device];
  return GORCH_CUDA_OK;
}

int ensure(Scratch& s, size_t bytes, char** errOut) {
  if (bytes <= s.cap) return GORCH_CUDA_OK;
  if (s.ptr) {
    CUDA_TRY(cudaFree(s.ptr), errOut);
    s.ptr = nullptr;
    s.cap = 0;
  }
  size_t want = bytes + (bytes >> 3);
  cudaError_t e = cudaMalloc(&s.ptr, want);
  if (e != cudaSuccess) {
    want = bytes;
    e = cudaMalloc(&s.ptr, want);
  }
  if (e != cudaSuccess) {
    s.ptr = nullptr;
    set_err(errOut, "cudaMalloc(%zu bytes) failed: %s", bytes, cudaGetErrorString(e));
    return GORCH_CUDA_ERR_CUDA;
  }
  s.cap = want;
  return GORCH_CUDA_OK;
}

int check_shape(int dtype, int64_t B, int64_t V, int64_t row_stride, char** errOut) {
  if (dtype != GORCH_CUDA_F32 && dtype != GORCH_CUDA_BF16) {
    set_err(errOut, "gorch_cuda: unknown dtype %d", dtype);
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  if (B < 0 || V < 1 || row_stride < V) {
    set_err(errOut, "gorch_cuda: bad shape B=%lld V=%lld row_stride=%lld", (long long)B,
            (long long)V, (long long)row_stride);
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  if (V > 0x7fffff00ll || B > 0x7fffffffll) {
    set_err(errOut, "gorch_cuda: shape beyond 31-bit row / batch limit");
    return GORCH_CUDA_ERR_LIMIT;
  }
  return GORCH_CUDA_OK;
}

size_t elem_size(int dtype) { return dtype == GORCH_CUDA_BF16 ? 2 : 4; }

// The narrow kernel's two instances: 256-thread CTAs (five per SM) while every row gets a CTA slot
// of its own, 128-thread CTAs (eight per SM) beyond that. Variants 6 / 7 force one of them (tests).
static cudaError_t launch_narrow(Ctx* c, const gs::BatchArgs& ba, int dtype, int64_t B) {
  const int64_t slots256 = static_cast<int64_t>(gs::n256::N_CTAS_PER_SM) * c->sm_count;
  const bool small_ctas = c->variant == 6 || (c->variant != 7 && B > slots256);
  if (small_ctas) {
    const int64_t slots = static_cast<int64_t>(gs::n128::N_CTAS_PER_SM) * c->sm_count;
    const unsigned g = static_cast<unsigned>(B < slots ? B : slots);
    if (dtype == GORCH_CUDA_F32) gs::n128::narrow_rows_kernel<float><<<g, gs::n128::N_NT, gs::n128::N_DYN_BYTES, c->stream>>>(ba);
    else gs::n128::narrow_rows_kernel<uint16_t><<<g, gs::n128::N_NT, gs::n128::N_DYN_BYTES, c->stream>>>(ba);
  } else {
    const unsigned g = static_cast<unsigned>(B < slots256 ? B : slots256);
    if (dtype == GORCH_CUDA_F32) gs::n256::narrow_rows_kernel<float><<<g, gs::n256::N_NT, gs::n256::N_DYN_BYTES, c->stream>>>(ba);
    else gs::n256::narrow_rows_kernel<uint16_t><<<g, gs::n256::N_NT, gs::n256::N_DYN_BYTES, c->stream>>>(ba);
  }
  return cudaGetLastError();
}

int launch_rows(Ctx* c, const void* logits, int dtype, int64_t B, int64_t V, int64_t row_stride,
                const GorchSampleCfg* cfgs, const double* uniforms, int32_t* out_ids,
                uint32_t* out_flags, double* out_probs, GorchSampleDebug* out_debug,
                int force_greedy, char** errOut, int32_t* fixed_lists = nullptr, const int32_t* row_done = nullptr) {
  // fixed_lists: caller-provided storage for the row work lists (16 + B + 1 words) instead of the
  // context's grow-only allocation; with it nothing in here allocates.
  if (B == 0) return GORCH_CUDA_OK;
  static_assert(sizeof(GorchSampleCfg) == sizeof(gs::RowCfg), "cfg layout");
  static_assert(sizeof(GorchSampleDebug) == sizeof(gs::RowDebug), "debug layout");
  if ((reinterpret_cast<uintptr_t>(logits) % elem_size(dtype)) != 0) {
    set_err(errOut, "gorch_cuda: logits pointer not aligned to its element size");
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  gs::KernelArgs a;
  a.logits = logits;
  a.row_stride = row_stride;
  a.V = static_cast<int32_t>(V);
  a.force_greedy = force_greedy;
  a.cfgs = reinterpret_cast<const gs::RowCfg*>(cfgs);
  a.uniforms = uniforms;
  a.out_ids = out_ids;
  a.out_flags = out_flags;
  a.out_probs = out_probs;
  a.out_debug = reinterpret_cast<gs::RowDebug*>(out_debug);
  a.exp_table = c->exp_table;
  a.row_offset = 0;
  a.worklist = nullptr;
  a.vs_records = nullptr;
  a.vs_col_offset = 0;
  a.vs_cand = gs::VS_CAND;
  a.vs_sumexp = 0;
  a.row_done = row_done;
  a.tk_values = nullptr;
  a.tk_indices = nullptr;
  a.tk_k = 0;
  if (c->timing) CUDA_TRY(cudaEventRecord(c->ev0, c->stream), errOut);
  int klaunch = 1;
  const bool batch_mode = c->variant == 2 || c->variant >= 4 || (c->variant == 0 && use_batch_mode(B, V * static_cast<int64_t>(elem_size(dtype))));
  if (batch_mode) {
    // narrow (greedy / top-k) beside wide (top-k off), then single-CTA (whatever was handed over)
    const size_t ints = 16 + static_cast<size_t>(B) + 1;
    int32_t* base = fixed_lists;
    if (!base) {
      int rc = ensure(c->worklist, ints * sizeof(int32_t), errOut);
      if (rc) return rc;
      base = static_cast<int32_t*>(c->worklist.ptr);
    }
    gs::BatchArgs ba;
    ba.k = a;
    ba.eb_table = c->eb_table;
    ba.hdr = base;
    // the hand-over list's count is the header's last word, its rows follow: one memset clears all
    ba.list_single = base + 15;
    ba.B = B;
    CUDA_TRY(cudaMemsetAsync(base, 0, 16 * sizeof(int32_t), c->stream), errOut);
    // at most one row per SM: a 1024-thread CTA finishes its row sooner than a 256-thread one, and no SM
    // would have held a second row anyway. Beyond that the 256-thread instance wins (measured), also
    // because a 1024-thread CTA takes the whole register file and keeps the narrow kernel off its SM
    const bool wide_big_ctas = c->variant == 5 || (c->variant != 4 && B <= c->sm_count);
    const int wctas = wide_big_ctas ? gs::w1024::W_CTAS : gs::w256::W_CTAS;
    const unsigned gw = static_cast<unsigned>(B < wctas * c->sm_count ? B : wctas * c->sm_count);
    const unsigned gsgl = static_cast<unsigned>(B < 2 * c->sm_count ? B : 2 * c->sm_count);
    gs::KernelArgs aw = a;
    aw.worklist = ba.list_single;
    // The narrow and the wide kernel work on disjoint rows: the wide one runs on a side stream
    // (fork before, join before the hand-over kernel), so that a mixed batch
    // does not pay for them one after the other.
    if (!force_greedy) {
      CUDA_TRY(cudaEventRecord(c->ev_fork, c->stream), errOut);
      CUDA_TRY(cudaStreamWaitEvent(c->side_stream, c->ev_fork, 0), errOut);
      if (dtype == GORCH_CUDA_F32) {
        if (wide_big_ctas) gs::w1024::wide_rows_kernel<float><<<gw, gs::w1024::W_NT, gs::w1024::W_DYN_BYTES, c->side_stream>>>(ba);
        else gs::w256::wide_rows_kernel<float><<<gw, gs::w256::W_NT, gs::w256::W_DYN_BYTES, c->side_stream>>>(ba);
      } else {
        if (wide_big_ctas) gs::w1024::wide_rows_kernel<uint16_t><<<gw, gs::w1024::W_NT, gs::w1024::W_DYN_BYTES, c->side_stream>>>(ba);
        else gs::w256::wide_rows_kernel<uint16_t><<<gw, gs::w256::W_NT, gs::w256::W_DYN_BYTES, c->side_stream>>>(ba);
      }
    }
    CUDA_TRY(launch_narrow(c, ba, dtype, B), errOut);
    if (!force_greedy) {
      CUDA_TRY(cudaEventRecord(c->ev_join, c->side_stream), errOut);
      CUDA_TRY(cudaStreamWaitEvent(c->stream, c->ev_join, 0), errOut);
      if (dtype == GORCH_CUDA_F32) gs::sample_rows_kernel<float><<<gsgl, gs::NT, gs::POOL_BYTES, c->stream>>>(aw);
      else gs::sample_rows_kernel<uint16_t><<<gsgl, gs::NT, gs::POOL_BYTES, c->stream>>>(aw);
    }
    CUDA_TRY(cudaGetLastError(), errOut);
    klaunch = force_greedy ? 1 : 3;
  } else if (c->variant == 1) {
    dim3 grid(static_cast<unsigned>(B)), block(gs::NT);
    if (dtype == GORCH_CUDA_F32) {
      gs::sample_rows_kernel<float><<<grid, block, gs::POOL_BYTES, c->stream>>>(a);
    } else {
      gs::sample_rows_kernel<uint16_t><<<grid, block, gs::POOL_BYTES, c->stream>>>(a);
    }
    CUDA_TRY(cudaGetLastError(), errOut);
  } else {
    // Cluster size: smallest power of two whose slice fits the shared-memory
    // budget, raised for small batches so that the whole GPU has work.
    const int vec = dtype == GORCH_CUDA_F32 ? 4 : 8;
    const int64_t nvec_max = (V + 2 * (vec - 1)) / vec + 1;
    int C = 1;
    while (C < gs::CL_MAX && ((nvec_max + C - 1) / C) * 16 > kSliceCap) C *= 2;
    // (two CTAs of this kernel fit an SM: stop while all clusters are still resident at once;
    // measured on 64 rows of 50257 f32: 43 us with 4 CTAs per row, 55 us with 8)
    while (C < gs::CL_MAX && B * 2 * C <= 2 * c->sm_count && ((nvec_max + 2 * C - 1) / (2 * C)) >= 64) C *= 2;
    if (c->force_cluster) C = c->force_cluster;
    const int64_t need = ((nvec_max + C - 1) / C) * 16;
    if (need > kSliceCap || B * C > 0x7fffffffll) {
      // rows too wide to keep in shared memory: the single-CTA kernel reads global memory
      dim3 grid(static_cast<unsigned>(B)), block(gs::NT);
      if (dtype == GORCH_CUDA_F32) {
        gs::sample_rows_kernel<float><<<grid, block, gs::POOL_BYTES, c->stream>>>(a);
      } else {
        gs::sample_rows_kernel<uint16_t><<<grid, block, gs::POOL_BYTES, c->stream>>>(a);
      }
      CUDA_TRY(cudaGetLastError(), errOut);
    } else {
      int32_t* wl = fixed_lists;
      if (!wl) {
        int rc = ensure(c->worklist, (static_cast<size_t>(B) + 1) * sizeof(int32_t), errOut);
        if (rc) return rc;
        wl = static_cast<int32_t*>(c->worklist.ptr);
      }
      CUDA_TRY(cudaMemsetAsync(wl, 0, sizeof(int32_t), c->stream), errOut);
      gs::ClusterArgs ca;
      ca.k = a;
      ca.slice_bytes = static_cast<int32_t>(need > gs::MIN_SLICE_BYTES ? need : gs::MIN_SLICE_BYTES);
      ca.eb_table = c->eb_table;
      ca.worklist = wl;
      const size_t dyn = static_cast<size_t>(ca.slice_bytes) + gs::REGION_A + gs::REGION_B;
      cudaLaunchConfig_t lc = {};
      lc.gridDim = dim3(static_cast<unsigned>(B * C));
      lc.blockDim = dim3(gs::NT);
      lc.dynamicSmemBytes = dyn;
      lc.stream = c->stream;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = static_cast<unsigned>(C);
      at[0].val.clusterDim.y = 1;
      at[0].val.clusterDim.z = 1;
      lc.attrs = at;
      lc.numAttrs = 1;
      if (dtype == GORCH_CUDA_F32) {
        CUDA_TRY(cudaLaunchKernelEx(&lc, gs::sample_cluster_kernel<float>, ca), errOut);
      } else {
        CUDA_TRY(cudaLaunchKernelEx(&lc, gs::sample_cluster_kernel<uint16_t>, ca), errOut);
      }
      // rows the cluster kernel handed over (rare): a fixed grid walks the list
      gs::KernelArgs aw = a;
      aw.worklist = ca.worklist;
      const int64_t wg = B < 2 * c->sm_count ? B : 2 * c->sm_count;
      dim3 grid(static_cast<unsigned>(wg)), block(gs::NT);
      if (dtype == GORCH_CUDA_F32) {
        gs::sample_rows_kernel<float><<<grid, block, gs::POOL_BYTES, c->stream>>>(aw);
      } else {
        gs::sample_rows_kernel<uint16_t><<<grid, block, gs::POOL_BYTES, c->stream>>>(aw);
      }
      CUDA_TRY(cudaGetLastError(), errOut);
      klaunch = 2;
    }
  }
  c->counters.kernel_launches += static_cast<uint64_t>(klaunch);
  if (force_greedy) c->counters.argmax_launches++; else c->counters.sample_launches++;
  c->counters.rows += static_cast<uint64_t>(B);
  if (c->timing) {
    CUDA_TRY(cudaEventRecord(c->ev1, c->stream), errOut);
    CUDA_TRY(cudaEventSynchronize(c->ev1), errOut);
    CUDA_TRY(cudaEventElapsedTime(&c->counters.last_kernel_ms, c->ev0, c->ev1), errOut);
  }
  return GORCH_CUDA_OK;
}

int validate_host_cfgs(const GorchSampleCfg* cfgs, int64_t B, char** errOut) {
  for (int64_t b = 0; b < B; b++) {
    float t = cfgs[b].temperature;
    if (!(t >= 0.0f) || !(t < std::numeric_limits<float>::infinity())) {
      set_err(errOut, "gorch_cuda: row %lld temperature %g is negative, NaN or infinite",
              (long long)b, (double)t);
      return GORCH_CUDA_ERR_BAD_ARG;
    }
    if (cfgs[b].topp_mode != GORCH_TOPP_MODE_A && cfgs[b].topp_mode != GORCH_TOPP_MODE_B) {
      set_err(errOut, "gorch_cuda: row %lld unknown topp_mode %d", (long long)b, cfgs[b].topp_mode);
      return GORCH_CUDA_ERR_BAD_ARG;
    }
  }
  return GORCH_CUDA_OK;
}

int host_run(Ctx* c, const void* logits, int dtype, int64_t B, int64_t V, int64_t row_stride,
             const GorchSampleCfg* cfgs, const double* uniforms, int32_t* out_ids,
             uint32_t* out_flags, int force_greedy, char** errOut) {
  int rc = check_shape(dtype, B, V, row_stride, errOut);
  if (rc) return rc;
  if (B == 0) return GORCH_CUDA_OK;
  if (!logits || !out_ids || (!force_greedy && (!cfgs || !uniforms))) {
    set_err(errOut, "gorch_cuda: null pointer argument");
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  if (!force_greedy) {
    rc = validate_host_cfgs(cfgs, B, errOut);
    if (rc) return rc;
  }
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  const size_t es = elem_size(dtype);
  const size_t lbytes = (static_cast<size_t>(B - 1) * row_stride + V) * es;
  if ((rc = ensure(c->st_logits, lbytes, errOut))) return rc;
  if ((rc = ensure(c->st_ids, B * sizeof(int32_t), errOut))) return rc;
  if ((rc = ensure(c->st_flags, B * sizeof(uint32_t), errOut))) return rc;
  CUDA_TRY(cudaMemcpyAsync(c->st_logits.ptr, logits, lbytes, cudaMemcpyHostToDevice, c->stream), errOut);
  c->counters.h2d_bytes += lbytes;
  if (!force_greedy) {
    if ((rc = ensure(c->st_cfgs, B * sizeof(GorchSampleCfg), errOut))) return rc;
    if ((rc = ensure(c->st_uniforms, B * sizeof(double), errOut))) return rc;
    CUDA_TRY(cudaMemcpyAsync(c->st_cfgs.ptr, cfgs, B * sizeof(GorchSampleCfg), cudaMemcpyHostToDevice, c->stream), errOut);
    CUDA_TRY(cudaMemcpyAsync(c->st_uniforms.ptr, uniforms, B * sizeof(double), cudaMemcpyHostToDevice, c->stream), errOut);
    c->counters.h2d_bytes += B * (sizeof(GorchSampleCfg) + sizeof(double));
  }
  rc = launch_rows(c, c->st_logits.ptr, dtype, B, V, row_stride,
                   static_cast<const GorchSampleCfg*>(c->st_cfgs.ptr),
                   static_cast<const double*>(c->st_uniforms.ptr),
                   static_cast<int32_t*>(c->st_ids.ptr), static_cast<uint32_t*>(c->st_flags.ptr),
                   nullptr, nullptr, force_greedy, errOut);
  if (rc) return rc;
  CUDA_TRY(cudaMemcpyAsync(out_ids, c->st_ids.ptr, B * sizeof(int32_t), cudaMemcpyDeviceToHost, c->stream), errOut);
  c->counters.d2h_bytes += B * sizeof(int32_t);
  if (out_flags) {
    CUDA_TRY(cudaMemcpyAsync(out_flags, c->st_flags.ptr, B * sizeof(uint32_t), cudaMemcpyDeviceToHost, c->stream), errOut);
    c->counters.d2h_bytes += B * sizeof(uint32_t);
  }
  CUDA_TRY(cudaStreamSynchronize(c->stream), errOut);
  return GORCH_CUDA_OK;
}

// ---- LM-head projection (lm_head.cuh) ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_tiled = nullptr;

int load_encode_tiled(char** errOut) {
  if (g_encode_tiled) return GORCH_CUDA_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres), errOut);
  if (!fn || qres != cudaDriverEntryPointSuccess) {
    set_err(errOut, "gorch_cuda: the driver does not offer cuTensorMapEncodeTiled");
    return GORCH_CUDA_ERR_CUDA;
  }
  g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
  return GORCH_CUDA_OK;
}

// Tensor map of a row-major [rows, K] bf16 matrix: boxes of 64 columns x 128 rows, 128-byte swizzle,
// zero fill outside the matrix.
int make_bf16_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld, char** errOut) {
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(gs::LMH_BK), static_cast<cuuint32_t>(gs::LMH_BM)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_err(errOut, "gorch_cuda: cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
    return GORCH_CUDA_ERR_CUDA;
  }
  return GORCH_CUDA_OK;
}

int check_lm_head(Ctx* c, const void* x, const void* w, int64_t B, int64_t V, int64_t K, int64_t ldx, int64_t ldw, char** errOut) {
  if (B < 0 || V < 1 || K < gs::LMH_BK || (K % gs::LMH_BK) != 0 || ldx < K || ldw < K) {
    set_err(errOut, "gorch_cuda: LM head needs B >= 0, V >= 1 and K a multiple of %d (got B=%lld V=%lld K=%lld)", gs::LMH_BK,
            (long long)B, (long long)V, (long long)K);
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  if (B > 0x7fffffffll || V > 0x7fffff00ll || K > 0x7fffffffll) { set_err(errOut, "gorch_cuda: LM head shape beyond 31 bits"); return GORCH_CUDA_ERR_LIMIT; }
  if (B == 0) return GORCH_CUDA_OK;
  if (!x || !w) { set_err(errOut, "gorch_cuda: null pointer argument"); return GORCH_CUDA_ERR_BAD_ARG; }
  if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(w) & 15u) || ((ldx * 2) & 15) || ((ldw * 2) & 15)) {
    set_err(errOut, "gorch_cuda: LM head operands must be 16-byte aligned with row pitches that are multiples of 16 bytes");
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  (void)c;
  return GORCH_CUDA_OK;
}

// One launch of lm_head_kernel over the vocabulary tiles tile0 + i * step, i < ntile.
int launch_lm_head(Ctx* c, gs::LmHeadArgs& a, char** errOut) {
  const int64_t ntile_total = (static_cast<int64_t>(a.V) + gs::LMH_BN - 1) / gs::LMH_BN;
  if (a.ntile < 1 || a.tile0 + static_cast<int64_t>(a.ntile - 1) * a.tile_step >= ntile_total) {
    set_err(errOut, "gorch_cuda: LM head tile range outside the vocabulary");
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  const unsigned grid = static_cast<unsigned>(a.ntile < c->sm_count ? a.ntile : c->sm_count);
  gs::lm_head_kernel<<<grid, gs::LMH_NT, gs::LMH_DYN_BYTES, c->stream>>>(a);
  CUDA_TRY(cudaGetLastError(), errOut);
  c->counters.kernel_launches += 1;
  return GORCH_CUDA_OK;
}

}  // namespace

extern "C" {

int gorch_cuda_device_count(int* count, char** errOut) {
  if (!count) { set_err(errOut, "gorch_cuda: null count"); return GORCH_CUDA_ERR_BAD_ARG; }
  CUDA_TRY(cudaGetDeviceCount(count), errOut);
  return GORCH_CUDA_OK;
}

GorchCudaCtxRef gorch_cuda_create_ctx(int device, char** errOut) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n <= 0) {
    set_err(errOut, "gorch_cuda: no CUDA device (%s)", cudaGetErrorString(e));
    return nullptr;
  }
  if (device < 0 || device >= n) {
    set_err(errOut, "gorch_cuda: device %d out of range [0,%d)", device, n);
    return nullptr;
  }
  Ctx* c = new (std::nothrow) Ctx();
  if (!c) { set_err(errOut, "gorch_cuda: out of host memory"); return nullptr; }
  c->device = device;
  auto fail = [&](const char* what, cudaError_t err) -> GorchCudaCtxRef {
    set_err(errOut, "gorch_cuda: %s failed: %s", what, cudaGetErrorString(err));
    gorch_cuda_release(c);
    return nullptr;
  };
  if ((e = cudaSetDevice(device)) != cudaSuccess) return fail("cudaSetDevice", e);
  cudaDeviceProp prop;
  if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) return fail("cudaGetDeviceProperties", e);
  if (prop.major < 10) {
    set_err(errOut, "gorch_cuda: device %d is sm_%d%d; this library is built for sm_100a only",
            device, prop.major, prop.minor);
    gorch_cuda_release(c);
    return nullptr;
  }
  c->sm_count = prop.multiProcessorCount;
  if (prop.l2CacheSize > 0) c->l2_bytes = prop.l2CacheSize;
  if ((e = cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking)) != cudaSuccess) return fail("cudaStreamCreate", e);
  c->stream = c->own_stream;
  if ((e = cudaStreamCreateWithFlags(&c->side_stream, cudaStreamNonBlocking)) != cudaSuccess) return fail("cudaStreamCreate", e);
  if ((e = cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming)) != cudaSuccess) return fail("cudaEventCreate", e);
  if ((e = cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming)) != cudaSuccess) return fail("cudaEventCreate", e);
  if ((e = cudaEventCreate(&c->ev0)) != cudaSuccess) return fail("cudaEventCreate", e);
  if ((e = cudaEventCreate(&c->ev1)) != cudaSuccess) return fail("cudaEventCreate", e);
  {
    // device address of the fixed work-list array of gorch_cuda_sample_dev_static on this device
    int32_t* unused = nullptr;
    char* msg = nullptr;
    if (static_lists_ptr(device, &unused, &msg) != GORCH_CUDA_OK) {
      if (errOut) *errOut = msg; else free(msg);
      gorch_cuda_release(c);
      return nullptr;
    }
  }
  double tab[256];
  for (int j = 0; j < 256; j++) tab[j] = static_cast<double>(exp2l(static_cast<long double>(j) / 256.0L));
  if ((e = cudaMalloc(&c->exp_table, sizeof tab)) != cudaSuccess) return fail("cudaMalloc(exp table)", e);
  if ((e = cudaMemcpy(c->exp_table, tab, sizeof tab, cudaMemcpyHostToDevice)) != cudaSuccess) return fail("cudaMemcpy(exp table)", e);
  static double ebt[gs::NB1];
  for (int j = 0; j < gs::NB1; j++) ebt[j] = static_cast<double>(expl(-static_cast<long double>(j) / 32.0L));
  if ((e = cudaMalloc(&c->eb_table, sizeof ebt)) != cudaSuccess) return fail("cudaMalloc(bucket table)", e);
  if ((e = cudaMemcpy(c->eb_table, ebt, sizeof ebt, cudaMemcpyHostToDevice)) != cudaSuccess) return fail("cudaMemcpy(bucket table)", e);
  if ((e = cudaFuncSetAttribute(gs::sample_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::POOL_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::sample_rows_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::POOL_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::sample_cluster_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 109 * 1024)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::sample_cluster_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, 109 * 1024)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::n256::narrow_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::n256::N_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::n256::narrow_rows_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::n256::N_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::n128::narrow_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::n128::N_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::n128::narrow_rows_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::n128::N_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::multinomial_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::MN_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::topk_large_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::TKL_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::topk_large_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::TKL_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::vocab_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::VM_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::w256::wide_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::w256::W_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::w1024::wide_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::w1024::W_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::w1024::wide_rows_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::w1024::W_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::LMH_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::lmh_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::LMH_F_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::row_softmax_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::RS_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::row_softmax_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::RS_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaFuncSetAttribute(gs::w256::wide_rows_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, gs::w256::W_DYN_BYTES)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  return c;
}

void gorch_cuda_release(GorchCudaCtxRef ctx) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) return;
  cudaSetDevice(c->device);
  if (c->own_stream) { cudaStreamSynchronize(c->own_stream); }
  for (Scratch* s : {&c->st_logits, &c->st_cfgs, &c->st_uniforms, &c->st_ids, &c->st_flags}) {
    if (s->ptr) cudaFree(s->ptr);
  }
  if (c->exp_table) cudaFree(c->exp_table);
  if (c->eb_table) cudaFree(c->eb_table);
  if (c->worklist.ptr) cudaFree(c->worklist.ptr);
  if (c->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(c->comm);
  if (c->lmh_scratch.ptr) cudaFree(c->lmh_scratch.ptr);
  if (c->lmh_logits.ptr) cudaFree(c->lmh_logits.ptr);
  if (c->vs_local.ptr) cudaFree(c->vs_local.ptr);
  if (c->vs_all.ptr) cudaFree(c->vs_all.ptr);
  if (c->vs_req.ptr) cudaFree(c->vs_req.ptr);
  if (c->vs_rows.ptr) cudaFree(c->vs_rows.ptr);
  if (c->vs_done.ptr) cudaFree(c->vs_done.ptr);
  for (cudaEvent_t e : c->ev_vs) if (e) cudaEventDestroy(e);
  if (c->ev0) cudaEventDestroy(c->ev0);
  if (c->ev1) cudaEventDestroy(c->ev1);
  if (c->own_stream) cudaStreamDestroy(c->own_stream);
  if (c->side_stream) cudaStreamDestroy(c->side_stream);
  if (c->ev_fork) cudaEventDestroy(c->ev_fork);
  if (c->ev_join) cudaEventDestroy(c->ev_join);
  delete c;
}

void gorch_cuda_free_string(char* s) { free(s); }

int gorch_cuda_sync(GorchCudaCtxRef ctx, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  CUDA_TRY(cudaStreamSynchronize(c->stream), errOut);
  return GORCH_CUDA_OK;
}

int gorch_cuda_set_stream(GorchCudaCtxRef ctx, void* stream, int external, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  c->stream = external ? static_cast<cudaStream_t>(stream) : c->own_stream;
  return GORCH_CUDA_OK;
}

int gorch_cuda_set_timing(GorchCudaCtxRef ctx, int on) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) return GORCH_CUDA_ERR_BAD_ARG;
  c->timing = on ? 1 : 0;
  return GORCH_CUDA_OK;
}

int gorch_cuda_set_kernel_variant(GorchCudaCtxRef ctx, int variant, int cluster_size, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  if ((variant < 0 || variant > 7) ||
      !(cluster_size == 0 || cluster_size == 1 || cluster_size == 2 || cluster_size == 4 || cluster_size == 8)) {
    set_err(errOut, "gorch_cuda: variant must be 0..7, cluster_size 0, 1, 2, 4 or 8");
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  c->variant = variant;
  c->force_cluster = cluster_size;
  return GORCH_CUDA_OK;
}

int gorch_cuda_get_counters(GorchCudaCtxRef ctx, GorchCudaCounters* out) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c || !out) return GORCH_CUDA_ERR_BAD_ARG;
  *out = c->counters;
  return GORCH_CUDA_OK;
}

GorchCudaBufferRef gorch_cuda_buffer_alloc(GorchCudaCtxRef ctx, uint64_t bytes, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return nullptr; }
  Buffer* b = new (std::nothrow) Buffer{c->device, nullptr, bytes};
  if (!b) { set_err(errOut, "gorch_cuda: out of host memory"); return nullptr; }
  cudaError_t e = cudaSetDevice(c->device);
  if (e == cudaSuccess) e = cudaMalloc(&b->ptr, bytes ? bytes : 1);
  if (e != cudaSuccess) {
    set_err(errOut, "gorch_cuda: cudaMalloc(%llu) failed: %s", (unsigned long long)bytes, cudaGetErrorString(e));
    delete b;
    return nullptr;
  }
  return b;
}

void gorch_cuda_buffer_free(GorchCudaBufferRef buf) {
  Buffer* b = static_cast<Buffer*>(buf);
  if (!b) return;
  cudaSetDevice(b->device);
  cudaFree(b->ptr);
  delete b;
}

uint64_t gorch_cuda_buffer_length(GorchCudaBufferRef buf) {
  Buffer* b = static_cast<Buffer*>(buf);
  return b ? b->bytes : 0;
}

void* gorch_cuda_buffer_device_ptr(GorchCudaBufferRef buf) {
  Buffer* b = static_cast<Buffer*>(buf);
  return b ? b->ptr : nullptr;
}

int gorch_cuda_buffer_upload(GorchCudaBufferRef buf, uint64_t offset, const void* host,
                             uint64_t bytes, char** errOut) {
  Buffer* b = static_cast<Buffer*>(buf);
  if (!b || (!host && bytes) || offset > b->bytes || bytes > b->bytes - offset) {
    set_err(errOut, "gorch_cuda: upload out of range");
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  CUDA_TRY(cudaSetDevice(b->device), errOut);
  CUDA_TRY(cudaMemcpy(static_cast<char*>(b->ptr) + offset, host, bytes, cudaMemcpyHostToDevice), errOut);
  return GORCH_CUDA_OK;
}

int gorch_cuda_buffer_download(GorchCudaBufferRef buf, uint64_t offset, void* host,
                               uint64_t bytes, char** errOut) {
  Buffer* b = static_cast<Buffer*>(buf);
  if (!b || (!host && bytes) || offset > b->bytes || bytes > b->bytes - offset) {
    set_err(errOut, "gorch_cuda: download out of range");
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  CUDA_TRY(cudaSetDevice(b->device), errOut);
  CUDA_TRY(cudaMemcpy(host, static_cast<char*>(b->ptr) + offset, bytes, cudaMemcpyDeviceToHost), errOut);
  return GORCH_CUDA_OK;
}

int gorch_cuda_sample_host(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                           int64_t V, int64_t row_stride, const GorchSampleCfg* cfgs,
                           const double* uniforms, int32_t* out_ids, uint32_t* out_flags,
                           char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  return host_run(c, logits, dtype, B, V, row_stride, cfgs, uniforms, out_ids, out_flags, 0, errOut);
}

int gorch_cuda_sample_dev(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                          int64_t V, int64_t row_stride, const GorchSampleCfg* cfgs,
                          const double* uniforms, int32_t* out_ids, uint32_t* out_flags,
                          double* out_probs, GorchSampleDebug* out_debug, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  int rc = check_shape(dtype, B, V, row_stride, errOut);
  if (rc) return rc;
  if (B == 0) return GORCH_CUDA_OK;
  if (!logits || !cfgs || !uniforms || !out_ids) {
    set_err(errOut, "gorch_cuda: null pointer argument");
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  return launch_rows(c, logits, dtype, B, V, row_stride, cfgs, uniforms, out_ids, out_flags,
                     out_probs, out_debug, 0, errOut);
}

static int vocab_local_launch(Ctx* c, const void* logits, int dtype, int64_t B, int64_t Vslice, int64_t row_stride,
                              int64_t col_offset, const GorchSampleCfg* cfgs, void* records, int cand, char** errOut,
                              bool sumexp_rows = true) {
  int rc = check_shape(dtype, B, Vslice, row_stride, errOut);
  if (rc) return rc;
  static_assert(sizeof(gs::VsRecord) == GORCH_VS_RECORD_BYTES, "record layout");
  if (col_offset < 0 || col_offset + Vslice > 0x7fffff00ll) {
    set_err(errOut, "gorch_cuda: column offset %lld out of range", (long long)col_offset);
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  if (cand < 1 || cand > gs::VS_CAND) {
    set_err(errOut, "gorch_cuda: %d candidates per record outside 1..%d", cand, gs::VS_CAND);
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  if (B == 0) return GORCH_CUDA_OK;
  if (!logits || !cfgs || !records) { set_err(errOut, "gorch_cuda: null pointer argument"); return GORCH_CUDA_ERR_BAD_ARG; }
  if ((reinterpret_cast<uintptr_t>(logits) % elem_size(dtype)) != 0) {
    set_err(errOut, "gorch_cuda: logits pointer not aligned to its element size");
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  // every row goes through the narrow kernel (row_kind says so when vs_records is set)
  const size_t ints = 16 + static_cast<size_t>(B) + 1;
  rc = ensure(c->worklist, ints * sizeof(int32_t), errOut);
  if (rc) return rc;
  int32_t* base = static_cast<int32_t*>(c->worklist.ptr);
  gs::BatchArgs ba;
  ba.k.logits = logits; ba.k.row_stride = row_stride; ba.k.V = static_cast<int32_t>(Vslice);
  ba.k.force_greedy = 0; ba.k.cfgs = reinterpret_cast<const gs::RowCfg*>(cfgs); ba.k.uniforms = nullptr;
  ba.k.out_ids = nullptr; ba.k.out_flags = nullptr; ba.k.out_probs = nullptr; ba.k.out_debug = nullptr;
  ba.k.exp_table = c->exp_table; ba.k.row_offset = 0; ba.k.worklist = nullptr;
  ba.k.vs_records = records; ba.k.vs_col_offset = static_cast<int32_t>(col_offset); ba.k.vs_cand = cand;
  ba.k.vs_sumexp = sumexp_rows ? 1 : 0;
  ba.k.tk_values = nullptr; ba.k.tk_indices = nullptr; ba.k.tk_k = 0; ba.k.row_done = nullptr;
  ba.eb_table = c->eb_table;
  ba.hdr = base; ba.list_single = base + 15;
  ba.B = B;
  CUDA_TRY(cudaMemsetAsync(base, 0, 16 * sizeof(int32_t), c->stream), errOut);
  CUDA_TRY(launch_narrow(c, ba, dtype, B), errOut);
  c->counters.kernel_launches += 1;
  if (sumexp_rows) {                                         // the records of rows without top-k: disjoint rows, same stream
    const unsigned g = static_cast<unsigned>(B < 4 * c->sm_count ? B : 4 * c->sm_count);
    if (dtype == GORCH_CUDA_F32) gs::vocab_sumexp_kernel<float><<<g, gs::VD_NT, 0, c->stream>>>(ba.k, c->eb_table, B);
    else gs::vocab_sumexp_kernel<uint16_t><<<g, gs::VD_NT, 0, c->stream>>>(ba.k, c->eb_table, B);
    c->counters.kernel_launches += 1;
  }
  CUDA_TRY(cudaGetLastError(), errOut);
  return GORCH_CUDA_OK;
}

static int vocab_merge_launch(Ctx* c, const void* all_records, int nranks, int cand, int64_t B, int64_t V,
                              const GorchSampleCfg* cfgs, const double* uniforms, int32_t* out_ids,
                              uint32_t* out_flags, char** errOut, int my_rank = -1, double* draw_req = nullptr) {
  if (nranks < 1 || nranks > gs::VM_MAX_RANKS) {
    set_err(errOut, "gorch_cuda: vocab merge takes 1..%d ranks, got %d", gs::VM_MAX_RANKS, nranks);
    return GORCH_CUDA_ERR_LIMIT;
  }
  int rc = check_shape(GORCH_CUDA_F32, B, V, V, errOut);
  if (rc) return rc;
  if (B == 0) return GORCH_CUDA_OK;
  if (!all_records || !cfgs || !uniforms || !out_ids) { set_err(errOut, "gorch_cuda: null pointer argument"); return GORCH_CUDA_ERR_BAD_ARG; }
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  gs::MergeArgs m;
  m.k.logits = nullptr; m.k.row_stride = V; m.k.V = static_cast<int32_t>(V); m.k.force_greedy = 0;
  m.k.cfgs = reinterpret_cast<const gs::RowCfg*>(cfgs); m.k.uniforms = uniforms;
  m.k.out_ids = out_ids; m.k.out_flags = out_flags; m.k.out_probs = nullptr; m.k.out_debug = nullptr;
  m.k.exp_table = c->exp_table; m.k.row_offset = 0; m.k.worklist = nullptr; m.k.vs_records = nullptr; m.k.vs_col_offset = 0;
  m.k.vs_cand = cand;
  m.k.vs_sumexp = 0;
  m.k.tk_values = nullptr; m.k.tk_indices = nullptr; m.k.tk_k = 0; m.k.row_done = nullptr;
  m.records = all_records;
  m.nranks = nranks;
  m.cand = cand;
  m.B = B;
  m.my_rank = my_rank;
  m.draw_req = draw_req;
  const unsigned g = static_cast<unsigned>(B < 8 * c->sm_count ? B : 8 * c->sm_count);
  gs::vocab_merge_kernel<<<g, gs::VM_NT, gs::vm_dyn_bytes(nranks, cand), c->stream>>>(m);
  CUDA_TRY(cudaGetLastError(), errOut);
  c->counters.kernel_launches += 1;
  c->counters.sample_launches += 1;
  c->counters.rows += B;
  return GORCH_CUDA_OK;
}

int gorch_cuda_vocab_local_dev(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                               int64_t Vslice, int64_t row_stride, int64_t col_offset,
                               const GorchSampleCfg* cfgs, void* records, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  return vocab_local_launch(c, logits, dtype, B, Vslice, row_stride, col_offset, cfgs, records, gs::VS_CAND, errOut);
}

int gorch_cuda_vocab_merge_dev(GorchCudaCtxRef ctx, const void* all_records, int nranks, int64_t B,
                               int64_t V, const GorchSampleCfg* cfgs, const double* uniforms,
                               int32_t* out_ids, uint32_t* out_flags, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  return vocab_merge_launch(c, all_records, nranks, gs::VS_CAND, B, V, cfgs, uniforms, out_ids, out_flags, errOut);
}

int gorch_cuda_vocab_merge_owner_dev(GorchCudaCtxRef ctx, const void* all_records, int nranks, int my_rank, int64_t B,
                                     int64_t V, const GorchSampleCfg* cfgs, const double* uniforms,
                                     int32_t* out_ids, uint32_t* out_flags, double* draw_req, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  if (my_rank < 0 || my_rank >= nranks || !draw_req) { set_err(errOut, "gorch_cuda: bad rank or null draw request buffer"); return GORCH_CUDA_ERR_BAD_ARG; }
  return vocab_merge_launch(c, all_records, nranks, gs::VS_CAND, B, V, cfgs, uniforms, out_ids, out_flags, errOut, my_rank, draw_req);
}

static int vocab_draw_launch(Ctx* c, const void* logits_slice, int dtype, int64_t B, int64_t Vslice, int64_t row_stride,
                             int64_t col_offset, const GorchSampleCfg* cfgs, const double* draw_req, int32_t* out_ids,
                             uint32_t* out_flags, char** errOut) {
  int rc = check_shape(dtype, B, Vslice, row_stride, errOut);
  if (rc) return rc;
  if (B == 0) return GORCH_CUDA_OK;
  if (!logits_slice || !cfgs || !draw_req || !out_ids) { set_err(errOut, "gorch_cuda: null pointer argument"); return GORCH_CUDA_ERR_BAD_ARG; }
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  gs::DrawArgs d;
  d.logits = logits_slice; d.row_stride = row_stride; d.V = static_cast<int32_t>(Vslice);
  d.col_offset = static_cast<int32_t>(col_offset);
  d.cfgs = reinterpret_cast<const gs::RowCfg*>(cfgs); d.draw_req = draw_req;
  d.eb_table = c->eb_table; d.exp_table = c->exp_table;
  d.out_ids = out_ids; d.out_flags = out_flags; d.B = B;
  const unsigned g = static_cast<unsigned>(B < 4 * c->sm_count ? B : 4 * c->sm_count);
  if (dtype == GORCH_CUDA_F32) gs::vocab_draw_kernel<float><<<g, gs::VD_NT, 0, c->stream>>>(d);
  else gs::vocab_draw_kernel<uint16_t><<<g, gs::VD_NT, 0, c->stream>>>(d);
  CUDA_TRY(cudaGetLastError(), errOut);
  c->counters.kernel_launches += 1;
  return GORCH_CUDA_OK;
}

int gorch_cuda_vocab_draw_dev(GorchCudaCtxRef ctx, const void* logits_slice, int dtype, int64_t B, int64_t Vslice,
                              int64_t row_stride, int64_t col_offset, const GorchSampleCfg* cfgs,
                              const double* draw_req, int32_t* out_ids, uint32_t* out_flags, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  return vocab_draw_launch(c, logits_slice, dtype, B, Vslice, row_stride, col_offset, cfgs, draw_req, out_ids, out_flags, errOut);
}

int gorch_cuda_comm_unique_id(void* id_bytes, char** errOut) {
  static_assert(sizeof(ncclUniqueId) == GORCH_CUDA_UNIQUE_ID_BYTES, "unique id size");
  if (!id_bytes) { set_err(errOut, "gorch_cuda: null unique-id buffer"); return GORCH_CUDA_ERR_BAD_ARG; }
  int rc = load_nccl(errOut);
  if (rc) return rc;
  ncclUniqueId id;
  NCCL_TRY(g_nccl.GetUniqueId(&id), errOut);
  memcpy(id_bytes, &id, sizeof id);
  return GORCH_CUDA_OK;
}

int gorch_cuda_comm_init(GorchCudaCtxRef ctx, int rank, int nranks, const void* unique_id_bytes, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  if (!unique_id_bytes || nranks < 1 || nranks > gs::VM_MAX_RANKS || rank < 0 || rank >= nranks) {
    set_err(errOut, "gorch_cuda: comm_init needs a unique id and 0 <= rank < nranks <= %d (got rank %d of %d)",
            gs::VM_MAX_RANKS, rank, nranks);
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  if (c->comm) { set_err(errOut, "gorch_cuda: the context already has a communicator"); return GORCH_CUDA_ERR_BAD_ARG; }
  int rc = load_nccl(errOut);
  if (rc) return rc;
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  ncclUniqueId id;
  memcpy(&id, unique_id_bytes, sizeof id);
  ncclComm_t comm = nullptr;
  NCCL_TRY(g_nccl.CommInitRank(&comm, nranks, id, rank), errOut);
  for (int i = 0; i < 4; i++) {
    if (!c->ev_vs[i]) CUDA_TRY(cudaEventCreate(&c->ev_vs[i]), errOut);
  }
  c->comm = comm;
  c->comm_rank = rank;
  c->comm_nranks = nranks;
  return GORCH_CUDA_OK;
}

int gorch_cuda_comm_release(GorchCudaCtxRef ctx, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  if (!c->comm) return GORCH_CUDA_OK;
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  CUDA_TRY(cudaStreamSynchronize(c->stream), errOut);
  ncclComm_t comm = c->comm;
  c->comm = nullptr;
  c->comm_nranks = 0;
  NCCL_TRY(g_nccl.CommDestroy(comm), errOut);
  return GORCH_CUDA_OK;
}

static int sample_vocab_sharded(GorchCudaCtxRef ctx, const void* logits_slice, int dtype, int64_t B,
                                int64_t Vslice, int64_t row_stride, int64_t col_offset, int64_t V,
                                int max_top_k, int rows_without_top_k, const GorchSampleCfg* cfgs, const double* uniforms,
                                int32_t* out_ids, uint32_t* out_flags, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  if (!c->comm) { set_err(errOut, "gorch_cuda: no communicator: call gorch_cuda_comm_init first"); return GORCH_CUDA_ERR_NCCL; }
  if (V < 1 || col_offset < 0 || col_offset + Vslice > V) {
    set_err(errOut, "gorch_cuda: slice [%lld, %lld) outside the vocabulary of %lld", (long long)col_offset,
            (long long)(col_offset + Vslice), (long long)V);
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  // candidates per record: the largest top_k of the batch plus room for ties at the local threshold,
  // in steps of eight (0: the full record)
  int cand = gs::VS_CAND;
  if (max_top_k > 0 && max_top_k <= gs::VS_CAND) cand = ((max_top_k + max_top_k / 4 + 8 + 7) / 8) * 8;
  if (cand > gs::VS_CAND) cand = gs::VS_CAND;
  if (B == 0) return GORCH_CUDA_OK;
  const size_t rec_bytes = 16 + 8 * static_cast<size_t>(cand);
  int rc = ensure(c->vs_local, static_cast<size_t>(B) * rec_bytes, errOut);
  if (rc) return rc;
  rc = ensure(c->vs_all, static_cast<size_t>(B) * rec_bytes * static_cast<size_t>(c->comm_nranks), errOut);
  if (rc) return rc;
  if (c->timing) CUDA_TRY(cudaEventRecord(c->ev_vs[0], c->stream), errOut);
  rc = vocab_local_launch(c, logits_slice, dtype, B, Vslice, row_stride, col_offset, cfgs, c->vs_local.ptr, cand, errOut,
                          (rows_without_top_k & 1) != 0);
  if (rc) return rc;
  if (c->timing) CUDA_TRY(cudaEventRecord(c->ev_vs[1], c->stream), errOut);
  // ONE collective: every rank's records to every rank, in rank order, on the context's stream
  NCCL_TRY(g_nccl.AllGather(c->vs_local.ptr, c->vs_all.ptr, static_cast<size_t>(B) * rec_bytes, ncclUint8, c->comm, c->stream), errOut);
  if (c->timing) CUDA_TRY(cudaEventRecord(c->ev_vs[2], c->stream), errOut);
  if (rows_without_top_k & 1) {
    // Rows without top-k: the merge names each such row's owner (the rank in whose slice u * S
    // falls), the owner finds the token in its slice, and an all-reduce (max) of ids and flags
    // hands it to every rank (the others wrote -1 and 0; rows with a top-k agree on every rank).
    if (!out_flags) { set_err(errOut, "gorch_cuda: rows without top-k need out_flags"); return GORCH_CUDA_ERR_BAD_ARG; }
    rc = ensure(c->vs_req, static_cast<size_t>(B) * 3 * sizeof(double), errOut);
    if (rc) return rc;
    double* req = static_cast<double*>(c->vs_req.ptr);
    rc = vocab_merge_launch(c, c->vs_all.ptr, c->comm_nranks, cand, B, V, cfgs, uniforms, out_ids, out_flags, errOut, c->comm_rank, req);
    if (rc) return rc;
    rc = vocab_draw_launch(c, logits_slice, dtype, B, Vslice, row_stride, col_offset, cfgs, req, out_ids, out_flags, errOut);
    if (rc) return rc;
    NCCL_TRY(g_nccl.AllReduce(out_ids, out_ids, static_cast<size_t>(B), ncclInt32, ncclMax, c->comm, c->stream), errOut);
    NCCL_TRY(g_nccl.AllReduce(out_flags, out_flags, static_cast<size_t>(B), ncclUint32, ncclMax, c->comm, c->stream), errOut);
  } else {
    rc = vocab_merge_launch(c, c->vs_all.ptr, c->comm_nranks, cand, B, V, cfgs, uniforms, out_ids, out_flags, errOut);
    if (rc) return rc;
  }
  if (rows_without_top_k & 2) {
    // Rows without top-k that the records cannot serve (a top-p cut over the whole vocabulary; with
    // bit 0 clear every row without top-k): the rows themselves are brought together — every rank
    // puts its slice into a zeroed [B, V] buffer and an all-reduce (sum) fills in the others' (x + 0
    // is x in any order; a -0 may come out as +0, which no comparison or exponential tells apart) —
    // and the ordinary kernels sample those rows on every rank, all others masked out. Correct, not
    // fast: V * B elements cross the links twice.
    if (!out_flags) { set_err(errOut, "gorch_cuda: gathered rows need out_flags"); return GORCH_CUDA_ERR_BAD_ARG; }
    const size_t es = elem_size(dtype);
    const int64_t ldv = (V + 15) & ~15ll;
    rc = ensure(c->vs_rows, static_cast<size_t>(B) * ldv * es, errOut);
    if (rc) return rc;
    rc = ensure(c->vs_done, static_cast<size_t>(B) * sizeof(int32_t), errOut);
    if (rc) return rc;
    CUDA_TRY(cudaMemsetAsync(c->vs_rows.ptr, 0, static_cast<size_t>(B) * ldv * es, c->stream), errOut);
    CUDA_TRY(cudaMemcpy2DAsync(static_cast<unsigned char*>(c->vs_rows.ptr) + static_cast<size_t>(col_offset) * es, ldv * es,
                               logits_slice, static_cast<size_t>(row_stride) * es, static_cast<size_t>(Vslice) * es,
                               static_cast<size_t>(B), cudaMemcpyDeviceToDevice, c->stream), errOut);
    const ncclDataType_t nt = dtype == GORCH_CUDA_F32 ? ncclFloat32 : static_cast<ncclDataType_t>(9);   // 9: ncclBfloat16
    NCCL_TRY(g_nccl.AllReduce(c->vs_rows.ptr, c->vs_rows.ptr, static_cast<size_t>(B) * ldv, nt, ncclSum, c->comm, c->stream), errOut);
    const unsigned gm = static_cast<unsigned>((B + 255) / 256);
    gs::vocab_gather_mask_kernel<<<gm, 256, 0, c->stream>>>(reinterpret_cast<const gs::RowCfg*>(cfgs), static_cast<int32_t>(V), B,
                                                            (rows_without_top_k & 1) != 0, static_cast<int32_t*>(c->vs_done.ptr));
    CUDA_TRY(cudaGetLastError(), errOut);
    c->counters.kernel_launches += 1;
    rc = launch_rows(c, c->vs_rows.ptr, dtype, B, V, ldv, cfgs, uniforms, out_ids, out_flags, nullptr, nullptr, 0, errOut, nullptr,
                     static_cast<const int32_t*>(c->vs_done.ptr));
    if (rc) return rc;
  }
  if (c->timing) {
    CUDA_TRY(cudaEventRecord(c->ev_vs[3], c->stream), errOut);
    CUDA_TRY(cudaEventSynchronize(c->ev_vs[3]), errOut);
    CUDA_TRY(cudaEventElapsedTime(&c->counters.vs_local_ms, c->ev_vs[0], c->ev_vs[1]), errOut);
    CUDA_TRY(cudaEventElapsedTime(&c->counters.vs_gather_ms, c->ev_vs[1], c->ev_vs[2]), errOut);
    CUDA_TRY(cudaEventElapsedTime(&c->counters.vs_merge_ms, c->ev_vs[2], c->ev_vs[3]), errOut);
    CUDA_TRY(cudaEventElapsedTime(&c->counters.last_kernel_ms, c->ev_vs[0], c->ev_vs[3]), errOut);
  }
  return GORCH_CUDA_OK;
}

int gorch_cuda_sample_vocab_sharded_dev(GorchCudaCtxRef ctx, const void* logits_slice, int dtype, int64_t B,
                                        int64_t Vslice, int64_t row_stride, int64_t col_offset, int64_t V,
                                        int max_top_k, const GorchSampleCfg* cfgs, const double* uniforms,
                                        int32_t* out_ids, uint32_t* out_flags, char** errOut) {
  return sample_vocab_sharded(ctx, logits_slice, dtype, B, Vslice, row_stride, col_offset, V, max_top_k, 0, cfgs, uniforms,
                              out_ids, out_flags, errOut);
}

int gorch_cuda_sample_vocab_sharded_ex_dev(GorchCudaCtxRef ctx, const void* logits_slice, int dtype, int64_t B,
                                           int64_t Vslice, int64_t row_stride, int64_t col_offset, int64_t V,
                                           int max_top_k, int rows_without_top_k, const GorchSampleCfg* cfgs,
                                           const double* uniforms, int32_t* out_ids, uint32_t* out_flags, char** errOut) {
  return sample_vocab_sharded(ctx, logits_slice, dtype, B, Vslice, row_stride, col_offset, V, max_top_k, rows_without_top_k,
                              cfgs, uniforms, out_ids, out_flags, errOut);
}

int gorch_cuda_topk_dev(GorchCudaCtxRef ctx, const void* x, int dtype, int64_t B, int64_t V,
                        int64_t row_stride, int64_t k, float* out_values, int32_t* out_indices,
                        uint32_t* out_flags, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  int rc = check_shape(dtype, B, V, row_stride, errOut);
  if (rc) return rc;
  if (k < 1 || k > V) {                                    // the reference panics here (index_ops.go:160-162)
    set_err(errOut, "gorch_cuda: TopK k=%lld out of range [1, %lld]", (long long)k, (long long)V);
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  if (k > gs::TKL_MAX_K) {
    set_err(errOut, "gorch_cuda: TopK supports k <= %d, got %lld", gs::TKL_MAX_K, (long long)k);
    return GORCH_CUDA_ERR_LIMIT;
  }
  if (B == 0) return GORCH_CUDA_OK;
  if (!x || !out_values || !out_indices) { set_err(errOut, "gorch_cuda: null pointer argument"); return GORCH_CUDA_ERR_BAD_ARG; }
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  if (k > gs::KFAST) {                                       // beyond the one-pass kernel's lists: select, gather, sort
    gs::TopKLargeArgs ta;
    ta.x = x; ta.row_stride = row_stride; ta.V = static_cast<int32_t>(V); ta.k = static_cast<int32_t>(k);
    ta.out_values = out_values; ta.out_indices = out_indices; ta.out_flags = out_flags; ta.B = B;
    const unsigned g = static_cast<unsigned>(B < c->sm_count ? B : c->sm_count);
    if (dtype == GORCH_CUDA_F32) gs::topk_large_kernel<float><<<g, gs::TKL_NT, gs::TKL_DYN_BYTES, c->stream>>>(ta);
    else gs::topk_large_kernel<uint16_t><<<g, gs::TKL_NT, gs::TKL_DYN_BYTES, c->stream>>>(ta);
    CUDA_TRY(cudaGetLastError(), errOut);
    c->counters.kernel_launches += 1;
    return GORCH_CUDA_OK;
  }
  const size_t ints = 16 + static_cast<size_t>(B) + 1;
  rc = ensure(c->worklist, ints * sizeof(int32_t), errOut);
  if (rc) return rc;
  int32_t* base = static_cast<int32_t*>(c->worklist.ptr);
  gs::BatchArgs ba;
  ba.k.logits = x; ba.k.row_stride = row_stride; ba.k.V = static_cast<int32_t>(V);
  ba.k.force_greedy = 0; ba.k.cfgs = nullptr; ba.k.uniforms = nullptr;
  ba.k.out_ids = nullptr; ba.k.out_flags = out_flags; ba.k.out_probs = nullptr; ba.k.out_debug = nullptr;
  ba.k.exp_table = c->exp_table; ba.k.row_offset = 0; ba.k.worklist = nullptr;
  ba.k.vs_records = nullptr; ba.k.vs_col_offset = 0; ba.k.vs_sumexp = 0;
  ba.k.tk_values = out_values; ba.k.tk_indices = out_indices; ba.k.tk_k = static_cast<int32_t>(k); ba.k.row_done = nullptr;
  ba.eb_table = c->eb_table;
  ba.hdr = base; ba.list_single = base + 15;
  ba.B = B;
  CUDA_TRY(cudaMemsetAsync(base, 0, 16 * sizeof(int32_t), c->stream), errOut);
  CUDA_TRY(launch_narrow(c, ba, dtype, B), errOut);
  CUDA_TRY(cudaGetLastError(), errOut);
  c->counters.kernel_launches += 1;
  return GORCH_CUDA_OK;
}

int gorch_cuda_multinomial_dev(GorchCudaCtxRef ctx, const float* probs, int64_t B, int64_t V,
                               int64_t row_stride, const double* uniforms, int32_t* out_ids,
                               uint32_t* out_flags, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  int rc = check_shape(GORCH_CUDA_F32, B, V, row_stride, errOut);
  if (rc) return rc;
  if (V > 8ll * gs::MN_MAX_STEPS * 256 - 64) {
    set_err(errOut, "gorch_cuda: Multinomial supports rows up to %d probabilities", 8 * gs::MN_MAX_STEPS * 256 - 64);
    return GORCH_CUDA_ERR_LIMIT;
  }
  if (B == 0) return GORCH_CUDA_OK;
  if (!probs || !uniforms || !out_ids) { set_err(errOut, "gorch_cuda: null pointer argument"); return GORCH_CUDA_ERR_BAD_ARG; }
  if ((reinterpret_cast<uintptr_t>(probs) % 4) != 0) { set_err(errOut, "gorch_cuda: probs pointer not aligned"); return GORCH_CUDA_ERR_BAD_ARG; }
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  gs::MultinomialArgs m;
  m.probs = probs; m.row_stride = row_stride; m.V = static_cast<int32_t>(V);
  m.uniforms = uniforms; m.out_ids = out_ids; m.out_flags = out_flags; m.B = B;
  const unsigned g = static_cast<unsigned>(B < 4 * c->sm_count ? B : 4 * c->sm_count);
  gs::multinomial_rows_kernel<<<g, gs::MN_NT, gs::MN_DYN_BYTES, c->stream>>>(m);
  CUDA_TRY(cudaGetLastError(), errOut);
  c->counters.kernel_launches += 1;
  return GORCH_CUDA_OK;
}

static int launch_generate_control(Ctx* c, const int32_t* ids, const uint32_t* flags,
                                   const GorchGenControl* gc, int64_t B, char** errOut) {
  static_assert(GORCH_GEN_MAX_STOPS == gs::GC_MAX_STOPS && GORCH_GEN_STOP == gs::GC_STOP &&
                GORCH_GEN_MAX_NEW == gs::GC_MAX_NEW && GORCH_GEN_MAX_SEQ == gs::GC_MAX_SEQ &&
                GORCH_GEN_ERROR == gs::GC_ERROR, "generate-control codes");
  if (!gc) { set_err(errOut, "gorch_cuda: null generate-control record"); return GORCH_CUDA_ERR_BAD_ARG; }
  if (B < 0 || B > 0x7fffffffll) { set_err(errOut, "gorch_cuda: bad batch size %lld", (long long)B); return GORCH_CUDA_ERR_BAD_ARG; }
  if (gc->n_stop < 0 || gc->n_stop > GORCH_GEN_MAX_STOPS) {
    set_err(errOut, "gorch_cuda: n_stop %d outside 0..%d", gc->n_stop, GORCH_GEN_MAX_STOPS);
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  if (gc->capacity < 0 || gc->max_seq < 0) { set_err(errOut, "gorch_cuda: negative capacity or max_seq"); return GORCH_CUDA_ERR_BAD_ARG; }
  if (B == 0) return GORCH_CUDA_OK;
  if (!ids || !gc->tokens || !gc->lengths || !gc->n_new || !gc->done || !gc->next_input || !gc->live_count ||
      (gc->cached && !gc->cache_len)) {
    set_err(errOut, "gorch_cuda: null pointer in the generate-control record");
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  gs::GenControlArgs a;
  a.ids = ids; a.flags = flags;
  a.tokens = gc->tokens; a.capacity = gc->capacity; a.lengths = gc->lengths; a.n_new = gc->n_new;
  a.cache_len = gc->cache_len; a.done = gc->done; a.next_input = gc->next_input;
  a.window_start = gc->window_start; a.live_count = gc->live_count;
  for (int i = 0; i < GORCH_GEN_MAX_STOPS; i++) a.stops[i] = (i < gc->n_stop && gc->stop_tokens[i] >= 0) ? gc->stop_tokens[i] : -1;
  a.n_stop = gc->n_stop; a.max_new = gc->max_new; a.max_seq = gc->max_seq; a.cached = gc->cached ? 1 : 0;
  a.bad_flags = GORCH_FLAG_INTERNAL | GORCH_FLAG_BAD_CFG;
  a.B = static_cast<int>(B);
  gs::generate_control_kernel<<<1, gs::GC_NT, 0, c->stream>>>(a);
  CUDA_TRY(cudaGetLastError(), errOut);
  c->counters.kernel_launches += 1;
  return GORCH_CUDA_OK;
}

int gorch_cuda_generate_control_dev(GorchCudaCtxRef ctx, const int32_t* ids, const uint32_t* flags,
                                    const GorchGenControl* gc, int64_t B, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  return launch_generate_control(c, ids, flags, gc, B, errOut);
}

int gorch_cuda_generate_step_dev(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                                 int64_t V, int64_t row_stride, const GorchSampleCfg* cfgs,
                                 const double* uniforms, int32_t* out_ids, uint32_t* out_flags,
                                 const GorchGenControl* gc, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  if (!gc) { set_err(errOut, "gorch_cuda: null generate-control record"); return GORCH_CUDA_ERR_BAD_ARG; }
  int rc = check_shape(dtype, B, V, row_stride, errOut);
  if (rc) return rc;
  if (B > 0) {
    if (!logits || !cfgs || !uniforms || !out_ids || !gc->done) {
      set_err(errOut, "gorch_cuda: null pointer argument");
      return GORCH_CUDA_ERR_BAD_ARG;
    }
    CUDA_TRY(cudaSetDevice(c->device), errOut);
    // rows whose sequence has ended are skipped by the sampling kernels (the reference leaves its loop,
    // model/generate.go:82-84); their out_ids / out_flags entries keep what they held
    rc = launch_rows(c, logits, dtype, B, V, row_stride, cfgs, uniforms, out_ids, out_flags, nullptr, nullptr, 0, errOut,
                     nullptr, gc->done);
    if (rc) return rc;
  }
  return launch_generate_control(c, out_ids, out_flags, gc, B, errOut);
}

static int launch_row_softmax(Ctx* c, int dtype, const gs::RowSoftmaxArgs& a, char** errOut) {
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  // A pair of CTAs per row where it was measured to pay: the two-pass ops when one row per SM in
  // flight would not fit in half of L2 (each pass-2 read then came from HBM again), and the
  // cross-entropy backward (no exchange, only finer work units) for rows of 256 KB and more. The
  // cross-entropy forward is one pass: the pair's barrier per row only costs there.
  const int64_t row_bytes = static_cast<int64_t>(a.V) * static_cast<int64_t>(elem_size(dtype));
  bool pair = false;
  if (a.mode == gs::RS_SOFTMAX || a.mode == gs::RS_LOG_SOFTMAX) pair = row_bytes * c->sm_count > (static_cast<int64_t>(c->l2_bytes) / 2);
  else if (a.mode == gs::RS_CE_BWD) pair = row_bytes >= 262144;
  const int C = (pair && c->sm_count >= 2) ? 2 : 1;
  const int64_t clusters = a.B < c->sm_count / C ? a.B : c->sm_count / C;
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(static_cast<unsigned>(clusters * C));
  lc.blockDim = dim3(gs::RS_NT);
  lc.dynamicSmemBytes = gs::RS_DYN_BYTES;
  lc.stream = c->stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = static_cast<unsigned>(C);
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  if (dtype == GORCH_CUDA_F32) { CUDA_TRY(cudaLaunchKernelEx(&lc, gs::row_softmax_kernel<float>, a), errOut); }
  else { CUDA_TRY(cudaLaunchKernelEx(&lc, gs::row_softmax_kernel<uint16_t>, a), errOut); }
  CUDA_TRY(cudaGetLastError(), errOut);
  c->counters.kernel_launches += 1;
  return GORCH_CUDA_OK;
}

int gorch_cuda_softmax_dev(GorchCudaCtxRef ctx, const void* x, int dtype, int64_t B, int64_t V,
                           int64_t row_stride, void* out, int64_t out_stride, int log_softmax,
                           char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  int rc = check_shape(dtype, B, V, row_stride, errOut);
  if (rc) return rc;
  if (out_stride < V) { set_err(errOut, "gorch_cuda: out_stride %lld below V", (long long)out_stride); return GORCH_CUDA_ERR_BAD_ARG; }
  if (B == 0) return GORCH_CUDA_OK;
  if (!x || !out) { set_err(errOut, "gorch_cuda: null pointer argument"); return GORCH_CUDA_ERR_BAD_ARG; }
  const size_t es = elem_size(dtype);
  if ((reinterpret_cast<uintptr_t>(x) % es) != 0 || (reinterpret_cast<uintptr_t>(out) % es) != 0) {
    set_err(errOut, "gorch_cuda: pointer not aligned to its element type");
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  gs::RowSoftmaxArgs a{};
  a.x = x; a.row_stride = row_stride; a.V = static_cast<int32_t>(V); a.B = B;
  a.mode = log_softmax ? gs::RS_LOG_SOFTMAX : gs::RS_SOFTMAX;
  a.out = out; a.out_stride = out_stride;
  return launch_row_softmax(c, dtype, a, errOut);
}

int gorch_cuda_cross_entropy_fwd_dev(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                                     int64_t V, int64_t row_stride, const int32_t* targets,
                                     float* row_loss, float* row_lse, float* mean_loss,
                                     char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  int rc = check_shape(dtype, B, V, row_stride, errOut);
  if (rc) return rc;
  if (B == 0) return GORCH_CUDA_OK;
  if (!logits || !targets || !row_loss || !row_lse) { set_err(errOut, "gorch_cuda: null pointer argument"); return GORCH_CUDA_ERR_BAD_ARG; }
  if ((reinterpret_cast<uintptr_t>(logits) % elem_size(dtype)) != 0) {
    set_err(errOut, "gorch_cuda: pointer not aligned to its element type");
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  gs::RowSoftmaxArgs a{};
  a.x = logits; a.row_stride = row_stride; a.V = static_cast<int32_t>(V); a.B = B;
  a.mode = gs::RS_CE_FWD; a.targets = targets; a.row_loss = row_loss; a.row_lse = row_lse;
  rc = launch_row_softmax(c, dtype, a, errOut);
  if (rc) return rc;
  if (mean_loss) {
    gs::mean_loss_kernel<<<1, 256, 0, c->stream>>>(row_loss, B, mean_loss);
    CUDA_TRY(cudaGetLastError(), errOut);
    c->counters.kernel_launches += 1;
  }
  return GORCH_CUDA_OK;
}

int gorch_cuda_cross_entropy_bwd_dev(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                                     int64_t V, int64_t row_stride, const int32_t* targets,
                                     const float* row_lse, float scale, float* dx,
                                     int64_t dx_stride, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  int rc = check_shape(dtype, B, V, row_stride, errOut);
  if (rc) return rc;
  if (dx_stride < V) { set_err(errOut, "gorch_cuda: dx_stride %lld below V", (long long)dx_stride); return GORCH_CUDA_ERR_BAD_ARG; }
  if (B == 0) return GORCH_CUDA_OK;
  if (!logits || !targets || !row_lse || !dx) { set_err(errOut, "gorch_cuda: null pointer argument"); return GORCH_CUDA_ERR_BAD_ARG; }
  if ((reinterpret_cast<uintptr_t>(logits) % elem_size(dtype)) != 0 || (reinterpret_cast<uintptr_t>(dx) % 4) != 0) {
    set_err(errOut, "gorch_cuda: pointer not aligned to its element type");
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  gs::RowSoftmaxArgs a{};
  a.x = logits; a.row_stride = row_stride; a.V = static_cast<int32_t>(V); a.B = B;
  a.mode = gs::RS_CE_BWD; a.targets = targets; a.row_lse = const_cast<float*>(row_lse);
  a.scale = scale; a.out = dx; a.out_stride = dx_stride;
  return launch_row_softmax(c, dtype, a, errOut);
}

int64_t gorch_cuda_sample_row(GorchCudaCtxRef ctx, const float* logits, int64_t n,
                              float temperature, int64_t top_k, float top_p, int topp_mode,
                              double uniform, uint32_t* out_flag, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return -1; }
  GorchSampleCfg cfg;
  cfg.temperature = temperature;
  // the reference takes a Go int; anything outside (0, n) disables top-k (generate.go:157)
  cfg.top_k = (top_k > 0 && top_k < n) ? static_cast<int32_t>(top_k) : 0;
  cfg.top_p = top_p;
  cfg.topp_mode = topp_mode;
  int32_t id = -1;
  uint32_t flag = 0;
  int rc = host_run(c, logits, GORCH_CUDA_F32, 1, n, n, &cfg, &uniform, &id, &flag, 0, errOut);
  if (rc) return -1;
  if (out_flag) *out_flag = flag;
  return id;
}

int gorch_cuda_argmax_host(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                           int64_t V, int64_t row_stride, int32_t* out_ids, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  return host_run(c, logits, dtype, B, V, row_stride, nullptr, nullptr, out_ids, nullptr, 1, errOut);
}

int gorch_cuda_argmax_dev(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                          int64_t V, int64_t row_stride, int32_t* out_ids, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  int rc = check_shape(dtype, B, V, row_stride, errOut);
  if (rc) return rc;
  if (B == 0) return GORCH_CUDA_OK;
  if (!logits || !out_ids) { set_err(errOut, "gorch_cuda: null pointer argument"); return GORCH_CUDA_ERR_BAD_ARG; }
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  return launch_rows(c, logits, dtype, B, V, row_stride, nullptr, nullptr, out_ids, nullptr,
                     nullptr, nullptr, 1, errOut);
}

int gorch_cuda_lm_head_logits_dev(GorchCudaCtxRef ctx, const void* x, int64_t ldx, const void* w, int64_t ldw, int64_t B,
                                  int64_t V, int64_t K, float* out_logits, int64_t ld_out, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  int rc = check_lm_head(c, x, w, B, V, K, ldx, ldw, errOut);
  if (rc) return rc;
  if (B == 0) return GORCH_CUDA_OK;
  if (!out_logits || ld_out < V) { set_err(errOut, "gorch_cuda: LM head output missing or its pitch below V"); return GORCH_CUDA_ERR_BAD_ARG; }
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  if ((rc = load_encode_tiled(errOut))) return rc;
  if ((rc = ensure(c->lmh_scratch, 256, errOut))) return rc;
  gs::LmHeadArgs a;
  memset(&a, 0, sizeof a);
  if ((rc = make_bf16_map(&a.map_x, x, B, K, ldx, errOut))) return rc;
  if ((rc = make_bf16_map(&a.map_w, w, V, K, ldw, errOut))) return rc;
  a.B = static_cast<int32_t>(B); a.V = static_cast<int32_t>(V); a.K = static_cast<int32_t>(K);
  a.tile0 = 0; a.tile_step = 1; a.ntile = static_cast<int32_t>((V + gs::LMH_BN - 1) / gs::LMH_BN);
  a.out_logits = out_logits; a.ld_out = ld_out; a.compact = 0;
  a.status = static_cast<uint32_t*>(c->lmh_scratch.ptr);
  CUDA_TRY(cudaMemsetAsync(a.status, 0, sizeof(uint32_t), c->stream), errOut);
  return launch_lm_head(c, a, errOut);
}

int gorch_cuda_lm_head_sample_dev(GorchCudaCtxRef ctx, const void* x, int64_t ldx, const void* w, int64_t ldw, int64_t B,
                                  int64_t V, int64_t K, int fuse_top_k, const GorchSampleCfg* cfgs, const double* uniforms,
                                  int32_t* out_ids, uint32_t* out_flags, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  int rc = check_lm_head(c, x, w, B, V, K, ldx, ldw, errOut);
  if (rc) return rc;
  if (B == 0) return GORCH_CUDA_OK;
  if (!cfgs || !uniforms || !out_ids) { set_err(errOut, "gorch_cuda: null pointer argument"); return GORCH_CUDA_ERR_BAD_ARG; }
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  if ((rc = load_encode_tiled(errOut))) return rc;
  gs::LmHeadArgs a;
  memset(&a, 0, sizeof a);
  if ((rc = make_bf16_map(&a.map_x, x, B, K, ldx, errOut))) return rc;
  if ((rc = make_bf16_map(&a.map_w, w, V, K, ldw, errOut))) return rc;
  a.B = static_cast<int32_t>(B); a.V = static_cast<int32_t>(V); a.K = static_cast<int32_t>(K);
  const int ntile = static_cast<int>((V + gs::LMH_BN - 1) / gs::LMH_BN);
  // the unfused form: logits to scratch, then the ordinary sampling kernels
  auto unfused = [&]() -> int {
    const int64_t ld = (V + 3) & ~3ll;
    int r2 = ensure(c->lmh_logits, static_cast<size_t>(B) * ld * sizeof(float), errOut);
    if (r2) return r2;
    if ((r2 = ensure(c->lmh_scratch, 256, errOut))) return r2;
    gs::LmHeadArgs u = a;
    u.tile0 = 0; u.tile_step = 1; u.ntile = ntile;
    u.out_logits = static_cast<float*>(c->lmh_logits.ptr); u.ld_out = ld; u.compact = 0;
    u.thr = nullptr; u.cand = nullptr; u.cand_cnt = nullptr; u.rowmax_key = nullptr; u.row_nan = nullptr;
    u.status = static_cast<uint32_t*>(c->lmh_scratch.ptr);
    CUDA_TRY(cudaMemsetAsync(u.status, 0, sizeof(uint32_t), c->stream), errOut);
    if ((r2 = launch_lm_head(c, u, errOut))) return r2;
    return launch_rows(c, c->lmh_logits.ptr, GORCH_CUDA_F32, B, V, ld, cfgs, uniforms, out_ids, out_flags, nullptr, nullptr, 0, errOut);
  };
  if (fuse_top_k < 1 || fuse_top_k > gs::KFAST || ntile < 4 * gs::LMH_SAMPLE_TILES_MIN || B > gs::LMH_ROWS_S) return unfused();
  int stiles = ntile / 32;
  if (stiles < gs::LMH_SAMPLE_TILES_MIN) stiles = gs::LMH_SAMPLE_TILES_MIN;
  if (stiles > gs::LMH_SAMPLE_TILES_MAX) stiles = gs::LMH_SAMPLE_TILES_MAX;

  // ---- the fused form: scratch = [status, nfail | thr | rowmax | nan | count | sample logits | candidates]
  const int nsample = stiles * gs::LMH_BN;
  // (candidates: one segment of LMH_SEG entries per row and CTA of the projection, and its count)
  const size_t nseg = static_cast<size_t>(ntile < c->sm_count ? ntile : c->sm_count);
  const size_t off_thr = 256, off_max = off_thr + 4 * B, off_nan = off_max + 4 * B;
  const size_t off_smp = (off_nan + 4 * B + 255) & ~static_cast<size_t>(255);
  const size_t off_cnt = (off_smp + sizeof(float) * B * nsample + 255) & ~static_cast<size_t>(255);
  const size_t off_cand = (off_cnt + 4 * static_cast<size_t>(B) * nseg + 255) & ~static_cast<size_t>(255);
  const size_t total = off_cand + sizeof(uint2) * static_cast<size_t>(B) * nseg * gs::LMH_SEG;
  if ((rc = ensure(c->lmh_scratch, total, errOut))) return rc;
  unsigned char* base = static_cast<unsigned char*>(c->lmh_scratch.ptr);
  CUDA_TRY(cudaMemsetAsync(base, 0, off_smp, c->stream), errOut);          // status, nfail, maxima, NaN bits (every CTA of the projection writes its counts)
  // 1. a sample of the vocabulary's tiles (all of them full tiles)
  gs::LmHeadArgs sa = a;
  sa.tile0 = 0; sa.tile_step = (ntile - 1) / stiles; sa.ntile = stiles;
  sa.out_logits = reinterpret_cast<float*>(base + off_smp); sa.ld_out = nsample; sa.compact = 1;
  sa.status = reinterpret_cast<uint32_t*>(base);
  if ((rc = launch_lm_head(c, sa, errOut))) return rc;
  // 2. thresholds
  gs::LmhSampleArgs fa;
  memset(&fa, 0, sizeof fa);
  fa.k.V = static_cast<int32_t>(V); fa.k.row_stride = V;
  fa.k.cfgs = reinterpret_cast<const gs::RowCfg*>(cfgs); fa.k.uniforms = uniforms;
  fa.k.out_ids = out_ids; fa.k.out_flags = out_flags; fa.k.exp_table = c->exp_table; fa.k.vs_cand = gs::VS_CAND; fa.k.vs_sumexp = 0;
  fa.sample = reinterpret_cast<const float*>(base + off_smp); fa.nsample = nsample; fa.fuse_top_k = fuse_top_k;
  fa.thr = reinterpret_cast<float*>(base + off_thr);
  fa.cand = reinterpret_cast<const uint2*>(base + off_cand);
  fa.cand_cnt = reinterpret_cast<const int32_t*>(base + off_cnt);
  fa.rowmax_key = reinterpret_cast<const uint32_t*>(base + off_max);
  fa.row_nan = reinterpret_cast<const int32_t*>(base + off_nan);
  fa.nfail = reinterpret_cast<int32_t*>(base + 4);
  fa.nseg = static_cast<int32_t>(nseg);
  fa.B = B;
  const unsigned g = static_cast<unsigned>(B < 4 * c->sm_count ? B : 4 * c->sm_count);
  gs::lmh_threshold_kernel<<<g, gs::LMH_F_NT, 0, c->stream>>>(fa);
  // 3. the whole vocabulary, candidates out of the epilogue
  gs::LmHeadArgs ma = a;
  ma.tile0 = 0; ma.tile_step = 1; ma.ntile = ntile;
  ma.out_logits = nullptr; ma.ld_out = 0; ma.compact = 0;
  ma.thr = fa.thr; ma.cand = reinterpret_cast<uint2*>(base + off_cand); ma.cand_cnt = reinterpret_cast<int32_t*>(base + off_cnt);
  ma.rowmax_key = reinterpret_cast<uint32_t*>(base + off_max); ma.row_nan = reinterpret_cast<int32_t*>(base + off_nan);
  ma.status = reinterpret_cast<uint32_t*>(base);
  if ((rc = launch_lm_head(c, ma, errOut))) return rc;
  // 4. finish every row from its candidates
  gs::lmh_finish_kernel<<<g, gs::LMH_F_NT, gs::LMH_F_DYN_BYTES, c->stream>>>(fa);
  CUDA_TRY(cudaGetLastError(), errOut);
  c->counters.kernel_launches += 2;
  c->counters.sample_launches += 1;
  c->counters.rows += static_cast<uint64_t>(B);
  // rows the fused form could not finish (their estimate failed, or their config is not served): the
  // count comes back to the host, which then recomputes the batch through the unfused form
  int32_t host_word[2] = {0, 0};
  CUDA_TRY(cudaMemcpyAsync(host_word, base, sizeof host_word, cudaMemcpyDeviceToHost, c->stream), errOut);
  CUDA_TRY(cudaStreamSynchronize(c->stream), errOut);
  if (host_word[0] != 0) {
    set_err(errOut, "gorch_cuda: the LM-head kernel gave up a bounded wait (status %d)", host_word[0]);
    return GORCH_CUDA_ERR_CUDA;
  }
  if (host_word[1] > 0) {
    c->counters.lm_head_refused_rows += static_cast<uint64_t>(host_word[1]);
    return unfused();
  }
  return GORCH_CUDA_OK;
}

int gorch_cuda_lm_head_status(GorchCudaCtxRef ctx, uint32_t* status, char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c || !status) { set_err(errOut, "gorch_cuda: null argument"); return GORCH_CUDA_ERR_BAD_ARG; }
  *status = 0;
  if (!c->lmh_scratch.ptr) return GORCH_CUDA_OK;
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  CUDA_TRY(cudaMemcpyAsync(status, c->lmh_scratch.ptr, sizeof(uint32_t), cudaMemcpyDeviceToHost, c->stream), errOut);
  CUDA_TRY(cudaStreamSynchronize(c->stream), errOut);
  return GORCH_CUDA_OK;
}

int gorch_cuda_sample_dev_static(GorchCudaCtxRef ctx, const void* logits, int dtype, int64_t B,
                                 int64_t V, int64_t row_stride, const GorchSampleCfg* cfgs,
                                 const double* uniforms, int32_t* out_ids, uint32_t* out_flags,
                                 char** errOut) {
  Ctx* c = static_cast<Ctx*>(ctx);
  if (!c) { set_err(errOut, "gorch_cuda: null context"); return GORCH_CUDA_ERR_BAD_ARG; }
  int rc = check_shape(dtype, B, V, row_stride, errOut);
  if (rc) return rc;
  if (B == 0) return GORCH_CUDA_OK;
  if (B > kStaticMaxRows) {
    set_err(errOut, "gorch_cuda: gorch_cuda_sample_dev_static serves at most %lld rows per call, got %lld",
            (long long)kStaticMaxRows, (long long)B);
    return GORCH_CUDA_ERR_LIMIT;
  }
  if (!logits || !cfgs || !uniforms || !out_ids) {
    set_err(errOut, "gorch_cuda: null pointer argument");
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  if ((reinterpret_cast<uintptr_t>(logits) % elem_size(dtype)) != 0) {
    set_err(errOut, "gorch_cuda: logits pointer not aligned to its element size");
    return GORCH_CUDA_ERR_BAD_ARG;
  }
  CUDA_TRY(cudaSetDevice(c->device), errOut);
  int32_t* base = nullptr;
  if ((rc = static_lists_ptr(c->device, &base, errOut))) return rc;   // looked up when the context was created
  // the same dispatch as gorch_cuda_sample_dev, with the work lists in the fixed array (it keeps the
  // previous call's contents: the dispatch clears the cursors and counts it uses before every launch)
  return launch_rows(c, logits, dtype, B, V, row_stride, cfgs, uniforms, out_ids, out_flags, nullptr, nullptr, 0,
                     errOut, base);
}

}  // extern "C"
