// C ABI and host-side launch policy of the sm_100a exact radix top-k indexer.
// Declarations and the reference interfaces each entry point replaces are in
// include/ff_topk.h.
#include "../../include/ff_topk.h"

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "ff_topk_kernel.cuh"

namespace {

thread_local char g_err[256] = "";
std::atomic<int64_t> g_launches{0};
std::atomic<int> g_cluster_override{0};
std::atomic<int> g_groups_override{0};
std::atomic<unsigned long long*> g_trace{nullptr};

std::atomic<int> g_self_seed{-1};   // -1: FF_TOPK_SELF_SEED or on; 0 / 1: set through ff_topk_set_self_seed

// Launch with programmatic stream serialization: the kernel is set up while the kernel before it on
// the stream still runs and waits for that kernel's completion itself (griddepcontrol.wait, its first
// instruction), so part of its launch latency hides behind that kernel's tail.
std::atomic<int> g_programmatic{-1};   // -1: FF_TOPK_PDL or on; 0 / 1: set through ff_topk_set_programmatic_launch
bool programmatic_launch_enabled() {
  const int v = g_programmatic.load(std::memory_order_relaxed);
  if (v >= 0) return v != 0;
  static const bool on = [] { const char* e = getenv("FF_TOPK_PDL"); return e == nullptr || atoi(e) != 0; }();
  return on;
}
bool self_seed_enabled() {
  const int v = g_self_seed.load(std::memory_order_relaxed);
  if (v >= 0) return v != 0;
  const char* env = getenv("FF_TOPK_SELF_SEED");
  return env == nullptr || atoi(env) != 0;
}

constexpr int kMaxDevices = 64;
std::once_flag g_init_once[kMaxDevices];
int g_init_rc[kMaxDevices];
int g_max_cluster[kMaxDevices];  // largest schedulable cluster size per device
int g_sm_count[kMaxDevices];
int g_active_clusters[kMaxDevices][5];  // co-resident clusters of size 1, 2, 4, 8, 16

int fail(int code, const char* msg) {
  snprintf(g_err, sizeof(g_err), "%s", msg);
  return code;
}
int fail_cuda(cudaError_t e, const char* where) {
  snprintf(g_err, sizeof(g_err), "%s: %s", where, cudaGetErrorString(e));
  return static_cast<int>(e);
}

template <typename K>
cudaError_t prepare_kernel(K kernel) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       ff::smem_bytes_for(ff::kMaxStages));
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
}

template <typename K>
int active_clusters_for(K kernel, int c) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(c, 1, 1);
  cfg.blockDim = dim3(ff::kThreads, 1, 1);
  cfg.dynamicSmemBytes = ff::smem_bytes_for(ff::kMaxStages);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = c;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

template <typename K>
int max_cluster_for(K kernel) {
  // Largest power-of-two cluster (<= 16) of which at least one fits on the device.
  for (int c = ff::kMaxCluster; c > 1; c >>= 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(c, 1, 1);
    cfg.blockDim = dim3(ff::kThreads, 1, 1);
    cfg.dynamicSmemBytes = ff::smem_bytes_for(ff::kMaxStages);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = c;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) == cudaSuccess && n > 0) return c;
    (void)cudaGetLastError();
  }
  return 1;
}

void init_device(int device) {
  int prev = 0;
  cudaError_t e = cudaGetDevice(&prev);
  if (e == cudaSuccess && prev != device) e = cudaSetDevice(device);
  if (e == cudaSuccess) e = prepare_kernel(ff::topk_cluster_kernel<false, ff::kModePlain>);
  if (e == cudaSuccess) e = prepare_kernel(ff::topk_cluster_kernel<false, ff::kModeHinted>);
  if (e == cudaSuccess) e = prepare_kernel(ff::topk_cluster_kernel<false, ff::kModePush>);
  if (e == cudaSuccess) e = prepare_kernel(ff::topk_cluster_kernel<false, ff::kModePushHinted>);
  if (e == cudaSuccess) e = prepare_kernel(ff::topk_cluster_kernel<false, ff::kModePushHintedSx>);
  if (e == cudaSuccess) e = prepare_kernel(ff::topk_cluster_kernel<true, ff::kModePlain>);
  if (e == cudaSuccess) e = prepare_kernel(ff::topk_cluster_kernel<false, ff::kModePlain, __nv_bfloat16>);
  if (e == cudaSuccess) e = prepare_kernel(ff::topk_cluster_kernel<false, ff::kModeHinted, __nv_bfloat16>);
  if (e == cudaSuccess) e = prepare_kernel(ff::topk_cluster_kernel<false, ff::kModePlain, __half>);
  if (e == cudaSuccess) e = prepare_kernel(ff::topk_cluster_kernel<false, ff::kModeHinted, __half>);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(ff::cp_merge_sorted_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             ff::kMaxPeers * ff::kMaxK * static_cast<int>(sizeof(uint32_t)));
  if (e == cudaSuccess) {
    g_max_cluster[device] = max_cluster_for(ff::topk_cluster_kernel<false, ff::kModePlain>);
    for (int i = 0; i < 5; ++i)
      g_active_clusters[device][i] = active_clusters_for(ff::topk_cluster_kernel<false, ff::kModePlain>, 1 << i);
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    g_sm_count[device] = sms > 0 ? sms : 148;
  }
  if (prev != device) (void)cudaSetDevice(prev);
  g_init_rc[device] = static_cast<int>(e);
}

int ensure_init(int* device_out) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  if (device < 0 || device >= kMaxDevices) return fail(FF_ERR_BAD_SHAPE, "device ordinal out of range");
  std::call_once(g_init_once[device], init_device, device);
  if (g_init_rc[device] != 0)
    return fail_cuda(static_cast<cudaError_t>(g_init_rc[device]), "ff_topk_init");
  *device_out = device;
  return 0;
}


// Cluster size per row.  One CTA sweeps about 16 Ki scores; the cluster grows
// with the row up to the largest size the device can schedule, but not beyond
// what lets every row of the batch run at the same time.
int choose_cluster(int device, int32_t B, int64_t L_width, int32_t k) {
  (void)k;
  int c = g_cluster_override.load();
  if (c == 0) {
    const char* env = getenv("FF_TOPK_CLUSTER");
    if (env != nullptr) c = atoi(env);
  }
  if (c == 0) {
    // Measured on B200: the widest cluster is fastest at every row length down
    // to 4 Ki (the finish is shared out over the cluster), so take the largest
    // size that keeps the whole batch in one wave of CTAs (one CTA per SM).
    c = ff::kMaxCluster;
    int fit = 1;
    while (fit * 2 * static_cast<int64_t>(B) <= g_sm_count[device] && fit < ff::kMaxCluster) fit *= 2;
    if (c > fit) c = fit;
  }
  if (c > ff::kMaxCluster) c = ff::kMaxCluster;
  if (c > g_max_cluster[device]) c = g_max_cluster[device];
  return c;
}

// Rows that are long and few are split over several clusters (groups) so that
// all SMs sweep them; that needs the caller's zero-filled workspace and a
// cooperative launch (all CTAs of a row wait for each other through global
// memory).  Returns the number of clusters per row and may lower `cluster`.
// Measured on B200 (B = 1, k = 2048, clusters of 8): with 15 or more clusters a split row beats one
// cluster of 16 from 128 Ki columns up (15.9 against 16.2 us; 16.8 against 20.3 us at 512 Ki), and
// with a threshold guess from 64 Ki up (10.1 against 12.5 us); with only 4 clusters it loses below
// 768 Ki columns.  So shorter rows are split only if at least 8 clusters are free for each.
constexpr int64_t kGroupMinWidth = 131072;
constexpr int64_t kGroupMinWidthHinted = 65536;
constexpr int64_t kGroupAlwaysWidth = 786432;
constexpr int kGroupCluster = 8;
int choose_groups(int device, int32_t B, int64_t L_width, size_t workspace_bytes, int* cluster, bool hinted = false) {
  int g = g_groups_override.load();
  if (g == 0) {
    const char* env = getenv("FF_TOPK_GROUPS");
    if (env != nullptr) g = atoi(env);
  }
  const size_t need = static_cast<size_t>(B) * ff::kWsRowWords * sizeof(uint32_t);
  if (workspace_bytes < need || g == 1) return 1;
  int c = *cluster;
  const bool automatic = g == 0;
  if (automatic) {
    if (L_width < (hinted ? kGroupMinWidthHinted : kGroupMinWidth) || g_cluster_override.load() != 0) return 1;
    c = kGroupCluster;
    g = 16;                                                     // more clusters than that bring nothing
    const int64_t by_size = L_width / (static_cast<int64_t>(c) * 1024);   // at least 1 Ki columns per CTA
    if (g > by_size) g = static_cast<int>(by_size);
  }
  int log2c = 0;
  while ((1 << log2c) < c) ++log2c;
  const int room = g_active_clusters[device][log2c] / (B > 0 ? B : 1);   // co-resident clusters per row
  if (g > room) g = room;
  if (automatic && L_width < kGroupAlwaysWidth && g < 8) return 1;
  if (g > 64) g = 64;
  if (g < 2) return 1;
  *cluster = c;
  return g;
}

template <bool HAS_MAP>
int launch(const ff::TopkParams& p, int cluster, cudaStream_t stream, int dtype = FF_DTYPE_F32) {
  cudaLaunchConfig_t cfg = {};
  const int groups = p.groups > 1 ? p.groups : 1;
  cfg.gridDim = dim3(static_cast<unsigned>(p.B) * cluster * groups, 1, 1);
  cfg.blockDim = dim3(ff::kThreads, 1, 1);
  cfg.dynamicSmemBytes = ff::smem_bytes_for(ff::kMaxStages);
  cfg.stream = stream;
  cudaLaunchAttribute attr[3];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // Cooperative whenever CTAs of the launch wait for each other through global memory: rows split
  // over clusters, and the single-kernel context-parallel step (its CTAs poll for entries that
  // CTAs of the same launch on the peers store), so that residency is guaranteed, not inferred.
  if (groups > 1 || p.push_fused != 0) {
    attr[cfg.numAttrs].id = cudaLaunchAttributeCooperative;
    attr[cfg.numAttrs].val.cooperative = 1;
    ++cfg.numAttrs;
  }
  if (programmatic_launch_enabled()) {
    attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
    ++cfg.numAttrs;
  }
  ff::TopkParams q = p;
  q.trace = g_trace.load(std::memory_order_relaxed);
  q.block_base = 0;
  q.grid_ctas = static_cast<int32_t>(cfg.gridDim.x);

  // one instantiation per mode: the plain select carries no code of the others
  cudaError_t e;
  // A row split over clusters that has no guess makes its own (FF_TOPK_SELF_SEED=0 or
  // ff_topk_set_self_seed(0) switch that off); the code lives in the instantiation with guesses.
  if (!HAS_MAP && groups > 1 && self_seed_enabled()) q.self_seed = 1;
  const bool hints = q.hint_in != nullptr || q.hint_out != nullptr || q.self_seed != 0;
  if (!HAS_MAP && dtype == FF_DTYPE_BF16)
    e = hints ? cudaLaunchKernelEx(&cfg, ff::topk_cluster_kernel<false, ff::kModeHinted, __nv_bfloat16>, q)
              : cudaLaunchKernelEx(&cfg, ff::topk_cluster_kernel<false, ff::kModePlain, __nv_bfloat16>, q);
  else if (!HAS_MAP && dtype == FF_DTYPE_F16)
    e = hints ? cudaLaunchKernelEx(&cfg, ff::topk_cluster_kernel<false, ff::kModeHinted, __half>, q)
              : cudaLaunchKernelEx(&cfg, ff::topk_cluster_kernel<false, ff::kModePlain, __half>, q);
  else if (!HAS_MAP && q.push_world > 0 && q.push_sx != 0)
    e = cudaLaunchKernelEx(&cfg, ff::topk_cluster_kernel<false, ff::kModePushHintedSx>, q);
  else if (!HAS_MAP && q.push_world > 0 && hints)
    e = cudaLaunchKernelEx(&cfg, ff::topk_cluster_kernel<false, ff::kModePushHinted>, q);
  else if (!HAS_MAP && q.push_world > 0)
    e = cudaLaunchKernelEx(&cfg, ff::topk_cluster_kernel<false, ff::kModePush>, q);
  else if (!HAS_MAP && hints)
    e = cudaLaunchKernelEx(&cfg, ff::topk_cluster_kernel<false, ff::kModeHinted>, q);
  else
    e = cudaLaunchKernelEx(&cfg, ff::topk_cluster_kernel<HAS_MAP, ff::kModePlain>, q);
  if (e != cudaSuccess) return fail_cuda(e, "cudaLaunchKernelEx(topk_cluster_kernel)");
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}

// Built-in scratch for ff_topk_launch_static: enough for FF_TOPK_STATIC_MAX_ROWS
// rows split over several clusters.  It lives in every GPU that loads this
// library until the process exits.  In host code the name below is only a
// handle for cudaGetSymbolAddress; it is never passed to a kernel.
static __device__ __align__(256) uint32_t g_static_scratch[FF_TOPK_STATIC_MAX_ROWS * ff::kWsRowWords];
std::mutex g_static_mutex;
std::atomic<uint32_t*> g_static_ptr[kMaxDevices];

// Device address of the built-in scratch on `device`, which must be current.  Only a success is
// remembered: a first call that fails (for instance because it was made while a stream capture
// was active) leaves nothing behind, and the next call simply tries again.
int static_scratch_address(int device, uint32_t** out) {
  uint32_t* ptr = g_static_ptr[device].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    ptr = g_static_ptr[device].load(std::memory_order_relaxed);
    if (ptr == nullptr) {
      void* sym = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&sym, g_static_scratch);
      if (e != cudaSuccess || sym == nullptr) {
        (void)cudaGetLastError();
        return fail_cuda(e == cudaSuccess ? cudaErrorInvalidSymbol : e, "cudaGetSymbolAddress(built-in scratch)");
      }
      ptr = static_cast<uint32_t*>(sym);
      g_static_ptr[device].store(ptr, std::memory_order_release);
    }
  }
  *out = ptr;
  return 0;
}

int check_common(int32_t B, int64_t L_width, int32_t k) {
  if (k < 1 || k > FF_TOPK_MAX_K) return fail(FF_ERR_BAD_K, "k must be in [1, 2048]");
  if (B < 0 || L_width < 0) return fail(FF_ERR_BAD_SHAPE, "negative B or L_width");
  if (L_width > 0x7fffffffLL) return fail(FF_ERR_TOO_LARGE, "L_width exceeds int32 indices");
  if (static_cast<int64_t>(B) * ff::kMaxCluster > 0x7fffffffLL)
    return fail(FF_ERR_TOO_LARGE, "B too large for one launch");
  return 0;
}

}  // namespace

extern "C" {

int32_t ff_topk_abi_version(void) { return 1; }

const char* ff_last_error_string(void) { return g_err; }

int64_t ff_topk_launch_count(void) { return g_launches.load(); }

int ff_topk_init(int device) {
  if (device < 0 || device >= kMaxDevices) return fail(FF_ERR_BAD_SHAPE, "device ordinal out of range");
  std::call_once(g_init_once[device], init_device, device);
  if (g_init_rc[device] != 0)
    return fail_cuda(static_cast<cudaError_t>(g_init_rc[device]), "ff_topk_init");
  return 0;
}

int ff_topk_set_cluster_override(int32_t c) {
  if (!(c == 0 || c == 1 || c == 2 || c == 4 || c == 8 || c == 16))
    return fail(FF_ERR_BAD_CLUSTER, "cluster override must be 0, 1, 2, 4, 8 or 16");
  g_cluster_override.store(c);
  return 0;
}

int ff_topk_set_trace_buffer(void* device_buffer) {
  g_trace.store(static_cast<unsigned long long*>(device_buffer));
  return 0;
}

int32_t ff_topk_policy_cluster_size(int32_t B, int64_t L_width, int32_t k) {
  int device = 0;
  if (ensure_init(&device) != 0) return -1;
  return choose_cluster(device, B, L_width, k);
}

int ff_topk_policy_launch_shape(int32_t B, int64_t L_width, int32_t k, int32_t has_workspace, int32_t hinted,
                                int32_t* out2) {
  if (out2 == nullptr) return fail(FF_ERR_NULL, "out2 must not be NULL");
  int device = 0;
  const int rc = ensure_init(&device);
  if (rc != 0) return rc;
  int cluster = choose_cluster(device, B, L_width, k);
  int groups = 1;
  if (has_workspace != 0)
    groups = choose_groups(device, B, L_width, ff_topk_workspace_bytes(B, L_width, k), &cluster, hinted != 0);
  out2[0] = cluster;
  out2[1] = groups;
  return 0;
}

size_t ff_topk_workspace_bytes(int32_t B, int64_t L_width, int32_t k) {
  (void)k;
  // Only rows split over several clusters use scratch: long rows, small batches.
  if (B < 1 || B > 16 || (L_width < kGroupMinWidthHinted && g_groups_override.load() < 2)) return 0;
  return static_cast<size_t>(B) * ff::kWsRowWords * sizeof(uint32_t);
}

int ff_topk_set_self_seed(int32_t on) {
  g_self_seed.store(on < 0 ? -1 : (on != 0 ? 1 : 0));
  return 0;
}

int ff_topk_set_programmatic_launch(int32_t on) {
  g_programmatic.store(on < 0 ? -1 : (on != 0 ? 1 : 0));
  return 0;
}

int ff_topk_set_groups_override(int32_t g) {
  if (g < 0 || g > 64) return fail(FF_ERR_BAD_CLUSTER, "groups override must be in [0, 64]");
  g_groups_override.store(g);
  return 0;
}

}  // extern "C"

namespace {

int transform_launch_impl(const void* scores_any, int dtype, int64_t row_stride, const int32_t* lengths,
                          const int32_t* row_starts, void* out_any, int index_bits, int32_t B, int64_t L_width,
                          int32_t k, int32_t epilogue, const int32_t* table,
                          int64_t table_stride, const int32_t* cu_seqlens_q,
                          int32_t n_table_rows, const int32_t* offsets, const float* hint_in,
                          float* hint_out, void* workspace, size_t workspace_bytes, int32_t* status,
                          void* stream, void* handover = nullptr) {
  int rc = check_common(B, L_width, k);
  if (rc != 0) return rc;
  if (B == 0) return 0;
  const float* scores = static_cast<const float*>(scores_any);
  if (scores == nullptr || lengths == nullptr || out_any == nullptr)
    return fail(FF_ERR_NULL, "scores, lengths and out must not be NULL");
  if (row_stride < 0) return fail(FF_ERR_BAD_SHAPE, "negative row_stride");
  if (dtype != FF_DTYPE_F32 && dtype != FF_DTYPE_BF16 && dtype != FF_DTYPE_F16)
    return fail(FF_ERR_BAD_SHAPE, "score_dtype must be FF_DTYPE_F32, FF_DTYPE_BF16 or FF_DTYPE_F16");
  if (index_bits != 32 && index_bits != 64) return fail(FF_ERR_BAD_SHAPE, "index_bits must be 32 or 64");
  if ((reinterpret_cast<uintptr_t>(scores) & (dtype == FF_DTYPE_F32 ? 3u : 1u)) != 0)
    return fail(FF_ERR_BAD_SHAPE, "scores must be aligned to their element size");
  if (epilogue == FF_EPILOGUE_PAGE_TABLE) {
    if (table == nullptr) return fail(FF_ERR_NULL, "page-table epilogue needs a table");
    if (cu_seqlens_q != nullptr && n_table_rows < 1)
      return fail(FF_ERR_BAD_SHAPE, "prefill page-table epilogue needs n_table_rows >= 1");
  } else if (epilogue == FF_EPILOGUE_ADD_OFFSET) {
    if (offsets == nullptr) return fail(FF_ERR_NULL, "offset epilogue needs offsets");
  } else if (epilogue != FF_EPILOGUE_INDEX) {
    return fail(FF_ERR_BAD_SHAPE, "unknown epilogue");
  }
  int device = 0;
  rc = ensure_init(&device);
  if (rc != 0) return rc;
  ff::TopkParams p = {};
  p.scores = scores;
  p.row_stride = row_stride;
  p.lengths = lengths;
  p.row_starts = row_starts;
  if (index_bits == 64) p.out_idx64 = static_cast<int64_t*>(out_any);
  else p.out_idx = static_cast<int32_t*>(out_any);
  p.B = B;
  p.k = k;
  p.L_width = L_width;
  p.fixed_len = -1;
  p.epilogue = epilogue;
  p.table = table;
  p.table_stride = table_stride;
  p.cu_seqlens_q = cu_seqlens_q;
  p.n_table_rows = n_table_rows;
  p.offsets = offsets;
  p.status = status;
  p.hint_in = hint_in;
  p.hint_out = hint_out;
  if (handover != nullptr) {
    if (hint_in == nullptr) return fail(FF_ERR_NULL, "a hand-over list needs the guesses it was built with (hint_in)");
    if ((reinterpret_cast<uintptr_t>(handover) & 63u) != 0) return fail(FF_ERR_BAD_SHAPE, "handover must be 64-byte aligned");
    if (dtype != FF_DTYPE_F32) return fail(FF_ERR_BAD_SHAPE, "the hand-over lists hold fp32 scores");
    static_assert(FF_TOPK_HANDOVER_ROW_BYTES == ff::kHandoverRowBytes, "hand-over layout");
    p.handover = static_cast<unsigned char*>(handover);
  }
  int cluster = choose_cluster(device, B, L_width, k);
  if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0) {
    p.groups = choose_groups(device, B, L_width, workspace_bytes, &cluster, hint_in != nullptr);
    p.workspace = static_cast<uint32_t*>(workspace);
  }
  return launch<false>(p, cluster, static_cast<cudaStream_t>(stream), dtype);
}

}  // namespace

extern "C" {

int ff_topk_launch_typed(const void* scores, int32_t score_dtype, int64_t row_stride, const int32_t* lengths,
                         const int32_t* row_starts, void* out_idx, int32_t index_bits, int32_t B, int64_t L_width,
                         int32_t k, const float* hint_in, float* hint_out, void* workspace, size_t workspace_bytes,
                         int32_t* status, void* stream) {
  return transform_launch_impl(scores, score_dtype, row_stride, lengths, row_starts, out_idx, index_bits, B, L_width,
                               k, FF_EPILOGUE_INDEX, nullptr, 0, nullptr, 0, nullptr, hint_in, hint_out, workspace,
                               workspace_bytes, status, stream);
}

int ff_topk_transform_launch(const float* scores, int64_t row_stride, const int32_t* lengths,
                             const int32_t* row_starts, int32_t* out, int32_t B, int64_t L_width,
                             int32_t k, int32_t epilogue, const int32_t* table,
                             int64_t table_stride, const int32_t* cu_seqlens_q,
                             int32_t n_table_rows, const int32_t* offsets, void* workspace,
                             size_t workspace_bytes, int32_t* status, void* stream) {
  return transform_launch_impl(scores, FF_DTYPE_F32, row_stride, lengths, row_starts, out, 32, B, L_width, k, epilogue,
                               table, table_stride, cu_seqlens_q, n_table_rows, offsets, nullptr, nullptr, workspace,
                               workspace_bytes, status, stream);
}

int ff_topk_launch_hinted(const float* scores, int64_t row_stride, const int32_t* lengths,
                          const int32_t* row_starts, int32_t* out_idx, int32_t B, int64_t L_width,
                          int32_t k, const float* hint_in, float* hint_out, void* workspace,
                          size_t workspace_bytes, int32_t* status, void* stream) {
  return transform_launch_impl(scores, FF_DTYPE_F32, row_stride, lengths, row_starts, out_idx, 32, B, L_width, k,
                               FF_EPILOGUE_INDEX, nullptr, 0, nullptr, 0, nullptr, hint_in, hint_out, workspace,
                               workspace_bytes, status, stream);
}

int ff_topk_launch_handover(const float* scores, int64_t row_stride, const int32_t* lengths,
                            const int32_t* row_starts, int32_t* out_idx, int32_t B, int64_t L_width, int32_t k,
                            const float* hint_in, float* hint_out, void* handover, void* workspace,
                            size_t workspace_bytes, int32_t* status, void* stream) {
  if (handover == nullptr) return fail(FF_ERR_NULL, "handover must not be NULL");
  return transform_launch_impl(scores, FF_DTYPE_F32, row_stride, lengths, row_starts, out_idx, 32, B, L_width, k,
                               FF_EPILOGUE_INDEX, nullptr, 0, nullptr, 0, nullptr, hint_in, hint_out, workspace,
                               workspace_bytes, status, stream, handover);
}

int ff_topk_launch(const float* scores, int64_t row_stride, const int32_t* lengths,
                   const int32_t* row_starts, int32_t* out_idx, int32_t B, int64_t L_width,
                   int32_t k, void* workspace, size_t workspace_bytes, int32_t* status,
                   void* stream) {
  return ff_topk_transform_launch(scores, row_stride, lengths, row_starts, out_idx, B, L_width, k,
                                  FF_EPILOGUE_INDEX, nullptr, 0, nullptr, 0, nullptr, workspace,
                                  workspace_bytes, status, stream);
}

int ff_topk_launch_static(const float* scores, int64_t row_stride, const int32_t* lengths,
                          const int32_t* row_starts, int32_t* out_idx, int32_t B, int64_t L_width,
                          int32_t k, int32_t* status, void* stream) {
  int rc = check_common(B, L_width, k);
  if (rc != 0) return rc;
  if (B > FF_TOPK_STATIC_MAX_ROWS)
    return fail(FF_ERR_TOO_LARGE, "ff_topk_launch_static: B exceeds FF_TOPK_STATIC_MAX_ROWS rows of built-in scratch");
  if (B == 0) return 0;
  if (scores == nullptr || lengths == nullptr || out_idx == nullptr)
    return fail(FF_ERR_NULL, "scores, lengths and out_idx must not be NULL");
  if (row_stride < 0) return fail(FF_ERR_BAD_SHAPE, "negative row_stride");
  if ((reinterpret_cast<uintptr_t>(scores) & 3u) != 0)
    return fail(FF_ERR_BAD_SHAPE, "scores must be 4-byte aligned");
  int device = 0;
  rc = ensure_init(&device);
  if (rc != 0) return rc;
  uint32_t* scratch = nullptr;
  rc = static_scratch_address(device, &scratch);
  if (rc != 0) return rc;
  const size_t row_bytes = static_cast<size_t>(ff::kWsRowWords) * sizeof(uint32_t);
  ff::TopkParams p = {};
  p.scores = scores;
  p.row_stride = row_stride;
  p.lengths = lengths;
  p.row_starts = row_starts;
  p.out_idx = out_idx;
  p.B = B;
  p.k = k;
  p.L_width = L_width;
  p.fixed_len = -1;
  p.epilogue = FF_EPILOGUE_INDEX;
  p.status = status;
  int cluster = choose_cluster(device, B, L_width, k);
  p.groups = choose_groups(device, B, L_width, FF_TOPK_STATIC_MAX_ROWS * row_bytes, &cluster);
  p.workspace = scratch;
  if (p.groups > 1) {
    // Only rows split over several clusters touch the scratch.  The array keeps whatever the
    // previous call left; the counters, histograms and lists must start at zero.
    const cudaError_t e =
        cudaMemsetAsync(scratch, 0, static_cast<size_t>(B) * row_bytes, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail_cuda(e, "cudaMemsetAsync(built-in scratch)");
  }
  return launch<false>(p, cluster, static_cast<cudaStream_t>(stream));
}

int ff_topk_cp_local(const float* scores, int64_t row_stride, const int32_t* lengths,
                     int32_t* cand_idx, float* cand_val, int32_t B, int64_t L_width, int32_t k,
                     int64_t shard_offset, void* workspace, size_t workspace_bytes,
                     int32_t* status, void* stream) {
  int rc = check_common(B, L_width, k);
  if (rc != 0) return rc;
  if (B == 0) return 0;
  if (scores == nullptr || lengths == nullptr || cand_idx == nullptr || cand_val == nullptr)
    return fail(FF_ERR_NULL, "scores, lengths, cand_idx and cand_val must not be NULL");
  if (shard_offset < 0 || shard_offset + L_width > 0x7fffffffLL)
    return fail(FF_ERR_TOO_LARGE, "shard_offset + L_width exceeds int32 indices");
  if (row_stride < 0) return fail(FF_ERR_BAD_SHAPE, "negative row_stride");
  int device = 0;
  rc = ensure_init(&device);
  if (rc != 0) return rc;
  ff::TopkParams p = {};
  p.scores = scores;
  p.row_stride = row_stride;
  p.lengths = lengths;
  p.out_idx = cand_idx;
  p.out_val = cand_val;
  p.B = B;
  p.k = k;
  p.L_width = L_width;
  p.shard_offset = shard_offset;
  p.fixed_len = -1;
  p.status = status;
  int cluster = choose_cluster(device, B, L_width, k);
  if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0) {
    p.groups = choose_groups(device, B, L_width, workspace_bytes, &cluster);
    p.workspace = static_cast<uint32_t*>(workspace);
  }
  return launch<false>(p, cluster, static_cast<cudaStream_t>(stream));
}

int ff_topk_cp_merge(const float* cand_val, const int32_t* cand_idx, int32_t n_ranks,
                     int64_t rank_stride, const int32_t* lengths, int32_t* out_idx, int32_t B,
                     int32_t k, void* workspace, size_t workspace_bytes, int32_t* status,
                     void* stream) {
  (void)workspace;
  (void)workspace_bytes;
  if (n_ranks < 1 || n_ranks > 1024) return fail(FF_ERR_BAD_SHAPE, "n_ranks must be in [1, 1024]");
  const int64_t n_cand = static_cast<int64_t>(n_ranks) * k;
  int rc = check_common(B, n_cand, k);
  if (rc != 0) return rc;
  if (B == 0) return 0;
  if (cand_val == nullptr || cand_idx == nullptr || lengths == nullptr || out_idx == nullptr)
    return fail(FF_ERR_NULL, "cand_val, cand_idx, lengths and out_idx must not be NULL");
  if (n_ranks > 1 && rank_stride < static_cast<int64_t>(B) * k)
    return fail(FF_ERR_BAD_SHAPE, "rank_stride < B*k");
  int device = 0;
  rc = ensure_init(&device);
  if (rc != 0) return rc;
  ff::TopkParams p = {};
  p.scores = cand_val;
  p.row_stride = k;
  p.lengths = lengths;
  p.idx_map = cand_idx;
  p.seg_len = k;
  p.seg_stride = rank_stride;
  p.out_idx = out_idx;
  p.B = B;
  p.k = k;
  p.L_width = n_cand;
  p.fixed_len = static_cast<int32_t>(n_cand);
  p.status = status;
  return launch<true>(p, choose_cluster(device, B, n_cand, k), static_cast<cudaStream_t>(stream));
}

// ---- context-parallel exchange over peer memory -----------------------------

struct FfCpExchange {
  int world, rank, B, k, device;
  size_t slot_words;     // one rank's candidate block: a 16-byte entry per (row, position) (4*B*k words)
  size_t ctrl_offset;    // words from the allocation's start to the control words
  size_t send_offset;    // words from the allocation's start to the send block
  size_t sx_offset;      // words from the allocation's start to the survivor-exchange regions
  size_t total_bytes;
  uint32_t* base;        // this rank's allocation
  void* peer[ff::kMaxPeers];
  bool opened[ff::kMaxPeers];
};

int ff_cp_exchange_create(int32_t world, int32_t rank, int32_t B, int32_t k, void** out) {
  if (out == nullptr) return fail(FF_ERR_NULL, "out must not be NULL");
  if (world < 1 || world > ff::kMaxPeers || rank < 0 || rank >= world)
    return fail(FF_ERR_BAD_SHAPE, "world must be in [1, 16] and rank in [0, world)");
  if (B < 1 || k < 1 || k > FF_TOPK_MAX_K) return fail(FF_ERR_BAD_K, "B >= 1 and k in [1, 2048] required");
  int device = 0;
  int rc = ensure_init(&device);
  if (rc != 0) return rc;
  FfCpExchange* ex = new FfCpExchange();
  ex->world = world;
  ex->rank = rank;
  ex->B = B;
  ex->k = k;
  ex->device = device;
  ex->slot_words = 4 * static_cast<size_t>(B) * k;
  ex->ctrl_offset = 2 * static_cast<size_t>(world) * ex->slot_words;
  ex->send_offset = ex->ctrl_offset + ff::kCtrlWords;
  ex->sx_offset = ex->send_offset + ex->slot_words;
  // survivor exchange: two step parities x world sending ranks x B rows x 128 regions of 528 bytes
  const size_t sx_words = 2 * static_cast<size_t>(world) * B * ff::kSxRegions * ff::kSxRegionWords;
  ex->total_bytes = (ex->sx_offset + sx_words) * sizeof(uint32_t);
  for (int i = 0; i < ff::kMaxPeers; ++i) {
    ex->peer[i] = nullptr;
    ex->opened[i] = false;
  }
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&ex->base), ex->total_bytes);
  if (e == cudaSuccess) e = cudaMemset(ex->base, 0, ex->total_bytes);
  if (e != cudaSuccess) {
    delete ex;
    return fail_cuda(e, "ff_cp_exchange_create");
  }
  ex->peer[rank] = ex->base;
  *out = ex;
  return 0;
}

int64_t ff_cp_exchange_bytes(void* handle) {
  return handle == nullptr ? 0 : static_cast<int64_t>(static_cast<FfCpExchange*>(handle)->total_bytes);
}

void* ff_cp_exchange_base(void* handle) {
  return handle == nullptr ? nullptr : static_cast<FfCpExchange*>(handle)->base;
}

int ff_cp_exchange_ipc_handle(void* handle, void* out64) {
  if (handle == nullptr || out64 == nullptr) return fail(FF_ERR_NULL, "NULL argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, static_cast<FfCpExchange*>(handle)->base);
  if (e != cudaSuccess) return fail_cuda(e, "cudaIpcGetMemHandle");
  memcpy(out64, &h, 64);
  return 0;
}

int ff_cp_exchange_open_peers(void* handle, const void* handles, int32_t n) {
  if (handle == nullptr || handles == nullptr) return fail(FF_ERR_NULL, "NULL argument");
  FfCpExchange* ex = static_cast<FfCpExchange*>(handle);
  if (n != ex->world) return fail(FF_ERR_BAD_SHAPE, "one handle per rank expected");
  for (int p = 0; p < ex->world; ++p) {
    if (p == ex->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const char*>(handles) + 64 * p, 64);
    void* ptr = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail_cuda(e, "cudaIpcOpenMemHandle");
    ex->peer[p] = ptr;
    ex->opened[p] = true;
  }
  return 0;
}

int ff_cp_exchange_set_peer(void* handle, int32_t p, void* peer_base) {
  if (handle == nullptr || peer_base == nullptr) return fail(FF_ERR_NULL, "NULL argument");
  FfCpExchange* ex = static_cast<FfCpExchange*>(handle);
  if (p < 0 || p >= ex->world) return fail(FF_ERR_BAD_SHAPE, "peer out of range");
  ex->peer[p] = peer_base;
  return 0;
}

int ff_cp_exchange_destroy(void* handle) {
  if (handle == nullptr) return 0;
  FfCpExchange* ex = static_cast<FfCpExchange*>(handle);
  for (int p = 0; p < ex->world; ++p) {
    if (ex->opened[p]) (void)cudaIpcCloseMemHandle(ex->peer[p]);
  }
  (void)cudaFree(ex->base);
  delete ex;
  return 0;
}

}  // extern "C"

namespace {

// Whether a context-parallel step may run as ONE kernel (select, announce, wait, merge).
// -1: decide from the launch shape; 0 / 1: forced by FF_TOPK_CP_FUSED (1 still needs a
// launch whose CTAs are all resident at once).
int cp_fused_setting() {
  const char* env = getenv("FF_TOPK_CP_FUSED");
  return env != nullptr ? atoi(env) : -1;
}

// How many of a rank's k candidates per row go to the peers right away in a single-kernel step.
// Each of `world` contiguous shards holds about k / world of the row's top-k; twice that (and never
// fewer than 256) is sent, so that on rows whose winners are spread over the shards the first round
// is enough, and the link carries 2 k entries per rank instead of world * k.  Rows whose winners
// crowd into few shards take the second round (exact either way).  FF_TOPK_CP_PREFIX overrides.
int cp_prefix(int world, int k) {
  const char* env = getenv("FF_TOPK_CP_PREFIX");
  int s = env != nullptr ? atoi(env) : 0;
  if (s <= 0) {
    if (world <= 2) return k;
    s = (2 * k + world - 1) / world;
    if (s < 256) s = 256;
  }
  return s < k ? (s < 1 ? 1 : s) : k;
}

// Whether a single-kernel step of `world` ranks first tries the exchange of survivors (every rank
// makes a guess for the whole row from its own shard and all finish from the same survivor list)
// before the exchange of sorted runs.  It needs the rows' own guesses (ff_topk_set_self_seed) and is
// not used when the caller carries guesses for the shards (those mean something else: a score
// between the SHARD's k-th and 4096-th largest).  Off unless FF_TOPK_CP_SX=1: on 4 GPUs it measured
// 21.9 us per step against 19.0 us with sorted runs (all 120 CTAs of a rank read every rank's regions,
// 14 MB through L2 per step); it is kept, exact and tested, for rows where ranking before the
// exchange costs more than here.  Every rank must decide alike, which they do when they make the
// same calls with the same settings.
int cp_survivor_exchange(int world, bool caller_hints, int k, int ctas_per_row) {
  if (world < 2 || caller_hints || !self_seed_enabled()) return 0;
  const char* on = getenv("FF_TOPK_CP_SX");
  if (on == nullptr || atoi(on) == 0) return 0;
  // a CTA's region takes kSxCap survivors: expected number plus six standard deviations must fit
  const double per_cta = 1.5 * k / (static_cast<double>(world) * ctas_per_row);
  if (ctas_per_row > ff::kSxRegions || per_cta + 6.0 * sqrt(per_cta) > ff::kSxCap) return 0;
  return 1;
}

// The parameter block of one rank's context-parallel send launch (shared by the real entry points
// and the several-ranks-in-one-launch test entry).  Returns 0 and the cluster size.
int cp_fill_params(FfCpExchange* ex, const float* scores, int64_t row_stride, const int32_t* lengths,
                   int64_t L_width, int64_t shard_offset, const float* hint_in, float* hint_out, void* workspace,
                   size_t workspace_bytes, int32_t* status, int device, ff::TopkParams* out, int* cluster_out);

// fused_out == nullptr: send only (the merge is a later launch).  Otherwise the launch
// merges too, if all its CTAs fit on the device together; *did_fuse tells.
int cp_send_impl(void* handle, const float* scores, int64_t row_stride, const int32_t* lengths,
                 int64_t L_width, int64_t shard_offset, const float* hint_in, float* hint_out,
                 void* workspace, size_t workspace_bytes, int32_t* status, void* stream, int32_t* fused_out,
                 bool* did_fuse) {
  if (did_fuse != nullptr) *did_fuse = false;
  if (handle == nullptr) return fail(FF_ERR_NULL, "exchange handle must not be NULL");
  FfCpExchange* ex = static_cast<FfCpExchange*>(handle);
  int device = 0;
  int rc = ensure_init(&device);
  if (rc != 0) return rc;
  ff::TopkParams p = {};
  int cluster = 1;
  rc = cp_fill_params(ex, scores, row_stride, lengths, L_width, shard_offset, hint_in, hint_out, workspace,
                      workspace_bytes, status, device, &p, &cluster);
  if (rc != 0) return rc;
  if (fused_out != nullptr && cp_fused_setting() != 0) {
    int log2c = 0;
    while ((1 << log2c) < cluster) ++log2c;
    const int64_t clusters = static_cast<int64_t>(ex->B) * (p.groups > 1 ? p.groups : 1);
    if (log2c < 5 && clusters <= g_active_clusters[device][log2c]) {
      p.push_fused = 1;
      p.push_prefix = cp_prefix(ex->world, ex->k);   // only a launch that merges itself can ask for the rest
      p.push_sx = cp_survivor_exchange(ex->world, hint_in != nullptr || hint_out != nullptr, ex->k,
                                       cluster * (p.groups > 1 ? p.groups : 1));
      p.out_idx = fused_out;
      if (did_fuse != nullptr) *did_fuse = true;
    }
  }
  return launch<false>(p, cluster, static_cast<cudaStream_t>(stream));
}

int cp_fill_params(FfCpExchange* ex, const float* scores, int64_t row_stride, const int32_t* lengths,
                   int64_t L_width, int64_t shard_offset, const float* hint_in, float* hint_out, void* workspace,
                   size_t workspace_bytes, int32_t* status, int device, ff::TopkParams* out, int* cluster_out) {
  for (int p = 0; p < ex->world; ++p)
    if (ex->peer[p] == nullptr) return fail(FF_ERR_NULL, "exchange: a peer is not mapped yet");
  // One launch: the shard-local select writes its candidates straight into the peers' receive
  // slots as self-validating entries (no separate push kernel, no flags).
  int rc = check_common(ex->B, L_width, ex->k);
  if (rc != 0) return rc;
  if (scores == nullptr || lengths == nullptr) return fail(FF_ERR_NULL, "scores and lengths must not be NULL");
  if (shard_offset < 0 || shard_offset + L_width > 0x7fffffffLL)
    return fail(FF_ERR_TOO_LARGE, "shard_offset + L_width exceeds int32 indices");
  ff::TopkParams p = {};
  p.scores = scores;
  p.row_stride = row_stride;
  p.lengths = lengths;
  p.out_idx = reinterpret_cast<int32_t*>(ex->base + ex->send_offset);   // unused in push mode
  p.out_val = reinterpret_cast<float*>(ex->base + ex->send_offset);     // non-null marks candidate mode
  p.B = ex->B;
  p.k = ex->k;
  p.L_width = L_width;
  p.shard_offset = shard_offset;
  p.fixed_len = -1;
  p.status = status;
  for (int q = 0; q < ff::kMaxPeers; ++q)
    p.push_peers.base[q] = static_cast<uint32_t*>(q < ex->world ? ex->peer[q] : nullptr);
  p.push_world = ex->world;
  p.push_rank = ex->rank;
  p.push_slot_words = static_cast<int64_t>(ex->slot_words);
  p.push_ctrl_offset = static_cast<int64_t>(ex->ctrl_offset);
  p.push_prefix = ex->k;   // a send whose merge is another launch delivers whole runs
  p.push_sx_offset = static_cast<int64_t>(ex->sx_offset);
  p.hint_in = hint_in;     // guesses of the shard-local threshold, as in ff_topk_launch_hinted
  p.hint_out = hint_out;
  int cluster = choose_cluster(device, ex->B, L_width, ex->k);
  if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0) {
    p.groups = choose_groups(device, ex->B, L_width, workspace_bytes, &cluster, hint_in != nullptr);
    p.workspace = static_cast<uint32_t*>(workspace);
  }
  *out = p;
  *cluster_out = cluster;
  return 0;
}

}  // namespace

extern "C" {

int ff_topk_cp_send(void* handle, const float* scores, int64_t row_stride, const int32_t* lengths,
                    int64_t L_width, int64_t shard_offset, void* workspace, size_t workspace_bytes,
                    int32_t* status, void* stream) {
  return cp_send_impl(handle, scores, row_stride, lengths, L_width, shard_offset, nullptr, nullptr, workspace,
                      workspace_bytes, status, stream, nullptr, nullptr);
}

int ff_topk_cp_send_hinted(void* handle, const float* scores, int64_t row_stride, const int32_t* lengths,
                           int64_t L_width, int64_t shard_offset, const float* hint_in, float* hint_out,
                           void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
  return cp_send_impl(handle, scores, row_stride, lengths, L_width, shard_offset, hint_in, hint_out, workspace,
                      workspace_bytes, status, stream, nullptr, nullptr);
}

int ff_topk_cp_recv_merge(void* handle, const int32_t* lengths, int32_t* out_idx, int32_t* status,
                          void* stream) {
  if (handle == nullptr || lengths == nullptr || out_idx == nullptr) return fail(FF_ERR_NULL, "NULL argument");
  FfCpExchange* ex = static_cast<FfCpExchange*>(handle);
  ff::CpMergeParams p = {};
  p.recv_even = ex->base;
  p.parity_words = static_cast<int64_t>(ex->world) * static_cast<int64_t>(ex->slot_words);
  p.slot_words = static_cast<int64_t>(ex->slot_words);
  p.ctrl = ex->base + ex->ctrl_offset;
  p.lengths = lengths;
  p.out_idx = out_idx;
  p.status = status;
  p.world = ex->world;
  p.B = ex->B;
  p.k = ex->k;
  const int n_cand = ex->world * ex->k;
  const dim3 grid((n_cand + 1023) / 1024, ex->B, 1);
  int sp = 1;
  while (sp < ex->k) sp *= 2;   // runs are staged at a power-of-two length
  const size_t key_bytes = static_cast<size_t>(ex->world) * sp * sizeof(uint32_t);   // <= 128 KiB
  ff::cp_merge_sorted_kernel<<<grid, 1024, key_bytes, static_cast<cudaStream_t>(stream)>>>(p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(e, "cp_merge_sorted_kernel");
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}

int ff_topk_cp_step(void* handle, const float* scores, int64_t row_stride, const int32_t* lengths,
                    int32_t* out_idx, int64_t L_width, int64_t shard_offset, void* workspace,
                    size_t workspace_bytes, int32_t* status, void* stream) {
  return ff_topk_cp_step_hinted(handle, scores, row_stride, lengths, out_idx, L_width, shard_offset, nullptr,
                                nullptr, workspace, workspace_bytes, status, stream);
}

int ff_topk_cp_step_emulated_ranks(int32_t n_ranks, void* const* handles, const float* const* scores,
                                   int64_t row_stride, const int32_t* lengths, int32_t* const* out_idx,
                                   const int64_t* L_width, const int64_t* shard_offset, float* const* hints,
                                   void* const* workspaces, size_t workspace_bytes, int32_t* status, void* stream) {
  if (n_ranks < 1 || n_ranks > ff::kMaxEmulatedRanks) return fail(FF_ERR_BAD_SHAPE, "n_ranks must be in [1, 8]");
  if (handles == nullptr || scores == nullptr || out_idx == nullptr || L_width == nullptr || shard_offset == nullptr)
    return fail(FF_ERR_NULL, "NULL argument");
  int device = 0;
  int rc = ensure_init(&device);
  if (rc != 0) return rc;
  static std::once_flag once;
  static cudaError_t prep = cudaSuccess;
  std::call_once(once, [] { prep = prepare_kernel(ff::topk_emulated_ranks_kernel<ff::kModePushHintedSx>); });
  if (prep != cudaSuccess) return fail_cuda(prep, "cudaFuncSetAttribute(topk_emulated_ranks_kernel)");
  ff::EmulatedRanks e = {};
  int cluster = 0, groups = 0;
  for (int r = 0; r < n_ranks; ++r) {
    FfCpExchange* ex = static_cast<FfCpExchange*>(handles[r]);
    if (ex == nullptr || ex->world != n_ranks || ex->rank != r) return fail(FF_ERR_BAD_SHAPE, "handles[r] must be rank r of n_ranks");
    int c = 1;
    float* hint = hints != nullptr ? hints[r] : nullptr;
    void* ws = workspaces != nullptr ? workspaces[r] : nullptr;
    rc = cp_fill_params(ex, scores[r], row_stride, lengths, L_width[r], shard_offset[r], hint, hint, ws,
                        ws != nullptr ? workspace_bytes : 0, status, device, &e.rank[r], &c);
    if (rc != 0) return rc;
    const int g = e.rank[r].groups > 1 ? e.rank[r].groups : 1;
    if (r == 0) {
      cluster = c;
      groups = g;
    } else if (c != cluster || g != groups) {
      return fail(FF_ERR_BAD_SHAPE, "emulated ranks need shards of one launch shape (force it with the overrides)");
    }
    e.rank[r].push_fused = 1;
    e.rank[r].push_prefix = cp_prefix(n_ranks, ex->k);
    e.rank[r].push_sx = cp_survivor_exchange(n_ranks, hint != nullptr, ex->k, c * g);
    e.rank[r].out_idx = out_idx[r];
    e.rank[r].trace = g_trace.load(std::memory_order_relaxed);
  }
  const int B = e.rank[0].B;
  const int per_rank = B * cluster * groups;
  int log2c = 0;
  while ((1 << log2c) < cluster) ++log2c;
  if (static_cast<int64_t>(n_ranks) * B * groups > g_active_clusters[device][log2c])
    return fail(FF_ERR_TOO_LARGE, "emulated ranks: the CTAs of all ranks must be resident at once");
  for (int r = 0; r < n_ranks; ++r) {
    e.rank[r].block_base = r * per_rank;
    e.rank[r].grid_ctas = per_rank;
  }
  e.ctas_per_rank = per_rank;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(n_ranks * per_rank), 1, 1);
  cfg.blockDim = dim3(ff::kThreads, 1, 1);
  cfg.dynamicSmemBytes = ff::smem_bytes_for(ff::kMaxStages);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeCooperative;   // the ranks' CTAs wait for one another
  attr[1].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  const cudaError_t err = cudaLaunchKernelEx(&cfg, ff::topk_emulated_ranks_kernel<ff::kModePushHintedSx>, e);
  if (err != cudaSuccess) return fail_cuda(err, "cudaLaunchKernelEx(topk_emulated_ranks_kernel)");
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}

int ff_topk_cp_step_hinted(void* handle, const float* scores, int64_t row_stride, const int32_t* lengths,
                           int32_t* out_idx, int64_t L_width, int64_t shard_offset, const float* hint_in,
                           float* hint_out, void* workspace, size_t workspace_bytes, int32_t* status,
                           void* stream) {
  if (out_idx == nullptr) return fail(FF_ERR_NULL, "out_idx must not be NULL");
  bool fused = false;
  const int rc = cp_send_impl(handle, scores, row_stride, lengths, L_width, shard_offset, hint_in, hint_out,
                              workspace, workspace_bytes, status, stream, out_idx, &fused);
  if (rc != 0 || fused) return rc;
  return ff_topk_cp_recv_merge(handle, lengths, out_idx, status, stream);
}

}  // extern "C"
