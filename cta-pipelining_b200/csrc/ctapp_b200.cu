// Host side of libctapp_b200.so: argument checking, tensor-map encoding, launches, and the small harness kernels.
// Every entry point is extern "C" with plain pointers and sizes; see include/ctapp_b200.h.
#include "../../include/ctapp_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "gemm_sm100.cuh"
#include "gemm2_sm100.cuh"
#include "reduce_sm100.cuh"

using namespace ctapp;

// ------------------------------------------------------------------------------------------ errors
static thread_local char g_err[512] = "";
static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
#define CU_OK(expr)                                                                                   \
  do {                                                                                                \
    cudaError_t e_ = (expr);                                                                          \
    if (e_ != cudaSuccess) return fail(static_cast<int>(e_), "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)
#define ARG(cond, ...)                           \
  do {                                           \
    if (!(cond)) return fail(-1, __VA_ARGS__);   \
  } while (0)

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    if (prev != dev) ok = cudaSetDevice(dev) == cudaSuccess;
  }
  ~DeviceGuard() {
    int cur = -1;
    if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
  }
};
#define GUARD(dev)   \
  DeviceGuard g_(dev); \
  if (!g_.ok) return fail(-2, "cannot select device %d", dev)

static std::atomic<long long> g_limit_ms{-1};   // entry points may be called from several host threads
static long long limit_ns() {
  long long ms = g_limit_ms.load(std::memory_order_relaxed);
  if (ms < 0) {
    const char* e = getenv("CTAPP_WAIT_LIMIT_MS");
    ms = e ? atoll(e) : 2000;
    if (ms <= 0) ms = 2000;
    g_limit_ms.store(ms, std::memory_order_relaxed);
  }
  return ms * 1000000ll;
}

// ------------------------------------------------------------------------------------------ driver entry points
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*StreamWaitValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

static void* driver_fn(const char* name) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
  return fn;
}

// bf16 row-major matrix (rows x cols, leading dimension ld elements), box box_cols x box_rows, 128-byte swizzle
static int make_tmap(CUtensorMap* tm, const void* base, long long rows, long long cols, long long ld, int box_cols, int box_rows,
                     bool swizzle128 = true) {
  static EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(driver_fn("cuTensorMapEncodeTiled"));
  if (!enc) return fail(-3, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return fail(-1, "matrix base %p is not 16-byte aligned", base);
  if ((ld * 2) % 16 != 0) return fail(-1, "leading dimension %lld is not a multiple of 8 elements", ld);
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-3, "cuTensorMapEncodeTiled failed with %d (rows %lld cols %lld ld %lld box %dx%d)", (int)r, rows, cols, ld, box_cols, box_rows);
  return 0;
}

// ------------------------------------------------------------------------------------------ configurations
// Reference ids 0-9 name wgmma tiles (64|128 x 128|256).  A 64-row UMMA tile has no place here (one CTA drives a
// 128-lane TMEM accumulator), so every id resolves to the 128-row tile with the same width.
// Ids 10 and up are this library's own: 10 = CTA pair (cta_group::2) working on a 256 x 256 tile, 11 = CTA pair on a
// 256 x 512 tile (single TMEM accumulator).
static int cfg_bn(int id) {
  switch (id) {
    case 0: case 1: case 5: case 7: return 128;
    case 2: case 3: case 4: case 6: case 8: case 9: case 10: return 256;
    case 11: return 512;
    default: return 0;
  }
}
static bool cfg_pair(int id) { return id == 10 || id == 11; }
static int sm_count(int dev) {
  static std::atomic<int> cache[64];
  if (dev < 0 || dev >= 64) return 0;
  int n = cache[dev].load(std::memory_order_relaxed);
  if (!n && cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) cache[dev].store(n, std::memory_order_relaxed);
  return n;
}
template <int BN> static int prepare_kernel() {
  CU_OK(cudaFuncSetAttribute(gemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::kSmemBytes));
  return 0;
}

static int launch_gemm(GemmParams& p, int bn, int sms, int pdl, int dev, cudaStream_t stream) {
  const int nsm = sm_count(dev);
  int grid = sms > 0 ? sms : nsm;
  if (grid > nsm) grid = nsm;
  if (grid > p.num_tiles) grid = p.num_tiles;
  if (grid < 1) return 0;   // nothing to do
  p.limit_ns = limit_ns();
  if (int r = bn == 256 ? prepare_kernel<256>() : prepare_kernel<128>()) return r;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = bn == 256 ? GemmCfg<256>::kSmemBytes : GemmCfg<128>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  if (bn == 256) CU_OK(cudaLaunchKernelEx(&cfg, gemm_kernel<256>, p));
  else CU_OK(cudaLaunchKernelEx(&cfg, gemm_kernel<128>, p));
  return 0;
}

// pair: the schedule's tile is 256 rows (two CTAs), and each CTA loads half of the B tile's rows
static int fill_common(GemmParams& p, const void* A, const void* B, int M, int N, int K, int bn, bool pair = false) {
  memset(&p, 0, sizeof(p));
  ARG(A && B, "null operand");
  ARG(M > 0 && N > 0 && K > 0, "bad shape M=%d N=%d K=%d", M, N, K);
  ARG(K % 8 == 0 && N % 8 == 0, "K=%d and N=%d must be multiples of 8", K, N);
  ARG(!pair || bn == 256 || bn == 512, "the CTA-pair kernel has 256- or 512-column tiles");
  p.M = M; p.N = N; p.K = K;
  p.panels = (M + BM - 1) / BM;
  p.tiles_m = pair ? (M + 2 * BM - 1) / (2 * BM) : p.panels;
  p.tiles_n = (N + bn - 1) / bn;
  p.num_tiles = p.tiles_m * p.tiles_n;
  if (int r = make_tmap(&p.tmA, A, M, K, K, BK, BM)) return r;
  if (int r = make_tmap(&p.tmB, B, N, K, K, BK, pair ? 128 : bn)) return r;   // pair: each CTA loads 128 weight rows per MMA
  return 0;
}

static int launch_gemm2(GemmParams& p, int sms, int pdl, int dev, cudaStream_t stream, bool wide = false) {
  const int nsm = sm_count(dev);
  int pairs = (sms > 0 && sms < nsm ? sms : nsm) / 2;
  if (pairs > p.num_tiles) pairs = p.num_tiles;
  if (pairs < 1) return 0;
  p.limit_ns = limit_ns();
  if (wide && p.act) return fail(-1, "the 256 x 512 tile has no activation epilogue");
  const unsigned smem = wide ? Gemm2CfgT<true>::kSmemBytes : Gemm2Cfg::kSmemBytes;
  CU_OK(cudaFuncSetAttribute(wide ? gemm2_kernel<false, true> : p.act ? gemm2_kernel<true> : gemm2_kernel<false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(wide ? Gemm2CfgT<true>::kThreads : Gemm2Cfg::kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  attr[na].id = cudaLaunchAttributeClusterDimension;
  attr[na].val.clusterDim.x = 2; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = 1;
  na++;
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    na++;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  if (wide) CU_OK(cudaLaunchKernelEx(&cfg, gemm2_kernel<false, true>, p));
  else if (p.act) CU_OK(cudaLaunchKernelEx(&cfg, gemm2_kernel<true>, p));
  else CU_OK(cudaLaunchKernelEx(&cfg, gemm2_kernel<false>, p));
  return 0;
}

// ------------------------------------------------------------------------------------------ small kernels
__global__ void chain_reset_kernel(Queue q, int* sb, const int* pristine, int sb_len, int* ready, int ready_value) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x, stride = gridDim.x * blockDim.x;
  if (q.entries) for (int k = i; k < q.cap; k += stride) q.entries[k] = -1;   // null: a pre-filled source queue keeps its ids and tail
  for (int k = i; k < sb_len; k += stride) sb[k] = pristine[k];
  if (i == 0) { *q.head = 0; if (q.entries) *q.tail = 0; }
  if (ready) {   // single CTA: everything above is ordered before the flag
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(ready, ready_value);
  }
}

template <int W> static int launch_reduce(const ReduceParams& p, int blocks, int threads, cudaStream_t s) {
  constexpr int R = RedRows<W>::value;
  if (p.partials_mc) tp_reduce_kernel<W, 4, true, true><<<blocks, threads, 0, s>>>(p);     // one reduced load per row: four rows in flight
  else if (p.x_mc) tp_reduce_kernel<W, R, true><<<blocks, threads, 0, s>>>(p);
  else tp_reduce_kernel<W, R><<<blocks, threads, 0, s>>>(p);
  CU_OK(cudaGetLastError());
  return 0;
}

__global__ void copy16_kernel(const int4* __restrict__ src, int4* __restrict__ dst, size_t n) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) dst[i] = src[i];
}

__global__ void stamp_kernel(unsigned long long* out) { *out = globaltimer(); }
__global__ void timer_reads_kernel(unsigned long long* out, int n) { for (int i = 0; i < n; i++) out[i] = globaltimer(); }

// A: t1; other = i; wait mine == i; t2.   B: wait mine == i; t; other = i.   Every wait is bounded.
__global__ void pingpong_kernel(int* mine, int* other, unsigned long long* out, int n, int is_a, int* status, long long limit) {
  for (int i = 1; i <= n; i++) {
    int seen;
    if (is_a) {
      const unsigned long long t1 = globaltimer();
      st_release_sys(other, i);
      if (!spin_acquire_sys(mine, PredEq{i}, limit, seen)) { report_status(status, kStatusTimeoutProbe, i, i, seen); return; }
      out[2 * (i - 1)] = t1; out[2 * (i - 1) + 1] = globaltimer();
    } else {
      if (!spin_acquire_sys(mine, PredEq{i}, limit, seen)) { report_status(status, kStatusTimeoutProbe, i, i, seen); return; }
      out[i - 1] = globaltimer();
      st_release_sys(other, i);
    }
  }
}

// ------------------------------------------------------------------------------------------ allocation-free reducer scratch
// Working memory of ctapp_tp_reduce_noalloc: the owner reducer's per-row accumulators (fp32) followed by its per-panel
// arrival counters (int32).  It lives in the library image, so every GPU that loads the library carries these
// 66 048 bytes until the process exits, and every call on a GPU shares them.
constexpr int kNoAllocMaxM = 16384;
constexpr size_t kNoAllocRowssBytes = static_cast<size_t>(kNoAllocMaxM) * sizeof(float);
constexpr size_t kNoAllocBytes = kNoAllocRowssBytes + (kNoAllocMaxM / 128) * sizeof(int);
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

// Device address of the scratch array on `device` (which must be current).  In host code the array's name is only a
// handle for the runtime, never an address a kernel could use; the address is asked for once per device and remembered.
static int noalloc_scratch_ptr(int device, unsigned char** out) {
  static std::mutex mu;
  static unsigned char* cache[64] = {};
  if (device < 0 || device >= 64) return fail(-1, "device index %d out of range", device);
  std::lock_guard<std::mutex> lock(mu);
  if (!cache[device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return fail(static_cast<int>(e), "cudaGetSymbolAddress(reducer scratch) on device %d: %s", device, cudaGetErrorString(e));
    cache[device] = static_cast<unsigned char*>(p);
  }
  *out = cache[device];
  return 0;
}

// Checks a reducer argument block and turns it into kernel parameters.  `own_scratch`: rowss_local / panel_done come from the
// caller (required); otherwise the caller of this function supplies them afterwards.
static int fill_reduce(const ctapp_tp_reduce_args* a, ReduceParams& p, bool own_scratch) {
  ARG(a, "null args");
  ARG(a->world == 1 || a->world == 2 || a->world == 4 || a->world == 8, "world %d is not supported (1 | 2 | 4 | 8)", a->world);
  ARG(a->rank >= 0 && a->rank < a->world, "bad rank %d", a->rank);
  ARG(a->M >= 0 && a->M % 128 == 0 && a->n1 > 0 && a->n1 % 256 == 0, "bad shape M=%d n1=%d", a->M, a->n1);
  ARG(a->tile_flags, "null tile_flags");
  ARG(!own_scratch || (a->rowss_local && a->panel_done), "null rowss_local / panel_done");
  ARG(a->tail_cols >= 0 && a->tail_cols <= a->n1 / 256, "bad tail_cols %d", a->tail_cols);
  ARG(a->order >= 0 && a->order <= 2 && a->swz >= 0, "bad unit order %d / swz %d", a->order, a->swz);
  // flags are indexed (source * panels_per_owner + owned panel): a smaller value than the panels this rank owns would make
  // the sources' flags alias each other, a larger one than the allocation reads out of bounds (the caller's to guarantee)
  ARG(a->panels_per_owner >= (a->M / 128 + a->world - 1) / a->world, "panels_per_owner %d is too small for M=%d on %d ranks (needs >= %d)",
      a->panels_per_owner, a->M, a->world, (a->M / 128 + a->world - 1) / a->world);
  memset(&p, 0, sizeof(p));
  p.M = a->M; p.n1 = a->n1; p.rank = a->rank; p.world = a->world;
  p.epoch = a->epoch; p.epoch_ptr = a->epoch_dev;
  p.tile_flags = a->tile_flags;
  for (int d = 0; d < a->world; d++) {
    ARG(a->inbox[d] && a->peer_x[d] && a->peer_rowss[d] && a->peer_panel_flag[d], "missing peer buffer %d", d);
    p.inbox[d] = static_cast<const uint4*>(a->inbox[d]);
    p.x[d] = static_cast<uint4*>(a->peer_x[d]);
    p.rowss[d] = a->peer_rowss[d];
    p.panel_flag[d] = a->peer_panel_flag[d];
  }
  p.resid = static_cast<const uint4*>(a->resid);
  p.rowss_local = a->rowss_local; p.panel_done = a->panel_done;
  p.ppo = a->panels_per_owner; p.tail = a->tail_cols;
  p.order = a->order ? a->order : 1; p.swz = a->swz;
  p.unit_ctr = a->unit_ctr; p.unit_log = a->unit_log; p.trace = a->trace; p.status = a->status;
  p.pdl_trigger = a->pdl_trigger; p.help_all = a->help_all;
  ARG(a->role_r >= 0 && a->role_r <= 1024 && (a->role_r == 0 || (a->role_ctr && !a->unit_ctr)),
      "role switching: role_r %d needs role_ctr and static unit shares (unit_ctr NULL)", a->role_r);
  p.role_ctr = a->role_r > 0 ? a->role_ctr : nullptr; p.role_r = a->role_r;
  if (a->x_mc || a->rowss_mc || a->panel_flag_mc) {   // NVLS variant: all three multicast addresses or none
    ARG(a->x_mc && a->rowss_mc && a->panel_flag_mc, "the NVLS variant needs x_mc, rowss_mc and panel_flag_mc");
    ARG(a->world >= 2, "the NVLS variant needs at least 2 ranks");
    p.x_mc = static_cast<uint4*>(a->x_mc); p.rowss_mc = a->rowss_mc; p.panel_flag_mc = a->panel_flag_mc;
  }
  if (a->partials_mc) {
    ARG(p.x_mc, "the in-switch reduction (partials_mc) needs the NVLS pushes too (x_mc, rowss_mc, panel_flag_mc)");
    ARG((!a->unit_ctr || !a->help_all) && !a->role_r, "the in-switch reduction is not available to helping consumer CTAs");
    p.partials_mc = static_cast<const uint4*>(a->partials_mc);
  }
  p.limit_ns = limit_ns();
  return 0;
}

static int launch_reduce_any(const ReduceParams& p, int blocks, int threads, cudaStream_t s) {
  switch (p.world) {
    case 1: return launch_reduce<1>(p, blocks, threads, s);
    case 2: return launch_reduce<2>(p, blocks, threads, s);
    case 4: return launch_reduce<4>(p, blocks, threads, s);
    default: return launch_reduce<8>(p, blocks, threads, s);
  }
}

extern "C" {

const char* ctapp_last_error(void) { return g_err; }
int ctapp_abi_version(void) { return 5; }   // 3: k-chunk flags in ctapp_chain_args; order / swz / unit_log / pdl_trigger in ctapp_tp_reduce_args (tma gone); red in ctapp_tp_qkv_args; tile_log in ctapp_tp_down_args
int ctapp_set_wait_limit_ms(int ms) {
  ARG(ms > 0, "limit must be positive");
  g_limit_ms = ms;
  return 0;
}
int ctapp_get_wait_limit_ms(void) { return static_cast<int>(limit_ns() / 1000000ll); }

int ctapp_config_info(int config_id, char* buf, int buf_len) {
  const int bn = cfg_bn(config_id);
  ARG(bn && buf && buf_len > 0, "bad config_id %d", config_id);
  if (cfg_pair(config_id)) {
    const bool wide = bn == 512;
    snprintf(buf, buf_len, "tcgen05 cta_group::2 tma-store-epi tile %dx%dx%d threads=%d smem=%u stages=%d tmem_cols=512 cluster=2", 2 * BM, bn, BK,
             wide ? Gemm2CfgT<true>::kThreads : Gemm2Cfg::kThreads, wide ? Gemm2CfgT<true>::kSmemBytes : Gemm2Cfg::kSmemBytes, wide ? Gemm2CfgT<true>::kStages : Gemm2Cfg::kStages);
    return 0;
  }
  const int stages = bn == 256 ? GemmCfg<256>::kStages : GemmCfg<128>::kStages;
  const unsigned smem = bn == 256 ? GemmCfg<256>::kSmemBytes : GemmCfg<128>::kSmemBytes;
  snprintf(buf, buf_len, "tcgen05 tma-store-epi tile %dx%dx%d threads=%d smem=%u stages=%d tmem_cols=%d", BM, bn, BK, kThreads, smem, stages, 2 * bn);
  return 0;
}
int ctapp_occupancy(int config_id) { return cfg_bn(config_id) ? 1 : fail(-1, "bad config_id %d", config_id); }

int ctapp_cluster_occupancy(int cluster_size, int device) {
  if (cluster_size < 1 || cluster_size > 16) return fail(-1, "bad cluster size %d", cluster_size);
  DeviceGuard g_(device);
  if (!g_.ok) return fail(-2, "cannot select device %d", device);
  cudaError_t e = cudaFuncSetAttribute(gemm2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Gemm2Cfg::kSmemBytes);
  if (e == cudaSuccess && cluster_size > 8) e = cudaFuncSetAttribute(gemm2_kernel<false>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  if (e != cudaSuccess) return fail(-static_cast<int>(e) - 100, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(sm_count(device) / cluster_size * cluster_size);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = Gemm2Cfg::kSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_size; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  e = cudaOccupancyMaxActiveClusters(&n, gemm2_kernel<false>, &cfg);
  if (e != cudaSuccess) return fail(-static_cast<int>(e) - 100, "cudaOccupancyMaxActiveClusters: %s", cudaGetErrorString(e));
  return n;
}

int ctapp_kernel_info(int which, char* buf, int buf_len) {
  ARG(buf && buf_len > 0, "null buffer");
  cudaFuncAttributes a;
  const void* fn = which == 0 ? (const void*)gemm_kernel<256> : which == 1 ? (const void*)gemm_kernel<128> : which == 3 ? (const void*)gemm2_kernel<false> : which == 4 ? (const void*)gemm2_kernel<true> : which == 5 ? (const void*)gemm2_kernel<false, true> : (const void*)tp_reduce_kernel<4, RedRows<4>::value>;
  CU_OK(cudaFuncGetAttributes(&a, fn));
  snprintf(buf, buf_len, "regs=%d local=%zu static_smem=%zu max_threads=%d", a.numRegs, a.localSizeBytes, a.sharedSizeBytes, a.maxThreadsPerBlock);
  return 0;
}

int ctapp_preload(int device) {
  GUARD(device);
  cudaFuncAttributes a;
  CU_OK(cudaFuncGetAttributes(&a, gemm_kernel<256>));
  CU_OK(cudaFuncGetAttributes(&a, gemm_kernel<128>));
  CU_OK(cudaFuncGetAttributes(&a, tp_reduce_kernel<1, RedRows<1>::value>));
  CU_OK(cudaFuncGetAttributes(&a, tp_reduce_kernel<2, RedRows<2>::value>));
  CU_OK(cudaFuncGetAttributes(&a, tp_reduce_kernel<4, RedRows<4>::value>));
  CU_OK(cudaFuncGetAttributes(&a, tp_reduce_kernel<8, RedRows<8>::value>));
  CU_OK(cudaFuncGetAttributes(&a, tp_reduce_kernel<2, RedRows<2>::value, true>));
  CU_OK(cudaFuncGetAttributes(&a, tp_reduce_kernel<4, RedRows<4>::value, true>));
  CU_OK(cudaFuncGetAttributes(&a, tp_reduce_kernel<8, RedRows<8>::value, true>));
  CU_OK(cudaFuncGetAttributes(&a, tp_reduce_kernel<2, 4, true, true>));
  CU_OK(cudaFuncGetAttributes(&a, tp_reduce_kernel<4, 4, true, true>));
  CU_OK(cudaFuncGetAttributes(&a, tp_reduce_kernel<8, 4, true, true>));
  CU_OK(cudaFuncGetAttributes(&a, tp_step_kernel));
  CU_OK(cudaFuncGetAttributes(&a, add_rmsnorm_kernel));
  CU_OK(cudaFuncGetAttributes(&a, gemm2_kernel<false>));
  CU_OK(cudaFuncGetAttributes(&a, gemm2_kernel<true>));
  CU_OK(cudaFuncGetAttributes(&a, gemm2_kernel<false, true>));
  CU_OK(cudaFuncGetAttributes(&a, silu_mul_kernel));
  CU_OK(cudaFuncGetAttributes(&a, chain_reset_kernel));
  unsigned char* scratch = nullptr;   // the allocation-free reducer's scratch address, so that its first call does no set-up either
  if (int r = noalloc_scratch_ptr(device, &scratch)) return r;
  if (int r = prepare_kernel<256>()) return r;
  if (int r = prepare_kernel<128>()) return r;
  CU_OK(cudaFuncSetAttribute(gemm2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Gemm2Cfg::kSmemBytes));
  CU_OK(cudaFuncSetAttribute(gemm2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Gemm2Cfg::kSmemBytes));
  CU_OK(cudaFuncSetAttribute(gemm2_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Gemm2CfgT<true>::kSmemBytes));
  return 0;
}

// ------------------------------------------------------------------------------------------ GEMM entry points
int ctapp_gemm(const void* X, const void* W, void* Y, int M, int N, int K, int config_id, int group_rows, int sms, int device, void* stream) {
  const int bn = cfg_bn(config_id);
  ARG(bn, "bad config_id %d", config_id);
  ARG(Y, "null output");
  GUARD(device);
  const bool pair = cfg_pair(config_id);
  GemmParams p;
  if (int r = fill_common(p, X, W, M, N, K, bn, pair)) return r;
  if (int r = make_tmap(&p.tmD[0], Y, M, N, N, kStoreCols, kStageRows)) return r;
  p.mode = kModePlain;
  p.order = kOrderGrouped;
  p.group_rows = group_rows > 0 ? group_rows : (pair ? 8 : 16);
  if (pair) return launch_gemm2(p, sms, 0, device, static_cast<cudaStream_t>(stream), bn == 512);
  return launch_gemm(p, bn, sms, 0, device, static_cast<cudaStream_t>(stream));
}

int ctapp_chain_gemm(const void* X, const void* W, void* Y, int M, int N, int K, int config_id, const ctapp_chain_args* a, int device, void* stream) {
  const int bn = cfg_bn(config_id);
  ARG(bn, "bad config_id %d", config_id);
  ARG(a && Y, "null argument");
  GUARD(device);
  const bool pair = cfg_pair(config_id);
  GemmParams p;
  if (int r = fill_common(p, X, W, M, N, K, bn, pair)) return r;
  ARG(a->src.entries && a->src.head && a->src.tail, "source queue pointers are required");
  ARG(a->src.cap == p.num_tiles, "source queue capacity %d != number of tiles %d", a->src.cap, p.num_tiles);
  ARG(a->tiles_n == p.tiles_n, "tiles_n %d does not match N=%d with tile width %d", a->tiles_n, N, bn);
  if (a->dep_offsets) {
    ARG(a->dep_consumers && a->scoreboard, "dep_consumers and scoreboard are required with dep_offsets");
    ARG(a->dst.entries && a->dst.tail && a->dst.cap > 0, "downstream queue is required with dep_offsets");
    ARG(!a->rowpanel || a->tiles_n2 > 0, "tiles_n2 is required in row-panel mode");
  }
  ARG(a->fence >= 0 && a->fence <= 3, "bad fence mode %d", a->fence);
  if (int r = make_tmap(&p.tmD[0], Y, M, N, N, kStoreCols, kStageRows)) return r;
  p.mode = kModeChain;
  p.src = Queue{a->src.entries, a->src.head, a->src.tail, a->src.cap};
  p.dep_offsets = a->dep_offsets; p.dep_consumers = a->dep_consumers; p.scoreboard = a->scoreboard;
  p.dst = Queue{a->dst.entries, a->dst.head, a->dst.tail, a->dst.cap};
  p.tiles_n2 = a->tiles_n2; p.rowpanel = a->rowpanel; p.skip_wait = a->skip_wait;
  ARG(a->src_group >= 0 && a->src_group <= 1024, "bad src_group %d", a->src_group);
  p.src_group = a->src_group;
  ARG(!a->src_windows || a->n_windows > 0, "src_windows needs n_windows > 0");
  p.src_windows = a->src_windows; p.n_windows = a->src_windows ? a->n_windows : 0;
  p.dst_ready = (a->dep_offsets || a->chunk_dst) ? a->dst_ready : nullptr; p.ready_value = a->ready_value;
  if (a->chunk_src) {
    ARG(a->chunk_kblocks > 0 && a->chunk_cols > 0 && a->chunk_cols * a->chunk_kblocks * BK >= K, "k-chunk flags: %d chunks of %d k-blocks do not cover K=%d",
        a->chunk_cols, a->chunk_kblocks, K);
    p.chunk_src = a->chunk_src; p.chunk_kblocks = a->chunk_kblocks; p.chunk_cols = a->chunk_cols;
  }
  p.chunk_dst = a->chunk_dst; p.chunk_value = a->chunk_value;
  p.status = a->status; p.stamps = a->stamps;
  if (pair) return launch_gemm2(p, a->sms, 0, device, static_cast<cudaStream_t>(stream), bn == 512);
  return launch_gemm(p, bn, a->sms, 0, device, static_cast<cudaStream_t>(stream));
}

int ctapp_chain_reset(ctapp_queue q, int* scoreboard, const int* pristine, int sb_len, int* ready_flag, int ready_value, int device, void* stream) {
  ARG(q.head && (!q.entries || (q.tail && q.cap > 0)), "bad queue");
  ARG(sb_len == 0 || (scoreboard && pristine), "scoreboard pointers are required when scoreboard_len > 0");
  GUARD(device);
  chain_reset_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(Queue{q.entries, q.head, q.tail, q.cap}, scoreboard, pristine, sb_len, ready_flag, ready_value);
  CU_OK(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------------ tensor-parallel boundary
int ctapp_tp_down(const ctapp_tp_down_args* a, int device, void* stream) {
  ARG(a, "null args");
  ARG(a->mode == 0 || a->mode == 7, "tp_down mode %d is not supported (0 | 7)", a->mode);
  ARG(a->world >= 1 && a->world <= CTAPP_MAX_WORLD && a->rank >= 0 && a->rank < a->world, "bad rank %d / world %d", a->rank, a->world);
  GUARD(device);
  const bool pair = a->cta_pair != 0, wide = a->cta_pair == 2;     // 2: CTA pairs on 256 x 512 tiles (two tile flags per tile)
  ARG(a->cta_pair >= 0 && a->cta_pair <= 2, "bad cta_pair %d", a->cta_pair);
  GemmParams p;
  if (int r = fill_common(p, a->A, a->W, a->M, a->N, a->K, wide ? 512 : 256, pair)) return r;
  ARG(a->N % (wide ? 512 : 256) == 0, "N=%d must be a multiple of %d", a->N, wide ? 512 : 256);
  p.status = a->status; p.stamps = a->trace; p.tile_log = a->tile_log;
  // mode 7 launched as a programmatic dependent follows the owner reducer, which waits for THIS kernel's tiles: it must not
  // wait for that grid to finish (the step kernel before the reducer has completed by then: stream order)
  p.pdl_trigger = a->pdl_trigger; p.pdl_wait = a->mode == 7 ? 0 : a->pdl;
  p.epoch = a->epoch; p.epoch_ptr = a->epoch_dev;
  if (a->raster == 2) p.order = kOrderNFast;
  else {
    ARG(a->tail_cols >= 0 && a->tail_cols <= a->N / 256, "bad tail_cols %d", a->tail_cols);
    p.order = kOrderMFastTail; p.tail_cols = wide ? a->tail_cols / 2 : a->tail_cols;      // tail_cols counts 256-column tiles
  }
  if (a->mode == 0) {
    ARG(a->D, "mode 0 needs D");
    if (int r = make_tmap(&p.tmD[0], a->D, a->M, a->N, a->N, kStoreCols, kStageRows)) return r;
    p.mode = kModePlain;
  } else {
    ARG(a->M % 128 == 0, "mode 7 needs M %% 128 == 0 (M=%d)", a->M);
    ARG(a->dst_rows >= ((a->M / 128 + a->world - 1) / a->world) * 128 && a->panels_per_owner * 128 <= a->dst_rows &&
            a->panels_per_owner >= (a->M / 128 + a->world - 1) / a->world,
        "inbox slot of %d rows / %d panels per owner does not fit M=%d on %d ranks (panels_per_owner must be >= ceil(M/128/world) and its rows <= dst_rows)",
        a->dst_rows, a->panels_per_owner, a->M, a->world);
    ARG(!a->dst_global || a->dst_rows >= a->M, "dst_global: every destination must hold all M=%d rows (dst_rows %d)", a->M, a->dst_rows);
    p.mode = kModeTpProducer; p.dst_global = a->dst_global != 0;
    p.world = a->world; p.rank = a->rank; p.ppo = a->panels_per_owner;
    for (int d = 0; d < a->world; d++) {
      ARG(a->dst_ptrs[d] && a->peer_tile_flags[d], "missing destination %d", d);
      if (int r = make_tmap(&p.tmD[d], a->dst_ptrs[d], a->dst_rows, a->N, a->N, kStoreCols, kStageRows)) return r;
      p.peer_tile_flags[d] = a->peer_tile_flags[d];
    }
  }
  if (pair) return launch_gemm2(p, a->sms, a->pdl, device, static_cast<cudaStream_t>(stream), wide);
  return launch_gemm(p, 256, a->sms, a->pdl, device, static_cast<cudaStream_t>(stream));
}

int ctapp_tp_qkv(const ctapp_tp_qkv_args* a, int device, void* stream) {
  ARG(a, "null args");
  ARG(a->mode == 0 || a->mode == 5 || a->mode == 8, "tp_qkv mode %d is not supported (0 | 5 | 8)", a->mode);
  ARG((a->mode == 8) == (a->red != nullptr), "mode 8 (the consumer's CTAs help the owner reducer) needs red, the other modes take none");
  ARG(a->tile == 256 || a->tile == 128 || a->tile == 0, "bad tile %d", a->tile);
  const int bn = a->tile == 128 ? 128 : 256;
  const bool pair = a->cta_pair != 0 && bn == 256;
  GUARD(device);
  GemmParams p;
  if (int r = fill_common(p, a->X, a->W, a->M, a->N, a->K, bn, pair)) return r;
  ARG(a->Y, "null output");
  ARG(a->act == 0 || a->act == 1, "bad act %d", a->act);
  ARG(!a->act || (pair && a->N % 256 == 0), "act needs the CTA-pair kernel and N %% 256 == 0 (N=%d)", a->N);
  const int ncols = a->act ? a->N / 2 : a->N;      // act: silu(gate) * up, 128 output columns per 256-column tile
  if (int r = make_tmap(&p.tmD[0], a->Y, a->M, ncols, ncols, kStoreCols, kStageRows)) return r;
  p.act = a->act;
  p.status = a->status; p.stamps = a->trace;
  p.epoch = a->epoch; p.epoch_ptr = a->epoch_dev;
  // raster 2: n fastest (panel by panel); 3: groups of `swizzle` tile rows, n-major inside a group (wide outputs: keeps a
  // weight panel in L2 across the group's rows); otherwise m fastest
  p.order = a->raster == 2 ? kOrderNFast : a->raster == 3 ? kOrderGrouped : kOrderMFastTail;
  p.group_rows = a->swizzle > 0 ? a->swizzle : 1;
  p.tail_cols = 0;
  p.rowss = a->rowss; p.inv_k = 1.0f / static_cast<float>(a->K); p.eps = a->eps;
  if (a->mode == 5 || a->mode == 8) {
    ARG(a->panel_flag, "mode %d needs panel_flag", a->mode);
    p.mode = kModeTpConsumer; p.panel_flag = a->panel_flag;
    p.pdl_wait = 0;            // the per-panel flags carry the dependency on the producer grid
    if (a->mode == 8) {
      if (int r = fill_reduce(a->red, p.red, true)) return r;
      ARG(p.red.unit_ctr || p.red.role_r > 0, "mode 8 needs red->unit_ctr (units shared out through that counter) or red->role_r > 0 (role switching)");
      ARG(!p.red.partials_mc, "mode 8: helping consumer CTAs read the inbox; the in-switch reduction (red->partials_mc) has no inbox");
      ARG(p.red.M == a->M && p.red.n1 == a->K, "mode 8: the reducer's shape (M=%d, n1=%d) must be this GEMM's (M=%d, K=%d)", p.red.M, p.red.n1, a->M, a->K);
      if (p.red.role_r > 0) {   // every static share needs a CTA: a launch of fewer CTAs than role_r splits the units among those it has
        const int nsm = sm_count(device);
        int ctas = a->sms > 0 && a->sms < nsm ? a->sms : nsm;
        if (pair) ctas = 2 * (ctas / 2 < p.num_tiles ? ctas / 2 : p.num_tiles); else if (ctas > p.num_tiles) ctas = p.num_tiles;
        if (p.red.role_r > ctas) p.red.role_r = ctas;
      }
    }
  } else {
    p.mode = a->rowss ? kModeTpConsumer : kModePlain;   // mode 0 with rowss: scale only, no waits
    p.panel_flag = nullptr;
    p.pdl_wait = a->pdl;
  }
  if (pair) return launch_gemm2(p, a->sms, a->pdl, device, static_cast<cudaStream_t>(stream));
  return launch_gemm(p, bn, a->sms, a->pdl, device, static_cast<cudaStream_t>(stream));
}

int ctapp_tp_reduce(const ctapp_tp_reduce_args* a, int device, void* stream) {
  ReduceParams p;
  if (int r = fill_reduce(a, p, true)) return r;
  ARG(a->threads >= 32 && a->threads <= 1024 && a->threads % 32 == 0 && a->blocks >= 1, "bad launch shape %d x %d", a->blocks, a->threads);
  GUARD(device);
  if (a->M == 0) return 0;
  return launch_reduce_any(p, a->blocks, a->threads, static_cast<cudaStream_t>(stream));
}

// The owner reducer for hosts that must not allocate device memory: same inputs, outputs and results as ctapp_tp_reduce,
// but the per-step working memory (row accumulators, panel arrival counters) is the library's own fixed array instead of
// caller buffers, and this call clears it itself.  Nothing here allocates: two cudaMemsetAsync and one launch (plus one
// cudaGetSymbolAddress per device on the first call, unless ctapp_preload has already run there).
int ctapp_tp_reduce_noalloc(const ctapp_tp_reduce_args* a, int device, void* stream) {
  ARG(a, "null args");
  ARG(a->M <= kNoAllocMaxM, "M=%d is beyond the built-in scratch of ctapp_tp_reduce_noalloc (at most %d rows); use ctapp_tp_reduce with caller buffers",
      a->M, kNoAllocMaxM);
  // what this variant does not do is refused, not dropped: a caller that set one of these would get other behaviour than it asked for
  ARG(!a->x_mc && !a->rowss_mc && !a->panel_flag_mc && !a->partials_mc,
      "ctapp_tp_reduce_noalloc pushes with unicast stores only: x_mc / rowss_mc / panel_flag_mc / partials_mc must be NULL");
  ARG(!a->unit_ctr && !a->unit_log && !a->pdl_trigger && !a->help_all && !a->role_r,
      "ctapp_tp_reduce_noalloc assigns units statically: unit_ctr / unit_log must be NULL, pdl_trigger, help_all and role_r 0");
  ReduceParams p;
  if (int r = fill_reduce(a, p, false)) return r;
  ARG(a->threads >= 32 && a->threads <= 1024 && a->threads % 32 == 0 && a->blocks >= 1, "bad launch shape %d x %d", a->blocks, a->threads);
  GUARD(device);
  unsigned char* scratch = nullptr;
  if (int r = noalloc_scratch_ptr(device, &scratch)) return r;
  p.rowss_local = reinterpret_cast<float*>(scratch);
  p.panel_done = reinterpret_cast<int*>(scratch + kNoAllocRowssBytes);
  if (a->M == 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the array keeps whatever the previous call left: the accumulators and counters of this step's rows start from zero
  CU_OK(cudaMemsetAsync(p.rowss_local, 0, static_cast<size_t>(a->M) * sizeof(float), s));
  CU_OK(cudaMemsetAsync(p.panel_done, 0, static_cast<size_t>(a->M / 128) * sizeof(int), s));
  return launch_reduce_any(p, a->blocks, a->threads, s);
}

// ------------------------------------------------------------------------------------------ read-back of the device-side integer maps
int ctapp_debug_tile_order(int order, int tiles_m, int tiles_n, int group_rows, int tail_cols, int* out_mn, int device, void* stream) {
  ARG(order >= 0 && order <= 2 && tiles_m > 0 && tiles_n > 0 && out_mn, "bad arguments");
  ARG(tail_cols >= 0 && tail_cols <= tiles_n, "bad tail_cols %d", tail_cols);
  GUARD(device);
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.tiles_m = tiles_m; p.tiles_n = tiles_n; p.num_tiles = tiles_m * tiles_n;
  p.order = order; p.group_rows = group_rows; p.tail_cols = tail_cols;
  tile_order_kernel<<<(p.num_tiles + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(p, out_mn);
  CU_OK(cudaGetLastError());
  return 0;
}
int ctapp_debug_unit_order(int owned_panels, int tiles_n, int tail_cols, int order, int swz, int* out_jnq, int device, void* stream) {
  ARG(owned_panels > 0 && tiles_n > 0 && tail_cols >= 0 && tail_cols <= tiles_n && (order == 1 || order == 2) && swz >= 0 && out_jnq, "bad arguments");
  GUARD(device);
  const int U = owned_panels * tiles_n * 4;
  unit_order_kernel<<<(U + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(owned_panels, tiles_n, tail_cols, order, swz, out_jnq);
  CU_OK(cudaGetLastError());
  return 0;
}
int ctapp_debug_queue_slots(int num_tiles, int tiles_n, int src_group, const int* src_windows, int n_windows, int* out_slots, int device, void* stream) {
  ARG(num_tiles > 0 && tiles_n > 0 && num_tiles % tiles_n == 0 && out_slots, "bad arguments");
  GUARD(device);
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.tiles_n = tiles_n; p.num_tiles = num_tiles; p.src.cap = num_tiles;
  p.src_group = src_group; p.src_windows = src_windows; p.n_windows = src_windows ? n_windows : 0;
  queue_slot_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p, out_slots);
  CU_OK(cudaGetLastError());
  return 0;
}

int ctapp_tp_step(int* epoch_dev, float* rowss_local, int* panel_done, int M, int* role_ctr, int device, void* stream) {
  ARG(epoch_dev && rowss_local && panel_done && M >= 0 && M % 128 == 0, "bad arguments");
  GUARD(device);
  int blocks = (M / 4 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 64) blocks = 64;
  tp_step_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(epoch_dev, reinterpret_cast<float4*>(rowss_local), panel_done, M, role_ctr);
  CU_OK(cudaGetLastError());
  return 0;
}

int ctapp_add_rmsnorm(const void* a, const void* resid, const void* gamma, void* x_out, void* y_out, int M, int n1, float eps, int device, void* stream) {
  ARG(a && gamma && y_out && M > 0 && n1 > 0 && n1 % 8 == 0 && n1 <= 16384, "bad arguments");
  GUARD(device);
  add_rmsnorm_kernel<<<M, 256, n1 * 2, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(a), static_cast<const uint4*>(resid), static_cast<const uint4*>(gamma),
                                                                           static_cast<uint4*>(x_out), static_cast<uint4*>(y_out), n1, eps);
  CU_OK(cudaGetLastError());
  return 0;
}

int ctapp_silu_mul(const void* in, void* out, int M, int I, int device, void* stream) {
  ARG(in && out && M > 0 && I > 0 && I % 8 == 0, "bad arguments (M=%d I=%d)", M, I);
  ARG(((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0, "buffers must be 16-byte aligned");
  GUARD(device);
  const long long total = static_cast<long long>(M) * (I / 8);
  const int blocks = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  silu_mul_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(in), static_cast<uint4*>(out), M, I);
  CU_OK(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------------ NVLS probes
int ctapp_mm_red_u32(void* mc, int n, unsigned v, int device, void* stream) {
  ARG(mc && n > 0, "bad arguments");
  GUARD(device);
  mm_red_u32_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<unsigned*>(mc), n, v);
  CU_OK(cudaGetLastError());
  return 0;
}
int ctapp_mm_red_f32(void* mc, const float* src, int n, int device, void* stream) {
  ARG(mc && src && n > 0, "bad arguments");
  GUARD(device);
  mm_red_f32_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<float*>(mc), src, n);
  CU_OK(cudaGetLastError());
  return 0;
}
int ctapp_mm_st_bf16(void* mc, const void* src, int n, int device, void* stream) {
  ARG(mc && src && n > 0 && n % 8 == 0, "bad arguments (n must be a multiple of 8 bf16)");
  GUARD(device);
  mm_st_bf16_kernel<<<(n / 8 + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint4*>(mc), static_cast<const uint4*>(src), n / 8);
  CU_OK(cudaGetLastError());
  return 0;
}
int ctapp_mm_ld_reduce_bf16(const void* mc, void* out, int n, int device, void* stream) {
  ARG(mc && out && n > 0 && n % 8 == 0, "bad arguments (n must be a multiple of 8 bf16)");
  GUARD(device);
  mm_ld_reduce_bf16_kernel<<<(n / 8 + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(mc), static_cast<uint4*>(out), n / 8);
  CU_OK(cudaGetLastError());
  return 0;
}
int ctapp_mm_order_stress(void* data_mc, const void* data_local, int* flag_mc, const int* flag_local, unsigned* ack_mc, const unsigned* ack_local,
                          int rank, int world, int iters, int slots, int* result, int device, void* stream) {
  ARG(data_mc && data_local && flag_mc && flag_local && ack_mc && ack_local && result, "null buffer");
  ARG(world >= 2 && rank >= 0 && rank < world && iters > 0 && slots > 0 && slots <= 128, "bad arguments");
  GUARD(device);
  mm_order_stress_kernel<<<slots, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint4*>(data_mc), static_cast<const uint4*>(data_local), flag_mc,
                                                                            flag_local, ack_mc, ack_local, rank, world, iters, result, limit_ns());
  CU_OK(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------------ harness natives
int ctapp_enable_peer_access(int device, int peer) {
  GUARD(device);
  int can = 0;
  CU_OK(cudaDeviceCanAccessPeer(&can, device, peer));
  ARG(can, "device %d cannot access device %d", device, peer);
  cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return 0; }
  CU_OK(e);
  return 0;
}

static volatile int* g_gate = nullptr;
static CUdeviceptr g_gate_dev = 0;
int ctapp_gate_alloc(void) {
  if (g_gate) return 0;
  void *h, *d;
  CU_OK(cudaHostAlloc(&h, sizeof(int), cudaHostAllocPortable | cudaHostAllocMapped));
  CU_OK(cudaHostGetDevicePointer(&d, h, 0));
  g_gate = static_cast<volatile int*>(h);
  g_gate_dev = reinterpret_cast<CUdeviceptr>(d);
  *g_gate = 0;
  return 0;
}
int ctapp_gate_set(int value) {
  ARG(g_gate, "gate_alloc has not been called");
  *g_gate = value;
  return 0;
}
int ctapp_gate_wait(int device, void* stream) {
  ARG(g_gate, "gate_alloc has not been called");
  static StreamWaitValue32Fn fn = reinterpret_cast<StreamWaitValue32Fn>(driver_fn("cuStreamWaitValue32"));
  ARG(fn, "cuStreamWaitValue32 is not available from this driver");
  GUARD(device);
  CUresult r = fn(static_cast<CUstream>(stream), g_gate_dev, 1, CU_STREAM_WAIT_VALUE_GEQ);
  if (r != CUDA_SUCCESS) return fail(-3, "cuStreamWaitValue32 failed with %d", (int)r);
  return 0;
}
int ctapp_peer_copy(void* dst, int dst_device, const void* src, int src_device, size_t bytes, void* stream) {
  GUARD(src_device);
  CU_OK(cudaMemcpyPeerAsync(dst, dst_device, src, src_device, bytes, static_cast<cudaStream_t>(stream)));
  return 0;
}

int ctapp_p2p_store_bw(const void* src, void* dst, size_t bytes, int device, void* stream) {
  ARG(src && dst && bytes % 16 == 0, "bad arguments");
  GUARD(device);
  copy16_kernel<<<sm_count(device) * 8, 512, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const int4*>(src), static_cast<int4*>(dst), bytes / 16);
  CU_OK(cudaGetLastError());
  return 0;
}

int ctapp_stamp_now(unsigned long long* out, int device, void* stream) {
  GUARD(device);
  stamp_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(out);
  CU_OK(cudaGetLastError());
  return 0;
}
int ctapp_timer_reads(unsigned long long* out, int n, int device, void* stream) {
  GUARD(device);
  timer_reads_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(out, n);
  CU_OK(cudaGetLastError());
  return 0;
}

int ctapp_pingpong(int* mine, int* other, unsigned long long* out, int n, int is_a, int* status, int device, void* stream) {
  ARG(mine && other && out && n > 0, "bad arguments");
  GUARD(device);
  pingpong_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(mine, other, out, n, is_a, status, limit_ns());
  CU_OK(cudaGetLastError());
  return 0;
}

int ctapp_malloc(void** out, size_t bytes, int device) {
  ARG(out && bytes > 0, "bad arguments");
  GUARD(device);
  CU_OK(cudaMalloc(out, bytes));
  return 0;
}
int ctapp_free(void* ptr, int device) {
  GUARD(device);
  CU_OK(cudaFree(ptr));
  return 0;
}
int ctapp_ipc_get_handle(void* ptr, unsigned char handle64[64], int device) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  GUARD(device);
  cudaIpcMemHandle_t h;
  CU_OK(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle64, &h, 64);
  return 0;
}
int ctapp_ipc_open(const unsigned char handle64[64], void** out, int device) {
  GUARD(device);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  CU_OK(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}
int ctapp_ipc_close(void* ptr, int device) {
  GUARD(device);
  CU_OK(cudaIpcCloseMemHandle(ptr));
  return 0;
}

}  // extern "C"
