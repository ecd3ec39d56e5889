/* C ABI of the B200-native CTA-pipelining library (libctapp_b200.so).
 *
 * Plain pointers and sizes only.  Every pointer named "device" is a CUDA device address valid on the GPU `device`
 * (peer addresses are device addresses of another GPU made reachable by peer access or an IPC mapping).  Work is
 * enqueued on `stream` (a cudaStream_t, may be NULL for the legacy default stream) of GPU `device`; the call
 * returns as soon as the work is enqueued.  Return value: 0 = ok, negative = argument error, positive = CUDA error
 * code; ctapp_last_error() gives the text.  Device-side waits are bounded: a wait that gives up writes a code into
 * the caller's `status` buffer (CTAPP_STATUS_INTS ints, zeroed by the caller) and the kernel drains and exits.
 *
 * Each entry point names the reference binding it replaces (file:line inside the reference project).
 */
#ifndef CTAPP_B200_H
#define CTAPP_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CTAPP_STATUS_INTS 8
#define CTAPP_MAX_WORLD 8

/* ---- library ---- */
const char* ctapp_last_error(void);
int ctapp_abi_version(void);   /* changes whenever an argument struct below changes layout; currently 5 */
/* Upper bound, in milliseconds, for every device-side wait on another GPU (default 2000, env CTAPP_WAIT_LIMIT_MS). */
int ctapp_set_wait_limit_ms(int ms);
int ctapp_get_wait_limit_ms(void);
/* Loads every kernel of the library on `device` (no launch), so that no lazy module load can happen while a
 * kernel that waits on a peer is resident.  Replaces the warm-up launches of ctapp/tp4.py:240-260. */
int ctapp_preload(int device);

/* ---- harness natives (csrc/gemm_tma.cu:167-248) ---- */
int ctapp_enable_peer_access(int device, int peer);                                     /* gemm_tma.cu:167-172 */
int ctapp_gate_alloc(void);                                                             /* gemm_tma.cu:192-197 */
int ctapp_gate_set(int value);                                                          /* gemm_tma.cu:198 */
int ctapp_gate_wait(int device, void* stream);                                          /* gemm_tma.cu:200-203 */
int ctapp_peer_copy(void* dst, int dst_device, const void* src, int src_device, size_t bytes, void* stream);   /* gemm_tma.cu:205-208 */
int ctapp_p2p_store_bw(const void* src, void* dst, size_t bytes, int device, void* stream);                    /* gemm_tma.cu:174-186 */
int ctapp_stamp_now(unsigned long long* out, int device, void* stream);                 /* gemm_tma.cu:214-218 */
int ctapp_timer_reads(unsigned long long* out, int n, int device, void* stream);        /* gemm_tma.cu:221-225 */
/* Bounded ping-pong between two GPUs; status may be NULL. */                            /* gemm_tma.cu:229-248 */
int ctapp_pingpong(int* mine, int* other, unsigned long long* out, int n, int is_a, int* status, int device, void* stream);
/* Cross-process mapping of device memory allocated by this library (one process per GPU). */
int ctapp_malloc(void** out, size_t bytes, int device);
int ctapp_free(void* ptr, int device);
int ctapp_ipc_get_handle(void* ptr, unsigned char handle64[64], int device);
int ctapp_ipc_open(const unsigned char handle64[64], void** out, int device);
int ctapp_ipc_close(void* ptr, int device);

/* ---- GEMM configurations (csrc/gemm_tma.cu:116-126, 155-165) ----
 * ids 0-9 are the reference's; each resolves to a one-CTA tcgen05 tile 128 x {128|256} x 64.  id 10 (no counterpart in
 * the reference) is the CTA-pair kernel: a cluster of two CTAs, cta_group::2, protocol tile 256 x 256 x 64; id 11 is the
 * same kernel on a 256 x 512 x 64 tile (a quarter less operand traffic per FLOP, one TMEM accumulator: for large plain or
 * chained GEMMs; the tensor-parallel entry points keep the 256-column tile). */
int ctapp_config_info(int config_id, char* buf, int buf_len);   /* text contains "tile BMxBNxBK" */
int ctapp_occupancy(int config_id);                              /* resident CTAs per SM */
/* How many clusters of `cluster_size` CTAs of the CTA-pair kernel (its threads and shared memory) the device can hold at
 * once (cudaOccupancyMaxActiveClusters); negative = error.  A cluster lives inside one GPC, so sizes that do not divide a
 * GPC's SM count leave SMs idle: the figure that decides whether a wider cluster can pay.  No counterpart in the reference. */
int ctapp_cluster_occupancy(int cluster_size, int device);

/* Y[M,N] = X[M,K] * W[N,K]^T, bf16 in, fp32 accumulate, bf16 out.  gemm_tma.cu:128-134 (gemm_tma), gemm_coop.cu:101-114
 * (coop_gemm).  group_rows: tile rows walked together (0 = library default); sms: CTAs to launch (0 = all SMs). */
int ctapp_gemm(const void* X, const void* W, void* Y, int M, int N, int K, int config_id, int group_rows, int sms,
               int device, void* stream);

/* ---- layer-per-GPU chain (csrc/ctapp.cuh:5-69, csrc/gemm_tma.cu:136-153) ---- */
typedef struct ctapp_queue {   /* ctapp.cuh:5 */
  int* entries;                /* cap ints, -1 = empty */
  int* head;
  int* tail;
  int cap;
} ctapp_queue;

typedef struct ctapp_chain_args {     /* ctapp.cuh:7-19 */
  unsigned long long* stamps;         /* NULL = off; else 8 u64 per CTA */
  ctapp_queue src;                    /* this GPU's work queue; cap == number of tiles of this GEMM */
  const int* dep_offsets;             /* CSR over this GEMM's tiles, NULL for the last stage */
  const int* dep_consumers;
  int* scoreboard;                    /* local counters, one per downstream tile or row panel (stride 32 ints) */
  ctapp_queue dst;                    /* the downstream GPU's queue (peer addresses) */
  int tiles_n;                        /* n-tiles of this GEMM */
  int skip_wait;                      /* negative control: take tile = pop index without waiting */
  int fence;                          /* accepted for compatibility; the TMA-store epilogue always orders as mode 1 */
  int tiles_n2;                       /* n-tiles of the downstream GEMM (row-panel mode) */
  int rowpanel;
  const int* dst_ready;               /* optional local flag the downstream GPU raises to `ready_value` once it has
                                         reset its queue; NULL = the caller orders the reset with stream events */
  int ready_value;
  int* status;                        /* CTAPP_STATUS_INTS ints or NULL */
  int sms;                            /* CTAs to launch, 0 = all SMs */
  int src_group;                      /* > 1: pop the source queue in windows of src_group published row panels, n-tile
                                         major inside a window (the L2-friendly order of a producer that finishes row
                                         panels in groups of that size); 0 | 1 = queue order.  No counterpart in the
                                         reference, whose consumer pops in queue order (ctapp.cuh:32-48). */
  const int* src_windows;             /* device array of n_windows + 1 ascending row-panel offsets (first 0, last = row
                                         panels of this GEMM): windows of any sizes, for a producer that finishes its
                                         row panels in groups of varying size; overrides src_group.  NULL = off. */
  int n_windows;
  /* k-chunk dependencies (no counterpart in the reference, whose consumer tile waits for its complete row panel,
   * ctapp.cuh:32-48, 51-69): value flags, one per tile of the PRODUCING GEMM, in the consuming GPU's memory.
   *   chunk_dst   producer side: peer address of the next GPU's flags; finished tile (m, n) raises chunk_dst[m * tiles_n + n] =
   *               chunk_value after its rows have landed (may be combined with dep_offsets; NULL = off)
   *   chunk_src   consumer side: this GPU's flags [row tiles][chunk_cols]; before loading the k-blocks
   *               [c * chunk_kblocks, (c + 1) * chunk_kblocks) of a tile of row tile m the loader waits (bounded) for
   *               chunk_src[m * chunk_cols + c] >= chunk_value, so a tile's main loop streams behind the producer.  The source
   *               queue is then pre-filled with this GEMM's own tile order (cap ids, tail = cap).  Both GEMMs must use tiles of the
   *               same height.  Values only grow from run to run, so the flags are never reset. */
  int* chunk_dst;
  const int* chunk_src;
  int chunk_kblocks, chunk_cols, chunk_value;
} ctapp_chain_args;

/* One stage of the chain: Y = X * W^T with tile ids popped from args->src and completion published into args->dst.
 * Y may be a peer address (the next GPU's input).  gemm_tma.cu:136-153 (ctapp_gemm). */
int ctapp_chain_gemm(const void* X, const void* W, void* Y, int M, int N, int K, int config_id,
                     const ctapp_chain_args* args, int device, void* stream);
/* Reset a stage's queue for the next run (entries = -1, head = tail = 0, scoreboard = pristine; q.entries == NULL
 * keeps a pre-filled source queue's ids and tail and only rewinds head) and then, if ready_flag != NULL, release
 * ready_flag[0] = ready_value at system scope (a flag in the upstream GPU's memory).
 * ctapp/pipeline.py:64-71 (Pipeline.reset), as one kernel. */
int ctapp_chain_reset(ctapp_queue q, int* scoreboard, const int* scoreboard_pristine, int scoreboard_len,
                      int* ready_flag, int ready_value, int device, void* stream);

/* ---- tensor-parallel layer boundary (csrc/ctapp_tp4.cuh, csrc/gemm_tp4.cu) ---- */
typedef struct ctapp_tp_down_args {   /* gemm_tp4.cu:156-199 (tp4_down); modes 0 and 7 */
  const void* A; const void* W; void* D;   /* A (M,K), W (N,K); D (M,N) used in mode 0 only */
  int M, N, K;
  int raster, swizzle, mode, rank, world;
  int epoch; const int* epoch_dev;         /* epoch_dev != NULL overrides epoch */
  void* dst_ptrs[CTAPP_MAX_WORLD];         /* mode 7: this rank's inbox slot at every owner, (dst_rows, N) bf16 */
  int dst_rows;
  int* peer_tile_flags[CTAPP_MAX_WORLD];   /* mode 7: every owner's tile_flags[world][ppo][N/256] */
  int panels_per_owner;
  int sms, pdl_trigger, pdl, tail_cols;
  unsigned long long* trace;
  int* status;
  int cta_pair;                            /* 0 = one CTA per 128-row tile; 1 = two CTAs per 256-row tile (cta_group::2), 256
                                              columns wide; 2 = the same on 256 x 512 tiles (N % 512 == 0; a tile raises the two
                                              256-column tile flags it covers; a quarter less operand traffic per FLOP) */
  int dst_global;                          /* mode 7: 1 = a tile keeps its own row position in every destination (each dst_ptrs[d]
                                              is then an (M, N) buffer, dst_rows >= M) instead of moving to row block m / world of
                                              the owner's inbox slot.  With every dst_ptrs[d] = this rank's partial buffer the
                                              producer stores locally and only the tile flag crosses the link: the layout the
                                              in-switch reduction reads (ctapp_tp_reduce_args.partials_mc; the reference's producer
                                              mode 4, csrc/ctapp_tp4.cuh:284-289) */
  int* tile_log;                           /* NULL, or [0] = 0 on entry and room for 1 + #tiles ints: the kernel appends one packed
                                              (m << 16 | n) per tile in the order its schedulers take them (m = tile row of the
                                              schedule: 256 rows with cta_pair); with one CTA (pair) that is the tile order itself */
} ctapp_tp_down_args;
int ctapp_tp_down(const ctapp_tp_down_args* args, int device, void* stream);

struct ctapp_tp_reduce_args;
typedef struct ctapp_tp_qkv_args {    /* gemm_tp4.cu:319-359 (tp4_qkv); modes 0, 5 and 8 */
  const void* X; const void* W; void* Y;   /* X (M,K) local, written by the owner reducers; W (N,K) gamma-folded; Y (M,N) */
  int M, N, K;
  int raster, swizzle, mode;               /* raster 2: n fastest; 3: groups of `swizzle` tile rows, n-major inside; else m fastest */
  int epoch; const int* epoch_dev;
  const int* panel_flag;                   /* [M/128], value flags */
  const float* rowss;                      /* [M] row sums of squares of X; NULL = no scaling */
  float eps;
  int sms, pdl, tile;                      /* tile: 256 | 128 */
  unsigned long long* trace;
  int* status;
  int cta_pair;                            /* as in ctapp_tp_down_args; needs tile 256 */
  int act;                                 /* 1: W holds gate and up rows interleaved in blocks of 128 (tile n = gate rows
                                              128n.. then up rows 128n..) and Y (M, N/2) receives silu(gate) * up, both
                                              factors rounded to bf16 first; needs cta_pair.  The reference runs the
                                              activation as a separate kernel (vllm_plugin/ctapp_vllm/model.py:183) and
                                              lists this fusion as future work (PLAN.md:597).  0 = off. */
  const struct ctapp_tp_reduce_args* red;  /* mode 8 (csrc/ctapp_tp4.cuh:913-925, the work-stealing form of tp4_role_preamble):
                                              every warp of every CTA first claims owner-reducer units from red->unit_ctr until
                                              none are left, then the CTA runs its GEMM tiles as in mode 5.  CTAs that become
                                              resident as the producer's retire thus drain what the dedicated reducer CTAs
                                              (ctapp_tp_reduce with the same unit_ctr) have not reached.  red->blocks / threads
                                              are ignored.  NULL in the other modes. */
} ctapp_tp_qkv_args;
int ctapp_tp_qkv(const ctapp_tp_qkv_args* args, int device, void* stream);

typedef struct ctapp_tp_reduce_args {  /* gemm_tp4.cu:243-312 (tp4_reduce, version 5 variant 1) */
  int M, n1, rank, world;
  int epoch; const int* epoch_dev;
  int blocks, threads;
  const int* tile_flags;                    /* local [world][ppo][n1/256] */
  const void* inbox[CTAPP_MAX_WORLD];       /* local inbox slot of every source rank */
  const void* resid;                        /* (M, n1) bf16 or NULL */
  void* peer_x[CTAPP_MAX_WORLD];            /* x buffer of every rank, (M, n1) bf16 */
  float* peer_rowss[CTAPP_MAX_WORLD];       /* rowss buffer of every rank, [M] */
  int* peer_panel_flag[CTAPP_MAX_WORLD];    /* panel_flag of every rank, [M/128] */
  float* rowss_local;                       /* [M] accumulators, zeroed by ctapp_tp_step */
  int* panel_done;                          /* [M/128] arrival counters, zeroed by ctapp_tp_step */
  int panels_per_owner, tail_cols;          /* panels_per_owner: the ppo the flags and inbox were allocated with; must be
                                               >= ceil(M / 128 / world) (checked) and not larger than the allocation (the caller's) */
  int order, swz;                           /* unit order when tail_cols == 0 (csrc/ctapp_tp4.cuh:551-565): order 0 | 1 = m fastest,
                                               in groups of swz n-tiles when swz > 1; 2 = panel by panel */
  int* unit_ctr;                            /* NULL = static unit assignment; else units are claimed from this counter (zeroed
                                               per step, e.g. role_ctr + 1 of ctapp_tp_step), which ctapp_tp_qkv mode 8 shares */
  int* unit_log;                            /* NULL, or [0] = 0 on entry and room for 1 + #units ints: one packed
                                               (j << 16 | n << 2 | q) per unit in the order the warps take them */
  int pdl_trigger;                          /* 1: raise the programmatic-launch trigger at entry, so that a producer GEMM
                                               launched behind this kernel with pdl = 1 starts beside it (ctapp/tp4.py:316-320) */
  int help_all;                             /* only read through ctapp_tp_qkv mode 8: 0 = a helping warp takes a unit only while
                                               the next unclaimed unit's tile has already arrived (the dedicated reducer CTAs are
                                               behind the producers) and otherwise goes on to its GEMM tiles; 1 = helpers take
                                               every unit and wait for tiles (no dedicated reducer CTAs are launched) */
  unsigned long long* trace;
  int* status;
  /* NVLS variant (csrc/ctapp_tp4.cuh:150-183, 458-536: multimem.st / multimem.red pushes): multicast addresses of the x
   * buffer, the row-sum buffer and the panel flags; all NULL = unicast pushes to peer_x / peer_rowss / peer_panel_flag */
  void* x_mc;
  float* rowss_mc;
  int* panel_flag_mc;
  /* In-switch reduction (csrc/ctapp_tp4.cuh:150-183, 458-536: multimem.ld_reduce): multicast address of the ranks' partial
   * buffers, (M, n1) bf16 each, written by producers launched with dst_global.  The W loads and adds per output become one
   * multimem.ld_reduce.add.acc::f32.v4.bf16x2; `inbox` is not read.  The switch returns the sum as bf16 and the residual is
   * added after that rounding: one bf16 rounding more than the inbox path, so results agree with it within the boundary's
   * max-error tolerance, not bit for bit (the mean error against the inbox path's rounding model doubles).  Needs the NVLS pushes above; NULL = read the inbox. */
  const void* partials_mc;
  /* Role switching (csrc/ctapp_tp4.cuh:913-925, ctapp/tp4.py:312-315), only read through ctapp_tp_qkv mode 8: with role_r > 0 no
   * reducer kernel is launched; every CTA of the consumer GEMM draws a ticket from role_ctr[0] (zeroed per step by
   * ctapp_tp_step), the first role_r to arrive run the owner reducer's static share ticket / role_r with all their warps and
   * then take GEMM tiles like the rest.  Launch the consumer as a programmatic dependent (pdl = 1) of a producer that raises
   * its trigger (pdl_trigger = 1) and leaves role_r SMs free, so that those CTAs are resident beside it.  unit_ctr must be
   * NULL (static shares); with unit_ctr and help_all = 1 instead, every CTA claims units (the reference's role + steal). */
  int* role_ctr;
  int role_r;
} ctapp_tp_reduce_args;
int ctapp_tp_reduce(const ctapp_tp_reduce_args* args, int device, void* stream);

/* Owner reducer for callers that cannot allocate device memory.  No counterpart in the reference.
 * Some hosts of this library never get to call cudaMalloc once they are running: an inference server that hands the
 * whole GPU to its own block pool at start-up, or a plugin called on a path where an allocation (which may synchronise
 * the device or fail in a full GPU) is not acceptable.  For them this variant of ctapp_tp_reduce keeps the reducer's
 * working memory -- the per-row fp32 accumulators and the per-panel arrival counters that ctapp_tp_reduce takes as
 * rowss_local / panel_done -- in a fixed array inside the library (66 048 bytes, resident on every GPU that loads the
 * library until the process exits).  The caller passes inputs and outputs exactly as for ctapp_tp_reduce;
 * args->rowss_local and args->panel_done are ignored, and no ctapp_tp_step is needed for them: the call zeroes the part of
 * the array it uses (stream-ordered, before the kernel).  What this variant does not offer is refused with an argument
 * error rather than ignored: the NVLS pushes (x_mc, rowss_mc, panel_flag_mc must be NULL: it pushes with unicast stores),
 * dynamic unit claims and the unit log (unit_ctr, unit_log must be NULL) and pdl_trigger (must be 0).
 *   Limit: M <= 16384 rows; larger M is refused with an error naming the limit.
 *   The first call on a device looks up the array's device address (one cudaGetSymbolAddress, no allocation) unless
 *   ctapp_preload has run on that device, which does the same look-up; make whichever comes first outside any stream capture.
 *   All calls on a GPU share the one array: two calls whose kernels overlap on the GPU (different streams) race on
 *   it.  Issue them on one stream, or order them with events.
 * The call performs no cudaMalloc / cudaFree and uses no allocating library routine. */
int ctapp_tp_reduce_noalloc(const ctapp_tp_reduce_args* args, int device, void* stream);

/* Read-back of the integer maps the kernels schedule by, computed by the same device functions (no counterpart in the
 * reference, where tp4_remap_tile / red5_map, csrc/ctapp_tp4.cuh:897-906, 551-565, exist only inside the kernels):
 *   tile order  out_mn[2 L], out_mn[2 L + 1] = (m, n) of schedule position L; order 0 = groups of group_rows tile rows, n-major
 *               inside a group; 1 = m fastest over the first tiles_n - tail_cols n-tiles, then tile row by tile row over the
 *               last tail_cols; 2 = n fastest
 *   unit order  out_jnq[3 u ..] = (owned panel j, n-tile, quarter) of the owner reducer's unit u
 *   queue slots out_slots[i] = source-queue slot read by the i-th pop of a consuming chain stage (src_group / src_windows) */
int ctapp_debug_tile_order(int order, int tiles_m, int tiles_n, int group_rows, int tail_cols, int* out_mn, int device, void* stream);
int ctapp_debug_unit_order(int owned_panels, int tiles_n, int tail_cols, int order, int swz, int* out_jnq, int device, void* stream);
int ctapp_debug_queue_slots(int num_tiles, int tiles_n, int src_group, const int* src_windows, int n_windows, int* out_slots,
                            int device, void* stream);

/* epoch_dev[0] += 1; zero rowss_local[0:M], panel_done[0:M/128] and role_ctr[0:2].  gemm_tp4.cu:362-372 (tp4_step). */
int ctapp_tp_step(int* epoch_dev, float* rowss_local, int* panel_done, int M, int* role_ctr, int device, void* stream);

/* NVLS known-answer probes on a multicast address `mc` (csrc/gemm_tp4.cu:393-502: mm_red_u32, mm_red_f32, mm_st_bf16,
 * mm_ld_reduce_bf16, mm_order_stress).  The ordering stress runs the reducer's publish sequence (multimem.st payload,
 * fence, releasing multimem.st flag) `iters` times per slot with bounded waits; result[0] = stale payload words seen,
 * result[1] != 0 = a wait gave up. */
int ctapp_mm_red_u32(void* mc, int n, unsigned v, int device, void* stream);
int ctapp_mm_red_f32(void* mc, const float* src, int n, int device, void* stream);
int ctapp_mm_st_bf16(void* mc, const void* src, int n, int device, void* stream);
int ctapp_mm_ld_reduce_bf16(const void* mc, void* out, int n, int device, void* stream);
int ctapp_mm_order_stress(void* data_mc, const void* data_local, int* flag_mc, const int* flag_local, unsigned* ack_mc,
                          const unsigned* ack_local, int rank, int world, int iters, int slots, int* result, int device, void* stream);

/* Comparison baseline only: x = a + resid (bf16), y = rmsnorm(x) * gamma, one pass (the fused add+RMSNorm a serving
 * stack runs after an all-reduce).  No counterpart in the reference (it used eager torch, ctapp/tp4.py:47-50). */
int ctapp_add_rmsnorm(const void* a, const void* resid, const void* gamma, void* x_out, void* y_out, int M, int n1,
                      float eps, int device, void* stream);

/* out (M, I) = silu(in[:, :I]) * in[:, I:] for in (M, 2 I) bf16, I % 8 == 0: the activation between the gate/up and the
 * down projection as one pass, for callers that do not fuse it into ctapp_tp_qkv (act = 1) and for the comparison
 * baselines.  No counterpart in the reference, which calls the serving stack's own kernel
 * (vllm_plugin/ctapp_vllm/model.py:183). */
int ctapp_silu_mul(const void* in, void* out, int M, int I, int device, void* stream);

/* registers / shared memory / spill of a kernel: which = 0 GEMM 128x256, 1 GEMM 128x128, 2 reducer, 3 CTA-pair GEMM,
 * 4 CTA-pair GEMM with the activation epilogue.  gemm_tp4.cu:374-390 */
int ctapp_kernel_info(int which, char* buf, int buf_len);

#ifdef __cplusplus
}
#endif
#endif /* CTAPP_B200_H */
