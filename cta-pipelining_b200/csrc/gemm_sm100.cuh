// Persistent, warp-specialised bf16 GEMM for sm_100a: D[M,N] = A[M,K] * B[N,K]^T, fp32 accumulation in TMEM.
//
//   warp 0   : scheduler + TMA loader.  Gets the next tile id (static order, or popped from a work queue and
//              acquired at system scope), publishes it to the other roles through a small ring, then streams the
//              A and B k-blocks of that tile into a multi-stage shared-memory ring with cp.async.bulk.tensor.
//   warp 1   : MMA issuer.  One thread issues tcgen05.mma (128 x BN x 16) over the ring into one of two TMEM
//              accumulators, so the epilogue of tile i overlaps the main loop of tile i+1.  Owns TMEM.
//   warps 2-5: epilogue.  tcgen05.ld -> (optional per-row scale) -> bf16 -> swizzled shared memory ->
//              cp.async.bulk.tensor store, each warp on its own 32-row slab with its own staging buffers.  The
//              destination tensor map may describe a peer GPU's memory.  After a tile's stores have completed the
//              warps publish it: chain scoreboard + downstream queue, or a per-tile value flag at the owner.
//
// Every wait on another GPU is bounded; a give-up is reported in the status buffer and the CTA drains and exits.
#pragma once
#include "ptx.cuh"
#include "reduce_sm100.cuh"

namespace ctapp {

constexpr int kMaxWorld = 8;
constexpr int BM = 128;   // tile rows == TMEM lanes
constexpr int BK = 64;    // k-block: 64 bf16 = one 128-byte swizzle row
constexpr int kThreads = 192;
constexpr int kSchedSlots = 4;
constexpr int kStageRows = 32;   // rows per epilogue warp
constexpr int kStoreCols = 64;   // columns per TMA store box (128 bytes)

// what the kernel does around the plain GEMM
enum GemmMode : int {
  kModePlain = 0,        // static tile order, local or peer D
  kModeChain = 1,        // tile ids from a work queue; optional downstream signalling
  kModeTpProducer = 7,   // scatter tile (m, n) to owner m % world and raise its tile flag
  kModeTpConsumer = 5,   // wait per 128-row panel for the owner's panel flag; scale rows by rsqrt(rowss/K + eps)
};                       // (with red.unit_ctr set its CTAs first help the owner reducer: every warp claims units until none are left)
enum TileOrder : int { kOrderGrouped = 0, kOrderMFastTail = 1, kOrderNFast = 2 };

struct Queue { int* entries; int* head; int* tail; int cap; };

struct alignas(64) GemmParams {
  CUtensorMap tmA;                 // A (M, K) row-major bf16, box 64 x 128
  CUtensorMap tmB;                 // B (N, K) row-major bf16, box 64 x BN
  CUtensorMap tmD[kMaxWorld];      // D (rows, N) row-major bf16, box 64 x 32; one per destination
  int M, N, K;
  int tiles_m, tiles_n, num_tiles;   // tile rows / columns of the schedule (CTA-pair kernel: 256-row tiles)
  int panels;                        // 128-row panels of M
  int mode, order, group_rows, tail_cols;
  // chain
  Queue src;
  const int* dep_offsets;
  const int* dep_consumers;
  int* scoreboard;
  Queue dst;
  int tiles_n2, rowpanel, skip_wait, src_group, n_windows;
  const int* src_windows;
  const int* dst_ready;
  int ready_value;
  // chain, k-chunk dependencies: instead of (or beside) the scoreboard, a finished tile (m, n) raises chunk_dst[m * tiles_n + n]
  // = chunk_value in the next GPU's memory; a consuming GEMM waits for chunk_src[m * chunk_cols + c] >= chunk_value before it
  // loads the k-blocks [c * chunk_kblocks, (c + 1) * chunk_kblocks) of a tile of row m: its main loop streams behind the producer
  int* chunk_dst;
  const int* chunk_src;
  int chunk_kblocks, chunk_cols, chunk_value;
  // tensor-parallel boundary
  int world, rank, ppo;
  int dst_global;                    // producer: a tile's destination rows are its own rows (every tmD describes an (M, N) buffer, e.g.
                                     // this rank's partial buffer for the in-switch reduction) instead of the owner's inbox rows
  int* peer_tile_flags[kMaxWorld];
  const int* epoch_ptr;
  int epoch;
  const int* panel_flag;
  const float* rowss;
  float inv_k, eps;
  // launch behaviour
  int pdl_trigger;                 // raise the programmatic-launch trigger right after the prologue
  int pdl_wait;                    // wait for the preceding grid's memory before touching global memory
  int act;                         // CTA-pair kernel only: 1 = silu(gate) * up epilogue over interleaved 128-column halves
  int* status;
  unsigned long long* stamps;      // 8 u64 per CTA or null
  int* tile_log;                   // null, or [0] = count followed by one packed (m << 16 | n) per scheduled tile, in schedule order
  long long limit_ns;
  ReduceParams red;                // tensor-parallel consumer: the owner reducer's arguments when its CTAs help (red.unit_ctr != null)
};

// Bounded wait of a consuming GEMM for k-chunk c of its A rows (written by the previous GPU's epilogue): one acquiring load
// when the chunk is there already.  Returns the first chunk index not known to be ready (c + 1), or c when the wait gave up
// (status written).  (Looking at several flags per poll with relaxed loads and one acquire fence for all of them measured
// 9-12 % slower over a whole chain run than one acquiring load per chunk.)
__device__ __forceinline__ int wait_chunks(const GemmParams& p, int m, int c, int nchunks, long long limit) {
  int seen;
  const int idx = m * p.chunk_cols + c;
  if (!spin_acquire_sys(p.chunk_src + idx, PredGe{p.chunk_value}, limit, seen)) {
    report_status(p.status, kStatusTimeoutChunk, idx, p.chunk_value, seen);
    return c;
  }
  fence_proxy_async_global();   // the rows were written through another GPU's async proxy; the loads below go through this one's
  return c + 1;
}

// Chain mode: which slot of the source queue the idx-th pop reads.  The producer publishes a finished row panel as tiles_n
// consecutive slots.  With windows the pops walk a window of g such panels n-tile major (slot 0 of every panel of the
// window, then slot 1, ...), so that g row panels share each weight tile while it is hot in L2.  src_group = g > 1: windows of
// constant size (the last one takes the panels that are left); src_windows: n_windows + 1 ascending panel offsets of windows
// of any sizes.  A permutation of the slots either way: every slot is still read exactly once.  `cur` is the caller's
// cursor into src_windows (pops of one CTA ascend).
__device__ __forceinline__ int queue_slot(const GemmParams& p, int idx, int& cur) {
  const int tn = p.tiles_n;
  int first, gw;   // first panel and panel count of the window idx falls into
  if (p.src_windows) {
    const int pi = idx / tn;
    while (cur + 1 < p.n_windows && __ldg(p.src_windows + cur + 1) <= pi) cur++;
    first = __ldg(p.src_windows + cur);
    gw = __ldg(p.src_windows + cur + 1) - first;
  } else {
    const int g = p.src_group;
    if (g <= 1) return idx % p.src.cap;
    first = (idx / (g * tn)) * g;
    const int left = p.src.cap / tn - first;
    gw = left < g ? left : g;
  }
  const int base = first * tn, r = idx - base;
  return base + (r % gw) * tn + r / gw;
}

__device__ __forceinline__ void decode_tile(const GemmParams& p, int L, int& m, int& n) {
  const int TM = p.tiles_m, TN = p.tiles_n;
  if (p.order == kOrderNFast) { m = L / TN; n = L - m * TN; return; }
  if (p.order == kOrderMFastTail) {
    const int C = p.tail_cols, head = TM * (TN - C);
    if (L < head) { n = L / TM; m = L - n * TM; }
    else { const int L2 = L - head; m = L2 / C; n = TN - C + (L2 - m * C); }
    return;
  }
  const int g = p.group_rows > 0 ? p.group_rows : 1;
  const int per = g * TN, grp = L / per, m0 = grp * g;
  const int rows = min(g, TM - m0), r = L - grp * per;
  n = r / rows; m = m0 + (r - n * rows);
}

// Read-back of the static tile order: out[2 L], out[2 L + 1] = (m, n) of schedule position L.
__global__ void tile_order_kernel(GemmParams p, int* out) {
  for (int L = blockIdx.x * blockDim.x + threadIdx.x; L < p.num_tiles; L += gridDim.x * blockDim.x) {
    int m, n;
    decode_tile(p, L, m, n);
    out[2 * L] = m; out[2 * L + 1] = n;
  }
}
// Read-back of the pop order of a consuming chain stage: out[i] = queue slot of the i-th pop.
__global__ void queue_slot_kernel(GemmParams p, int* out) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    int cur = 0;
    for (int i = 0; i < p.num_tiles; i++) out[i] = queue_slot(p, i, cur);
  }
}

template <int BN> struct GemmCfg {
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr uint32_t kABytes = BM * BK * 2;
  static constexpr uint32_t kBBytes = BN * BK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kEpiBytes = 4 * 2 * kStageRows * kStoreCols * 2;   // 4 warps x 2 buffers x 4 KB
  static constexpr uint32_t kBarBytes = 512;
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + kEpiBytes + kBarBytes + 1024;   // + alignment slack
  static constexpr uint32_t kTmemCols = 2 * BN;
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1) gemm_kernel(const __grid_constant__ GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + S * Cfg::kABytes;
  uint8_t* sD = sB + S * Cfg::kBBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sD + Cfg::kEpiBytes);
  uint64_t* full = bars;                    // [S]  TMA -> MMA
  uint64_t* empty = full + S;               // [S]  MMA -> TMA
  uint64_t* tfull = empty + S;              // [2]  MMA -> epilogue
  uint64_t* tempty = tfull + 2;             // [2]  epilogue -> MMA
  uint64_t* sfull = tempty + 2;             // [kSchedSlots] scheduler -> MMA, epilogue
  uint64_t* sempty = sfull + kSchedSlots;   // [kSchedSlots]
  uint64_t* drain = sempty + kSchedSlots;   // [1]  abort path only
  uint64_t* epi = drain + 1;                // [1]  epilogue warps -> publishing warp, one phase per published tile
  int* s_tile = reinterpret_cast<int*>(epi + 1);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_tile + kSchedSlots);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  int* s_ticket = const_cast<int*>(s_abort) + 1;   // role switching: this CTA's ticket

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = (p.K + BK - 1) / BK;
  const long long limit = p.limit_ns;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; i++) { mbar_init(full + i, 1); mbar_init(empty + i, 1); }
    for (int i = 0; i < 2; i++) { mbar_init(tfull + i, 1); mbar_init(tempty + i, 4); }
    for (int i = 0; i < kSchedSlots; i++) { mbar_init(sfull + i, 1); mbar_init(sempty + i, 5); }
    mbar_init(drain, 1);
    mbar_init(epi, 4);
    *s_abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.tmA);
    tma_prefetch_desc(&p.tmB);
    if (p.stamps) { p.stamps[blockIdx.x * 8 + 0] = globaltimer(); p.stamps[blockIdx.x * 8 + 6] = smid(); }
  }
  if (warp == 1) { tmem_alloc(s_tmem, Cfg::kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  if (p.pdl_trigger) pdl_launch_dependents();
  if (p.pdl_wait) pdl_wait();
  const int epoch = p.epoch_ptr ? __ldcg(p.epoch_ptr) : p.epoch;
  if (p.mode == kModeTpConsumer) {   // mode 8: every warp, before it takes up its role in the GEMM
    if (p.red.role_r > 0) reduce_role(p.red, epoch, s_ticket);
    else if (p.red.unit_ctr) reduce_help(p.red, epoch, p.red.help_all != 0);
  }

  if (warp == 0) {
    // ============================================================ scheduler + TMA loader
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; int sq = 0; uint32_t sphase = 0;
      uint32_t armed = 0, armed_parity = 0;   // per stage: has a load been issued, and in which phase
      int k_static = 0, ntiles_done = 0;
      uint32_t panel_seen[4] = {0, 0, 0, 0};
      int win_cur = 0;
      auto pop = [&]() -> int {
        if (p.mode == kModeChain) { const int idx = atomicAdd(p.src.head, 1); return idx < p.num_tiles ? idx : -1; }
        const int idx = static_cast<int>(blockIdx.x) + (k_static++) * static_cast<int>(gridDim.x);
        return idx < p.num_tiles ? idx : -1;
      };
      int next = pop();
      bool ok = true;
      while (ok) {
        int tile = next;
        if (tile >= 0 && p.status && ld_relaxed_gpu(p.status) != 0) tile = -1;   // another CTA gave up: stop taking work
        if (tile >= 0 && p.mode == kModeChain && !p.skip_wait) {
          int seen;
          const int slot = queue_slot(p, tile, win_cur);
          if (!spin_acquire_sys(p.src.entries + slot, PredNe{-1}, limit, seen)) {
            report_status(p.status, kStatusTimeoutQueue, slot, 0, seen); *s_abort = kStatusTimeoutQueue; break;
          }
          if (seen < 0 || seen >= p.num_tiles) {
            report_status(p.status, kStatusBadIndex, slot, p.num_tiles, seen); *s_abort = kStatusBadIndex; break;
          }
          tile = seen;
          fence_proxy_async_global();   // peer-written A rows must be visible to the TMA loads below
        }
        if (!mbar_wait(sempty + sq, sphase ^ 1, s_abort, limit)) break;
        s_tile[sq] = tile;
        mbar_arrive(sfull + sq);
        if (++sq == kSchedSlots) { sq = 0; sphase ^= 1; }
        if (tile < 0) break;
        int m, n;
        if (p.mode == kModeChain) { m = tile / p.tiles_n; n = tile - m * p.tiles_n; } else decode_tile(p, tile, m, n);
        if (p.tile_log) p.tile_log[1 + atomicAdd(p.tile_log, 1)] = (m << 16) | n;
        if (p.stamps && ntiles_done == 0) { p.stamps[blockIdx.x * 8 + 1] = globaltimer(); }
        if (p.mode == kModeTpConsumer && p.panel_flag && !(m < 128 && (panel_seen[m >> 5] >> (m & 31) & 1u))) {
          int seen;
          if (!spin_acquire_sys(p.panel_flag + m, PredGe{epoch}, limit, seen)) {
            report_status(p.status, kStatusTimeoutPanel, m, epoch, seen); *s_abort = kStatusTimeoutPanel; break;
          }
          fence_proxy_async_global();
          if (m < 128) panel_seen[m >> 5] |= 1u << (m & 31);   // a panel flag never goes back within a launch: ask once
        }
        next = -2;
        int chunk_upto = 0;   // k-chunks [0, chunk_upto) of this tile's rows are known to have landed
        const int nchunks = p.chunk_src ? (KB + p.chunk_kblocks - 1) / p.chunk_kblocks : 0;
        for (int kb = 0; kb < KB; kb++) {
          if (p.chunk_src && !p.skip_wait && kb % p.chunk_kblocks == 0 && kb / p.chunk_kblocks >= chunk_upto) {
            chunk_upto = wait_chunks(p, m, kb / p.chunk_kblocks, nchunks, limit);
            if (chunk_upto <= kb / p.chunk_kblocks) { *s_abort = kStatusTimeoutChunk; ok = false; break; }
          }
          if (!mbar_wait(empty + stage, phase ^ 1, s_abort, limit)) { ok = false; break; }
          mbar_arrive_expect_tx(full + stage, Cfg::kStageBytes);
          tma_load_2d(sA + stage * Cfg::kABytes, &p.tmA, kb * BK, m * BM, full + stage);
          tma_load_2d(sB + stage * Cfg::kBBytes, &p.tmB, kb * BK, n * BN, full + stage);
          armed |= 1u << stage;
          armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
          if (++stage == S) { stage = 0; phase ^= 1; }
          if (kb == (KB >> 1)) next = pop();   // claim the next tile early enough to hide the atomic's latency
        }
        if (next == -2) next = pop();
        ntiles_done++;
      }
      if (*s_abort) {   // let the loads already issued land before the CTA goes away
        for (int s = 0; s < S; s++)
          if (armed & (1u << s)) {
            const unsigned long long t0 = globaltimer();
            while (!mbar_try_wait(full + s, (armed_parity >> s) & 1u) && globaltimer() - t0 < 2000000ull) {}
          }
      }
      if (p.stamps) p.stamps[blockIdx.x * 8 + 5] = static_cast<unsigned long long>(ntiles_done);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ============================================================ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
      int stage = 0; uint32_t phase = 0; int sq = 0; uint32_t sphase = 0; uint32_t it = 0;
      bool ok = true;
      while (ok) {
        if (!mbar_wait(sfull + sq, sphase, s_abort, limit)) break;
        const int tile = s_tile[sq];
        mbar_arrive(sempty + sq);
        if (++sq == kSchedSlots) { sq = 0; sphase ^= 1; }
        if (tile < 0) break;
        const uint32_t a = it & 1u, aphase = (it >> 1) & 1u;
        if (!mbar_wait(tempty + a, aphase ^ 1, s_abort, limit)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + a * BN;
        for (int kb = 0; kb < KB; kb++) {
          if (!mbar_wait(full + stage, phase, s_abort, limit)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = umma_desc_k128(sA + stage * Cfg::kABytes);
          const uint64_t bdesc = umma_desc_k128(sB + stage * Cfg::kBBytes);
#pragma unroll
          for (int k = 0; k < BK / 16; k++)   // +32 bytes (2 descriptor units) per 16-element k step inside the swizzle row
            tc_mma_f16(d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          tc_commit(empty + stage);
          if (++stage == S) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(tfull + a);
        if (p.stamps) p.stamps[blockIdx.x * 8 + 2] = globaltimer();
        it++;
      }
      if (*s_abort) {   // make sure no MMA is still writing TMEM when it is released
        tc_commit(drain);
        const unsigned long long t0 = globaltimer();
        while (!mbar_try_wait(drain, 0) && globaltimer() - t0 < 2000000ull) {}
      }
    }
    __syncwarp();
  } else {
    // ============================================================ epilogue (warps 2..5)
    const int ew = warp - 2;
    const int lane_base = (warp & 3) * 32;              // the TMEM lane quarter this warp may read
    const int row_in_tile = lane_base + lane;
    uint8_t* stage_buf = sD + ew * (2 * kStageRows * kStoreCols * 2);
    int sq = 0; uint32_t sphase = 0; uint32_t it = 0; uint32_t cbuf = 0; uint32_t epi_phase = 0;
    bool ready_checked = p.dst_ready == nullptr;
    uint32_t epi_seen[4] = {0, 0, 0, 0};
    // every lane polls (each needs its own acquire); the outcome is made warp-uniform so the warp never splits
    auto warp_wait = [&](uint64_t* bar, uint32_t parity) -> bool {
      const bool ok = mbar_wait(bar, parity, s_abort, limit);
      return __all_sync(0xffffffffu, ok);
    };
    while (true) {
      if (!warp_wait(sfull + sq, sphase)) break;
      const int tile = s_tile[sq];
      __syncwarp();
      if (lane == 0) mbar_arrive(sempty + sq);
      if (++sq == kSchedSlots) { sq = 0; sphase ^= 1; }
      if (tile < 0) break;
      int m, n;
      if (p.mode == kModeChain) { m = tile / p.tiles_n; n = tile - m * p.tiles_n; } else decode_tile(p, tile, m, n);
      const uint32_t a = it & 1u, aphase = (it >> 1) & 1u;
      it++;
      if (!warp_wait(tfull + a, aphase)) break;
      tc_fence_after();

      float scale = 1.0f;
      if (p.mode == kModeTpConsumer && p.rowss) {
        if (p.panel_flag && !(m < 128 && (epi_seen[m >> 5] >> (m & 31) & 1u))) {   // rowss was pushed before the flag: acquire once per panel
          if (lane == 0) (void)ld_acquire_sys(p.panel_flag + m);
          if (m < 128) epi_seen[m >> 5] |= 1u << (m & 31);
        }
        __syncwarp();
        const int row = m * BM + row_in_tile;
        if (row < p.M) scale = rsqrtf(__ldcg(p.rowss + row) * p.inv_k + p.eps);
      }
      if (!ready_checked) {   // downstream must have reset its queue / may still be reading the previous run's rows
        int okr = 1;
        if (lane == 0) {
          int seen;
          if (!spin_acquire_sys(p.dst_ready, PredGe{p.ready_value}, limit, seen)) {
            report_status(p.status, kStatusTimeoutReady, 0, p.ready_value, seen); *s_abort = kStatusTimeoutReady; okr = 0;
          }
        }
        okr = __shfl_sync(0xffffffffu, okr, 0);
        if (!okr) break;
        ready_checked = true;
      }
      // destination of this tile
      int dst = 0, drow = m * BM;
      if (p.mode == kModeTpProducer) { dst = m % p.world; drow = p.dst_global ? m * BM : (m / p.world) * BM; }
      const CUtensorMap* tmD = &p.tmD[dst];

      const uint32_t tcol = tmem_base + (static_cast<uint32_t>(lane_base) << 16) + a * BN;
#pragma unroll 1
      for (int c = 0; c < BN / kStoreCols; c++) {
        uint32_t v[2][32];
        tc_ld_32x32b_x32(tcol + c * kStoreCols, v[0]);
        tc_ld_32x32b_x32(tcol + c * kStoreCols + 32, v[1]);
        tc_wait_ld();
        if (c == BN / kStoreCols - 1) {   // accumulator fully read: hand it back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty + a);
        }
        uint8_t* buf = stage_buf + (cbuf & 1u) * (kStageRows * kStoreCols * 2);
        cbuf++;
        if (lane == 0) bulk_wait_read<1>();   // the store issued two chunks ago has finished reading this buffer
        __syncwarp();
#pragma unroll
        for (int h = 0; h < 2; h++) {
#pragma unroll
          for (int q = 0; q < 4; q++) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[h][8 * q + 0]) * scale, __uint_as_float(v[h][8 * q + 1]) * scale);
            o.y = pack_bf16x2(__uint_as_float(v[h][8 * q + 2]) * scale, __uint_as_float(v[h][8 * q + 3]) * scale);
            o.z = pack_bf16x2(__uint_as_float(v[h][8 * q + 4]) * scale, __uint_as_float(v[h][8 * q + 5]) * scale);
            o.w = pack_bf16x2(__uint_as_float(v[h][8 * q + 6]) * scale, __uint_as_float(v[h][8 * q + 7]) * scale);
            const int chunk = h * 4 + q;   // 16-byte chunk inside the 128-byte row; swizzled like the tensor map expects
            *reinterpret_cast<uint4*>(buf + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = o;
          }
        }
        fence_proxy_async_shared();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(tmD, buf, n * BN + c * kStoreCols, drow + lane_base);
          bulk_commit();
        }
      }
      if (p.stamps && threadIdx.x == 64) p.stamps[blockIdx.x * 8 + 3] = globaltimer();

      // ---- publish the tile
      const bool chain_signal = p.mode == kModeChain && (p.dep_offsets != nullptr || p.chunk_dst != nullptr);
      if (chain_signal || p.mode == kModeTpProducer) {
        if (lane == 0) { bulk_wait<0>(); fence_proxy_async(); mbar_arrive(epi); }   // this warp's rows have reached the destination
        if (ew == 0) {
          if (!warp_wait(epi, epi_phase)) break;   // ... and so have the other three warps' rows
          epi_phase ^= 1;
          fence_acq_rel_sys();   // every publishing lane orders the tile's rows before whatever it stores below
          if (p.mode == kModeTpProducer) {
            if (lane == 0) {
              fence_acq_rel_sys();
              st_relaxed_sys(p.peer_tile_flags[dst] + (p.rank * p.ppo + m / p.world) * p.tiles_n + n, epoch);
            }
          } else {
            if (p.chunk_dst && lane == 0) st_relaxed_sys(p.chunk_dst + tile, p.chunk_value);   // tile == m * tiles_n + n
            if (p.dep_offsets) {
            const int begin = p.dep_offsets[tile], deg = p.dep_offsets[tile + 1] - begin;
            for (int i0 = 0; i0 < deg; i0 += 32) {
              const int i = i0 + lane;
              int old = 0, c = 0;
              if (i < deg) {
                c = p.dep_consumers[begin + i];
                fence_acq_rel_sys();
                old = atom_add_acq_rel_gpu(p.scoreboard + (p.rowpanel ? c * 32 : c), -1);
              }
              if (p.rowpanel) {
                // a completed row panel publishes tiles_n2 consecutive ids; the warp shares the stores
                unsigned done = __ballot_sync(0xffffffffu, i < deg && old == 1);
                while (done) {
                  const int src_lane = __ffs(done) - 1;
                  done &= done - 1;
                  const int cc = __shfl_sync(0xffffffffu, c, src_lane);
                  int base = 0;
                  if (lane == src_lane) { base = atom_add_relaxed_sys(p.dst.tail, p.tiles_n2); fence_acq_rel_sys(); }
                  base = __shfl_sync(0xffffffffu, base, src_lane);
                  for (int j = lane; j < p.tiles_n2; j += 32) st_relaxed_sys(p.dst.entries + (base + j) % p.dst.cap, cc * p.tiles_n2 + j);
                }
              } else if (i < deg && old == 1) {
                const int slot = atom_add_relaxed_sys(p.dst.tail, 1);
                st_release_sys(p.dst.entries + slot % p.dst.cap, c);
              }
            }
            }
          }
          if (p.stamps && lane == 0) p.stamps[blockIdx.x * 8 + 4] = globaltimer();
        }
      }
    }
    if (lane == 0) bulk_wait<0>();   // no bulk store may still read this CTA's shared memory at exit
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
  if (threadIdx.x == 0) {
    if (*s_abort && p.status) report_status(p.status, *s_abort, -1, 0, 0);
    if (p.stamps) p.stamps[blockIdx.x * 8 + 7] = globaltimer();
  }
}

}  // namespace ctapp
