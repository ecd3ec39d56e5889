// CTA-pair variant of the persistent GEMM: two CTAs on the two SMs of a TPC (a cluster of 2) work on one 256 x 256 output
// tile with tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows of A and ITS HALF of the B tile (128 of the 256
// weight rows), so an SM pulls 32 KiB per k-block through the L2 fabric instead of 48 KiB; the leader CTA's MMA thread
// issues one 256 x 256 x 16 instruction that reads both CTAs' shared memory and writes both CTAs' TMEM (128 accumulator
// rows each).  No TMA multicast anywhere: every load is a plain per-CTA tiled load whose completion bytes are counted on
// the leader's barrier.
//
//   leader CTA (cluster rank 0)                         peer CTA (cluster rank 1)
//   warp 0  scheduler + loader (A rows 0-127, B half 0)  warp 0  loader (A rows 128-255, B half 1), follows the leader's tile ids
//   warp 1  MMA issuer for the pair; TMEM alloc          warp 1  TMEM alloc only
//   warps 2-5 epilogue of rows 0-127                     warps 2-5 epilogue of rows 128-255
//   (256 x 512 tile: warps 2-9, two per 32-row quarter, one for either 256-column half)
//
// The protocol around the GEMM is the one of gemm_sm100.cuh.  In chain mode the protocol's tile is the pair's 256 x 256
// tile (one queue entry, one CSR row; published by the leader once both halves have landed).  In the tensor-parallel modes
// the unit stays the 128-row panel: each CTA scatters, flags and waits for its own panel.
#pragma once
#include "gemm_sm100.cuh"

namespace ctapp {

// kWide: the pair's tile is 256 x 512 (two 256-column MMAs per k step that share the A operand in shared memory): 48 KiB of
// operands per CTA and k-block for twice the work, a quarter less traffic L2 -> shared memory per FLOP than the 256 x 256
// tile.  The price: the accumulator takes all 512 TMEM columns, so the main loop of the next tile cannot start before the
// epilogue has read the accumulator, and tiles are twice as coarse.  To keep that read short the wide tile has eight epilogue
// warps; each pulls its 32 rows x 256 columns out of TMEM into registers (rounded to bf16, 128 registers), hands the
// accumulator back, and only then feeds its rows through its staging buffer to the TMA stores, beside the next tile's main
// loop.  With stores into another GPU's memory the staging buffers drain slowly; done the other way round (store a chunk,
// wait for the buffer, read the next chunk) that wait sat between two tiles' main loops: 0.725 against 0.666 ms for an
// 8192^3 stage with a peer destination.
template <bool kWide> struct Gemm2CfgT {
  static constexpr int BN = kWide ? 512 : 256;
  static constexpr int kStages = kWide ? 4 : 6;               // 192 KiB of operands in flight either way
  static constexpr int kAccs = kWide ? 1 : 2;                 // TMEM accumulators
  static constexpr int kEpiWarps = kWide ? 8 : 4;             // per CTA
  static constexpr int kThreads = 32 * (2 + kEpiWarps);
  static constexpr uint32_t kABytes = BM * BK * 2;            // this CTA's 128 rows of A
  static constexpr uint32_t kBBytes = (BN / 2) * BK * 2;      // this CTA's half of the B tile
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;  // per CTA
  static constexpr uint32_t kEpiBytes = 4 * 2 * kStageRows * kStoreCols * 2;
  static constexpr uint32_t kBarBytes = 512;
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + kEpiBytes + kBarBytes + 1024;
  static constexpr uint32_t kTmemCols = 512;
};
using Gemm2Cfg = Gemm2CfgT<false>;

// kAct: the tile's columns 0-127 are "gate" and 128-255 the matching "up" columns (the weight rows are interleaved that way
// by the caller); the epilogue writes silu(gate) * up, 128 output columns per tile, into a D of N / 2 columns.  Both factors
// are rounded to bf16 first, as a separate activation kernel reading the GEMM's bf16 output would see them.
template <bool kAct, bool kWide = false>
__global__ void __launch_bounds__(Gemm2CfgT<kWide>::kThreads, 1) gemm2_kernel(const __grid_constant__ GemmParams p) {
  static_assert(!(kAct && kWide), "the activation epilogue is built for the 256-column tile");
  using Cfg = Gemm2CfgT<kWide>;
  constexpr int kEpiWarps = Cfg::kEpiWarps;
  constexpr int S = Cfg::kStages, BN = Cfg::BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + S * Cfg::kABytes;
  uint8_t* sD = sB + S * Cfg::kBBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sD + Cfg::kEpiBytes);
  uint64_t* full = bars;                    // [S]  leader only: both CTAs' loads -> MMA
  uint64_t* empty = full + S;               // [S]  both CTAs: MMA (multicast commit) -> loaders
  uint64_t* tfull = empty + S;              // [2]  both CTAs: MMA (multicast commit) -> epilogue
  uint64_t* tempty = tfull + 2;             // [2]  leader only: both CTAs' epilogues -> MMA
  uint64_t* sfull = tempty + 2;             // [kSchedSlots] both CTAs: scheduler -> consumers of the tile id
  uint64_t* sempty = sfull + kSchedSlots;   // [kSchedSlots] leader only: all consumers of both CTAs -> scheduler
  uint64_t* drain = sempty + kSchedSlots;   // [1]  abort path only
  uint64_t* epi = drain + 1;                // [1]  this CTA's epilogue warps -> its publishing warp
  int* s_tile = reinterpret_cast<int*>(epi + 1);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_tile + kSchedSlots);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  // leader only: how many tile halves the peer has landed.  A counter, not an mbarrier: nothing stops the peer from
  // finishing two tiles before the leader's publishing warp looks, and a barrier phase that flips twice is lost.
  uint32_t* s_peer_done = reinterpret_cast<uint32_t*>(const_cast<int*>(s_abort) + 1);
  int* s_ticket = reinterpret_cast<int*>(s_peer_done + 1);   // role switching: this CTA's ticket

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();
  const bool leader = crank == 0;
  const int pair = static_cast<int>(blockIdx.x >> 1), npairs = static_cast<int>(gridDim.x >> 1);
  const int KB = (p.K + BK - 1) / BK;
  const long long limit = p.limit_ns;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; i++) { mbar_init(full + i, 1); mbar_init(empty + i, 1); }
    for (int i = 0; i < 2; i++) { mbar_init(tfull + i, 1); mbar_init(tempty + i, 2 * kEpiWarps); }
    for (int i = 0; i < kSchedSlots; i++) { mbar_init(sfull + i, 1); mbar_init(sempty + i, 2 + 2 * kEpiWarps); }   // the other loader, the MMA thread, every epilogue warp
    mbar_init(drain, 1);
    mbar_init(epi, kEpiWarps);
    *s_abort = 0;
    *s_peer_done = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.tmA);
    tma_prefetch_desc(&p.tmB);
    if (p.stamps) { p.stamps[blockIdx.x * 8 + 0] = globaltimer(); p.stamps[blockIdx.x * 8 + 6] = smid(); }
  }
  if (warp == 1) { tmem_alloc_pair(s_tmem, Cfg::kTmemCols); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();   // the other CTA's barriers are initialised before anything is sent to them
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  if (p.pdl_trigger) pdl_launch_dependents();
  if (p.pdl_wait) pdl_wait();
  const int epoch = p.epoch_ptr ? __ldcg(p.epoch_ptr) : p.epoch;
  if constexpr (!kWide) {   // the wide tile is never a tensor-parallel consumer
    if (p.mode == kModeTpConsumer) {   // mode 8: every warp, before it takes up its role in the GEMM
      if (p.red.role_r > 0) reduce_role(p.red, epoch, s_ticket);   // either CTA of a pair draws its own ticket
      else if (p.red.unit_ctr) reduce_help(p.red, epoch, p.red.help_all != 0);
    }
  }

  // a give-up in one CTA stops both
  auto abort_pair = [&](int code) {
    *s_abort = code;
    st_cluster_u32(mapa_u32(const_cast<int*>(s_abort), crank ^ 1u), static_cast<uint32_t>(code));
  };

  if (warp == 0) {
    // ============================================================ loaders (the leader's also schedules)
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; int sq = 0; uint32_t sphase = 0;
      int k_static = 0, ntiles_done = 0;
      uint32_t armed = 0, armed_parity = 0;
      uint32_t panel_seen[4] = {0, 0, 0, 0};
      int win_cur = 0;
      auto pop = [&]() -> int {
        if (p.mode == kModeChain) { const int idx = atomicAdd(p.src.head, 1); return idx < p.num_tiles ? idx : -1; }
        const int idx = pair + (k_static++) * npairs;
        return idx < p.num_tiles ? idx : -1;
      };
      int next = leader ? pop() : -1;
      bool ok = true;
      while (ok) {
        int tile;
        if (leader) {
          tile = next;
          if (tile >= 0 && p.status && ld_relaxed_gpu(p.status) != 0) tile = -1;
          if (tile >= 0 && p.mode == kModeChain && !p.skip_wait) {
            int seen;
            const int slot = queue_slot(p, tile, win_cur);
            if (!spin_acquire_sys(p.src.entries + slot, PredNe{-1}, limit, seen)) {
              report_status(p.status, kStatusTimeoutQueue, slot, 0, seen); abort_pair(kStatusTimeoutQueue); break;
            }
            if (seen < 0 || seen >= p.num_tiles) {
              report_status(p.status, kStatusBadIndex, slot, p.num_tiles, seen); abort_pair(kStatusBadIndex); break;
            }
            tile = seen;
          }
          if (!mbar_wait_cluster(sempty + sq, sphase ^ 1, s_abort, limit)) break;
          s_tile[sq] = tile;
          st_cluster_u32(mapa_u32(s_tile + sq, 1), static_cast<uint32_t>(tile));
          mbar_arrive_cluster_local(sfull + sq);
          mbar_arrive_remote(mapa_u32(sfull + sq, 1));
        } else {
          if (!mbar_wait_cluster(sfull + sq, sphase, s_abort, limit)) break;
          tile = s_tile[sq];
          mbar_arrive_remote(mapa_u32(sempty + sq, 0));
        }
        if (++sq == kSchedSlots) { sq = 0; sphase ^= 1; }
        if (tile < 0) break;
        int mp, n;
        if (p.mode == kModeChain) { mp = tile / p.tiles_n; n = tile - mp * p.tiles_n; } else decode_tile(p, tile, mp, n);
        const int m = 2 * mp + static_cast<int>(crank);   // this CTA's 128-row panel
        if (p.tile_log && leader) p.tile_log[1 + atomicAdd(p.tile_log, 1)] = (mp << 16) | n;
        if (p.stamps && ntiles_done == 0) p.stamps[blockIdx.x * 8 + 1] = globaltimer();
        if (p.mode == kModeChain && !p.skip_wait) fence_proxy_async_global();   // peer-written A rows vs the TMA loads below
        if (p.mode == kModeTpConsumer && p.panel_flag && m < p.panels && !(m < 128 && (panel_seen[m >> 5] >> (m & 31) & 1u))) {
          int seen;
          if (!spin_acquire_sys(p.panel_flag + m, PredGe{epoch}, limit, seen)) {
            report_status(p.status, kStatusTimeoutPanel, m, epoch, seen); abort_pair(kStatusTimeoutPanel); break;
          }
          fence_proxy_async_global();
          if (m < 128) panel_seen[m >> 5] |= 1u << (m & 31);   // a panel flag never goes back within a launch: ask once
        }
        const uint32_t full0 = mapa_u32(full, 0);   // the leader's full[0] as a cluster address; stages are 8 bytes apart
        next = -2;
        int chunk_upto = 0;   // k-chunks [0, chunk_upto) of this tile's rows are known to have landed
        const int nchunks = p.chunk_src ? (KB + p.chunk_kblocks - 1) / p.chunk_kblocks : 0;
        for (int kb = 0; kb < KB; kb++) {
          // k-chunk dependencies: the flag covers the pair's 256 rows; each CTA asks for itself before it loads its half
          if (p.chunk_src && !p.skip_wait && kb % p.chunk_kblocks == 0 && kb / p.chunk_kblocks >= chunk_upto) {
            chunk_upto = wait_chunks(p, mp, kb / p.chunk_kblocks, nchunks, limit);
            if (chunk_upto <= kb / p.chunk_kblocks) { abort_pair(kStatusTimeoutChunk); ok = false; break; }
          }
          if (!mbar_wait(empty + stage, phase ^ 1, s_abort, limit)) { ok = false; break; }
          if (leader) mbar_arrive_expect_tx(full + stage, 2 * Cfg::kStageBytes);   // both CTAs' bytes are counted here
          tma_load_2d_pair(sA + stage * Cfg::kABytes, &p.tmA, kb * BK, m * BM, full0 + stage * 8);
          if constexpr (kWide) {   // accumulator columns 0-255 and 256-511: each CTA supplies 128 weight rows of either half
            tma_load_2d_pair(sB + stage * Cfg::kBBytes, &p.tmB, kb * BK, n * BN + static_cast<int>(crank) * 128, full0 + stage * 8);
            tma_load_2d_pair(sB + stage * Cfg::kBBytes + Cfg::kBBytes / 2, &p.tmB, kb * BK, n * BN + 256 + static_cast<int>(crank) * 128, full0 + stage * 8);
          } else {
            tma_load_2d_pair(sB + stage * Cfg::kBBytes, &p.tmB, kb * BK, n * BN + static_cast<int>(crank) * (BN / 2), full0 + stage * 8);
          }
          armed |= 1u << stage;
          armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
          if (++stage == S) { stage = 0; phase ^= 1; }
          if (leader && kb == (KB >> 1)) next = pop();
        }
        if (leader && next == -2) next = pop();
        ntiles_done++;
      }
      if (*s_abort) {   // let the loads already issued land before the CTA goes away
        if (leader) {
          for (int s = 0; s < S; s++)
            if (armed & (1u << s)) {
              const unsigned long long t0 = globaltimer();
              while (!mbar_try_wait_cluster(full + s, (armed_parity >> s) & 1u) && globaltimer() - t0 < 2000000ull) {}
            }
        } else {
          // This CTA's loads complete on the LEADER's barriers, which it cannot wait on for itself.  Loads of stages the leader
          // armed are covered by the leader's wait above: this CTA stays resident until the closing cluster barrier, which the
          // leader reaches only after that wait.  For a stage this CTA loaded but the leader never armed (the leader gave up
          // first) there is no barrier phase to wait for; a TMA load lands within microseconds, so pause well beyond that.
          const unsigned long long t0 = globaltimer();
          while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
        }
      }
      if (p.stamps) p.stamps[blockIdx.x * 8 + 5] = static_cast<unsigned long long>(ntiles_done);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ============================================================ MMA issuer (leader only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, 256);
      int stage = 0; uint32_t phase = 0; int sq = 0; uint32_t sphase = 0; uint32_t it = 0;
      bool ok = true;
      while (ok) {
        if (!mbar_wait_cluster(sfull + sq, sphase, s_abort, limit)) break;
        const int tile = s_tile[sq];
        mbar_arrive_cluster_local(sempty + sq);
        if (++sq == kSchedSlots) { sq = 0; sphase ^= 1; }
        if (tile < 0) break;
        const uint32_t a = kWide ? 0u : (it & 1u), aphase = kWide ? (it & 1u) : ((it >> 1) & 1u);
        if (!mbar_wait_cluster(tempty + a, aphase ^ 1, s_abort, limit)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + a * BN;
        for (int kb = 0; kb < KB; kb++) {
          if (!mbar_wait_cluster(full + stage, phase, s_abort, limit)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = umma_desc_k128(sA + stage * Cfg::kABytes);
          const uint64_t bdesc = umma_desc_k128(sB + stage * Cfg::kBBytes);
          const uint64_t bdesc2 = umma_desc_k128(sB + stage * Cfg::kBBytes + Cfg::kBBytes / 2);   // wide tile: each CTA's other 128 weight rows
#pragma unroll
          for (int k = 0; k < BK / 16; k++) {
            tc_mma_f16_pair(d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
            if constexpr (kWide) tc_mma_f16_pair(d + 256, adesc + 2 * k, bdesc2 + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);   // same A
          }
          tc_commit_pair(empty + stage, 3);   // frees the stage in both CTAs
          if (++stage == S) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit_pair(tfull + a, 3);         // both CTAs' epilogues
        if (p.stamps) p.stamps[blockIdx.x * 8 + 2] = globaltimer();
        it++;
      }
      if (*s_abort) {
        tc_commit_pair(drain, 1);
        const unsigned long long t0 = globaltimer();
        while (!mbar_try_wait(drain, 0) && globaltimer() - t0 < 2000000ull) {}
      }
    }
    __syncwarp();
  } else {
    // ============================================================ epilogue (warps 2..5; wide tile: 2..9), this CTA's 128 rows
    const int ew = warp - 2;
    const int lane_base = (warp & 3) * 32;    // a warp reads the TMEM lanes of its index modulo 4
    const int row_in_tile = lane_base + lane;
    // two staging buffers per warp; the wide tile's eight warps have one each (their stores are off the critical path)
    uint8_t* stage_buf = sD + ew * ((kWide ? 1 : 2) * kStageRows * kStoreCols * 2);
    int sq = 0; uint32_t sphase = 0; uint32_t it = 0; uint32_t cbuf = 0; uint32_t epi_phase = 0, published = 0;
    bool ready_checked = p.dst_ready == nullptr;
    uint32_t epi_seen[4] = {0, 0, 0, 0};
    auto warp_wait = [&](uint64_t* bar, uint32_t parity) -> bool {
      const bool ok = mbar_wait_cluster(bar, parity, s_abort, limit);
      return __all_sync(0xffffffffu, ok);
    };
    while (true) {
      if (!warp_wait(sfull + sq, sphase)) break;
      const int tile = s_tile[sq];
      __syncwarp();
      if (lane == 0) { if (leader) mbar_arrive_cluster_local(sempty + sq); else mbar_arrive_remote(mapa_u32(sempty + sq, 0)); }
      if (++sq == kSchedSlots) { sq = 0; sphase ^= 1; }
      if (tile < 0) break;
      int mp, n;
      if (p.mode == kModeChain) { mp = tile / p.tiles_n; n = tile - mp * p.tiles_n; } else decode_tile(p, tile, mp, n);
      const int m = 2 * mp + static_cast<int>(crank);
      const bool valid = m < p.panels;            // an odd panel count leaves the last pair's second half empty
      const uint32_t a = kWide ? 0u : (it & 1u), aphase = kWide ? (it & 1u) : ((it >> 1) & 1u);
      it++;
      if (!warp_wait(tfull + a, aphase)) break;
      tc_fence_after();

      float scale = 1.0f;
      if (p.mode == kModeTpConsumer && p.rowss && valid) {
        if (p.panel_flag && !(m < 128 && (epi_seen[m >> 5] >> (m & 31) & 1u))) {   // rowss was pushed before the flag: acquire once per panel
          if (lane == 0) (void)ld_acquire_sys(p.panel_flag + m);
          if (m < 128) epi_seen[m >> 5] |= 1u << (m & 31);
        }
        __syncwarp();
        const int row = m * BM + row_in_tile;
        if (row < p.M) scale = rsqrtf(__ldcg(p.rowss + row) * p.inv_k + p.eps);
      }
      if (!ready_checked) {
        int okr = 1;
        if (lane == 0) {
          int seen;
          if (!spin_acquire_sys(p.dst_ready, PredGe{p.ready_value}, limit, seen)) {
            report_status(p.status, kStatusTimeoutReady, 0, p.ready_value, seen); abort_pair(kStatusTimeoutReady); okr = 0;
          }
        }
        okr = __shfl_sync(0xffffffffu, okr, 0);
        if (!okr) break;
        ready_checked = true;
      }
      int dst = 0, drow = m * BM;
      if (p.mode == kModeTpProducer) { dst = m % p.world; drow = p.dst_global ? m * BM : (m / p.world) * BM; }
      const CUtensorMap* tmD = &p.tmD[dst];

      const uint32_t tcol = tmem_base + (static_cast<uint32_t>(lane_base) << 16) + a * BN;
      constexpr int kChunks = kAct ? BN / (2 * kStoreCols) : BN / kStoreCols;   // 64 output columns per chunk
      if constexpr (kWide) {
        // this warp's 32 rows x 256 columns: four chunks of 64 columns, all of them into registers as bf16 pairs, then the
        // accumulator goes back to the MMA thread, then the stores
        constexpr int kMine = kChunks / 2;
        const int col_half = (ew >> 2) * (BN / 2);
        uint32_t pk[kMine][32];
#pragma unroll
        for (int c = 0; c < kMine; c++) {
          uint32_t v[2][32];
          tc_ld_32x32b_x32(tcol + col_half + c * kStoreCols, v[0]);
          tc_ld_32x32b_x32(tcol + col_half + c * kStoreCols + 32, v[1]);
          tc_wait_ld();
          if (c == kMine - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { if (leader) mbar_arrive_cluster_local(tempty + a); else mbar_arrive_remote(mapa_u32(tempty + a, 0)); }
          }
#pragma unroll
          for (int h = 0; h < 2; h++)
#pragma unroll
            for (int j = 0; j < 16; j++) pk[c][h * 16 + j] = pack_bf16x2(__uint_as_float(v[h][2 * j]), __uint_as_float(v[h][2 * j + 1]));
        }
        if (valid) {
#pragma unroll
          for (int c = 0; c < kMine; c++) {
            if (lane == 0) bulk_wait_read<0>();   // this warp's one staging buffer
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 8; q++) {      // 16-byte piece q of this lane's 128-byte row, in the 128-byte swizzle TMA expects
              const uint4 o = make_uint4(pk[c][4 * q], pk[c][4 * q + 1], pk[c][4 * q + 2], pk[c][4 * q + 3]);
              *reinterpret_cast<uint4*>(stage_buf + lane * 128 + ((q ^ (lane & 7)) << 4)) = o;
            }
            fence_proxy_async_shared();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(tmD, stage_buf, n * BN + col_half + c * kStoreCols, drow + lane_base);
              bulk_commit();
            }
          }
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < kChunks; c++) {
        uint32_t v[2][32];
        uint32_t u[kAct ? 2 : 1][kAct ? 32 : 1];
        tc_ld_32x32b_x32(tcol + c * kStoreCols, v[0]);
        tc_ld_32x32b_x32(tcol + c * kStoreCols + 32, v[1]);
        if constexpr (kAct) {
          tc_ld_32x32b_x32(tcol + BN / 2 + c * kStoreCols, u[0]);
          tc_ld_32x32b_x32(tcol + BN / 2 + c * kStoreCols + 32, u[1]);
        }
        tc_wait_ld();
        if (c == kChunks - 1) {   // accumulator fully read: hand it back to the pair's MMA thread
          tc_fence_before();
          __syncwarp();
          if (lane == 0) { if (leader) mbar_arrive_cluster_local(tempty + a); else mbar_arrive_remote(mapa_u32(tempty + a, 0)); }
        }
        if (!valid) continue;
        uint8_t* buf = stage_buf + (cbuf & 1u) * (kStageRows * kStoreCols * 2);
        cbuf++;
        if (lane == 0) bulk_wait_read<1>();
        __syncwarp();
        auto val = [&](int h, int i) -> float {
          const float g = __uint_as_float(v[h][i]) * scale;
          if constexpr (kAct) {
            const float gb = bf16_round(g), ub = bf16_round(__uint_as_float(u[h][i]) * scale);
            return gb / (1.0f + __expf(-gb)) * ub;
          } else {
            return g;
          }
        };
#pragma unroll
        for (int h = 0; h < 2; h++) {
#pragma unroll
          for (int q = 0; q < 4; q++) {
            uint4 o;
            o.x = pack_bf16x2(val(h, 8 * q + 0), val(h, 8 * q + 1));
            o.y = pack_bf16x2(val(h, 8 * q + 2), val(h, 8 * q + 3));
            o.z = pack_bf16x2(val(h, 8 * q + 4), val(h, 8 * q + 5));
            o.w = pack_bf16x2(val(h, 8 * q + 6), val(h, 8 * q + 7));
            const int chunk = h * 4 + q;
            *reinterpret_cast<uint4*>(buf + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = o;
          }
        }
        fence_proxy_async_shared();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(tmD, buf, n * (kAct ? BN / 2 : BN) + c * kStoreCols, drow + lane_base);
          bulk_commit();
        }
      }
      }
      if (p.stamps && threadIdx.x == 64) p.stamps[blockIdx.x * 8 + 3] = globaltimer();

      // ---- publish
      const bool chain_signal = p.mode == kModeChain && (p.dep_offsets != nullptr || p.chunk_dst != nullptr);
      if (chain_signal || (p.mode == kModeTpProducer && valid)) {
        if (lane == 0) { bulk_wait<0>(); fence_proxy_async(); mbar_arrive(epi); }
        if (ew == 0) {
          if (!warp_wait(epi, epi_phase)) break;
          epi_phase ^= 1;
          fence_acq_rel_sys();
          if (p.mode == kModeTpProducer) {
            // the owners index their tile flags in 256-column tiles: a 512-column tile raises two of them
            constexpr int kFlags = BN / 256;
            if (lane < kFlags) st_relaxed_sys(p.peer_tile_flags[dst] + (p.rank * p.ppo + m / p.world) * (kFlags * p.tiles_n) + kFlags * n + lane, epoch);
          } else if (!leader) {
            if (lane == 0) red_add_release_cluster(mapa_u32(s_peer_done, 0), 1);   // this half of the pair tile has landed
          } else {
            published++;
            int okp = 1;
            if (lane == 0) {                                       // ... and so has the peer's half
              const unsigned long long t0 = globaltimer();
              unsigned polls = 0;
              while (ld_acquire_cluster_u32(s_peer_done) < published) {
                if ((++polls & 255u) == 0 && (*s_abort || static_cast<long long>(globaltimer() - t0) > 4 * limit)) {
                  if (!*s_abort) abort_pair(kStatusTimeoutPipe);
                  okp = 0;
                  break;
                }
              }
            }
            if (!__shfl_sync(0xffffffffu, okp, 0)) break;
            fence_acq_rel_sys();
            if (p.chunk_dst && lane == 0) st_relaxed_sys(p.chunk_dst + tile, p.chunk_value);   // tile == mp * tiles_n + n
            const int begin = p.dep_offsets ? p.dep_offsets[tile] : 0, deg = p.dep_offsets ? p.dep_offsets[tile + 1] - begin : 0;
            for (int i0 = 0; i0 < deg; i0 += 32) {
              const int i = i0 + lane;
              int old = 0, c = 0;
              if (i < deg) {
                c = p.dep_consumers[begin + i];
                old = atom_add_acq_rel_gpu(p.scoreboard + (p.rowpanel ? c * 32 : c), -1);
              }
              if (p.rowpanel) {
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
          if (p.stamps && lane == 0) p.stamps[blockIdx.x * 8 + 4] = globaltimer();
        }
      }
    }
    if (lane == 0) bulk_wait<0>();
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  cluster_arrive();   // nothing of this CTA (barriers, shared memory, TMEM) is touched by the other one after this point
  cluster_wait();
  if (warp == 1) tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
  if (threadIdx.x == 0) {
    if (*s_abort && p.status) report_status(p.status, *s_abort, -1, 0, 0);
    if (p.stamps) p.stamps[blockIdx.x * 8 + 7] = globaltimer();
  }
}

}  // namespace ctapp
