// TMA-fed owner reducer: the same work and the same protocol as tp_reduce_kernel (reduce_sm100.cuh), restructured so that
// the bytes in flight per SM are set by shared memory, not by registers.
//
//   warp 0      : loader.  For each unit of this CTA, in the producer's tile order: waits (bounded) for the `world` tile flags,
//                 then brings the unit's 32 x 256 patch of every inbox slice and of the residual into a shared-memory stage
//                 with one cp.async.bulk.tensor load per source (one 16 KiB box each), completion on the stage's mbarrier.
//   warps 1-8   : adders.  Each takes 4 of the 32 rows: per row a lane reads its 16 bytes of every source from shared memory,
//                 adds left to right in fp32 (slot 0 .. world-1, then the residual), rounds once to bf16, pushes the 16 bytes
//                 to every rank (unicast st.relaxed.sys.v4, or one multimem.st), and the warp adds the row's sum of squares
//                 of the rounded values to rowss_local.
//   warp 9      : publisher.  When all adders are done with a stage it releases the stage to the loader, counts the unit on
//                 its panel (fence.acq_rel.sys + atomic) and, as the panel's last arrival, pushes the 128 row sums and the
//                 panel flag to every rank.
//
// With world = 8 a stage holds half a unit's columns (128), so three stages fit; arrivals are still counted per unit.
#pragma once
#include "reduce_sm100.cuh"

namespace ctapp {

constexpr int kRedAdders = 8;                      // adder warps
constexpr int kRedThreads = 32 * (kRedAdders + 2);  // + loader + publisher
constexpr int kRedUnitRows = 32;

struct alignas(64) ReduceTmaParams {
  CUtensorMap tmIn[9];     // [0..world-1] inbox slices (rows = ppo * 128, cols = n1); [world] residual (rows = M)
  ReduceParams r;
  int has_resid;
};

template <int W> struct RedTmaCfg {
  static constexpr int kChunkCols = W <= 4 ? 256 : 128;
  static constexpr int kChunksPerUnit = 256 / kChunkCols;
  static constexpr int kSources = W + 1;
  static constexpr uint32_t kSrcBytes = kRedUnitRows * kChunkCols * 2;
  static constexpr uint32_t kStageBytes = kSources * kSrcBytes;
  static constexpr int kStages = (200 * 1024) / kStageBytes < 2 ? 2 : ((200 * 1024) / kStageBytes > 6 ? 6 : (200 * 1024) / kStageBytes);
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

template <int W, bool MC>
__global__ void __launch_bounds__(kRedThreads, 1) tp_reduce_tma_kernel(const __grid_constant__ ReduceTmaParams tp) {
  using Cfg = RedTmaCfg<W>;
  constexpr int S = Cfg::kStages;
  const ReduceParams& p = tp.r;
  extern __shared__ uint8_t red_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(red_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S * Cfg::kStageBytes);   // loader -> adders
  uint64_t* done = full + S;                                                   // adders -> publisher
  uint64_t* empty = done + S;                                                  // publisher -> loader
  int* s_unit = reinterpret_cast<int*>(empty + S);                             // [S] which (unit, chunk) a stage holds, -1 = stop
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_unit + S);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int epoch = p.epoch_ptr ? __ldcg(p.epoch_ptr) : p.epoch;
  const int P = p.M / 128;
  const int Pr = P > p.rank ? (P - 1 - p.rank) / W + 1 : 0;
  const int tiles_n = p.n1 / 256;
  const int units_per_panel = tiles_n * 4;
  const int U = Pr * units_per_panel;
  const int row_vecs = p.n1 / 8;
  const long long limit = p.limit_ns;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; i++) { mbar_init(full + i, 1); mbar_init(done + i, kRedAdders); mbar_init(empty + i, 1); }
    *s_abort = 0;
    fence_mbar_init();
  }
  __syncthreads();

  if (warp == 0) {
    // ============================================================ loader
    int stage = 0; uint32_t phase = 0;
    bool ok = true;
    for (int u = static_cast<int>(blockIdx.x); ok; u += static_cast<int>(gridDim.x)) {
      const bool stop = u >= U || (p.status && ld_relaxed_gpu(p.status) != 0);
      int j = 0, n = 0, q = 0;
      if (!stop) {
        unit_map(u, Pr, tiles_n, p.tail, j, n, q);
        bool got = true;
        if (lane < W) {
          int seen;
          const int idx = (lane * p.ppo + j) * tiles_n + n;
          if (!spin_acquire_sys(p.tile_flags + idx, PredGe{epoch}, limit, seen)) {
            report_status(p.status, kStatusTimeoutTile, idx, epoch, seen);
            got = false;
          }
        }
        if (!__all_sync(0xffffffffu, got)) { if (lane == 0) *s_abort = kStatusTimeoutTile; break; }
        fence_proxy_async_global();   // the inbox rows were written by other GPUs; the loads below go through the async proxy
      }
      for (int c = 0; c < (stop ? 1 : Cfg::kChunksPerUnit); c++) {
        int okw = 1;
        if (lane == 0) {
          okw = mbar_wait(empty + stage, phase ^ 1, s_abort, limit) ? 1 : 0;
          if (okw) {
            s_unit[stage] = stop ? -1 : u * Cfg::kChunksPerUnit + c;
            if (stop) {
              mbar_arrive(full + stage);
            } else {
              mbar_arrive_expect_tx(full + stage, (W + tp.has_resid) * Cfg::kSrcBytes);
              uint8_t* dst = smem + stage * Cfg::kStageBytes;
              const int col = n * 256 + c * Cfg::kChunkCols;
#pragma unroll
              for (int s = 0; s < W; s++) tma_load_2d(dst + s * Cfg::kSrcBytes, &tp.tmIn[s], col, j * 128 + q * 32, full + stage);
              if (tp.has_resid) tma_load_2d(dst + W * Cfg::kSrcBytes, &tp.tmIn[W], col, (j * W + p.rank) * 128 + q * 32, full + stage);
            }
          }
        }
        okw = __shfl_sync(0xffffffffu, okw, 0);
        if (!okw) { ok = false; break; }
        if (++stage == S) { stage = 0; phase ^= 1; }
      }
      if (stop) break;
    }
    if (*s_abort && lane == 0) {   // give loads that are still in flight time to land before the CTA goes away
      const unsigned long long t0 = globaltimer();
      while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
    }
  } else if (warp <= kRedAdders) {
    // ============================================================ adders
    const int aw = warp - 1;                       // rows aw * 4 .. aw * 4 + 3 of the unit
    int stage = 0; uint32_t phase = 0;
    while (true) {
      const bool okw = __all_sync(0xffffffffu, mbar_wait(full + stage, phase, s_abort, limit));
      if (!okw) break;
      const int uc = s_unit[stage];
      if (uc < 0) break;
      const int u = uc / Cfg::kChunksPerUnit, c = uc - u * Cfg::kChunksPerUnit;
      int j, n, q;
      unit_map(u, Pr, tiles_n, p.tail, j, n, q);
      const int m = j * W + p.rank;
      const uint8_t* src = smem + stage * Cfg::kStageBytes;
      constexpr int kLanesPerRow = Cfg::kChunkCols / 8;           // 16-byte pieces per row of the chunk: 32 or 16
      constexpr int kRowsPerPass = 32 / kLanesPerRow;             // 1 or 2 rows per warp pass
#pragma unroll
      for (int rr = 0; rr < 4; rr += kRowsPerPass) {
        const int r = aw * 4 + rr + lane / kLanesPerRow;          // row inside the unit
        const int piece = lane % kLanesPerRow;
        const uint32_t soff = static_cast<uint32_t>(r) * (Cfg::kChunkCols * 2) + piece * 16;
        uint4 a[W];
#pragma unroll
        for (int s = 0; s < W; s++) a[s] = *reinterpret_cast<const uint4*>(src + s * Cfg::kSrcBytes + soff);
        const uint4 rv = tp.has_resid ? *reinterpret_cast<const uint4*>(src + W * Cfg::kSrcBytes + soff) : make_uint4(0, 0, 0, 0);
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
          float lo = 0.f, hi = 0.f;
#pragma unroll
          for (int s = 0; s < W; s++) {
            const float2 f = unpack_bf16x2((&a[s].x)[i]);
            if (s == 0) { lo = f.x; hi = f.y; } else { lo += f.x; hi += f.y; }
          }
          const float2 fr = unpack_bf16x2((&rv.x)[i]);
          o[i] = pack_bf16x2(lo + fr.x, hi + fr.y);
        }
        const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
        const int xrow = m * 128 + q * 32 + r;
        const size_t xoff = static_cast<size_t>(xrow) * row_vecs + n * 32 + c * (Cfg::kChunkCols / 8) + piece;
        if (MC) {
          multimem_st_v4(p.x_mc + xoff, ov);
        } else {
#pragma unroll
          for (int d = 1; d <= W; d++) st_relaxed_sys_v4(p.x[(p.rank + d) % W] + xoff, ov);
        }
        float ss = sumsq_bf16x8(ov);
#pragma unroll
        for (int sh = kLanesPerRow / 2; sh > 0; sh >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sh);
        if (piece == 0) atomicAdd(p.rowss_local + xrow, ss);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(done + stage);   // release: this warp's stores and atomics are ordered before the publisher's fence
      if (++stage == S) { stage = 0; phase ^= 1; }
    }
  } else {
    // ============================================================ publisher
    int stage = 0; uint32_t phase = 0;
    // the stop marker is not added by anyone: the publisher sees it when the loader's bare arrive completes `full`
    while (true) {
      bool okw = __all_sync(0xffffffffu, mbar_wait(full + stage, phase, s_abort, limit));
      if (!okw) break;
      const int uc = s_unit[stage];
      if (uc < 0) break;
      okw = __all_sync(0xffffffffu, mbar_wait(done + stage, phase, s_abort, limit));
      if (!okw) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(empty + stage);   // every adder has read the stage: the loader may refill it
      const int u = uc / Cfg::kChunksPerUnit, c = uc - u * Cfg::kChunksPerUnit;
      if (c == Cfg::kChunksPerUnit - 1) {          // the unit is complete
        int j, n, q;
        unit_map(u, Pr, tiles_n, p.tail, j, n, q);
        const int m = j * W + p.rank;
        int last = 0;
        if (lane == 0) {
          fence_acq_rel_sys();
          last = atom_add_relaxed_gpu(p.panel_done + m, 1) == units_per_panel - 1;
        }
        if (__shfl_sync(0xffffffffu, last, 0)) {
          if (lane == 0) fence_acq_rel_sys();
          __syncwarp();
          const float4 v = __ldcg(reinterpret_cast<const float4*>(p.rowss_local + m * 128) + lane);
          if (MC) {
            multimem_st_f32x4(p.rowss_mc + m * 128 + lane * 4, v);
          } else {
#pragma unroll
            for (int d = 1; d <= W; d++) st_relaxed_sys_f32x4(p.rowss[(p.rank + d) % W] + m * 128 + lane * 4, v);
          }
          __syncwarp();
          if (lane == 0) {
            fence_acq_rel_sys();
            if (MC) {
              multimem_st_release_b32(p.panel_flag_mc + m, epoch);
            } else {
#pragma unroll
              for (int d = 1; d <= W; d++) st_relaxed_sys(p.panel_flag[(p.rank + d) % W] + m, epoch);
            }
            if (p.trace) p.trace[m] = globaltimer();
          }
          __syncwarp();
        }
      }
      if (++stage == S) { stage = 0; phase ^= 1; }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && *s_abort && p.status) report_status(p.status, *s_abort, -1, 0, 0);
}

}  // namespace ctapp
