// Owner reducer of the tensor-parallel boundary (panel ownership, unicast value flags) and its helpers.
//
// Rank r owns the 128-row panels m with m % world == r.  Every rank's producer GEMM stores its partial of tile
// (m, n) into slot `src` of the owner's inbox and raises tile_flags[src][m / world][n] = epoch there.  The owner
// walks its units -- (owned panel j, 256-column tile n, 32-row quarter q), one warp per unit, in the producer's
// tile order -- waits for the `world` flags of the unit's tile, and for each row computes
//     x = bf16( p_0 + p_1 + ... + p_{world-1} + resid )         fp32, added left to right
// stores x to every rank (local copy last), accumulates the row's sum of squares of the ROUNDED x, and counts the
// unit on the panel.  The warp that completes a panel pushes the panel's 128 row sums and then panel_flag[m] = epoch
// to every rank.
#pragma once
#include "ptx.cuh"

namespace ctapp {

struct ReduceParams {
  int M, n1, rank, world;
  int epoch; const int* epoch_ptr;
  const int* tile_flags;
  const uint4* inbox[8];
  const uint4* resid;
  uint4* x[8];
  float* rowss[8];
  int* panel_flag[8];
  float* rowss_local;
  int* panel_done;
  int ppo, tail;
  int order, swz;            // unit order when tail == 0: 1 = m fastest in groups of swz n-tiles, 2 = panel by panel
  int* unit_ctr;             // non-null: units are claimed from this counter (shared with consumer CTAs that help)
  int* unit_log;             // non-null: [0] = count, then one packed (j << 16 | n << 2 | q) per processed unit, in claim order
  unsigned long long* trace;
  int* status;
  long long limit_ns;
  int pdl_trigger;           // raise the programmatic-launch trigger at entry (the producer GEMM is this kernel's dependent)
  int help_all;              // helpers (consumer CTAs): 1 = take every unit, waiting for tiles (no dedicated reducer CTAs run)
  // NVLS variant: multicast addresses of the x buffer, the row-sum buffer and the panel flags (null = unicast pushes)
  uint4* x_mc;
  float* rowss_mc;
  int* panel_flag_mc;
  // in-switch reduction: multicast address of the ranks' partial-sum buffers ((M, n1) bf16, every rank's own producer output at
  // the same offset); null = the partials are read from the local inbox slices
  const uint4* partials_mc;
  // role switching (consumer mode 8 only): the first role_r CTAs of the consumer GEMM to arrive (tickets from role_ctr, zeroed
  // per step) ARE the owner reducer -- each runs the static share `ticket` of `role_r` -- before they take GEMM tiles
  int* role_ctr;
  int role_r;
};

// Unit u -> (owned panel j, n-tile, quarter).  The order follows the producer's tile order so that units become ready in
// the order they are visited:
//   tail > 0            m-fast head over the first tiles_n - tail n-tiles, then panel-major over the last `tail` n-tiles
//   order 1, swz <= 1   n-major: for each n-tile, every owned panel
//   order 1, swz > 1    groups of swz n-tiles: for each group, for each owned panel, the group's n-tiles
//   order 2             panel by panel
// Same integer function as the reference's red5_map (csrc/ctapp_tp4.cuh:551-565) with the n-tile count as a parameter.
__device__ __forceinline__ void unit_map(int u, int Pr, int tiles_n, int tail, int order, int swz, int& j, int& n, int& q) {
  q = u & 3;
  const int t = u >> 2;
  if (tail > 0) {
    const int head = Pr * (tiles_n - tail);
    if (t < head) { n = t / Pr; j = t - n * Pr; }
    else { const int t2 = t - head; j = t2 / tail; n = tiles_n - tail + (t2 - j * tail); }
    return;
  }
  if (order == 2) { j = t / tiles_n; n = t - j * tiles_n; return; }
  if (swz <= 1) { n = t / Pr; j = t - n * Pr; return; }
  const int g = t / swz;
  j = g % Pr;
  n = (g / Pr) * swz + t % swz;
}

// acc + (low | high) half of a packed bf16 pair, in fp32: the conversion is part of the add (sm_100 mixed-precision add)
__device__ __forceinline__ float add_bf16_lo(float acc, uint32_t v) {
  float d;
  asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tadd.rn.f32.bf16 %0, lo, %1;\n\t}" : "=f"(d) : "f"(acc), "r"(v));
  return d;
}
__device__ __forceinline__ float add_bf16_hi(float acc, uint32_t v) {
  float d;
  asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tadd.rn.f32.bf16 %0, hi, %1;\n\t}" : "=f"(d) : "f"(acc), "r"(v));
  return d;
}
// acc + h * h for both halves of a packed bf16 pair
__device__ __forceinline__ float sq_bf16x2(float acc, uint32_t v) {
  float d;
  asm("{\n\t.reg .b16 lo, hi;\n\t.reg .f32 t;\n\tmov.b32 {lo, hi}, %2;\n\tfma.rn.f32.bf16 t, lo, lo, %1;\n\tfma.rn.f32.bf16 %0, hi, hi, t;\n\t}"
      : "=f"(d) : "f"(acc), "r"(v));
  return d;
}

__device__ __forceinline__ float sumsq_bf16x8(uint4 o) {
  float s = 0.f;
  const uint32_t w[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
  for (int i = 0; i < 4; i++) { const float2 f = unpack_bf16x2(w[i]); s = fmaf(f.x, f.x, s); s = fmaf(f.y, f.y, s); }
  return s;
}

// One unit, by one warp: 32 rows x 256 columns of x.  Returns false when a tile flag never arrived (status written).
//   * lanes 0..W-1 wait (bounded) for the W tile flags of the unit's tile
//   * per batch of ROWS rows: every lane loads its 16 bytes of every source and of the residual, adds them in fp32 in slot
//     order (the residual last) starting from -0.0 so that the first add is exact, rounds once to bf16, pushes the 16 bytes
//     to every rank (remote copies first, the local one last; or one multimem store), and squares the ROUNDED values
//   * the ROWS row sums are folded across the warp by halving (ROWS values -> one per lane group) and added to rowss_local
//     by ROWS lanes at once
//   * lane 0 orders everything above before the panel's arrival count; the warp that completes the panel pushes the panel's
//     128 row sums and then panel_flag[m] = epoch to every rank
// LR (needs MC): the W partials are not read from the inbox but summed by the NVSwitch: one multimem.ld_reduce (fp32
// accumulation in the switch, bf16 result) on the multicast address of the ranks' partial buffers replaces the W loads and adds.
template <int W, int ROWS, bool MC, bool LR = false>
__device__ __forceinline__ bool reduce_unit(const ReduceParams& p, int epoch, int u, int Pr, int tiles_n, int lane) {
  static_assert(ROWS == 1 || ROWS == 2 || ROWS == 4, "rows per batch");
  int j, n, q;
  unit_map(u, Pr, tiles_n, p.tail, p.order, p.swz, j, n, q);
  if (p.unit_log && lane == 0) p.unit_log[1 + atomicAdd(p.unit_log, 1)] = (j << 16) | (n << 2) | q;
  bool ok = true;
  if (lane < W) {
    int seen;
    const int idx = (lane * p.ppo + j) * tiles_n + n;
    if (!spin_acquire_sys(p.tile_flags + idx, PredGe{epoch}, p.limit_ns, seen)) {
      report_status(p.status, kStatusTimeoutTile, idx, epoch, seen);
      ok = false;
    }
  }
  if (!__all_sync(0xffffffffu, ok)) return false;
  const int row_vecs = p.n1 / 8;                 // 16-byte vectors per row
  const int m = j * W + p.rank;
  const int xrow0 = m * 128 + q * 32;
  // every source slice has the same geometry: one running offset serves all of them (the bases sit in the parameter bank)
  size_t ioff = static_cast<size_t>(j * 128 + q * 32) * row_vecs + n * 32 + lane;
  size_t xoff0 = static_cast<size_t>(xrow0) * row_vecs + n * 32 + lane;
  const bool rsrc = p.resid != nullptr;
#pragma unroll 1
  for (int r = 0; r < 32; r += ROWS, ioff += static_cast<size_t>(ROWS) * row_vecs, xoff0 += static_cast<size_t>(ROWS) * row_vecs) {
    constexpr int kParts = LR ? 1 : W;
    uint4 part[ROWS][kParts], res[ROWS];
#pragma unroll
    for (int rr = 0; rr < ROWS; rr++) {
      if (LR) {
        part[rr][0] = multimem_ld_reduce_bf16x8(p.partials_mc + xoff0 + rr * row_vecs);   // the partials sit at x's own offsets
      } else {
#pragma unroll
        for (int s = 0; s < kParts; s++) part[rr][s] = __ldcg(p.inbox[s] + ioff + rr * row_vecs);
      }
    }
    if (rsrc) {
#pragma unroll
      for (int rr = 0; rr < ROWS; rr++) res[rr] = __ldg(p.resid + xoff0 + rr * row_vecs);
    }
    float ss[ROWS];
#pragma unroll
    for (int rr = 0; rr < ROWS; rr++) {
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        float lo = -0.0f, hi = -0.0f;
#pragma unroll
        for (int s = 0; s < kParts; s++) { const uint32_t w = (&part[rr][s].x)[i]; lo = add_bf16_lo(lo, w); hi = add_bf16_hi(hi, w); }
        if (rsrc) { const uint32_t w = (&res[rr].x)[i]; lo = add_bf16_lo(lo, w); hi = add_bf16_hi(hi, w); }
        o[i] = pack_bf16x2(lo, hi);
      }
      const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
      const size_t xoff = xoff0 + rr * row_vecs;
      if (MC) {
        multimem_st_v4(p.x_mc + xoff, ov);
      } else {
#pragma unroll
        for (int d = 1; d <= W; d++) st_relaxed_sys_v4(p.x[(p.rank + d) % W] + xoff, ov);
      }
      ss[rr] = sq_bf16x2(sq_bf16x2(sq_bf16x2(sq_bf16x2(0.f, o[0]), o[1]), o[2]), o[3]);
    }
    // fold ROWS sums across the warp: after the halving steps lane l holds (part of) row (l / (32 / ROWS))'s sum
    float v;
    if (ROWS == 4) {
      const bool up = lane & 16;
      float k0 = up ? ss[2] : ss[0], k1 = up ? ss[3] : ss[1];
      k0 += __shfl_xor_sync(0xffffffffu, up ? ss[0] : ss[2], 16);
      k1 += __shfl_xor_sync(0xffffffffu, up ? ss[1] : ss[3], 16);
      const bool up8 = lane & 8;
      v = (up8 ? k1 : k0) + __shfl_xor_sync(0xffffffffu, up8 ? k0 : k1, 8);
#pragma unroll
      for (int sh = 4; sh > 0; sh >>= 1) v += __shfl_xor_sync(0xffffffffu, v, sh);
      if ((lane & 7) == 0) atomicAdd(p.rowss_local + xrow0 + r + (lane >> 3), v);
    } else if (ROWS == 2) {
      const bool up = lane & 16;
      v = (up ? ss[1] : ss[0]) + __shfl_xor_sync(0xffffffffu, up ? ss[0] : ss[1], 16);
#pragma unroll
      for (int sh = 8; sh > 0; sh >>= 1) v += __shfl_xor_sync(0xffffffffu, v, sh);
      if ((lane & 15) == 0) atomicAdd(p.rowss_local + xrow0 + r + (lane >> 4), v);
    } else {
      v = ss[0];
#pragma unroll
      for (int sh = 16; sh > 0; sh >>= 1) v += __shfl_xor_sync(0xffffffffu, v, sh);
      if (lane == 0) atomicAdd(p.rowss_local + xrow0 + r, v);
    }
  }
  __syncwarp();
  const int units_per_panel = tiles_n * 4;
  int last = 0;
  if (lane == 0) {
    fence_acq_rel_sys();   // this warp's x stores and row-sum atomics before the arrival count
    last = atom_add_relaxed_gpu(p.panel_done + m, 1) == units_per_panel - 1;
  }
  if (__shfl_sync(0xffffffffu, last, 0)) {
    if (lane == 0) fence_acq_rel_sys();   // acquire side: the other warps' stores and atomics of this panel
    __syncwarp();
    const float4 sums = __ldcg(reinterpret_cast<const float4*>(p.rowss_local + m * 128) + lane);
    if (MC) {
      multimem_st_f32x4(p.rowss_mc + m * 128 + lane * 4, sums);
    } else {
#pragma unroll
      for (int d = 1; d <= W; d++) st_relaxed_sys_f32x4(p.rowss[(p.rank + d) % W] + m * 128 + lane * 4, sums);
    }
    __syncwarp();
    if (lane == 0) {
      fence_acq_rel_sys();   // x (all warps, through the arrival chain) and the row sums before the flags
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
  return true;
}

// The unit loop of one warp.  Static assignment: unit = first, first + stride, ...; with p.unit_ctr every warp claims its
// next unit from the shared counter instead (first / stride unused), which lets CTAs of another kernel join in.
// kOnlyReady (helpers from another kernel): a warp takes a unit only while the NEXT unclaimed unit's tile has already arrived,
// i.e. while the dedicated reducer CTAs are behind the producers; once the reducers keep pace it leaves instead of waiting.
template <int W, int ROWS, bool MC, bool kOnlyReady = false, bool LR = false>
__device__ __forceinline__ void reduce_units(const ReduceParams& p, int epoch, int first, int stride, int lane) {
  const int P = p.M / 128;
  const int Pr = P > p.rank ? (P - 1 - p.rank) / W + 1 : 0;
  const int tiles_n = p.n1 / 256;
  const int U = Pr * tiles_n * 4;
  auto claim = [&]() -> int {
    if (kOnlyReady) {
      int next = 0;
      if (lane == 0) next = ld_relaxed_gpu(p.unit_ctr);
      next = __shfl_sync(0xffffffffu, next, 0);
      if (next >= U) return U;
      int j, n, q;
      unit_map(next, Pr, tiles_n, p.tail, p.order, p.swz, j, n, q);
      const bool up = lane >= W || ld_relaxed_sys(p.tile_flags + (lane * p.ppo + j) * tiles_n + n) >= epoch;
      if (!__all_sync(0xffffffffu, up)) return U;
    }
    int v = 0;
    if (lane == 0) v = atomicAdd(p.unit_ctr, 1);
    return __shfl_sync(0xffffffffu, v, 0);
  };
  for (int u = p.unit_ctr ? claim() : first; u < U; u = p.unit_ctr ? claim() : u + stride)
    if (!reduce_unit<W, ROWS, MC, LR>(p, epoch, u, Pr, tiles_n, lane)) return;   // a producer never delivered: the host reads the status
}

// rows per batch: as many as the register file of a 1024-thread CTA allows (64 registers per thread)
template <int W> struct RedRows { static constexpr int value = W >= 8 ? 1 : (W >= 2 ? 2 : 4); };

// MC: the pushes to every rank (x rows, row sums, panel flags) are single multimem stores on a multicast address, replicated
// by the NVSwitch, instead of one unicast store per rank; everything else is the same kernel.
template <int W, int ROWS, bool MC = false, bool LR = false>
__global__ void __launch_bounds__(1024, 1) tp_reduce_kernel(const ReduceParams p) {
  if (p.pdl_trigger) pdl_launch_dependents();
  const int epoch = p.epoch_ptr ? __ldcg(p.epoch_ptr) : p.epoch;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  reduce_units<W, ROWS, MC, false, LR>(p, epoch, warp * static_cast<int>(gridDim.x) + static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x) * nwarps, lane);
}

// Consumer CTAs helping the owner reducer (any CTA shape): every warp claims units while there are units whose tiles have
// arrived and that nobody has taken (`all`: until no unit is left at all, waiting for tiles where necessary: for a launch without
// dedicated reducer CTAs).
__device__ __forceinline__ void reduce_help(const ReduceParams& p, int epoch, bool all) {
  const int lane = threadIdx.x & 31;
  if (!p.unit_ctr) return;
  const bool mc = p.x_mc != nullptr;
#define CTAPP_HELP(W, R)                                                                                          \
  do {                                                                                                              \
    if (all) { if (mc) reduce_units<W, R, true, false>(p, epoch, 0, 0, lane); else reduce_units<W, R, false, false>(p, epoch, 0, 0, lane); } \
    else { if (mc) reduce_units<W, R, true, true>(p, epoch, 0, 0, lane); else reduce_units<W, R, false, true>(p, epoch, 0, 0, lane); }     \
  } while (0)
  switch (p.world) {
    case 1: if (all) reduce_units<1, 4, false, false>(p, epoch, 0, 0, lane); else reduce_units<1, 4, false, true>(p, epoch, 0, 0, lane); break;
    case 2: CTAPP_HELP(2, 2); break;
    case 4: CTAPP_HELP(4, 2); break;
    default: CTAPP_HELP(8, 1); break;
  }
#undef CTAPP_HELP
}

// Role switching (same integer contract as the reference's tp4_role_preamble, csrc/ctapp_tp4.cuh:913-925): every CTA of the
// consumer GEMM draws a ticket; tickets below role_r run the owner reducer's static share ticket / role_r with all their warps,
// the others return at once.  `s_ticket`: one word of shared memory nothing else uses.  Every thread of the CTA calls this.
__device__ __forceinline__ void reduce_role(const ReduceParams& p, int epoch, int* s_ticket) {
  if (threadIdx.x == 0) *s_ticket = atomicAdd(p.role_ctr, 1);
  __syncthreads();
  const int role = *s_ticket;
  if (role >= p.role_r) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int first = warp * p.role_r + role, stride = p.role_r * nwarps;
  const bool mc = p.x_mc != nullptr;
  switch (p.world) {
    case 1: reduce_units<1, 4, false>(p, epoch, first, stride, lane); break;
    case 2: if (mc) reduce_units<2, 2, true>(p, epoch, first, stride, lane); else reduce_units<2, 2, false>(p, epoch, first, stride, lane); break;
    case 4: if (mc) reduce_units<4, 2, true>(p, epoch, first, stride, lane); else reduce_units<4, 2, false>(p, epoch, first, stride, lane); break;
    default: if (mc) reduce_units<8, 1, true>(p, epoch, first, stride, lane); else reduce_units<8, 1, false>(p, epoch, first, stride, lane); break;
  }
}

// Read-back of the unit order: out[3 u .. 3 u + 2] = (j, n, q) for every unit of a rank with Pr owned panels.
__global__ void unit_order_kernel(int Pr, int tiles_n, int tail, int order, int swz, int* out) {
  const int U = Pr * tiles_n * 4;
  for (int u = blockIdx.x * blockDim.x + threadIdx.x; u < U; u += gridDim.x * blockDim.x) {
    int j, n, q;
    unit_map(u, Pr, tiles_n, tail, order, swz, j, n, q);
    out[3 * u] = j; out[3 * u + 1] = n; out[3 * u + 2] = q;
  }
}

// ------------------------------------------------------------------------------------------ NVLS known-answer probes
__global__ void mm_red_u32_kernel(unsigned* mc, int n, unsigned v) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) multimem_red_add_u32(mc + i, v);
}
__global__ void mm_red_f32_kernel(float* mc, const float* src, int n) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) multimem_red_add_f32(mc + i, src[i]);
}
__global__ void mm_st_bf16_kernel(uint4* mc, const uint4* src, int n16) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += gridDim.x * blockDim.x) multimem_st_v4(mc + i, src[i]);
}
__global__ void mm_ld_reduce_bf16_kernel(const uint4* mc, uint4* out, int n16) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += gridDim.x * blockDim.x) out[i] = multimem_ld_reduce_bf16x8(mc + i);
}
// Ordering stress for the reducer's publish sequence: one block per slot.  In iteration `it` the slot's writer (rank
// slot % world) broadcasts 512 bytes of payload with multimem.st, fences, and raises the slot's flag on every rank with a
// releasing multimem.st; every rank (the writer too) waits for its local flag, checks that the payload it sees is the
// one of this iteration, and acknowledges with a multimem reduction the writer waits for before it writes again.
// Every wait is bounded; `result[0]` counts stale payload words, `result[1]` is set when a wait gave up.
__global__ void __launch_bounds__(32) mm_order_stress_kernel(uint4* data_mc, const uint4* data_local, int* flag_mc, const int* flag_local,
                                                             unsigned* ack_mc, const unsigned* ack_local, int rank, int world, int iters,
                                                             int* result, long long limit_ns) {
  const int slot = blockIdx.x, lane = threadIdx.x;
  const bool writer = slot % world == rank;
  for (int it = 1; it <= iters; it++) {
    int seen;
    if (writer) {
      const unsigned v = static_cast<unsigned>(it) * 0x10001u + static_cast<unsigned>(slot);
      multimem_st_v4(data_mc + slot * 32 + lane, make_uint4(v, v, v, v));
      __syncwarp();
      if (lane == 0) { fence_acq_rel_sys(); multimem_st_release_b32(flag_mc + slot, it); }
    }
    int ok = 1;
    if (lane == 0) ok = spin_acquire_sys(flag_local + slot, PredGe{it}, limit_ns, seen) ? 1 : 0;
    if (!__shfl_sync(0xffffffffu, ok, 0)) { if (lane == 0) atomicExch(result + 1, 1); return; }
    const unsigned want = static_cast<unsigned>(it) * 0x10001u + static_cast<unsigned>(slot);
    const uint4 got = __ldcg(data_local + slot * 32 + lane);
    int bad = (got.x != want) + (got.y != want) + (got.z != want) + (got.w != want);
    if (bad) atomicAdd(result, bad);
    __syncwarp();
    if (lane == 0) { fence_acq_rel_sys(); multimem_red_release_add_u32(ack_mc + slot, 1u); }
    if (writer) {
      if (lane == 0) ok = spin_acquire_sys(reinterpret_cast<const int*>(ack_local) + slot, PredGe{it * world}, limit_ns, seen) ? 1 : 0;
      if (!__shfl_sync(0xffffffffu, ok, 0)) { if (lane == 0) atomicExch(result + 1, 1); return; }
    }
  }
}

// Per-step reset: epoch += 1, zero the per-step accumulators.
__global__ void tp_step_kernel(int* epoch, float4* rowss_local4, int* panel_done, int M, int* role_ctr) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x, stride = gridDim.x * blockDim.x;
  if (i == 0) { epoch[0] += 1; if (role_ctr) { role_ctr[0] = 0; role_ctr[1] = 0; } }
  for (int k = i; k < M / 4; k += stride) rowss_local4[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int k = i; k < M / 128; k += stride) panel_done[k] = 0;
}

// Comparison baseline: x = a + resid, y = x * rsqrt(mean(x^2) + eps) * gamma, one CTA per row, one pass over the row.
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const uint4* a, const uint4* resid, const uint4* gamma, uint4* x_out, uint4* y_out,
                                                          int n1, float eps) {
  extern __shared__ uint4 s_row[];
  __shared__ float s_part[8];
  const int row = blockIdx.x, vecs = n1 / 8;
  float ss = 0.f;
  for (int i = threadIdx.x; i < vecs; i += blockDim.x) {
    const uint4 av = a[static_cast<size_t>(row) * vecs + i];
    const uint4 rv = resid ? resid[static_cast<size_t>(row) * vecs + i] : make_uint4(0, 0, 0, 0);
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const float2 fa = unpack_bf16x2((&av.x)[k]), fr = unpack_bf16x2((&rv.x)[k]);
      o[k] = pack_bf16x2(fa.x + fr.x, fa.y + fr.y);
    }
    const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
    s_row[i] = ov;
    if (x_out) x_out[static_cast<size_t>(row) * vecs + i] = ov;
    ss += sumsq_bf16x8(ov);
  }
#pragma unroll
  for (int sh = 16; sh > 0; sh >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sh);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); w++) tot += s_part[w];
  const float scale = rsqrtf(tot / n1 + eps);
  for (int i = threadIdx.x; i < vecs; i += blockDim.x) {
    const uint4 xv = s_row[i], gv = gamma[i];
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const float2 fx = unpack_bf16x2((&xv.x)[k]), fg = unpack_bf16x2((&gv.x)[k]);
      // bf16(x * scale) then * gamma in bf16, as the eager formulation rounds
      const float2 nx = unpack_bf16x2(pack_bf16x2(fx.x * scale, fx.y * scale));
      o[k] = pack_bf16x2(nx.x * fg.x, nx.y * fg.y);
    }
    y_out[static_cast<size_t>(row) * vecs + i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// out[r, c] = silu(in[r, c]) * in[r, I + c] for a (rows, 2 I) bf16 input: the activation between the gate/up projection and
// the down projection when it is not fused into the GEMM epilogue.  8 columns per thread, 16-byte accesses; I % 8 == 0.
__global__ void silu_mul_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, long long rows, int I) {
  const int vec = I / 8;
  const long long total = rows * vec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec;
    const int c = static_cast<int>(i - r * vec);
    const uint4 g = in[r * 2 * vec + c], u = in[r * 2 * vec + vec + c];
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const float2 fg = unpack_bf16x2((&g.x)[k]), fu = unpack_bf16x2((&u.x)[k]);
      o[k] = pack_bf16x2(fg.x / (1.0f + __expf(-fg.x)) * fu.x, fg.y / (1.0f + __expf(-fg.y)) * fu.y);
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace ctapp
