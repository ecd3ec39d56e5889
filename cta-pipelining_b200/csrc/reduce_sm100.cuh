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
  int* unit_ctr;
  unsigned long long* trace;
  int* status;
  long long limit_ns;
  // NVLS variant: multicast addresses of the x buffer, the row-sum buffer and the panel flags (null = unicast pushes)
  uint4* x_mc;
  float* rowss_mc;
  int* panel_flag_mc;
};

// unit u -> (owned panel j, n-tile, quarter), following the producer order "m-fast head, panel-major tail"
__device__ __forceinline__ void unit_map(int u, int Pr, int tiles_n, int tail, int& j, int& n, int& q) {
  q = u & 3;
  const int t = u >> 2;
  const int head = Pr * (tiles_n - tail);
  if (t < head) { n = t / Pr; j = t - n * Pr; }
  else { const int t2 = t - head; j = t2 / tail; n = tiles_n - tail + (t2 - j * tail); }
}

__device__ __forceinline__ float sumsq_bf16x8(uint4 o) {
  float s = 0.f;
  const uint32_t w[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
  for (int i = 0; i < 4; i++) { const float2 f = unpack_bf16x2(w[i]); s = fmaf(f.x, f.x, s); s = fmaf(f.y, f.y, s); }
  return s;
}

// MC: the pushes to every rank (x rows, row sums, panel flags) are single multimem stores on a multicast address, replicated
// by the NVSwitch, instead of one unicast store per rank; everything else is the same kernel.
template <int W, int ROWS, bool MC = false>
__global__ void __launch_bounds__(1024, 1) tp_reduce_kernel(const ReduceParams p) {
  const int epoch = p.epoch_ptr ? __ldcg(p.epoch_ptr) : p.epoch;
  const int P = p.M / 128;
  const int Pr = P > p.rank ? (P - 1 - p.rank) / W + 1 : 0;
  const int tiles_n = p.n1 / 256;
  const int units_per_panel = tiles_n * 4;
  const int U = Pr * units_per_panel;
  const int row_vecs = p.n1 / 8;                 // uint4 per row
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int stride = gridDim.x * nwarps;
  auto claim = [&]() -> int {
    int v = 0;
    if (lane == 0) v = atomicAdd(p.unit_ctr, 1);
    return __shfl_sync(0xffffffffu, v, 0);
  };
  for (int u = p.unit_ctr ? claim() : warp * static_cast<int>(gridDim.x) + static_cast<int>(blockIdx.x); u < U;
       u = p.unit_ctr ? claim() : u + stride) {
    int j, n, q;
    unit_map(u, Pr, tiles_n, p.tail, j, n, q);
    bool ok = true;
    if (lane < W) {
      int seen;
      const int idx = (lane * p.ppo + j) * tiles_n + n;
      if (!spin_acquire_sys(p.tile_flags + idx, PredGe{epoch}, p.limit_ns, seen)) {
        report_status(p.status, kStatusTimeoutTile, idx, epoch, seen);
        ok = false;
      }
    }
    if (!__all_sync(0xffffffffu, ok)) return;   // a producer never delivered: give up (bounded), the host reads the status
    const int m = j * W + p.rank;
    const int xrow0 = m * 128 + q * 32;
    const size_t ioff0 = static_cast<size_t>(j * 128 + q * 32) * row_vecs + n * 32 + lane;
    const size_t xoff0 = static_cast<size_t>(xrow0) * row_vecs + n * 32 + lane;
#pragma unroll 1
    for (int r = 0; r < 32; r += ROWS) {
      uint4 a[ROWS][W], rv[ROWS];
#pragma unroll
      for (int rr = 0; rr < ROWS; rr++) {
#pragma unroll
        for (int s = 0; s < W; s++) a[rr][s] = __ldcg(p.inbox[s] + ioff0 + static_cast<size_t>(r + rr) * row_vecs);
      }
#pragma unroll
      for (int rr = 0; rr < ROWS; rr++)
        rv[rr] = p.resid ? __ldg(p.resid + xoff0 + static_cast<size_t>(r + rr) * row_vecs) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int rr = 0; rr < ROWS; rr++) {
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
          float lo = 0.f, hi = 0.f;
#pragma unroll
          for (int s = 0; s < W; s++) {
            const float2 f = unpack_bf16x2((&a[rr][s].x)[i]);
            if (s == 0) { lo = f.x; hi = f.y; } else { lo += f.x; hi += f.y; }
          }
          const float2 fr = unpack_bf16x2((&rv[rr].x)[i]);
          o[i] = pack_bf16x2(lo + fr.x, hi + fr.y);
        }
        const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
        const size_t xoff = xoff0 + static_cast<size_t>(r + rr) * row_vecs;
        if (MC) {
          multimem_st_v4(p.x_mc + xoff, ov);
        } else {
#pragma unroll
          for (int d = 1; d <= W; d++) {   // remote copies first, the local one last
            const int dst = (p.rank + d) % W;
            st_relaxed_sys_v4(p.x[dst] + xoff, ov);
          }
        }
        float ss = sumsq_bf16x8(ov);
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sh);
        if (lane == 0) atomicAdd(p.rowss_local + xrow0 + r + rr, ss);
      }
    }
    __syncwarp();
    int last = 0;
    if (lane == 0) {
      fence_acq_rel_sys();   // this warp's x stores and row-sum atomics before the arrival count
      last = atom_add_relaxed_gpu(p.panel_done + m, 1) == units_per_panel - 1;
    }
    if (__shfl_sync(0xffffffffu, last, 0)) {
      if (lane == 0) fence_acq_rel_sys();   // acquire side: the other warps' stores and atomics of this panel
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
