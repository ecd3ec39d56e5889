"""Bindings of the native library: builds ``libctapp_b200.so`` with nvcc (sm_100a) and exposes it through ctypes.

``load()`` and ``load_tp4()`` return module-like objects with the function names and argument meaning of the
reference's two extension modules (reference ctapp/ext.py:15-43, csrc/gemm_tma.cu:252-269, csrc/gemm_tp4.cu:837-865);
arguments are torch CUDA tensors, work is enqueued on the current torch stream of the tensor's device, and every
argument error or CUDA error raises ``RuntimeError``.  There is no CPU fallback: without the built library (or
without nvcc to build it) ``load()`` raises.
"""
from __future__ import annotations

import ctypes as C
import os
import shutil
import subprocess

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REPO = os.path.dirname(ROOT)
CSRC = os.path.join(ROOT, "csrc")
LIB_PATH = os.path.join(ROOT, "libctapp_b200.so")
BD = BD4 = ROOT   # build directory (the reference kept one per module; here one library serves both)
SOURCES = ["ctapp_b200.cu"]
HEADERS = ["ptx.cuh", "gemm_sm100.cuh", "gemm2_sm100.cuh", "reduce_sm100.cuh", os.path.join(REPO, "include", "ctapp_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--shared",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
ABI_VERSION = 5
STATUS_INTS = 8
MAX_WORLD = 8

STATUS_TEXT = {1: "source work-queue entry never arrived", 2: "panel flag never arrived", 3: "tile flag never arrived",
               4: "downstream ready flag never arrived", 5: "intra-CTA pipeline barrier never completed",
               6: "probe wait gave up", 7: "index outside its table", 8: "k-chunk flag never arrived"}


def _nvcc():
    for cand in (os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"), shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    return None


def _stale():
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False, verbose=False):
    """Compile the library in-tree for sm_100a.  Returns the path of the shared object."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = _nvcc()
    if nvcc is None:
        if os.path.exists(LIB_PATH):
            return LIB_PATH            # cannot rebuild here; use what was shipped
        raise RuntimeError("libctapp_b200.so is not built and nvcc was not found (set CUDA_HOME)")
    tmp = f"{LIB_PATH}.{os.getpid()}.tmp"     # built beside the target and renamed: a process that has the old file mapped keeps it
    cmd = [nvcc, *NVCC_FLAGS, "-o", tmp, *[os.path.join(CSRC, s) for s in SOURCES]]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        print(" ".join(cmd)); print(r.stdout); print(r.stderr)
    if r.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise RuntimeError(f"nvcc failed ({r.returncode}):\n{r.stderr[-4000:]}")
    os.replace(tmp, LIB_PATH)
    with open(os.path.join(ROOT, "build_ptxas.log"), "w") as f:
        f.write(r.stderr)
    return LIB_PATH


# ------------------------------------------------------------------------------------------ C structs
class Queue(C.Structure):
    _fields_ = [("entries", C.c_void_p), ("head", C.c_void_p), ("tail", C.c_void_p), ("cap", C.c_int)]


class ChainArgs(C.Structure):
    _fields_ = [("stamps", C.c_void_p), ("src", Queue), ("dep_offsets", C.c_void_p), ("dep_consumers", C.c_void_p),
                ("scoreboard", C.c_void_p), ("dst", Queue), ("tiles_n", C.c_int), ("skip_wait", C.c_int), ("fence", C.c_int),
                ("tiles_n2", C.c_int), ("rowpanel", C.c_int), ("dst_ready", C.c_void_p), ("ready_value", C.c_int),
                ("status", C.c_void_p), ("sms", C.c_int), ("src_group", C.c_int),
                ("src_windows", C.c_void_p), ("n_windows", C.c_int),
                ("chunk_dst", C.c_void_p), ("chunk_src", C.c_void_p), ("chunk_kblocks", C.c_int), ("chunk_cols", C.c_int), ("chunk_value", C.c_int)]


class TpDownArgs(C.Structure):
    _fields_ = [("A", C.c_void_p), ("W", C.c_void_p), ("D", C.c_void_p), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
                ("raster", C.c_int), ("swizzle", C.c_int), ("mode", C.c_int), ("rank", C.c_int), ("world", C.c_int),
                ("epoch", C.c_int), ("epoch_dev", C.c_void_p), ("dst_ptrs", C.c_void_p * MAX_WORLD), ("dst_rows", C.c_int),
                ("peer_tile_flags", C.c_void_p * MAX_WORLD), ("panels_per_owner", C.c_int), ("sms", C.c_int),
                ("pdl_trigger", C.c_int), ("pdl", C.c_int), ("tail_cols", C.c_int), ("trace", C.c_void_p), ("status", C.c_void_p),
                ("cta_pair", C.c_int), ("dst_global", C.c_int), ("tile_log", C.c_void_p)]


class TpQkvArgs(C.Structure):
    _fields_ = [("X", C.c_void_p), ("W", C.c_void_p), ("Y", C.c_void_p), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
                ("raster", C.c_int), ("swizzle", C.c_int), ("mode", C.c_int), ("epoch", C.c_int), ("epoch_dev", C.c_void_p),
                ("panel_flag", C.c_void_p), ("rowss", C.c_void_p), ("eps", C.c_float), ("sms", C.c_int), ("pdl", C.c_int),
                ("tile", C.c_int), ("trace", C.c_void_p), ("status", C.c_void_p), ("cta_pair", C.c_int), ("act", C.c_int), ("red", C.c_void_p)]


class TpReduceArgs(C.Structure):
    _fields_ = [("M", C.c_int), ("n1", C.c_int), ("rank", C.c_int), ("world", C.c_int), ("epoch", C.c_int), ("epoch_dev", C.c_void_p),
                ("blocks", C.c_int), ("threads", C.c_int), ("tile_flags", C.c_void_p), ("inbox", C.c_void_p * MAX_WORLD),
                ("resid", C.c_void_p), ("peer_x", C.c_void_p * MAX_WORLD), ("peer_rowss", C.c_void_p * MAX_WORLD),
                ("peer_panel_flag", C.c_void_p * MAX_WORLD), ("rowss_local", C.c_void_p), ("panel_done", C.c_void_p),
                ("panels_per_owner", C.c_int), ("tail_cols", C.c_int), ("order", C.c_int), ("swz", C.c_int), ("unit_ctr", C.c_void_p),
                ("unit_log", C.c_void_p), ("pdl_trigger", C.c_int), ("help_all", C.c_int), ("trace", C.c_void_p),
                ("status", C.c_void_p), ("x_mc", C.c_void_p), ("rowss_mc", C.c_void_p), ("panel_flag_mc", C.c_void_p), ("partials_mc", C.c_void_p),
                ("role_ctr", C.c_void_p), ("role_r", C.c_int)]


_SIGS = {
    "ctapp_last_error": (C.c_char_p, []),
    "ctapp_abi_version": (C.c_int, []),
    "ctapp_set_wait_limit_ms": (C.c_int, [C.c_int]),
    "ctapp_get_wait_limit_ms": (C.c_int, []),
    "ctapp_preload": (C.c_int, [C.c_int]),
    "ctapp_enable_peer_access": (C.c_int, [C.c_int, C.c_int]),
    "ctapp_gate_alloc": (C.c_int, []),
    "ctapp_gate_set": (C.c_int, [C.c_int]),
    "ctapp_gate_wait": (C.c_int, [C.c_int, C.c_void_p]),
    "ctapp_peer_copy": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_size_t, C.c_void_p]),
    "ctapp_p2p_store_bw": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]),
    "ctapp_stamp_now": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "ctapp_timer_reads": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "ctapp_pingpong": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "ctapp_malloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t, C.c_int]),
    "ctapp_free": (C.c_int, [C.c_void_p, C.c_int]),
    "ctapp_ipc_get_handle": (C.c_int, [C.c_void_p, C.c_char_p, C.c_int]),
    "ctapp_ipc_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p), C.c_int]),
    "ctapp_ipc_close": (C.c_int, [C.c_void_p, C.c_int]),
    "ctapp_config_info": (C.c_int, [C.c_int, C.c_char_p, C.c_int]),
    "ctapp_occupancy": (C.c_int, [C.c_int]),
    "ctapp_cluster_occupancy": (C.c_int, [C.c_int, C.c_int]),
    "ctapp_gemm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "ctapp_chain_gemm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(ChainArgs), C.c_int, C.c_void_p]),
    "ctapp_chain_reset": (C.c_int, [Queue, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "ctapp_tp_down": (C.c_int, [C.POINTER(TpDownArgs), C.c_int, C.c_void_p]),
    "ctapp_tp_qkv": (C.c_int, [C.POINTER(TpQkvArgs), C.c_int, C.c_void_p]),
    "ctapp_tp_reduce": (C.c_int, [C.POINTER(TpReduceArgs), C.c_int, C.c_void_p]),
    "ctapp_tp_reduce_noalloc": (C.c_int, [C.POINTER(TpReduceArgs), C.c_int, C.c_void_p]),
    "ctapp_debug_tile_order": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "ctapp_debug_unit_order": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "ctapp_debug_queue_slots": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "ctapp_tp_step": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "ctapp_mm_red_u32": (C.c_int, [C.c_void_p, C.c_int, C.c_uint, C.c_int, C.c_void_p]),
    "ctapp_mm_red_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "ctapp_mm_st_bf16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "ctapp_mm_ld_reduce_bf16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "ctapp_mm_order_stress": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                        C.c_void_p, C.c_int, C.c_void_p]),
    "ctapp_add_rmsnorm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p]),
    "ctapp_silu_mul": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "ctapp_kernel_info": (C.c_int, [C.c_int, C.c_char_p, C.c_int]),
}
EXPORTS = tuple(_SIGS)

_lib = None


def lib():
    """The loaded shared object with argument types set (built on first use if the sources are newer)."""
    global _lib
    if _lib is None:
        path = build()
        l = C.CDLL(path)
        for name, (res, args) in _SIGS.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        if l.ctapp_abi_version() != ABI_VERSION:     # the ctypes structs below must match the library's argument structs
            raise RuntimeError(f"{path} has ABI version {l.ctapp_abi_version()}, these bindings need {ABI_VERSION}: rebuild it")
        _lib = l
    return _lib


def _check(rc):
    if rc != 0:
        raise RuntimeError(f"ctapp_b200: {lib().ctapp_last_error().decode()} (code {rc})")


def _stream(dev):
    return C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, int):
        return C.c_void_p(t) if t else None
    return C.c_void_p(t.data_ptr())


def _bf16_matrix(t, name):
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.is_contiguous()):
        raise RuntimeError(f"{name} must be a contiguous 2-D bf16 CUDA tensor")
    return t


def _i32(t, name, optional=False):
    if t is None and optional:
        return None
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.int32 and t.is_contiguous()):
        raise RuntimeError(f"{name} must be a contiguous int32 CUDA tensor")
    return t


def new_status(device):
    """A zeroed status buffer for the bounded device-side waits."""
    return torch.zeros(STATUS_INTS, dtype=torch.int32, device=device)


def check_status(status, what="kernel"):
    """Raise RuntimeError if a device-side wait gave up (synchronises the device the buffer lives on)."""
    s = status.cpu().tolist()
    if s[0] != 0:
        status.zero_()
        raise RuntimeError(f"ctapp_b200: {what}: {STATUS_TEXT.get(s[0], 'unknown')} (code {s[0]}, block {s[1]}, index {s[2]}, "
                           f"expected {s[3]}, seen {s[4]}, {s[5]} waiters gave up)")


def _ptr_array(values):
    arr = (C.c_void_p * MAX_WORLD)()
    for i, v in enumerate(values):
        arr[i] = v.data_ptr() if isinstance(v, torch.Tensor) else int(v)
    return arr


# ------------------------------------------------------------------------------------------ module 1: chain
class ChainModule:
    """Function-compatible stand-in for the reference's ``gemm_tma_ext`` (csrc/gemm_tma.cu:252-269, gemm_coop.cu:116-119)."""

    def __init__(self):
        self.lib = lib()

    # ---- GEMMs
    def gemm_tma(self, X, W, Y, config_id, group_rows=0, sms=0):
        X, W, Y = _bf16_matrix(X, "X"), _bf16_matrix(W, "W"), _bf16_matrix(Y, "Y")
        M, K = X.shape
        N = W.shape[0]
        if W.shape[1] != K or tuple(Y.shape) != (M, N):
            raise RuntimeError(f"shape mismatch X{tuple(X.shape)} W{tuple(W.shape)} Y{tuple(Y.shape)}")
        dev = X.device.index
        _check(self.lib.ctapp_gemm(_ptr(X), _ptr(W), _ptr(Y), M, N, K, int(config_id), int(group_rows), int(sms), dev, _stream(dev)))

    def coop_gemm(self, X, W, Y, cfg, raster=0, swizzle=1):
        # the persistent kernel serves both roles; cfg 0/2 are 128x256 tiles, 1 is 256x128 in the reference (-> 128x256 here)
        self.gemm_tma(X, W, Y, 3, group_rows=8)

    def coop_info(self, cfg):
        return self.config_info(3)

    def ctapp_gemm(self, X, W, Y, config_id, src_entries, src_head, src_tail, dep_offsets, dep_consumers, scoreboard,
                   dst_entries, dst_head, dst_tail, tiles_n, skip_wait, fence, stamps=None, tiles_n2=0, rowpanel=0,
                   status=None, dst_ready=None, ready_value=0, sms=0, src_group=0, src_windows=None,
                   chunk_dst=None, chunk_src=None, chunk_kblocks=0, chunk_value=0):
        X, W, Y = _bf16_matrix(X, "X"), _bf16_matrix(W, "W"), _bf16_matrix(Y, "Y")
        M, K = X.shape
        N = W.shape[0]
        if W.shape[1] != K or tuple(Y.shape) != (M, N):
            raise RuntimeError(f"shape mismatch X{tuple(X.shape)} W{tuple(W.shape)} Y{tuple(Y.shape)}")
        a = ChainArgs()
        a.stamps = _ptr(stamps)
        a.src = Queue(_ptr(_i32(src_entries, "src_entries")), _ptr(_i32(src_head, "src_head")), _ptr(_i32(src_tail, "src_tail")), src_entries.numel())
        a.dep_offsets, a.dep_consumers = _ptr(_i32(dep_offsets, "dep_offsets", True)), _ptr(_i32(dep_consumers, "dep_consumers", True))
        a.scoreboard = _ptr(_i32(scoreboard, "scoreboard", True))
        a.dst = Queue(_ptr(_i32(dst_entries, "dst_entries", True)), _ptr(_i32(dst_head, "dst_head", True)), _ptr(_i32(dst_tail, "dst_tail", True)),
                      dst_entries.numel() if dst_entries is not None else 1)
        a.tiles_n, a.skip_wait, a.fence, a.tiles_n2, a.rowpanel = int(tiles_n), int(skip_wait), int(fence), int(tiles_n2), int(rowpanel)
        a.dst_ready, a.ready_value = _ptr(dst_ready), int(ready_value)
        a.status, a.sms, a.src_group = _ptr(status), int(sms), int(src_group)
        if src_windows is not None:      # int32 device tensor of window offsets in row panels: [0, ..., panels]
            a.src_windows, a.n_windows = _ptr(_i32(src_windows, "src_windows")), src_windows.numel() - 1
        # k-chunk dependencies: chunk_dst = the next GPU's flags (one per tile of this GEMM); chunk_src = this GPU's flags, a 2-D
        # int32 tensor (row tiles, producer n-tiles), with chunk_kblocks 64-wide k-blocks per flag
        a.chunk_dst, a.chunk_value = _ptr(_i32(chunk_dst, "chunk_dst", True)), int(chunk_value)
        if chunk_src is not None:
            a.chunk_src, a.chunk_kblocks, a.chunk_cols = _ptr(_i32(chunk_src, "chunk_src")), int(chunk_kblocks), chunk_src.shape[-1]
        dev = X.device.index
        _check(self.lib.ctapp_chain_gemm(_ptr(X), _ptr(W), _ptr(Y), M, N, K, int(config_id), C.byref(a), dev, _stream(dev)))

    def chain_reset(self, entries, head, tail, scoreboard=None, pristine=None, ready_flag=None, ready_value=0):
        """One kernel: entries = -1, head = tail = 0, scoreboard = pristine, then ready_flag = ready_value (release, system
        scope).  entries None: only head is rewound (a pre-filled source queue)."""
        q = Queue(_ptr(entries), _ptr(head), _ptr(tail), entries.numel() if entries is not None else 0)
        dev = head.device.index
        _check(self.lib.ctapp_chain_reset(q, _ptr(scoreboard), _ptr(pristine), scoreboard.numel() if scoreboard is not None else 0,
                                          _ptr(ready_flag), int(ready_value), dev, _stream(dev)))

    def config_info(self, config_id):
        buf = C.create_string_buffer(256)
        _check(self.lib.ctapp_config_info(int(config_id), buf, 256))
        return buf.value.decode()

    def cluster_occupancy(self, cluster_size, device=0):
        """Clusters of ``cluster_size`` CTAs of the CTA-pair kernel the device holds at once."""
        n = self.lib.ctapp_cluster_occupancy(int(cluster_size), int(device))
        if n < 0:
            raise RuntimeError(f"ctapp_cluster_occupancy: {self.lib.ctapp_last_error().decode()}")
        return n

    def occupancy(self, config_id):
        n = self.lib.ctapp_occupancy(int(config_id))
        if n < 0:
            _check(n)
        return n

    def kernel_info(self, which):
        buf = C.create_string_buffer(256)
        _check(self.lib.ctapp_kernel_info(int(which), buf, 256))
        return buf.value.decode()

    def preload(self, device):
        _check(self.lib.ctapp_preload(int(device)))

    # ---- read-back of the device-side integer maps
    def debug_tile_order(self, order, tiles_m, tiles_n, group_rows=0, tail_cols=0, device=0):
        """(tiles, 2) int32 CPU tensor: the (m, n) the kernels' ``decode_tile`` gives for every schedule position."""
        out = torch.empty(tiles_m * tiles_n, 2, dtype=torch.int32, device=torch.device("cuda", device))
        _check(self.lib.ctapp_debug_tile_order(int(order), int(tiles_m), int(tiles_n), int(group_rows), int(tail_cols), _ptr(out), device, _stream(device)))
        return out.cpu()

    def debug_unit_order(self, owned_panels, tiles_n, tail_cols=0, order=1, swz=1, device=0):
        """(units, 3) int32 CPU tensor: the (j, n, q) the owner reducer's ``unit_map`` gives for every unit."""
        out = torch.empty(owned_panels * tiles_n * 4, 3, dtype=torch.int32, device=torch.device("cuda", device))
        _check(self.lib.ctapp_debug_unit_order(int(owned_panels), int(tiles_n), int(tail_cols), int(order), int(swz), _ptr(out), device, _stream(device)))
        return out.cpu()

    def debug_queue_slots(self, num_tiles, tiles_n, src_group=0, src_windows=None, device=0):
        """int32 CPU tensor: the queue slot the kernels' ``queue_slot`` reads at every pop."""
        out = torch.empty(num_tiles, dtype=torch.int32, device=torch.device("cuda", device))
        nw = src_windows.numel() - 1 if src_windows is not None else 0
        _check(self.lib.ctapp_debug_queue_slots(int(num_tiles), int(tiles_n), int(src_group), _ptr(src_windows), nw, _ptr(out), device, _stream(device)))
        return out.cpu()

    # ---- harness natives
    def enable_peer_access(self, dev, peer):
        _check(self.lib.ctapp_enable_peer_access(int(dev), int(peer)))

    def p2p_store_bw_kernel(self, src, dst):
        dev = src.device.index
        _check(self.lib.ctapp_p2p_store_bw(_ptr(src), _ptr(dst), src.numel() * src.element_size(), dev, _stream(dev)))

    def gate_alloc(self):
        _check(self.lib.ctapp_gate_alloc())

    def gate_set(self, v):
        _check(self.lib.ctapp_gate_set(int(v)))

    def gate_wait(self):
        dev = torch.cuda.current_device()
        _check(self.lib.ctapp_gate_wait(dev, _stream(dev)))

    def peer_copy(self, dst, src):
        dev = src.device.index
        _check(self.lib.ctapp_peer_copy(_ptr(dst), dst.device.index, _ptr(src), dev, src.numel() * src.element_size(), _stream(dev)))

    def stamp_now(self, out):
        dev = out.device.index
        _check(self.lib.ctapp_stamp_now(_ptr(out), dev, _stream(dev)))

    def timer_reads(self, out):
        dev = out.device.index
        _check(self.lib.ctapp_timer_reads(_ptr(out), out.numel(), dev, _stream(dev)))

    def pingpong(self, mine, other, out, n, is_a, status=None):
        dev = mine.device.index
        _check(self.lib.ctapp_pingpong(_ptr(mine), _ptr(other), _ptr(out), int(n), int(is_a), _ptr(status), dev, _stream(dev)))

    def set_wait_limit_ms(self, ms):
        _check(self.lib.ctapp_set_wait_limit_ms(int(ms)))


# ------------------------------------------------------------------------------------------ module 2: TP boundary
class Tp4Module:
    """Function-compatible stand-in for the reference's ``ctapp_tp4_ext`` (csrc/gemm_tp4.cu:837-865), protocol v5 subset:
    tp4_down modes {0, 7}, tp4_qkv modes {0, 5}, tp4_reduce version 5, tp4_step.  Pointer-valued arguments accept ints
    (device addresses) or tensors, as in the reference."""

    def __init__(self):
        self.lib = lib()

    def tp4_down(self, A, W, D, raster, swizzle, mode, rank, world, epoch, tile_cnt_mc=0, tile_cnt=None, partials_mc=0, x_mc=0,
                 resid=None, rowss_mc=0, panel_cnt_mc=0, sms=0, epoch_dev=None, rowss_mc_base=0, rowss_stride=0, d_ptr=0,
                 dst_ptrs=(), dst_rows=0, peer_tile_flags=(), panels_per_owner=0, pdl_trigger=0, trace=0, tail_cols=0, pdl=0, status=None, cta_pair=0,
                 tile_log=None, dst_global=0):
        A, W = _bf16_matrix(A, "A"), _bf16_matrix(W, "W")
        if mode not in (0, 7):
            raise RuntimeError(f"tp4_down: mode {mode} is not available in this build (0 | 7)")
        a = TpDownArgs()
        a.A, a.W, a.D = _ptr(A), _ptr(W), _ptr(D) if mode == 0 else None
        a.M, a.K = A.shape
        a.N = W.shape[0]
        if W.shape[1] != a.K:
            raise RuntimeError(f"shape mismatch A{tuple(A.shape)} W{tuple(W.shape)}")
        a.raster, a.swizzle, a.mode, a.rank, a.world, a.epoch = int(raster), int(swizzle), int(mode), int(rank), int(world), int(epoch)
        a.epoch_dev = _ptr(epoch_dev)
        a.dst_ptrs, a.dst_rows = _ptr_array(dst_ptrs), int(dst_rows)
        a.peer_tile_flags, a.panels_per_owner = _ptr_array(peer_tile_flags), int(panels_per_owner)
        a.sms, a.pdl_trigger, a.pdl, a.tail_cols = int(sms), int(pdl_trigger), int(pdl), int(tail_cols)
        a.trace, a.status, a.cta_pair, a.tile_log, a.dst_global = _ptr(trace), _ptr(status), int(cta_pair), _ptr(tile_log), int(dst_global)
        dev = A.device.index
        _check(self.lib.ctapp_tp_down(C.byref(a), dev, _stream(dev)))

    @staticmethod
    def _reduce_args(M, rank, world, epoch, epoch_dev, blocks, threads, tile_flags, inbox_ptrs, resid, peer_x, peer_rowss, peer_panel_flag,
                     rowss_local, panel_done, panels_per_owner, tail_cols, n1, status, order=1, swz=1, unit_ctr=0, unit_log=None, pdl_trigger=0,
                     red_trace=0, x_mc_ptr=0, rowss_mc_ptr=0, panel_flag_mc_ptr=0, help_all=0, partials_mc_ptr=0, role_ctr=None, role_r=0):
        """The owner reducer's argument block (``ctapp_tp_reduce_args``), shared by tp4_reduce, tp4_reduce_noalloc and the mode-8
        consumer.  ``panels_per_owner`` is required: the flags are indexed with it, and a wrong value aliases the sources."""
        if panels_per_owner <= 0:
            raise RuntimeError("panels_per_owner is required (the value the tile flags and the inbox were allocated with)")
        a = TpReduceArgs()
        a.M, a.n1, a.rank, a.world, a.epoch, a.epoch_dev = int(M), int(n1), int(rank), int(world), int(epoch), _ptr(epoch_dev)
        a.blocks, a.threads = int(blocks), int(threads)
        a.tile_flags = _ptr(tile_flags)
        a.inbox, a.peer_x = _ptr_array(inbox_ptrs), _ptr_array(peer_x)
        a.peer_rowss, a.peer_panel_flag = _ptr_array(peer_rowss), _ptr_array(peer_panel_flag)
        a.resid = _ptr(resid)
        a.rowss_local, a.panel_done = _ptr(rowss_local), _ptr(panel_done)
        a.panels_per_owner, a.tail_cols, a.order, a.swz = int(panels_per_owner), int(tail_cols), int(order), int(swz)
        a.unit_ctr, a.unit_log, a.pdl_trigger, a.help_all = _ptr(unit_ctr), _ptr(unit_log), int(pdl_trigger), int(help_all)
        a.trace, a.status = _ptr(red_trace), _ptr(status)
        a.x_mc, a.rowss_mc, a.panel_flag_mc = _ptr(x_mc_ptr), _ptr(rowss_mc_ptr), _ptr(panel_flag_mc_ptr)
        a.partials_mc = _ptr(partials_mc_ptr)
        a.role_ctr, a.role_r = _ptr(role_ctr), int(role_r)
        return a

    def tp4_qkv(self, X, W, Y, raster, swizzle, mode, epoch, panel_cnt=None, panel_target=1, rowss=None, sms=0, pdl=0, epoch_dev=None,
                tile=256, R=0, role_ctr=None, rank=0, red_order=1, red_swz=1, tile_flags=None, resid=None, inbox_ptrs=(), peer_x=(),
                peer_rowss=(), peer_panel_flag=(), rowss_local=0, panel_done=0, panels_per_owner=0, red_rows=4, trace=0, red_trace=0,
                red_stages=0, red_dyn=0, red_tail=0, status=None, eps=1e-5, cta_pair=0, act=0, world=1, unit_ctr=None, help_all=0,
                x_mc_ptr=0, rowss_mc_ptr=0, panel_flag_mc_ptr=0):
        """Modes 0 (plain, optional row scaling), 5 (per-panel waits) and 8: as 5, and every CTA first helps the owner reducer by
        claiming units from ``unit_ctr`` (default ``role_ctr[1:]``), for which the reducer's arguments (``rank`` .. ``red_tail``,
        named as in the reference binding) are needed.  Mode 8 with ``R > 0`` and ``red_dyn=0`` is role switching instead: the
        first R CTAs to arrive (tickets from ``role_ctr[0]``) run the reducer's static shares, no unit counter.  ``act=1``: W is (2 I, K) with gate and up rows interleaved in blocks of
        128 (``interleave_gate_up``) and Y is (M, I) = silu(gate) * up; needs ``cta_pair``."""
        X, W, Y = _bf16_matrix(X, "X"), _bf16_matrix(W, "W"), _bf16_matrix(Y, "Y")
        if mode not in (0, 5, 8):
            raise RuntimeError(f"tp4_qkv: mode {mode} is not available in this build (0 | 5 | 8)")
        a = TpQkvArgs()
        a.X, a.W, a.Y = _ptr(X), _ptr(W), _ptr(Y)
        a.M, a.K = X.shape
        a.N = W.shape[0]
        if W.shape[1] != a.K or tuple(Y.shape) != (a.M, a.N // 2 if act else a.N):
            raise RuntimeError(f"shape mismatch X{tuple(X.shape)} W{tuple(W.shape)} Y{tuple(Y.shape)} act={act}")
        a.act = int(act)
        a.raster, a.swizzle, a.mode, a.epoch, a.epoch_dev = int(raster), int(swizzle), int(mode), int(epoch), _ptr(epoch_dev)
        a.panel_flag = _ptr(panel_cnt) if mode in (5, 8) else None
        a.rowss = _ptr(rowss)
        a.eps, a.sms, a.pdl, a.tile = float(eps), int(sms), int(pdl), int(tile)
        a.trace, a.status, a.cta_pair = _ptr(trace), _ptr(status), int(cta_pair)
        red = None
        if mode == 8:
            role = R > 0 and not red_dyn
            if role:
                if role_ctr is None:
                    raise RuntimeError("tp4_qkv: role switching (R > 0) needs role_ctr")
                unit_ctr = None
            elif unit_ctr is None:
                unit_ctr = role_ctr[1:] if role_ctr is not None else None
            red = self._reduce_args(a.M, rank, world, epoch, epoch_dev, 1, 32, tile_flags, inbox_ptrs, resid, peer_x, peer_rowss, peer_panel_flag,
                                    rowss_local, panel_done, panels_per_owner, red_tail, a.K, status, order=red_order, swz=red_swz,
                                    unit_ctr=unit_ctr, red_trace=red_trace, x_mc_ptr=x_mc_ptr, rowss_mc_ptr=rowss_mc_ptr,
                                    panel_flag_mc_ptr=panel_flag_mc_ptr, help_all=help_all, role_ctr=role_ctr if role else None,
                                    role_r=R if role else 0)
            a.red = C.cast(C.pointer(red), C.c_void_p)
        dev = X.device.index
        _check(self.lib.ctapp_tp_qkv(C.byref(a), dev, _stream(dev)))

    def tp4_reduce(self, M, rank, world, epoch, raster, blocks, tile_cnt, partials_mc=0, x_mc=0, resid=None, rowss_mc=0, panel_cnt_mc=0,
                   unicast=0, peer_partials=(), peer_x=(), version=5, epoch_dev=None, inbox_ptrs=(), peer_rowss=(), peer_panel_flag=(),
                   rowss_local=0, panel_done=0, panels_per_owner=0, threads=1024, variant=1, swz=1, rows=2, red_trace=0, dsmem=0, stages=0,
                   unit_ctr=0, tail_cols=0, pdl_trigger=0, n1=8192, status=None, x_mc_ptr=0, rowss_mc_ptr=0, panel_flag_mc_ptr=0, unit_log=None,
                   partials_mc_ptr=0):
        """Owner reducer, protocol version 5 (``raster`` = the producer's tile order: 1 = m fastest, 2 = n fastest; ``swz`` = its
        n-tile group size).  ``variant`` / ``rows`` / ``stages`` / ``dsmem`` of the reference select kernels that have one
        counterpart here and are accepted without effect."""
        if version != 5:
            raise RuntimeError(f"tp4_reduce: version {version} is not available in this build (5)")
        a = self._reduce_args(M, rank, world, epoch, epoch_dev, blocks, threads, tile_cnt, inbox_ptrs, resid, peer_x, peer_rowss, peer_panel_flag,
                              rowss_local, panel_done, panels_per_owner, tail_cols, n1, status, order=2 if raster == 2 else 1, swz=swz,
                              unit_ctr=unit_ctr, unit_log=unit_log, pdl_trigger=pdl_trigger, red_trace=red_trace, x_mc_ptr=x_mc_ptr,
                              rowss_mc_ptr=rowss_mc_ptr, panel_flag_mc_ptr=panel_flag_mc_ptr, partials_mc_ptr=partials_mc_ptr)
        dev = tile_cnt.device.index
        _check(self.lib.ctapp_tp_reduce(C.byref(a), dev, _stream(dev)))

    # ---- NVLS probes (reference csrc/gemm_tp4.cu:393-502); ``mc`` is a multicast device address (int)
    def mm_red_u32(self, mc, n, v):
        dev = torch.cuda.current_device()
        _check(self.lib.ctapp_mm_red_u32(_ptr(mc), int(n), int(v), dev, _stream(dev)))

    def mm_red_f32(self, mc, src):
        dev = src.device.index
        _check(self.lib.ctapp_mm_red_f32(_ptr(mc), _ptr(src), src.numel(), dev, _stream(dev)))

    def mm_st_bf16(self, mc, src):
        dev = src.device.index
        _check(self.lib.ctapp_mm_st_bf16(_ptr(mc), _ptr(src), src.numel(), dev, _stream(dev)))

    def mm_ld_reduce_bf16(self, mc, out):
        dev = out.device.index
        _check(self.lib.ctapp_mm_ld_reduce_bf16(_ptr(mc), _ptr(out), out.numel(), dev, _stream(dev)))

    def mm_order_stress(self, data_mc, data, flag_mc, flag, ack_mc, ack, rank, world, iters, slots):
        """Returns (stale payload words seen, 1 if a wait gave up else 0); synchronises the device."""
        dev = data.device.index
        res = torch.zeros(2, dtype=torch.int32, device=data.device)
        _check(self.lib.ctapp_mm_order_stress(_ptr(data_mc), _ptr(data), _ptr(flag_mc), _ptr(flag), _ptr(ack_mc), _ptr(ack), int(rank), int(world),
                                              int(iters), int(slots), _ptr(res), dev, _stream(dev)))
        torch.cuda.synchronize(dev)
        r = res.cpu().tolist()
        return r[0], r[1]

    def tp4_reduce_noalloc(self, M, rank, world, epoch, blocks, tile_flags, resid=None, peer_x=(), epoch_dev=None, inbox_ptrs=(),
                           peer_rowss=(), peer_panel_flag=(), panels_per_owner=0, threads=1024, tail_cols=0, n1=8192, status=None, **refused):
        """The owner reducer without caller scratch buffers and without any allocation (``ctapp_tp_reduce_noalloc``): for hosts
        that may not allocate device memory while running.  M <= 16384; calls that overlap on the GPU race on the shared
        built-in scratch; make the first call on a device (or ``preload``) outside stream capture.  Multicast addresses, a unit
        counter or a unit log (``x_mc_ptr`` ..., ``unit_ctr``, ``unit_log``) are passed on and refused by the library."""
        a = self._reduce_args(M, rank, world, epoch, epoch_dev, blocks, threads, tile_flags, inbox_ptrs, resid, peer_x, peer_rowss, peer_panel_flag,
                              0, 0, panels_per_owner, tail_cols, n1, status, **refused)
        dev = tile_flags.device.index
        _check(self.lib.ctapp_tp_reduce_noalloc(C.byref(a), dev, _stream(dev)))

    def tp4_step(self, epoch_dev, rowss_local, panel_done, M, role_ctr=None):
        dev = epoch_dev.device.index
        _check(self.lib.ctapp_tp_step(_ptr(epoch_dev), _ptr(rowss_local), _ptr(panel_done), int(M), _ptr(role_ctr), dev, _stream(dev)))

    def silu_mul(self, g, out=None):
        """out (M, I) = silu(g[:, :I]) * g[:, I:] for a contiguous bf16 (M, 2 I) tensor, one pass."""
        g = _bf16_matrix(g, "g")
        M, I2 = g.shape
        if out is None:
            out = torch.empty(M, I2 // 2, dtype=torch.bfloat16, device=g.device)
        if I2 % 16 or tuple(out.shape) != (M, I2 // 2) or not out.is_contiguous():
            raise RuntimeError(f"silu_mul: bad shapes g{tuple(g.shape)} out{tuple(out.shape)}")
        dev = g.device.index
        _check(self.lib.ctapp_silu_mul(_ptr(g), _ptr(out), M, I2 // 2, dev, _stream(dev)))
        return out

    def add_rmsnorm(self, a, resid, gamma, x_out, y_out, eps=1e-5):
        M, n1 = a.shape
        dev = a.device.index
        _check(self.lib.ctapp_add_rmsnorm(_ptr(a), _ptr(resid), _ptr(gamma), _ptr(x_out), _ptr(y_out), M, n1, float(eps), dev, _stream(dev)))

    def tp4_info(self, which):
        buf = C.create_string_buffer(256)
        _check(self.lib.ctapp_kernel_info({"down": 0, "qkv": 0, "qkv128": 1, "reduce": 2}.get(which, which) if not isinstance(which, int) else which, buf, 256))
        return buf.value.decode()

    def tp4_set_debug(self, mask):
        if mask:
            raise RuntimeError("tp4_set_debug: the ablation bit mask of the reference has no counterpart in this build")

    def preload(self, device):
        _check(self.lib.ctapp_preload(int(device)))

    def set_wait_limit_ms(self, ms):
        _check(self.lib.ctapp_set_wait_limit_ms(int(ms)))


_chain = _tp4 = None


def load():
    """The chain module (reference ctapp/ext.py:15-26)."""
    global _chain
    if _chain is None:
        _chain = ChainModule()
    return _chain


def load_tp4():
    """The tensor-parallel boundary module (reference ctapp/ext.py:29-43)."""
    global _tp4
    if _tp4 is None:
        _tp4 = Tp4Module()
    return _tp4
