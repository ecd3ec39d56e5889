"""The C-ABI shared library builds, loads without a GPU, and exports every symbol the public header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "ctapp_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ctapp_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_header_symbols():
    from ctapp import ext
    path = ext.build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    syms = header_symbols()
    assert len(syms) >= 25
    for s in syms:
        assert hasattr(lib, s), f"{s} is declared in include/ctapp_b200.h but not exported"
    # the binding table covers the header, and nothing else
    assert sorted(ext.EXPORTS) == syms


def test_argument_errors_without_gpu():
    """Calls that fail in argument checking never touch CUDA, so they can run here."""
    from ctapp import ext
    lib = ext.lib()
    assert lib.ctapp_abi_version() == ext.ABI_VERSION == 5
    buf = ctypes.create_string_buffer(256)
    assert lib.ctapp_config_info(3, buf, 256) == 0 and b"tile 128x256x64" in buf.value
    assert lib.ctapp_config_info(5, buf, 256) == 0 and b"tile 128x128x64" in buf.value
    assert lib.ctapp_config_info(77, buf, 256) < 0 and b"bad config_id" in lib.ctapp_last_error()
    assert lib.ctapp_occupancy(3) == 1
    assert lib.ctapp_set_wait_limit_ms(0) < 0
    assert lib.ctapp_set_wait_limit_ms(1500) == 0 and lib.ctapp_get_wait_limit_ms() == 1500
    assert lib.ctapp_set_wait_limit_ms(2000) == 0
    assert lib.ctapp_gemm(None, None, None, 128, 128, 128, 42, 0, 0, 0, None) < 0
    assert lib.ctapp_gate_set(1) < 0 and b"gate_alloc" in lib.ctapp_last_error()


def _reduce_args(**over):
    """A reducer argument block with fake (never dereferenced) addresses: argument checking happens before any CUDA call."""
    from ctapp import ext
    fake = 0x1000
    kw = dict(M=1024, rank=0, world=2, epoch=1, epoch_dev=None, blocks=4, threads=1024, tile_flags=fake, inbox_ptrs=[fake, fake], resid=None,
              peer_x=[fake, fake], peer_rowss=[fake, fake], peer_panel_flag=[fake, fake], rowss_local=fake, panel_done=fake, panels_per_owner=4,
              tail_cols=8, n1=8192, status=None)
    kw.update(over)
    return ext.Tp4Module._reduce_args(**kw)


def test_reducer_argument_checks_without_gpu():
    """panels_per_owner is validated (a value below ceil(M / 128 / world) would make the sources' tile flags alias each other),
    and the allocation-free variant refuses what it does not do instead of ignoring it."""
    from ctapp import ext
    lib = ext.lib()
    a = _reduce_args(panels_per_owner=3)
    assert lib.ctapp_tp_reduce(ctypes.byref(a), 0, None) == -1 and b"panels_per_owner" in lib.ctapp_last_error()
    assert lib.ctapp_tp_reduce_noalloc(ctypes.byref(a), 0, None) == -1 and b"panels_per_owner" in lib.ctapp_last_error()
    with pytest.raises(RuntimeError):
        _reduce_args(panels_per_owner=0)                       # the binding insists on the argument
    for over, word in ((dict(x_mc_ptr=0x2000, rowss_mc_ptr=0x2000, panel_flag_mc_ptr=0x2000), b"unicast"), (dict(unit_ctr=0x2000), b"unit_ctr"),
                       (dict(unit_log=0x2000), b"unit_ctr"), (dict(pdl_trigger=1), b"pdl_trigger"), (dict(partials_mc_ptr=0x2000), b"unicast"), (dict(M=32768, panels_per_owner=128), b"16384"),
                       (dict(role_ctr=0x2000, role_r=4), b"role_r")):
        a = _reduce_args(**over)
        assert lib.ctapp_tp_reduce_noalloc(ctypes.byref(a), 0, None) == -1, over
        assert word in lib.ctapp_last_error(), (over, lib.ctapp_last_error())
    a = _reduce_args(order=3)
    assert lib.ctapp_tp_reduce(ctypes.byref(a), 0, None) == -1
    for over in (dict(role_r=4), dict(role_r=4, role_ctr=0x2000, unit_ctr=0x2000), dict(role_r=-1, role_ctr=0x2000)):   # role switching: its counter, static shares
        a = _reduce_args(**over)
        assert lib.ctapp_tp_reduce(ctypes.byref(a), 0, None) == -1 and b"role" in lib.ctapp_last_error(), over
    q = ext.TpQkvArgs()
    q.mode = 8
    assert lib.ctapp_tp_qkv(ctypes.byref(q), 0, None) == -1 and b"mode 8" in lib.ctapp_last_error()


def test_python_module_surface():
    """The two module objects carry the function names of the reference's extension modules."""
    from ctapp import ext
    m1, m2 = ext.load(), ext.load_tp4()
    for name in ("gemm_tma", "ctapp_gemm", "coop_gemm", "coop_info", "config_info", "occupancy", "enable_peer_access",
                 "p2p_store_bw_kernel", "gate_alloc", "gate_set", "gate_wait", "peer_copy", "stamp_now", "timer_reads", "pingpong"):
        assert callable(getattr(m1, name)), name
    for name in ("tp4_down", "tp4_qkv", "tp4_reduce", "tp4_reduce_noalloc", "tp4_step", "tp4_info", "tp4_set_debug"):
        assert callable(getattr(m2, name)), name
    assert "tile 128x256x64" in m1.config_info(3)
    with pytest.raises(RuntimeError):
        m1.config_info(99)


def test_build_entry_point_runs():
    """``__graft_entry__.build()`` is what decides "does it build": it must compile the library in-tree, load it, agree with
    the bindings on the ABI version and import the package."""
    import importlib
    import os
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if root not in sys.path:
        sys.path.insert(0, root)
    entry = importlib.import_module("__graft_entry__")
    entry.build()
    from ctapp import ext
    assert os.path.exists(ext.LIB_PATH) and ext.lib().ctapp_abi_version() == ext.ABI_VERSION
