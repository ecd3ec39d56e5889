"""The allocation-free owner reducer (``ctapp_tp_reduce_noalloc``), called through the C ABI.

Some hosts of the library may not allocate device memory once they are serving (the GPU has been handed to their own
memory pool, or an allocation's implicit synchronisation is not acceptable on the calling path).  For them the reducer's
working memory lives in a fixed array inside the library.  This test feeds the same inputs to the regular entry point
(caller-provided scratch) and to the allocation-free one, twice in a row, and requires the same x (bit for bit), the same
panel flags, and the same row sums (fp32 atomics accumulate in any order: relative 1e-5).  The second call has to cope
with what the first one left in the shared array.  The file sorts last so that a stop at the first failure has run
everything else before.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(M, n1, seed, epoch, dev):
    g = torch.Generator().manual_seed(seed)
    ppo, tn = M // 128, n1 // 256
    inbox = torch.randn(1, ppo * 128, n1, generator=g).to(torch.bfloat16).to(dev)
    resid = torch.randn(M, n1, generator=g).to(torch.bfloat16).to(dev)
    flags = torch.full((1, ppo, tn), epoch, dtype=torch.int32, device=dev)     # every producer tile has "arrived"
    return inbox, resid, flags, ppo


def _args(ext, M, n1, epoch, inbox, resid, flags, ppo, x, rowss, pflag, rowss_local=None, panel_done=None, status=None):
    a = ext.TpReduceArgs()
    a.M, a.n1, a.rank, a.world, a.epoch = M, n1, 0, 1, epoch
    a.blocks, a.threads = 4, 1024
    a.tile_flags, a.resid = flags.data_ptr(), resid.data_ptr()
    a.inbox[0], a.peer_x[0], a.peer_rowss[0], a.peer_panel_flag[0] = inbox.data_ptr(), x.data_ptr(), rowss.data_ptr(), pflag.data_ptr()
    if rowss_local is not None:
        a.rowss_local, a.panel_done = rowss_local.data_ptr(), panel_done.data_ptr()
    a.panels_per_owner, a.tail_cols = ppo, min(8, n1 // 256)
    a.status = status.data_ptr() if status is not None else None
    return a


def _outputs(M, n1, dev):
    return (torch.full((M, n1), float("nan"), dtype=torch.bfloat16, device=dev), torch.full((M,), float("nan"), device=dev),
            torch.zeros(M // 128, dtype=torch.int32, device=dev))


def test_noalloc_reducer_matches_regular_entry_point_twice():
    from ctapp import ext
    lib = ext.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    n1 = 512
    for call, (M, seed, epoch) in enumerate([(512, 1, 5), (384, 2, 9)]):     # two calls in a row, different sizes and data
        inbox, resid, flags, ppo = _case(M, n1, seed, epoch, dev)
        # regular entry point: scratch from the caller
        x0, rs0, pf0 = _outputs(M, n1, dev)
        st0 = ext.new_status(dev)
        a0 = _args(ext, M, n1, epoch, inbox, resid, flags, ppo, x0, rs0, pf0, torch.zeros(M, device=dev),
                   torch.zeros(M // 128, dtype=torch.int32, device=dev), st0)
        assert lib.ctapp_tp_reduce(C.byref(a0), 0, stream) == 0, lib.ctapp_last_error()
        # allocation-free entry point: inputs and outputs only
        x1, rs1, pf1 = _outputs(M, n1, dev)
        st1 = ext.new_status(dev)
        a1 = _args(ext, M, n1, epoch, inbox, resid, flags, ppo, x1, rs1, pf1, status=st1)
        assert lib.ctapp_tp_reduce_noalloc(C.byref(a1), 0, stream) == 0, lib.ctapp_last_error()
        torch.cuda.synchronize(dev)
        assert st0.cpu()[0].item() == 0 and st1.cpu()[0].item() == 0, (st0.cpu().tolist(), st1.cpu().tolist())
        assert not torch.isnan(x0.float()).any(), "the regular entry point left rows unwritten"
        assert torch.equal(x1, x0), f"call {call}: x differs in {(x1 != x0).sum().item()} elements"
        assert torch.equal(pf1, pf0) and bool((pf1 == epoch).all()), f"call {call}: panel flags {pf1.tolist()} vs {pf0.tolist()}"
        torch.testing.assert_close(rs1, rs0, rtol=1e-5, atol=1e-6)
        # and both agree with plain arithmetic on the same inputs
        ref = (inbox[0, :M].float() + resid.float()).to(torch.bfloat16)
        assert torch.equal(x1, ref)
        torch.testing.assert_close(rs1, ref.float().pow(2).sum(-1), rtol=1e-4, atol=1e-3)


def test_noalloc_reducer_rejects_sizes_beyond_its_scratch():
    from ctapp import ext
    lib = ext.lib()
    a = ext.TpReduceArgs()
    a.M, a.n1, a.rank, a.world, a.blocks, a.threads = 16384 + 128, 512, 0, 1, 4, 1024
    a.tile_flags = 256     # never dereferenced: the size check comes first
    assert lib.ctapp_tp_reduce_noalloc(C.byref(a), 0, None) < 0
    msg = lib.ctapp_last_error().decode()
    assert "16384" in msg and "ctapp_tp_reduce" in msg, msg
