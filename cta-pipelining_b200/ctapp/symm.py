"""Symmetric buffers: every rank allocates the same buffer and learns the device address of every other rank's copy.

Three providers behind one call (``symm_empty``), mirroring what the reference gets from torch symmetric memory
(reference ctapp/tp4.py:31-35: ``buffer_ptrs[r]`` and ``multicast_ptr``):

* ``LocalGroup``: one process drives all ranks' GPUs; peer addresses are plain UVA pointers after
  ``cudaDeviceEnablePeerAccess``.  world == 1 needs no peer at all.
* process group (a group name or None with torch.distributed initialised): one process per GPU; buffers come from the
  library's own ``cudaMalloc`` and are mapped into the other processes with CUDA IPC handles exchanged through
  ``torch.distributed.all_gather_object``.
* ``CTAPP_SYMM=torch``: torch's symmetric memory, which also yields a multicast address on NVSwitch systems.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from ctapp.ext import _check, lib


class SymmHandle:
    """What a kernel launch needs to know about a symmetric buffer."""

    def __init__(self, buffer_ptrs, multicast_ptr=0, keep=None):
        self.buffer_ptrs = list(buffer_ptrs)
        self.multicast_ptr = multicast_ptr
        self._keep = keep      # objects that must outlive the handle (owning tensors, allocations)


class _RawCuda:
    """Adapter that lets torch view foreign device memory (``__cuda_array_interface__``)."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _numel(shape):
    n = 1
    for s in (shape if isinstance(shape, (tuple, list)) else (shape,)):
        n *= int(s)
    return n


def _shape(shape):
    return tuple(shape) if isinstance(shape, (tuple, list)) else (int(shape),)


def view_ptr(ptr, shape, dtype, device):
    """A torch tensor over foreign device memory (a peer's buffer mapped into this process): a typed pointer carrier for
    the bindings, never read or written by torch itself."""
    nbytes = _numel(shape) * torch.empty((), dtype=dtype).element_size()
    dev = device if isinstance(device, torch.device) else torch.device("cuda", device)
    return torch.as_tensor(_RawCuda(ptr, nbytes), device=dev).view(dtype).view(_shape(shape))


class _Allocation:
    """Device memory from the library's allocator (eligible for CUDA IPC), freed with the object."""

    def __init__(self, nbytes, device):
        self.device = device
        p = C.c_void_p()
        _check(lib().ctapp_malloc(C.byref(p), max(nbytes, 16), device))
        self.ptr = p.value

    def tensor(self, shape, dtype):
        nbytes = _numel(shape) * torch.empty((), dtype=dtype).element_size()
        return torch.as_tensor(_RawCuda(self.ptr, nbytes), device=torch.device("cuda", self.device)).view(dtype).view(_shape(shape))

    def __del__(self):
        try:
            lib().ctapp_free(C.c_void_p(self.ptr), self.device)
        except Exception:
            pass


class _IpcMappings:
    """This rank's allocation plus its mappings of the peers' copies; the mappings are closed before the allocation is freed.
    Peers may still have this rank's copy mapped: callers drop their handles only after a barrier (the worker harness does)."""

    def __init__(self, alloc, opened, device):
        self.alloc, self.opened, self.device = alloc, opened, device

    def __del__(self):
        for p in self.opened:
            try:
                lib().ctapp_ipc_close(C.c_void_p(p), self.device)
            except Exception:
                pass
        self.opened = []


class LocalGroup:
    """All ranks live in this process: rank r uses ``devices[r]`` (devices may repeat; world 1 is one GPU talking to
    itself).  The k-th ``symm_empty`` call of every rank refers to the same logical buffer."""

    def __init__(self, devices):
        self.devices = [int(d) for d in devices]
        self.world = len(self.devices)
        self._bufs = []                      # per logical buffer: list of per-rank tensors
        self._next = [0] * self.world        # per rank: index of its next symm_empty call
        uniq = sorted(set(self.devices))
        for a in uniq:
            for b in uniq:
                if a != b:
                    _check(lib().ctapp_enable_peer_access(a, b))

    def alloc(self, shape, dtype, rank):
        k = self._next[rank]
        self._next[rank] += 1
        if k == len(self._bufs):
            self._bufs.append([torch.zeros(_shape(shape), dtype=dtype, device=torch.device("cuda", d)) for d in self.devices])
        ts = self._bufs[k]
        assert tuple(ts[rank].shape) == _shape(shape) and ts[rank].dtype == dtype, "ranks disagree on the order of symmetric allocations"
        return ts[rank], SymmHandle([t.data_ptr() for t in ts], 0, keep=ts)

    def barrier(self):
        for d in set(self.devices):
            torch.cuda.synchronize(d)


def _process_group(group):
    """torch.distributed group object for a group name (None = the default group)."""
    import torch.distributed as dist
    if group is None or not dist.is_initialized():
        return None
    if isinstance(group, str):
        return dist.distributed_c10d._resolve_process_group(group)
    return group


def symm_empty(shape, dtype, dev, group, rank=None, multicast=False):
    """-> (this rank's tensor, SymmHandle).  ``group``: a LocalGroup, or a torch.distributed group name / None for the
    default process group.  Collective over the group in the multi-process case.  ``multicast``: the buffer must also
    have a multicast address (NVLS): only torch's symmetric memory provides one."""
    if isinstance(group, LocalGroup):
        return group.alloc(shape, dtype, rank)
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(_process_group(group)) == 1:
        t = torch.zeros(_shape(shape), dtype=dtype, device=dev)
        return t, SymmHandle([t.data_ptr()], 0, keep=t)
    if multicast or os.environ.get("CTAPP_SYMM", "ipc") == "torch":
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(*_shape(shape), dtype=dtype, device=dev)
        t.zero_()
        torch.cuda.synchronize(dev)          # zeroed before any peer learns the address (the rendezvous is the barrier):
        hdl = symm_mem.rendezvous(t, group if isinstance(group, str) else dist.group.WORLD.group_name)   # a late zero_ could erase a peer's flag
        return t, SymmHandle(list(hdl.buffer_ptrs), getattr(hdl, "multicast_ptr", 0) or 0, keep=(t, hdl))
    device = dev.index if isinstance(dev, torch.device) else int(dev)
    nbytes = _numel(shape) * torch.empty((), dtype=dtype).element_size()
    alloc = _Allocation(nbytes, device)
    t = alloc.tensor(shape, dtype)
    t.zero_()
    torch.cuda.synchronize(device)
    handle = C.create_string_buffer(64)
    _check(lib().ctapp_ipc_get_handle(C.c_void_p(alloc.ptr), handle, device))
    pg = _process_group(group)
    me, world = dist.get_rank(pg), dist.get_world_size(pg)
    gathered = [None] * world
    dist.all_gather_object(gathered, bytes(handle.raw), group=pg)
    ptrs, opened = [], []
    for r in range(world):
        if r == me:
            ptrs.append(alloc.ptr)
            continue
        p = C.c_void_p()
        _check(lib().ctapp_ipc_open(gathered[r], C.byref(p), device))
        ptrs.append(p.value)
        opened.append(p.value)
    return t, SymmHandle(ptrs, 0, keep=_IpcMappings(alloc, opened, device))
