"""What the chain is compared with, all driven from one process on devices 0 and 1: one GPU doing both layers (half of it
is the chain's ideal), micro-batching with peer copies, tensor parallelism with an NCCL all-reduce, and the CTA-pipelined
chain itself.  Same class names and constructor arguments as reference ctapp/methods.py:27-141; every method has
``prepare()`` (untimed) and ``enqueue()`` (timed) and ``result()``."""
from __future__ import annotations

import torch

from ctapp.ext import load
from ctapp.pipeline import Pipeline

BF = torch.bfloat16


def ext():
    return load()


def dev(i):
    return torch.device("cuda", i)


def _out(M, W, device):
    return torch.empty(M, W.shape[0], device=device, dtype=BF)


class Base:
    def prepare(self):
        pass

    def result(self):
        return self.Y2


class OneGpuCublas(Base):
    """Both layers on device 0 with the library GEMM."""

    def __init__(self, M, X, W1, W2):
        self.X, self.W1, self.W2 = X, W1, W2
        self.Y1, self.Y2 = _out(M, W1, dev(0)), _out(M, W2, dev(0))

    def _mm(self, x, w, y):
        torch.mm(x, w.t(), out=y)

    def enqueue(self):
        with torch.cuda.device(0):
            self._mm(self.X, self.W1, self.Y1)
            self._mm(self.Y1, self.W2, self.Y2)


class OneGpuTma(OneGpuCublas):
    """Both layers on device 0 with this library's GEMM (config id ``cfg``)."""

    def __init__(self, M, X, W1, W2, cfg):
        super().__init__(M, X, W1, W2)
        self.cfg = cfg

    def _mm(self, x, w, y):
        ext().gemm_tma(x, w, y, self.cfg)


class MicroBatchCublas(Base):
    """Layer 1 on device 0, layer 2 on device 1, the M rows cut into chunks: compute chunk i, copy it across on a copy
    stream, compute on the other side.  chunk == M is the plain sequential two-GPU pipeline."""

    def __init__(self, M, X, W1, W2, chunk):
        ext().enable_peer_access(0, 1); ext().enable_peer_access(1, 0)     # otherwise the copies bounce through the host
        self.X, self.W1, self.W2 = X, W1, W2
        step = min(chunk, M)
        self.slices = [slice(a, min(a + step, M)) for a in range(0, M, step)]
        self.Y1a, self.Y1b, self.Y2 = _out(M, W1, dev(0)), _out(M, W1, dev(1)), _out(M, W2, dev(1))
        self.compute0, self.compute1 = torch.cuda.current_stream(0), torch.cuda.current_stream(1)
        with torch.cuda.device(0):
            self.copier = torch.cuda.Stream()
        self.done0 = [torch.cuda.Event() for _ in self.slices]
        self.copied = [torch.cuda.Event() for _ in self.slices]

    def gemm(self, x, w, y):
        torch.mm(x, w.t(), out=y)

    def enqueue(self):
        for i, rows in enumerate(self.slices):
            with torch.cuda.device(0):
                with torch.cuda.stream(self.compute0):
                    self.gemm(self.X[rows], self.W1, self.Y1a[rows])
                    self.done0[i].record(self.compute0)
                with torch.cuda.stream(self.copier):
                    self.copier.wait_event(self.done0[i])
                    ext().peer_copy(self.Y1b[rows], self.Y1a[rows])
                    self.copied[i].record(self.copier)
            with torch.cuda.device(1), torch.cuda.stream(self.compute1):
                self.compute1.wait_event(self.copied[i])
                self.gemm(self.Y1b[rows], self.W2, self.Y2[rows])


class MicroBatchTma(MicroBatchCublas):
    def __init__(self, M, X, W1, W2, chunk, cfg):
        super().__init__(M, X, W1, W2, chunk)
        self.cfg = cfg

    def gemm(self, x, w, y):
        ext().gemm_tma(x, w, y, self.cfg)


class TensorParallel2(Base):
    """Megatron split over two GPUs: W1 by rows, W2 by columns, all-reduce of the (M, N2) partial sums with single-process
    NCCL.  X is replicated."""

    def __init__(self, M, X, W1, W2):
        half = W1.shape[0] // 2
        W2 = W2.to(dev(0))
        cut = [slice(g * half, (g + 1) * half) for g in range(2)]
        self.X = [X, X.to(dev(1))]
        self.W1 = [W1[cut[g]].contiguous().to(dev(g)) for g in range(2)]
        self.W2 = [W2[:, cut[g]].contiguous().to(dev(g)) for g in range(2)]
        self.Y1 = [_out(M, self.W1[g], dev(g)) for g in range(2)]
        self.P = [_out(M, W2, dev(g)) for g in range(2)]
        self.streams = [torch.cuda.current_stream(g) for g in range(2)]
        for _ in range(3):      # NCCL communicator set-up happens on first use
            self.enqueue()
        torch.cuda.synchronize(0); torch.cuda.synchronize(1)

    def enqueue(self):
        for g in range(2):
            with torch.cuda.device(g):
                torch.mm(self.X[g], self.W1[g].t(), out=self.Y1[g])
                torch.mm(self.Y1[g], self.W2[g].t(), out=self.P[g])
        torch.cuda.nccl.all_reduce(self.P, streams=self.streams)

    def result(self):
        return self.P[1]


class Ctapp(Base):
    """The CTA-pipelined chain: ``prepare`` resets the queues, ``enqueue`` launches both stages."""

    def __init__(self, M, X, W1, W2, cfg_p, cfg_c, group_rows, fence=1, scoreboard="rowpanel"):
        self.pl = Pipeline(M, X.shape[1], W1.shape[0], W2.shape[0], cfg_p, cfg_c, devA=0, devB=1, fence=fence, group_rows=group_rows,
                           scoreboard=scoreboard)
        self.X, self.W1, self.W2 = X, W1, W2

    def prepare(self):
        self.pl.reset()

    def enqueue(self):
        self.pl.chain.enqueue(self.X, [self.W1, self.W2])

    def result(self):
        return self.pl.Y2
