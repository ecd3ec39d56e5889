"""The methods the chain is compared with, all driven from one process on devices 0 and 1 (mirrors reference
ctapp/methods.py:27-141): one GPU doing both layers (the "ideal" is half of it), micro-batching with peer copies, tensor
parallelism with an NCCL all-reduce, and the CTA-pipelined chain.  Each has ``prepare()`` (untimed) and ``enqueue()``."""
from __future__ import annotations

import torch

from ctapp.ext import load
from ctapp.pipeline import Pipeline

BF = torch.bfloat16
_ext = None


def ext():
    global _ext
    if _ext is None:
        _ext = load()
    return _ext


def dev(i):
    return torch.device("cuda", i)


class Base:
    def prepare(self):
        pass

    def result(self):
        return self.Y2


class OneGpuCublas(Base):
    """Both layers on device 0 with the library GEMM; half of its time is the chain's ideal (one GEMM's time)."""

    def __init__(self, M, X, W1, W2):
        self.X, self.W1, self.W2 = X, W1, W2
        self.Y1 = torch.empty(M, W1.shape[0], device=dev(0), dtype=BF)
        self.Y2 = torch.empty(M, W2.shape[0], device=dev(0), dtype=BF)

    def enqueue(self):
        with torch.cuda.device(0):
            torch.mm(self.X, self.W1.t(), out=self.Y1)
            torch.mm(self.Y1, self.W2.t(), out=self.Y2)


class OneGpuTma(OneGpuCublas):
    """Both layers on device 0 with this library's GEMM (config id ``cfg``)."""

    def __init__(self, M, X, W1, W2, cfg):
        super().__init__(M, X, W1, W2)
        self.cfg = cfg

    def enqueue(self):
        with torch.cuda.device(0):
            ext().gemm_tma(self.X, self.W1, self.Y1, self.cfg)
            ext().gemm_tma(self.Y1, self.W2, self.Y2, self.cfg)


class MicroBatchCublas(Base):
    """Layer 1 on device 0 and layer 2 on device 1, M split into chunks: GEMM chunk i, copy it over, GEMM on the other side,
    each on its own stream.  chunk == M is the plain sequential two-GPU pipeline."""

    def __init__(self, M, X, W1, W2, chunk):
        ext().enable_peer_access(0, 1); ext().enable_peer_access(1, 0)
        self.M, self.chunk, self.X, self.W1, self.W2 = M, min(chunk, M), X, W1, W2
        N1, N2 = W1.shape[0], W2.shape[0]
        self.Y1a = torch.empty(M, N1, device=dev(0), dtype=BF)
        self.Y1b = torch.empty(M, N1, device=dev(1), dtype=BF)
        self.Y2 = torch.empty(M, N2, device=dev(1), dtype=BF)
        self.sA, self.sB = torch.cuda.current_stream(0), torch.cuda.current_stream(1)
        with torch.cuda.device(0):
            self.sC = torch.cuda.Stream()
        self.n = -(-M // self.chunk)
        self.evA = [torch.cuda.Event() for _ in range(self.n)]
        self.evC = [torch.cuda.Event() for _ in range(self.n)]

    def gemm(self, x, w, y):
        torch.mm(x, w.t(), out=y)

    def enqueue(self):
        c = self.chunk
        for i in range(self.n):
            sl = slice(i * c, min((i + 1) * c, self.M))
            with torch.cuda.device(0):
                with torch.cuda.stream(self.sA):
                    self.gemm(self.X[sl], self.W1, self.Y1a[sl]); self.evA[i].record(self.sA)
                with torch.cuda.stream(self.sC):
                    self.sC.wait_event(self.evA[i]); ext().peer_copy(self.Y1b[sl], self.Y1a[sl]); self.evC[i].record(self.sC)
            with torch.cuda.device(1), torch.cuda.stream(self.sB):
                self.sB.wait_event(self.evC[i])
                self.gemm(self.Y1b[sl], self.W2, self.Y2[sl])


class MicroBatchTma(MicroBatchCublas):
    def __init__(self, M, X, W1, W2, chunk, cfg):
        super().__init__(M, X, W1, W2, chunk)
        self.cfg = cfg

    def gemm(self, x, w, y):
        ext().gemm_tma(x, w, y, self.cfg)


class TensorParallel2(Base):
    """Megatron split over two GPUs: W1 by rows, W2 by columns, all-reduce of the (M, N2) partial sums (single-process
    NCCL).  X is replicated."""

    def __init__(self, M, X, W1, W2):
        N1, N2 = W1.shape[0], W2.shape[0]
        h = N1 // 2
        W2 = W2.to(dev(0))
        self.X = [X, X.to(dev(1))]
        self.W1 = [W1[g * h:(g + 1) * h].contiguous().to(dev(g)) for g in range(2)]
        self.W2 = [W2[:, g * h:(g + 1) * h].contiguous().to(dev(g)) for g in range(2)]
        self.Y1 = [torch.empty(M, h, device=dev(g), dtype=BF) for g in range(2)]
        self.P = [torch.empty(M, N2, device=dev(g), dtype=BF) for g in range(2)]
        self.s = [torch.cuda.current_stream(g) for g in range(2)]
        for _ in range(3):
            self.enqueue()
        torch.cuda.synchronize(0); torch.cuda.synchronize(1)

    def enqueue(self):
        for g in range(2):
            with torch.cuda.device(g):
                torch.mm(self.X[g], self.W1[g].t(), out=self.Y1[g])
                torch.mm(self.Y1[g], self.W2[g].t(), out=self.P[g])
        torch.cuda.nccl.all_reduce(self.P, streams=self.s)

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
