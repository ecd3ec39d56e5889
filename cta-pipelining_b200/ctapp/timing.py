"""Gated latency measurement (the role of reference ctapp/timing.py:10-35).

A run is timed from the moment the GPUs are let loose to the moment the last of them is done, with the host's launch cost
kept out of the window: while the ``Gate`` is closed every participating stream sits on a ``cuStreamWaitValue32`` of a word
in pinned host memory, the work is queued up behind those waits, and opening the gate releases all streams at once.
``measure`` keeps the reference's signature: ``method.prepare()`` (untimed), ``method.enqueue()`` (timed)."""
from __future__ import annotations

import contextlib
import statistics

import torch

from ctapp.ext import load


class Gate:
    """The pinned host word all streams wait on.  ``with gate.closed(streams): ...`` queues a wait on every stream, runs the body
    (which enqueues the work to be released), and opens the gate on exit."""

    _ext = None

    def __init__(self):
        if Gate._ext is None:
            Gate._ext = load()
            Gate._ext.gate_alloc()
        self.ext = Gate._ext

    @contextlib.contextmanager
    def closed(self, streams):
        self.ext.gate_set(0)
        for s in streams:
            with torch.cuda.device(s.device), torch.cuda.stream(s):
                self.ext.gate_wait()
        try:
            yield self
        finally:
            self.ext.gate_set(1)


class _Span:
    """Start / stop events on the first stream; ``stop`` first makes that stream wait for everything queued on the others."""

    def __init__(self, streams):
        self.streams = streams
        self.lead = streams[0]
        self.t0 = torch.cuda.Event(enable_timing=True)
        self.t1 = torch.cuda.Event(enable_timing=True)

    def start(self):
        with torch.cuda.device(self.lead.device):
            self.t0.record(self.lead)

    def stop(self):
        for s in self.streams[1:]:
            with torch.cuda.device(s.device):
                done = torch.cuda.Event()
                done.record(s)
            self.lead.wait_event(done)
        with torch.cuda.device(self.lead.device):
            self.t1.record(self.lead)

    def microseconds(self):
        for s in self.streams:
            s.synchronize()
        return self.t0.elapsed_time(self.t1) * 1e3


def gated_run(gate, streams, prepare, enqueue):
    """One gated run -> device time in microseconds between the gate opening and the last stream finishing."""
    prepare()
    span = _Span(streams)
    with gate.closed(streams):
        span.start()         # queued behind the gate on the lead stream: fires when the gate opens
        enqueue()
        span.stop()
    return span.microseconds()


def measure(method, reps=20, warmup=5, devs=(0, 1), times=None):
    """(median, 10th percentile, 90th percentile) in microseconds over ``reps`` gated runs of ``method`` on the current streams
    of ``devs`` (the events live on ``devs[0]``).  One ungated run comes first, so that nothing has to be loaded or allocated
    while the streams are blocked."""
    gate = Gate()
    streams = [torch.cuda.current_stream(d) for d in devs]
    method.prepare()
    method.enqueue()
    for s in streams:
        s.synchronize()
    samples = [gated_run(gate, streams, method.prepare, method.enqueue) for _ in range(warmup + reps)][warmup:]
    if times is not None:
        times.extend(samples)
    deciles = statistics.quantiles(samples, n=10, method="inclusive")
    return statistics.median(samples), deciles[0], deciles[-1]
