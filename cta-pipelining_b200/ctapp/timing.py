"""Gated latency measurement (mirrors reference ctapp/timing.py:10-35): every participating stream first blocks on a flag in
pinned host memory (``cuStreamWaitValue32``), the work is enqueued behind it, and the gate is opened once everything is
queued, so host launch cost stays outside the timed window."""
from __future__ import annotations

import statistics

import torch

from ctapp.ext import load

ext = None


def _ext():
    global ext
    if ext is None:
        ext = load()
        ext.gate_alloc()
    return ext


def measure(method, reps=20, warmup=5, devs=(0, 1), times=None):
    """``method.prepare()`` runs before the gate closes; ``method.enqueue()`` is what is timed.  Returns (median, p10, p90) in
    microseconds, measured with CUDA events on ``devs[0]``'s stream, which waits for every other device's last work."""
    e = _ext()
    streams = [torch.cuda.current_stream(d) for d in devs]
    # one ungated run first: nothing may have to be loaded or allocated while the streams are blocked
    method.prepare(); method.enqueue()
    for d in devs:
        torch.cuda.synchronize(d)
    ts = []
    for i in range(warmup + reps):
        method.prepare()
        e.gate_set(0)
        for d, s in zip(devs, streams):
            with torch.cuda.device(d), torch.cuda.stream(s):
                e.gate_wait()
        with torch.cuda.device(devs[0]):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(streams[0])
        method.enqueue()
        for d, s in zip(devs[1:], streams[1:]):
            with torch.cuda.device(d):
                ev = torch.cuda.Event(); ev.record(s)
            streams[0].wait_event(ev)
        with torch.cuda.device(devs[0]):
            end.record(streams[0])
        e.gate_set(1)
        for d in devs:
            torch.cuda.synchronize(d)
        if i >= warmup:
            ts.append(start.elapsed_time(end) * 1e3)
    if times is not None:
        times.extend(ts)
    q = statistics.quantiles(ts, n=10, method="inclusive")
    return statistics.median(ts), q[0], q[-1]
