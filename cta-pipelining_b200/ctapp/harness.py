"""Process harness and timers for the one-process-per-GPU tests and benches: ``launch`` spawns ``world`` workers that
join an NCCL (or, on the CPU, gloo) process group plus a gloo side group, runs a function in each and collects the
results; ``time_step`` / ``time_one_gpu`` are the boundary's timers (reference ctapp/tp4.py:689-790)."""
from __future__ import annotations

import os
import queue as _queue
import statistics
import sys
import time
import traceback

import torch
import torch.distributed as dist


def _event_ms(fn, dev, reps=1):
    """Device time of ``reps`` back-to-back calls of ``fn`` in ms (CUDA events on the current stream, synchronised)."""
    torch.cuda.synchronize(dev)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(reps):
        fn()
    t1.record()
    torch.cuda.synchronize(dev)
    return t0.elapsed_time(t1)


def time_step(step, dev, iters, warmup, side_group):
    """Two figures for a multi-rank step, each the maximum over ranks: the median of ``iters`` isolated calls (all ranks
    meet at a barrier before every call) and the mean of ``iters`` calls issued back to back."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize(dev)
    singles = []
    for _ in range(iters):
        dist.barrier(group=side_group)
        singles.append(_event_ms(step, dev))
    dist.barrier(group=side_group)
    b2b = _event_ms(step, dev, iters) / iters
    both = torch.tensor([statistics.median(singles), b2b], dtype=torch.float64)
    dist.all_reduce(both, op=dist.ReduceOp.MAX, group=side_group)
    return both.tolist()


def time_one_gpu(fn, dev, iters, warmup):
    """Median device time in ms of ``iters`` isolated calls on one GPU."""
    for _ in range(warmup):
        fn()
    return statistics.median(_event_ms(fn, dev) for _ in range(iters))


def _quiesce(dev, side_group, seconds):
    """Drain this rank's GPU, then meet the other ranks (bounded: a rank that is already gone must not hold the others)."""
    import datetime
    try:
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
        if side_group is not None:
            dist.monitored_barrier(group=side_group, timeout=datetime.timedelta(seconds=seconds))
        return True
    except BaseException:  # noqa: BLE001
        return False


def _worker(rank, world, port, fn, args, results, backend):
    """Body of one spawned rank: join the groups, run ``fn``, report.  A rank leaves only with its GPU idle and its symmetric
    buffers (which may be bound to an NVLink multicast object) released, and after having waited (bounded) for the other
    ranks to be idle too: a peer may still be storing into this rank's memory while its own kernels finish.  The process
    groups themselves are not torn down (a peer may already be gone, and a teardown that waits for it would never return)."""
    import gc
    from ctapp import tp4
    os.environ.setdefault("TORCH_NCCL_ENABLE_MONITORING", "0")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    pkg = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if pkg not in sys.path:
        sys.path.insert(0, pkg)
    status, dev, report = 0, torch.device("cpu"), None
    try:
        url = f"tcp://127.0.0.1:{port}"
        if backend == "nccl":
            dev = torch.device("cuda", rank)
            torch.cuda.set_device(dev)
            dist.init_process_group("nccl", init_method=url, rank=rank, world_size=world, device_id=dev)
            tp4.GLOO = dist.new_group(backend="gloo")
        else:
            dist.init_process_group("gloo", init_method=url, rank=rank, world_size=world)
            tp4.GLOO = dist.group.WORLD
        value = fn(rank, world, dev, dist.group.WORLD.group_name, *args)
        if backend == "nccl":
            torch.cuda.synchronize(dev)
        tp4.barrier()
        report = (rank, True, value)
    except BaseException:  # noqa: BLE001
        traceback.print_exc()
        report = (rank, False, traceback.format_exc())
        status = 1
    results.put(report)
    # leave in order: everybody idle -> drop the buffers (frames of a raised exception would keep them alive) -> idle again
    side = tp4.GLOO if dist.is_initialized() else None
    _quiesce(dev, side, 20.0)
    sys.last_traceback = sys.last_value = None
    gc.collect()
    if dev.type == "cuda":
        torch.cuda.empty_cache()
    _quiesce(dev, side, 20.0)
    sys.stdout.flush(); sys.stderr.flush()
    results.close(); results.join_thread()
    os._exit(status)


def launch(fn, world, port, *args, backend="nccl", grace_s=60.0):
    """Run ``fn(rank, world, dev, group_name, *args)`` in ``world`` spawned processes (one per GPU; backend "gloo" runs them on
    the CPU).  Returns (per-rank results, bad): a rank that raised or vanished leaves None and makes ``bad`` true.  Once a
    rank has failed the others get ``grace_s`` seconds and are then stopped.  That is long enough for every device-side wait
    to have given up (they are bounded at two seconds) and for the survivors' own exit sequence (GPU idle, buffers released),
    so a rank is only ever stopped with no kernel of its own in flight."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, args, q, backend)) for r in range(world)]
    for p in procs:
        p.start()
    results, reported, first_failure = [None] * world, 0, None
    while reported < world:
        try:
            r, ok, value = q.get(timeout=1)
            reported += 1
            if ok:
                results[r] = value
            elif first_failure is None:
                first_failure = time.time()
        except _queue.Empty:
            if not any(p.is_alive() for p in procs):
                break
            if first_failure is None and any(p.exitcode not in (None, 0) for p in procs):
                first_failure = time.time()
        if first_failure is not None and time.time() - first_failure > grace_s:
            break
    for p in procs:
        p.join(timeout=0.5 if first_failure is not None else 30)
        if p.is_alive():
            p.kill()
            p.join(timeout=5)
    bad = reported < world or any(r is None for r in results)
    return results, bad
