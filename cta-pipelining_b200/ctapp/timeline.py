"""Per-CTA time stamps of a chain run on one time base (what reference bench/timeline.py:43-58,119-160 extracts).

Both GEMM kernels record ``%globaltimer`` per CTA when given a stamp buffer: slot 0 entry, 1 first tile acquired, 2 last main
loop issued, 3 last epilogue stores issued, 4 last tile published, 5 tiles processed, 6 SM id, 7 exit.  ``%globaltimer`` is
per GPU; ``clock_offset`` measures the offset between two GPUs with a bounded flag ping-pong (the midpoint of each round
trip on A is taken as the moment B stamped), so that stamps of different stages can be put on stage 0's clock."""
from __future__ import annotations

import statistics

import torch

from ctapp.ext import check_status, load, new_status


def clock_offset(dev_a, dev_b, n=64):
    """(offset_ns, round_trip_ns): add ``offset_ns`` to a ``%globaltimer`` value of ``dev_b`` to express it on ``dev_a``'s clock.
    Launches one single-thread kernel on each GPU; both wait (bounded) on flags the other one writes."""
    ext = load()
    a, b = torch.device("cuda", dev_a), torch.device("cuda", dev_b)
    if dev_a == dev_b:
        return 0.0, 0.0
    ext.enable_peer_access(dev_a, dev_b); ext.enable_peer_access(dev_b, dev_a)
    fa, fb = torch.zeros(1, dtype=torch.int32, device=a), torch.zeros(1, dtype=torch.int32, device=b)
    oa, ob = torch.zeros(2 * n, dtype=torch.int64, device=a), torch.zeros(n, dtype=torch.int64, device=b)
    sa, sb = new_status(a), new_status(b)
    torch.cuda.synchronize(a); torch.cuda.synchronize(b)
    with torch.cuda.device(b):
        ext.pingpong(fb, fa, ob, n, 0, sb)      # B: wait own flag == i, stamp, raise A's flag
    with torch.cuda.device(a):
        ext.pingpong(fa, fb, oa, n, 1, sa)      # A: stamp, raise B's flag, wait own flag == i, stamp
    torch.cuda.synchronize(a); torch.cuda.synchronize(b)
    check_status(sa, "ping-pong A"); check_status(sb, "ping-pong B")
    ta, tb = oa.cpu().view(n, 2), ob.cpu()
    rtt = (ta[:, 1] - ta[:, 0]).double()
    keep = rtt <= rtt.median() * 1.5                       # drop rounds disturbed by anything else on the link
    mid = (ta[:, 0] + ta[:, 1]).double() / 2
    off = (mid - tb.double())[keep]
    return float(off.median()), float(rtt[keep].median())


def chain_timeline(chain):
    """Stage-by-stage summary (microseconds on stage 0's clock, relative to stage 0's first CTA entry) of the most recent run
    of a ``Chain`` built with ``stamps=True``.  Synchronises every device."""
    assert chain.stamps, "build the Chain with stamps=True"
    for d in chain.devs:
        torch.cuda.synchronize(d)
    out, t0 = [], None
    for g, st in enumerate(chain.stamps):
        off = 0.0 if g == 0 else clock_offset(chain.devs[0].index, chain.devs[g].index)[0]
        s = st.view(-1, 8).cpu()
        s = s[s[:, 0] > 0].double()
        if s.shape[0] == 0:
            out.append({"stage": g, "ctas": 0})
            continue
        t = s.clone()
        for k in (0, 1, 2, 3, 4, 7):
            t[:, k] = torch.where(s[:, k] > 0, s[:, k] + off, s[:, k])
        if t0 is None:
            t0 = float(t[:, 0].min())
        us = lambda v: (float(v) - t0) / 1e3  # noqa: E731
        pub = t[:, 4][t[:, 4] > 0]
        out.append({"stage": g, "ctas": int(s.shape[0]), "sms": int(s[:, 6].unique().numel()), "tiles": int(s[:, 5].sum()),
                    "entry_min_us": us(t[:, 0].min()), "entry_max_us": us(t[:, 0].max()),
                    "first_tile_min_us": us(t[:, 1][t[:, 1] > 0].min()), "first_tile_median_us": us(t[:, 1][t[:, 1] > 0].median()),
                    "last_publish_max_us": us(pub.max()) if pub.numel() else None,
                    "exit_min_us": us(t[:, 7].min()), "exit_max_us": us(t[:, 7].max()),
                    "tiles_per_cta_median": float(statistics.median(s[:, 5].tolist()))})
    return out
