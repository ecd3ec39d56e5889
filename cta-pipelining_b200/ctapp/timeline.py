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


_SEGMENTS = (("wait for the first tile", 0, 1, "#bdbdbd"), ("main loops", 1, 2, "#3b6fb6"),
             ("last epilogue", 2, 3, "#4daf4a"), ("publish and exit", 3, 7, "#ff7f00"))


def gantt_svg(stages, path=None, width=1200, row_h=3, title="CTA timeline"):
    """Gantt chart of per-CTA stamps as an SVG document (reference bench/timeline.py:119-160 draws the same picture with
    matplotlib, which this library does not depend on).

    ``stages``: list of (label, stamps, offset_ns): ``stamps`` an (n, 8) integer array or tensor in the kernels' slot layout
    (rows with entry == 0 are CTAs that did not run), ``offset_ns`` what to add to put them on the first stage's clock.
    One row per CTA, stages stacked top to bottom, rows ordered by SM id; colours: grey = waiting for the first tile,
    blue = first tile acquired to last main loop issued, green = last epilogue, orange = publish and exit.
    Returns the SVG text and writes it to ``path`` when given."""
    rows, t0, t1 = [], None, None
    for label, st, off in stages:
        s = torch.as_tensor(st).reshape(-1, 8).double()
        s = s[s[:, 0] > 0]
        s = s[torch.argsort(s[:, 6], stable=True)]
        for r in s.tolist():
            t = [v + off if (k in (0, 1, 2, 3, 4, 7) and v > 0) else v for k, v in enumerate(r)]
            rows.append((label, t))
            t0 = t[0] if t0 is None else min(t0, t[0])
            t1 = t[7] if t1 is None else max(t1, t[7])
    if not rows:
        raise ValueError("no CTA left a stamp")
    span = max(t1 - t0, 1.0)
    left, top = 90, 30
    x = lambda v: left + (v - t0) / span * (width - left - 10)  # noqa: E731
    height = top + len(rows) * row_h + 40
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="monospace" font-size="11">',
           f'<text x="{left}" y="14">{title}: {span / 1e3:.1f} us, {len(rows)} CTAs</text>']
    y, prev = top, None
    for label, t in rows:
        if label != prev:
            out.append(f'<text x="2" y="{y + 10}">{label}</text>')
            prev = label
        for _, a, b, colour in _SEGMENTS:
            ta, tb = t[a], t[b]
            if a == 1 and ta <= 0:        # a CTA that never got a tile: grey from entry to exit
                continue
            if ta > 0 and tb > ta:
                out.append(f'<rect x="{x(ta):.1f}" y="{y}" width="{max(x(tb) - x(ta), 0.3):.1f}" height="{row_h}" fill="{colour}"/>')
        if t[1] <= 0:
            out.append(f'<rect x="{x(t[0]):.1f}" y="{y}" width="{max(x(t[7]) - x(t[0]), 0.3):.1f}" height="{row_h}" fill="#bdbdbd"/>')
        y += row_h
    for i in range(6):
        v = t0 + span * i / 5
        out.append(f'<text x="{x(v) - 10:.0f}" y="{y + 14}">{(v - t0) / 1e3:.0f}</text>')
    lx = left
    for name, _, _, colour in _SEGMENTS:
        out.append(f'<rect x="{lx}" y="{y + 22}" width="10" height="10" fill="{colour}"/><text x="{lx + 14}" y="{y + 31}">{name}</text>')
        lx += 14 + 8 * len(name) + 20
    out.append("</svg>")
    text = "\n".join(out)
    if path:
        with open(path, "w") as f:
            f.write(text)
    return text


def chain_gantt_svg(chain, path=None):
    """``gantt_svg`` of the most recent run of a ``Chain`` built with ``stamps=True`` (clock offsets measured here)."""
    assert chain.stamps, "build the Chain with stamps=True"
    for d in chain.devs:
        torch.cuda.synchronize(d)
    stages = []
    for g, st in enumerate(chain.stamps):
        off = 0.0 if g == 0 else clock_offset(chain.devs[0].index, chain.devs[g].index)[0]
        stages.append((f"stage {g} gpu {chain.devs[g].index}", st.cpu(), off))
    return gantt_svg(stages, path, title=f"{len(stages)}-stage chain, M={chain.M}")
