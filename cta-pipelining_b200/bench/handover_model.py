"""Timing model of one chain link with k-chunk dependencies: when does the consuming GEMM end, given the order and the
tile time of the producing one?  No GPU, no kernels: a discrete-event walk over both tile orders.

    python cta-pipelining_b200/bench/handover_model.py [--ms 4096,8192,16384] [--groups 1,2,4,8]

Model.  ``pairs`` CTA pairs per GPU.  The producer pops its tiles in ``producer_order`` (groups of tile rows, n-major inside
a group) as pairs fall free; a tile takes ``tile_us`` and raises its flag when it ends.  The consumer pops its own grouped
order the same way; a tile walks its k-chunks in order, and chunk c of a tile of row m starts no earlier than the flag of
producer tile (m, c) and takes ``consumer_tile_us / chunks``.  Nothing else is modelled (no launch skew, no cold first wave, no
polling cost), so the model is a floor for the order it is given.  Against gated measurements on two B200s (N = K = 8192,
producer 256x256 tiles of 50 us, consumer 256x512 tiles of 97 us, groups of 4): model 438 / 814 / 1505 us at M = 4096 / 8192 /
16384, measured 431-435 / 797-812 / 1528-1533 us; groups of 8: model 503 / 862, measured 497 / 871; producer on 256x512 tiles
of 100 us as well: model 488 / 861 / 1555, measured 489 / 867 / 1594.

What it shows: the consumer ends T_producer + L, where L is the work it has fallen behind; it runs at the producer's speed and
is throttled by the flags, so L never shrinks during a run.  L is at least one producer wave (the tiles of a wave end
together: their consumer work can only start then) and in practice nearer two, because consumer tiles popped late in a group
start behind the flags and run their full length.
"""
from __future__ import annotations

import argparse
import heapq


def grouped_order(tm, tn, group_rows):
    """(m, n) in the order ``ctapp.pipeline.producer_order`` gives for a constant group size."""
    g = max(1, group_rows)
    return [(m, n) for m0 in range(0, tm, g) for n in range(tn) for m in range(m0, min(tm, m0 + g))]


def producer_times(order, pairs, tile_us):
    """End time of every tile when ``pairs`` workers pop ``order`` as they fall free -> ({(m, n): t}, end of the last one)."""
    free = [(0.0, p) for p in range(pairs)]
    done = {}
    for tile in order:
        t, p = heapq.heappop(free)
        done[tile] = t + tile_us
        heapq.heappush(free, (t + tile_us, p))
    return done, max(done.values())


def consumer_end(done, order, pairs, chunks, tile_us):
    """End of the consuming GEMM: every tile of row m needs producer tile (m, c) before its chunk c."""
    free = [(0.0, p) for p in range(pairs)]
    per_chunk = tile_us / chunks
    end = 0.0
    for m, _ in order:
        t, p = heapq.heappop(free)
        for c in range(chunks):
            t = max(t, done[(m, c)]) + per_chunk
        end = max(end, t)
        heapq.heappush(free, (t, p))
    return end


def link(M, N=8192, group_rows=4, pairs=74, tile_us=50.0, consumer_tile_us=97.0, producer_bn=256, consumer_bn=512, consumer_group=None):
    """(T_producer, end of the consumer) in us for a link of M rows; both GEMMs N wide on 256-row tiles."""
    tm, tn1, tn2 = -(-M // 256), N // producer_bn, N // consumer_bn
    done, tp = producer_times(grouped_order(tm, tn1, group_rows), pairs, tile_us)
    return tp, consumer_end(done, grouped_order(tm, tn2, consumer_group or group_rows), pairs, tn1, consumer_tile_us)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ms", default="4096,8192,16384")
    ap.add_argument("--groups", default="1,2,4,8")
    ap.add_argument("--tile-us", type=float, default=50.0, help="one 256x256 producer tile at K=8192")
    ap.add_argument("--consumer-tile-us", type=float, default=97.0, help="one 256x512 consumer tile at K=8192")
    a = ap.parse_args()
    for M in (int(v) for v in a.ms.split(",")):
        cells = []
        for g in (int(v) for v in a.groups.split(",")):
            tp, end = link(M, group_rows=g, tile_us=a.tile_us, consumer_tile_us=a.consumer_tile_us)
            cells.append(f"groups of {g}: {end:.0f} us (T_producer {tp:.0f} + {end - tp:.0f})")
        print(f"M={M}  " + "  ".join(cells))


if __name__ == "__main__":
    main()
