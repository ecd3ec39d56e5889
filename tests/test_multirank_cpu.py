"""The multi-rank host logic on the CPU: world_size-2 process groups over gloo (no GPU)."""
from oracle import boundary as ob
from oracle import chain as oc


def _plans_agree(rank, world, dev, group_name, M, K, widths):
    """Every rank computes its own stage plan; neighbours must agree on the link between them."""
    import torch.distributed as dist
    from ctapp.pipeline import build_deps, stage_plan
    plan = stage_plan(M, K, widths, rank)
    plans = [None] * world
    dist.all_gather_object(plans, plan)
    for g in range(world - 1):
        assert plans[g]["dst_cap"] == plans[g + 1]["ntiles"]
        assert plans[g]["dst_cols"] == plans[g + 1]["k_in"]
        assert plans[g]["tiles_n2"] == plans[g + 1]["tiles_n"]
    total = 0
    if not plan["last"]:
        off, cons, sb = build_deps(M, plan["n_out"], widths[rank + 1], 128, 256, 128, 256, True)
        assert int(sb.sum()) == plan["ntiles"] and off.numel() == plan["ntiles"] + 1
        total = int(sb.sum())
    return {"rank": rank, "ntiles": plan["ntiles"], "deps": total}


def _shards_cover(rank, world, dev, group_name, seed):
    """K-shards of the down projection and N-shards of the next projection, gathered over the group, rebuild the full
    weights; the owners of the 128-row panels partition the panels."""
    import torch
    import torch.distributed as dist
    from ctapp.tp4 import fold_gamma, shard_weights
    Wd, gamma, Wq = ob.make_weights(seed=seed, K=256 * world, N2_=128 * world, n1=256)
    wd, wq, wqf = shard_weights(Wd, Wq, gamma, rank, world)
    parts = [None] * world
    dist.all_gather_object(parts, (wd, wq, wqf, [m for m in range(10) if m % world == rank]))
    assert torch.equal(torch.cat([p[0] for p in parts], dim=1), Wd)
    assert torch.equal(torch.cat([p[1] for p in parts], dim=0), Wq)
    assert torch.equal(torch.cat([p[2] for p in parts], dim=0), fold_gamma(Wq, gamma))
    assert sorted(sum((p[3] for p in parts), [])) == list(range(10))
    assert len(parts[rank][3]) == ob.panels_owned(1280, rank, world)
    return rank


def _orders_and_windows_agree(rank, world, dev, group_name, tm, tn, group_rows):
    """Rank 0 computes the order it works in, every later rank the windows it pops its queue in: when the producer publishes
    its row panels group by group, the consuming rank's tile order is the producer's own, all the way down the chain; and the
    set the ranks use for step e of a link with doubled buffers is the same on both sides."""
    import torch
    import torch.distributed as dist
    from ctapp.pipeline import consumer_window, pop_slots, producer_order
    n = tm * tn
    mine = producer_order(n, tn, group_rows) if rank == 0 else None
    win = 0 if rank == 0 else consumer_window(group_rows, 1, 256, 256, tm)
    got = [None] * world
    dist.all_gather_object(got, (mine, win, [(e, e & 1) for e in range(1, 6)]))
    order0 = got[0][0]
    if rank > 0:
        slots = pop_slots(n, tn, win if win else 1)
        # the producer finishes its groups in order, so panel p sits in queue slots [p * tn, (p + 1) * tn) as tile ids p * tn + j
        assert torch.equal(slots, order0), (rank, group_rows)
    assert all(g[2] == got[0][2] for g in got)
    return rank


def _one_rank_raises(rank, world, dev, group_name):
    if rank == 1:
        raise RuntimeError("injected failure on rank 1")
    return rank


def _one_rank_never_joins(rank, world, dev, group_name):
    import os
    if rank == 1:
        os._exit(3)          # dies without a word before the closing barrier
    return rank


def test_stage_plans_agree_over_gloo():
    from ctapp.tp4 import launch
    res, bad = launch(_plans_agree, 2, 29631, 1024, 512, [768, 1024], backend="gloo")
    assert not bad, res
    assert [r["ntiles"] for r in res] == [8 * 3, 8 * 4] and res[0]["deps"] == 24


def test_producer_order_and_consumer_windows_agree_over_gloo():
    from ctapp.tp4 import launch
    for port, (tm, tn, gr) in enumerate([(32, 32, "head"), (16, 8, 8), (9, 4, "ramp"), (12, 4, [3, 4, 5])]):
        res, bad = launch(_orders_and_windows_agree, 2, 29640 + port, tm, tn, gr, backend="gloo")
        assert not bad and res == [0, 1], (res, tm, tn, gr)


def test_weight_shards_cover_over_gloo():
    from ctapp.tp4 import launch
    res, bad = launch(_shards_cover, 2, 29632, 7, backend="gloo")
    assert not bad and res == [0, 1]


def test_launch_reports_a_raising_rank():
    from ctapp.tp4 import launch
    res, bad = launch(_one_rank_raises, 2, 29633, backend="gloo", grace_s=3.0)
    assert bad and res[1] is None


def test_launch_reports_a_vanished_rank_and_does_not_hang():
    import time
    from ctapp.tp4 import launch
    t = time.time()
    res, bad = launch(_one_rank_never_joins, 2, 29634, backend="gloo", grace_s=3.0)
    assert bad and res[1] is None
    assert time.time() - t < 60


def test_protocol_model_detects_a_dropped_flag():
    """Host-side fault injection in the protocol model: a producer tile that never reports leaves its panel unpublished."""
    entries, tail, sb = oc.simulate_link(512, 512, 512, 128, 256, 128, 256, True, 0, order=[0, 1, 2, 3, 4, 5, 7])
    assert tail == 6 and (entries[6:] == -1).all() and sb[3 * 32] == 1
