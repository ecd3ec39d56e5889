"""The oracle against the golden fixtures generated from the reference's own Python functions, plus
hand-derived known answers for the device-side index maps."""
import os

import numpy as np
import pytest
import torch

from oracle import boundary as ob
from oracle import chain as oc

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


@pytest.fixture(scope="module")
def deps():
    return np.load(os.path.join(GOLD, "chain_deps.npz"))


@pytest.fixture(scope="module")
def bsmall():
    return np.load(os.path.join(GOLD, "boundary_small.npz"))


def test_build_deps_matches_reference(deps):
    n = sum(1 for k in deps.files if k.endswith("_args") and k.startswith("case"))
    assert n >= 12
    for i in range(n):
        a = [int(v) for v in deps[f"case{i}_args"]]
        off, cons, init = oc.build_deps(*a[:7], rowpanel=bool(a[7]))
        assert off.dtype == cons.dtype == init.dtype == np.int32
        assert np.array_equal(off, deps[f"case{i}_off"]), a
        assert np.array_equal(cons, deps[f"case{i}_cons"]), a
        assert np.array_equal(init, deps[f"case{i}_init"]), a


def test_build_deps_headline_known_answer():
    # the 2-rank chain config with 128x128 tiles: one dependency per producer tile, consumer panel == m, 64 per panel
    off, cons, init = oc.build_deps(1024, 8192, 8192, 128, 128, 128, 128, True)
    assert np.array_equal(off, np.arange(513))
    assert np.array_equal(cons, np.repeat(np.arange(8), 64))
    assert init.shape == (8 * 32,) and np.all(init[::32] == 64) and init.sum() == 512


def test_producer_order_matches_reference(deps):
    n = sum(1 for k in deps.files if k.startswith("order") and k.endswith("_args"))
    assert n >= 5
    for j in range(n):
        P, tn1, g = (int(v) for v in deps[f"order{j}_args"])
        assert np.array_equal(oc.producer_order(P, tn1, g), deps[f"order{j}"])
    assert np.array_equal(oc.producer_order(12, 4, 0), np.arange(12))


@pytest.mark.parametrize("case", [(1024, 8192, 8192, 128, 256, 128, 256, True, 0), (1024, 8192, 8192, 128, 256, 128, 256, True, 8),
                                  (512, 1024, 1536, 128, 128, 128, 256, False, 0), (1000, 1000, 520, 128, 128, 64, 256, True, 2),
                                  (4096, 8192, 8192, 64, 256, 128, 128, True, 8)])
def test_link_simulation_invariants(case):
    M, N1, N2, BM1, BN1, BM2, BN2, rp, g = case
    entries, tail, sb = oc.simulate_link(M, N1, N2, BM1, BN1, BM2, BN2, rp, g)
    tn2 = oc.cdiv(N2, BN2)
    C = oc.cdiv(M, BM2) * tn2
    assert oc.check_link_invariants(entries, tail, sb, C, tn2, rp) == []


def test_link_simulation_order_known_answer():
    # 2 panels x 2 n-tiles feeding 2 panels x 3 n-tiles, ascending producer order: panel 0 completes first
    entries, tail, sb = oc.simulate_link(256, 512, 768, 128, 256, 128, 256, True, 0)
    assert entries.tolist() == [0, 1, 2, 3, 4, 5] and tail == 6 and not sb.any()
    # producer walks panel 1 first
    entries, _, _ = oc.simulate_link(256, 512, 768, 128, 256, 128, 256, True, 0, order=[2, 3, 0, 1])
    assert entries.tolist() == [3, 4, 5, 0, 1, 2]
    # a dropped producer tile leaves its panel unpublished (what a lost flag looks like)
    entries, tail, sb = oc.simulate_link(256, 512, 768, 128, 256, 128, 256, True, 0, order=[0, 1, 2])
    assert tail == 3 and entries.tolist() == [0, 1, 2, -1, -1, -1] and sb[32] == 1
    assert oc.check_link_invariants(entries, tail, sb, 6, 3, True) != []


def test_remap_tile_known_answers_and_bijection():
    # TM=4 panels, TN=8 n-tiles, tail C=2: head = 4*6 = 24 indices m-fast, then panel-major over n in {6,7}
    assert ob.remap_tile(0, 4, 8, 2) == (0, 0)
    assert ob.remap_tile(3, 4, 8, 2) == (3, 0)
    assert ob.remap_tile(4, 4, 8, 2) == (0, 1)
    assert ob.remap_tile(23, 4, 8, 2) == (3, 5)
    assert ob.remap_tile(24, 4, 8, 2) == (0, 6)
    assert ob.remap_tile(25, 4, 8, 2) == (0, 7)
    assert ob.remap_tile(26, 4, 8, 2) == (1, 6)
    assert ob.remap_tile(31, 4, 8, 2) == (3, 7)
    for TM, TN, C in [(32, 32, 16), (8, 32, 8), (1, 32, 8), (5, 32, 16), (64, 32, 16), (7, 4, 0), (3, 32, 32)]:
        seen = {ob.remap_tile(L, TM, TN, C) for L in range(TM * TN)}
        assert seen == {(m, n) for m in range(TM) for n in range(TN)}


def test_unit_map_follows_producer_order():
    # every unit exactly once, and the (panel, n) sequence of a rank's units is the producer sequence filtered to its panels
    for M, world in [(4096, 4), (4096, 8), (1024, 2), (512, 4), (896, 4), (128, 4), (8192, 8)]:
        TM, TN = M // 128, 32
        C = ob.tail_cols(M)
        prod = [ob.remap_tile(L, TM, TN, C) for L in range(TM * TN)]
        for rank in range(world):
            Pr = ob.panels_owned(M, rank, world)
            assert Pr == len([m for m in range(TM) if m % world == rank])
            units = [ob.unit_map(u, Pr, TN, C) for u in range(Pr * TN * 4)]
            assert len(set(units)) == len(units)
            seq = [(j * world + rank, n) for (j, n, q) in units if q == 0]
            assert seq == [(m, n) for (m, n) in prod if m % world == rank]
            assert all(units[4 * i + q] == (units[4 * i][0], units[4 * i][1], q) for i in range(len(units) // 4) for q in range(4))


def test_unit_map_for_panel_major_and_plain_m_fast_orders():
    # tail == all n-tiles: the producer walks panel by panel (short producers); tail == 0: m fastest everywhere
    for M, world, C in [(1024, 4, 32), (1024, 2, 0), (640, 4, 32), (2048, 8, 0)]:
        TM, TN = M // 128, 32
        prod = [ob.remap_tile(L, TM, TN, C) for L in range(TM * TN)]
        if C == TN:
            assert prod[:TN] == [(0, n) for n in range(TN)]
        for rank in range(world):
            Pr = ob.panels_owned(M, rank, world)
            units = [ob.unit_map(u, Pr, TN, C) for u in range(Pr * TN * 4)]
            assert [(j * world + rank, n) for (j, n, q) in units if q == 0] == [(m, n) for (m, n) in prod if m % world == rank]


def test_tail_and_ppo_rules():
    assert ob.tail_cols(4096) == 16 and ob.tail_cols(2048) == 16 and ob.tail_cols(1920) == 8 and ob.tail_cols(128) == 8
    assert ob.tail_cols(4096, raster=2) == 0 and ob.tail_cols(4096, swizzle=2) == 0
    assert ob.panels_per_owner(8192, 4) == 16 and ob.panels_per_owner(8192, 8) == 8 and ob.panels_per_owner(640, 4) == 2
    assert ob.tile_flag_index(2, 3, 5, 16) == (2 * 16 + 3) * 32 + 5


@pytest.mark.parametrize("world", [2, 4, 8])
def test_boundary_protocol_state(world):
    sim = ob.BoundarySim(2048, world)
    for epoch, M in enumerate((2048, 512, 1280), start=1):
        sim.step(M, epoch)
        P = M // 128
        assert np.all(sim.panel_flag[:, :P] == epoch)
        for r in range(world):
            Pr = ob.panels_owned(M, r, world)
            assert np.all(sim.tile_flags[r, :, :Pr, :] == epoch)
            own = [m for m in range(P) if m % world == r]
            assert np.all(sim.panel_done[r, own] == 128)


def test_boundary_arithmetic_matches_reference(bsmall):
    for k in range(2):
        M, K, H, N2_, world, seed = (int(v) for v in bsmall[f"b{k}_args"])
        h, resid, Wd, gamma, Wq = (bf16(bsmall[f"b{k}_{n}"]) for n in ("h", "resid", "Wd", "gamma", "Wq"))
        x, out = ob.boundary_reference(h, Wd, resid, gamma, Wq)
        assert torch.equal(x, torch.from_numpy(bsmall[f"b{k}_x"]))
        assert torch.equal(out, torch.from_numpy(bsmall[f"b{k}_out"]))
        x, out = ob.boundary_reference(h, Wd, None, gamma, Wq)
        assert torch.equal(x, torch.from_numpy(bsmall[f"b{k}_x_noresid"]))
        assert torch.equal(out, torch.from_numpy(bsmall[f"b{k}_out_noresid"]))
        assert torch.equal(ob.fold_gamma(Wq, gamma), bf16(bsmall[f"b{k}_fold"]))
        for r in range(world):
            wd, wq, wqf = ob.shard_weights(Wd, Wq, gamma, r, world)
            assert torch.equal(wd, bf16(bsmall[f"b{k}_r{r}_Wd"]))
            assert torch.equal(wq, bf16(bsmall[f"b{k}_r{r}_Wq"]))
            assert torch.equal(wqf, bf16(bsmall[f"b{k}_r{r}_Wqf"]))
        # the device rounding model stays within the acceptance tolerance of the fp32 reference
        xr, outr = ob.boundary_reference(h, Wd, resid, gamma, Wq)
        xm, outm = ob.boundary_device_model(h, Wd, resid, gamma, Wq, world)
        mx, mean = oc.error_stats(outm, outr)
        assert mx <= 2e-2 and mean <= 5e-3, (mx, mean)
        mx, mean = oc.error_stats(xm, xr)
        assert mx <= 2e-2 and mean <= 5e-3, (mx, mean)


def test_chain_reference_small():
    X, Ws = oc.make_chain_inputs(64, 128, [96, 80], seed=0)
    ys = oc.chain_reference(X, Ws, keep=True)
    assert ys[0].shape == (64, 96) and ys[1].shape == (64, 80) and ys[1].dtype == torch.bfloat16
    ref = torch.nn.functional.linear(torch.nn.functional.linear(X.float(), Ws[0].float()), Ws[1].float())
    mx, mean = oc.error_stats(ys[1], ref)
    assert mx <= 2e-2 and mean <= 5e-3
    X2, Ws2 = oc.make_chain_inputs(64, 128, [96, 80], seed=0)
    assert torch.equal(X, X2) and all(torch.equal(a, b) for a, b in zip(Ws, Ws2))


def test_unit_map_orders_are_bijections_and_follow_the_producer():
    """Every unit order visits each (panel, n-tile, quarter) once; the tail order is the producer's ``remap_tile`` restricted to
    a rank's panels; order 2 is panel by panel; swizzle groups keep ``swz`` n-tiles together."""
    for Pr, tn, tail, order, swz in ((4, 8, 0, 1, 1), (4, 8, 0, 1, 2), (4, 8, 0, 1, 4), (3, 6, 0, 2, 1), (5, 8, 3, 1, 1)):
        units = [ob.unit_map(u, Pr, tn, tail, order, swz) for u in range(Pr * tn * 4)]
        assert sorted(units) == [(j, n, q) for j in range(Pr) for n in range(tn) for q in range(4)]
    assert [ob.unit_map(4 * t, 2, 4, 0, 1, 2)[:2] for t in range(8)] == [(0, 0), (0, 1), (1, 0), (1, 1), (0, 2), (0, 3), (1, 2), (1, 3)]
    assert [ob.unit_map(4 * t, 2, 3, 0, 2)[:2] for t in range(6)] == [(0, 0), (0, 1), (0, 2), (1, 0), (1, 1), (1, 2)]
    # tail order == the producer's order when one rank owns every panel
    assert [ob.unit_map(4 * t, 4, 8, 3)[:2] for t in range(32)] == [ob.remap_tile(L, 4, 8, 3) for L in range(32)]


def test_tile_orders_are_bijections():
    for order, TM, TN, g, tail in ((0, 7, 5, 3, 0), (0, 4, 4, 8, 0), (1, 6, 8, 0, 3), (1, 6, 8, 0, 0), (2, 5, 3, 0, 0)):
        tiles = ob.tile_order(order, TM, TN, g, tail)
        assert sorted(tiles) == [(m, n) for m in range(TM) for n in range(TN)]
    assert ob.tile_order(0, 3, 2, 2) == [(0, 0), (1, 0), (0, 1), (1, 1), (2, 0), (2, 1)]


def test_kchunk_link_model():
    """Flags all carry the run's number afterwards; a consumer tile can complete only after the LAST producer tile of its row
    (in producer order) has finished, and a consumer walking the same grouped order as its producer never needs a tile from a
    later group than its own."""
    tm, tn1, tn2, g = 8, 4, 6, 2
    o1, o2 = oc.producer_order(tm * tn1, tn1, g), oc.producer_order(tm * tn2, tn2, g)
    flags, need = oc.simulate_kchunk_link(o1, tn1, o2, tn2, tn1, run_id=3)
    assert flags.shape == (tm, tn1) and (flags == 3).all()
    rows = o2 // tn2
    assert (need <= (rows // g + 1) * g * tn1).all() and (need > (rows // g) * g * tn1).all()
    assert (np.diff(need.reshape(-1, g * tn2).max(axis=1)) > 0).all()          # groups become ready in order
