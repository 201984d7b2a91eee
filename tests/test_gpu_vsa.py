"""VSA on the device against vsa_attention_host (the oracle): tile selection exact (as sets), coarse
scores bit-identical, outputs within tolerance."""
import math
from pathlib import Path

import numpy as np
import pytest
import torch

from _util import assert_close, to_dev_bf16, to_host_f32

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def inputs(oracle, seed, bh, seq, sigmoid_gate=True):
    q, k, v, g = (oracle.bf16_round(oracle.seeded_normal(seed, i, (bh, seq, 128))) for i in range(4))
    if sigmoid_gate:  # the bench configuration: sigmoid applied to seeded logits before the call
        g = oracle.bf16_round((1.0 / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32))
    return q, k, v, g


def test_plan_equals_oracle(fvlib, oracle):
    from fastvideo_rs_b200 import vsa
    for grid in ((4, 4, 4), (33, 28, 52), (3, 5, 7), (1, 1, 1), (8, 8, 8), (1, 1, 5), (21, 30, 52)):
        a, b = vsa.TilePlan(grid), oracle.TilePlan(grid)
        assert a.num_tiles == b.num_tiles and a.seq == b.seq and a.padded == b.padded and a.tiles == b.tiles
        assert np.array_equal(a.slot_src, b.slot_src) and np.array_equal(a.token_slot, b.token_slot)
        assert np.array_equal(a.block_sizes, b.block_sizes)
    assert vsa.topk_for(0.8, 819) == 164 and vsa.topk_for(0.0, 819) == 819 and vsa.topk_for(1.0, 819) == 1
    assert vsa.topk_for(0.9, 10) == 1 and vsa.topk_for(0.875, 624) == 78


@pytest.mark.parametrize("grid,bh,topk", [((5, 6, 9), 2, 4), ((4, 8, 8), 2, 3), ((8, 8, 8), 1, 8), ((3, 5, 7), 3, 2),
                                           ((6, 12, 16), 2, 9), ((1, 1, 5), 1, 1), ((4, 4, 12), 2, 3)])
def test_vsa_matches_host(fvlib, oracle, grid, bh, topk):
    from fastvideo_rs_b200 import sdpa, vsa
    seq = grid[0] * grid[1] * grid[2]
    q, k, v, g = inputs(oracle, 500 + seq, bh, seq)
    ctx = vsa.VsaCtx(grid, topk=topk)
    out, sel, sc, co = vsa.vsa_attention(to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v), to_dev_bf16(g), ctx, want_aux=True)
    assert sdpa.device_status() == 0
    want, wsel, wsc, wco = oracle.vsa_attention_host(q, k, v, g, grid, topk, want_aux=True)
    assert np.array_equal(to_host_f32(sc).view(np.uint32), wsc.view(np.uint32)), "coarse scores must be bit-identical"
    got_sel = sel.cpu().numpy()
    assert np.array_equal(got_sel, np.sort(got_sel, axis=-1)), "selection is emitted in ascending tile order"
    assert np.array_equal(got_sel, np.sort(wsel.astype(np.int64), axis=-1)), "selected tile sets differ"
    assert np.abs(to_host_f32(co) - wco).max() < 1e-5
    assert_close(to_host_f32(out), want, f"vsa {grid}")


def test_vsa_golden_fixture(fvlib, oracle):
    from fastvideo_rs_b200 import vsa
    g = np.load(ROOT / "tests" / "golden" / "vsa_small.npz")
    grid, heads, topk = tuple(int(x) for x in g["grid"]), int(g["heads"]), int(g["topk"])
    seq = grid[0] * grid[1] * grid[2]
    q, k, v, gate = inputs(oracle, int(g["seed"]), heads, seq)
    ctx = vsa.VsaCtx(grid, topk=topk)
    out, sel, sc, _ = vsa.vsa_attention(to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v), to_dev_bf16(gate), ctx, want_aux=True)
    assert np.array_equal(sel.cpu().numpy(), g["selected_sorted"].astype(np.int64))
    assert np.array_equal(to_host_f32(sc), g["scores"])
    assert_close(to_host_f32(out)[:, g["rows"]], g["out"], "vsa golden")


def test_ties_go_to_the_lower_tile(fvlib, oracle):
    """Identical tiles give identical scores: the selection must keep the lowest indices (rt/vsa.rs:203-212)."""
    from fastvideo_rs_b200 import vsa
    grid, bh, topk = (4, 4, 16), 1, 2  # 4 tiles along w
    seq = 256
    plan = oracle.TilePlan(grid)
    base = oracle.bf16_round(oracle.seeded_normal(9, 0, (64, 128)))
    q = np.zeros((bh, seq, 128), np.float32)
    for tile in range(4):  # every tile holds the same 64 rows -> all coarse scores equal
        q[0, plan.slot_src[tile * 64:(tile + 1) * 64]] = base
    ctx = vsa.VsaCtx(grid, topk=topk)
    tq = to_dev_bf16(q)
    _, sel, sc, _ = vsa.vsa_attention(tq, tq, tq, None, ctx, want_aux=True)
    _, wsel, wsc, _ = oracle.vsa_attention_host(q, q, q, None, grid, topk, want_aux=True)
    assert np.array_equal(to_host_f32(sc), wsc)
    assert np.array_equal(sel.cpu().numpy(), np.sort(wsel.astype(np.int64), axis=-1))
    assert (sel.cpu().numpy() == np.array([0, 1])).all()


def test_all_tiles_selected_and_zero_gate_is_dense_attention(fvlib, oracle):
    """rt/vsa.rs:536-597 on the device: the load-bearing invariant, against the dense kernel."""
    from fastvideo_rs_b200 import sdpa, vsa
    grid, bh = (5, 7, 9), 2  # partial tiles on every axis
    seq = 5 * 7 * 9
    q, k, v, _ = inputs(oracle, 77, bh, seq)
    ctx = vsa.VsaCtx(grid, topk=10 ** 6)
    tq, tk, tv = to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v)
    got = vsa.vsa_attention(tq, tk, tv, torch.zeros_like(tq), ctx, out_bf16=False)
    dense = sdpa.dense_fwd(tq, tk, tv, out_bf16=False)
    assert float((got - dense).abs().max()) < 2e-3
    assert_close(to_host_f32(got), oracle.sdpa_rows(q, k, v), "all tiles == dense")
    # gate of ones == no gate; and the coarse branch changes the result
    one = vsa.vsa_attention(tq, tk, tv, torch.ones_like(tq), ctx, out_bf16=False)
    none = vsa.vsa_attention(tq, tk, tv, None, ctx, out_bf16=False)
    assert torch.equal(one, none)
    assert float((one - got).abs().max()) > 1e-4


def test_vsa_wan_480p_grid_selection_exact(fvlib, oracle):
    """The benchmark configuration's grid (21 x 30 x 52 -> 624 tiles, keep 78) on one head pair: every one
    of the 1248 rows of tile indices equals the host's (as sets), scores are bit-identical, and sampled output
    rows are within tolerance."""
    from fastvideo_rs_b200 import sdpa, vsa
    grid, bh, topk = (21, 30, 52), 2, 78
    seq = 32760
    q, k, v, g = inputs(oracle, 2026, bh, seq)
    ctx = vsa.VsaCtx(grid, sparsity=0.875)
    assert ctx.topk == topk and ctx.plan.num_tiles == 624
    out, sel, sc, _ = vsa.vsa_attention(to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v), to_dev_bf16(g), ctx, want_aux=True)
    assert sdpa.device_status() == 0
    want, wsel, wsc, _ = oracle.vsa_attention_host(q, k, v, g, grid, topk, want_aux=True)
    assert np.array_equal(to_host_f32(sc).view(np.uint32), wsc.view(np.uint32))
    assert np.array_equal(sel.cpu().numpy(), np.sort(wsel.astype(np.int64), axis=-1))
    assert_close(to_host_f32(out), want, "vsa 480p")
