"""The committed fixtures are what the oracle computes today (a changed oracle fails here), and they
carry the invariants the reference's tests state for these quantities."""
import sys
from pathlib import Path

import numpy as np

GOLD = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLD))


def test_dense_fixtures_reproduce(oracle):
    import make_golden as M
    for name in ("wan_dense_tiny", "wan_causal_small"):
        g = np.load(GOLD / f"{name}.npz")
        causal = tuple(int(x) for x in g["causal"])
        case = M.wan_dense_case(int(g["seed"]), int(g["batch"]), tuple(int(x) for x in g["grid"]), int(g["heads"]),
                                g["rows"], causal if causal[0] else None)
        assert np.array_equal(case["out"], g["out"])
        assert np.array_equal(case["q_rows"], g["q_rows"])
        # softmax rows are convex combinations of V: bounded by V's range
        assert np.isfinite(g["out"]).all() and np.abs(g["out"]).max() < 6.0


def test_causal_fixture_first_chunk_sees_only_itself(oracle):
    import make_golden as M
    g = np.load(GOLD / "wan_causal_small.npz")
    grid, heads, seed = tuple(int(x) for x in g["grid"]), int(g["heads"]), int(g["seed"])
    proj, w, seq, dim = M.wan_inputs(seed, 1, grid, heads)
    cos, sin = oracle.wan_rope(*grid)
    q = oracle.qk_norm_rope_bhsd(proj, w, cos, sin, 1, seq, heads, 128, 3 * dim, 0)
    k = oracle.qk_norm_rope_bhsd(proj, w, cos, sin, 1, seq, heads, 128, 3 * dim, dim)
    v = oracle.split_heads_bhsd(proj, 1, seq, heads, 128, 3 * dim, 2 * dim)
    # rows 0 and 39 lie in chunk 0 (40 tokens): dense attention over the first 40 keys alone
    first = oracle.sdpa_rows(q[:, :40], k[:, :40], v[:, :40], rows=np.array([0, 39], np.int32))
    assert np.abs(first - g["out"][:, :2]).max() < 1e-6


def test_vsa_fixture_reproduces(oracle):
    g = np.load(GOLD / "vsa_small.npz")
    grid, heads, topk = tuple(int(x) for x in g["grid"]), int(g["heads"]), int(g["topk"])
    seq = grid[0] * grid[1] * grid[2]
    q, k, v, lg = (oracle.bf16_round(oracle.seeded_normal(int(g["seed"]), i, (heads, seq, 128))) for i in range(4))
    gate = oracle.bf16_round((1.0 / (1.0 + np.exp(-lg.astype(np.float64)))).astype(np.float32))
    out, sel, scores, coarse = oracle.vsa_attention_host(q, k, v, gate, grid, topk, want_aux=True)
    assert np.array_equal(np.sort(sel, axis=-1), g["selected_sorted"])
    assert np.array_equal(scores, g["scores"]) and np.array_equal(out[:, g["rows"]], g["out"])
    assert g["selected_sorted"].shape == (heads, 12, 4)


def test_rope_fixture(oracle):
    g = np.load(GOLD / "rope_480p_rows.npz")
    c, s = oracle.wan_rope(21, 30, 52)
    assert np.array_equal(c[g["rows"]], g["cos"]) and np.array_equal(s[g["rows"]], g["sin"])
