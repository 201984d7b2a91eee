"""The reference's own closed-form unit tests, re-run against the CPU oracle (file:line of each
reference test in its docstring; paths inside zaitrarrio/fastvideo-rs).  These pin the oracle."""
import math

import numpy as np
import pytest


def lcg_stream(seed, n, inc=1442695040888963407):
    """s = s*6364136223846793005 + inc; x = (s >> 33) / 2^31 - 0.5  (rt/vsa.rs:541-551, :663-667)."""
    out = np.empty(n, np.float32)
    s = seed
    mask = (1 << 64) - 1
    for i in range(n):
        s = (s * 6364136223846793005 + inc) & mask
        out[i] = np.float32(np.float32(s >> 33) / np.float32(1 << 31)) - np.float32(0.5)
    return out


def sin_fill(shape, k, amp=0.9, off=0.0):
    """t(n, k) = sin(i*k)*amp (+ off)  (rt/sdpa.rs:513-519, wan/fuse.rs:627-632)."""
    n = int(np.prod(shape))
    i = np.arange(n, dtype=np.float32)
    return (np.sin(i * np.float32(k)).astype(np.float32) * np.float32(amp) + np.float32(off)).reshape(shape)


def test_bf16_round_matches_numpy_twin(oracle):
    x = np.concatenate([oracle.seeded_normal(3, 0, (4096,)), np.array([0.0, -0.0, 1.0, 65280.0, 3.3895314e38, np.inf,
                                                                          -np.inf, 1e-40], np.float32)])
    assert np.array_equal(oracle.bf16_round(x).view(np.uint32), oracle.bf16_round_np(x).view(np.uint32))
    # ties go to even: 1 + 2^-8 sits halfway between 1 and 1 + 2^-7
    assert oracle.bf16_round(np.array([1.00390625], np.float32))[0] == 1.0
    assert oracle.bf16_round(np.array([1.01171875], np.float32))[0] == np.float32(1.015625)
    assert np.isnan(oracle.bf16_round(np.array([np.nan], np.float32))[0])


def test_shard_ranges_cover_seq(oracle):
    """rt/sp.rs:66-73"""
    assert oracle.shard_ranges(10, 2) == [(0, 5), (5, 5)]
    assert oracle.shard_ranges(11, 2) == [(0, 6), (6, 5)]
    assert sum(l for _, l in oracle.shard_ranges(11, 2)) == 11
    assert oracle.shard_ranges(75600, 8) == [(9450 * r, 9450) for r in range(8)]
    assert oracle.shard_ranges(32760, 8) == [(4095 * r, 4095) for r in range(8)]


def test_shard_gather_round_trip(oracle):
    """rt/sp.rs:75-84"""
    a = np.arange(12, dtype=np.float32).reshape(1, 1, 4, 3)
    parts = [a[:, :, s : s + l] for s, l in oracle.shard_ranges(4, 2)]
    assert np.array_equal(np.concatenate(parts, axis=2), a)


@pytest.mark.parametrize("grid", [(4, 4, 4), (33, 28, 52), (3, 5, 7), (1, 1, 1)])
def test_tiling_is_a_permutation_with_padding(oracle, grid):
    """rt/vsa.rs:481-507"""
    p = oracle.TilePlan(grid)
    assert p.seq == grid[0] * grid[1] * grid[2]
    assert p.padded == p.num_tiles * 64
    real = p.slot_src[p.slot_src >= 0]
    assert sorted(real.tolist()) == list(range(p.seq))
    slots = np.nonzero(p.slot_src >= 0)[0]
    assert np.array_equal(p.token_slot[p.slot_src[slots]], slots.astype(np.uint32))
    assert int(p.block_sizes.sum()) == p.seq
    assert (p.block_sizes <= 64).all()


def test_full_tiles_have_no_padding(oracle):
    """rt/vsa.rs:509-514"""
    p = oracle.TilePlan((8, 8, 8))
    assert (p.slot_src >= 0).all() and (p.block_sizes == 64).all()


def test_partial_tile_keeps_subcube_order(oracle):
    """rt/vsa.rs:516-526"""
    p = oracle.TilePlan((1, 1, 5))
    assert p.num_tiles == 2
    assert p.block_sizes.tolist() == [4, 1]
    assert p.slot_src[:4].tolist() == [0, 1, 2, 3]
    assert (p.slot_src[4:64] == -1).all()
    assert p.slot_src[64] == 4


def test_topk_matches_upstream_rule(oracle):
    """rt/vsa.rs:528-534"""
    assert oracle.topk_for(0.8, 819) == 164
    assert oracle.topk_for(0.0, 819) == 819
    assert oracle.topk_for(1.0, 819) == 1
    assert oracle.topk_for(0.9, 10) == 1
    assert oracle.topk_for(0.875, 624) == 78  # the 12.5 % of the VSA bench configuration


def test_wan_480p_grid_tiles(oracle):
    p = oracle.TilePlan((21, 30, 52))
    assert p.tiles == (6, 8, 13) and p.num_tiles == 624 and p.padded == 39936


def test_all_tiles_selected_and_zero_gate_is_dense_attention(oracle):
    """rt/vsa.rs:536-597: LCG inputs seeds 1, 2, 3, grid (2, 3, 5), 2 heads, dim 8."""
    heads, dim, grid = 2, 8, (2, 3, 5)
    seq = 30
    n = heads * seq * dim
    q, k, v = (lcg_stream(s, n).reshape(heads, seq, dim) for s in (1, 2, 3))
    gate = np.zeros_like(q)
    scale = 1.0 / math.sqrt(dim)
    got = oracle.vsa_attention_host(q, k, v, gate, grid, oracle.TilePlan(grid).num_tiles, scale)
    # plain dense attention: f32 scores, f64 softmax and PV
    want = np.zeros_like(q)
    for h in range(heads):
        s = np.zeros((seq, seq), np.float32)
        for i in range(seq):
            for j in range(seq):
                acc = np.float32(0)
                for d in range(dim):
                    acc = np.float32(acc + np.float32(q[h, i, d] * k[h, j, d]))
                s[i, j] = np.float32(acc * np.float32(scale))
        m = s.max(axis=1, keepdims=True)
        e = np.exp((s - m).astype(np.float64))
        want[h] = ((e @ v[h].astype(np.float64)) / e.sum(axis=1, keepdims=True)).astype(np.float32)
    assert np.abs(got - want).max() < 2e-5


def test_gate_adds_the_coarse_branch(oracle):
    """rt/vsa.rs:601-656"""
    dim, grid = 4, (1, 4, 4)
    n = 16 * dim
    i = np.arange(n)
    q = ((i % 7).astype(np.float32) * np.float32(0.1) - np.float32(0.3)).reshape(1, 16, dim)
    k = ((i % 5).astype(np.float32) * np.float32(0.2) - np.float32(0.4)).reshape(1, 16, dim)
    v = ((i % 3).astype(np.float32) * np.float32(0.3) - np.float32(0.3)).reshape(1, 16, dim)
    nb = oracle.TilePlan(grid).num_tiles
    scale = 1.0 / math.sqrt(dim)
    zero = oracle.vsa_attention_host(q, k, v, np.zeros_like(q), grid, nb, scale)
    one = oracle.vsa_attention_host(q, k, v, np.ones_like(q), grid, nb, scale)
    none = oracle.vsa_attention_host(q, k, v, None, grid, nb, scale)
    assert np.abs(one - none).max() < 1e-6
    assert np.abs(one - zero).max() > 1e-4


def test_fewer_tiles_changes_the_result_but_stays_finite(oracle):
    """rt/vsa.rs:659-695: LCG with increment 1, seed 99, one stream feeding q, k, v in turn."""
    dim, grid = 8, (4, 8, 8)
    n = 256 * dim
    stream = lcg_stream(99, 3 * n, inc=1)
    q, k, v = (stream[i * n : (i + 1) * n].reshape(1, 256, dim) for i in range(3))
    nb = oracle.TilePlan(grid).num_tiles
    scale = 1.0 / math.sqrt(dim)
    sparse = oracle.vsa_attention_host(q, k, v, None, grid, oracle.topk_for(0.8, nb), scale)
    dense = oracle.vsa_attention_host(q, k, v, None, grid, nb, scale)
    assert np.isfinite(sparse).all() and np.isfinite(dense).all()
    assert (np.abs(sparse - dense) > 1e-6).any()


def test_vsa_selection_is_descending_with_low_index_ties(oracle):
    """rt/vsa.rs:203-212: emission order is score descending, ties to the lower tile index."""
    dim, grid = 8, (4, 8, 8)
    n = 256 * dim
    q, k, v = (oracle.seeded_normal(5, i, (1, 256, dim)) for i in range(3))
    _, sel, scores, _ = oracle.vsa_attention_host(q, k, v, None, grid, 3, want_aux=True)
    for qt in range(sel.shape[1]):
        order = sorted(range(scores.shape[2]), key=lambda j: (-scores[0, qt, j], j))
        assert sel[0, qt].tolist() == order[:3]


@pytest.mark.parametrize("window,fpb", [(-1, 3), (3, 3), (6, 3), (-1, 1), (1, 1), (2, 1)])
def test_block_causal_predicate_equals_the_models_mask(oracle, window, fpb):
    """rt/attn.rs:883-903: frames 9, h 6, w 4 with patch (1, 2, 2) -> 9 x 3 x 2 tokens."""
    frame_tokens, seq = 3 * 2, 9 * 3 * 2
    bc = oracle.block_causal_for(fpb, window, frame_tokens)
    assert bc is not None
    want = oracle.causal_temporal_mask(seq, frame_tokens, fpb, window)
    got = oracle.block_causal_mask(*bc, seq, seq)
    assert np.array_equal(got, want)
    for qi in (0, 5, 17, seq - 1):
        for ki in (0, 6, 23, seq - 1):
            assert oracle.block_causal_allows(*bc, qi, ki) == (want[qi, ki] == 0.0)


def test_token_granular_window_has_no_block_form(oracle):
    """rt/attn.rs:899-902: local_attn_size 4 with 3 frames per block is not whole blocks."""
    assert oracle.block_causal_for(3, 4, 6) is None


def test_block_causal_rows_equal_masked_composed(oracle):
    """rt/attn.rs:906-930: {block 5, window 2, sink 1} on (1, 2, 24, 8): the parameterised mask and the
    additive dense mask give the same bits."""
    q = sin_fill((2, 24, 8), 0.37)
    k = sin_fill((2, 24, 8), 0.71)
    v = sin_fill((2, 24, 8), 1.13)
    mask = oracle.block_causal_mask(5, 2, 1, 24, 24)
    a = oracle.sdpa_rows(q, k, v, mask=mask)
    b = oracle.sdpa_rows(q, k, v, block_causal=(5, 2, 1))
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    f = oracle.sdpa_rows_f64(q, k, v, block_causal=(5, 2, 1))
    assert np.abs(a - f).max() < 1e-5


def test_composed_sdpa_closed_form_inputs(oracle):
    """rt/sdpa.rs:513-542: t(n, k) = sin(i k) 0.9 on (1, 2, 5, 7, 8); the default scale is 1/sqrt(d) and
    another scale gives another result.  The C++ restatement and its numpy twin agree to a few ulp
    (they differ only in the libm behind exp)."""
    q = sin_fill((2, 5, 8), 0.37)
    k = sin_fill((2, 7, 8), 0.71)
    v = sin_fill((2, 7, 8), 1.13)
    a = oracle.sdpa_rows(q, k, v)
    b = oracle.sdpa_composed_np(q, k, v)
    assert np.abs(a - b).max() < 5e-7
    assert np.array_equal(a, oracle.sdpa_rows(q, k, v, scale=1.0 / math.sqrt(8)))
    assert np.abs(a - oracle.sdpa_rows(q, k, v, scale=0.5)).max() > 1e-4
    assert np.abs(a - oracle.sdpa_rows_f64(q, k, v)).max() < 1e-6
    # a zero additive mask changes nothing, bit for bit
    assert np.array_equal(a, oracle.sdpa_rows(q, k, v, mask=np.zeros((5, 7), np.float32)))


def test_rope_tables_layout_and_twin(oracle):
    """wan/transformer.rs:447-544: 44/42/42 split, values repeated in pairs, position 0 is identity."""
    c, s = oracle.wan_rope(3, 8, 8)
    assert c.shape == (192, 128)
    assert np.array_equal(c[0], np.ones(128, np.float32)) and np.array_equal(s[0], np.zeros(128, np.float32))
    assert np.array_equal(c[:, 0::2], c[:, 1::2]) and np.array_equal(s[:, 0::2], s[:, 1::2])
    # token (t=1, h=0, w=0) rotates only the first 44 dims; (0, 1, 0) only dims 44..85; (0, 0, 1) only 86..127
    t1, h1, w1 = 64, 8, 1
    assert (s[t1, :44] != 0).any() and not s[t1, 44:].any()
    assert (s[h1, 44:86] != 0).any() and not s[h1, :44].any() and not s[h1, 86:].any()
    assert (s[w1, 86:] != 0).any() and not s[w1, :86].any()
    assert s[t1, 0] == np.float32(math.sin(1.0))  # correctly rounded sin(1)
    c2, s2 = oracle.wan_rope_np(3, 8, 8)
    assert np.abs(c - c2).max() < 2e-7 and np.abs(s - s2).max() < 2e-7


def test_qk_norm_rope_matches_definition(oracle):
    """rt/ops.rs:2304-2350 against a direct numpy evaluation; wan/fuse.rs:627-662's fill vals(n, k) =
    sin(i k) 1.3 + 0.1."""
    b, seq, heads, d = 1, 6, 3, 128
    width = 3 * heads * d
    src = sin_fill((b, seq, width), 0.013, 1.3, 0.1)
    w = sin_fill((heads * d,), 0.21, 0.5, 1.0)
    c, s = oracle.wan_rope(1, 2, 3)
    out = oracle.qk_norm_rope_bhsd(src, w, c, s, b, seq, heads, d, width, heads * d, 1e-6)
    x = src[0, :, heads * d : 2 * heads * d].astype(np.float64)
    inv = 1.0 / np.sqrt((x * x).mean(axis=1, keepdims=True) + 1e-6)
    y = (x * inv * w.astype(np.float64)).reshape(seq, heads, d).transpose(1, 0, 2)
    ye, yo = y[..., 0::2], y[..., 1::2]
    ce, so = c[None, :, 0::2].astype(np.float64), s[None, :, 1::2].astype(np.float64)
    want = np.empty_like(y)
    want[..., 0::2] = ye * ce - yo * so
    want[..., 1::2] = ye * so + yo * ce
    assert np.abs(out - want).max() < 2e-5
    # no rope: plain norm * w
    plain = oracle.qk_norm_rope_bhsd(src, w, None, None, b, seq, heads, d, width, heads * d, 1e-6)
    assert np.abs(plain - y).max() < 2e-5
    # the statistic spans all heads: per-head differs
    per = oracle.qk_norm_rope_bhsd(src, w, None, None, b, seq, heads, d, width, heads * d, 1e-6, per_head=True)
    assert np.abs(per - plain).max() > 1e-3


def test_block_glue_twins_closed_form(oracle):
    """The restatements of ln_adaln_e (C/rt/kernels/act16.cu:184-209) and of the fused residual + norm
    (C/wan/kernels/block.cu:17-78) on inputs whose answer is known in closed form: a zero AdaLN table leaves a
    plain LayerNorm (zero mean, unit variance), scale / shift rows act as (1 + s) and + t, a zero gate leaves the
    hidden state as it was, and the norm of the residual reads the UNROUNDED sum (a sum that rounds to a
    constant row still has a non-zero normalised output)."""
    x = oracle.seeded_normal(5, 0, (2, 9, 64))
    e = np.zeros((2, 6, 64), np.float32)
    y = oracle.ln_adaln_e(x, e, 1, 0)
    assert np.abs(y.mean(-1)).max() < 1e-6 and np.abs(y.var(-1) - 1.0).max() < 1e-4
    e[:, 1] = 0.5
    e[:, 0] = -2.0
    assert np.allclose(oracle.ln_adaln_e(x, e, 1, 0), y * 1.5 - 2.0, atol=1e-6)
    h = oracle.bf16_round(x)
    a = oracle.bf16_round(oracle.seeded_normal(5, 1, (2, 9, 64)))
    w, b = np.full(64, 2.0, np.float32), np.full(64, 0.25, np.float32)
    hid, normed = oracle.self_residual_norm(h, a, np.zeros((2, 6, 64), np.float32), 2, w, b)
    assert np.array_equal(hid, h)
    assert np.allclose(normed, 2.0 * oracle.ln_adaln_e(h, np.zeros((2, 6, 64), np.float32), 0, 0) + 0.25, atol=1e-5)
    # unrounded sum: h = 1 everywhere, attn * gate = tiny alternating values that vanish in bf16(h + .)
    h1 = np.ones((1, 1, 64), np.float32)
    a1 = (np.where(np.arange(64) % 2 == 0, 1.0, -1.0) * 2.0 ** -12).astype(np.float32).reshape(1, 1, 64)
    g = np.ones((1, 6, 64), np.float32)
    hid1, n1 = oracle.self_residual_norm(h1, a1, g, 2, np.ones(64, np.float32), np.zeros(64, np.float32))
    assert np.array_equal(hid1, h1) and np.abs(n1).min() > 0.2  # 2^-12 / sqrt(2^-24 + eps)


def test_rope_bhsd_twin_follows_the_host_loop(oracle):
    """apply_rotary_bshd (C/rt/ops.rs:1903-1933) restated as the plain loop on a small case, against the
    vectorised twin; rotating back with the negated sine (C/wan/causal.rs:764-771) returns the input up to
    one rounding."""
    import numpy as np
    cos, sin = oracle.wan_rope(2, 2, 3)
    x = oracle.seeded_normal(77, 0, (3, 12, 128))
    got = oracle.rope_bhsd(x, cos, sin)
    want = np.empty_like(x)
    for b in range(3):
        for t in range(12):
            for i in range(64):
                x1, x2 = x[b, t, 2 * i], x[b, t, 2 * i + 1]
                cs, sn = cos[t, 2 * i], sin[t, 2 * i]
                want[b, t, 2 * i] = np.float32(x1 * cs) - np.float32(x2 * sn)
                want[b, t, 2 * i + 1] = np.float32(x1 * sn) + np.float32(x2 * cs)
    assert np.array_equal(got, want)
    back = oracle.rope_bhsd(got, cos, sin, negate_sin=True)
    assert np.abs(back - x).max() < 1e-6
