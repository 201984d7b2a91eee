"""The q/k prologue kernel against the oracle's qk_norm_rope_bhsd / split_heads_bhsd."""
import numpy as np
import pytest
import torch

from _util import assert_close, to_dev_bf16, to_host_f32

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("batch,grid,heads,per_head", [(1, (3, 8, 8), 12, False), (2, (2, 5, 7), 12, False),
                                                       (1, (2, 4, 6), 40, False), (1, (2, 3, 5), 12, True),
                                                       (1, (1, 1, 1), 1, False)])
def test_prep_matches_oracle(fvlib, oracle, batch, grid, heads, per_head):
    from fastvideo_rs_b200 import wan
    seq = grid[0] * grid[1] * grid[2]
    dim = heads * 128
    proj = oracle.bf16_round(oracle.seeded_normal(31, 0, (batch, seq, 3 * dim)))
    wq = (1.0 + 0.1 * oracle.seeded_normal(31, 1, (dim,))).astype(np.float32)
    wk = (1.0 + 0.1 * oracle.seeded_normal(31, 2, (dim,))).astype(np.float32)
    cos, sin = oracle.wan_rope(*grid)
    tc, ts = wan.wan_rope_tables(grid)
    assert np.array_equal(to_host_f32(tc), cos) and np.array_equal(to_host_f32(ts), sin)
    q, k, v = wan.qk_prep(to_dev_bf16(proj), torch.from_numpy(wq).cuda(), torch.from_numpy(wk).cuda(), tc, ts, heads,
                          norm_scope=wan.NORM_PER_HEAD if per_head else wan.NORM_ACROSS_HEADS)
    want_q = oracle.qk_norm_rope_bhsd(proj, wq, cos, sin, batch, seq, heads, 128, 3 * dim, 0, 1e-6, per_head)
    want_k = oracle.qk_norm_rope_bhsd(proj, wk, cos, sin, batch, seq, heads, 128, 3 * dim, dim, 1e-6, per_head)
    want_v = oracle.split_heads_bhsd(proj, batch, seq, heads, 128, 3 * dim, 2 * dim)
    gq = to_host_f32(q).reshape(batch * heads, seq, 128)
    gk = to_host_f32(k).reshape(batch * heads, seq, 128)
    gv = to_host_f32(v).reshape(batch * heads, seq, 128)
    assert np.array_equal(gv, want_v)  # a copy: bit exact
    # f32 arithmetic identical up to the order of the sum of squares, then ONE rounding to bf16: the
    # result is the bf16 rounding of the oracle's value except where that value sits on a rounding tie
    for got, want in ((gq, want_q), (gk, want_k)):
        rounded = oracle.bf16_round(want)
        mism = np.mean(got != rounded)
        assert mism < 2e-3, f"{mism:.2e} of the elements differ from the rounded oracle"
        assert np.abs(got - want).max() <= np.abs(want).max() * 2.0 ** -8


@pytest.mark.parametrize("batch,grid,heads,per_head", [(1, (3, 40, 50), 12, False), (2, (2, 30, 40), 40, False),
                                                       (1, (3, 30, 40), 20, False), (1, (3, 20, 25), 48, False),
                                                       (1, (3, 40, 50), 12, True), (1, (5, 40, 50), 1, False), (1, (3, 20, 25), 64, False),
                                                       (1, (3, 20, 25), 7, False), (2, (3, 20, 25), 16, True), (1, (2, 20, 25), 33, False)])
def test_prep_group_kernel_equals_the_row_kernel(fvlib, oracle, batch, grid, heads, per_head, monkeypatch):
    """Enough rows that every persistent group of warps walks several rows, in each launch configuration of the
    default kernel (1, 2, 4 and 8 warps per row; 1 to 5 chunks per thread, ragged last chunk): equal to the oracle
    on sampled rows, and bit for bit to the one-CTA-per-row kernel everywhere (same reduction tree)."""
    from fastvideo_rs_b200 import wan
    seq = grid[0] * grid[1] * grid[2]
    dim = heads * 128
    proj = oracle.bf16_round(oracle.seeded_normal(33, heads, (batch, seq, 3 * dim)))
    wq = (1.0 + 0.1 * oracle.seeded_normal(33, 1, (dim,))).astype(np.float32)
    wk = (1.0 + 0.1 * oracle.seeded_normal(33, 2, (dim,))).astype(np.float32)
    tc, ts = wan.wan_rope_tables(grid)
    scope = wan.NORM_PER_HEAD if per_head else wan.NORM_ACROSS_HEADS
    args = (to_dev_bf16(proj), torch.from_numpy(wq).cuda(), torch.from_numpy(wk).cuda(), tc, ts, heads)
    monkeypatch.delenv("FV_PREP_KERNEL", raising=False)
    q, k, v = wan.qk_prep(*args, norm_scope=scope)
    from fastvideo_rs_b200 import sdpa
    assert sdpa.device_status() == 0
    monkeypatch.setenv("FV_PREP_KERNEL", "row")
    q2, k2, v2 = wan.qk_prep(*args, norm_scope=scope)
    monkeypatch.delenv("FV_PREP_KERNEL")
    assert torch.equal(q, q2) and torch.equal(k, k2) and torch.equal(v, v2)
    cos, sin = oracle.wan_rope(*grid)
    want_q = oracle.qk_norm_rope_bhsd(proj, wq, cos, sin, batch, seq, heads, 128, 3 * dim, 0, 1e-6, per_head)
    want_v = oracle.split_heads_bhsd(proj, batch, seq, heads, 128, 3 * dim, 2 * dim)
    assert np.array_equal(to_host_f32(v).reshape(batch * heads, seq, 128), want_v)
    gq = to_host_f32(q).reshape(batch * heads, seq, 128)
    assert np.mean(gq != oracle.bf16_round(want_q)) < 2e-3
    assert np.abs(gq - want_q).max() <= np.abs(want_q).max() * 2.0 ** -8


def test_prep_without_rope_and_partial_outputs(fvlib, oracle):
    from fastvideo_rs_b200 import wan
    batch, seq, heads = 1, 50, 12
    dim = heads * 128
    proj = oracle.bf16_round(oracle.seeded_normal(32, 0, (batch, seq, dim)))
    w = np.ones(dim, np.float32)
    # cross-attention K: RMS-normed, no rotation, projection of width dim at column 0
    _, k, _ = wan.qk_prep(to_dev_bf16(proj), None, torch.from_numpy(w).cuda(), None, None, heads, col_k=0,
                          want_q=False, want_v=False)
    want = oracle.qk_norm_rope_bhsd(proj, w, None, None, batch, seq, heads, 128, dim, 0, 1e-6)
    got = to_host_f32(k).reshape(heads, seq, 128)
    assert np.mean(got != oracle.bf16_round(want)) < 2e-3


def test_prep_rejects_bad_columns(fvlib, oracle):
    from fastvideo_rs_b200 import FvError, wan
    proj = torch.zeros((1, 8, 1536), dtype=torch.bfloat16, device="cuda")
    w = torch.ones(1536, device="cuda")
    with pytest.raises(FvError):
        wan.qk_prep(proj, w, w, None, None, 12)  # k and v columns fall outside a width-1536 row


def test_prep_slab_of_wan14b_rows(fvlib, oracle):
    """7 200 token rows of the Wan-14B width (40 heads, 30 KB per row in, 30 KB out: past L2 in both directions),
    the case the profile of the default kernel is captured on: V bit-exact, q and k against the oracle on sampled
    tokens."""
    from fastvideo_rs_b200 import sdpa, wan
    batch, grid, heads = 1, (2, 45, 80), 40
    seq, dim = grid[0] * grid[1] * grid[2], heads * 128
    proj = oracle.bf16_round(oracle.seeded_normal(34, 0, (batch, seq, 3 * dim)))
    w = (1.0 + 0.1 * oracle.seeded_normal(34, 1, (dim,))).astype(np.float32)
    tc, ts = wan.wan_rope_tables(grid)
    tw = torch.from_numpy(w).cuda()
    q, k, v = wan.qk_prep(to_dev_bf16(proj), tw, tw, tc, ts, heads)
    assert sdpa.device_status() == 0
    assert "group_kernel" in sdpa._lib.last_kernel()
    tok = np.unique(np.concatenate([[0, 1, seq - 1], np.random.default_rng(5).integers(0, seq, 61)]))
    cos, sin = oracle.wan_rope(*grid)
    sub = np.ascontiguousarray(proj[:, tok])
    want_q = oracle.qk_norm_rope_bhsd(sub, w, cos[tok], sin[tok], batch, len(tok), heads, 128, 3 * dim, 0)
    want_k = oracle.qk_norm_rope_bhsd(sub, w, cos[tok], sin[tok], batch, len(tok), heads, 128, 3 * dim, dim)
    want_v = oracle.split_heads_bhsd(sub, batch, len(tok), heads, 128, 3 * dim, 2 * dim)
    tt = torch.from_numpy(tok).cuda()
    assert np.array_equal(to_host_f32(v[:, :, tt]).reshape(heads, len(tok), 128), want_v)
    for got, want in ((q, want_q), (k, want_k)):
        g = to_host_f32(got[:, :, tt]).reshape(heads, len(tok), 128)
        assert np.mean(g != oracle.bf16_round(want)) < 2e-3
        assert np.abs(g - want).max() <= np.abs(want).max() * 2.0 ** -8


def test_prep_writes_the_block_into_the_cache_tail(fvlib, oracle):
    """fv_wan_qk_prep_cache_bf16: K and V of a block land in rows [row0, row0 + seq) of the cache planes, bit for
    bit what the plain call plus two copies give (the append of wan/causal.rs:541-628); other rows untouched."""
    from fastvideo_rs_b200 import wan
    batch, heads, grid, cap, row0 = 2, 12, (1, 6, 13), 300, 150
    seq, dim = grid[0] * grid[1] * grid[2], heads * 128
    proj = to_dev_bf16(oracle.bf16_round(oracle.seeded_normal(35, 0, (batch, seq, 3 * dim))))
    w = torch.from_numpy((1.0 + 0.1 * oracle.seeded_normal(35, 1, (dim,))).astype(np.float32)).cuda()
    tc, ts = wan.wan_rope_tables(grid)
    q0, k0, v0 = wan.qk_prep(proj, w, w, tc, ts, heads)
    kc = torch.full((batch, heads, cap, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    vc = torch.full_like(kc, -3.0)
    q1, k1, v1 = wan.qk_prep(proj, w, w, tc, ts, heads, cache=(kc, vc, row0))
    assert torch.equal(q0, q1) and torch.equal(k0, k1) and torch.equal(v0, v1)
    assert torch.equal(kc[:, :, row0:row0 + seq], k0) and torch.equal(vc[:, :, row0:row0 + seq], v0)
    assert (kc[:, :, :row0] == 7.0).all() and (kc[:, :, row0 + seq:] == 7.0).all()
    assert (vc[:, :, :row0] == -3.0).all() and (vc[:, :, row0 + seq:] == -3.0).all()
    for kern in ("row",):
        import os
        os.environ["FV_PREP_KERNEL"] = kern
        try:
            kc2 = torch.zeros_like(kc)
            wan.qk_prep(proj, w, w, tc, ts, heads, cache=(kc2, torch.zeros_like(vc), cap - seq))
        finally:
            del os.environ["FV_PREP_KERNEL"]
        assert torch.equal(kc2[:, :, cap - seq:], k0)
    with pytest.raises(Exception):
        wan.qk_prep(proj, w, w, tc, ts, heads, cache=(kc, vc, cap - seq + 1))


def test_rope_bhsd_rebases_a_sink(fvlib, oracle):
    """fv_wan_rope_bhsd against the oracle's apply_rotary twin: f32 results bit for bit, bf16 results = RNE of
    those; and the rebased-sink sequence of wan/causal.rs:734-812 -- un-rope the cached sink keys with their own
    tables (sin negated) into an f32 buffer, rope that buffer at the target frames into the cache head."""
    from fastvideo_rs_b200 import wan
    b, h, cap, sink = 1, 3, 500, 2 * 78
    grid = (6, 6, 13)   # 78 tokens per frame
    cos, sin = oracle.wan_rope(*grid)
    own = slice(0, sink)             # the sink's own frames 0, 1
    new = slice(3 * 78, 3 * 78 + sink)  # target frames 3, 4
    x = oracle.bf16_round(oracle.seeded_normal(36, 0, (b * h, cap, 128)))
    kc = to_dev_bf16(x).view(b, h, cap, 128).clone()
    tco, tso = torch.from_numpy(cos[own].copy()).cuda(), torch.from_numpy(sin[own].copy()).cuda()
    tcn, tsn = torch.from_numpy(cos[new].copy()).cuda(), torch.from_numpy(sin[new].copy()).cuda()
    raw = torch.empty((b, h, sink, 128), dtype=torch.float32, device="cuda")
    wan.rope_bhsd(kc, tco, tso, raw, negate_sin=True)
    want_raw = oracle.rope_bhsd(x[:, :sink], cos[own], sin[own], negate_sin=True)
    assert np.array_equal(raw.cpu().numpy().reshape(b * h, sink, 128), want_raw)
    wan.rope_bhsd(raw, tcn, tsn, kc)
    want_head = oracle.bf16_round(oracle.rope_bhsd(want_raw, cos[new], sin[new]))
    got = to_host_f32(kc).reshape(b * h, cap, 128)
    assert np.array_equal(got[:, :sink], want_head)
    assert np.array_equal(got[:, sink:], x[:, sink:])
    # rows in the middle of both tensors, bf16 -> bf16 in place
    mid = kc.clone()
    wan.rope_bhsd(mid, tcn, tsn, mid, src_row0=200, dst_row0=200)
    want_mid = oracle.bf16_round(oracle.rope_bhsd(got[:, 200:200 + sink], cos[new], sin[new]))
    assert np.array_equal(to_host_f32(mid).reshape(b * h, cap, 128)[:, 200:200 + sink], want_mid)
    with pytest.raises(Exception):
        wan.rope_bhsd(kc, tcn, tsn, raw, src_row0=cap - sink + 1)
    # the same through the cache object: un-roped copy taken once, sink re-roped in place, second call a no-op
    cache = wan.CausalKvCache(wan.KvSpec(78, cap, sink, cap, True), b, h)
    cache.k.copy_(to_dev_bf16(x).view(b, h, cap, 128))
    cache.local_end = cap
    cache.rebase_sink(3, (tco, tso), (tcn, tsn))
    assert np.array_equal(to_host_f32(cache.k).reshape(b * h, cap, 128), got)
    before = cache.k.clone()
    cache.rebase_sink(3, (tco, tso), (tcn, tsn))
    assert torch.equal(cache.k, before) and cache.sink_at == 3


def test_kv_cache_update_keeps_prefix_and_window(fvlib):
    """update_keeps_prefix_and_window of the reference (wan/causal.rs:1113-1155) on the device cache: blocks of four
    tokens into a rolling cache of eight rows with a two-row sink; every row carries one value."""
    from fastvideo_rs_b200 import wan
    cache = wan.CausalKvCache(wan.KvSpec(2, 8, 2, 8, True), 1, 1)

    def blk(base):
        return (base + torch.arange(4, dtype=torch.float32, device="cuda")).view(1, 1, 4, 1).expand(1, 1, 4, 128).contiguous().bfloat16()

    def rows(t):
        assert (t == t[..., :1]).all()
        return t[0, 0, :, 0].float().tolist()

    k, _ = cache.update(blk(0.0), blk(0.0), 0)
    assert rows(k) == [0.0, 1.0, 2.0, 3.0]
    k, _ = cache.update(blk(10.0), blk(10.0), 0)       # the same block again (next step): overwritten
    assert rows(k) == [10.0, 11.0, 12.0, 13.0]
    k, _ = cache.update(blk(20.0), blk(20.0), 4)
    assert k.shape[2] == 8
    k, v = cache.update(blk(30.0), blk(30.0), 8)       # third block: 4 evicted after the 2-row sink
    assert rows(k) == [10.0, 11.0, 22.0, 23.0, 30.0, 31.0, 32.0, 33.0] and rows(v) == rows(k)
    assert len(cache) == 8
    k, _ = cache.update(blk(40.0), blk(40.0), 12)      # fourth block: the roll moves 2 rows down by 4
    assert rows(k) == [10.0, 11.0, 32.0, 33.0, 40.0, 41.0, 42.0, 43.0]
    cache.reset()
    assert len(cache) == 0


def test_kv_cache_roll_with_overlap_prep_and_window_attention(fvlib, oracle):
    """A roll whose source and destination overlap (more rows move than are evicted), blocks written by the prologue
    kernel, and the block's queries attending to the window in place -- against the oracle over the same rows."""
    from fastvideo_rs_b200 import sdpa, wan
    batch, heads, ft, n = 1, 3, 26, 52          # 2 frames of 26 tokens per block
    grid = (2, 2, 13)
    dim = heads * 128
    spec = wan.KvSpec.rolling_window(ft, 7, 1)  # 182 rows, sink 26: the third roll moves 104 rows down by 52
    cache = wan.CausalKvCache(spec, batch, heads)
    w = np.ones(dim, np.float32)
    tw = torch.from_numpy(w).cuda()
    host_k, host_v = [], []                     # the cache as the host would hold it: lists of [heads, rows, 128]
    for b in range(5):
        proj = oracle.bf16_round(oracle.seeded_normal(37, b, (batch, n, 3 * dim)))
        cos, sin = oracle.wan_rope(*grid, start_frame=2 * b)
        tc, ts = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
        q = cache.prep(to_dev_bf16(proj), tw, tw, tc, ts, b * n)
        out = cache.attend(q)
        assert sdpa.device_status() == 0
        kq = oracle.bf16_round(oracle.qk_norm_rope_bhsd(proj, w, cos, sin, batch, n, heads, 128, 3 * dim, 0))
        kk = oracle.bf16_round(oracle.qk_norm_rope_bhsd(proj, w, cos, sin, batch, n, heads, 128, 3 * dim, dim))
        vv = oracle.split_heads_bhsd(proj, batch, n, heads, 128, 3 * dim, 2 * dim)
        if sum(x.shape[1] for x in host_k) + n > spec.capacity:   # roll: the sink stays, the oldest rows after it go
            allk, allv = np.concatenate(host_k, 1), np.concatenate(host_v, 1)
            ev = allk.shape[1] + n - spec.capacity
            host_k = [np.concatenate([allk[:, :spec.sink], allk[:, spec.sink + ev:]], 1)]
            host_v = [np.concatenate([allv[:, :spec.sink], allv[:, spec.sink + ev:]], 1)]
        host_k.append(kk)
        host_v.append(vv)
        allk, allv = np.concatenate(host_k, 1), np.concatenate(host_v, 1)
        L = allk.shape[1]
        assert len(cache) == L
        got_k = to_host_f32(cache.k[0, :, :L])
        assert np.mean(got_k != allk) < 2e-3     # (one rounding of the prologue, ties aside)
        assert np.array_equal(to_host_f32(cache.v[0, :, :L]), allv)
        want = oracle.sdpa_rows(kq, to_host_f32(cache.k[0, :, :L]), allv)
        assert_close(to_host_f32(out).reshape(heads, n, 128), want, f"window attention, block {b}")
    merged = cache.attend(q, merged=True)
    assert torch.equal(merged, out.permute(0, 2, 1, 3).reshape(batch, n, dim))
