"""The Wan callers around the kernels (WanAttention::{forward_self, attend_vsa, cross_kv, forward_cross},
crates/fastvideo-cudarc/src/wan/transformer.rs:163-445) against the oracle's host math on seeded projections."""
import numpy as np
import pytest
import torch

from _util import assert_close, sample_rows, to_dev_bf16, to_host_f32

pytestmark = pytest.mark.gpu


def test_forward_cross_and_cross_kv(fvlib, oracle):
    from fastvideo_rs_b200 import wan
    batch, heads, grid, text = 2, 12, (3, 10, 13), 77
    seq, dim = grid[0] * grid[1] * grid[2], heads * 128
    q_proj = oracle.bf16_round(oracle.seeded_normal(71, 0, (batch, seq, dim)))
    kv_proj = oracle.bf16_round(oracle.seeded_normal(71, 1, (batch, text, 2 * dim)))
    wq = (1.0 + 0.1 * oracle.seeded_normal(71, 2, (dim,))).astype(np.float32)
    wk = (1.0 + 0.1 * oracle.seeded_normal(71, 3, (dim,))).astype(np.float32)
    attn = wan.WanSelfAttention(grid, heads, torch.from_numpy(wq).cuda(), torch.from_numpy(wk).cuda())
    k, v = attn.cross_kv(to_dev_bf16(kv_proj))
    assert k.shape == (batch, heads, text, 128) and v.shape == k.shape
    want_k = oracle.bf16_round(oracle.qk_norm_rope_bhsd(kv_proj, wk, None, None, batch, text, heads, 128, 2 * dim, 0))
    want_v = oracle.split_heads_bhsd(kv_proj, batch, text, heads, 128, 2 * dim, dim)
    assert np.array_equal(to_host_f32(v).reshape(-1, text, 128), want_v)
    assert np.mean(to_host_f32(k).reshape(-1, text, 128) != want_k) < 2e-3  # one rounding, ties aside
    out = attn.forward_cross(to_dev_bf16(q_proj), (k, v))
    want_q = oracle.bf16_round(oracle.qk_norm_rope_bhsd(q_proj, wq, None, None, batch, seq, heads, 128, dim, 0))
    want = oracle.sdpa_rows(want_q, want_k, want_v)
    assert_close(to_host_f32(out).reshape(-1, seq, 128), want, "forward_cross")
    merged = attn.forward_cross(to_dev_bf16(q_proj), (k, v), merged=True)
    assert torch.equal(merged, out.permute(0, 2, 1, 3).reshape(batch, seq, dim))


def test_forward_self_merged_and_causal(fvlib, oracle):
    from fastvideo_rs_b200 import sdpa, wan
    batch, heads, grid = 1, 12, (4, 6, 7)
    seq, dim = grid[0] * grid[1] * grid[2], heads * 128
    qkv = oracle.bf16_round(oracle.seeded_normal(72, 0, (batch, seq, 3 * dim)))
    w = np.ones(dim, np.float32)
    causal = sdpa.BlockCausal(2 * grid[1] * grid[2], 0, 0)
    attn = wan.WanSelfAttention(grid, heads, torch.from_numpy(w).cuda(), torch.from_numpy(w).cuda(), causal=causal)
    out = attn.forward_self(to_dev_bf16(qkv))
    cos, sin = oracle.wan_rope(*grid)
    q = oracle.bf16_round(oracle.qk_norm_rope_bhsd(qkv, w, cos, sin, batch, seq, heads, 128, 3 * dim, 0))
    k = oracle.bf16_round(oracle.qk_norm_rope_bhsd(qkv, w, cos, sin, batch, seq, heads, 128, 3 * dim, dim))
    v = oracle.split_heads_bhsd(qkv, batch, seq, heads, 128, 3 * dim, 2 * dim)
    want = oracle.sdpa_rows(q, k, v, block_causal=(causal.block_tokens, 0, 0))
    assert_close(to_host_f32(out).reshape(-1, seq, 128), want, "forward_self causal")
    merged = attn.forward_self(to_dev_bf16(qkv), merged=True)
    assert torch.equal(merged, out.permute(0, 2, 1, 3).reshape(batch, seq, dim))


def test_attend_vsa_takes_the_gate_projection(fvlib, oracle):
    """forward_self on the VSA route: the gate is the gate projection split into heads, nothing else
    (wan/transformer.rs:336-347); the result equals the VSA operator called by hand and, against the oracle's
    vsa_attention_host on a small grid, stays within the stated tolerance."""
    from fastvideo_rs_b200 import vsa, wan
    batch, heads, grid = 1, 2, (5, 6, 9)
    seq, dim = grid[0] * grid[1] * grid[2], heads * 128
    qkv = oracle.bf16_round(oracle.seeded_normal(73, 0, (batch, seq, 3 * dim)))
    gate = oracle.bf16_round(0.5 * oracle.seeded_normal(73, 1, (batch, seq, dim)))
    w = np.ones(dim, np.float32)
    ctx = vsa.VsaCtx(grid, sparsity=0.5)
    attn = wan.WanSelfAttention(grid, heads, torch.from_numpy(w).cuda(), torch.from_numpy(w).cuda(), vsa=ctx)
    out = attn.forward_self(to_dev_bf16(qkv), gate=to_dev_bf16(gate))
    cos, sin = oracle.wan_rope(*grid)
    q = oracle.bf16_round(oracle.qk_norm_rope_bhsd(qkv, w, cos, sin, batch, seq, heads, 128, 3 * dim, 0))
    k = oracle.bf16_round(oracle.qk_norm_rope_bhsd(qkv, w, cos, sin, batch, seq, heads, 128, 3 * dim, dim))
    v = oracle.split_heads_bhsd(qkv, batch, seq, heads, 128, 3 * dim, 2 * dim)
    g = oracle.split_heads_bhsd(gate, batch, seq, heads, 128, dim, 0)
    want = oracle.vsa_attention_host(q, k, v, g, grid, ctx.topk)
    assert_close(to_host_f32(out).reshape(-1, seq, 128), want, "attend_vsa")
    with pytest.raises(ValueError):
        attn.forward_self(to_dev_bf16(qkv))


def test_f32_operands_are_rounded_like_act16(fvlib, oracle):
    """act16_operands and the tail of dense (rt/sdpa.rs:167-181,206-213): float32 operands are rounded to bf16
    (RNE, bit-exact against the oracle's rounding, ragged tail included), attention runs on those, and the
    float32 result holds bf16-representable values equal to the bf16 call's."""
    from fastvideo_rs_b200 import sdpa
    b, h, sq, sk = 1, 3, 333, 517   # 3 * 333 * 128 and 3 * 517 * 128 are multiples of 8; the tail case is below
    q = oracle.seeded_normal(74, 0, (b, h, sq, 128))
    k = oracle.seeded_normal(74, 1, (b, h, sk, 128))
    v = oracle.seeded_normal(74, 2, (b, h, sk, 128))
    tq, tk, tv = (torch.from_numpy(x).cuda() for x in (q, k, v))
    q16, k16, v16 = sdpa.act16_operands(tq, tk, tv)
    for got, src in ((q16, q), (k16, k), (v16, v)):
        assert np.array_equal(to_host_f32(got), oracle.bf16_round(src))
    out32 = sdpa.sdpa(tq, tk, tv, sdpa.Plan.dense(None))
    assert out32.dtype == torch.float32
    out16 = sdpa.sdpa(q16, k16, v16, sdpa.Plan.dense(None))
    assert torch.equal(out32, out16.float())
    want = oracle.sdpa_rows(oracle.bf16_round(q).reshape(-1, sq, 128), oracle.bf16_round(k).reshape(-1, sk, 128),
                            oracle.bf16_round(v).reshape(-1, sk, 128))
    assert_close(out32.cpu().numpy().reshape(-1, sq, 128), want, "f32 entrance")
    # ragged tail: 13 values
    a = torch.from_numpy(oracle.seeded_normal(75, 0, (13,))).cuda()
    r, _, _ = sdpa.act16_operands(a, a.clone(), a.clone())
    assert np.array_equal(to_host_f32(r), oracle.bf16_round(a.cpu().numpy()))
    assert torch.equal(sdpa.act16_widen(r), r.float())
    with pytest.raises(ValueError):
        sdpa.sdpa(tq, k16, v16, sdpa.Plan.dense(None))
