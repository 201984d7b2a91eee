"""Parity of the sm_100a attention kernel with the CPU oracle, through the C ABI (ctypes) on seeded
inputs.  Tolerance: bf16 outputs within max-abs 2e-2 and mean-abs 2e-3 of the fp32 oracle."""
import math
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from _util import assert_close, sample_rows, to_dev_bf16, to_host_f32

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def qkv(oracle, seed, bh, sq, sk):
    q = oracle.bf16_round(oracle.seeded_normal(seed, 0, (bh, sq, 128)))
    k = oracle.bf16_round(oracle.seeded_normal(seed, 1, (bh, sk, 128)))
    v = oracle.bf16_round(oracle.seeded_normal(seed, 2, (bh, sk, 128)))
    return q, k, v


# the reference's parity shapes (scripts/gpu/upstream/attn_dc_bench.cu:466-471;
# crates/fastvideo-gpucheck/src/kernels/attn2.rs:83-175) plus tile-edge lengths
SHAPES = [(1, 1, 1), (2, 64, 64), (2, 128, 128), (1, 129, 127), (2, 256, 256), (3, 192, 192), (2, 63, 4097), (2, 130, 1),
          (2, 300, 512), (2, 1000, 333), (4, 1024, 1024), (2, 257, 640), (2, 2048, 2048), (1, 65, 65)]


@pytest.mark.parametrize("bh,sq,sk", SHAPES)
def test_dense_matches_oracle(fvlib, oracle, bh, sq, sk):
    from fastvideo_rs_b200 import sdpa
    q, k, v = qkv(oracle, 100 + sq + sk, bh, sq, sk)
    out = sdpa.dense_fwd(to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v))
    assert sdpa.device_status() == 0
    want = oracle.sdpa_rows(q, k, v)
    assert_close(to_host_f32(out), want, f"dense {bh}x{sq}x{sk}")


def test_bf16_output_is_the_rounded_f32_output(fvlib, oracle):
    """crates/fastvideo-gpucheck/src/kernels/attn2.rs:611-694: bf16 out == RNE(f32 out)."""
    from fastvideo_rs_b200 import sdpa
    q, k, v = (to_dev_bf16(x) for x in qkv(oracle, 7, 3, 300, 700))
    o16 = sdpa.dense_fwd(q, k, v, out_bf16=True)
    o32 = sdpa.dense_fwd(q, k, v, out_bf16=False)
    assert torch.equal(o16, o32.to(torch.bfloat16))
    # and two runs give the same bits
    assert torch.equal(o16, sdpa.dense_fwd(q, k, v, out_bf16=True))


def test_scale_argument(fvlib, oracle):
    from fastvideo_rs_b200 import sdpa
    q, k, v = qkv(oracle, 8, 2, 200, 300)
    out = sdpa.dense_fwd(to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v), scale=0.05)
    assert_close(to_host_f32(out), oracle.sdpa_rows(q, k, v, scale=0.05), "scale 0.05")


CAUSAL = [(2, 600, 600, 100, 0, 0), (2, 600, 600, 100, 2, 1), (2, 1000, 1000, 130, 0, 0), (1, 24, 24, 5, 2, 1),
          (2, 2340, 2340, 780, 0, 0), (2, 54, 54, 6, 0, 0), (2, 54, 54, 18, 1, 0), (1, 700, 700, 256, 3, 0),
          (1, 700, 700, 1, 0, 0), (1, 520, 520, 128, 0, 2)]


@pytest.mark.parametrize("bh,sq,sk,bt,win,sink", CAUSAL)
def test_block_causal_matches_masked_oracle(fvlib, oracle, bh, sq, sk, bt, win, sink):
    """crates/fastvideo-gpucheck/src/kernels_wan.rs:89-364: the causal kernel against the masked
    composed SDPA, including windows, sinks and blocks that do not divide the key tile."""
    from fastvideo_rs_b200 import sdpa
    q, k, v = qkv(oracle, 300 + bt + win, bh, sq, sk)
    out = sdpa.dense_fwd(to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v), causal=sdpa.BlockCausal(bt, win, sink))
    assert sdpa.device_status() == 0
    want = oracle.sdpa_rows(q, k, v, block_causal=(bt, win, sink))
    assert_close(to_host_f32(out), want, f"causal bt{bt} w{win} s{sink}")


def test_one_block_mask_is_dense(fvlib, oracle):
    """kernels_wan.rs: a mask whose single block covers everything == the dense kernel, bit for bit."""
    from fastvideo_rs_b200 import sdpa
    q, k, v = (to_dev_bf16(x) for x in qkv(oracle, 9, 2, 500, 500))
    a = sdpa.dense_fwd(q, k, v)
    b = sdpa.dense_fwd(q, k, v, causal=sdpa.BlockCausal(500, 0, 0))
    assert torch.equal(a, b)


def test_entry_plans(fvlib, oracle):
    """rt/sdpa.rs:508-575 on the device: each Plan the Wan caller builds runs and equals the oracle; plans
    that belong to other kernels decline instead of falling back."""
    from fastvideo_rs_b200 import Declined, sdpa
    b, h, sq, sk = 2, 3, 260, 390
    q, k, v = qkv(oracle, 11, b * h, sq, sk)
    tq, tk, tv = (to_dev_bf16(x).view(b, h, -1, 128) for x in (q, k, v))
    want = oracle.sdpa_rows(q, k, v)
    assert_close(to_host_f32(sdpa.sdpa(tq, tk, tv, sdpa.Plan.dense(None))).reshape(b * h, sq, 128), want, "Plan.dense")
    assert_close(to_host_f32(sdpa.sdpa(tq, tk, tv, sdpa.Plan.kv_window())).reshape(b * h, sq, 128), want, "Plan.kv_window")
    want5 = oracle.sdpa_rows(q, k, v, scale=0.5)
    assert_close(to_host_f32(sdpa.sdpa(tq, tk, tv, sdpa.Plan.dense(0.5))).reshape(b * h, sq, 128), want5, "scale 0.5")
    bc = sdpa.BlockCausal(65, 0, 0)
    wantc = oracle.sdpa_rows(q, k, v, block_causal=(65, 0, 0))
    assert_close(to_host_f32(sdpa.sdpa(tq, tk, tv, sdpa.Plan.block_causal(None, bc))).reshape(b * h, sq, 128), wantc,
                 "Plan.block_causal")
    with pytest.raises(Declined):
        sdpa.sdpa(tq, tk, tv, sdpa.Plan.composed(None, None))
    with pytest.raises(Declined):
        sdpa.sdpa(tq, tk, tv, sdpa.Plan.masked(None, torch.zeros(sq, sk, device="cuda")))
    with pytest.raises(ValueError, match="BHSD"):
        sdpa.sdpa(tq[0], tk[0], tv[0], sdpa.Plan.dense(None))


def test_golden_tiny_wan_through_prep_and_attention(fvlib, oracle):
    """Config 0 end to end against the committed fixture: projection -> RMSNorm (across heads) + RoPE ->
    dense attention."""
    import sys
    sys.path.insert(0, str(ROOT / "tests" / "golden"))
    import make_golden as M
    from fastvideo_rs_b200 import wan
    for name in ("wan_dense_tiny", "wan_causal_small"):
        g = np.load(ROOT / "tests" / "golden" / f"{name}.npz")
        grid, heads = tuple(int(x) for x in g["grid"]), int(g["heads"])
        proj, w, seq, dim = M.wan_inputs(int(g["seed"]), 1, grid, heads)
        causal = tuple(int(x) for x in g["causal"])
        from fastvideo_rs_b200.sdpa import BlockCausal
        attn = wan.WanSelfAttention(grid, heads, torch.from_numpy(w).cuda(), torch.from_numpy(w).cuda(),
                                    causal=BlockCausal(*causal) if causal[0] else None)
        out = attn.forward_self(to_dev_bf16(proj))
        got = to_host_f32(out).reshape(heads, seq, 128)[:, g["rows"]]
        assert_close(got, g["out"], name)


def test_full_size_rows_wan_1p3b(fvlib, oracle):
    """Config 1's self-attention shape (32 760 tokens) on 2 heads, sampled rows against the oracle, plus
    size-independent properties at full size: rows are convex combinations of V (bounded by V's range),
    and a constant V gives that constant."""
    from fastvideo_rs_b200 import sdpa
    bh, s = 2, 32760
    q, k, v = qkv(oracle, 21, bh, s, s)
    tq, tk, tv = to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v)
    out = sdpa.dense_fwd(tq, tk, tv)
    assert sdpa.device_status() == 0
    rows = sample_rows(s, 40, 3)
    want = oracle.sdpa_rows(q, k, v, rows=rows)
    assert_close(to_host_f32(out[:, torch.from_numpy(rows).long().cuda()]), want, "32760 rows")
    assert float(out.float().abs().max()) <= float(tv.float().abs().max())
    ones = torch.full_like(tv, 0.5)
    const = sdpa.dense_fwd(tq, tk, ones)
    assert torch.equal(const, ones)


def test_full_size_rows_wan_14b(fvlib, oracle):
    """Config 3's shape (75 600 tokens: 295 work items of 256 rows + one of 80, 590 key tiles + one of 80 keys)
    on 2 heads: sampled rows (item and tile edges, the tail) against the oracle over all keys; constant V."""
    from fastvideo_rs_b200 import sdpa
    bh, s = 2, 75600
    q, k, v = qkv(oracle, 23, bh, s, s)
    tq, tk, tv = to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v)
    out = sdpa.dense_fwd(tq, tk, tv)
    assert sdpa.device_status() == 0
    rows = np.unique(np.concatenate([sample_rows(s, 24, 4), [75519, 75520, 75521, 75599, 37799, 37888]])).astype(np.int32)
    want = oracle.sdpa_rows(q, k, v, rows=rows)
    assert_close(to_host_f32(out[:, torch.from_numpy(rows).long().cuda()]), want, "75600 rows")
    ones = torch.full_like(tv, -0.25)
    assert torch.equal(sdpa.dense_fwd(tq, tk, ones), ones)


def test_full_size_chunk_causal_self_forcing(fvlib, oracle):
    """Config 4's real shape: 32 760 tokens in 7 chunks of 4 680 (block-lower-triangular), 2 heads; rows at the
    start, end and both sides of every chunk border against the masked oracle.  4 680 is not a multiple of the
    128-key tile: every chunk border cuts through a key tile and through a work item."""
    from fastvideo_rs_b200 import sdpa
    bh, s, bt = 2, 32760, 4680
    q, k, v = qkv(oracle, 24, bh, s, s)
    out = sdpa.dense_fwd(to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v), causal=sdpa.BlockCausal(bt, 0, 0))
    assert sdpa.device_status() == 0
    edges = [c * bt + d for c in range(1, 7) for d in (-129, -1, 0, 1, 127)]
    rows = np.unique(np.concatenate([sample_rows(s, 16, 6), edges])).astype(np.int32)
    want = oracle.sdpa_rows(q, k, v, rows=rows, block_causal=(bt, 0, 0))
    assert_close(to_host_f32(out[:, torch.from_numpy(rows).long().cuda()]), want, "chunk-causal 32760")
    # a row of chunk 0 sees chunk 0 only: equal to dense attention over the first 4 680 keys
    first = sdpa.dense_fwd(to_dev_bf16(q[:, :bt]), to_dev_bf16(k[:, :bt]), to_dev_bf16(v[:, :bt]))
    assert float((out[:, :bt].float() - first.float()).abs().max()) <= 2e-2


def test_cross_attention_shape(fvlib, oracle):
    """Config 1's cross-attention: 32 760 queries over 512 text keys."""
    from fastvideo_rs_b200 import sdpa
    q, k, v = qkv(oracle, 22, 2, 32760, 512)
    out = sdpa.dense_fwd(to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v))
    rows = sample_rows(32760, 64, 5)
    assert_close(to_host_f32(out)[:, rows], oracle.sdpa_rows(q, k, v, rows=rows), "cross 32760x512")


def test_two_pass_segments_equal_one_pass(fvlib, oracle):
    """The sequence-parallel evaluation on one GPU: keys split into 3 uneven segments, pass 1 over the
    middle one, pass 2 over the others merging pass 1 -- equals the oracle over all keys, and the
    log-sum-exp it returns is the oracle's."""
    from fastvideo_rs_b200 import sp
    bh, sq, sk = 2, 333, 1000
    q, k, v = qkv(oracle, 23, bh, sq, sk)
    ranges = oracle.shard_ranges(sk, 3)  # (0,334) (334,333) (667,333)
    rows = max(l for _, l in ranges)
    k_all = np.zeros((3, bh, rows, 128), np.float32)
    v_all = np.zeros_like(k_all)
    for r, (s0, l) in enumerate(ranges):
        k_all[r, :, :l] = k[:, s0 : s0 + l]
        v_all[r, :, :l] = v[:, s0 : s0 + l]
    tq, tk, tv = to_dev_bf16(q), to_dev_bf16(k_all), to_dev_bf16(v_all)
    scale = 1.0 / math.sqrt(128)
    o1 = torch.empty((bh, sq, 128), dtype=torch.float32, device="cuda")
    lse1 = torch.empty((bh, sq), dtype=torch.float32, device="cuda")
    mid = ranges[1]
    sp.segments_fwd(tq, tk[1].contiguous(), tv[1].contiguous(), [mid[1]], [mid[0]], rows, scale, out=o1, lse_out=lse1)
    lens = [ranges[0][1], 0, ranges[2][1]]
    starts = [r[0] for r in ranges]
    lse = torch.empty_like(lse1)
    out = sp.segments_fwd(tq, tk, tv, lens, starts, rows, scale, prev_o=o1, prev_lse=lse1, lse_out=lse)
    assert_close(to_host_f32(out), oracle.sdpa_rows(q, k, v), "two-pass")
    # pass 1 alone is attention over the middle segment
    assert_close(to_host_f32(o1), oracle.sdpa_rows(q, k[:, mid[0] : mid[0] + mid[1]], v[:, mid[0] : mid[0] + mid[1]]),
                 "pass 1", 2e-3, 2e-4)
    s = (q.astype(np.float64) @ k.astype(np.float64).transpose(0, 2, 1)) * scale
    want_lse = (np.log(np.exp(s - s.max(-1, keepdims=True)).sum(-1)) + s.max(-1)) / math.log(2.0)
    assert np.abs(to_host_f32(lse) - want_lse).max() < 2e-2


@pytest.mark.parametrize("world,bt,win,sink", [(2, 100, 0, 0), (3, 130, 0, 0), (4, 64, 2, 1), (3, 1000, 0, 0), (4, 37, 3, 0)])
def test_sequence_parallel_block_causal_rank_by_rank(fvlib, oracle, world, bt, win, sink):
    """What each rank of SpAttention.forward(causal=...) launches, run rank after rank on one GPU: pass 1 over the
    rank's own keys, pass 2 over the shards SpLayout says it needs, both under the mask with global row and key
    indices.  The shards put together equal the one-launch masked kernel and the masked oracle."""
    from fastvideo_rs_b200 import sdpa, sp
    bh, seq = 2, 1001  # uneven shards: the gathered buffer is padded
    q, k, v = qkv(oracle, 77 + world, bh, seq, seq)
    tq, tk, tv = to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v)
    causal = sdpa.BlockCausal(bt, win, sink)
    scale = 1.0 / math.sqrt(128)
    layouts = [sp.SpLayout(seq, world, r) for r in range(world)]
    rows = layouts[0].seg_rows
    k_all = torch.zeros((world, bh, rows, 128), dtype=torch.bfloat16, device="cuda")
    v_all = torch.zeros_like(k_all)
    for r, lay in enumerate(layouts):
        k_all[r, :, : lay.len] = tk[:, lay.start : lay.start + lay.len]
        v_all[r, :, : lay.len] = tv[:, lay.start : lay.start + lay.len]
    parts = []
    for r, lay in enumerate(layouts):
        qr = tq[:, lay.start : lay.start + lay.len].contiguous()
        l1, s1 = lay.pass1()
        l2, s2 = lay.pass2_for(causal)
        # a rank holds nothing of the shards it does not need: poison them
        ka, va = k_all.clone(), v_all.clone()
        for o in range(world):
            if o != r and o not in lay.needed_ranks(causal):
                ka[o].fill_(float("nan"))
                va[o].fill_(float("nan"))
        if not any(l2):
            parts.append(sp.segments_fwd(qr, k_all[r].contiguous(), v_all[r].contiguous(), l1, s1, rows, scale, causal=causal,
                                         q_row0=lay.start))
            continue
        o1 = torch.empty((bh, lay.len, 128), dtype=torch.float32, device="cuda")
        lse1 = torch.empty((bh, lay.len), dtype=torch.float32, device="cuda")
        sp.segments_fwd(qr, k_all[r].contiguous(), v_all[r].contiguous(), l1, s1, rows, scale, out=o1, lse_out=lse1,
                        causal=causal, q_row0=lay.start)
        parts.append(sp.segments_fwd(qr, ka, va, l2, s2, rows, scale, prev_o=o1, prev_lse=lse1, causal=causal,
                                     q_row0=lay.start))
    assert sdpa.device_status() == 0
    got = torch.cat(parts, dim=1)
    assert torch.isfinite(got.float()).all()
    one = sdpa.dense_fwd(tq, tk, tv, causal=causal)
    assert float((got.float() - one.float()).abs().max()) <= 2e-2
    assert_close(to_host_f32(got), oracle.sdpa_rows(q, k, v, block_causal=(bt, win, sink)), f"sp{world} causal bt{bt} w{win} s{sink}")


@pytest.mark.parametrize("grouped", [True, False])
@pytest.mark.parametrize("world,zigzag,mask", [(2, False, None), (4, False, None), (4, True, (130, 0, 0)), (3, True, (64, 2, 1)),
                                               (8, True, (100, 0, 0)), (4, True, None), (8, False, None)])
def test_sequence_parallel_chained_passes_rank_by_rank(fvlib, oracle, world, zigzag, mask, grouped):
    """The launches of SpAttention.forward with the copy-engine exchange, run rank after rank on one GPU: pass 1
    over the rank's own runs, then the passes of SpLayout.source_groups (one, two, four ... sources per pass, or one
    source each), each continuing the previous pass' f32 state -- contiguous shards and the zig-zag split (two runs of query rows per rank), dense
    and block-causal.  Runs a rank does not fetch are poisoned with NaN.  Put back in sequence order the rows
    equal the one-launch kernel and the oracle."""
    from fastvideo_rs_b200 import sdpa, sp
    bh, seq = 2, 1001
    q, k, v = qkv(oracle, 91 + world, bh, seq, seq)
    tq, tk, tv = to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v)
    causal = sdpa.BlockCausal(*mask) if mask else None
    scale = 1.0 / math.sqrt(128)
    layouts = [sp.SpLayout(seq, world, r, zigzag=zigzag) for r in range(world)]
    L0 = layouts[0]

    def block(t, lay):  # a rank's [runs, bh, run_rows, 128] block
        b = torch.zeros((lay.nrun, bh, lay.run_rows, 128), dtype=torch.bfloat16, device="cuda")
        for r, (s0, l) in enumerate(lay.runs[lay.rank]):
            b[r, :, :l] = t[:, s0:s0 + l]
        return b

    kb = [block(tk, lay) for lay in layouts]
    vb = [block(tv, lay) for lay in layouts]
    got = torch.zeros((bh, seq, 128), dtype=torch.bfloat16, device="cuda")
    for lay in layouts:
        rows = torch.tensor(lay.rows(), device="cuda", dtype=torch.long)
        if rows.numel() == 0:
            continue
        qr = tq[:, rows].contiguous()
        q_row0, q_split, q_row1 = lay.q_runs()
        common = dict(causal=causal, q_row0=q_row0, q_split=q_split, q_row1=q_row1)
        l1, s1 = lay.pass1()
        order = lay.source_order(causal)
        if not order:
            o = sp.segments_fwd(qr, kb[lay.rank], vb[lay.rank], l1, s1, lay.run_rows, scale, **common)
        else:
            ob = [torch.empty((bh, lay.len, 128), dtype=torch.float32, device="cuda") for _ in range(2)]
            lb = [torch.empty((bh, lay.len), dtype=torch.float32, device="cuda") for _ in range(2)]
            sp.segments_fwd(qr, kb[lay.rank], vb[lay.rank], l1, s1, lay.run_rows, scale, out=ob[0], lse_out=lb[0], **common)
            o = None
            groups = lay.source_groups(causal, grouped)
            assert [s for g in groups for s in g] == order
            for n, srcs in enumerate(groups):
                if len(srcs) == 1:
                    ln, st = lay.source_segments(srcs[0], causal)
                    ks, vs = kb[srcs[0]].clone(), vb[srcs[0]].clone()
                else:  # several sources in one pass: segments over the whole gathered buffer
                    ln, st = lay.group_segments(srcs, causal)
                    ks, vs = torch.cat(kb).clone(), torch.cat(vb).clone()
                for run, l in enumerate(ln):
                    if l == 0:  # not fetched, or not this pass'
                        ks[run].fill_(float("nan"))
                        vs[run].fill_(float("nan"))
                last = n == len(groups) - 1
                a, b = n & 1, 1 - (n & 1)
                o = sp.segments_fwd(qr, ks, vs, ln, st, lay.run_rows, scale, out=None if last else ob[b],
                                    lse_out=None if last else lb[b], prev_o=ob[a], prev_lse=lb[a], **common)
        got[:, rows] = o
    assert sdpa.device_status() == 0
    assert torch.isfinite(got.float()).all()
    one = sdpa.dense_fwd(tq, tk, tv, causal=causal)
    assert float((got.float() - one.float()).abs().max()) <= 2e-2
    assert_close(to_host_f32(got), oracle.sdpa_rows(q, k, v, block_causal=mask), f"sp{world} zigzag={zigzag} mask={mask}")
    assert L0.nrun == (2 if zigzag else 1)


def test_merged_heads_output_is_the_permuted_bhsd_output(fvlib, oracle):
    """merge_heads folded into the store (rt/ops.rs:2373-2385): same bits as the BHSD call, [b, s, h*d] order."""
    from fastvideo_rs_b200 import sdpa
    b, h, sq, sk = 2, 3, 300, 421
    q, k, v = qkv(oracle, 25, b * h, sq, sk)
    tq, tk, tv = (to_dev_bf16(x).view(b, h, -1, 128) for x in (q, k, v))
    for bf16 in (True, False):
        want = sdpa.dense_fwd(tq.view(b * h, sq, 128), tk.view(b * h, sk, 128), tv.view(b * h, sk, 128), out_bf16=bf16)
        got = sdpa.dense_fwd_merged(tq, tk, tv, out_bf16=bf16)
        assert got.shape == (b, sq, h * 128)
        assert torch.equal(got, want.view(b, h, sq, 128).permute(0, 2, 1, 3).reshape(b, sq, h * 128))
    bc = sdpa.BlockCausal(64, 0, 0)
    want = sdpa.dense_fwd(tq.view(b * h, sq, 128), tk.view(b * h, sk, 128), tv.view(b * h, sk, 128), causal=bc)
    got = sdpa.dense_fwd_merged(tq, tk, tv, causal=bc)
    assert torch.equal(got, want.view(b, h, sq, 128).permute(0, 2, 1, 3).reshape(b, sq, h * 128))


def test_relative_l2_error_is_inside_the_reference_kernel_bounds(fvlib, oracle):
    """crates/fastvideo-gpucheck/src/kernels/attn2.rs:83-175,611-694: rel-L2 against the f32 reference <= 1e-2."""
    from fastvideo_rs_b200 import sdpa
    for bh, sq, sk in ((2, 2048, 2048), (2, 300, 512), (1, 63, 4097)):
        q, k, v = qkv(oracle, 26 + sq, bh, sq, sk)
        got = to_host_f32(sdpa.dense_fwd(to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v), out_bf16=False)).astype(np.float64)
        want = oracle.sdpa_rows_f64(q, k, v)
        rel = np.sqrt(((got - want) ** 2).sum() / (want ** 2).sum())
        assert rel <= 1e-2, rel


def test_invalid_arguments_are_errors_not_launches(fvlib, oracle):
    from fastvideo_rs_b200 import FvError, sdpa
    q, k, v = (to_dev_bf16(x) for x in qkv(oracle, 24, 1, 64, 64))
    with pytest.raises(FvError):
        sdpa.dense_fwd(q, k, v, scale=-1.0)
    with pytest.raises(ValueError):
        sdpa.dense_fwd(q.float(), k, v)
    with pytest.raises(ValueError):
        sdpa.dense_fwd(q.cpu(), k.cpu(), v.cpu())


def test_native_checker_passes(fvlib):
    """The torch-free bring-up binary agrees (its own f64 host evaluation, NaN-poisoned outputs)."""
    from fastvideo_rs_b200 import _build
    exe = _build.build_native_checker()
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:]


def test_spare_sms_hint_shrinks_one_launch_and_changes_no_bit(fvlib, oracle):
    """fv_hint_spare_sms: the next launch of the calling thread leaves SMs free (for a collective's copy kernels beside
    it), the one after that uses every SM again; the work deal changes, the results do not."""
    from fastvideo_rs_b200 import sdpa, _lib
    q, k, v = qkv(oracle, 97, 24, 4096, 2048)
    tq, tk, tv = to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v)
    full = sdpa.dense_fwd(tq, tk, tv)
    line_full = _lib.last_kernel()
    assert fvlib.fv_hint_spare_sms(24) == 0
    fewer = sdpa.dense_fwd(tq, tk, tv)
    line_fewer = _lib.last_kernel()
    again = sdpa.dense_fwd(tq, tk, tv)
    assert sdpa.device_status() == 0
    import re
    n_full, n_fewer, n_again = (int(re.search(r"(\d+) CTAs", s).group(1)) for s in (line_full, line_fewer, _lib.last_kernel()))
    assert n_fewer == n_full - 24 and n_again == n_full
    assert torch.equal(full, fewer) and torch.equal(full, again)
    assert fvlib.fv_hint_spare_sms(-1) != 0 and fvlib.fv_hint_spare_sms(1000) != 0
