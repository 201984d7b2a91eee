"""The sequence-parallel path's host logic on CPU ranks (gloo, world size 2 and 3): shard ranges, the
padded all-gather layout, the two passes' segment tables and the log-sum-exp merge.  The attention of
each pass is evaluated by a numpy stand-in that follows the kernel's segment contract
(include/fv_sdpa.h, fv_sdpa_segments_bf16), so what is checked is everything around the kernel."""
import math
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def segments_attention_np(q, k_all, v_all, seg_len, seg_start, scale, prev=None):
    """Softmax attention of q [bh, sq, d] over the listed segments of k_all / v_all [nseg, bh, rows, d];
    returns (normalised out f32, lse in the base-2 domain).  prev = (out, lse) of another key set merges."""
    bh, sq, d = q.shape
    ks, vs = [], []
    for s, n in enumerate(seg_len):
        ks.append(k_all[s, :, :n])
        vs.append(v_all[s, :, :n])
    k, v = np.concatenate(ks, axis=1).astype(np.float64), np.concatenate(vs, axis=1).astype(np.float64)
    sc = (q.astype(np.float64) @ k.transpose(0, 2, 1)) * scale * math.log2(math.e)
    m = sc.max(-1, keepdims=True)
    p = np.exp2(sc - m)
    l = p.sum(-1, keepdims=True)
    out, lse = (p @ v) / l, (m + np.log2(l))[..., 0]
    if prev is not None:
        po, pl = prev
        M = np.maximum(lse, pl)
        wn, wp = np.exp2(lse - M), np.exp2(pl - M)
        out = (out * wn[..., None] + po * wp[..., None]) / (wn + wp)[..., None]
        lse = M + np.log2(wn + wp)
    return out, lse


def worker(rank, world, seq, port, q_out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fastvideo_rs_b200 import sp
        from oracle import oracle as O
        bh, d = 2, 16
        q, k, v = (O.bf16_round(O.seeded_normal(5, i, (bh, seq, d))) for i in range(3))
        lay = sp.SpLayout(seq, world, rank)
        assert lay.ranges == O.shard_ranges(seq, world)
        ql = sp.shard_tensor(torch.from_numpy(q), 1, rank, world).numpy()
        kl = sp.shard_tensor(torch.from_numpy(k), 1, rank, world).numpy()
        vl = sp.shard_tensor(torch.from_numpy(v), 1, rank, world).numpy()
        assert ql.shape[1] == lay.len
        # the exchange: zero-padded shards gathered rank-major, exactly the layout the kernel indexes
        pad = lambda x: np.concatenate([x, np.zeros((bh, lay.seg_rows - x.shape[1], d), np.float32)], axis=1)
        k_all = torch.zeros((world, bh, lay.seg_rows, d))
        v_all = torch.zeros((world, bh, lay.seg_rows, d))
        dist.all_gather_into_tensor(k_all.view(world * bh, lay.seg_rows, d), torch.from_numpy(pad(kl)))
        dist.all_gather_into_tensor(v_all.view(world * bh, lay.seg_rows, d), torch.from_numpy(pad(vl)))
        scale = 1.0 / math.sqrt(d)
        l1, s1 = lay.pass1()
        assert l1 == [lay.len] and s1 == [lay.start]
        o1 = segments_attention_np(ql, pad(kl)[None], pad(vl)[None], l1, s1, scale)
        l2, s2 = lay.pass2()
        assert l2[rank] == 0 and sum(l2) == seq - lay.len and s2 == [s for s, _ in lay.ranges]
        keep = [r for r in range(world) if l2[r] > 0]
        out, _ = segments_attention_np(ql, k_all.numpy()[keep], v_all.numpy()[keep], [l2[r] for r in keep],
                                       [s2[r] for r in keep], scale, prev=o1)
        rows = np.arange(lay.start, lay.start + lay.len, dtype=np.int32)
        want = O.sdpa_rows(q, k, v, scale=scale, rows=rows)
        err = float(np.abs(out - want).max())
        # outputs stay sharded; gathering them reproduces the full result (sp::all_gather_seq)
        outs = [torch.zeros((bh, lay.seg_rows, d), dtype=torch.float64) for _ in range(world)]
        mine = torch.zeros((bh, lay.seg_rows, d), dtype=torch.float64)
        mine[:, : lay.len] = torch.from_numpy(out)
        dist.all_gather(outs, mine)
        full = sp.all_gather_seq([o[:, :l] for o, (_, l) in zip(outs, lay.ranges)], 1).numpy()
        err_full = float(np.abs(full - O.sdpa_rows(q, k, v, scale=scale)).max())
        q_out.put((rank, err, err_full))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,seq", [(2, 11), (2, 64), (3, 100)])
def test_two_pass_sp_on_gloo_ranks(fvlib, oracle, world, seq):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + world * 7 + seq) % 2000
    procs = [ctx.Process(target=worker, args=(r, world, seq, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=90) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r for r, _, _ in res) == list(range(world))
    for r, err, err_full in res:
        assert err < 1e-5 and err_full < 1e-5, (r, err, err_full)


def test_layout_tables(fvlib):
    from fastvideo_rs_b200 import sp
    lay = sp.SpLayout(75600, 8, 3)
    assert (lay.start, lay.len, lay.seg_rows) == (28350, 9450, 9450) and not lay.needs_padding()
    lay = sp.SpLayout(11, 2, 1)
    assert (lay.start, lay.len, lay.seg_rows) == (6, 5, 6) and lay.needs_padding()
    assert lay.pass2() == ([6, 0], [0, 6])
    with pytest.raises(ValueError):
        sp.SpLayout(10, 2, 2)
    x = torch.arange(12.0).reshape(1, 1, 4, 3)
    parts = [sp.shard_tensor(x, 2, r, 2) for r in range(2)]
    assert torch.equal(sp.all_gather_seq(parts, 2), x)
    with pytest.raises(ValueError):
        sp.all_gather_seq([], 2)


def test_needed_ranks_under_the_block_causal_mask():
    """Which shards a rank fetches: checked against the predicate itself on every (row, key) pair."""
    from fastvideo_rs_b200 import sp
    from fastvideo_rs_b200.sdpa import BlockCausal
    for seq, world in ((1001, 4), (960, 8), (37, 3), (5, 8)):
        for bc in (BlockCausal(100), BlockCausal(64, 2, 1), BlockCausal(37, 3, 0), BlockCausal(1000), BlockCausal(1, 1, 0),
                   BlockCausal(7, 0, 2)):
            for rank in range(world):
                lay = sp.SpLayout(seq, world, rank)
                need = set(lay.needed_ranks(bc))
                truth = set()
                for o, (s0, l) in enumerate(lay.ranges):
                    if o == rank:
                        continue
                    if any(bc.allows(qi, ki) for qi in range(lay.start, lay.start + lay.len) for ki in range(s0, s0 + l)):
                        truth.add(o)
                # never misses a shard a row can see; may keep one whose keys fall between two rows' windows
                assert truth <= need, (seq, world, bc, rank, truth, need)
                if bc.window == 0:
                    assert truth == need, (seq, world, bc, rank, truth, need)
                lens, starts = lay.pass2_for(bc)
                assert [i for i, l in enumerate(lens) if l] == sorted(need)
                assert starts == [s for s, _ in lay.ranges]
        lay = sp.SpLayout(seq, world, 0)
        assert lay.needed_ranks(None) == [r for r in range(1, world) if lay.ranges[r][1] > 0] or lay.len == 0


def test_native_sp_handle_argument_checks_without_a_gpu():
    """fv_sp_create validates before it touches a device; with no sm_100 device it says so instead of
    computing anywhere else."""
    import ctypes
    import torch
    from fastvideo_rs_b200 import _lib
    L = _lib.lib()
    h = ctypes.c_void_p()
    for world, rank, seq, bh in ((2, 2, 100, 4), (0, 0, 100, 4), (17, 0, 100, 4), (1, 0, 0, 4), (1, 0, 100, 0), (2, -1, 100, 4)):
        assert L.fv_sp_create(None, world, rank, seq, bh, 0, ctypes.byref(h)) == _lib.ERR_INVALID, (world, rank, seq, bh)
        assert not h.value
    assert L.fv_sp_create(None, 2, 0, 100, 4, 0, ctypes.byref(h)) == _lib.ERR_INVALID  # two ranks need an id
    assert "communicator id" in _lib.last_error()
    assert L.fv_sp_info(None, None, None, None, None) == _lib.ERR_INVALID
    assert L.fv_sp_forward_bf16(None, None, None, None, None, None, 1, ctypes.c_float(0.1), 0, 0, 0, 0) == _lib.ERR_INVALID
    assert L.fv_sp_destroy(None) == _lib.RAN
    if not torch.cuda.is_available():
        assert L.fv_sp_create(None, 1, 0, 100, 4, 0, ctypes.byref(h)) == _lib.ERR_NO_DEVICE
        assert not h.value
    # the id comes from NCCL itself when it can be loaded; either way the call answers, it does not crash
    buf = ctypes.create_string_buffer(128)
    rc = L.fv_sp_unique_id(buf)
    assert rc in (_lib.RAN, _lib.ERR_NCCL), _lib.last_error()
    assert L.fv_sp_unique_id(None) == _lib.ERR_INVALID


def test_dense_second_pass_table_is_unchanged_by_the_mask_plumbing():
    """Without a mask the shard selection keeps every other rank: pass2_for(None) is pass2()."""
    from fastvideo_rs_b200 import sp
    for seq, world in ((75600, 8), (75600, 4), (32760, 2), (1001, 3), (5, 8)):
        for rank in range(world):
            lay = sp.SpLayout(seq, world, rank)
            if lay.len:
                assert lay.pass2_for(None) == lay.pass2()
                assert lay.needed_ranks(None) == [r for r in range(world) if r != rank and lay.ranges[r][1] > 0]


def test_native_second_pass_table_equals_the_python_layout():
    """The shard selection inside fv_sp_forward_bf16 (C++) against SpLayout.pass2_for (Python), masks and none."""
    import ctypes
    from fastvideo_rs_b200 import _lib, sp
    from fastvideo_rs_b200.sdpa import BlockCausal
    L = _lib.lib()
    masks = [None, BlockCausal(100), BlockCausal(64, 2, 1), BlockCausal(37, 3, 0), BlockCausal(1000), BlockCausal(1, 1, 0),
             BlockCausal(7, 0, 2), BlockCausal(4680), BlockCausal(390, 4, 1)]
    for seq, world in ((1001, 4), (960, 8), (37, 3), (5, 8), (32760, 8), (75600, 2), (1, 1)):
        for bc in masks:
            for rank in range(world):
                lens = (ctypes.c_int * world)()
                mode, bt, win, sink = (1, bc.block_tokens, bc.window, bc.sink) if bc else (0, 0, 0, 0)
                assert L.fv_sp_second_pass_lens(seq, world, rank, mode, bt, win, sink, lens) == _lib.RAN
                lay = sp.SpLayout(seq, world, rank)
                want = lay.pass2_for(bc)[0] if lay.len else [0 if r == rank else l for r, (_, l) in enumerate(lay.ranges)]
                if lay.len == 0 and bc is not None:
                    continue  # a rank without rows computes nothing: its table is not used
                assert list(lens) == want, (seq, world, rank, bc, list(lens), want)
    lens = (ctypes.c_int * 32)()
    assert L.fv_sp_second_pass_lens(100, 17, 0, 0, 0, 0, 0, lens) == _lib.ERR_INVALID
    assert L.fv_sp_second_pass_lens(100, 2, 2, 0, 0, 0, 0, lens) == _lib.ERR_INVALID


def test_zigzag_layout_balances_the_causal_work_and_covers_the_sequence():
    """Zig-zag split: rank r holds piece r and piece 2 * world - 1 - r of 2 * world pieces.  Every token is held
    once; under the chunk-causal mask of the Self-Forcing shape the ranks' visible (row, key) pairs differ by
    well under one per cent, where contiguous shards differ by a factor of several."""
    from fastvideo_rs_b200 import sp
    from fastvideo_rs_b200.sdpa import BlockCausal
    seq, world, bc = 32760, 8, BlockCausal(4680)
    work = lambda rows: sum(min(seq, (i // bc.block_tokens + 1) * bc.block_tokens) for i in rows)
    held, zz, contiguous = [], [], []
    for r in range(world):
        lay = sp.SpLayout(seq, world, r, zigzag=True)
        rows = lay.rows()
        held += rows
        zz.append(work(rows))
        q0, split, q1 = lay.q_runs()
        assert rows[0] == q0 and rows[split] == q1 and split == lay.runs[r][0][1]
        contiguous.append(work(sp.SpLayout(seq, world, r).rows()))
    assert sorted(held) == list(range(seq))
    assert max(zz) / min(zz) < 1.005 and max(contiguous) / min(contiguous) > 3.0
    # what a rank fetches under the mask, against the predicate itself (small case, every pair)
    for seq, world in ((200, 4), (37, 3)):
        for bc in (BlockCausal(25), BlockCausal(16, 2, 1), BlockCausal(7, 0, 2)):
            for rank in range(world):
                lay = sp.SpLayout(seq, world, rank, zigzag=True)
                need = lay.needed(bc)
                for src in range(world):
                    if src == rank:
                        continue
                    for run, (s0, l) in enumerate(lay.runs[src]):
                        truth = any(bc.allows(qi, ki) for qi in lay.rows() for ki in range(s0, s0 + l))
                        got = need.get(src, [False] * lay.nrun)[run]
                        assert got or not truth, (seq, world, bc, rank, src, run)
                        if bc.window == 0:
                            assert got == truth, (seq, world, bc, rank, src, run)
                lens, starts = lay.pass2_for(bc)
                assert len(lens) == world * lay.nrun and all(l == 0 for l in lens[rank * lay.nrun:(rank + 1) * lay.nrun])


def test_source_groups_cover_the_order_once_and_double():
    """SpLayout.source_groups: the pull order cut into passes of 1, 2, 4, ... sources (or one each); group_segments
    leaves exactly the group's visible runs non-empty at their global offsets."""
    from fastvideo_rs_b200 import sp
    from fastvideo_rs_b200.sdpa import BlockCausal
    for world in (2, 3, 4, 8):
        for zigzag, causal in ((False, None), (True, BlockCausal(100, 0, 0))):
            for rank in range(world):
                lay = sp.SpLayout(1001, world, rank, zigzag=zigzag)
                order = lay.source_order(causal)
                groups = lay.source_groups(causal, True)
                assert [s for g in groups for s in g] == order
                assert [len(g) for g in groups[:-1]] == [2 ** i for i in range(len(groups) - 1)]
                assert lay.source_groups(causal, False) == [[s] for s in order]
                need = lay.needed(causal)
                for g in groups:
                    lens, starts = lay.group_segments(g, causal)
                    assert len(lens) == world * lay.nrun
                    for r in range(world):
                        for run, (s0, l) in enumerate(lay.runs[r]):
                            i = r * lay.nrun + run
                            assert starts[i] == s0
                            assert lens[i] == (l if (r in g and need.get(r, [False] * lay.nrun)[run]) else 0)
