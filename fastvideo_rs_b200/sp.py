"""Sequence parallelism for the attention call: one process per GPU, contiguous token shards
(sp::shard_ranges, crates/fastvideo-cudarc/src/rt/sp.rs:16-28), ONE exchange -- an NCCL all-gather
of the rank's bf16 K and V shards into every rank's own HBM -- overlapped with attention over the
local keys; the output stays sharded.  (The reference replicates K/V on every rank and gathers the
outputs through the host, rt/sdpa.rs:354-410; this replaces that.)

Pass 1 (compute stream): softmax(Q_r K_r^T) V_r, f32, with its log-sum-exp.
Exchange (communication stream, concurrently): all-gather K, all-gather V.
Pass 2 (compute stream, after the exchange): the same kernel over the other ranks' segments,
merging pass 1 in its epilogue -- exactly the softmax over all keys."""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Tuple

import torch

from . import _lib
from .sdpa import BlockCausal, _stream_ptr


def shard_ranges(seq: int, world: int) -> List[Tuple[int, int]]:
    """[(start, len)] per rank: contiguous, remainder to the low ranks."""
    world = max(world, 1)
    st = (ctypes.c_int * world)()
    ln = (ctypes.c_int * world)()
    _lib.lib().fv_shard_ranges(seq, world, st, ln)
    return [(st[i], ln[i]) for i in range(world)]


def shard_tensor(x: torch.Tensor, dim: int, rank: int, world: int) -> torch.Tensor:
    """This rank's slice of `x` along `dim` (sp::shard_tensor, rt/sp.rs:41-49)."""
    ranges = shard_ranges(x.shape[dim], world)
    if not 0 <= rank < len(ranges):
        raise ValueError(f"SP rank {rank} out of world {world}")
    start, length = ranges[rank]
    return x.narrow(dim, start, length)


def all_gather_seq(shards: List[torch.Tensor], dim: int) -> torch.Tensor:
    """Concatenate sequence shards (sp::all_gather_seq, rt/sp.rs:31-37)."""
    if not shards:
        raise ValueError("all_gather empty")
    return torch.cat(shards, dim)


def _i32(vals):
    return (ctypes.c_int * len(vals))(*[int(v) for v in vals])


def segments_fwd(q, k_all, v_all, seg_len, seg_start, seg_rows, scale, *, out=None, out_bf16=True, causal=None,
                 q_row0=0, q_split=0, q_row1=0, lse_out=None, prev_o=None, prev_lse=None):
    """fv_sdpa_segments_runs_bf16: q [bh, sq, 128]; k_all / v_all [nseg, bh, seg_rows, 128].  Rows from q_split on
    (when > 0) are a second run of the sequence starting at global row q_row1."""
    bh, sq, d = q.shape
    nseg = len(seg_len)
    if out is None:
        out = torch.empty((bh, sq, d), dtype=torch.bfloat16 if out_bf16 else torch.float32, device=q.device)
    mode, bt, win, sink = (1, causal.block_tokens, causal.window, causal.sink) if causal else (0, 0, 0, 0)
    vp = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
    fp = lambda t: ctypes.cast(ctypes.c_void_p(t.data_ptr()), ctypes.POINTER(ctypes.c_float)) if t is not None else None
    with torch.cuda.device(q.device):
        rc = _lib.lib().fv_sdpa_segments_runs_bf16(_stream_ptr(), vp(q), vp(k_all), vp(v_all), vp(out),
                                                   int(out.dtype == torch.bfloat16), bh, sq, nseg, _i32(seg_len),
                                                   _i32(seg_start), seg_rows, ctypes.c_float(scale), mode, bt, win, sink,
                                                   q_row0, q_split, q_row1, fp(lse_out), fp(prev_o), fp(prev_lse))
    _lib.check(rc, "segments_fwd")
    return out


class SpLayout:
    """Host-side bookkeeping of the exchange, pure Python: which runs of the sequence each rank holds, how the
    staging and gathered buffers are laid out, and the segment tables of the passes.

    contiguous (the reference's split, rt/sp.rs:16-28): rank r holds ONE run, shard_ranges(seq, world)[r].
    zigzag: the sequence is cut into 2 * world pieces and rank r holds piece r and piece 2 * world - 1 - r, an
    early and a late one.  Under a causal mask a row sees about as many keys as its index, so contiguous shards
    give the last rank several times the first rank's work; a zig-zag pair always adds up to about the same.

    Every run lives in a slot of `run_rows` rows (the longest run of any rank; shorter ones are zero-padded), so
    that one rank's K (or V) is a [runs, bh, run_rows, 128] block: `runs` key segments of the attention call."""

    def __init__(self, seq: int, world: int, rank: int, zigzag: bool = False):
        if not 0 <= rank < max(world, 1):
            raise ValueError(f"SP rank {rank} out of world {world}")
        self.seq, self.world, self.rank, self.zigzag = seq, max(world, 1), rank, bool(zigzag) and world > 1
        if self.zigzag:
            pieces = shard_ranges(seq, 2 * self.world)
            self.runs = [[pieces[r], pieces[2 * self.world - 1 - r]] for r in range(self.world)]
        else:
            self.runs = [[rg] for rg in shard_ranges(seq, self.world)]
        self.nrun = len(self.runs[0])
        self.ranges = [rr[0] for rr in self.runs]           # first run of every rank (the contiguous shard)
        self.start, _ = self.runs[rank][0]
        self.len = sum(l for _, l in self.runs[rank])      # rows this rank holds
        self.run_rows = max(max(l for _, l in rr) for rr in self.runs)
        self.seg_rows = self.run_rows

    # ---- this rank's query rows
    def q_runs(self):
        """(q_row0, q_split, q_row1) of this rank's rows for the attention call."""
        rr = self.runs[self.rank]
        if len(rr) == 1 or rr[1][1] == 0:
            return rr[0][0], 0, 0
        if rr[0][1] == 0:
            return rr[1][0], 0, 0
        return rr[0][0], rr[0][1], rr[1][0]

    def rows(self, rank: Optional[int] = None):
        """Global row indices this rank (or `rank`) holds, in its local order."""
        rr = self.runs[self.rank if rank is None else rank]
        return [i for s, l in rr for i in range(s, s + l)]

    # ---- key segments
    def pass1(self):
        """(seg_len, seg_start) of the local-keys pass: this rank's own runs."""
        rr = self.runs[self.rank]
        return [l for _, l in rr], [s for s, _ in rr]

    def needed(self, causal: Optional[BlockCausal]):
        """{source rank: [run is needed]} over the other ranks: the runs that hold a key some row of this rank may
        see.  Dense: every non-empty run.  Under the block-causal mask (rt/attn.rs:448-453) rows [a, b) see the
        keys [lo, hi) and [0, sink * block): hi = the end of row b-1's block (it may reach past the run), lo = the
        start of the oldest block inside row a's window (0 without a window)."""
        mine = [(s, l) for s, l in self.runs[self.rank] if l > 0]
        out = {}
        for r in range(self.world):
            if r == self.rank or not mine:
                continue
            flags = []
            for s0, l in self.runs[r]:
                need = l > 0
                if need and causal is not None:
                    bt = max(causal.block_tokens, 1)
                    sink_hi = min(self.seq, causal.sink * bt)
                    need = s0 < sink_hi
                    for a, n in mine:
                        hi = min(self.seq, ((a + n - 1) // bt + 1) * bt)
                        lo = max(0, a // bt - causal.window + 1) * bt if causal.window > 0 else 0
                        need = need or (s0 < hi and s0 + l > lo)
                flags.append(need)
            if any(flags):
                out[r] = flags
        return out

    def needed_ranks(self, causal: Optional[BlockCausal]) -> List[int]:
        return sorted(self.needed(causal))

    def source_order(self, causal: Optional[BlockCausal]) -> List[int]:
        """The needed source ranks, nearest first (rank - 1, rank - 2, ...): every rank then pulls from a different
        peer at any one time."""
        need = self.needed(causal)
        return [r for r in ((self.rank - step) % self.world for step in range(1, self.world)) if r in need]

    def source_segments(self, src: int, causal: Optional[BlockCausal]):
        """(seg_len, seg_start) of one source rank's block, runs nobody here can see emptied."""
        flags = self.needed(causal).get(src, [False] * self.nrun)
        return [l if f else 0 for (_, l), f in zip(self.runs[src], flags)], [s for s, _ in self.runs[src]]

    def source_groups(self, causal: Optional[BlockCausal], grouped: bool = True) -> List[List[int]]:
        """The needed sources in the order they are pulled, cut into the passes that consume them: one source, then
        two, then four, ... (grouped) or one per pass.  A pass costs a fixed amount per work item (the first key tile
        of an item takes the exact softmax path, the pipeline fills and drains, the epilogue reads and writes the f32
        state), so at 8 ranks seven passes of one source each spend a fifth of their time there; doubling the group
        keeps the first remote pass as early as it can be and every later one no longer than what hides its copies."""
        order = self.source_order(causal)
        if not grouped:
            return [[s] for s in order]
        groups, size, i = [], 1, 0
        while i < len(order):
            groups.append(order[i:i + size])
            i += size
            size *= 2
        return groups

    def group_segments(self, srcs, causal: Optional[BlockCausal]):
        """(seg_len, seg_start) over the whole gathered buffer [world, runs, ...] with only the runs of `srcs` that
        somebody here can see left non-empty."""
        need = self.needed(causal)
        lens, starts = [], []
        for r in range(self.world):
            flags = need.get(r, [False] * self.nrun)
            for (s0, l), f in zip(self.runs[r], flags):
                lens.append(l if (f and r in srcs and r != self.rank) else 0)
                starts.append(s0)
        return lens, starts

    def pass2(self):
        """(seg_len, seg_start) of ONE remote-keys pass over the whole gathered buffer [world, runs, ...]: every
        run at its global offset, this rank's own ones emptied (pass 1 covered them)."""
        return self.pass2_for(None)

    def pass2_for(self, causal: Optional[BlockCausal]):
        need = self.needed(causal)
        lens, starts = [], []
        for r in range(self.world):
            flags = need.get(r, [False] * self.nrun)
            for (s0, l), f in zip(self.runs[r], flags):
                lens.append(l if (f and r != self.rank) else 0)
                starts.append(s0)
        return lens, starts

    def needs_padding(self) -> bool:
        return any(l != self.run_rows for _, l in self.runs[self.rank])


class SpAttention:
    """Sequence-parallel attention for one (seq, bh) shape; buffers allocated once.

    Per call: this rank's K and V go into a staging block; the exchange brings every other rank's block into
    this rank's own HBM on a communication stream while pass 1 (local keys) runs; then passes over the nearest
    source rank, the next two, the next four, ... (SpLayout.source_groups), each as soon as its blocks have
    landed, each continuing the previous pass' softmax state (f32 result + log-sum-exp).  Only the first
    block's transfer has to hide under pass 1; every later one hides under the passes before it.

    exchange="ce" (default): the staging block is peer-mapped (torch symmetric memory, multicast off) and the
      other ranks PULL it with plain device-to-device copies that the copy engines carry out over NVLink -- no SM
      is used, which matters because the attention kernel holds every SM for the whole launch.  The staging
      block is double-buffered, so one device-side barrier per call is enough (when a rank passes the barrier of
      call n + 1 every peer has finished pulling call n, and call n + 2 is the next one to write that half).
    exchange="nccl": ncclAllGather of K and of V, then one remote pass over all of it."""

    def __init__(self, seq: int, bh: int, group=None, device=None, zigzag: bool = False, exchange: Optional[str] = None,
                 grouped: Optional[bool] = None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        # remote passes over one, two, four, ... sources (default) or one pass per source (FV_SP_PASSES=per-source)
        self.grouped = grouped if grouped is not None else os.environ.get("FV_SP_PASSES", "grouped") != "per-source"
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.seq, self.bh = seq, bh
        self.layout = L = SpLayout(seq, self.world, self.rank, zigzag)
        self.ranges, self.start, self.len, self.seg_rows = L.ranges, L.start, L.len, L.run_rows
        self.calls = 0
        d = 128
        if self.world == 1:
            return
        blk = (L.nrun, bh, L.run_rows, d)
        self.k_all = torch.zeros((self.world,) + blk, dtype=torch.bfloat16, device=self.device)
        self.v_all = torch.zeros((self.world,) + blk, dtype=torch.bfloat16, device=self.device)
        self.o_buf = [torch.empty((bh, self.len, d), dtype=torch.float32, device=self.device) for _ in range(2)]
        self.lse_buf = [torch.empty((bh, self.len), dtype=torch.float32, device=self.device) for _ in range(2)]
        prio = int(os.environ.get("FV_SP_COMM_PRIORITY", "-1"))
        self.comm_stream = torch.cuda.Stream(device=self.device, priority=prio)
        self.exchange = exchange or os.environ.get("FV_SP_EXCHANGE", "ce")
        self.stage = self.hdl = None
        self.fenced = [None, None]  # per staging half: the event after which it may be rewritten
        if self.exchange == "ce":
            try:
                os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
                import torch.distributed._symmetric_memory as symm_mem
                shape = (2, 2) + blk  # [half][k | v][run][bh][rows][d]
                self.stage = symm_mem.empty(shape, dtype=torch.bfloat16, device=self.device)
                self.stage.zero_()
                self.hdl = symm_mem.rendezvous(self.stage, group if group is not None else dist.group.WORLD)
                self.peer = [self.hdl.get_buffer(r, shape, torch.bfloat16) for r in range(self.world)]
            except Exception as e:  # no peer mapping on this machine: say so and use NCCL
                import sys
                print(f"sp: peer-mapped staging unavailable ({type(e).__name__}: {e}); using the NCCL all-gather", file=sys.stderr)
                self.exchange, self.stage, self.hdl = "nccl", None, None
        if self.exchange != "ce":
            self.local = torch.zeros((2,) + blk, dtype=torch.bfloat16, device=self.device)  # [k | v] padded block

    def _fill(self, dst: torch.Tensor, x: torch.Tensor) -> None:
        """This rank's [bh, len, d] rows into a [runs, bh, run_rows, d] block (padding rows stay zero)."""
        off = 0
        for r, (_, l) in enumerate(self.layout.runs[self.rank]):
            if l:
                dst[r, :, :l].copy_(x[:, off:off + l])
            off += l

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None,
                out: Optional[torch.Tensor] = None, causal: Optional[BlockCausal] = None) -> torch.Tensor:
        """q, k, v: this rank's [bh, len_r, 128] bf16 rows (zig-zag: the early run followed by the late one).
        Returns this rank's [bh, len_r, 128] bf16.  causal: the block-causal mask over GLOBAL token indices; a rank
        then fetches only the runs its rows can see."""
        L, d = self.layout, q.shape[-1]
        scale = float(scale) if scale is not None else 1.0 / d ** 0.5
        q_row0, q_split, q_row1 = L.q_runs()
        if self.world == 1:
            return segments_fwd(q, k, v, [self.len], [0], self.len, scale, out=out, causal=causal)
        cur = torch.cuda.current_stream(self.device)
        if out is None:
            out = torch.empty((self.bh, self.len, d), dtype=torch.bfloat16, device=q.device)
        order = L.source_order(causal)
        half = self.calls & 1
        self.calls += 1
        arrived = {}
        if self.exchange == "ce":
            if self.fenced[half] is not None:
                cur.wait_event(self.fenced[half])  # every rank has pulled what this half held two calls ago
            mine_k, mine_v = self.stage[half, 0], self.stage[half, 1]
            self._fill(mine_k, k)
            self._fill(mine_v, v)
            ready = torch.cuda.Event()
            ready.record(cur)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ready)
                self.hdl.barrier(channel=0)  # every rank's staging half is written (and its previous pulls are done)
                fence = torch.cuda.Event()
                fence.record(self.comm_stream)
                self.fenced[1 - half] = fence   # the OTHER half was last read one call ago: free from here on
                for src in order:
                    flags = L.needed(causal)[src]
                    for r, f in enumerate(flags):
                        if f:  # contiguous blocks: the copy engines move them, no kernel touches peer memory
                            self.k_all[src, r].copy_(self.peer[src][half, 0, r], non_blocking=True)
                            self.v_all[src, r].copy_(self.peer[src][half, 1, r], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self.comm_stream)
                    arrived[src] = ev
        else:
            mine_k, mine_v = self.local[0], self.local[1]
            self._fill(mine_k, k)
            self._fill(mine_v, v)
            ready = torch.cuda.Event()
            ready.record(cur)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ready)
                self.dist.all_gather_into_tensor(self.k_all, mine_k, group=self.group)
                self.dist.all_gather_into_tensor(self.v_all, mine_v, group=self.group)
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
                arrived = {src: ev for src in order}
        # pass 1: the local keys, while the exchange is in flight
        if self.exchange == "nccl":
            # the all-gather's copy kernels need SMs beside the persistent attention CTAs of pass 1
            _lib.lib().fv_hint_spare_sms(int(os.environ.get("FV_SP_SPARE_SMS", "24")))
        l1, s1 = L.pass1()
        common = dict(causal=causal, q_row0=q_row0, q_split=q_split, q_row1=q_row1)
        if not order:  # no row of this rank sees a key of another rank: pass 1 is the result
            segments_fwd(q, mine_k, mine_v, l1, s1, L.run_rows, scale, out=out, **common)
            for ev in set(arrived.values()):
                cur.wait_event(ev)  # (nccl: the gather still reads this rank's block)
            return out
        segments_fwd(q, mine_k, mine_v, l1, s1, L.run_rows, scale, out=self.o_buf[0], lse_out=self.lse_buf[0], **common)
        if self.exchange == "ce":
            # one pass per source rank as its block lands, each continuing the state of the one before
            groups = L.source_groups(causal, self.grouped)
            k_flat = self.k_all.view(-1, self.bh, L.run_rows, d)
            v_flat = self.v_all.view(-1, self.bh, L.run_rows, d)
            for n, srcs in enumerate(groups):
                cur.wait_event(arrived[srcs[-1]])  # (the copies are in stream order: the last one's event covers the group)
                last = n == len(groups) - 1
                a, b = n & 1, 1 - (n & 1)
                if len(srcs) == 1:
                    ln, st = L.source_segments(srcs[0], causal)
                    kk, vv = self.k_all[srcs[0]], self.v_all[srcs[0]]
                else:
                    ln, st = L.group_segments(srcs, causal)
                    kk, vv = k_flat, v_flat
                segments_fwd(q, kk, vv, ln, st, L.run_rows, scale,
                             out=out if last else self.o_buf[b], lse_out=None if last else self.lse_buf[b],
                             prev_o=self.o_buf[a], prev_lse=self.lse_buf[a], **common)
        else:
            cur.wait_event(arrived[order[0]])
            ln, st = L.pass2_for(causal)
            segments_fwd(q, self.k_all.view(-1, self.bh, L.run_rows, d), self.v_all.view(-1, self.bh, L.run_rows, d), ln, st,
                         L.run_rows, scale, out=out, prev_o=self.o_buf[0], prev_lse=self.lse_buf[0], **common)
        return out


class NativeSp:
    """The same sequence-parallel attention with the whole sequence of launches behind the C ABI
    (fv_sp_create / fv_sp_forward_bf16: NCCL all-gather on the handle's own high-priority stream, two passes),
    for hosts that are not Python.  `unique_id`: the 128 bytes of `NativeSp.unique_id()` made on rank 0 and handed
    to every rank (here: by torch.distributed, in a Rust host: by whatever it has).  One handle per rank."""

    def __init__(self, seq: int, bh: int, world: int, rank: int, unique_id: Optional[bytes] = None, groups: int = 0):
        self.seq, self.bh, self.world, self.rank = seq, bh, world, rank
        self._h = ctypes.c_void_p()
        buf = ctypes.create_string_buffer(unique_id, 128) if unique_id is not None else None
        rc = _lib.lib().fv_sp_create(buf, world, rank, seq, bh, groups, ctypes.byref(self._h))
        _lib.check(rc, "fv_sp_create")
        st, ln, rows, gr = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        _lib.check(_lib.lib().fv_sp_info(self._h, ctypes.byref(st), ctypes.byref(ln), ctypes.byref(rows), ctypes.byref(gr)),
                   "fv_sp_info")
        self.start, self.len, self.seg_rows, self.groups = st.value, ln.value, rows.value, gr.value

    @staticmethod
    def unique_id() -> bytes:
        buf = ctypes.create_string_buffer(128)
        _lib.check(_lib.lib().fv_sp_unique_id(buf), "fv_sp_unique_id")
        return buf.raw

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None,
                out: Optional[torch.Tensor] = None, out_bf16: bool = True,
                causal: Optional[BlockCausal] = None) -> torch.Tensor:
        """q, k, v: this rank's [bh, len, 128] bf16 shards -> this rank's [bh, len, 128]."""
        scale = float(scale) if scale is not None else 1.0 / q.shape[-1] ** 0.5
        if out is None:
            out = torch.empty((self.bh, self.len, 128), dtype=torch.bfloat16 if out_bf16 else torch.float32, device=q.device)
        mode, bt, win, sink = (1, causal.block_tokens, causal.window, causal.sink) if causal else (0, 0, 0, 0)
        vp = lambda t: ctypes.c_void_p(t.data_ptr())
        with torch.cuda.device(q.device):
            rc = _lib.lib().fv_sp_forward_bf16(self._h, _stream_ptr(), vp(q), vp(k), vp(v), vp(out),
                                               int(out.dtype == torch.bfloat16), ctypes.c_float(scale), mode, bt, win, sink)
        _lib.check(rc, "fv_sp_forward_bf16")
        return out

    def close(self) -> None:
        if self._h:
            _lib.lib().fv_sp_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
