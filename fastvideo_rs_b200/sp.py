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
                 q_row0=0, lse_out=None, prev_o=None, prev_lse=None):
    """fv_sdpa_segments_bf16: q [bh, sq, 128]; k_all / v_all [nseg, bh, seg_rows, 128]."""
    bh, sq, d = q.shape
    nseg = len(seg_len)
    if out is None:
        out = torch.empty((bh, sq, d), dtype=torch.bfloat16 if out_bf16 else torch.float32, device=q.device)
    mode, bt, win, sink = (1, causal.block_tokens, causal.window, causal.sink) if causal else (0, 0, 0, 0)
    vp = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
    fp = lambda t: ctypes.cast(ctypes.c_void_p(t.data_ptr()), ctypes.POINTER(ctypes.c_float)) if t is not None else None
    with torch.cuda.device(q.device):
        rc = _lib.lib().fv_sdpa_segments_bf16(_stream_ptr(), vp(q), vp(k_all), vp(v_all), vp(out),
                                              int(out.dtype == torch.bfloat16), bh, sq, nseg, _i32(seg_len),
                                              _i32(seg_start), seg_rows, ctypes.c_float(scale), mode, bt, win, sink,
                                              q_row0, fp(lse_out), fp(prev_o), fp(prev_lse))
    _lib.check(rc, "segments_fwd")
    return out


class SpLayout:
    """Host-side bookkeeping of the exchange, pure Python: who holds which tokens, how the gathered
    buffer is laid out ([world, bh, seg_rows, 128], shorter shards zero-padded to seg_rows), and the
    segment tables of the two passes."""

    def __init__(self, seq: int, world: int, rank: int):
        if not 0 <= rank < max(world, 1):
            raise ValueError(f"SP rank {rank} out of world {world}")
        self.seq, self.world, self.rank = seq, max(world, 1), rank
        self.ranges = shard_ranges(seq, self.world)
        self.start, self.len = self.ranges[rank]
        self.seg_rows = max(l for _, l in self.ranges)

    def pass1(self):
        """(seg_len, seg_start) of the local-keys pass: one segment, this rank's shard."""
        return [self.len], [self.start]

    def pass2(self):
        """(seg_len, seg_start) of the remote-keys pass over the gathered buffer: every rank's segment at
        its global offset, this rank's own one emptied (pass 1 covered it)."""
        lens = [l if r != self.rank else 0 for r, (_, l) in enumerate(self.ranges)]
        return lens, [s for s, _ in self.ranges]

    def needs_padding(self) -> bool:
        return self.len != self.seg_rows

    def needed_ranks(self, causal: Optional[BlockCausal]) -> List[int]:
        """The other ranks whose shard holds a key some row of this shard may see.  Dense: all of them.  Under
        the block-causal mask (rt/attn.rs:448-453) the rows [start, start + len) see the keys
        [lo, hi) and [0, sink * block): hi = the end of the last row's block (it may reach into the next shard),
        lo = the start of the oldest block inside the first row's window (0 without a window)."""
        others = [r for r in range(self.world) if r != self.rank]
        if causal is None or self.len == 0:
            return others if self.len else []
        bt = max(causal.block_tokens, 1)
        first, last = self.start, self.start + self.len - 1
        hi = min(self.seq, (last // bt + 1) * bt)
        lo = max(0, first // bt - causal.window + 1) * bt if causal.window > 0 else 0
        sink_hi = min(self.seq, causal.sink * bt)
        need = []
        for r in others:
            s0, l = self.ranges[r]
            if l > 0 and ((s0 < hi and s0 + l > lo) or s0 < sink_hi):
                need.append(r)
        return need

    def pass2_for(self, causal: Optional[BlockCausal]):
        """pass2() with the segments of ranks no row can see emptied: their shards are not fetched."""
        need = set(self.needed_ranks(causal))
        lens = [l if r in need else 0 for r, (_, l) in enumerate(self.ranges)]
        return lens, [s for s, _ in self.ranges]


class SpAttention:
    """Sequence-parallel dense attention for one (seq, bh) shape; buffers allocated once.

    groups: the heads are cut into that many contiguous groups, each with its own pair of all-gathers; the remote pass
    of group g starts when group g has arrived, so only the first group's exchange has to hide under the local pass
    (at 8 GPUs the whole exchange is longer than the local pass).  Default: 2 groups from 8 ranks on, else 1."""

    def __init__(self, seq: int, bh: int, group=None, device=None, groups: Optional[int] = None):
        import os
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.seq, self.bh = seq, bh
        self.layout = SpLayout(seq, self.world, self.rank)
        self.ranges, self.start, self.len, self.seg_rows = (self.layout.ranges, self.layout.start, self.layout.len,
                                                            self.layout.seg_rows)
        d = 128
        if groups is None:
            groups = int(os.environ.get("FV_SP_GROUPS", "0")) or (2 if self.world >= 8 else 1)
        if groups < 1 or bh % groups != 0:
            groups = 1
        self.groups, self.bh_g = groups, bh // groups
        if self.world > 1:
            mk = lambda: torch.zeros((self.world, self.bh_g, self.seg_rows, d), dtype=torch.bfloat16, device=self.device)
            self.k_all = [mk() for _ in range(groups)]
            self.v_all = [mk() for _ in range(groups)]
            self.o1 = torch.empty((bh, self.len, d), dtype=torch.float32, device=self.device)
            self.lse1 = torch.empty((bh, self.len), dtype=torch.float32, device=self.device)
            # The exchange runs on a HIGH-priority stream: the attention kernel keeps every SM busy with one large CTA each,
            # and NCCL's copy CTAs only make progress once all of them are resident -- at default priority they trickle in
            # as attention CTAs retire and the gather takes longer than the compute it should hide under (measured at 8
            # GPUs: 14.3 ms per step against 9.9 ms without the exchange).
            prio = int(os.environ.get("FV_SP_COMM_PRIORITY", "-1"))
            self.comm_stream = torch.cuda.Stream(device=self.device, priority=prio)
            # extra streams so that pulls from different peers run on different copy engines at the same time
            ncopy = max(1, min(int(os.environ.get("FV_SP_COPY_STREAMS", "1")), self.world - 1))
            self.copy_streams = [self.comm_stream] + [torch.cuda.Stream(device=self.device, priority=prio) for _ in range(ncopy - 1)]
            self.pad = None
            if self.layout.needs_padding():
                self.pad = (torch.zeros((bh, self.seg_rows, d), dtype=torch.bfloat16, device=self.device),
                            torch.zeros((bh, self.seg_rows, d), dtype=torch.bfloat16, device=self.device))
            # How the shards travel.  "nccl": ncclAllGather (its copy CTAs compete with the attention CTAs for SMs).
            # "ce": every rank keeps its K/V shard in a peer-mapped staging buffer and PULLS the other ranks' shards with
            # plain device-to-device copies, which the copy engines carry out over NVLink without using any SM; two
            # device-side barriers per call fence the staging buffer (written / everybody has pulled).
            self.exchange = os.environ.get("FV_SP_EXCHANGE", "ce")
            self.stage = self.hdl = self.released = None
            if self.exchange == "ce":
                try:
                    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
                    import torch.distributed._symmetric_memory as symm_mem
                    self.stage = symm_mem.empty((2, bh, self.seg_rows, d), dtype=torch.bfloat16, device=self.device)
                    self.stage.zero_()
                    self.hdl = symm_mem.rendezvous(self.stage, group if group is not None else dist.group.WORLD)
                    self.peer = [self.hdl.get_buffer(r, (2, bh, self.seg_rows, d), torch.bfloat16) for r in range(self.world)]
                except Exception as e:  # no peer mapping on this machine: say so and use NCCL
                    import sys
                    print(f"sp: peer-mapped staging unavailable ({type(e).__name__}: {e}); using the NCCL all-gather", file=sys.stderr)
                    self.exchange, self.stage, self.hdl = "nccl", None, None

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None,
                out: Optional[torch.Tensor] = None, causal: Optional[BlockCausal] = None) -> torch.Tensor:
        """q, k, v: this rank's [bh, len_r, 128] bf16 shards.  Returns this rank's [bh, len_r, 128] bf16.
        causal: the block-causal mask over GLOBAL token indices; a rank then fetches only the shards its rows
        can see (later ranks do more work than earlier ones: contiguous shards are kept, as the reference's)."""
        d = q.shape[-1]
        scale = float(scale) if scale is not None else 1.0 / d ** 0.5
        if self.world == 1:
            return segments_fwd(q, k, v, [self.len], [0], self.len, scale, out=out, causal=causal)
        need = self.layout.needed_ranks(causal)
        cur = torch.cuda.current_stream(self.device)
        if out is None:
            out = torch.empty((self.bh, self.len, d), dtype=torch.bfloat16, device=q.device)
        G, n = self.groups, self.bh_g
        no_comm = os.environ.get("FV_SP_NO_COMM") == "1"  # diagnosis only: compute without the exchange (wrong results)
        arrived = []
        if self.exchange == "ce":
            if self.released is not None:
                cur.wait_event(self.released)  # every rank has pulled the previous call's shard out of the staging buffer
            self.stage[0, :, : self.len].copy_(k)
            self.stage[1, :, : self.len].copy_(v)
            ks, vs = self.stage[0], self.stage[1]
            ready = torch.cuda.Event()
            ready.record(cur)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ready)
                if not no_comm:
                    self.hdl.barrier(channel=0)  # every rank's staging buffer is written
                fence = torch.cuda.Event()
                fence.record(self.comm_stream)
                for cs in self.copy_streams[1:]:
                    cs.wait_event(fence)
                for g in range(G):
                    for step in range(1, self.world):
                        r = (self.rank - step) % self.world
                        if not no_comm and r in need:
                            with torch.cuda.stream(self.copy_streams[(step - 1) % len(self.copy_streams)]):
                                self.k_all[g][r].copy_(self.peer[r][0, g * n:(g + 1) * n], non_blocking=True)
                                self.v_all[g][r].copy_(self.peer[r][1, g * n:(g + 1) * n], non_blocking=True)
                    for cs in self.copy_streams[1:]:  # group g has arrived when every copy stream got this far
                        e2 = torch.cuda.Event()
                        e2.record(cs)
                        self.comm_stream.wait_event(e2)
                    ev = torch.cuda.Event()
                    ev.record(self.comm_stream)
                    arrived.append(ev)
                if not no_comm:
                    self.hdl.barrier(channel=1)  # every rank has pulled: the staging buffers may be rewritten
                self.released = torch.cuda.Event()
                self.released.record(self.comm_stream)
        else:
            if self.pad is not None:
                self.pad[0][:, : self.len].copy_(k)
                self.pad[1][:, : self.len].copy_(v)
                ks, vs = self.pad
            else:
                ks, vs = k, v
            ready = torch.cuda.Event()
            ready.record(cur)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ready)
                for g in range(G):
                    if not no_comm:
                        self.dist.all_gather_into_tensor(self.k_all[g].view(-1, self.seg_rows, d), ks[g * n:(g + 1) * n], group=self.group)
                        self.dist.all_gather_into_tensor(self.v_all[g].view(-1, self.seg_rows, d), vs[g * n:(g + 1) * n], group=self.group)
                    ev = torch.cuda.Event()
                    ev.record(self.comm_stream)
                    arrived.append(ev)
        # pass 1: the local keys, every head, while the exchange is in flight
        l1, s1 = self.layout.pass1()
        l2, s2 = self.layout.pass2_for(causal)
        if not any(l2):  # no row of this shard sees a key of another shard: pass 1 is the result
            segments_fwd(q, ks, vs, l1, s1, self.seg_rows, scale, out=out, causal=causal, q_row0=self.start)
            return out
        segments_fwd(q, ks, vs, l1, s1, self.seg_rows, scale, out=self.o1, lse_out=self.lse1, causal=causal,
                     q_row0=self.start)
        # pass 2 per head group, as it arrives: every other rank's keys, merged with pass 1
        for g in range(G):
            cur.wait_event(arrived[g])
            sl = slice(g * n, (g + 1) * n)
            segments_fwd(q[sl], self.k_all[g], self.v_all[g], l2, s2, self.seg_rows, scale, out=out[sl],
                         prev_o=self.o1[sl], prev_lse=self.lse1[sl], causal=causal, q_row0=self.start)
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
