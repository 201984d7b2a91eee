"""Video sparse attention: rt::vsa (crates/fastvideo-cudarc/src/rt/vsa.rs) over the kernels in csrc/vsa.cu.
TilePlan, topk_for and VsaCtx keep the reference's names; vsa_attention is vsa_attention_device
(rt/vsa.rs:358-470) for bf16 tensors on the device."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import numpy as np
import torch

from . import _lib
from .sdpa import _stream_ptr

TILE = (4, 4, 4)
TILE_ELEMS = 64


def topk_for(sparsity: float, num_tiles: int) -> int:
    """Tiles kept for a sparsity level (rt/vsa.rs:34-37)."""
    return _lib.lib().fv_vsa_topk_for(ctypes.c_double(sparsity), int(num_tiles))


class TilePlan:
    """Tiling geometry of one latent grid (rt/vsa.rs:39-109): which token lands in which padded slot and
    how many real tokens each 4x4x4 tile holds."""

    def __init__(self, grid: Tuple[int, int, int]):
        t, h, w = (int(x) for x in grid)
        self._h = ctypes.c_void_p()
        _lib.check(_lib.lib().fv_vsa_plan_create(t, h, w, ctypes.byref(self._h)), f"vsa: grid {grid}")
        nt, seq, padded = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        tiles = (ctypes.c_int * 3)()
        _lib.lib().fv_vsa_plan_info(self._h, ctypes.byref(nt), ctypes.byref(seq), ctypes.byref(padded), tiles)
        self.grid, self.tiles = (t, h, w), tuple(tiles)
        self.seq, self.padded, self._nt = seq.value, padded.value, nt.value
        self.slot_src = np.empty(self.padded, np.int32)
        self.token_slot = np.empty(self.seq, np.uint32)
        self.block_sizes = np.empty(self._nt, np.uint32)
        _lib.lib().fv_vsa_plan_host(self._h, self.slot_src.ctypes.data_as(ctypes.c_void_p),
                                    self.token_slot.ctypes.data_as(ctypes.c_void_p),
                                    self.block_sizes.ctypes.data_as(ctypes.c_void_p))

    @property
    def num_tiles(self) -> int:
        return self._nt

    def __del__(self):
        try:
            if self._h:
                _lib.lib().fv_vsa_plan_destroy(self._h)
        except Exception:
            pass


class VsaCtx:
    """Everything a VSA layer needs for one grid (rt/vsa.rs:329-356): the plan, how many tiles each query
    tile attends, and the workspace (allocated once per (bh) and reused by every layer and step)."""

    def __init__(self, grid, sparsity: float = 0.8, topk: Optional[int] = None):
        self.plan = TilePlan(grid)
        self.topk = topk if topk is not None else topk_for(sparsity, self.plan.num_tiles)
        self.seq = self.plan.seq
        self._ws = {}

    def workspace(self, bh: int, device) -> torch.Tensor:
        key = (bh, str(device))
        if key not in self._ws:
            n = _lib.lib().fv_vsa_workspace_bytes(self.plan._h, bh, self.topk)
            self._ws[key] = torch.empty(n, dtype=torch.uint8, device=device)
        return self._ws[key]


_lib_size_t_set = False


def vsa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: Optional[torch.Tensor], ctx: VsaCtx,
                  scale: Optional[float] = None, out_bf16: bool = True, want_aux: bool = False):
    """VSA on the device: q, k, v, gate [bh, seq, 128] bf16 (gate may be None) -> [bh, seq, 128].
    out = coarse * gate + fine (linear gate).  With want_aux also returns (selected [bh, nt, topk] int64
    ascending, scores [bh, nt, nt] f32, coarse [bh, nt, 128] f32)."""
    global _lib_size_t_set
    L = _lib.lib()
    if not _lib_size_t_set:
        L.fv_vsa_workspace_bytes.restype = ctypes.c_size_t
        _lib_size_t_set = True
    for name, t in (("q", q), ("k", k), ("v", v), ("gate", gate)):
        if t is None:
            continue
        if not t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ValueError(f"vsa: {name} must be a contiguous CUDA bf16 tensor")
    bh, seq, d = q.shape
    if seq != ctx.seq or d != 128:
        raise ValueError(f"vsa: q has {seq} tokens x {d}, the plan has {ctx.seq} x 128")
    nt, topk = ctx.plan.num_tiles, min(max(ctx.topk, 1), ctx.plan.num_tiles)
    scale = float(scale) if scale is not None else 1.0 / d ** 0.5
    out = torch.empty((bh, seq, d), dtype=torch.bfloat16 if out_bf16 else torch.float32, device=q.device)
    ws = ctx.workspace(bh, q.device)
    sel = sc = co = None
    if want_aux:
        sel = torch.empty((bh, nt, topk), dtype=torch.int32, device=q.device)
        sc = torch.empty((bh, nt, nt), dtype=torch.float32, device=q.device)
        co = torch.empty((bh, nt, 128), dtype=torch.float32, device=q.device)
    vp = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
    with torch.cuda.device(q.device):
        rc = L.fv_vsa_forward_bf16(_stream_ptr(), ctx.plan._h, vp(q), vp(k), vp(v), vp(gate), bh, topk,
                                   ctypes.c_float(scale), vp(out), int(out_bf16), vp(ws), ctypes.c_size_t(ws.numel()),
                                   vp(sel), vp(sc), vp(co))
    _lib.check(rc, "vsa_attention")
    if want_aux:
        return out, sel.long(), sc, co
    return out
