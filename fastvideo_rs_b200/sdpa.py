"""The one attention entry: rt::sdpa::sdpa(q, k, v, &Plan) (crates/fastvideo-cudarc/src/rt/sdpa.rs:27-164)
over torch CUDA tensors.  The Plan constructors keep the reference's names.  Which kernel runs is
sdpa_rule's choice; when that choice is not this library's sm_100a kernel the call raises
``Declined`` -- this package has no other kernel and no CPU path."""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from . import sdpa_rule


@dataclass(frozen=True)
class BlockCausal:
    """Wan's block-causal temporal mask as kernel parameters (rt/attn.rs:434-453): query q sees key k
    iff (block(k) <= block(q) and (window == 0 or block(q) - block(k) < window)) or block(k) < sink."""
    block_tokens: int
    window: int = 0
    sink: int = 0

    def allows(self, q: int, k: int) -> bool:
        bt = max(self.block_tokens, 1)
        tq, tk = q // bt, k // bt
        return (tk <= tq and (self.window == 0 or tq - tk < self.window)) or tk < self.sink


_DENSE, _COMPOSED, _BLOCK_CAUSAL, _VDN_WINDOW, _KV_WINDOW = range(5)


@dataclass(frozen=True, eq=False)
class Plan:
    """What one attention call computes (rt/sdpa.rs:27-139)."""
    kind: int = _DENSE
    scale: Optional[float] = None
    mask: Optional[torch.Tensor] = None
    fp8_first_: bool = False
    causal: Optional[BlockCausal] = None
    flash: Optional[bool] = None

    @staticmethod
    def dense(scale: Optional[float] = None) -> "Plan":
        return Plan(_DENSE, scale)

    @staticmethod
    def masked(scale: Optional[float], mask: Optional[torch.Tensor]) -> "Plan":
        return Plan(_DENSE, scale, mask)

    def fp8_first(self) -> "Plan":
        if self.kind == _DENSE and self.mask is None:
            return Plan(_DENSE, self.scale, None, True)
        return self

    @staticmethod
    def composed(scale: Optional[float], mask: Optional[torch.Tensor]) -> "Plan":
        return Plan(_COMPOSED, scale, mask)

    @staticmethod
    def block_causal(scale: Optional[float], mask: BlockCausal) -> "Plan":
        return Plan(_BLOCK_CAUSAL, scale, causal=mask)

    @staticmethod
    def kv_window() -> "Plan":
        return Plan(_KV_WINDOW)

    @staticmethod
    def kv_window_with(flash: bool) -> "Plan":
        return Plan(_KV_WINDOW, flash=flash)

    def to_c(self) -> _lib.PlanC:
        c = _lib.PlanC()
        c.kind = self.kind
        c.has_scale = int(self.scale is not None)
        c.scale = float(self.scale or 0.0)
        c.has_mask = int(self.mask is not None)
        c.fp8_first = int(self.fp8_first_)
        if self.causal is not None:
            c.block_tokens, c.window, c.sink = self.causal.block_tokens, self.causal.window, self.causal.sink
        c.kv_flash = -1 if self.flash is None else int(self.flash)
        return c


def _stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check_bf16_cuda(name: str, t: torch.Tensor) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor: this package has no CPU path")
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bfloat16 (the reference rounds operands to bf16 under bf16 activations)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous BHSD")


def sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, plan: Plan, *, out_bf16: bool = True,
         probe: Optional[sdpa_rule.Probe] = None) -> torch.Tensor:
    """Scaled dot-product attention over BHSD q [b, h, sq, d], k / v [b, h, sk, d], as `plan` says.
    Returns [b, h, sq, d] (bf16, or f32 with out_bf16=False).  Operands are bf16; three float32 operands are
    rounded to bf16 first and the result comes back as float32 holding bf16-rounded values, as the reference
    does under bf16 activations.  Mixed dtypes are an error.  Asynchronous on the current stream."""
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("sdpa expects BHSD")
    if q.dtype == torch.float32 and k.dtype == torch.float32 and v.dtype == torch.float32:
        # f32-stored activations: operands rounded to bf16 first, the result rounded again and handed back in
        # the caller's storage type (act16_operands and the tail of dense, rt/sdpa.rs:167-181,206-213)
        q16, k16, v16 = act16_operands(q, k, v)
        return act16_widen(sdpa(q16, k16, v16, plan, out_bf16=True, probe=probe))
    for n, t in (("q", q), ("k", k), ("v", v)):
        _check_bf16_cuda(n, t)
    cs4 = ctypes.c_size_t * 4
    pc = plan.to_c()
    pr = probe.to_c() if probe is not None else None
    out = torch.empty(q.shape, dtype=torch.bfloat16 if out_bf16 else torch.float32, device=q.device)
    L = _lib.lib()
    prp = ctypes.byref(pr) if pr is not None else None
    with torch.cuda.device(q.device):
        # A short query block against a long window is cut along the keys when that fills the SMs better.
        L.fv_sdpa_ws_bytes.restype = ctypes.c_size_t
        need = int(L.fv_sdpa_ws_bytes(cs4(*q.shape), cs4(*k.shape), ctypes.byref(pc), prp)) \
            if os.environ.get("FV_SPLITKV", "1") != "0" else 0
        ws = _workspace(q.device, need) if need else None
        rc = L.fv_sdpa_ws(_stream_ptr(), ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()),
                          ctypes.c_void_p(v.data_ptr()), cs4(*q.shape), cs4(*k.shape), cs4(*v.shape),
                          ctypes.byref(pc), prp, ctypes.c_void_p(out.data_ptr()), int(out_bf16),
                          ctypes.c_void_p(ws.data_ptr() if ws is not None else None),
                          ctypes.c_size_t(ws.numel() if ws is not None else 0))
    _lib.check(rc, "sdpa")
    return out


def act16_operands(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
    """bf16-rounded copies of three f32 operands in one launch (act16_operands, rt/sdpa.rs:167-181)."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        if not t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous():
            raise ValueError(f"act16_operands: {n} must be a contiguous CUDA float32 tensor")
    if k.shape != v.shape:
        raise ValueError("act16_operands: k and v differ in shape")
    outs = [torch.empty(t.shape, dtype=torch.bfloat16, device=t.device) for t in (q, k, v)]
    fp = lambda t: ctypes.cast(ctypes.c_void_p(t.data_ptr()), ctypes.POINTER(ctypes.c_float))
    with torch.cuda.device(q.device):
        rc = _lib.lib().fv_act16_operands(_stream_ptr(), fp(q), fp(k), fp(v), ctypes.c_longlong(q.numel()),
                                          ctypes.c_longlong(k.numel()), *[ctypes.c_void_p(o.data_ptr()) for o in outs])
    _lib.check(rc, "act16_operands")
    return tuple(outs)


def act16_widen(x: torch.Tensor) -> torch.Tensor:
    """A bf16 result in f32 storage (the values stay the bf16-rounded ones)."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("act16_widen: a contiguous CUDA bf16 tensor")
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.lib().fv_act16_widen(_stream_ptr(), ctypes.c_void_p(x.data_ptr()), ctypes.c_longlong(x.numel()),
                                       ctypes.cast(ctypes.c_void_p(out.data_ptr()), ctypes.POINTER(ctypes.c_float)))
    _lib.check(rc, "act16_widen")
    return out


def dense_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: Optional[float] = None,
              out_bf16: bool = True, causal: Optional[BlockCausal] = None, q_row0: int = 0,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The kernel-level call (attn_dc::dense_fwd, rt/attn_dc.rs:213-273): q [bh, sq, 128],
    k / v [bh, sk, 128] bf16 -> [bh, sq, 128]."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _check_bf16_cuda(n, t)
    bh, sq, d = q.shape
    sk = k.shape[1]
    if k.shape != (bh, sk, d) or v.shape != k.shape:
        raise ValueError("dense_fwd: k and v must be [bh, sk, d] of q")
    scale = float(scale) if scale is not None else 1.0 / d ** 0.5
    if out is None:
        out = torch.empty((bh, sq, d), dtype=torch.bfloat16 if out_bf16 else torch.float32, device=q.device)
    mode, bt, win, sink = (1, causal.block_tokens, causal.window, causal.sink) if causal else (0, 0, 0, 0)
    with torch.cuda.device(q.device):
        rc = _lib.lib().fv_sdpa_dense_bf16(_stream_ptr(), ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()),
                                           ctypes.c_void_p(v.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                           int(out.dtype == torch.bfloat16), bh, sq, sk, d, ctypes.c_float(scale),
                                           mode, bt, win, sink, q_row0)
    _lib.check(rc, "dense_fwd")
    return out


def dense_fwd_merged(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: Optional[float] = None,
                     out_bf16: bool = True, causal: Optional[BlockCausal] = None) -> torch.Tensor:
    """dense_fwd on BHSD q [b, h, sq, 128], k / v [b, h, sk, 128] with the head merge folded into the store:
    returns [b, sq, h * 128] (what merge_heads gives, rt/ops.rs:2373-2385)."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _check_bf16_cuda(n, t)
    if q.dim() != 4 or k.dim() != 4 or v.shape != k.shape or k.shape[:2] != q.shape[:2] or k.shape[3] != q.shape[3]:
        raise ValueError("sdpa expects BHSD")
    b, h, sq, d = q.shape
    sk = k.shape[2]
    scale = float(scale) if scale is not None else 1.0 / d ** 0.5
    out = torch.empty((b, sq, h * d), dtype=torch.bfloat16 if out_bf16 else torch.float32, device=q.device)
    mode, bt, win, sink = (1, causal.block_tokens, causal.window, causal.sink) if causal else (0, 0, 0, 0)
    with torch.cuda.device(q.device):
        rc = _lib.lib().fv_sdpa_dense_merged_bf16(_stream_ptr(), ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()),
                                                  ctypes.c_void_p(v.data_ptr()), ctypes.c_void_p(out.data_ptr()), int(out_bf16),
                                                  b, h, sq, sk, d, ctypes.c_float(scale), mode, bt, win, sink, 0)
    _lib.check(rc, "dense_fwd_merged")
    return out


_split_ws: dict = {}  # device index -> workspace tensor, grown on demand


def _workspace(device: torch.device, need: int) -> torch.Tensor:
    """One split-KV workspace per device, reused by every call on it (calls on one device share its stream
    order; a caller with several streams passes workspaces of its own to splitkv_fwd)."""
    ws = _split_ws.get(device.index)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device=device)
        _split_ws[device.index] = ws
    return ws


def splitkv_choose(bh: int, sq: int, sk: int, sm_count: int) -> int:
    """How many key ranges the cost model cuts this shape into on a GPU of `sm_count` SMs (1 = no split)."""
    return int(_lib.lib().fv_sdpa_splitkv_choose(bh, sq, sk, sm_count))


def splitkv_workspace_bytes(bh: int, sq: int, splits: int) -> int:
    L = _lib.lib()
    L.fv_sdpa_splitkv_workspace_bytes.restype = ctypes.c_size_t
    return int(L.fv_sdpa_splitkv_workspace_bytes(bh, sq, splits))


def splitkv_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, splits: int, *, scale: Optional[float] = None,
                out_bf16: bool = True, out_heads: int = 0, workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Unmasked attention of a short query block over a long key window (Plan::kv_window, rt/sdpa.rs:122-133) with
    each head's keys cut into `splits` ranges that run side by side: q [bh, sq, 128], k / v [bh, sk, 128] ->
    [bh, sq, 128], or [bh / out_heads, sq, out_heads * 128] with out_heads > 0."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _check_bf16_cuda(n, t)
    bh, sq, d = q.shape
    sk = k.shape[1]
    if k.shape != (bh, sk, d) or v.shape != k.shape:
        raise ValueError("splitkv_fwd: k and v must be [bh, sk, d] of q")
    scale = float(scale) if scale is not None else 1.0 / d ** 0.5
    if workspace is None:
        workspace = _workspace(q.device, splitkv_workspace_bytes(bh, sq, splits))
    shape = (bh // out_heads, sq, out_heads * d) if out_heads > 0 else (bh, sq, d)
    out = torch.empty(shape, dtype=torch.bfloat16 if out_bf16 else torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        rc = _lib.lib().fv_sdpa_splitkv_bf16(_stream_ptr(), ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()),
                                             ctypes.c_void_p(v.data_ptr()), ctypes.c_void_p(out.data_ptr()), int(out_bf16),
                                             bh, sq, sk, d, ctypes.c_float(scale), int(splits), int(out_heads),
                                             ctypes.c_void_p(workspace.data_ptr()), ctypes.c_size_t(workspace.numel()))
    _lib.check(rc, "splitkv_fwd")
    return out


def device_status() -> int:
    """Synchronises the current stream and returns the kernels' status word (0 = every bounded wait
    completed); raises FvError when a kernel gave up."""
    code = ctypes.c_int(0)
    rc = _lib.lib().fv_device_status(_stream_ptr(), ctypes.byref(code))
    _lib.check(rc, "device_status")
    return code.value
