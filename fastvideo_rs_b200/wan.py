"""The Wan caller side of the path: 3-D RoPE tables, the fused q/k RMSNorm + RoPE + head-split
prologue, and the self-attention forward that strings them to sdpa() -- the slice of
WanAttention::{qk, attend, forward_self} (crates/fastvideo-cudarc/src/wan/transformer.rs:163-349)
between the QKV projection and the output projection."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import numpy as np
import torch

from . import _lib
from .sdpa import BlockCausal, Plan, _stream_ptr, sdpa

NORM_ACROSS_HEADS, NORM_PER_HEAD = 0, 1
_f32p = ctypes.POINTER(ctypes.c_float)


def wan_rope_tables_host(grid: Tuple[int, int, int], d: int = 128, theta: float = 10000.0,
                         start_frame: int = 0) -> Tuple[np.ndarray, np.ndarray]:
    """cos, sin [ppf*pph*ppw, d] f32 on the host (wan_rope_at, wan/transformer.rs:490-544)."""
    ppf, pph, ppw = grid
    seq = ppf * pph * ppw
    cos = np.empty((seq, d), np.float32)
    sin = np.empty((seq, d), np.float32)
    rc = _lib.lib().fv_wan_rope_tables(ppf, pph, ppw, d, ctypes.c_double(theta), start_frame,
                                       cos.ctypes.data_as(_f32p), sin.ctypes.data_as(_f32p))
    _lib.check(rc, "wan_rope_tables")
    return cos, sin


def wan_rope_tables(grid, d: int = 128, theta: float = 10000.0, start_frame: int = 0, device="cuda"):
    """The tables uploaded once per grid (the reference caches them per grid, wan/transformer.rs:2221-2244)."""
    cos, sin = wan_rope_tables_host(grid, d, theta, start_frame)
    return torch.from_numpy(cos).to(device), torch.from_numpy(sin).to(device)


def qk_prep(proj: torch.Tensor, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], cos: Optional[torch.Tensor],
            sin: Optional[torch.Tensor], heads: int, col_q: int = 0, col_k: Optional[int] = None,
            col_v: Optional[int] = None, eps: float = 1e-6, norm_scope: int = NORM_ACROSS_HEADS,
            want_q: bool = True, want_k: bool = True, want_v: bool = True):
    """RMSNorm * w, RoPE, head split of q and k (and the head split of v) in one pass over the fused
    projection `proj` [batch, seq, width] bf16.  Default column layout is [q | k | v].  Returns
    (q, k, v) as [batch, heads, seq, 128] bf16 tensors (None for the ones not asked for)."""
    if not proj.is_cuda or proj.dtype != torch.bfloat16 or not proj.is_contiguous() or proj.dim() != 3:
        raise ValueError("qk_prep: proj must be a contiguous CUDA bf16 [batch, seq, width] tensor")
    b, seq, width = proj.shape
    d = 128
    dim = heads * d
    col_k = dim if col_k is None else col_k
    col_v = 2 * dim if col_v is None else col_v
    mk = lambda want: torch.empty((b, heads, seq, d), dtype=torch.bfloat16, device=proj.device) if want else None
    q, k, v = mk(want_q), mk(want_k), mk(want_v)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
    fptr = lambda t: ctypes.cast(ctypes.c_void_p(t.data_ptr()), _f32p) if t is not None else None
    for name, t in (("wq", wq), ("wk", wk), ("cos", cos), ("sin", sin)):
        if t is not None and (t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous()):
            raise ValueError(f"qk_prep: {name} must be a contiguous CUDA float32 tensor")
    with torch.cuda.device(proj.device):
        rc = _lib.lib().fv_wan_qk_prep_bf16(_stream_ptr(), ptr(proj), width, col_q, col_k, col_v, fptr(wq), fptr(wk),
                                            fptr(cos), fptr(sin), b, seq, heads, d, ctypes.c_float(eps), norm_scope,
                                            ptr(q), ptr(k), ptr(v))
    _lib.check(rc, "qk_prep")
    return q, k, v


class WanSelfAttention:
    """forward_self without the two GEMMs: fused QKV projection in, attention out (BHSD).

    grid: token grid in patches (frames, height, width); heads x 128 = model dim.  causal: optional
    BlockCausal (Self-Forcing chunk-causal mask)."""

    def __init__(self, grid, heads: int, wq: torch.Tensor, wk: torch.Tensor, eps: float = 1e-6,
                 theta: float = 10000.0, causal: Optional[BlockCausal] = None, device="cuda"):
        self.grid, self.heads, self.eps, self.causal = tuple(grid), heads, eps, causal
        self.wq, self.wk = wq, wk
        self.cos, self.sin = wan_rope_tables(grid, 128, theta, 0, device)

    def forward_self(self, qkv: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
        q, k, v = qk_prep(qkv, self.wq, self.wk, self.cos, self.sin, self.heads, eps=self.eps)
        plan = Plan.block_causal(scale, self.causal) if self.causal is not None else Plan.dense(scale)
        return sdpa(q, k, v, plan)


class HostStaged:
    """Runs a device step over a sequence of HOST batches with the copies off the critical path: inputs come
    from pinned host tensors, results go back to pinned host tensors, and while step i computes, the input of
    step i + 1 is already arriving and the result of step i - 1 is leaving -- two device buffers each way, one
    stream for host-to-device copies, one for device-to-host copies, events in between.  This is what the
    denoising loop does around attention when its activations live on the host (offload), and what the
    benchmark's end-to-end leg measures.

    step(dev_in) -> dev_out runs on the current stream and may return a view of a buffer it reuses: the result
    is copied into this object's own output buffer on the compute stream before the next step starts."""

    def __init__(self, in_shape, out_shape, device, dtype=torch.bfloat16):
        self.device = device
        self.h2d, self.d2h = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
        self.dev_in = [torch.empty(in_shape, dtype=dtype, device=device) for _ in range(2)]
        self.dev_out = [torch.empty(out_shape, dtype=dtype, device=device) for _ in range(2)]

    def run(self, host_ins, host_outs, step):
        """host_ins / host_outs: equally long lists of pinned host tensors (entries may repeat)."""
        cur = torch.cuda.current_stream(self.device)
        n = len(host_ins)
        arrived = [None, None]   # input buffer i % 2 holds batch i
        consumed = [None, None]  # ... and the step that read it has finished
        left = [None, None]      # output buffer i % 2 has been copied out

        def fetch(i):
            with torch.cuda.stream(self.h2d):
                if consumed[i & 1] is not None:
                    self.h2d.wait_event(consumed[i & 1])
                self.dev_in[i & 1].copy_(host_ins[i], non_blocking=True)
                arrived[i & 1] = torch.cuda.Event()
                arrived[i & 1].record(self.h2d)

        if n:
            fetch(0)
        for i in range(n):
            if i + 1 < n:
                fetch(i + 1)
            cur.wait_event(arrived[i & 1])
            out = step(self.dev_in[i & 1])
            consumed[i & 1] = torch.cuda.Event()
            consumed[i & 1].record(cur)
            if left[i & 1] is not None:
                cur.wait_event(left[i & 1])
            self.dev_out[i & 1].view(-1)[: out.numel()].copy_(out.reshape(-1))
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_event(done)
                host_outs[i].view(-1)[: out.numel()].copy_(self.dev_out[i & 1].view(-1)[: out.numel()], non_blocking=True)
                left[i & 1] = torch.cuda.Event()
                left[i & 1].record(self.d2h)
        for ev in left:
            if ev is not None:
                cur.wait_event(ev)
