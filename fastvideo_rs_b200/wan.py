"""The Wan caller side of the path: 3-D RoPE tables, the fused q/k RMSNorm + RoPE + head-split
prologue, and the self-attention forward that strings them to sdpa() -- the slice of
WanAttention::{qk, attend, forward_self} (crates/fastvideo-cudarc/src/wan/transformer.rs:163-349)
between the QKV projection and the output projection."""
from __future__ import annotations

import ctypes
from typing import NamedTuple, Optional, Tuple

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
            want_q: bool = True, want_k: bool = True, want_v: bool = True, cache=None):
    """RMSNorm * w, RoPE, head split of q and k (and the head split of v) in one pass over the fused
    projection `proj` [batch, seq, width] bf16.  Default column layout is [q | k | v].  Returns
    (q, k, v) as [batch, heads, seq, 128] bf16 tensors (None for the ones not asked for).
    cache = (k_cache, v_cache, row0): K and V of the block go straight into rows [row0, row0 + seq) of the
    [batch, heads, cache_rows, 128] bf16 cache tensors (the append of wan/causal.rs:541-628 without its two
    copies); k and v of the result are then views of those rows."""
    if not proj.is_cuda or proj.dtype != torch.bfloat16 or not proj.is_contiguous() or proj.dim() != 3:
        raise ValueError("qk_prep: proj must be a contiguous CUDA bf16 [batch, seq, width] tensor")
    b, seq, width = proj.shape
    d = 128
    dim = heads * d
    col_k = dim if col_k is None else col_k
    col_v = 2 * dim if col_v is None else col_v
    mk = lambda want: torch.empty((b, heads, seq, d), dtype=torch.bfloat16, device=proj.device) if want else None
    ptr = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
    if cache is not None:
        kc, vc, row0 = cache
        for n, t in (("k_cache", kc), ("v_cache", vc)):
            if t.dtype != torch.bfloat16 or not t.is_cuda or not t.is_contiguous() or t.dim() != 4 or \
                    t.shape[0] != b or t.shape[1] != heads or t.shape[3] != d:
                raise ValueError(f"qk_prep: {n} must be a contiguous CUDA bf16 [batch, heads, rows, 128] tensor")
        if kc.shape != vc.shape:
            raise ValueError("qk_prep: k_cache and v_cache differ in shape")
        q = mk(want_q)
        for name, t in (("wq", wq), ("wk", wk), ("cos", cos), ("sin", sin)):
            if t is not None and (t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous()):
                raise ValueError(f"qk_prep: {name} must be a contiguous CUDA float32 tensor")
        fp = lambda t: ctypes.cast(ctypes.c_void_p(t.data_ptr()), _f32p) if t is not None else None
        with torch.cuda.device(proj.device):
            rc = _lib.lib().fv_wan_qk_prep_cache_bf16(_stream_ptr(), ptr(proj), width, col_q, col_k, col_v, fp(wq), fp(wk),
                                                      fp(cos), fp(sin), b, seq, heads, d, ctypes.c_float(eps), norm_scope,
                                                      ptr(q), ptr(kc), ptr(vc), kc.shape[2], int(row0))
        _lib.check(rc, "qk_prep (cache)")
        return q, kc[:, :, row0:row0 + seq], vc[:, :, row0:row0 + seq]
    q, k, v = mk(want_q), mk(want_k), mk(want_v)
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
    """WanAttention without its GEMMs (wan/transformer.rs:163-445): projections in, attention out.

    grid: token grid in patches (frames, height, width); heads x 128 = model dim.  causal: optional
    BlockCausal (Self-Forcing chunk-causal mask).  vsa: optional vsa.VsaCtx of the same grid -- forward_self
    then takes the VSA route (attend_vsa) and needs the gate projection."""

    def __init__(self, grid, heads: int, wq: torch.Tensor, wk: torch.Tensor, eps: float = 1e-6,
                 theta: float = 10000.0, causal: Optional[BlockCausal] = None, device="cuda", vsa=None):
        self.grid, self.heads, self.eps, self.causal, self.vsa = tuple(grid), heads, eps, causal, vsa
        self.wq, self.wk = wq, wk
        self.cos, self.sin = wan_rope_tables(grid, 128, theta, 0, device)

    def forward_self(self, qkv: torch.Tensor, scale: Optional[float] = None, gate: Optional[torch.Tensor] = None,
                     merged: bool = False) -> torch.Tensor:
        """forward_self (wan/transformer.rs:265-349) between the QKV projection and the output projection.
        qkv [batch, seq, 3 * dim] bf16; gate [batch, seq, dim] bf16 (the gate projection) with a VSA context.
        merged: return [batch, seq, dim] (merge_heads folded into the store) instead of BHSD."""
        q, k, v = qk_prep(qkv, self.wq, self.wk, self.cos, self.sin, self.heads, eps=self.eps)
        if self.vsa is not None:
            if gate is None:
                raise ValueError("forward_self: the VSA route needs the gate projection")
            out = self.attend_vsa(q, k, v, gate)
            return out.permute(0, 2, 1, 3).reshape(out.shape[0], out.shape[2], -1) if merged else out
        if merged:
            from .sdpa import dense_fwd_merged
            return dense_fwd_merged(q, k, v, scale=scale, causal=self.causal)
        plan = Plan.block_causal(scale, self.causal) if self.causal is not None else Plan.dense(scale)
        return sdpa(q, k, v, plan)

    def attend_vsa(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate_proj: torch.Tensor) -> torch.Tensor:
        """attend_vsa (wan/transformer.rs:354-390): q, k normed and roped, v split, BHSD; the gate is the gate
        projection split into heads with no norm and no rotation (wan/transformer.rs:336-347), linear."""
        from . import vsa as _vsa
        b, h, seq, d = q.shape
        if gate_proj.shape != (b, seq, h * d):
            raise ValueError(f"attend_vsa: gate projection {tuple(gate_proj.shape)} for {tuple(q.shape)}")
        # head split of the gate: the prologue kernel's V path is exactly that copy
        _, _, g = qk_prep(gate_proj, None, None, None, None, h, col_q=0, col_k=0, col_v=0, want_q=False, want_k=False)
        out = _vsa.vsa_attention(q.view(b * h, seq, d), k.view(b * h, seq, d), v.view(b * h, seq, d), g.view(b * h, seq, d), self.vsa)
        return out.view(b, h, seq, d)

    def cross_kv(self, kv_proj: torch.Tensor, wk: Optional[torch.Tensor] = None):
        """cross_kv (wan/transformer.rs:406-419): the text tokens' fused K|V projection [batch, text, 2 * dim] ->
        (RMS-normed K without rotation, V), both BHSD bf16 -- the layout the attention kernel reads, computed
        once per denoise and cached by the caller."""
        dim = self.heads * 128
        _, k, v = qk_prep(kv_proj, None, wk if wk is not None else self.wk, None, None, self.heads, col_q=0, col_k=0, col_v=dim,
                          eps=self.eps, want_q=False)
        return k, v

    def forward_cross(self, q_proj: torch.Tensor, cached_kv, scale: Optional[float] = None, merged: bool = False) -> torch.Tensor:
        """forward_cross (wan/transformer.rs:420-444): q = RMSNorm(q projection) without rotation, attention over
        the cached text K / V.  q_proj [batch, seq, dim] bf16."""
        q, _, _ = qk_prep(q_proj, self.wq, None, None, None, self.heads, col_q=0, col_k=0, col_v=0, eps=self.eps,
                          want_k=False, want_v=False)
        k, v = cached_kv
        if merged:
            from .sdpa import dense_fwd_merged
            return dense_fwd_merged(q, k, v, scale=scale)
        return sdpa(q, k, v, Plan.dense(scale))


def rope_bhsd(src: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, dst: torch.Tensor, *, src_row0: int = 0,
              dst_row0: int = 0, negate_sin: bool = False) -> torch.Tensor:
    """Wan's interleaved RoPE over rows of BHSD tensors (rope_bhsd_f32 / rope_bhsd, wan/causal.rs:246-275, and the
    copy_tokens that follows it in KvRope::RebasedSink, :734-812): rows [src_row0, src_row0 + n) of src
    [b, h, rows, 128] (bf16 or f32) rotated with table rows 0 .. n-1 of cos / sin [n, 128] f32 into rows
    [dst_row0, dst_row0 + n) of dst (bf16 or f32).  negate_sin rotates back.  Returns dst."""
    n = cos.shape[0]
    for name, t in (("src", src), ("dst", dst)):
        if not t.is_cuda or t.dtype not in (torch.bfloat16, torch.float32) or not t.is_contiguous() or t.dim() != 4 or t.shape[3] != 128:
            raise ValueError(f"rope_bhsd: {name} must be a contiguous CUDA bf16 or float32 [b, h, rows, 128] tensor")
    if src.shape[:2] != dst.shape[:2] or cos.shape != (n, 128) or sin.shape != (n, 128):
        raise ValueError("rope_bhsd: shapes")
    for name, t in (("cos", cos), ("sin", sin)):
        if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"rope_bhsd: {name} must be a contiguous CUDA float32 tensor")
    fp = lambda t: ctypes.cast(ctypes.c_void_p(t.data_ptr()), _f32p)
    with torch.cuda.device(src.device):
        rc = _lib.lib().fv_wan_rope_bhsd(_stream_ptr(), ctypes.c_void_p(src.data_ptr()), int(src.dtype == torch.bfloat16),
                                         src.shape[2], int(src_row0), fp(cos), fp(sin), int(negate_sin),
                                         src.shape[0] * src.shape[1], n, ctypes.c_void_p(dst.data_ptr()),
                                         int(dst.dtype == torch.bfloat16), dst.shape[2], int(dst_row0))
    _lib.check(rc, "rope_bhsd")
    return dst


class _KvSpecC(ctypes.Structure):
    _fields_ = [("frame_tokens", ctypes.c_int), ("capacity", ctypes.c_int), ("sink", ctypes.c_int),
                ("max_attention", ctypes.c_int), ("rolling", ctypes.c_int)]


class _KvMoveC(ctypes.Structure):
    _fields_ = [("evicted", ctypes.c_longlong), ("local_start", ctypes.c_longlong), ("local_end", ctypes.c_longlong),
                ("window_start", ctypes.c_longlong)]


class KvMove(NamedTuple):
    """Where the cache pointers moved for one write (KvMove, wan/causal.rs:276-287)."""
    evicted: int
    local_start: int
    local_end: int
    window_start: int


class KvSpec:
    """Token geometry of one causal K/V cache (KvSpec, wan/causal.rs:38-147): tokens per latent frame, rows of a
    cache plane, rows kept at the head when it rolls, keys a block reads back from its end, and whether it rolls
    (local_attn_size given) or refuses clips longer than its window."""

    def __init__(self, frame_tokens: int, capacity: int, sink: int, max_attention: int, rolling: bool):
        self.frame_tokens, self.capacity, self.sink = int(frame_tokens), int(capacity), int(sink)
        self.max_attention, self.rolling = int(max_attention), bool(rolling)

    @staticmethod
    def rolling_window(frame_tokens: int, local_attn_frames: int, sink_frames: int) -> "KvSpec":
        """KvSpec::rolling (wan/causal.rs:110-133): a cache of local_attn_frames frames that keeps the first
        sink_frames frames when it rolls."""
        if local_attn_frames == 0 or sink_frames >= local_attn_frames:
            raise ValueError(f"causal kv: sink {sink_frames} frames must be below the window ({local_attn_frames} frames)")
        n = local_attn_frames * frame_tokens
        return KvSpec(frame_tokens, n, sink_frames * frame_tokens, n, True)

    @staticmethod
    def global_window(frame_tokens: int, frames: int = 21, sink_frames: int = 0) -> "KvSpec":
        """local_attn_size == -1 (KvSpec::for_config, wan/causal.rs:80-107): sliding_window_num_frames frames, no roll."""
        n = frames * frame_tokens
        return KvSpec(frame_tokens, n, sink_frames * frame_tokens, n, False)

    def window_frames(self) -> int:
        return self.max_attention // max(self.frame_tokens, 1)

    def sink_target(self, end_frame: int) -> int:
        """First frame the sink keys should sit at once the write that ends at end_frame is done (wan/causal.rs:136-138)."""
        return max(end_frame - self.window_frames(), 0)

    def plan(self, global_end: int, local_end_prev: int, current_start: int, n: int) -> KvMove:
        """KvSpec::plan (wan/causal.rs:289-336) through the library (host arithmetic, no device needed)."""
        c = _KvSpecC(self.frame_tokens, self.capacity, self.sink, self.max_attention, int(self.rolling))
        mv = _KvMoveC()
        rc = _lib.lib().fv_kv_plan(ctypes.byref(c), ctypes.c_longlong(global_end), ctypes.c_longlong(local_end_prev),
                                   ctypes.c_longlong(current_start), ctypes.c_longlong(n), ctypes.byref(mv))
        _lib.check(rc, "kv plan")
        return KvMove(mv.evicted, mv.local_start, mv.local_end, mv.window_start)


class CausalKvCache:
    """One layer's causal K/V cache as persistent buffers (CausalKvCache in static mode, wan/causal.rs:338-730):
    k, v [batch, heads, capacity, 128] bf16 written in place, the pointers (global_end, local_end) on the host.
    A block is planned (KvSpec.plan), the cache rolled past its sink when full (fv_kv_roll), the block written at
    [local_start, local_end) -- by `update` from BHSD tensors like the reference, or by `prep` straight out of the
    prologue kernel -- and its queries attend to rows [window_start, local_end) in place (`attend`,
    Plan::kv_window)."""

    def __init__(self, spec: KvSpec, batch: int, heads: int, device="cuda"):
        self.spec, self.batch, self.heads = spec, batch, heads
        self.k = torch.zeros((batch, heads, spec.capacity, 128), dtype=torch.bfloat16, device=device)
        self.v = torch.zeros_like(self.k)
        self.global_end = self.local_end = 0
        self.last: Optional[KvMove] = None
        self.raw_sink: Optional[torch.Tensor] = None  # KvRope::RebasedSink: the sink keys without RoPE (f32), taken once
        self.sink_at = 0                              # first frame the cached sink keys are roped at now

    def __len__(self) -> int:
        return self.local_end

    def reset(self) -> None:
        self.global_end = self.local_end = 0
        self.last = None
        self.raw_sink, self.sink_at = None, 0

    def rebase_sink(self, target: int, orig, new) -> None:
        """CausalKvCache::rebase_sink (wan/causal.rs:734-812): re-rope the sink keys to start at frame `target`
        (KvSpec.sink_target).  orig = (cos, sin) tables of the sink's own frames 0 .. sink (to take the un-roped copy
        the first time, by rotating back), new = those of frames target .. target + sink ([sink_tokens, 128] f32
        each).  Two launches of the BHSD rope kernel, the second writing the cache head in place; a no-op when the
        sink is already there."""
        sink = self.spec.sink
        if sink == 0 or self.local_end < sink or self.sink_at == target:
            return
        if self.raw_sink is None:
            self.raw_sink = torch.empty((self.batch, self.heads, sink, 128), dtype=torch.float32, device=self.k.device)
            rope_bhsd(self.k, orig[0], orig[1], self.raw_sink, negate_sin=True)
        rope_bhsd(self.raw_sink, new[0], new[1], self.k)
        self.sink_at = target

    def _advance(self, current_start: int, n: int) -> KvMove:
        mv = self.spec.plan(self.global_end, self.local_end, current_start, n)
        if mv.evicted > 0:
            for t in (self.k, self.v):
                with torch.cuda.device(t.device):
                    rc = _lib.lib().fv_kv_roll(_stream_ptr(), ctypes.c_void_p(t.data_ptr()), 2, self.batch * self.heads,
                                               self.spec.capacity, self.spec.sink, int(mv.evicted), self.local_end)
                _lib.check(rc, "kv roll")
        return mv

    def _commit(self, mv: KvMove, current_start: int, n: int) -> None:
        self.global_end, self.local_end, self.last = current_start + n, mv.local_end, mv

    def update(self, k: torch.Tensor, v: torch.Tensor, current_start: int):
        """CausalKvCache::update (wan/causal.rs:541-628): write a block's roped K and V [batch, heads, n, 128] at
        rollout position current_start; returns the (k, v) windows its queries read, as views of the cache."""
        n = k.shape[2]
        mv = self._advance(current_start, n)
        self.k[:, :, mv.local_start:mv.local_end].copy_(k)
        self.v[:, :, mv.local_start:mv.local_end].copy_(v)
        self._commit(mv, current_start, n)
        return self.k[:, :, mv.window_start:mv.local_end], self.v[:, :, mv.window_start:mv.local_end]

    def prep(self, proj: torch.Tensor, wq, wk, cos, sin, current_start: int, eps: float = 1e-6) -> torch.Tensor:
        """The block's fused QKV projection [batch, n, 3 * dim] through the prologue kernel with K and V landing in
        the cache rows of the block (no copy launches); returns q [batch, heads, n, 128].  cos / sin: the table rows
        of the block's own frames."""
        n = proj.shape[1]
        mv = self._advance(current_start, n)
        q, _, _ = qk_prep(proj, wq, wk, cos, sin, self.heads, eps=eps, cache=(self.k, self.v, mv.local_start))
        self._commit(mv, current_start, n)
        return q

    def attend(self, q: torch.Tensor, scale: Optional[float] = None, merged: bool = False) -> torch.Tensor:
        """Plan::kv_window over the cache (rt/sdpa.rs:122-133; wan/transformer.rs:290-313): the block's queries
        [batch, heads, n, 128] against rows [window_start, local_end) of the cache, read in place."""
        if self.last is None:
            raise ValueError("attend: nothing has been written to the cache")
        if q.dtype != torch.bfloat16 or not q.is_cuda or not q.is_contiguous() or q.dim() != 4 or q.shape[:2] != (self.batch, self.heads):
            raise ValueError("attend: q must be a contiguous CUDA bf16 [batch, heads, n, 128] tensor")
        b, h, n, d = q.shape
        scale = float(scale) if scale is not None else 1.0 / d ** 0.5
        out = torch.empty((b, n, h * d) if merged else (b, h, n, d), dtype=torch.bfloat16, device=q.device)
        ws, we = self.last.window_start, self.last.local_end
        with torch.cuda.device(q.device):
            rc = _lib.lib().fv_sdpa_window_bf16(_stream_ptr(), ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(self.k.data_ptr()),
                                                ctypes.c_void_p(self.v.data_ptr()), ctypes.c_void_p(out.data_ptr()), 1, b * h, n,
                                                self.spec.capacity, int(ws), int(we - ws), d, ctypes.c_float(scale),
                                                h if merged else 0)
        _lib.check(rc, "sdpa window")
        return out


def ln_adaln_e(x: torch.Tensor, e: torch.Tensor, scale_slot: int, shift_slot: int, eps: float = 1e-6) -> torch.Tensor:
    """CudaTensor::ln_adaln_e under bf16 activations (rt/fused.rs:20-70), the pass before attention:
    x [batch, seq, dim] bf16, e [batch, e_rows, dim] f32 -> bf16(LN(x) * (1 + e[b, scale]) + e[b, shift])."""
    if x.dtype != torch.bfloat16 or not x.is_cuda or not x.is_contiguous() or x.dim() != 3:
        raise ValueError("ln_adaln_e: x must be a contiguous CUDA bf16 [batch, seq, dim] tensor")
    b, seq, dim = x.shape
    if e.dtype != torch.float32 or not e.is_cuda or not e.is_contiguous() or e.dim() != 3 or e.shape[0] != b or e.shape[2] != dim:
        raise ValueError(f"ln_adaln_e: table {tuple(e.shape)} for {tuple(x.shape)}")
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        rc = _lib.lib().fv_wan_ln_adaln_bf16(_stream_ptr(), ctypes.c_void_p(x.data_ptr()),
                                             ctypes.cast(ctypes.c_void_p(e.data_ptr()), _f32p), scale_slot, shift_slot, b, seq, dim,
                                             e.shape[1], ctypes.c_float(eps), ctypes.c_void_p(out.data_ptr()))
    _lib.check(rc, "ln_adaln_e")
    return out


def self_residual_norm(hidden: torch.Tensor, attn: torch.Tensor, e: torch.Tensor, gate_slot: int, w: torch.Tensor,
                       b: torch.Tensor, eps: float = 1e-6):
    """wan::fuse::self_residual_norm (wan/fuse.rs:108-166), the pass after attention: returns
    (bf16(hidden + attn * e[b, gate]), bf16(LayerNorm(that sum, unrounded) * w + b))."""
    for n, t in (("hidden", hidden), ("attn", attn)):
        if t.dtype != torch.bfloat16 or not t.is_cuda or not t.is_contiguous() or t.dim() != 3:
            raise ValueError(f"self_residual_norm: {n} must be a contiguous CUDA bf16 [batch, seq, dim] tensor")
    bt, seq, dim = hidden.shape
    if attn.shape != hidden.shape or e.dtype != torch.float32 or e.shape[0] != bt or e.shape[2] != dim or not e.is_contiguous():
        raise ValueError("self_residual_norm: shapes")
    for n, t in (("w", w), ("b", b)):
        if t.dtype != torch.float32 or not t.is_cuda or t.numel() != dim or not t.is_contiguous():
            raise ValueError(f"self_residual_norm: {n} must be CUDA float32 [dim]")
    hid, normed = torch.empty_like(hidden), torch.empty_like(hidden)
    fp = lambda t: ctypes.cast(ctypes.c_void_p(t.data_ptr()), _f32p)
    with torch.cuda.device(hidden.device):
        rc = _lib.lib().fv_wan_self_residual_norm_bf16(_stream_ptr(), ctypes.c_void_p(hidden.data_ptr()), ctypes.c_void_p(attn.data_ptr()),
                                                       fp(e), gate_slot, fp(w), fp(b), bt, seq, dim, e.shape[1], ctypes.c_float(eps),
                                                       ctypes.c_void_p(hid.data_ptr()), ctypes.c_void_p(normed.data_ptr()))
    _lib.check(rc, "self_residual_norm")
    return hid, normed


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
