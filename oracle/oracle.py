"""TEST INFRASTRUCTURE, NOT PRODUCT.

Python face of the CPU oracle: ctypes bindings of ``libfvoracle.so`` (built from
``fv_oracle.cpp`` by ``oracle/Makefile``) plus a few pure-numpy twins used to cross-check
the C++ restatement on small cases, and the seeded input generator shared by tests and
bench.  Only ``tests/``, ``__graft_entry__.smoke`` and the CPU-baseline leg of ``bench.py``
may import this module; the library under test never does.

Reference lines restated are cited next to each C++ function in ``fv_oracle.cpp`` and, for
the numpy twins, below (paths inside zaitrarrio/fastvideo-rs, ``C/`` =
``crates/fastvideo-cudarc/src/``).

Parity pin: the reference keeps no golden tensors for this path; its closed-form unit tests
are re-run against this oracle by ``tests/test_oracle_kat.py``.  Cases seeded by the
reference's ``rand`` crate streams (fv-gpucheck) are not reproducible here and stay
"parity unpinned"; inputs come from :func:`seeded_normal` instead.
"""
from __future__ import annotations

import ctypes
import math
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libfvoracle.so"
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_i32p = ctypes.POINTER(ctypes.c_int32)
_u32p = ctypes.POINTER(ctypes.c_uint32)
_u16p = ctypes.POINTER(ctypes.c_uint16)


def build(force: bool = False) -> Path:
    """Compile the oracle with g++ (no GPU involved)."""
    src = _HERE / "fv_oracle.cpp"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "libfvoracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        _lib.fvo_topk_for.restype = ctypes.c_int
        _lib.fvo_topk_for.argtypes = [ctypes.c_double, ctypes.c_int]
        _lib.fvo_tile_plan.restype = ctypes.c_int
        _lib.fvo_num_threads.restype = ctypes.c_int
    return _lib


def _p(a: np.ndarray, typ):
    return a.ctypes.data_as(typ)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


# --------------------------------------------------------------------------- inputs
def seeded_normal(seed: int, tensor_index: int, shape) -> np.ndarray:
    """i.i.d. N(0,1) float32 from a counter-based generator (numpy Philox, key = seed,
    stream = tensor_index).  The same (seed, tensor_index, shape) always gives the same
    values on any machine."""
    bitgen = np.random.Philox(key=int(seed) + (int(tensor_index) << 32))
    return np.random.Generator(bitgen).standard_normal(size=shape, dtype=np.float32)


def bf16_round(x) -> np.ndarray:
    """Round to bf16 (nearest even, NaN kept quiet) and widen back to f32."""
    x = _f32(x)
    y = np.empty_like(x)
    lib().fvo_bf16_round(_p(x, _f32p), _p(y, _f32p), ctypes.c_size_t(x.size))
    return y


def bf16_round_np(x) -> np.ndarray:
    """numpy twin of the rounding in C/rt/kernels/core.cu:2-15."""
    u = _f32(x).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    r = np.where(nan, (u >> 16) | 0x40, r).astype(np.uint32) << 16
    return r.astype(np.uint32).view(np.float32).reshape(np.shape(x))


def to_bf16_bits(x) -> np.ndarray:
    x = _f32(x)
    y = np.empty(x.shape, dtype=np.uint16)
    lib().fvo_f32_to_bf16(_p(x, _f32p), _p(y, _u16p), ctypes.c_size_t(x.size))
    return y


def from_bf16_bits(h) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    y = np.empty(h.shape, dtype=np.float32)
    lib().fvo_bf16_to_f32(_p(h, _u16p), _p(y, _f32p), ctypes.c_size_t(h.size))
    return y


# --------------------------------------------------------------------------- rope / norm
def wan_rope(ppf: int, pph: int, ppw: int, d: int = 128, theta: float = 10000.0, start_frame: int = 0):
    """cos, sin tables [ppf*pph*ppw, d] (C/wan/transformer.rs:447-544)."""
    seq = ppf * pph * ppw
    c = np.empty((seq, d), np.float32)
    s = np.empty((seq, d), np.float32)
    lib().fvo_wan_rope(ppf, pph, ppw, d, ctypes.c_double(theta), start_frame, _p(c, _f32p), _p(s, _f32p))
    return c, s


def wan_rope_np(ppf, pph, ppw, d=128, theta=10000.0, start_frame=0):
    """numpy twin of wan_rope (same rounding points)."""
    h_dim = 2 * (d // 6)
    w_dim = h_dim
    t_dim = d - h_dim - w_dim

    def rot(dim, seq):
        half = dim // 2
        i = np.arange(half, dtype=np.float64)
        freq = (1.0 / np.power(theta, 2.0 * i / dim)).astype(np.float32)
        arg = (np.arange(seq, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32)
        return np.repeat(np.cos(arg), 2, axis=1).astype(np.float32), np.repeat(np.sin(arg), 2, axis=1).astype(np.float32)

    ct, st = rot(t_dim, start_frame + ppf)
    ch, sh = rot(h_dim, pph)
    cw, sw = rot(w_dim, ppw)
    ft, fh, fw = np.meshgrid(np.arange(start_frame, start_frame + ppf), np.arange(pph), np.arange(ppw), indexing="ij")
    ft, fh, fw = ft.ravel(), fh.ravel(), fw.ravel()
    return (np.concatenate([ct[ft], ch[fh], cw[fw]], axis=1), np.concatenate([st[ft], sh[fh], sw[fw]], axis=1))


def qk_norm_rope_bhsd(src, w, cos, sin, batch, seq, heads, d, src_width, col_off, eps=1e-6, per_head=False):
    """RMSNorm over the heads*d row (or one head) times w, RoPE, -> [batch*heads, seq, d]
    (C/rt/ops.rs:2304-2350)."""
    src = _f32(src)
    w = _f32(w)
    out = np.empty((batch * heads, seq, d), np.float32)
    cp = _p(_f32(cos), _f32p) if cos is not None else None
    sp = _p(_f32(sin), _f32p) if sin is not None else None
    if cos is not None:
        cos_c, sin_c = _f32(cos), _f32(sin)
        cp, sp = _p(cos_c, _f32p), _p(sin_c, _f32p)
    lib().fvo_qk_norm_rope_bhsd(_p(src, _f32p), _p(w, _f32p), cp, sp, batch, seq, heads, d, src_width, col_off,
                                ctypes.c_float(eps), 1 if per_head else 0, _p(out, _f32p))
    return out


def split_heads_bhsd(src, batch, seq, heads, d, src_width, col_off):
    src = _f32(src)
    out = np.empty((batch * heads, seq, d), np.float32)
    lib().fvo_split_heads_bhsd(_p(src, _f32p), batch, seq, heads, d, src_width, col_off, _p(out, _f32p))
    return out


# --------------------------------------------------------------------------- masks
def block_causal_allows(bt: int, window: int, sink: int, q: int, k: int) -> bool:
    """BlockCausal::allows (C/rt/attn.rs:448-453)."""
    bt = max(bt, 1)
    tq, tk = q // bt, k // bt
    return (tk <= tq and (window == 0 or tq - tk < window)) or tk < sink


def block_causal_mask(bt, window, sink, sq, sk) -> np.ndarray:
    m = np.empty((sq, sk), np.float32)
    lib().fvo_block_causal_mask(bt, window, sink, sq, sk, _p(m, _f32p))
    return m


def causal_temporal_mask(seq, frame_tokens, frames_per_block, local_attn_size) -> np.ndarray:
    """crates/fastvideo-models/src/wan/family.rs:80-109 (local_attn_size < 0: no window)."""
    m = np.empty((seq, seq), np.float32)
    lib().fvo_causal_temporal_mask(seq, frame_tokens, frames_per_block, local_attn_size, _p(m, _f32p))
    return m


def block_causal_for(frames_per_block: int, local_attn_size: int, frame_tokens: int):
    """block_causal_for (C/rt/attn.rs:630-645): (block_tokens, window, sink) or None."""
    fpb = max(frames_per_block, 1)
    if local_attn_size < 0:
        window = 0
    elif local_attn_size > 0 and local_attn_size % fpb == 0:
        window = local_attn_size // fpb
    else:
        return None
    return (fpb * frame_tokens, window, 0)


# --------------------------------------------------------------------------- sdpa
def sdpa_rows(q, k, v, scale=None, rows=None, mask=None, block_causal=None, q_row0=0) -> np.ndarray:
    """The composed f32 SDPA (C/rt/sdpa.rs:328-342) on query rows `rows` of every head.
    q [bh, sq, d], k/v [bh, sk, d] -> [bh, len(rows), d]."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    bh, sq, d = q.shape
    sk = k.shape[1]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    rows = np.arange(sq, dtype=np.int32) if rows is None else np.ascontiguousarray(rows, dtype=np.int32)
    out = np.empty((bh, len(rows), d), np.float32)
    mp = None
    if mask is not None:
        mask = _f32(mask)
        assert mask.shape == (sq, sk)
        mp = _p(mask, _f32p)
    mode, bt, win, sink = (1, *block_causal) if block_causal is not None else (0, 0, 0, 0)
    lib().fvo_sdpa_rows(_p(q, _f32p), _p(k, _f32p), _p(v, _f32p), bh, sq, sk, d, ctypes.c_float(scale), mp, mode, bt,
                        win, sink, q_row0, _p(rows, _i32p), len(rows), _p(out, _f32p))
    return out


def sdpa_rows_f64(q, k, v, scale=None, rows=None, block_causal=None, q_row0=0) -> np.ndarray:
    """f64 evaluation with -inf masking (crates/fastvideo-gpucheck/src/kernels.rs:156-186)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    bh, sq, d = q.shape
    sk = k.shape[1]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    rows = np.arange(sq, dtype=np.int32) if rows is None else np.ascontiguousarray(rows, dtype=np.int32)
    out = np.empty((bh, len(rows), d), np.float64)
    mode, bt, win, sink = (1, *block_causal) if block_causal is not None else (0, 0, 0, 0)
    lib().fvo_sdpa_rows_f64(_p(q, _f32p), _p(k, _f32p), _p(v, _f32p), bh, sq, sk, d, ctypes.c_float(scale), mode, bt, win,
                            sink, q_row0, _p(rows, _i32p), len(rows), _p(out, _f64p))
    return out


def sdpa_composed_np(q, k, v, scale=None, mask=None) -> np.ndarray:
    """Pure-numpy twin of sdpa_rows with the reference's operation order (small cases only):
    scores accumulate over the head dim in index order with separate multiply and add."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    bh, sq, d = q.shape
    sk = k.shape[1]
    scale = np.float32(1.0 / math.sqrt(d) if scale is None else scale)
    out = np.zeros((bh, sq, d), np.float32)
    for h in range(bh):
        sc = np.zeros((sq, sk), np.float32)
        for t in range(d):
            sc = (sc + (q[h, :, t : t + 1] * k[h, :, t][None, :]).astype(np.float32)).astype(np.float32)
        sc = (sc * scale).astype(np.float32)
        if mask is not None:
            sc = (sc + _f32(mask)).astype(np.float32)
        m = sc.max(axis=1, keepdims=True)
        e = np.exp((sc - m).astype(np.float32)).astype(np.float32)
        ssum = np.zeros((sq,), np.float32)
        for j in range(sk):
            ssum = (ssum + e[:, j]).astype(np.float32)
        p = (e * (np.float32(1.0) / ssum)[:, None]).astype(np.float32)
        o = np.zeros((sq, d), np.float32)
        for t in range(sk):
            o = (o + (p[:, t : t + 1] * v[h, t][None, :]).astype(np.float32)).astype(np.float32)
        out[h] = o
    return out


# --------------------------------------------------------------------------- sp
def shard_ranges(seq: int, world: int):
    """sp::shard_ranges (C/rt/sp.rs:16-28): [(start, len)] contiguous, remainder to low ranks."""
    world = max(world, 1)
    st = (ctypes.c_int * world)()
    ln = (ctypes.c_int * world)()
    lib().fvo_shard_ranges(seq, world, st, ln)
    return [(st[i], ln[i]) for i in range(world)]


# --------------------------------------------------------------------------- vsa
TILE = (4, 4, 4)
TILE_ELEMS = 64


def topk_for(sparsity: float, num_tiles: int) -> int:
    return lib().fvo_topk_for(ctypes.c_double(sparsity), num_tiles)


class TilePlan:
    """TilePlan::new (C/rt/vsa.rs:63-108)."""

    def __init__(self, grid):
        t, h, w = grid
        if t <= 0 or h <= 0 or w <= 0:
            raise ValueError(f"vsa: empty grid {grid}")
        self.grid = (t, h, w)
        self.tiles = (-(-t // 4), -(-h // 4), -(-w // 4))
        n = lib().fvo_tile_plan(t, h, w, None, None, None)
        self.seq = t * h * w
        self.padded = n * TILE_ELEMS
        self.slot_src = np.empty(self.padded, np.int32)
        self.token_slot = np.empty(self.seq, np.uint32)
        self.block_sizes = np.empty(n, np.uint32)
        lib().fvo_tile_plan(t, h, w, _p(self.slot_src, _i32p), _p(self.token_slot, _u32p), _p(self.block_sizes, _u32p))

    @property
    def num_tiles(self) -> int:
        return len(self.block_sizes)


def vsa_attention_host(q, k, v, gate, grid, topk, scale=None, want_aux=False):
    """vsa_attention_host (C/rt/vsa.rs:116-262).  q, k, v, gate: [bh, seq, dim] f32 (gate may be
    None).  Returns out, or (out, selected [bh, nt, topk], scores [bh, nt, nt], coarse [bh, nt, dim])."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    bh, seq, dim = q.shape
    t, h, w = grid
    assert seq == t * h * w
    scale = 1.0 / math.sqrt(dim) if scale is None else scale
    nt = lib().fvo_tile_plan(t, h, w, None, None, None)
    topk = min(max(topk, 1), nt)
    out = np.zeros((bh, seq, dim), np.float32)
    gp = None
    if gate is not None:
        gate = _f32(gate)
        gp = _p(gate, _f32p)
    sel = np.empty((bh, nt, topk), np.uint32)
    sc = np.empty((bh, nt, nt), np.float32)
    co = np.empty((bh, nt, dim), np.float32)
    lib().fvo_vsa_attention_host(_p(q, _f32p), _p(k, _f32p), _p(v, _f32p), gp, t, h, w, topk, bh, dim,
                                 ctypes.c_float(scale), _p(out, _f32p), _p(sel, _u32p), _p(sc, _f32p), _p(co, _f32p))
    return (out, sel, sc, co) if want_aux else out


# --------------------------------------------------------------------------- block glue
def rope_bhsd(x, cos, sin, negate_sin: bool = False) -> np.ndarray:
    """apply_rotary_bshd on BHSD rows (C/rt/ops.rs:1903-1933 through rope_bhsd_f32, C/wan/causal.rs:246-263):
    x [planes, n, d] f32, cos / sin [n, d]; pairs (2i, 2i+1) use the tables' even index; products and sums
    rounded separately in f32.  Result f32."""
    x = _f32(x)
    c = _f32(cos)[None, :, 0::2]
    s = _f32(sin)[None, :, 0::2] * np.float32(-1.0 if negate_sin else 1.0)
    x0, x1 = x[..., 0::2], x[..., 1::2]
    out = np.empty_like(x)
    out[..., 0::2] = (x0 * c).astype(np.float32) - (x1 * s).astype(np.float32)
    out[..., 1::2] = (x0 * s).astype(np.float32) + (x1 * c).astype(np.float32)
    return out


def ln_adaln_e(x, e, scale_slot: int, shift_slot: int, eps: float = 1e-6) -> np.ndarray:
    """Unaffine LayerNorm + AdaLN modulation, f32 (C/rt/kernels/act16.cu:184-209, mx_ln_adaln_e):
    x [batch, seq, dim], e [batch, e_rows, dim] -> (x - mean) * rsqrt(var + eps) * (1 + e[b, scale]) + e[b, shift],
    biased variance of the deviations from the mean.  The bf16 kernel rounds this once."""
    x, e = _f32(x), _f32(e)
    mean = x.mean(axis=-1, keepdims=True, dtype=np.float32)
    d = x - mean
    inv = (1.0 / np.sqrt((d * d).mean(axis=-1, keepdims=True, dtype=np.float32) + np.float32(eps))).astype(np.float32)
    return (d * inv) * (np.float32(1.0) + e[:, scale_slot][:, None, :]) + e[:, shift_slot][:, None, :]


def self_residual_norm(h, attn, e, gate_slot: int, w, b, eps: float = 1e-6):
    """wan_res_ln with res_mode 0 / ln_mode 0 (C/wan/kernels/block.cu:17-78; host twin C/wan/fuse.rs:108-166):
    s = h + attn * e[b, gate] in f32; returns (bf16(s), LN(s) * w + b) -- the norm reads the UNROUNDED s; the
    kernel rounds the second once."""
    h, attn, e, w, b = _f32(h), _f32(attn), _f32(e), _f32(w), _f32(b)
    s = h + attn * e[:, gate_slot][:, None, :]
    mean = s.mean(axis=-1, keepdims=True, dtype=np.float32)
    d = s - mean
    inv = (1.0 / np.sqrt((d * d).mean(axis=-1, keepdims=True, dtype=np.float32) + np.float32(eps))).astype(np.float32)
    return bf16_round(s), (d * inv) * w + b


def num_threads() -> int:
    return lib().fvo_num_threads()
