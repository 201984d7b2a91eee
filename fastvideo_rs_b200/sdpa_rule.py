"""The kernel-selection plugin: rt::sdpa_rule (crates/fastvideo-cudarc/src/rt/sdpa_rule.rs) over the
C++ chooser in csrc/sdpa_rule.cpp.  Names, argument meaning and results follow the reference; the one
addition is ``FlashKernel.B200`` (seam value ``"b200"``; the ``auto`` pick where ``b200_loaded``).
Everything here is pure and runs without a GPU."""
from __future__ import annotations

import ctypes
import enum
from dataclasses import dataclass, field
from typing import Optional, Sequence

from . import _lib


class Backend(enum.IntEnum):
    Dense = 0
    Cublas = 1
    Flash = 2
    Host = 3
    Sparse = 4


class FlashKernel(enum.IntEnum):
    V1 = 0
    V2 = 1
    V3 = 2
    V3s = 3
    Cudnn = 4
    Dc = 5
    B200 = 6


class AutoMode(enum.IntEnum):
    Rule = 0
    Timed = 1


class DensePick(enum.IntEnum):
    Cudnn = 0
    V2 = 1


class StepKind(enum.IntEnum):
    Retired = 0
    FlashF32 = 1
    Sage = 2
    Mma = 3
    Cublas = 4
    Composed = 5


@dataclass(frozen=True)
class Step:
    kind: StepKind
    out_bf16: bool = False
    retired: Optional[Backend] = None


@dataclass(frozen=True)
class MmaKernel:
    kind: str  # "fixed" | "rule" | "timed"
    kernel: Optional[FlashKernel] = None
    sm_major: Optional[int] = None


MMA_TILE = 64


@dataclass
class Probe:
    """What the chooser reads (the reference's Probe trait, sdpa_rule.rs:321-350, as data)."""
    backend: Backend = Backend.Dense
    sp_world: int = 1
    mma_default: bool = True
    sage_min_seq: Optional[int] = None
    fp8_dense: bool = False
    causal_flash: bool = True
    kernel_choice: str = "auto"
    sm_major: Optional[int] = 10
    sms: int = 148
    dc_loaded: bool = False
    b200_loaded: bool = True
    auto_mode: AutoMode = AutoMode.Rule
    cudnn_has_plan: bool = False

    def to_c(self) -> _lib.Probe:
        c = _lib.Probe()
        c.backend = int(self.backend)
        c.sp_world = max(int(self.sp_world), 1)
        c.mma_default = int(self.mma_default)
        c.has_sage = int(self.sage_min_seq is not None)
        c.sage_min_seq = int(self.sage_min_seq or 0)
        c.fp8_dense = int(self.fp8_dense)
        c.causal_flash = int(self.causal_flash)
        c.kernel_choice = self.kernel_choice.encode()[:31]
        c.has_sm = int(self.sm_major is not None)
        c.sm_major = int(self.sm_major or 0)
        c.sms = max(int(self.sms), 1)
        c.dc_loaded = int(self.dc_loaded)
        c.b200_loaded = int(self.b200_loaded)
        c.auto_timed = int(self.auto_mode == AutoMode.Timed)
        c.cudnn_has_plan = int(self.cudnn_has_plan)
        return c

    @staticmethod
    def from_c(c: _lib.Probe) -> "Probe":
        return Probe(Backend(c.backend), c.sp_world, bool(c.mma_default), c.sage_min_seq if c.has_sage else None,
                     bool(c.fp8_dense), bool(c.causal_flash), c.kernel_choice.decode(),
                     c.sm_major if c.has_sm else None, c.sms, bool(c.dc_loaded), bool(c.b200_loaded),
                     AutoMode.Timed if c.auto_timed else AutoMode.Rule, bool(c.cudnn_has_plan))


def live() -> Probe:
    """The settings (FASTVIDEO_* variables) and the current device: the reference's `Live`."""
    c = _lib.Probe()
    _lib.lib().fv_probe_live(ctypes.byref(c))
    return Probe.from_c(c)


def _shape4(s: Sequence[int]):
    if len(s) != 4:
        raise ValueError("sdpa expects BHSD")
    return (ctypes.c_size_t * 4)(*[int(x) for x in s])


def parse_backend(v: str) -> Backend:
    return Backend(_lib.lib().fv_rule_parse_backend(v.encode()))


def parse_auto_mode(v: str) -> AutoMode:
    return AutoMode.Timed if _lib.lib().fv_rule_parse_auto_timed(v.encode()) else AutoMode.Rule


def parse_kernel_override(v: str) -> Optional[FlashKernel]:
    r = _lib.lib().fv_rule_parse_kernel_override(v.encode())
    return None if r < 0 else FlashKernel(r)


def flash_v2_fills(sq: int, bh: int, sms: int) -> bool:
    return bool(_lib.lib().fv_rule_flash_v2_fills(ctypes.c_size_t(sq), ctypes.c_size_t(bh), ctypes.c_size_t(sms)))


def pick(sm_major: int, sq: int, sk: int, d: int) -> DensePick:
    return DensePick(_lib.lib().fv_rule_pick(sm_major, ctypes.c_size_t(sq), ctypes.c_size_t(sk), ctypes.c_size_t(d)))


@dataclass(frozen=True)
class Dims:
    b: int
    h: int
    sq: int
    sk: int
    d: int


@dataclass(frozen=True)
class Shape:
    sq: int
    sk: int
    dims: Optional[Dims]
    _q: tuple = field(default=(), compare=False, repr=False)
    _k: tuple = field(default=(), compare=False, repr=False)
    _v: tuple = field(default=(), compare=False, repr=False)

    @staticmethod
    def of(q: Sequence[int], k: Sequence[int], v: Sequence[int]) -> "Shape":
        sq, sk, ok = ctypes.c_size_t(), ctypes.c_size_t(), ctypes.c_int()
        _lib.lib().fv_rule_shape_of(_shape4(q), _shape4(k), _shape4(v), ctypes.byref(sq), ctypes.byref(sk),
                                    ctypes.byref(ok))
        dims = Dims(q[0], q[1], q[2], k[2], q[3]) if ok.value else None
        return Shape(sq.value, sk.value, dims, tuple(q), tuple(k), tuple(v))


def dense_route(shape: Shape, masked: bool, out_bf16: bool, p: Probe) -> list[Step]:
    steps = (_lib.Step * 8)()
    n = _lib.lib().fv_rule_dense_route(_shape4(shape._q), _shape4(shape._k), _shape4(shape._v), int(masked),
                                       int(out_bf16), ctypes.byref(p.to_c()), steps)
    out = []
    for i in range(n):
        kind = StepKind(steps[i].kind)
        if kind == StepKind.Retired:
            out.append(Step(kind, False, Backend(steps[i].retired)))
        elif kind in (StepKind.Sage, StepKind.Mma):
            out.append(Step(kind, bool(steps[i].out_bf16)))
        else:
            out.append(Step(kind))
    return out


def run_route(route, attempt):
    """Each step through `attempt` until one returns a result (sdpa_rule.rs:441-454)."""
    for step in route:
        out = attempt(step)
        if out is not None:
            return out
    return None


def flash_kernel_for(sq: int, bh: int, sms: int, p: Probe) -> FlashKernel:
    return FlashKernel(_lib.lib().fv_rule_flash_kernel_for(ctypes.c_size_t(sq), ctypes.c_size_t(bh),
                                                           ctypes.c_size_t(sms), ctypes.byref(p.to_c())))


def mma_kernel(shape: Shape, out_bf16: bool, p: Probe) -> MmaKernel:
    kern, sm = ctypes.c_int(), ctypes.c_int()
    kind = _lib.lib().fv_rule_mma_kernel(_shape4(shape._q), _shape4(shape._k), _shape4(shape._v), int(out_bf16),
                                         ctypes.byref(p.to_c()), ctypes.byref(kern), ctypes.byref(sm))
    if kind == 0:
        return MmaKernel("fixed", FlashKernel(kern.value))
    if kind == 1:
        return MmaKernel("rule", FlashKernel(kern.value), sm.value)
    return MmaKernel("timed")


def fp8_first(p: Probe) -> bool:
    return bool(_lib.lib().fv_rule_fp8_first(ctypes.byref(p.to_c())))


def block_causal_first(p: Probe) -> bool:
    return bool(_lib.lib().fv_rule_block_causal_first(ctypes.byref(p.to_c())))


def vdn_window_first(p: Probe) -> bool:
    return bool(_lib.lib().fv_rule_vdn_window_first(ctypes.byref(p.to_c())))


def kv_window_flash(flash: Optional[bool], p: Probe) -> bool:
    f = -1 if flash is None else int(flash)
    return bool(_lib.lib().fv_rule_kv_window_flash(f, ctypes.byref(p.to_c())))


def mma_sdpa_supported(b: int, h: int, sq: int, sk: int, d: int, sm_major: int) -> bool:
    cs = ctypes.c_size_t
    return bool(_lib.lib().fv_rule_mma_sdpa_supported(cs(b), cs(h), cs(sq), cs(sk), cs(d), sm_major))
