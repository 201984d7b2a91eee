"""The chooser (csrc/sdpa_rule.cpp through the C ABI) against the reference's own unit tests
(crates/fastvideo-cudarc/src/rt/sdpa_rule.rs:549-652) and against an independent restatement of its
rules over a table of probes (the reference's identity test, rt/sdpa_rule_identity.rs, in spirit:
every reachable input, two implementations, equal traces)."""
import itertools

import pytest

from fastvideo_rs_b200 import sdpa_rule as R


def test_the_measured_shapes_get_the_faster_kernel_or_a_tie(fvlib):
    for n in (27_280, 36_080, 37_710, 124_440):
        assert R.pick(12, n, n, 128) == R.DensePick.Cudnn
    for sq, sk in ((130_560, 130_560), (23_616, 23_616), (6_144, 6_144), (27_280, 512), (38_760, 1_024), (124_440, 151)):
        assert R.pick(12, sq, sk, 128) == R.DensePick.V2


def test_only_sm12x_d128_has_rows(fvlib):
    assert R.pick(9, 37_710, 37_710, 128) == R.DensePick.V2
    assert R.pick(10, 37_710, 37_710, 128) == R.DensePick.V2
    assert R.pick(12, 37_710, 37_710, 64) == R.DensePick.V2


def test_auto_mode_parses(fvlib):
    assert R.parse_auto_mode("timed") == R.AutoMode.Timed
    assert R.parse_auto_mode(" timed ") == R.AutoMode.Timed
    assert R.parse_auto_mode("rule") == R.AutoMode.Rule
    assert R.parse_auto_mode("") == R.AutoMode.Rule


def test_backend_parses_like_the_string_compares_it_replaces(fvlib):
    assert R.parse_backend("dense") == R.Backend.Dense
    assert R.parse_backend("cublas") == R.Backend.Cublas
    assert R.parse_backend("flash") == R.Backend.Flash
    assert R.parse_backend("host") == R.Backend.Host
    assert R.parse_backend("sparse") == R.Backend.Sparse
    for v in ("", "fused", " cublas", "dense "):
        assert R.parse_backend(v) == R.Backend.Dense


def test_the_h3_vae_override_parses(fvlib):
    assert R.parse_kernel_override("v3s") == R.FlashKernel.V3s
    assert R.parse_kernel_override("cudnn") == R.FlashKernel.Cudnn
    for v in ("auto", "dc", "", "V2", "b200"):
        assert R.parse_kernel_override(v) is None


def test_flash_v2_only_where_its_grid_fills_the_gpu(fvlib):
    assert R.flash_v2_fills(37_710, 56, 188)
    assert R.flash_v2_fills(124_440, 32, 188)
    assert R.flash_v2_fills(130_560, 32, 188)
    assert not R.flash_v2_fills(6_144, 32, 188)
    assert not R.flash_v2_fills(1, 1, 188)


def test_shapes_agree_only_when_k_and_v_match_q(fvlib):
    s = R.Shape.of([1, 2, 5, 64], [1, 2, 7, 64], [1, 2, 7, 64])
    assert s.dims == R.Dims(1, 2, 5, 7, 64) and (s.sq, s.sk) == (5, 7)
    assert R.Shape.of([1, 2, 5, 64], [1, 2, 7, 64], [1, 2, 6, 64]).dims is None
    assert R.Shape.of([1, 2, 5, 64], [1, 3, 7, 64], [1, 3, 7, 64]).dims is None
    assert R.Shape.of([1, 2, 5, 64], [1, 2, 7, 32], [1, 2, 7, 32]).dims is None


def test_mma_sdpa_supported_table(fvlib):
    """rt/attn.rs:107-128"""
    assert R.mma_sdpa_supported(1, 12, 32760, 32760, 128, 10)
    assert R.mma_sdpa_supported(2, 4, 1, 1, 64, 8)
    assert not R.mma_sdpa_supported(1, 12, 32760, 32760, 80, 10)
    assert not R.mma_sdpa_supported(1, 12, 0, 7, 128, 10)
    assert not R.mma_sdpa_supported(1, 12, 7, 0, 128, 10)
    assert not R.mma_sdpa_supported(1, 12, 7, 7, 128, 7)
    assert not R.mma_sdpa_supported(1, 65536, 7, 7, 128, 10)
    assert R.mma_sdpa_supported(1, 65535, 7, 7, 128, 10)


# ---- an independent restatement of the reference rules (written from the Rust, not from the C++) ----
def ref_flash_kernel_for(sq, bh, sms, p):
    fixed = {"v1": "V1", "v2": "V2", "v3": "V3", "v3s": "V3s", "cudnn": "Cudnn", "dc": "Dc"}
    if p.kernel_choice in fixed:
        return fixed[p.kernel_choice]
    if p.dc_loaded:
        return "Dc"
    fills = -(-sq // 128) * bh >= 16 * max(sms, 1)
    return "V2" if fills else "V1"


def ref_dense_route(shape, masked, out_bf16, p):
    route = []
    if not masked:
        if p.backend in (R.Backend.Host, R.Backend.Sparse):
            return [("Retired", p.backend)]
        if p.backend == R.Backend.Flash:
            route.append(("FlashF32",))
        if p.backend != R.Backend.Cublas and p.mma_default:
            if p.sage_min_seq is not None and shape.sq >= p.sage_min_seq and shape.sk >= p.sage_min_seq:
                route.append(("Sage", out_bf16))
            route.append(("Mma", out_bf16))
        route.append(("Cublas",))
    route.append(("Composed",))
    return route


def ref_mma_kernel(shape, out_bf16, p):
    if shape.dims is None or p.sm_major is None:
        return ("fixed", ref_flash_kernel_for(2**64 - 1, 1, 1, p))
    d = shape.dims
    k = ref_flash_kernel_for(d.sq, d.b * d.h, p.sms, p)
    if k == "V2" and out_bf16 and p.sm_major == 12 and p.kernel_choice == "auto":
        if p.auto_mode == R.AutoMode.Timed:
            return ("timed",)
        cud = d.d == 128 and d.sq >= 24576 and 24576 <= d.sk <= 128000
        return ("rule", "Cudnn" if (cud and p.cudnn_has_plan) else "V2", 12)
    return ("fixed", k)


SHAPES = [
    ([1, 12, 192, 128], [1, 12, 192, 128]), ([2, 12, 32760, 128], [2, 12, 32760, 128]),
    ([2, 12, 32760, 128], [2, 12, 512, 128]), ([1, 40, 75600, 128], [1, 40, 75600, 128]),
    ([1, 32, 6144, 128], [1, 32, 6144, 128]), ([1, 56, 37710, 128], [1, 56, 37710, 128]),
    ([1, 2, 5, 64], [1, 2, 7, 64]), ([1, 2, 5, 64], [1, 3, 7, 64]), ([1, 24, 27280, 80], [1, 24, 27280, 80]),
]


def as_tuple_step(s):
    if s.kind == R.StepKind.Retired:
        return ("Retired", s.retired)
    if s.kind in (R.StepKind.Sage, R.StepKind.Mma):
        return (s.kind.name, s.out_bf16)
    return (s.kind.name,)


def test_identity_with_the_reference_rules_when_the_b200_kernel_is_absent(fvlib):
    n = 0
    for backend, mma_default, sage, choice, sm, dc, auto, plan, sp in itertools.product(
            list(R.Backend), (False, True), (None, 4096), ("auto", "v1", "v2", "v3", "v3s", "cudnn", "dc", "bogus"),
            (None, 8, 9, 10, 12), (False, True), list(R.AutoMode), (False, True), (1, 2)):
        p = R.Probe(backend=backend, sp_world=sp, mma_default=mma_default, sage_min_seq=sage, kernel_choice=choice,
                    sm_major=sm, sms=148 if sm != 12 else 188, dc_loaded=dc, b200_loaded=False, auto_mode=auto,
                    cudnn_has_plan=plan)
        for q, k in SHAPES:
            shape = R.Shape.of(q, k, k)
            for masked, out_bf16 in ((False, True), (False, False), (True, True)):
                got = [as_tuple_step(s) for s in R.dense_route(shape, masked, out_bf16, p)]
                assert got == ref_dense_route(shape, masked, out_bf16, p)
            for out_bf16 in (True, False):
                m = R.mma_kernel(shape, out_bf16, p)
                want = ref_mma_kernel(shape, out_bf16, p)
                got = (m.kind,) if m.kind == "timed" else ((m.kind, m.kernel.name) if m.kind == "fixed" else
                                                           (m.kind, m.kernel.name, m.sm_major))
                assert got == want, (p, q, k, out_bf16)
                n += 1
        assert R.block_causal_first(p) == (p.causal_flash and sp == 1 and mma_default)
        assert R.vdn_window_first(p) == (sp == 1 and mma_default)
    assert n > 100_000


def test_the_b200_kernel_is_the_auto_pick_where_loaded_and_a_seam_value(fvlib):
    q = [1, 40, 75600, 128]
    shape = R.Shape.of(q, q, q)
    auto = R.Probe(sm_major=10, b200_loaded=True, dc_loaded=True)
    assert R.flash_kernel_for(75600, 40, 148, auto) == R.FlashKernel.B200
    assert R.mma_kernel(shape, True, auto) == R.MmaKernel("fixed", R.FlashKernel.B200)
    # an explicit choice still wins, in both directions
    assert R.flash_kernel_for(75600, 40, 148, R.Probe(kernel_choice="dc", b200_loaded=True)) == R.FlashKernel.Dc
    assert R.flash_kernel_for(75600, 40, 148, R.Probe(kernel_choice="v2", b200_loaded=True)) == R.FlashKernel.V2
    assert R.flash_kernel_for(75600, 40, 148, R.Probe(kernel_choice="b200", b200_loaded=False)) == R.FlashKernel.B200
    # not loaded: the reference's answer
    assert R.flash_kernel_for(75600, 40, 148, R.Probe(b200_loaded=False, dc_loaded=True)) == R.FlashKernel.Dc
    assert R.flash_kernel_for(75600, 40, 148, R.Probe(b200_loaded=False)) == R.FlashKernel.V2


def test_route_predicates(fvlib):
    p = R.Probe()
    assert R.block_causal_first(p) and R.vdn_window_first(p)
    assert not R.block_causal_first(R.Probe(sp_world=2))
    assert not R.block_causal_first(R.Probe(causal_flash=False))
    assert R.kv_window_flash(None, p) and not R.kv_window_flash(None, R.Probe(causal_flash=False))
    assert R.kv_window_flash(True, R.Probe(causal_flash=False)) and not R.kv_window_flash(False, p)
    assert not R.fp8_first(p) and R.fp8_first(R.Probe(fp8_dense=True))


def test_run_route_takes_the_first_step_that_answers(fvlib):
    route = [R.Step(R.StepKind.Mma, True), R.Step(R.StepKind.Cublas), R.Step(R.StepKind.Composed)]
    seen = []

    def attempt(step):
        seen.append(step.kind)
        return "ran" if step.kind == R.StepKind.Cublas else None

    assert R.run_route(route, attempt) == "ran" and seen == [R.StepKind.Mma, R.StepKind.Cublas]
    assert R.run_route(route, lambda s: None) is None


def test_live_probe_without_a_device_says_so(fvlib, monkeypatch):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    monkeypatch.setenv("FASTVIDEO_SDPA", "cublas")
    monkeypatch.setenv("FASTVIDEO_SP_WORLD", "4")
    monkeypatch.setenv("FASTVIDEO_FLASH_KERNEL", "B200")
    p = R.live()
    assert p.sm_major is None and not p.mma_default and not p.b200_loaded
    assert p.backend == R.Backend.Cublas and p.sp_world == 4 and p.kernel_choice == "b200"
