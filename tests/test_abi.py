"""The C ABI: the shared library loads, exports every symbol include/fv_sdpa.h declares, and -- on a
machine without an sm_100 device -- refuses to compute instead of falling back."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "fv_sdpa.h").read_text()
    return sorted(set(re.findall(r"FV_API\s+[\w\s\*]+?\b(fv_\w+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    for must in ("fv_sdpa", "fv_sdpa_dense_bf16", "fv_sdpa_dense_merged_bf16", "fv_sdpa_two_pass_noalloc_bf16", "fv_sdpa_segments_bf16", "fv_wan_qk_prep_bf16", "fv_wan_rope_tables",
                 "fv_rule_dense_route", "fv_rule_mma_kernel", "fv_shard_ranges", "fv_last_error", "fv_device_status"):
        assert must in names


def test_library_exports_every_declared_symbol(fvlib):
    for name in declared_symbols():
        assert hasattr(fvlib, name), f"libfvsdpa.so does not export {name}"


def test_no_torch_types_in_the_signatures():
    text = (ROOT / "include" / "fv_sdpa.h").read_text()
    code = re.sub(r"/\*.*?\*/", "", text, flags=re.S)  # comments may cite the reference's CudaTensor
    assert "torch" not in code.lower() and "at::" not in code and "Tensor" not in code


def test_version_and_error_strings(fvlib):
    assert b"sm_100a" in fvlib.fv_version()
    assert isinstance(fvlib.fv_last_error(), bytes)


def test_compute_entries_refuse_without_a_device(fvlib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    rc = fvlib.fv_sdpa_dense_bf16(None, ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16),
                                  ctypes.c_void_p(16), 1, 1, 128, 128, 128, ctypes.c_float(0.088), 0, 0, 0, 0, 0)
    assert rc == -3  # FV_ERR_NO_DEVICE
    assert b"no CPU path" in fvlib.fv_last_error() or b"sm_100a" in fvlib.fv_last_error()


def test_declines_are_not_errors(fvlib):
    # head dim 64 is outside what the kernel runs: declined before any device is touched
    rc = fvlib.fv_sdpa_dense_bf16(None, None, None, None, None, 1, 1, 128, 128, 64, ctypes.c_float(0.125), 0, 0, 0, 0, 0)
    assert rc == 1
    rc = fvlib.fv_sdpa_dense_bf16(None, None, None, None, None, 1, 0, 128, 128, 128, ctypes.c_float(0.088), 0, 0, 0, 0, 0)
    assert rc == 1


def test_host_rope_tables_equal_the_oracle(fvlib, oracle):
    from fastvideo_rs_b200 import wan
    import numpy as np
    for grid, start in (((3, 8, 8), 0), ((2, 3, 5), 4), ((21, 30, 52), 0)):
        c, s = wan.wan_rope_tables_host(grid, 128, 10000.0, start)
        co, so = oracle.wan_rope(*grid, 128, 10000.0, start)
        assert np.array_equal(c, co) and np.array_equal(s, so)


def test_shard_ranges_equal_the_oracle(fvlib, oracle):
    from fastvideo_rs_b200 import sp
    for seq, world in ((10, 2), (11, 2), (75600, 8), (32760, 8), (7, 8), (1, 1), (32761, 4)):
        assert sp.shard_ranges(seq, world) == oracle.shard_ranges(seq, world)


def test_the_entry_declines_what_is_not_ours(fvlib):
    from fastvideo_rs_b200 import _lib, sdpa_rule as R
    cs4 = ctypes.c_size_t * 4
    shape = cs4(1, 12, 192, 128)

    def call(plan_kind, probe, has_mask=0, d=128):
        pc = _lib.PlanC()
        pc.kind = plan_kind
        pc.has_mask = has_mask
        pc.block_tokens = 64
        pc.kv_flash = -1
        pr = probe.to_c()
        sh = cs4(1, 12, 192, d)
        return fvlib.fv_sdpa(None, None, None, None, sh, sh, sh, ctypes.byref(pc), ctypes.byref(pr), None, 1)

    assert call(1, R.Probe()) == 1                                  # Plan::composed
    assert call(3, R.Probe()) == 1                                  # Plan::vdn_window
    assert call(0, R.Probe(), has_mask=1) == 1                      # additive mask -> composed step
    assert call(0, R.Probe(backend=R.Backend.Cublas)) == 1          # FASTVIDEO_SDPA=cublas
    assert call(0, R.Probe(kernel_choice="v2")) == 1                # another fused kernel fixed by the seam
    assert call(0, R.Probe(b200_loaded=False, dc_loaded=True)) == 1 # library not the auto pick
    assert call(2, R.Probe(sp_world=2)) == 1                        # block-causal under SP: dense-mask fallback
    assert call(0, R.Probe(), d=80) == 1                            # head dim the kernel does not run
    assert call(0, R.Probe(backend=R.Backend.Host)) == -1           # retired backend is an error
    assert b"retired" in fvlib.fv_last_error()
