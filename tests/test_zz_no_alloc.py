"""The entry point that allocates nothing (fv_sdpa_two_pass_noalloc_bf16), called through the C ABI.

It exists for hosts that may not allocate device memory at the point where they run attention -- a
serving loop on a fixed memory budget, a latency-critical thread that must not pay the allocator's
device-wide synchronisation.  It keeps its status word and the pass-1 result of the two-pass evaluation
in an array built into the library, so successive calls share that array.  The checks: its output equals
the existing entry point's (fv_sdpa_segments_bf16 over all keys in one pass) within the tolerance of the
other parity tests, on two calls in a row with different inputs (the second call must not see anything
of the first), and a call beyond the built-in limit is refused with a message instead of running.

Collected last on purpose: a failure here cannot hide another test's result in a run that stops at the
first failure."""
import ctypes
import math

import numpy as np
import pytest
import torch

from _util import MAX_ABS, MEAN_ABS, to_dev_bf16, to_host_f32

pytestmark = pytest.mark.gpu


def _i32(vals):
    return (ctypes.c_int * len(vals))(*[int(v) for v in vals])


def _vp(t):
    return ctypes.c_void_p(t.data_ptr())


def _case(oracle, seed, bh, sq, lens):
    """q and K/V split into len(lens) segments, padded to the longest, segment-major like an all-gather."""
    sk = sum(lens)
    q = oracle.bf16_round(oracle.seeded_normal(seed, 0, (bh, sq, 128)))
    k = oracle.bf16_round(oracle.seeded_normal(seed, 1, (bh, sk, 128)))
    v = oracle.bf16_round(oracle.seeded_normal(seed, 2, (bh, sk, 128)))
    rows = max(lens)
    starts = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(int).tolist()
    k_all = np.zeros((len(lens), bh, rows, 128), np.float32)
    v_all = np.zeros_like(k_all)
    for s, (s0, n) in enumerate(zip(starts, lens)):
        k_all[s, :, :n] = k[:, s0:s0 + n]
        v_all[s, :, :n] = v[:, s0:s0 + n]
    return q, k, v, k_all, v_all, starts, rows


def _run_both(fvlib, oracle, seed, bh, sq, lens, local, check_memory=False):
    q, k, v, k_all, v_all, starts, rows = _case(oracle, seed, bh, sq, lens)
    tq, tk, tv = to_dev_bf16(q), to_dev_bf16(k_all), to_dev_bf16(v_all)
    scale = ctypes.c_float(1.0 / math.sqrt(128))
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # existing entry point: every segment in one pass
    ref = torch.empty((bh, sq, 128), dtype=torch.bfloat16, device="cuda")
    rc = fvlib.fv_sdpa_segments_bf16(stream, _vp(tq), _vp(tk), _vp(tv), _vp(ref), 1, bh, sq, len(lens), _i32(lens),
                                     _i32(starts), rows, scale, 0, 0, 0, 0, 0, None, None, None)
    assert rc == 0, fvlib.fv_last_error()
    # new entry point: pass 1 over segment `local`, pass 2 over the others, nothing allocated
    out = torch.full((bh, sq, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    k_loc, v_loc = tk[local].contiguous(), tv[local].contiguous()
    lens2 = [n if s != local else 0 for s, n in enumerate(lens)]
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = fvlib.fv_sdpa_two_pass_noalloc_bf16(stream, _vp(tq), _vp(k_loc), _vp(v_loc), lens[local], starts[local], rows,
                                             _vp(tk), _vp(tv), len(lens), _i32(lens2), _i32(starts), rows, _vp(out), 1,
                                             bh, sq, scale, None)
    assert rc == 0, fvlib.fv_last_error()
    # the status word the call's kernels report to is the library's own: a wait that ran out inside this call
    # would show here, and reading it allocates nothing either
    code = ctypes.c_int(-1)
    assert fvlib.fv_device_status(stream, ctypes.byref(code)) == 0, fvlib.fv_last_error()
    assert code.value == 0
    if check_memory:
        # cudaMemGetInfo around a warm call (the module image was loaded by the call before it): not one byte
        assert torch.cuda.mem_get_info()[0] == free_before
    got, want = to_host_f32(out), to_host_f32(ref)
    assert np.isfinite(got).all()
    err = np.abs(got - want)
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS, (err.max(), err.mean())
    # and both agree with the oracle over all keys
    orc = oracle.sdpa_rows(q, k, v)
    err = np.abs(got - orc)
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS, (err.max(), err.mean())


def test_no_alloc_entry_matches_the_existing_entry_twice_in_a_row(fvlib, oracle):
    # first call: 3 segments, the middle one local; second call right after it: other sizes, other data,
    # the first segment local -- it reuses the built-in array the first call wrote
    _run_both(fvlib, oracle, 901, 3, 300, [334, 333, 333], local=1)
    _run_both(fvlib, oracle, 902, 2, 513, [200, 457], local=0, check_memory=True)


def test_a_wait_that_runs_out_is_seen_after_a_no_alloc_call(fvlib, oracle):
    """The status word is shared: a kernel that gave up before the call (the wait self-test, one warp, a
    barrier nobody arrives at, 1e5 cycles) is still reported by the status read that follows the call."""
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    fvlib.fv_selftest_wait_timeout.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
    assert fvlib.fv_selftest_wait_timeout(stream, 100000) == 0, fvlib.fv_last_error()
    q, k, v, k_all, v_all, starts, rows = _case(oracle, 903, 1, 128, [128, 128])
    tq, tk, tv = to_dev_bf16(q), to_dev_bf16(k_all), to_dev_bf16(v_all)
    out = torch.empty((1, 128, 128), dtype=torch.bfloat16, device="cuda")
    rc = fvlib.fv_sdpa_two_pass_noalloc_bf16(stream, _vp(tq), _vp(tk[0]), _vp(tv[0]), 128, 0, rows, _vp(tk), _vp(tv), 2,
                                             _i32([0, 128]), _i32(starts), rows, _vp(out), 1, 1, 128,
                                             ctypes.c_float(1.0 / math.sqrt(128)), None)
    assert rc == 0, fvlib.fv_last_error()
    code = ctypes.c_int(0)
    assert fvlib.fv_device_status(stream, ctypes.byref(code)) != 0
    assert code.value == 109
    assert fvlib.fv_device_status(stream, ctypes.byref(code)) == 0 and code.value == 0   # read once, cleared
    assert np.isfinite(to_host_f32(out)).all()


def test_no_alloc_entry_refuses_calls_beyond_its_built_in_scratch(fvlib):
    # 66 000 rows > 65 024: refused before anything is launched (the pointers are never dereferenced)
    dummy = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = fvlib.fv_sdpa_two_pass_noalloc_bf16(stream, _vp(dummy), _vp(dummy), _vp(dummy), 128, 0, 128, _vp(dummy),
                                             _vp(dummy), 1, _i32([128]), _i32([0]), 128, _vp(dummy), 1, 66, 1000,
                                             ctypes.c_float(0.088), None)
    assert rc == -1
    msg = fvlib.fv_last_error().decode()
    assert "66000" in msg and "65024" in msg
