"""The block glue either side of self-attention (ln_adaln_e before, self_residual_norm after) against the
oracle's f32 restatements.  The kernels reduce in another order than the reference's (one read of the row,
warp shuffles), so the comparison is a rounding bound, not bit equality: the result is the bf16 rounding of a
value within f32 reduction error of the oracle's, i.e. equal to the rounded oracle except at rounding ties."""
import numpy as np
import pytest
import torch

from _util import to_dev_bf16, to_host_f32

pytestmark = pytest.mark.gpu

# (batch, seq, dim): one, two and four warps per row; a width that leaves the last vectors of a lane empty
SHAPES = [(1, 7, 128), (2, 333, 1536), (1, 200, 2048), (2, 150, 5120), (1, 64, 6144), (1, 33, 3080)]


def _close_to_rounded(got, want, what):
    assert np.isfinite(got).all(), what
    # |got - want| <= half an ulp of bf16 at |want| plus slack for the f32 reduction order
    bound = np.abs(want) * 2.0 ** -8 + 2e-5 * (1.0 + np.abs(want))
    bad = np.abs(got - want) > bound
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside the rounding bound, worst {np.abs(got - want).max():.3e}"


@pytest.mark.parametrize("batch,seq,dim", SHAPES)
def test_ln_adaln_matches_oracle(fvlib, oracle, batch, seq, dim):
    from fastvideo_rs_b200 import wan
    x = oracle.bf16_round(2.0 * oracle.seeded_normal(51, dim, (batch, seq, dim)) + 0.3)
    e = (0.2 * oracle.seeded_normal(52, dim, (batch, 6, dim))).astype(np.float32)
    out = wan.ln_adaln_e(to_dev_bf16(x), torch.from_numpy(e).cuda(), 1, 0, 1e-6)
    _close_to_rounded(to_host_f32(out), oracle.ln_adaln_e(x, e, 1, 0, 1e-6), f"ln_adaln {batch}x{seq}x{dim}")


@pytest.mark.parametrize("batch,seq,dim", SHAPES)
def test_self_residual_norm_matches_oracle(fvlib, oracle, batch, seq, dim):
    from fastvideo_rs_b200 import wan
    h = oracle.bf16_round(oracle.seeded_normal(53, dim, (batch, seq, dim)))
    a = oracle.bf16_round(0.5 * oracle.seeded_normal(54, dim, (batch, seq, dim)))
    e = (0.3 * oracle.seeded_normal(55, dim, (batch, 6, dim))).astype(np.float32)
    w = (1.0 + 0.1 * oracle.seeded_normal(56, dim, (dim,))).astype(np.float32)
    b = (0.1 * oracle.seeded_normal(57, dim, (dim,))).astype(np.float32)
    hid, normed = wan.self_residual_norm(to_dev_bf16(h), to_dev_bf16(a), torch.from_numpy(e).cuda(), 2, torch.from_numpy(w).cuda(),
                                         torch.from_numpy(b).cuda(), 1e-6)
    want_h, want_n = oracle.self_residual_norm(h, a, e, 2, w, b, 1e-6)
    assert np.array_equal(to_host_f32(hid), want_h)  # elementwise, separately rounded product and sum: bit exact
    _close_to_rounded(to_host_f32(normed), want_n, f"self_residual_norm {batch}x{seq}x{dim}")


def test_glue_argument_errors(fvlib):
    import ctypes
    from fastvideo_rs_b200 import _lib
    L = _lib.lib()
    x = torch.zeros((1, 4, 128), dtype=torch.bfloat16, device="cuda")
    e = torch.zeros((1, 6, 128), dtype=torch.float32, device="cuda")
    fp = lambda t: ctypes.cast(ctypes.c_void_p(t.data_ptr()), ctypes.POINTER(ctypes.c_float))
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    assert L.fv_wan_ln_adaln_bf16(None, vp(x), fp(e), 6, 0, 1, 4, 128, 6, ctypes.c_float(1e-6), vp(x)) == _lib.ERR_INVALID
    assert L.fv_wan_ln_adaln_bf16(None, None, fp(e), 1, 0, 1, 4, 128, 6, ctypes.c_float(1e-6), vp(x)) == _lib.ERR_INVALID
    assert L.fv_wan_ln_adaln_bf16(None, vp(x), fp(e), 1, 0, 1, 4, 132, 6, ctypes.c_float(1e-6), vp(x)) == _lib.DECLINED
    assert L.fv_wan_ln_adaln_bf16(None, vp(x), fp(e), 1, 0, 1, 4, 8192, 6, ctypes.c_float(1e-6), vp(x)) == _lib.DECLINED
