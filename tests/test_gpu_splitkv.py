"""Split-KV (a short query block against a long key window, Plan::kv_window of rt/sdpa.rs:122-133, :300-326)
through the C ABI: the parts merged by their log-sum-exp equal the oracle and the one-launch kernel.
Tolerance: bf16 outputs within max-abs 2e-2 and mean-abs 2e-3 of the fp32 oracle; against the one-launch
kernel in f32, relative L2 4e-3 (the reference's kernel-against-kernel bound, crates/fastvideo-gpucheck/src/
kernels/attn2.rs:83-175: each range rounds its probabilities to bf16 about a maximum of its own)."""
import numpy as np
import pytest
import torch

from _util import assert_close, sample_rows, to_dev_bf16, to_host_f32
from test_gpu_sdpa import qkv

pytestmark = pytest.mark.gpu

# (bh, sq, sk, splits): ranges that are whole key tiles, ranges that end inside a tile, one query row,
# more ranges than key tiles per range, the widest split
CASES = [(2, 300, 1536, 2), (2, 300, 1536, 3), (3, 130, 1500, 3), (1, 1, 1024, 4), (2, 257, 640, 5), (2, 64, 48, 8),
         (1, 520, 4096, 8), (4, 256, 777 * 7, 7)]


@pytest.mark.parametrize("bh,sq,sk,splits", CASES)
def test_splitkv_matches_oracle_and_one_launch(fvlib, oracle, bh, sq, sk, splits):
    from fastvideo_rs_b200 import sdpa
    q, k, v = qkv(oracle, 500 + sk + splits, bh, sq, sk)
    tq, tk, tv = to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v)
    out = sdpa.splitkv_fwd(tq, tk, tv, splits)
    assert sdpa.device_status() == 0
    assert_close(to_host_f32(out), oracle.sdpa_rows(q, k, v), f"split {splits} of {bh}x{sq}x{sk}")
    o32 = sdpa.splitkv_fwd(tq, tk, tv, splits, out_bf16=False)
    one = sdpa.dense_fwd(tq, tk, tv, out_bf16=False)
    rel = float(((o32 - one).double().pow(2).sum() / one.double().pow(2).sum()).sqrt())
    assert rel <= 4e-3, rel
    # bf16 out is the rounded f32 out, and the call is deterministic
    assert torch.equal(out, o32.to(torch.bfloat16))
    assert torch.equal(out, sdpa.splitkv_fwd(tq, tk, tv, splits))


def test_splitkv_merged_heads_and_scale(fvlib, oracle):
    from fastvideo_rs_b200 import sdpa
    b, h, sq, sk = 2, 3, 200, 900
    q, k, v = qkv(oracle, 41, b * h, sq, sk)
    tq, tk, tv = to_dev_bf16(q), to_dev_bf16(k), to_dev_bf16(v)
    bhsd = sdpa.splitkv_fwd(tq, tk, tv, 3, scale=0.05)
    assert_close(to_host_f32(bhsd), oracle.sdpa_rows(q, k, v, scale=0.05), "split scale 0.05")
    merged = sdpa.splitkv_fwd(tq, tk, tv, 3, scale=0.05, out_heads=h)
    assert merged.shape == (b, sq, h * 128)
    assert torch.equal(merged, bhsd.view(b, h, sq, 128).permute(0, 2, 1, 3).reshape(b, sq, h * 128))


def test_splitkv_bad_arguments_are_errors(fvlib, oracle):
    from fastvideo_rs_b200 import FvError, sdpa
    q, k, v = (to_dev_bf16(x) for x in qkv(oracle, 42, 2, 64, 600))
    with pytest.raises(FvError, match="divide"):
        sdpa.splitkv_fwd(q, k, v, 7)
    with pytest.raises(FvError, match="splits"):
        sdpa.splitkv_fwd(q, k, v, 1)
    with pytest.raises(FvError, match="splits"):
        sdpa.splitkv_fwd(q, k, v, 10)
    with pytest.raises(FvError, match="workspace"):
        sdpa.splitkv_fwd(q, k, v, 2, workspace=torch.empty(1024, dtype=torch.uint8, device="cuda"))
    assert sdpa.device_status() == 0


def test_kv_window_plan_at_the_causal_wan_shape(fvlib, oracle):
    """One block of 3 latent frames (4 680 rows) against the 21-frame window (32 760 keys), 12 heads
    (crates/fastvideo-cudarc/src/wan/transformer.rs:250-313): Plan.kv_window takes the split path on a
    148-SM GPU and equals the oracle on sampled rows and the one-launch kernel everywhere."""
    from fastvideo_rs_b200 import sdpa, sdpa_rule
    b, h, sq, sk = 1, 12, 4680, 32760
    q, k, v = qkv(oracle, 43, b * h, sq, sk)
    tq, tk, tv = (to_dev_bf16(x).view(b, h, -1, 128) for x in (q, k, v))
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert sdpa.splitkv_choose(b * h, sq, sk, sms) > 1 or sms != 148
    out = sdpa.sdpa(tq, tk, tv, sdpa.Plan.kv_window())
    assert sdpa.device_status() == 0
    one = sdpa.dense_fwd(tq.view(b * h, sq, 128), tk.view(b * h, sk, 128), tv.view(b * h, sk, 128))
    diff = (out.view(b * h, sq, 128).float() - one.float()).abs()
    assert float(diff.max()) <= 4e-3  # one bf16 step of values below 1
    rows = sample_rows(sq, 24, 5)
    heads = [0, 5, 11]
    want = oracle.sdpa_rows(q[heads], k[heads], v[heads], rows=rows)
    got = to_host_f32(out.view(b * h, sq, 128)[heads][:, torch.from_numpy(rows).long().cuda()])
    assert_close(got, want, "kv_window 4680 x 32760")
    # a probe that forces the composed reference still declines instead of running something else
    from fastvideo_rs_b200 import Declined
    with pytest.raises(Declined):
        sdpa.sdpa(tq, tk, tv, sdpa.Plan.kv_window_with(False))
