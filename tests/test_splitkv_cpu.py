"""Host side of split-KV: the cost model's choice and the workspace size (no GPU needed)."""
import ctypes

from fastvideo_rs_b200 import _lib, sdpa


def test_choice_is_one_for_grids_that_fill_the_gpu():
    # the Wan denoising shapes: thousands of CTAs, nothing to even out
    for bh, sq, sk in ((24, 32760, 32760), (40, 75600, 75600), (24, 32760, 512), (12, 192, 192), (12, 4680, 4680)):
        assert sdpa.splitkv_choose(bh, sq, sk, 148) == 1


def test_choice_for_a_block_against_the_window():
    # 19 query blocks x 12 heads = 228 CTAs = 1.54 waves of 148; three ranges make 4.6 waves of a third the length
    s = sdpa.splitkv_choose(12, 4680, 32760, 148)
    assert s == 3
    # fewer CTAs than SMs: always worth cutting
    assert sdpa.splitkv_choose(12, 1560, 32760, 148) > 1
    # whatever is chosen divides the keys and leaves at least four key tiles per range
    for bh, sq, sk in ((12, 4680, 32760), (12, 1560, 32760), (40, 4680, 14040), (2, 256, 4099), (1, 128, 1 << 20)):
        for sms in (148, 132, 64):
            c = sdpa.splitkv_choose(bh, sq, sk, sms)
            assert 1 <= c <= 8 and sk % c == 0 and (c == 1 or sk // c >= 512)
    # degenerate arguments never split
    assert sdpa.splitkv_choose(0, 10, 10, 148) == 1 and sdpa.splitkv_choose(4, 10, 10, 0) == 1


def test_workspace_size():
    assert sdpa.splitkv_workspace_bytes(12, 4680, 3) == 12 * 3 * 4680 * 129 * 4
    assert sdpa.splitkv_workspace_bytes(12, 4680, 1) == 0
    assert sdpa.splitkv_workspace_bytes(12, 4680, 9) == 0
    assert sdpa.splitkv_workspace_bytes(0, 4680, 2) == 0


def test_entry_workspace_query_follows_the_plan_kind():
    L = _lib.lib()
    L.fv_sdpa_ws_bytes.restype = ctypes.c_size_t
    cs4 = ctypes.c_size_t * 4
    probe = _lib.Probe()
    L.fv_probe_default(ctypes.byref(probe))
    probe.sms = 148
    q, k = cs4(1, 12, 4680, 128), cs4(1, 12, 32760, 128)
    kvw, dense, causal = sdpa.Plan.kv_window().to_c(), sdpa.Plan.dense(None).to_c(), \
        sdpa.Plan.block_causal(None, sdpa.BlockCausal(1560)).to_c()
    want = 12 * 3 * 4680 * 129 * 4
    assert L.fv_sdpa_ws_bytes(q, k, ctypes.byref(kvw), ctypes.byref(probe)) == want
    assert L.fv_sdpa_ws_bytes(q, k, ctypes.byref(dense), ctypes.byref(probe)) == want
    assert L.fv_sdpa_ws_bytes(q, k, ctypes.byref(causal), ctypes.byref(probe)) == 0
    big = cs4(1, 40, 75600, 128)
    assert L.fv_sdpa_ws_bytes(big, big, ctypes.byref(dense), ctypes.byref(probe)) == 0
    d64 = cs4(1, 12, 4680, 64)
    assert L.fv_sdpa_ws_bytes(d64, k, ctypes.byref(kvw), ctypes.byref(probe)) == 0
