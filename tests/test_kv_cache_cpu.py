"""KvSpec::plan through the C ABI against the reference's own unit tests (wan/causal.rs:858-912: blocks_append_and_steps_
overwrite, rolling_cache_keeps_the_sink) and the pointer sequence of update_keeps_prefix_and_window (:1113-1155).
Host arithmetic only: no device is needed."""
import pytest


def test_blocks_append_and_steps_overwrite(fvlib):
    from fastvideo_rs_b200.wan import KvSpec
    from fastvideo_rs_b200._lib import FvError
    s = KvSpec(10, 210, 0, 210, False)
    m = s.plan(0, 0, 0, 30)
    assert (m.local_start, m.local_end, m.window_start) == (0, 30, 0)
    m = s.plan(30, 30, 0, 30)          # the next denoising step of block 0: same slots
    assert (m.local_start, m.local_end) == (0, 30)
    m = s.plan(30, 30, 30, 30)         # block 1 appends and reads blocks 0 and 1
    assert (m.local_start, m.local_end, m.window_start) == (30, 60, 0)
    with pytest.raises(FvError, match="local_attn_size"):   # 22 frames with a global window: refused
        s.plan(210, 210, 210, 10)


def test_rolling_cache_keeps_the_sink(fvlib):
    from fastvideo_rs_b200.wan import KvSpec
    s = KvSpec(10, 60, 10, 60, True)
    assert s.plan(0, 0, 0, 30).local_end == 30
    assert s.plan(30, 30, 30, 30).local_end == 60
    m = s.plan(60, 60, 60, 30)         # block 2: 30 tokens evicted after the sink, written at the end
    assert (m.evicted, m.local_start, m.local_end, m.window_start) == (30, 30, 60, 0)
    m = s.plan(90, 60, 60, 30)         # the next step of block 2 overwrites in place
    assert (m.evicted, m.local_start, m.local_end) == (0, 30, 60)


def test_pointer_sequence_of_a_rolling_cache_and_errors(fvlib):
    from fastvideo_rs_b200.wan import KvSpec
    from fastvideo_rs_b200._lib import FvError
    s = KvSpec(2, 8, 2, 8, True)
    state = (0, 0)
    seen = []
    for start in (0, 0, 4, 8, 12):
        m = s.plan(state[0], state[1], start, 4)
        seen.append((m.evicted, m.local_start, m.local_end, m.window_start))
        state = (start + 4, m.local_end)
    assert seen == [(0, 0, 4, 0), (0, 0, 4, 0), (0, 4, 8, 0), (4, 4, 8, 0), (4, 4, 8, 0)]
    with pytest.raises(FvError, match="before the cache start"):
        s.plan(100, 8, 0, 4)
    w = KvSpec.rolling_window(10, 6, 1)
    assert (w.capacity, w.sink, w.max_attention, w.rolling) == (60, 10, 60, True)
    assert w.window_frames() == 6 and w.sink_target(9) == 3 and w.sink_target(4) == 0
    with pytest.raises(ValueError):
        KvSpec.rolling_window(10, 3, 3)
    g = KvSpec.global_window(1560)
    assert g.capacity == 32760 and not g.rolling


def _plan_py(spec, global_end, local_end_prev, current_start, n):
    """KvSpec::plan (wan/causal.rs:289-336) restated in plain Python; None where the reference returns an error."""
    current_end = current_start + n
    if not spec.rolling and current_end > spec.max_attention:
        return None
    if current_end < global_end and current_end + local_end_prev < global_end:
        return None
    advance = max(current_end - global_end, 0)
    evicted = n + local_end_prev - spec.capacity if (spec.rolling and current_end > global_end and n + local_end_prev > spec.capacity) else 0
    local_end = local_end_prev + advance - max(global_end - current_end, 0)
    if local_end < 0 or local_end - evicted < 0:
        return None
    local_end -= evicted
    if local_end < n or local_end > max(spec.capacity, n):
        return None
    return (evicted, local_end - n, local_end, max(local_end - spec.max_attention, 0))


def test_plan_equals_its_restatement_on_random_states(fvlib):
    import random
    from fastvideo_rs_b200.wan import KvSpec
    from fastvideo_rs_b200._lib import FvError
    rng = random.Random(5)
    for _ in range(3000):
        ft = rng.choice([1, 2, 10, 78])
        frames = rng.randint(1, 9)
        spec = KvSpec(ft, frames * ft, rng.randint(0, frames - 1) * ft if frames > 1 else 0, rng.randint(1, frames) * ft, rng.random() < 0.7)
        ge, le = rng.randint(0, 40 * ft), rng.randint(0, frames * ft)
        cs, n = rng.randint(0, 40 * ft), rng.randint(0, 4 * ft)
        want = _plan_py(spec, ge, le, cs, n)
        try:
            got = tuple(spec.plan(ge, le, cs, n))
        except FvError:
            got = None
        assert got == want, (vars(spec), ge, le, cs, n, got, want)
