"""Shared helpers of the GPU parity tests."""
import numpy as np
import torch

MAX_ABS, MEAN_ABS = 2e-2, 2e-3  # bf16 outputs against the fp32 oracle (the stated tolerance of this path)


def to_dev_bf16(x: np.ndarray) -> torch.Tensor:
    """x holds bf16-representable f32 values: the conversion is exact."""
    return torch.from_numpy(np.ascontiguousarray(x)).to(device="cuda", dtype=torch.bfloat16)


def to_host_f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def assert_close(got: np.ndarray, want: np.ndarray, what: str, max_abs=MAX_ABS, mean_abs=MEAN_ABS):
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert err.max() <= max_abs and err.mean() <= mean_abs, f"{what}: max-abs {err.max():.3e} mean-abs {err.mean():.3e}"


def sample_rows(sq: int, n: int, seed: int = 0) -> np.ndarray:
    """Tile edges, the ends, and a seeded spread."""
    fixed = [r for r in (0, 1, 63, 64, 127, 128, 129, 255, 256, 257, 383, 384, 511, 512) if r < sq]
    fixed += [max(sq - 1 - i, 0) for i in range(4)]
    rng = np.random.default_rng(seed)
    extra = rng.integers(0, sq, size=max(n - len(fixed), 0)).tolist()
    return np.unique(np.asarray(fixed + extra, np.int32))
