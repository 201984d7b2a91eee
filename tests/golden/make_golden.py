"""Generates the committed fixtures under tests/golden/ from the CPU oracle.

    python tests/golden/make_golden.py

The reference (Rust) cannot be run where this repository is built and keeps no golden tensors for
this path, so the fixtures are outputs of the oracle -- the restatement of the reference's host math
that tests/test_oracle_kat.py pins to the reference's closed-form unit tests.  They freeze the
oracle (a later edit that changes its numbers fails tests/test_golden.py) and give the GPU tests
vectors that do not depend on the oracle being built on the GPU box.

Inputs are never stored: they are seeded_normal(seed, tensor_index, shape) rounded to bf16, so a
fixture is (seed, shape, rows, expected values)."""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import oracle as O  # noqa: E402

OUT = Path(__file__).resolve().parent


def wan_inputs(seed, batch, grid, heads):
    """The fused QKV projection [batch, seq, 3*heads*128] (bf16-rounded N(0,1)) and unit norm weights."""
    seq = grid[0] * grid[1] * grid[2]
    dim = heads * 128
    proj = O.bf16_round(O.seeded_normal(seed, 0, (batch, seq, 3 * dim)))
    w = np.ones(dim, np.float32)
    return proj, w, seq, dim


def wan_dense_case(seed, batch, grid, heads, rows, causal=None):
    proj, w, seq, dim = wan_inputs(seed, batch, grid, heads)
    cos, sin = O.wan_rope(*grid)
    q = O.qk_norm_rope_bhsd(proj, w, cos, sin, batch, seq, heads, 128, 3 * dim, 0, 1e-6)
    k = O.qk_norm_rope_bhsd(proj, w, cos, sin, batch, seq, heads, 128, 3 * dim, dim, 1e-6)
    v = O.split_heads_bhsd(proj, batch, seq, heads, 128, 3 * dim, 2 * dim)
    rows = np.asarray(rows, np.int32)
    out = O.sdpa_rows(q, k, v, rows=rows, block_causal=causal)
    return dict(seed=seed, batch=batch, grid=np.asarray(grid), heads=heads, rows=rows,
                causal=np.asarray(causal if causal else (0, 0, 0)), q_rows=q[:, rows], k_rows=k[:, rows], out=out)


def main():
    # config 0: tiny Wan dense self-attention, grid 3x8x8 = 192 tokens, 12 heads
    np.savez_compressed(OUT / "wan_dense_tiny.npz",
                        **wan_dense_case(1234, 1, (3, 8, 8), 12, [0, 1, 63, 64, 65, 127, 128, 191]))
    # chunk-causal at a small grid: 6 frames of 4x5 tokens, chunks of 2 frames (40 tokens)
    np.savez_compressed(OUT / "wan_causal_small.npz",
                        **wan_dense_case(4321, 1, (6, 4, 5), 2, [0, 39, 40, 41, 79, 80, 119], causal=(40, 0, 0)))
    # VSA at a grid with partial tiles: (5, 6, 9) -> tiles (2, 2, 3) = 12, keep 4
    grid, heads = (5, 6, 9), 2
    seq = 5 * 6 * 9
    q, k, v, g = (O.bf16_round(O.seeded_normal(777, i, (heads, seq, 128))) for i in range(4))
    gate = 1.0 / (1.0 + np.exp(-g.astype(np.float64)))
    gate = O.bf16_round(gate.astype(np.float32))
    out, sel, scores, coarse = O.vsa_attention_host(q, k, v, gate, grid, 4, want_aux=True)
    rows = np.asarray([0, 1, 35, 36, 100, 143, 144, 200, 269], np.int32)
    np.savez_compressed(OUT / "vsa_small.npz", seed=777, grid=np.asarray(grid), heads=heads, topk=4, rows=rows,
                        selected_sorted=np.sort(sel, axis=-1), scores=scores, coarse=coarse, out=out[:, rows])
    # rope rows
    cos, sin = O.wan_rope(21, 30, 52)
    pick = np.asarray([0, 1, 51, 52, 1559, 1560, 32759], np.int32)
    np.savez_compressed(OUT / "rope_480p_rows.npz", rows=pick, cos=cos[pick], sin=sin[pick])
    for f in sorted(OUT.glob("*.npz")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
