"""Sequence-parallel attention across real GPUs (NCCL all-gather of K/V overlapped with the local pass).
Needs at least two B200s in the box; skipped otherwise."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("seq,block,impl", [(3001, 0, "python"), (4096, 0, "python"), (3001, 390, "python"),
                                            (3001, 0, "native"), (4096, 390, "native")])
def test_sp_matches_oracle_on_all_gpus(fvlib, oracle, seq, block, impl):
    """block > 0: the block-causal mask over global token indices; every rank fetches only the shards it can see
    (the rank-by-rank launches are also checked on one GPU in test_gpu_sdpa.py)."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("one GPU in this box")
    world = 8 if n >= 8 else (4 if n >= 4 else 2)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", "29631", str(ROOT / "tests" / "sp_worker.py"), str(seq), "3", str(block), impl]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env={**__import__("os").environ, "NCCL_NVLS_ENABLE": "0"})
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
