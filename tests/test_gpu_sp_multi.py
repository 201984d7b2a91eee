"""Sequence-parallel attention across real GPUs: the K/V exchange (copy-engine pulls from peer-mapped staging,
or the NCCL all-gather) overlapped with the local pass, per-source chained passes, contiguous and zig-zag
shards, the Python class and the C-ABI handle.  Needs at least two B200s in the box; skipped otherwise.
NVLS is off in the children (a rank that dies must not hold a multicast binding)."""
import ctypes
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

CASES = [  # seq, block, impl, zigzag, exchange
    (3001, 0, "python", "", "ce"), (4096, 0, "python", "", "nccl"), (3001, 390, "python", "", "ce"),
    (3001, 390, "python", "zigzag", "ce"), (4099, 512, "python", "zigzag", "nccl"), (3001, 0, "python", "zigzag", "ce"),
    (3001, 0, "native", "", ""), (4096, 390, "native", "", ""), (3001, 0, "mismatch", "", ""),
]


@pytest.mark.parametrize("seq,block,impl,zigzag,exchange", CASES)
def test_sp_matches_oracle_on_all_gpus(fvlib, oracle, seq, block, impl, zigzag, exchange):
    """block > 0: the block-causal mask over global token indices; every rank fetches only the runs it can see
    (the rank-by-rank launches are also checked on one GPU in test_gpu_sdpa.py)."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("one GPU in this box")
    world = 8 if n >= 8 else (4 if n >= 4 else 2)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", "29631", str(ROOT / "tests" / "sp_worker.py"), str(seq), "3", str(block), impl, zigzag or "-", exchange or "ce"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600,
                         env={**os.environ, "NCCL_NVLS_ENABLE": "0", "FV_SP_INIT_TIMEOUT_S": "60"})
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]


def test_rendezvous_gives_up_when_a_rank_never_comes(fvlib):
    """Host-side failure, no kernel involved: rank 0 of a two-rank communicator whose peer never calls.  The
    non-blocking rendezvous is abandoned after the deadline and the call returns FV_ERR_NCCL; the process and
    the GPU stay usable (a one-rank handle is created right after)."""
    from fastvideo_rs_b200 import _lib, sp
    L = _lib.lib()
    try:
        uid = sp.NativeSp.unique_id()
    except _lib.FvError:
        pytest.skip("NCCL cannot be loaded here")
    L.fv_sp_create_timeout.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                       ctypes.c_double, ctypes.POINTER(ctypes.c_void_p)]
    h = ctypes.c_void_p()
    buf = ctypes.create_string_buffer(uid, 128)
    rc = L.fv_sp_create_timeout(buf, 2, 0, 1000, 4, 0, 3.0, ctypes.byref(h))
    assert rc == _lib.ERR_NCCL and not h.value, (rc, _lib.last_error())
    assert "rendezvous abandoned" in _lib.last_error() or "failed to form" in _lib.last_error(), _lib.last_error()
    one = sp.NativeSp(1000, 4, 1, 0)
    assert (one.start, one.len) == (0, 1000)
    one.close()
