"""One rank of the multi-GPU sequence-parallel check (run under torch.distributed.run by
tests/test_gpu_sp_multi.py): this rank's output rows against the CPU oracle over ALL keys."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def main():
    seq = int(sys.argv[1]) if len(sys.argv) > 1 else 3001
    bh = int(sys.argv[2]) if len(sys.argv) > 2 else 3
    block = int(sys.argv[3]) if len(sys.argv) > 3 else 0  # > 0: block-causal mask with that many tokens per block
    native = len(sys.argv) > 4 and sys.argv[4] == "native"  # the C-ABI handle (fv_sp_*) instead of the Python class
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from fastvideo_rs_b200 import sdpa, sp
    from oracle import oracle as O
    q, k, v = (O.bf16_round(O.seeded_normal(61, i, (bh, seq, 128))) for i in range(3))
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to("cuda", torch.bfloat16)
    if native:
        ids = [sp.NativeSp.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        attn = sp.NativeSp(seq, bh, world, rank, ids[0])
    else:
        attn = sp.SpAttention(seq, bh)
    s0, n = attn.start, attn.len
    causal = sdpa.BlockCausal(block, 0, 0) if block else None
    out = None
    for _ in range(2):  # twice: the gather buffers are reused
        out = attn.forward(dev(q[:, s0:s0 + n]), dev(k[:, s0:s0 + n]), dev(v[:, s0:s0 + n]), causal=causal)
    torch.cuda.synchronize()
    assert sdpa.device_status() == 0
    rows = np.unique(np.concatenate([np.arange(s0, s0 + min(n, 40)), np.arange(s0 + max(n - 40, 0), s0 + n)])).astype(np.int32)
    want = O.sdpa_rows(q, k, v, rows=rows, block_causal=(block, 0, 0) if block else None)
    got = out.float().cpu().numpy()[:, rows - s0]
    err = np.abs(got - want)
    ok = bool(err.max() <= 2e-2 and err.mean() <= 2e-3 and np.isfinite(got).all())
    flag = torch.tensor([0 if ok else 1], device="cuda")
    dist.all_reduce(flag)
    print(f"rank {rank}/{world}: rows {s0}..{s0 + n} max-abs {err.max():.3e} mean-abs {err.mean():.3e} {'ok' if ok else 'FAIL'}",
          flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 0 else 1)


if __name__ == "__main__":
    main()
