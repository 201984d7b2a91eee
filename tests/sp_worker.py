"""One rank of the multi-GPU sequence-parallel check (run under torch.distributed.run by
tests/test_gpu_sp_multi.py): this rank's output rows against the CPU oracle over ALL keys.

    sp_worker.py seq bh block impl [zigzag] [exchange]
impl: python (SpAttention), native (the C-ABI handle fv_sp_*), mismatch (native handles created with different
shapes on different ranks: every rank must get an error, none may hang)."""
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
    impl = sys.argv[4] if len(sys.argv) > 4 else "python"
    zigzag = len(sys.argv) > 5 and sys.argv[5] == "zigzag"
    exchange = sys.argv[6] if len(sys.argv) > 6 else None
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from fastvideo_rs_b200 import _lib, sdpa, sp
    from oracle import oracle as O
    if impl in ("native", "mismatch"):
        ids = [sp.NativeSp.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
    if impl == "mismatch":
        # the last rank describes another problem: the handshake inside fv_sp_create must fail on every rank
        try:
            sp.NativeSp(seq + (1 if rank == world - 1 else 0), bh, world, rank, ids[0])
            ok = False
        except _lib.FvError as e:
            ok = e.code == _lib.ERR_INVALID and "created with" in str(e)
        flag = torch.tensor([0 if ok else 1], device="cuda")
        dist.all_reduce(flag)
        print(f"rank {rank}/{world}: mismatched shapes {'refused' if ok else 'NOT refused'}", flush=True)
        dist.destroy_process_group()
        sys.exit(0 if int(flag.item()) == 0 else 1)
    q, k, v = (O.bf16_round(O.seeded_normal(61, i, (bh, seq, 128))) for i in range(3))
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to("cuda", torch.bfloat16)
    if impl == "native":
        attn = sp.NativeSp(seq, bh, world, rank, ids[0])
        rows = np.arange(attn.start, attn.start + attn.len)
    else:
        attn = sp.SpAttention(seq, bh, zigzag=zigzag, exchange=exchange)
        rows = np.asarray(attn.layout.rows(), np.int64)
    causal = sdpa.BlockCausal(block, 0, 0) if block else None
    out = None
    for _ in range(3):  # three times: the staging halves and the gather buffers are reused
        out = attn.forward(dev(q[:, rows]), dev(k[:, rows]), dev(v[:, rows]), causal=causal)
    torch.cuda.synchronize()
    assert sdpa.device_status() == 0
    n = len(rows)
    pick = np.unique(np.concatenate([np.arange(min(n, 40)), np.arange(max(n - 40, 0), n), np.arange(max(n // 2 - 20, 0), min(n // 2 + 20, n))]))
    want = O.sdpa_rows(q, k, v, rows=rows[pick].astype(np.int32), block_causal=(block, 0, 0) if block else None)
    got = out.float().cpu().numpy()[:, pick]
    err = np.abs(got - want)
    ok = bool(err.max() <= 2e-2 and err.mean() <= 2e-3 and np.isfinite(got).all())
    flag = torch.tensor([0 if ok else 1], device="cuda")
    dist.all_reduce(flag)
    print(f"rank {rank}/{world} {impl} zigzag={zigzag} exchange={getattr(attn, 'exchange', 'nccl')}: {n} rows, max-abs {err.max():.3e} "
          f"mean-abs {err.mean():.3e} {'ok' if ok else 'FAIL'}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 0 else 1)


if __name__ == "__main__":
    main()
