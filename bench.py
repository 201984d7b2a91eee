#!/usr/bin/env python
"""Benchmark of the Wan self-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" = one pass of the path over one synthetic batch: the fused QKV projection (bf16, seeded
N(0,1)) goes through the q/k prologue kernel (RMSNorm across heads + 3-D RoPE + head split) and the
attention kernel.  Default workload: Wan2.1-14B 720p x 81 frames dense self-attention (1 x 40 heads x
75 600 tokens x 128), sequence-parallel over N GPUs (token shards; one NCCL all-gather of K and V per
step, overlapped with attention over the local keys).  Total work is fixed as N grows ("strong").

Prints ONE JSON line (rank 0).  FLOPs = 4 * bh * sq * sk_visible * d (the reference's formula,
crates/fastvideo-gpucheck/src/kernels/attn2.rs:466).  `value` is whole-job TFLOP/s with inputs resident
in HBM; `e2e` is the same metric with the projection coming from pinned host memory and the result
going back to the host inside the timed region.

--impl reference times the reference's CPU path (its composed f32 SDPA after the host q/k norm + RoPE,
restated in oracle/fv_oracle.cpp because the reference is Rust and no Rust toolchain exists here) on all
host threads, on a bounded sample of query rows of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: batch, heads, grid (frames, h, w in patches), causal block tokens (0 = dense), cross keys
    "wan14b_720p_dense": dict(batch=1, heads=40, grid=(21, 45, 80), block=0, desc="Wan2.1-14B 720p x81f dense self-attention"),
    "wan1p3b_480p_dense": dict(batch=2, heads=12, grid=(21, 30, 52), block=0, desc="Wan2.1-1.3B 480p x81f dense self-attention, CFG pair"),
    "wan1p3b_480p_causal": dict(batch=1, heads=12, grid=(21, 30, 52), block=4680, desc="Self-Forcing chunk-causal (7 chunks x 3 frames) at the Wan-1.3B shape"),
    "wan1p3b_480p_vsa": dict(batch=1, heads=12, grid=(21, 30, 52), block=0, vsa_topk=78,
                             desc="VSA block-sparse self-attention at the Wan-1.3B 480p grid: 624 tiles of 64 tokens, top-k 78 (12.5 %), "
                                  "sigmoid gate applied to seeded logits before the call"),
    "wan1p3b_ar_kvwindow": dict(batch=1, heads=12, grid=(3, 30, 52), block=0, window=32760, rope_grid=(21, 30, 52),
                                desc="causal (Self-Forcing) Wan-1.3B inference step: one block of 3 latent frames (4 680 rows) "
                                     "against the cached 21-frame window (32 760 keys), Plan.kv_window; the step is prologue of the "
                                     "block + write of its k/v into the cache tail + attention (keys cut in ranges when that fills "
                                     "the SMs better; FV_SPLITKV=0 turns that off)"),
    "tiny": dict(batch=1, heads=12, grid=(3, 8, 8), block=0, desc="tiny Wan-arch dense self-attention (192 tokens)"),
}
def _metric_name():
    """The metric string of the benchmark contract file when it sits beside this script."""
    try:
        return json.loads((ROOT / "BASELINE.json").read_text())["metric"]
    except Exception:
        return "Wan self-attn TFLOP/s/GPU (% of BF16 peak), dense+VSA, at 1/2/4/8 B200"


METRIC = _metric_name()
UNIT_NOTE = "value = whole-job TFLOP/s (prologue + attention); per GPU in per_gpu_tflops, fraction of peak in frac_of_bf16_peak_*"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(burst=float(d["bf16_tflops"]), sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    hbm=float(d["hbm_gbs"]), source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


def visible_pairs(seq: int, block: int) -> float:
    """Query-key pairs the mask lets through (dense: seq^2)."""
    if block <= 0:
        return float(seq) * seq
    total = 0.0
    for c0 in range(0, seq, block):
        rows = min(block, seq - c0)
        total += rows * float(min(seq, c0 + block))
    return total


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs (read-only)."""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index, self.lines, self.proc, self.note = index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); pw.append(float(f[3]))
            except ValueError:
                continue
            for n, val in zip(names, f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
        sm.sort()
        out = dict(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(mx), power_w_max=max(pw), samples=len(sm), reasons=sorted(reasons))
        if self.note:
            out["note"] = self.note
        return out


def reference_arm(args, wl):
    """The reference's CPU path on the host cores, on a bounded sample of the workload.

    Attention: `cpu_rows` query rows x `cpu_heads` heads against ALL keys of those heads (the composed f32
    SDPA).  Prologue: the host q/k RMSNorm + RoPE + head split on `cpu_tokens` tokens, all heads.  Both
    are scaled to the full workload by the work they cover (rows x heads, tokens) and combined into the
    same whole-step TFLOP/s the GPU arm reports."""
    import numpy as np
    from oracle import oracle as O
    O.build()
    batch, heads, grid, block = wl["batch"], wl["heads"], wl["grid"], wl["block"]
    seq = grid[0] * grid[1] * grid[2]
    dim = heads * 128
    hs = min(args.cpu_heads, heads)
    rows = np.sort(np.random.default_rng(0).choice(seq, size=min(args.cpu_rows, seq), replace=False)).astype(np.int32)
    window = wl.get("window", 0)
    keys = window or seq
    q, k, v = (O.bf16_round(O.seeded_normal(args.seed, 10 + i, (hs, seq if i == 0 else keys, 128))) for i in range(3))
    causal = (block, 0, 0) if block else None
    ntok = min(args.cpu_tokens, seq)
    proj = O.bf16_round(O.seeded_normal(args.seed, 0, (1, ntok, 3 * dim)))
    w = np.ones(dim, np.float32)
    cos, sin = O.wan_rope(*grid)
    cos, sin = cos[:ntok].copy(), sin[:ntok].copy()  # which positions the sample ropes does not change its cost
    t_attn, t_prep = [], []
    for i in range(args.warmup_cpu + args.steps_cpu):
        t0 = time.perf_counter()
        O.sdpa_rows(q, k, v, rows=rows, block_causal=causal)
        t1 = time.perf_counter()
        O.qk_norm_rope_bhsd(proj, w, cos, sin, 1, ntok, heads, 128, 3 * dim, 0)
        O.qk_norm_rope_bhsd(proj, w, cos, sin, 1, ntok, heads, 128, 3 * dim, dim)
        O.split_heads_bhsd(proj, 1, ntok, heads, 128, 3 * dim, 2 * dim)
        t2 = time.perf_counter()
        if i >= args.warmup_cpu:
            t_attn.append(t1 - t0)
            t_prep.append(t2 - t1)
    ta, tp = sorted(t_attn)[len(t_attn) // 2], sorted(t_prep)[len(t_prep) // 2]
    if block:
        vis_rows = sum(min(seq, (int(r) // block + 1) * block) for r in rows)
    else:
        vis_rows = len(rows) * keys
    sample_flops = 4.0 * hs * vis_rows * 128
    total_flops = 4.0 * batch * heads * (float(seq) * window if window else visible_pairs(seq, block)) * 128
    full_seconds = ta * (total_flops / sample_flops) + tp * (batch * seq / ntok)
    return dict(value=total_flops / full_seconds / 1e12, seconds=ta + tp, cores=O.num_threads(), attn_tflops=sample_flops / ta / 1e12,
                sample=f"attention: {len(rows)} of {seq} query rows x {hs} of {heads} heads x all keys ({sample_flops / 1e9:.1f} GFLOP in "
                       f"{ta:.2f} s); prologue: {ntok} of {batch * seq} tokens x all heads ({tp:.2f} s); scaled to the whole step by "
                       f"rows x heads and tokens (extrapolated whole step: {full_seconds:.0f} s)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="wan14b_720p_dense", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seed", type=int, default=20260927)
    ap.add_argument("--cpu-rows", type=int, default=2048, help="query rows of the CPU-baseline sample")
    ap.add_argument("--cpu-heads", type=int, default=4, help="heads of the CPU-baseline sample")
    ap.add_argument("--cpu-tokens", type=int, default=4096, help="tokens of the CPU-baseline prologue sample")
    ap.add_argument("--steps-cpu", type=int, default=1)
    ap.add_argument("--warmup-cpu", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    batch, heads, grid, block = wl["batch"], wl["heads"], wl["grid"], wl["block"]
    seq = grid[0] * grid[1] * grid[2]
    dim = heads * 128
    total_flops = 4.0 * batch * heads * visible_pairs(seq, block) * 128
    window = wl.get("window", 0)
    if window:
        total_flops = 4.0 * batch * heads * float(seq) * window * 128
    vsa_topk = wl.get("vsa_topk", 0)
    if vsa_topk:
        # the reference's count for the fine stage (padded slots, crates/fastvideo-gpucheck/src/kernels/vsa_dc.rs:648)
        # plus the coarse tile attention
        ntile = math.prod(-(-g // 4) for g in grid)
        total_flops = 4.0 * batch * heads * (ntile * 64.0) * (vsa_topk * 64.0) * 128 + 4.0 * batch * heads * ntile * ntile * 128
    # inputs read by one step; below 4 x the 126 MB L2 the bench writes a flush buffer between steps
    needs_flush = batch * seq * dim * 2 * 3 + 2 * batch * heads * window * 128 * 2 < 4 * 126e6
    cfg = dict(workload=f"{args.workload}: {wl['desc']}; b{batch} h{heads} S{seq} d128", seed=args.seed,
               l2="inputs exceed L2 (no flush needed)" if not needs_flush else
                  "L2 flushed between steps (512 MB written before each step, outside the per-step event pairs that are summed)",
               parallelism=f"sp{world}" if world > 1 else "single")

    if args.impl == "reference":
        if rank != 0:
            return
        if vsa_topk:
            print(json.dumps(dict(impl="reference", unavailable="the VSA workload's CPU arm is the oracle's vsa_attention_host, timed by "
                                  "tests only; run --impl reference on a dense workload")))
            return
        # whole --steps/--warmup run of bounded samples
        args.steps_cpu, args.warmup_cpu = max(1, min(args.steps, 3)), min(args.warmup, 1)
        r = reference_arm(args, wl)
        line = dict(metric=METRIC, value=r["value"], unit="TFLOP/s", n_gpus=args.gpus, steps=args.steps_cpu, warmup=args.warmup_cpu,
                    ms_per_step=r["seconds"] * 1e3, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="f32",
                    data="synthetic", config=cfg, impl="reference",
                    cpu_baseline=dict(value=r["value"], unit="TFLOP/s", cores=r["cores"], kind="port", sample=r["sample"]),
                    e2e=dict(value=r["value"], unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist
    from fastvideo_rs_b200 import sdpa, sp, wan

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the kernels have no CPU path (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if world != args.gpus and rank == 0:
        print(f"note: --gpus {args.gpus} but WORLD_SIZE {world}; using {world}", file=sys.stderr)

    # ---- synthetic inputs, resident in HBM: this rank's token shard of the fused QKV projection
    start, length = sp.shard_ranges(seq, world)[rank]
    gen = torch.Generator(device=dev)
    gen.manual_seed(args.seed + rank)
    proj = torch.randn((batch, length, 3 * dim), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    wq = torch.ones(dim, device=dev)
    wk = torch.ones(dim, device=dev)
    cos_all, sin_all = wan.wan_rope_tables_host(wl.get("rope_grid", grid))
    if window:  # the block is the last frames of the window's grid
        start = window - seq
    cos = torch.from_numpy(cos_all[start:start + length].copy()).to(dev)
    sin = torch.from_numpy(sin_all[start:start + length].copy()).to(dev)
    bh = batch * heads
    causal = sdpa.BlockCausal(block, 0, 0) if block else None
    if world > 1 and causal is not None:
        raise SystemExit("the chunk-causal workload is single-GPU in this bench")
    if vsa_topk and world > 1:
        raise SystemExit("the VSA workload is single-GPU in this bench")
    if window and world > 1:
        raise SystemExit("the KV-window workload is single-GPU in this bench")
    k_cache = v_cache = None
    if window:  # earlier blocks' keys and values, as the cache holds them: [b, h, window, 128] bf16
        k_cache, v_cache = (torch.randn((batch, heads, window, 128), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
                            for _ in range(2))
    spa = sp.SpAttention(seq, bh, device=dev) if world > 1 else None
    vsa_in = None
    if vsa_topk:
        from fastvideo_rs_b200 import vsa
        vctx = vsa.VsaCtx(grid, topk=vsa_topk)
        mk = lambda: torch.randn((bh, seq, 128), generator=gen, device=dev, dtype=torch.float32)
        vq, vk, vv = (mk().to(torch.bfloat16) for _ in range(3))
        vgate = torch.sigmoid(mk()).to(torch.bfloat16)
        vsa_in = torch.stack([vq, vk, vv, vgate])  # one tensor so the end-to-end leg copies it in one go
        proj = vsa_in
    out_buf = torch.empty((bh, length, 128), dtype=torch.bfloat16, device=dev)
    launches_per_step = 5 if vsa_topk else (2 if world == 1 else 2 + spa.groups)
    if window:  # prologue, attention, and the merge of the key ranges when the keys are cut
        split = os.environ.get("FV_SPLITKV", "1") != "0" and sdpa.splitkv_choose(
            bh, seq, window, torch.cuda.get_device_properties(dev).multi_processor_count) > 1
        launches_per_step = 3 if split else 2
    attn_events = []

    def step(p, record=False):
        if vsa_topk:
            if record:
                e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
            o = vsa.vsa_attention(p[0], p[1], p[2], p[3], vctx)
            if record:
                e1.record()
                attn_events.append((e0, e1))
            return o
        q, k, v = wan.qk_prep(p, wq, wk, cos, sin, heads)
        q, k, v = q.view(bh, length, 128), k.view(bh, length, 128), v.view(bh, length, 128)
        if record:
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
        if window:
            k_cache[:, :, window - seq:].copy_(k.view(batch, heads, seq, 128))
            v_cache[:, :, window - seq:].copy_(v.view(batch, heads, seq, 128))
            o = sdpa.sdpa(q.view(batch, heads, seq, 128), k_cache, v_cache, sdpa.Plan.kv_window()).view(bh, seq, 128)
        elif spa is not None:
            o = spa.forward(q, k, v, out=out_buf)
        else:
            o = sdpa.dense_fwd(q, k, v, causal=causal, out=out_buf)
        if record:
            e1.record()
            attn_events.append((e0, e1))
        return o

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step(proj)
    barrier()
    assert sdpa.device_status() == 0
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    step_events = []
    flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device=dev) if needs_flush else None
    for _ in range(args.steps):
        if needs_flush:
            flush_buf.fill_(1)
            s0 = torch.cuda.Event(enable_timing=True); s1 = torch.cuda.Event(enable_timing=True)
            s0.record()
        step(proj, record=True)
        if needs_flush:
            s1.record()
            step_events.append((s0, s1))
    t1.record()
    barrier()
    if world == 1 and len(sampler.lines) < 3:
        # a timed region shorter than nvidia-smi's start-up: keep the same load running until it has sampled
        deadline = time.time() + 4.0
        while len(sampler.lines) < 3 and time.time() < deadline:
            for _ in range(10):
                step(proj)
            torch.cuda.synchronize()
        sampler.note = "timed region shorter than the sampler's start-up: sampled under the same steps repeated right after it"
    clocks = sampler.stop() if rank == 0 else None
    ms_total = sum(a.elapsed_time(b) for a, b in step_events) if needs_flush else t0.elapsed_time(t1)
    attn_ms = sum(a.elapsed_time(b) for a, b in attn_events) / len(attn_events)
    assert sdpa.device_status() == 0

    # ---- end to end through the public API: pinned host projection in, host result out, every step
    e2e = None
    if not args.no_e2e:
        host_in = torch.empty(proj.shape, dtype=torch.bfloat16, pin_memory=True)
        host_in.copy_(proj)
        host_out = torch.empty(out_buf.shape, dtype=torch.bfloat16, pin_memory=True)
        dev_in = torch.empty_like(proj)
        n_e2e = max(2, min(args.steps, 5))

        def e2e_step():
            dev_in.copy_(host_in, non_blocking=True)
            o = step(dev_in)
            host_out.copy_(o, non_blocking=True)

        e2e_step()
        barrier()
        a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_e2e):
            e2e_step()
        b.record()
        barrier()
        e2e_ms = a.elapsed_time(b) / n_e2e
    t = torch.tensor([ms_total, attn_ms, e2e_ms if not args.no_e2e else 0.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, attn_ms, e2e_ms = (float(x) for x in t.tolist())
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    ms_step = ms_total / args.steps
    value = total_flops / (ms_step * 1e-3) / 1e12
    pk = peaks()
    rank_flops = total_flops / world
    achieved = rank_flops / (attn_ms * 1e-3) / 1e12
    # DRAM bytes per attention launch: measured on a smaller case of the same kernel (ncu dram__bytes_read.sum +
    # dram__bytes_write.sum of a 24-head x 8192-token capture: reads = 1.0007 x (Q + K + V), every output byte written
    # once) and scaled by the bytes of Q, K, V and O, which is what the traffic is proportional to.
    traffic = None if (vsa_topk or window) else int(4 * bh * length * 128 * 2 * 1.0005) + (2 * bh * (seq - length) * 128 * 2 if world > 1 else 0)
    line = dict(metric=METRIC, value=value, unit="TFLOP/s", n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
                ms_per_step=ms_step, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16", data="synthetic",
                config=cfg, value_note=UNIT_NOTE, per_gpu_tflops=value / world, frac_of_bf16_peak_burst=value / world / pk["burst"],
                frac_of_bf16_peak_sustained=value / world / pk["sustained"], peaks=pk,
                roofline=dict(bound="tensor", kernel="fv_vsa_fine_kernel (+4 small kernels in the timed span)" if vsa_topk else
                              ("fv_sdpa_fwd_d128 (+ cache-tail copies and fv_splitkv_merge_kernel in the timed span)" if window
                               else "fv_sdpa_fwd_d128"),
                              achieved=achieved, peak=pk["sustained"], unit="TFLOP/s",
                              frac=achieved / pk["sustained"], frac_of_burst=achieved / pk["burst"], of=pk["source"],
                              ms_per_launch_set=attn_ms, traffic=traffic,
                              note="attention launch(es) of one step timed with CUDA events inside the timed region; "
                                   "at N>1 this includes waiting for the K/V all-gather"),
                clocks=clocks, gpu_launches=launches_per_step * args.steps)
    if not args.no_e2e:
        line["e2e"] = dict(value=total_flops / (e2e_ms * 1e-3) / 1e12, unit="TFLOP/s", ms_per_step=e2e_ms,
                           h2d_bytes_per_step=proj.numel() * 2 * world, d2h_bytes_per_step=out_buf.numel() * 2 * world)
    if world == 1 and not args.no_cpu_baseline:
        r = reference_arm(args, wl)
        line["cpu_baseline"] = dict(value=r["value"], unit="TFLOP/s", cores=r["cores"], kind="port", sample=r["sample"],
                                    seconds=r["seconds"])
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
