#!/usr/bin/env python
"""Benchmark of the Wan self-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]
                    [--sp-impl python|native] [--sp-exchange ce|nccl] [--no-extra]

One "step" = one pass of the path over one synthetic batch: the fused QKV projection (bf16, seeded
N(0,1), generated on the host with a counter-based generator so that every value is known there) goes
through the q/k prologue kernel (RMSNorm across heads + 3-D RoPE + head split) and the attention
kernel.  Default workload: Wan2.1-14B 720p x 81 frames dense self-attention (1 x 40 heads x 75 600
tokens x 128), sequence-parallel over N GPUs: token shards, the ranks' K and V blocks exchanged once
per step (copy-engine pulls from peer-mapped staging by default, --sp-exchange nccl for the NCCL
all-gather) under the attention over the local keys.  Total work is fixed as N grows ("strong").

Prints ONE JSON line (rank 0).  FLOPs = 4 * bh * sq * sk_visible * d (the reference's formula,
crates/fastvideo-gpucheck/src/kernels/attn2.rs:466).
  value     whole-job TFLOP/s with inputs resident in HBM
  e2e       the same metric with every step's projection coming from pinned host memory and its result
            going back to the host inside the timed region (double-buffered, copies on their own streams)
  parity    the step's output checked OUTSIDE the timed region against the CPU oracle on sampled rows of
            every rank (all keys), and the prologue on sampled tokens; the run exits non-zero when it fails
  extra     (1 GPU, default workload only) short runs of the other configurations, each with its own
            clocks record and parity check

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
    # name: batch, heads, grid (frames, h, w in patches), causal block tokens (0 = dense)
    "wan14b_720p_dense": dict(batch=1, heads=40, grid=(21, 45, 80), block=0, desc="Wan2.1-14B 720p x81f dense self-attention"),
    "wan1p3b_480p_dense": dict(batch=2, heads=12, grid=(21, 30, 52), block=0, desc="Wan2.1-1.3B 480p x81f dense self-attention, CFG pair"),
    "wan1p3b_480p_cross": dict(batch=2, heads=12, grid=(21, 30, 52), block=0, cross=512,
                               desc="Wan2.1-1.3B 480p cross-attention to 512 text tokens, CFG pair (q through the prologue without RoPE; "
                                    "text K/V seeded N(0,1) bf16, as a per-denoise cache holds them)"),
    "wan1p3b_480p_causal": dict(batch=1, heads=12, grid=(21, 30, 52), block=4680, desc="Self-Forcing chunk-causal (7 chunks x 3 frames) at the Wan-1.3B shape"),
    "wan1p3b_480p_vsa": dict(batch=1, heads=12, grid=(21, 30, 52), block=0, vsa_topk=78,
                             desc="VSA block-sparse self-attention at the Wan-1.3B 480p grid: 624 tiles of 64 tokens, top-k 78 (12.5 %), "
                                  "sigmoid gate applied to seeded logits before the call"),
    "wan1p3b_ar_kvwindow": dict(batch=1, heads=12, grid=(3, 30, 52), block=0, window=32760, rope_grid=(21, 30, 52),
                                desc="causal (Self-Forcing) Wan-1.3B inference step: one block of 3 latent frames (4 680 rows) "
                                     "against the cached 21-frame window (32 760 keys), Plan.kv_window; the step is prologue of the "
                                     "block, which writes its k/v into the cache tail, + attention (keys cut in ranges when that fills "
                                     "the SMs better; FV_SPLITKV=0 turns that off)"),
    "tiny": dict(batch=1, heads=12, grid=(3, 8, 8), block=0, desc="tiny Wan-arch dense self-attention (192 tokens)"),
}
EXTRA = ["wan1p3b_480p_dense", "wan1p3b_480p_cross", "wan1p3b_480p_vsa", "wan1p3b_480p_causal", "wan1p3b_ar_kvwindow"]


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


def workload_flops(wl) -> float:
    batch, heads, grid, block = wl["batch"], wl["heads"], wl["grid"], wl["block"]
    seq = grid[0] * grid[1] * grid[2]
    if wl.get("window"):
        return 4.0 * batch * heads * float(seq) * wl["window"] * 128
    if wl.get("cross"):
        return 4.0 * batch * heads * float(seq) * wl["cross"] * 128
    if wl.get("vsa_topk"):
        # the reference's count for the fine stage (padded slots, crates/fastvideo-gpucheck/src/kernels/vsa_dc.rs:648)
        # plus the coarse tile attention
        ntile = math.prod(-(-g // 4) for g in grid)
        return 4.0 * batch * heads * (ntile * 64.0) * (wl["vsa_topk"] * 64.0) * 128 + 4.0 * batch * heads * ntile * ntile * 128
    return 4.0 * batch * heads * visible_pairs(seq, block) * 128


# ---------------------------------------------------------------------------------- seeded inputs
GEN_BLOCK = 1050  # tokens per generator stream: a shard of any rank count is cut out of whole streams


def seeded_normal(seed: int, stream: int, shape):
    """i.i.d. N(0,1) float32 from numpy's counter-based Philox generator, key = seed, stream in the high word:
    the same (seed, stream, shape) gives the same values on any machine."""
    import numpy as np
    return np.random.Generator(np.random.Philox(key=int(seed) + (int(stream) << 32))).standard_normal(size=shape, dtype=np.float32)


def seeded_rows(seed: int, tensor: int, t0: int, t1: int, width: int):
    """Rows [t0, t1) of the seeded [*, width] tensor number `tensor`, whatever the caller's shard: the tensor is
    defined in streams of GEN_BLOCK rows."""
    import numpy as np
    parts = []
    for blk in range(t0 // GEN_BLOCK, (t1 - 1) // GEN_BLOCK + 1 if t1 > t0 else 0):
        rows = seeded_normal(seed, 1000 + tensor * 100000 + blk, (GEN_BLOCK, width))
        lo, hi = max(t0 - blk * GEN_BLOCK, 0), min(t1 - blk * GEN_BLOCK, GEN_BLOCK)
        parts.append(rows[lo:hi])
    return np.concatenate(parts, 0) if parts else np.empty((0, width), np.float32)


def to_dev_bf16(x, dev):
    import torch
    return torch.from_numpy(x).to(dev).to(torch.bfloat16)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs (read-only)."""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index, self.lines, self.proc, self.note = index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "25",
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
    keys = wl.get("window", 0) or wl.get("cross", 0) or seq
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
    total_flops = workload_flops(wl)
    full_seconds = ta * (total_flops / sample_flops) + tp * (batch * seq / ntok)
    return dict(value=total_flops / full_seconds / 1e12, seconds=ta + tp, cores=O.num_threads(), attn_tflops=sample_flops / ta / 1e12,
                sample=f"attention: {len(rows)} of {seq} query rows x {hs} of {heads} heads x all keys ({sample_flops / 1e9:.1f} GFLOP in "
                       f"{ta:.2f} s); prologue: {ntok} of {batch * seq} tokens x all heads ({tp:.2f} s); scaled to the whole step by "
                       f"rows x heads and tokens (extrapolated whole step: {full_seconds:.0f} s)")


# ------------------------------------------------------------------------------------- the GPU arm
class Bench:
    """One workload on this rank's GPU: seeded inputs, the step, its timing and its parity check."""

    def __init__(self, name, args, rank, world, dev):
        import numpy as np
        import torch
        from fastvideo_rs_b200 import sdpa, sp, wan
        self.torch, self.np, self.sdpa, self.sp, self.wan = torch, np, sdpa, sp, wan
        self.name, self.wl, self.args, self.rank, self.world, self.dev = name, WORKLOADS[name], args, rank, world, dev
        wl = self.wl
        self.batch, self.heads, self.grid, self.block = wl["batch"], wl["heads"], wl["grid"], wl["block"]
        self.seq = self.grid[0] * self.grid[1] * self.grid[2]
        self.dim, self.bh = self.heads * 128, self.batch * self.heads
        self.window, self.cross, self.vsa_topk = wl.get("window", 0), wl.get("cross", 0), wl.get("vsa_topk", 0)
        if world > 1 and (self.window or self.cross or self.vsa_topk):
            raise SystemExit(f"the {name} workload is single-GPU in this bench")
        self.causal = sdpa.BlockCausal(self.block, 0, 0) if self.block else None
        # sequence-parallel layout: contiguous shards; zig-zag pieces under the causal mask (balanced work)
        self.layout = sp.SpLayout(self.seq, world, rank, zigzag=bool(self.block) and world > 1)
        self.rows = self.layout.rows()
        self.length = len(self.rows)
        seed = args.seed
        runs = [(s, l) for s, l in self.layout.runs[rank] if l > 0]
        # ---- inputs, resident in HBM (every value reproducible on the host)
        cos_all, sin_all = wan.wan_rope_tables_host(wl.get("rope_grid", self.grid))
        off = self.window - self.seq if self.window else 0  # the block is the last frames of the window's grid
        idx = np.asarray(self.rows, np.int64) + off
        self.cos_h, self.sin_h = cos_all[idx].copy(), sin_all[idx].copy()
        self.cos = None if self.cross else torch.from_numpy(self.cos_h).to(dev)
        self.sin = None if self.cross else torch.from_numpy(self.sin_h).to(dev)
        self.wq = torch.ones(self.dim, device=dev)
        self.wk = torch.ones(self.dim, device=dev)
        if self.vsa_topk:
            from fastvideo_rs_b200 import vsa
            self.vsa = vsa
            self.vctx = vsa.VsaCtx(self.grid, topk=self.vsa_topk)
            ts = [seeded_rows(seed, 20 + i, 0, self.bh * self.seq, 128).reshape(self.bh, self.seq, 128) for i in range(4)]
            ts[3] = 1.0 / (1.0 + np.exp(-ts[3]))  # the gate is linear in the reference: the sigmoid is the caller's
            self.proj = torch.stack([to_dev_bf16(t, dev) for t in ts])  # one tensor: the end-to-end leg copies it in one go
        else:
            parts = [np.concatenate([seeded_rows(seed, b, s, s + l, 3 * self.dim) for s, l in runs], 0) if runs
                     else np.empty((0, 3 * self.dim), np.float32) for b in range(self.batch)]
            self.proj = to_dev_bf16(np.stack(parts), dev)  # [batch, length, 3 * dim]
        self.k_cache = self.v_cache = self.text_k = self.text_v = None
        if self.window:  # earlier blocks' keys and values, as the cache holds them: [b, h, window, 128] bf16
            self.k_cache, self.v_cache = (to_dev_bf16(seeded_rows(seed, 30 + i, 0, self.bh * self.window, 128)
                                                      .reshape(self.batch, self.heads, self.window, 128), dev) for i in range(2))
        if self.cross:
            self.text_k, self.text_v = (to_dev_bf16(seeded_rows(seed, 40 + i, 0, self.bh * self.cross, 128)
                                                    .reshape(self.bh, self.cross, 128), dev) for i in range(2))
        self.spa = None
        if world > 1:
            if args.sp_impl == "native":
                import torch.distributed as dist
                ids = [sp.NativeSp.unique_id() if rank == 0 else None]
                dist.broadcast_object_list(ids, src=0)
                self.spa = sp.NativeSp(self.seq, self.bh, world, rank, ids[0])
                if self.block:
                    raise SystemExit("the native handle shards contiguously: run the causal workload with --sp-impl python")
            else:
                self.spa = sp.SpAttention(self.seq, self.bh, device=dev, zigzag=self.layout.zigzag, exchange=args.sp_exchange)
        self.out_buf = torch.empty((self.bh, self.length, 128), dtype=torch.bfloat16, device=dev)
        self.attn_events = []
        self.last_qkv = None
        props = torch.cuda.get_device_properties(dev)
        self.split = bool(self.window) and os.environ.get("FV_SPLITKV", "1") != "0" and \
            sdpa.splitkv_choose(self.bh, self.seq, self.window, props.multi_processor_count) > 1
        # inputs read by one step; below 4 x the 126 MB L2 the bench writes a flush buffer between steps
        self.needs_flush = self.proj.numel() * 2 + 2 * self.bh * (self.window + self.cross) * 128 * 2 < 4 * 126e6
        self.flops = workload_flops(self.wl)

    def remote_passes(self):
        """Attention launches of one step after the local pass."""
        if getattr(self.spa, "exchange", "nccl") != "ce":
            # Python nccl exchange: one pass over everything the all-gather brought; the native handle: one remote pass
            # per head group
            return 1 if hasattr(self.spa, "exchange") else getattr(self.spa, "groups", 1)
        return len(self.layout.source_groups(self.causal, self.spa.grouped))

    def launches_per_step(self):
        if self.vsa_topk:
            return 5
        if self.window:
            return 3 if self.split else 2  # prologue, attention, and the merge of the key ranges when the keys are cut
        if self.spa is not None:
            return 2 + self.remote_passes()
        return 2

    def step(self, p, record=False, keep=False):
        torch = self.torch
        e0 = e1 = None
        if self.vsa_topk:
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            o = self.vsa.vsa_attention(p[0], p[1], p[2], p[3], self.vctx)
            if record:
                e1.record()
                self.attn_events.append((e0, e1))
            return o
        n = self.length
        if self.window:  # the block's K and V go straight into the cache tail (no copy launches)
            q, k, v = self.wan.qk_prep(p, self.wq, self.wk, self.cos, self.sin, self.heads,
                                       cache=(self.k_cache, self.v_cache, self.window - self.seq))
        else:
            q, k, v = self.wan.qk_prep(p, self.wq, self.wk, self.cos, self.sin, self.heads, want_k=not self.cross, want_v=not self.cross)
        q = q.view(self.bh, n, 128)
        if not self.cross and not self.window:
            k, v = k.view(self.bh, n, 128), v.view(self.bh, n, 128)
        if keep:
            self.last_qkv = (q, k, v)
        if record:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        if self.window:
            o = self.sdpa.sdpa(q.view(self.batch, self.heads, self.seq, 128), self.k_cache, self.v_cache,
                               self.sdpa.Plan.kv_window()).view(self.bh, self.seq, 128)
        elif self.cross:
            o = self.sdpa.dense_fwd(q, self.text_k, self.text_v, out=self.out_buf)
        elif self.spa is not None:
            o = self.spa.forward(q, k, v, out=self.out_buf, causal=self.causal)
        else:
            o = self.sdpa.dense_fwd(q, k, v, causal=self.causal, out=self.out_buf)
        if record:
            e1.record()
            self.attn_events.append((e0, e1))
        return o

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        self.torch.cuda.synchronize()

    def timed(self, steps, warmup, local_rank, min_seconds=0.0):
        """W warm-up steps, then `steps` timed ones bracketed by a barrier and a synchronize on both sides; at least
        `min_seconds` of them (more steps are added, all inside the timed region) so that the clock sampler sees
        the load.  Returns (ms per step, attention ms per step, clocks, steps run)."""
        torch = self.torch
        for _ in range(max(warmup, 3)):
            self.step(self.proj)
        self.barrier()
        assert self.sdpa.device_status() == 0
        if min_seconds > 0:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            self.step(self.proj)
            b.record()
            torch.cuda.synchronize()
            steps = max(steps, int(min_seconds * 1e3 / max(a.elapsed_time(b), 1e-3)) + 1)
        sampler = ClockSampler(local_rank)
        if self.rank == 0:
            sampler.start()
            if min_seconds > 0:
                time.sleep(0.35)  # nvidia-smi's start-up
        self.attn_events = []
        step_events = []
        flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device=self.dev) if self.needs_flush else None
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        t0.record()
        for _ in range(steps):
            if self.needs_flush:
                flush_buf.fill_(1)
                s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s0.record()
            self.step(self.proj, record=True)
            if self.needs_flush:
                s1.record()
                step_events.append((s0, s1))
        t1.record()
        self.barrier()
        clocks = sampler.stop() if self.rank == 0 else None
        ms_total = sum(a.elapsed_time(b) for a, b in step_events) if self.needs_flush else t0.elapsed_time(t1)
        attn_ms = sum(a.elapsed_time(b) for a, b in self.attn_events) / len(self.attn_events)
        assert self.sdpa.device_status() == 0
        return ms_total / steps, attn_ms, clocks, steps

    def e2e(self, steps):
        """The same step through the public API with HOST buffers: every step's input is copied from pinned host
        memory and its result copied back, all inside the timed region.  The copies run on their own streams and
        the device buffers are double-buffered (wan.HostStaged), so step i computes while step i + 1 arrives and
        step i - 1 leaves."""
        torch = self.torch
        host_in = torch.empty(self.proj.shape, dtype=torch.bfloat16, pin_memory=True)
        host_in.copy_(self.proj)
        host_out = torch.empty(self.out_buf.shape if not self.vsa_topk else (self.bh, self.seq, 128), dtype=torch.bfloat16, pin_memory=True)
        pipe = self.wan.HostStaged(host_in.shape, host_out.shape, self.dev)
        pipe.run([host_in] * 2, [host_out] * 2, self.step)  # warm-up (allocations, first-touch of the pinned pages)
        self.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        pipe.run([host_in] * steps, [host_out] * steps, self.step)
        b.record()
        self.barrier()
        return a.elapsed_time(b) / steps, host_in.numel() * 2, host_out.numel() * 2

    # ------------------------------------------------------------------------------------ parity
    def parity(self):
        """Outside any timed region: (1) the prologue on sampled tokens of this rank against the oracle's host
        prologue of the same seeded projection rows; (2) this rank's output on sampled rows (shard ends, work-item
        and tile edges, a random spread) x 2 planes against the oracle's composed f32 SDPA over ALL keys, the K
        and V of every rank gathered to the host.  Tolerance of the attention output: max-abs 2e-2, mean-abs 2e-3
        (BASELINE.json); of the prologue: 2^-7 relative + 1e-2 (one bf16 rounding of values up to ~4)."""
        torch, np = self.torch, self.np
        from oracle import oracle as O
        O.build()
        if self.vsa_topk:
            return dict(ok=None, note="not checked here: the VSA operator is checked on this very grid, every row of the tile selection "
                                      "included, by tests/test_gpu_vsa.py; its CPU oracle takes minutes at this size")
        o = self.step(self.proj, keep=True).float()
        torch.cuda.synchronize()
        q, k, v = self.last_qkv
        rng = np.random.default_rng(1234 + self.rank)
        n = self.length
        planes = sorted({0, self.bh - 1})
        tix = lambda a: torch.from_numpy(np.asarray(a, np.int64)).to(self.dev)
        res = dict(planes=planes)
        # (1) prologue
        if n:
            toks = np.unique(np.concatenate([[0, n - 1], rng.integers(0, n, 14)])).astype(np.int64)
            b_of = lambda pl: pl // self.heads
            worst = 0.0
            for b in sorted({b_of(pl) for pl in planes}):
                rows_h = O.bf16_round(self.proj[b][tix(toks)].float().cpu().numpy()[None])  # [1, t, 3 dim], exactly the bf16 values
                w = np.ones(self.dim, np.float32)
                if self.cross:
                    cos = np.ones((len(toks), 128), np.float32); sin = np.zeros((len(toks), 128), np.float32)
                else:
                    cos, sin = self.cos_h[toks], self.sin_h[toks]
                cols = [(q, 0)] if self.cross else [(q, 0), (k, self.dim)]
                for t, col in cols:
                    want = O.qk_norm_rope_bhsd(rows_h, w, cos, sin, 1, len(toks), self.heads, 128, 3 * self.dim, col)  # [heads, t, 128]
                    got = t.view(self.batch, self.heads, n, 128)[b][:, tix(toks)].float().cpu().numpy()
                    worst = max(worst, float(np.max(np.abs(got - want) - np.abs(want) * 2.0 ** -7)))
                if not self.cross:
                    want = O.split_heads_bhsd(rows_h, 1, len(toks), self.heads, 128, 3 * self.dim, 2 * self.dim)
                    got = v.view(self.batch, self.heads, n, 128)[b][:, tix(toks)].float().cpu().numpy()
                    worst = max(worst, float(np.max(np.abs(got - want))))
            res["prologue_excess"] = worst
            res["prologue_ok"] = bool(worst <= 1e-2)
        # (2) attention over all keys
        edges = [0, 1, 127, 128, 255, 256, 257, n // 2, n - 258, n - 257, n - 256, n - 2, n - 1]
        if self.layout.nrun == 2:
            edges += [self.layout.runs[self.rank][0][1] - 1, self.layout.runs[self.rank][0][1]]
        local = np.unique(np.concatenate([[e for e in edges if 0 <= e < n], rng.integers(0, max(n, 1), 20)])).astype(np.int64) if n else \
            np.empty(0, np.int64)
        glob = np.asarray(self.rows, np.int64)[local] if n else local
        got = o[planes][:, tix(local)].cpu().numpy() if n else np.empty((len(planes), 0, 128), np.float32)
        if self.window:
            kk, vv = (t.view(self.bh, self.window, 128)[planes].float().cpu().numpy() for t in (self.k_cache, self.v_cache))
            qq = q[planes].float().cpu().numpy()
            want = O.sdpa_rows(qq, kk, vv, rows=local.astype(np.int32))
        elif self.cross:
            kk, vv = (t[planes].float().cpu().numpy() for t in (self.text_k, self.text_v))
            want = O.sdpa_rows(q[planes].float().cpu().numpy(), kk, vv, rows=local.astype(np.int32))
        else:
            # every rank's q, k, v rows of the two planes, put back in sequence order on rank 0
            mine = torch.stack([q[planes], k[planes], v[planes]]).contiguous()  # [3, planes, n, 128]
            full = None
            if self.world > 1:
                import torch.distributed as dist
                lens = [len(self.layout.rows(r)) for r in range(self.world)]
                pad = torch.zeros((3, len(planes), max(lens), 128), dtype=torch.bfloat16, device=self.dev)
                pad[:, :, :n] = mine
                bufs = [torch.empty_like(pad) for _ in range(self.world)] if self.rank == 0 else None
                dist.gather(pad, bufs, dst=0)
                pg = torch.zeros((len(planes), 64, 128), dtype=torch.float32, device=self.dev)
                pr = torch.full((64,), -1, dtype=torch.int64, device=self.dev)
                pg[:, :len(local)] = torch.from_numpy(got).to(self.dev)
                pr[:len(local)] = torch.from_numpy(glob).to(self.dev)
                gots = [torch.empty_like(pg) for _ in range(self.world)] if self.rank == 0 else None
                rws = [torch.empty_like(pr) for _ in range(self.world)] if self.rank == 0 else None
                dist.gather(pg, gots, dst=0)
                dist.gather(pr, rws, dst=0)
                if self.rank != 0:
                    return None
                full = np.zeros((3, len(planes), self.seq, 128), np.float32)
                for r in range(self.world):
                    rr = np.asarray(self.layout.rows(r), np.int64)
                    full[:, :, rr] = bufs[r][:, :, :len(rr)].float().cpu().numpy()
                keep = [(rws[r] >= 0).cpu().numpy() for r in range(self.world)]
                glob = np.concatenate([rws[r].cpu().numpy()[keep[r]] for r in range(self.world)])
                got = np.concatenate([gots[r].cpu().numpy()[:, keep[r]] for r in range(self.world)], 1)
            else:
                full = mine.float().cpu().numpy()
            want = O.sdpa_rows(full[0], full[1], full[2], rows=glob.astype(np.int32),
                               block_causal=(self.block, 0, 0) if self.block else None)
        err = np.abs(got - want)
        res.update(max_abs=float(err.max()) if err.size else 0.0, mean_abs=float(err.mean()) if err.size else 0.0,
                   rows=int(got.shape[1]), keys="all", finite=bool(np.isfinite(got).all()))
        res["ok"] = bool(res["finite"] and res["max_abs"] <= 2e-2 and res["mean_abs"] <= 2e-3 and res.get("prologue_ok", True))
        return res


def roofline_of(b: Bench, attn_ms, pk):
    rank_flops = b.flops / b.world
    achieved = rank_flops / (attn_ms * 1e-3) / 1e12
    kernel = "fv_vsa_fine_kernel (+4 small kernels in the timed span)" if b.vsa_topk else \
        ("fv_attn_fwd_d128 (+ fv_splitkv_merge_kernel in the timed span)" if b.window else "fv_attn_fwd_d128")
    # DRAM bytes per attention launch: measured on a smaller case of the same kernel (ncu dram__bytes_read.sum +
    # dram__bytes_write.sum of a 24-head x 8192-token capture: reads = 1.0007 x (Q + K + V), every output byte written
    # once) and scaled by the bytes of Q, K, V and O, which is what the traffic is proportional to.
    traffic = None if (b.vsa_topk or b.window or b.cross) else \
        int(4 * b.bh * b.length * 128 * 2 * 1.0005) + (2 * b.bh * (b.seq - b.length) * 128 * 2 if b.world > 1 else 0)
    return dict(bound="tensor", kernel=kernel, achieved=achieved, peak=pk["sustained"], unit="TFLOP/s", frac=achieved / pk["sustained"],
                frac_of_burst=achieved / pk["burst"], of=pk["source"], ms_per_launch_set=attn_ms, traffic=traffic,
                note="attention launch(es) of one step timed with CUDA events inside the timed region; at N>1 this includes "
                     "waiting for the K/V exchange")


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
    ap.add_argument("--no-extra", action="store_true", help="skip the short runs of the other configurations")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--sp-impl", default="python", choices=["python", "native"],
                    help="N > 1: the Python SpAttention or the C-ABI handle fv_sp_* (what a host that is not Python binds)")
    ap.add_argument("--sp-exchange", default=None, choices=["ce", "nccl"],
                    help="N > 1, --sp-impl python: copy-engine pulls from peer-mapped staging (default) or the NCCL all-gather")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    seq = wl["grid"][0] * wl["grid"][1] * wl["grid"][2]

    def config_of(b=None, name=args.workload):
        w = WORKLOADS[name]
        s = w["grid"][0] * w["grid"][1] * w["grid"][2]
        cfg = dict(workload=f"{name}: {w['desc']}; b{w['batch']} h{w['heads']} S{s} d128", seed=args.seed,
                   parallelism=f"sp{world}" if world > 1 else "single")
        if b is not None:
            cfg["l2"] = "inputs exceed L2 (no flush needed)" if not b.needs_flush else \
                "L2 flushed between steps (512 MB written before each step, outside the per-step event pairs that are summed)"
            if world > 1:
                cfg["sp"] = dict(impl=args.sp_impl, exchange=getattr(b.spa, "exchange", "nccl"), shards="zigzag" if b.layout.zigzag else "contiguous",
                                 passes=1 + b.remote_passes())
        return cfg

    if args.impl == "reference":
        if rank != 0:
            return
        if wl.get("vsa_topk"):
            print(json.dumps(dict(impl="reference", unavailable="the VSA workload's CPU arm is the oracle's vsa_attention_host, timed by "
                                  "tests only; run --impl reference on a dense workload")))
            return
        # whole --steps/--warmup run of bounded samples
        args.steps_cpu, args.warmup_cpu = max(1, min(args.steps, 3)), min(args.warmup, 1)
        r = reference_arm(args, wl)
        line = dict(metric=METRIC, value=r["value"], unit="TFLOP/s", n_gpus=args.gpus, steps=args.steps_cpu, warmup=args.warmup_cpu,
                    ms_per_step=r["seconds"] * 1e3, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="f32",
                    data="synthetic", config=config_of(), impl="reference",
                    cpu_baseline=dict(value=r["value"], unit="TFLOP/s", cores=r["cores"], kind="port", sample=r["sample"]),
                    e2e=dict(value=r["value"], unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist
    from fastvideo_rs_b200 import _lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the kernels have no CPU path (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if world != args.gpus and rank == 0:
        print(f"note: --gpus {args.gpus} but WORLD_SIZE {world}; using {world}", file=sys.stderr)

    pk = peaks()
    b = Bench(args.workload, args, rank, world, dev)
    ms_step, attn_ms, clocks, steps = b.timed(args.steps, args.warmup, local_rank)
    kernel_line = _lib.last_kernel()
    e2e_ms = h2d = d2h = 0.0
    if not args.no_e2e:
        e2e_ms, h2d, d2h = b.e2e(max(args.steps, 2))
    par = None if args.no_parity else b.parity()
    t = torch.tensor([ms_step, attn_ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step, attn_ms, e2e_ms = (float(x) for x in t.tolist())
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    value = b.flops / (ms_step * 1e-3) / 1e12
    line = dict(metric=METRIC, value=value, unit="TFLOP/s", n_gpus=world, steps=steps, warmup=max(args.warmup, 3),
                ms_per_step=ms_step, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16", data="synthetic",
                config=config_of(b), value_note=UNIT_NOTE, per_gpu_tflops=value / world, frac_of_bf16_peak_burst=value / world / pk["burst"],
                frac_of_bf16_peak_sustained=value / world / pk["sustained"], peaks=pk, roofline=roofline_of(b, attn_ms, pk),
                clocks=clocks, gpu_launches=b.launches_per_step() * steps, last_kernel=kernel_line, parity=par)
    if clocks and clocks.get("sm_mhz"):
        # time x clock: comparable across rank counts that run at different clocks under the power cap
        line["ms_x_ghz"] = ms_step * clocks["sm_mhz"] / 1e3
    if not args.no_e2e:
        line["e2e"] = dict(value=b.flops / (e2e_ms * 1e-3) / 1e12, unit="TFLOP/s", ms_per_step=e2e_ms,
                           h2d_bytes_per_step=int(h2d) * world, d2h_bytes_per_step=int(d2h) * world,
                           host_link_gbs_per_gpu=(h2d + d2h) / (e2e_ms * 1e-3) / 1e9,
                           note="pinned host buffers, double-buffered device staging, copies on their own streams, all inside the timed region")
    if world == 1 and not args.no_cpu_baseline:
        r = reference_arm(args, wl)
        line["cpu_baseline"] = dict(value=r["value"], unit="TFLOP/s", cores=r["cores"], kind="port", sample=r["sample"],
                                    seconds=r["seconds"])
    if world == 1 and not args.no_extra and args.workload == "wan14b_720p_dense":
        del b
        torch.cuda.empty_cache()
        extra = []
        for name in EXTRA:
            x = Bench(name, args, rank, world, dev)
            ms, ams, clk, n = x.timed(5, 3, local_rank, min_seconds=1.0)
            xp = None if args.no_parity else x.parity()
            tf = x.flops / (ms * 1e-3) / 1e12
            extra.append(dict(workload=config_of(x, name)["workload"], ms_per_step=ms, steps=n, tflops=tf, attention_ms=ams,
                              attention_tflops=x.flops / (ams * 1e-3) / 1e12, frac_of_sustained=tf / pk["sustained"],
                              frac_of_burst=tf / pk["burst"], l2=config_of(x, name)["l2"], clocks=clk, parity=xp,
                              gpu_launches=x.launches_per_step() * n))
            del x
            torch.cuda.empty_cache()
        line["extra"] = extra
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    bad = [p for p in [par] + [e["parity"] for e in line.get("extra", [])] if p and p.get("ok") is False]
    if bad:
        print(f"parity check failed: {bad}", file=sys.stderr)
        sys.exit(3)


if __name__ == "__main__":
    main()
