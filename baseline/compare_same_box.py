#!/usr/bin/env python
"""Times this repository's attention kernel and the reference's own kernels (baseline/_ref/incumbent_driver,
built by baseline/build_incumbent.sh) back to back on ONE GPU at the benchmark configurations' shapes, and
prints a markdown table.  CUDA events, median of 5 launches after 2 warm-ups, both sides; clocks sampled with
nvidia-smi while each side runs.

    python baseline/compare_same_box.py [--quick]

Ours runs through tests/native/sdpa_check.bin (the torch-free checker, C ABI), theirs through the driver.
"""
import json
import subprocess
import sys
import threading
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
OURS = ROOT / "tests" / "native" / "sdpa_check.bin"
THEIRS = ROOT / "baseline" / "_ref" / "incumbent_driver"

# (label, bh, sq, sk, mask or None, reference kernel)
SHAPES = [
    ("config 1 self: 24 x 32 760^2", 24, 32760, 32760, None, "dc100"),
    ("config 1 cross: 24 x 32 760 x 512", 24, 32760, 512, None, "dc100"),
    ("config 3: 40 x 75 600^2", 40, 75600, 75600, None, "dc100"),
    ("config 4 chunk-causal: 12 x 32 760, 7 x 4 680", 12, 32760, 32760, (4680, 0, 0), "causal"),
    ("AR step: 12 x 4 680 x 32 760", 12, 4680, 32760, None, "dc100"),
    ("config 1 self, mma.sync V2", 24, 32760, 32760, None, "v2"),
]


class Clocks:
    def __init__(self):
        self.lines, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=clocks.sm,power.draw", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", "0"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True).start()
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()

    def median_mhz(self):
        v = sorted(float(l.split(",")[0]) for l in self.lines if l.strip())
        return v[len(v) // 2] if v else None


def last_json(out: str):
    for line in reversed(out.strip().splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    return {}


def main():
    quick = "--quick" in sys.argv
    if not OURS.exists() or not THEIRS.exists():
        raise SystemExit(f"need {OURS} and {THEIRS}")
    print("| shape | reference kernel | theirs ms | theirs TFLOP/s | ours ms | ours TFLOP/s | ours / theirs | SM MHz theirs / ours |")
    print("|---|---|---:|---:|---:|---:|---:|---|")
    for label, bh, sq, sk, mask, kern in SHAPES:
        if quick and bh * sq * sk > 3e10:
            continue
        case = f"{bh},{sq},{sk}" + (f",{mask[0]},{mask[1]},{mask[2]}" if mask else "")
        cmd_t = [str(THEIRS), kern, str(bh), str(sq), str(sk), "--bench", "5"] + (["--mask", ",".join(map(str, mask))] if mask else [])
        with Clocks() as ct:
            t = last_json(subprocess.run(cmd_t, capture_output=True, text=True, timeout=900).stdout)
        with Clocks() as co:
            o = last_json(subprocess.run([str(OURS), "--bench", "--case", case], capture_output=True, text=True, timeout=900).stdout.replace("OK (0 failing)", ""))
        if not t.get("ms") or not o.get("ms"):
            print(f"| {label} | {kern} | failed: {t} / {o} |")
            continue
        print(f"| {label} | `{kern}` | {t['ms']:.3f} | {t['tflops']:.0f} | {o['ms']:.3f} | {o['tflops']:.0f} | {t['ms'] / o['ms']:.2f} x | "
              f"{ct.median_mhz()} / {co.median_mhz()} |", flush=True)


if __name__ == "__main__":
    main()
