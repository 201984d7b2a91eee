#!/bin/bash
# Compiles, from the read-only reference tree where its sources lie, into the git-ignored baseline/_ref/:
#   attn_dc_bench      the reference's own standalone harness of its sm_100a attention kernels
#   incumbent_driver   this repository's driver (baseline/incumbent_driver.cu) around the reference's kernels
# Nothing of the reference is copied into this repository.  Recipe: scripts/gpu/upstream/pod.sh:221-246 of
# the reference, without its -DDC_DEBUG_HANG debug build.
#   usage: baseline/build_incumbent.sh <reference root>     (or FV_REFERENCE_ROOT=<reference root>)
set -e
REF=${1:-${FV_REFERENCE_ROOT:-}}
[ -n "$REF" ] || { echo "usage: $0 <reference root>"; exit 2; }
HERE=$(cd "$(dirname "$0")" && pwd)
SRC=$REF/scripts/gpu/upstream/attn_dc_bench.cu
[ -f "$SRC" ] || { echo "no reference tree at $REF: nothing built"; exit 0; }
mkdir -p "$HERE/_ref"
FLAGS="-std=c++17 -O3 -arch=sm_100a --fmad=true --prec-div=true --prec-sqrt=true --ftz=false"
OUT=$HERE/_ref/attn_dc_bench
if [ -x "$OUT" ] && [ "$OUT" -nt "$SRC" ]; then echo "$OUT is up to date"; else nvcc $FLAGS -o "$OUT" "$SRC"; echo "built $OUT"; fi
DRV=$HERE/_ref/incumbent_driver
if [ -x "$DRV" ] && [ "$DRV" -nt "$HERE/incumbent_driver.cu" ]; then echo "$DRV is up to date"; else
  nvcc $FLAGS -I "$REF" -o "$DRV" "$HERE/incumbent_driver.cu"; echo "built $DRV"; fi
