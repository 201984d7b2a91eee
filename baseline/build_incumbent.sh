#!/bin/bash
# Compiles the reference's own standalone harness of its sm_100a attention kernels (the incumbent this
# repository is measured against) from the read-only reference tree, where its sources lie, into the
# git-ignored baseline/_ref/.  Nothing of the reference is copied into this repository.  Recipe:
# scripts/gpu/upstream/pod.sh:221-246 of the reference, without its -DDC_DEBUG_HANG debug build.
#   usage: baseline/build_incumbent.sh <reference root>     (or FV_REFERENCE_ROOT=<reference root>)
set -e
REF=${1:-${FV_REFERENCE_ROOT:-}}
[ -n "$REF" ] || { echo "usage: $0 <reference root>"; exit 2; }
HERE=$(cd "$(dirname "$0")" && pwd)
SRC=$REF/scripts/gpu/upstream/attn_dc_bench.cu
[ -f "$SRC" ] || { echo "no reference tree at $REF: nothing built"; exit 0; }
mkdir -p "$HERE/_ref"
OUT=$HERE/_ref/attn_dc_bench
if [ -x "$OUT" ] && [ "$OUT" -nt "$SRC" ]; then echo "$OUT is up to date"; exit 0; fi
nvcc -std=c++17 -O3 -arch=sm_100a --fmad=true --prec-div=true --prec-sqrt=true --ftz=false -o "$OUT" "$SRC"
echo "built $OUT"
