#!/bin/bash
# Per-layer sweep over batch sizes and implementations, in the spirit of the reference's comparison/test.sh:
# for one VGG-16 layer (1..9) run layoutCompare for batch 1..64 in NCHW / NHWC / CHWN and for the cuDNN modes,
# scrape the "time:<ms> ms" lines and write one row of 20 timings per batch to result/layer<L>.out.
# Usage: sweep.sh <layer> [dtype=fp32|tf32|bf16] [outdir=result]
set -u
layer=${1:-6}
dtype=${2:-fp32}
outdir=${3:-result}
here=$(cd "$(dirname "$0")" && pwd)
exe=$here/bin/layoutCompare
mkdir -p "$outdir"
out=$outdir/layer${layer}_${dtype}.out
: > "$out"
for name_opt in NCHW:0 NHWC:1 CHWN:2 cuDNN_nonfused_NCHW:3 cuDNN_fused_NCHW:4 cuDNN_best_NCHW:7 cuDNN_best_NHWC:8; do
    name=${name_opt%%:*}; opt=${name_opt##*:}
    if [ "$dtype" != fp32 ] && { [ "$opt" = 3 ] || [ "$opt" = 4 ]; }; then continue; fi
    echo "$name" >> "$out"
    for batch in 1 2 4 8 16 32 64; do
        "$exe" batch=$batch opt=$opt layer=$layer dtype=$dtype | grep -Eo 'time:[0-9]+(\.[0-9]+)? ms' | grep -Eo '[0-9]+(\.[0-9]+)?' | tr '\n' '\t' >> "$out"
        echo "" >> "$out"
    done
done
echo "wrote $out"
