#!/usr/bin/env bash
# Compiles the reference's OWN general kernel (HipGraph/FusedMM fusedMM.c, read where it lies) with
# oracle/ref_harness.c into oracle/_ref/libfusedmm_ref_<s|d>_<i32|i64>.so.  TEST INFRASTRUCTURE ONLY.
# No reference source is copied; the only outputs are the shared objects under oracle/_ref/.
#   usage: oracle/build_ref.sh [reference-dir]      (default: $FUSEDMM_REFERENCE_DIR, else the read-only mount of the reference)
# Flags: the macros are the reference's own switches (kernels/CONFIG/make.base:199-223: PTTIME,
# LOAD_BALANCE, SREAL/DREAL, INDEXTYPE).  -ffp-contract=off keeps mul+add unfused so that the
# restatement in fusedmm_oracle.c can be required to match bit for bit.
set -euo pipefail
here="$(cd "$(dirname "$0")" && pwd)"
ref="${1:-${FUSEDMM_REFERENCE_DIR:-/root/reference}}"
if [ ! -f "$ref/fusedMM.c" ]; then echo "build_ref: no reference at $ref" >&2; exit 3; fi
out="$here/_ref"; mkdir -p "$out"
pids=()
for pre in s d; do
  for ib in 32 64; do
    real=SREAL; [ "$pre" = d ] && real=DREAL
    gcc -O3 -mavx2 -ffp-contract=off -fopenmp -fPIC -shared -w \
        -D$real -DINDEXTYPE=int${ib}_t -DPTTIME -DLOAD_BALANCE "-DNTHREADS=fusedmm_ref_nthreads()" \
        -include "$here/ref_prelude.h" -I"$ref" -I"$here" \
        "$ref/fusedMM.c" "$here/ref_harness.c" -lm -o "$out/libfusedmm_ref_${pre}_i${ib}.so" &
    pids+=($!)
  done
done
for p in "${pids[@]}"; do wait "$p"; done
ls -l "$out"
