#!/usr/bin/env bash
# Builds the reference's OPTIMISED OpenMP path (HipGraph/FusedMM: the generated SIMD kernels behind
# {s,d}gfusedMM_csr, kernels/src/kernels.c:456-631, and fusedMM.c with -DENABLE_OPT_FUSEDMM) into
#     oracle/_ref/libfusedmm_refopt_<s|d>_i64_<avxz|avx2>.so
# and, beside each, the reference's general kernel alone (fusedMM.c without ENABLE_OPT_FUSEDMM) compiled with
# the same optimising flags, as the second timed figure:
#     oracle/_ref/libfusedmm_refgen_<s|d>_i64_<avxz|avx2>.so
# (oracle/build_ref.sh builds the general kernel too, but with -ffp-contract=off for the bit-for-bit pin of
# the oracle: right for parity, wrong for a timed baseline).
# TEST / BASELINE INFRASTRUCTURE ONLY: this is the CPU code the benchmark times beside the GPU.
#
# What it does is what the reference's `./configure && make` does, step by step, without running
# either (the reference tree is read-only and its Makefiles write into it):
#   1. compile the reference's generator tool (kernels/codegen/extract.c) into a scratch directory;
#   2. expand kernels/codegen/genheader.base and genkern.base with the arguments of
#      kernels/CONFIG/make.base:122-125 and rungen.top:86-113 (kruntime=1, bestK=512, regblk=bacrb,
#      the shipped defaults make.base:160-185) into that scratch directory;
#   3. compile the generated kernels with the flags of kernels/codegen/genmake.base:29-33,81-86
#      (-O3 <simd flags> -DBLC_ARCH -DBLC_X86 -DBLC_<simd> -fopenmp -DPTTIME -DLDB -DBETA{0,1}),
#      kernels.c, and fusedMM.c with make.base:325-330's flags (-O3 -fopenmp -DPTTIME -DLOAD_BALANCE
#      -DENABLE_OPT_FUSEDMM), and link them with oracle/ref_harness.c.
# The scratch directory (generated C files, objects) is deleted at the end; no reference source and no
# generated source enters the repository.  Two SIMD levels are built because the machine that runs the
# benchmark need not be the machine that builds: the loader picks the one the host CPU supports
# (configure:150-225 makes the same choice from lscpu).  NTHREADS is bound to a function
# (ref_prelude.h) so one binary uses the cores of whatever host runs it (configure:276-286 bakes the
# build host's core count in).  int64 indices only (the reference's default, make.base:151).
#   usage: oracle/build_ref_opt.sh [reference-dir]
set -euo pipefail
here="$(cd "$(dirname "$0")" && pwd)"
ref="${1:-${FUSEDMM_REFERENCE_DIR:-/root/reference}}"
if [ ! -f "$ref/kernels/codegen/genkern.base" ]; then echo "build_ref_opt: no reference at $ref" >&2; exit 3; fi
out="$here/_ref"; mkdir -p "$out"
jobs="$(nproc 2>/dev/null || echo 4)"
work="$(mktemp -d /tmp/fusedmm_refopt.XXXXXX)"
trap 'rm -rf "$work"' EXIT
BESTK=512

gcc -O3 -w -o "$work/xextract" "$ref/kernels/codegen/extract.c" 2>/dev/null
ext="$work/xextract"

build_one() {  # pre (s|d)  simd tag (avxz|avx2)  vlen  simd flags  simd macro
  local pre="$1" tag="$2" vlen="$3" cflags="$4" simd="$5"
  local lib="$out/libfusedmm_refopt_${pre}_i64_${tag}.so"
  if [ -f "$lib" ] && [ "$lib" -nt "$0" ] && [ "$lib" -nt "$here/ref_harness.c" ]; then echo "up to date: $lib"; return 0; fi
  local top="$work/${pre}_${tag}/kernels"
  local gsrc="$top/generated/src" ginc="$top/generated/include"
  mkdir -p "$gsrc" "$ginc" "$top/src" "$top/obj"
  ln -s "$ref/kernels/simd" "$top/simd"     # the generated sources include "../../simd/simd.h"
  local real=SREAL; [ "$pre" = d ] && real=DREAL
  # ---- step 2: headers and sources -------------------------------------------------------------------
  "$ext" -b "$ref/kernels/codegen/genheader.base" -langC pre=$pre rout=misc -o "$ginc/${pre}gmisc.h" >/dev/null
  for kn in sigmoid tdist spmm gcn; do
    "$ext" -b "$ref/kernels/codegen/genheader.base" -langC -def MDIM $BESTK pre=$pre -def VLEN $vlen rout=ghead \
           -def frc $kn -def kruntime 1 -def bestK $BESTK -o "$ginc/${pre}gkernels_${kn}.h" >/dev/null
    for ((d = vlen; d <= BESTK; d += vlen)); do
      local kr=0; [ "$d" -eq "$BESTK" ] && kr=1
      "$ext" -b "$ref/kernels/codegen/genkern.base" -langC -def DIM $d pre=$pre rblk=bacrb -def VLEN $vlen rout=$kn \
             -def kruntime $kr -o "$gsrc/${pre}gfusedMM_K${d}_${kn}_csr.c" >/dev/null
    done
  done
  # ---- step 3: compile ---------------------------------------------------------------------------------
  local common="-O3 $cflags -DBLC_ARCH -DBLC_X86 -D$simd -DINDEXTYPE=int64_t -fopenmp -DPTTIME -DLDB -D$real -fPIC -w"
  ( cd "$gsrc"
    for f in *.c; do for b in 0 1; do echo "$f $b"; done; done |
      xargs -P "$jobs" -n 2 sh -c 'gcc '"$common"' "-DNTHREADS=fusedmm_ref_nthreads()" -include "'"$here"'/ref_prelude.h" -DBETA$1 -I"'"$ref"'/kernels/simd" -c "$0" -o "'"$top"'/obj/${0%.c}_b$1.o"'
  )
  gcc $common "-DNTHREADS=fusedmm_ref_nthreads()" -include "$here/ref_prelude.h" -I"$ginc" -I"$top/src" \
      -c "$ref/kernels/src/kernels.c" -o "$top/obj/${pre}kernels_pt.o"
  gcc -O3 $cflags -fopenmp -fPIC -w -DINDEXTYPE=int64_t -DINT64 -D$real -DPTTIME -DLOAD_BALANCE -DENABLE_OPT_FUSEDMM \
      "-DNTHREADS=fusedmm_ref_nthreads()" -include "$here/ref_prelude.h" -I"$ref/kernels/include" -I"$ref" \
      -c "$ref/fusedMM.c" -o "$top/obj/${pre}OptFusedMM_pt.o"
  gcc -O3 $cflags -fopenmp -fPIC -w -DINDEXTYPE=int64_t -D$real -I"$ref" -I"$here" \
      -c "$here/ref_harness.c" -o "$top/obj/harness.o"
  gcc -shared -fopenmp -o "$lib.tmp" "$top"/obj/*.o -lm
  mv "$lib.tmp" "$lib"
  # the general kernel alone, same flags minus ENABLE_OPT_FUSEDMM (make.base:325-330, the FusedMM target)
  gcc -O3 $cflags -fopenmp -fPIC -shared -w -DINDEXTYPE=int64_t -DINT64 -D$real -DPTTIME -DLOAD_BALANCE \
      "-DNTHREADS=fusedmm_ref_nthreads()" -include "$here/ref_prelude.h" -I"$ref/kernels/include" -I"$ref" -I"$here" \
      "$ref/fusedMM.c" "$here/ref_harness.c" -lm -o "$out/libfusedmm_refgen_${pre}_i64_${tag}.so"
  rm -rf "$work/${pre}_${tag}"
  echo "built $lib"
}

# simd flags per level: configure:160-180 (-mavx512f -mavx512dq | -mavx -mfma); vector lengths configure:163-164,177-178
build_one s avxz 16 "-mavx512f -mavx512dq" BLC_AVXZ
build_one d avxz 8  "-mavx512f -mavx512dq" BLC_AVXZ
build_one s avx2 8  "-mavx -mfma" BLC_AVX2
build_one d avx2 4  "-mavx -mfma" BLC_AVX2
ls -l "$out"
