"""Time ``fusedMM_csr`` on a MatrixMarket graph and print the reference tester's CSV line.

The command line and the output columns follow the reference's timing driver (``test/fusedMMtime.cpp:1807-1826``
for the flags, ``:1760-1805`` for the line ``Filename,NNZ,M,N,K,Trusted_exe_time,Test_exe_time,Speedup_exe_time``),
so a loop like the one in ``runtime.sh:176-186`` can append the output of this program to the same ``.csv`` files::

    python -m fusedmm_b200.mtx_run -input graph.mtx -K 128 -t s -nrep 20 -skHd 1

The reference builds one executable per kernel; here ``-t`` selects it: ``s`` sigmoid (table look-up, the tester's
scalar function ``fusedMMtime.cpp:586-633``), ``t`` t-distribution (clamped, ``:640-646``), ``f`` Fruchterman-Reingold
(``:635-639``), ``m`` SpMM, ``g`` GCN.  "Trusted" is this library's flag-interpreting vector kernel (option
``force_generic``: the stage codes are read at run time), "test" its kernels specialised for the message, both on the GPU with the arrays resident there;
times are seconds per call, the median of ``-nrep`` calls measured with CUDA events by the library itself.
``-T 1`` also compares the two results, the tester's PASSED/FAILED check (``fusedMMtime.cpp:1690-1712``).
There is no CPU path: without a CUDA device the program stops with an error.
"""
from __future__ import annotations

import argparse
import sys

import numpy as np

from . import messages as M

KERNELS = {
    "s": (M.MSG_SIGMOID, M.SOP_SIGMOID_TABLE_C),
    "t": (M.MSG_TDIST, M.SOP_TDIST_CLAMPED),
    "f": (M.MSG_TDIST, M.SOP_FR),
    "m": (M.MSG_SPMM, M.SOP_IDENTITY),
    "g": (M.MSG_GCN, M.SOP_IDENTITY),
}
HEADER = "Filename,NNZ,M,N,K,Trusted_exe_time,Test_exe_time,Speedup_exe_time"


def parse_args(argv):
    """Single-dash long options, as the reference's tester spells them."""
    p = argparse.ArgumentParser(prog="python -m fusedmm_b200.mtx_run", description=__doc__.split("\n\n")[0])
    p.add_argument("-input", required=True, help="MatrixMarket coordinate file")
    p.add_argument("-M", type=int, default=0, help="rows of S to process (0: all)")
    p.add_argument("-K", type=int, default=128, help="feature dimension of X, Y and Z")
    p.add_argument("-nrep", type=int, default=20, help="timed repetitions")
    p.add_argument("-T", type=int, default=0, choices=(0, 1), help="1: also compare trusted and test results")
    p.add_argument("-t", default="t", choices=sorted(KERNELS), help="kernel: s t f m g")
    p.add_argument("-skHd", type=int, default=0, choices=(0, 1), help="1: do not print the header line")
    p.add_argument("-ibeta", type=int, default=0, choices=(0, 1), help="beta: 0 overwrite Z, 1 accumulate")
    p.add_argument("-dtype", default="f32", choices=("f32", "f64"))
    p.add_argument("-seed", type=int, default=1)
    p.add_argument("-C", type=int, default=0, help="accepted for compatibility; the GPU caches are not flushed")
    p.add_argument("-ialpha", type=int, default=1, help="accepted for compatibility; alpha is never read")
    return p.parse_args(argv)


def _time_calls(call, nrep, api):
    ms = []
    for _ in range(max(1, nrep)):
        st = call()
        if st != 0:
            raise api.FusedMMError(f"fusedMM_csr returned {st}: {api.status_string(st)}")
        ms.append(api.call_info().device_ms)
    return float(np.median(ms)) * 1e-3


def run(args, out=sys.stdout):
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("fusedmm_b200.mtx_run needs a CUDA device; there is no CPU implementation")
    from . import api, mtx, synth
    dev = torch.device("cuda", torch.cuda.current_device())
    dtype = torch.float32 if args.dtype == "f32" else torch.float64
    csr = mtx.read_mtx(args.input, val_dtype=np.float32 if args.dtype == "f32" else np.float64)
    n = csr.n
    m = args.M if 0 < args.M <= n else n
    k = args.K
    msg, sop = KERNELS[args.t]
    rowptr, indx, val = csr.rowptr.to(dev), csr.indx.to(dev), csr.val.to(dev)
    pb, pe = rowptr[:-1].contiguous(), rowptr[1:].contiguous()
    nnz = int(rowptr[m].item() - rowptr[0].item())
    x = synth.dense_uniform(n, k, -0.5, 0.5, args.seed, device=dev, dtype=dtype)
    z0 = torch.zeros((m, k), device=dev, dtype=dtype)
    z1 = torch.zeros((m, k), device=dev, dtype=dtype)
    beta = float(args.ibeta)

    def call(z):
        return api.fusedMM_csr(msg, m, n, k, 1.0, nnz, n, n, val, indx, pb, pe, x, k, x, k, beta, z, k, sop=sop)

    old = api.get_option("force_generic")
    try:
        api.set_option("force_generic", 1)
        call(z0)                                  # warm-up, also sizes the library's scratch
        t0 = _time_calls(lambda: call(z0), args.nrep, api)
        api.set_option("force_generic", 0)
        call(z1)
        t1 = _time_calls(lambda: call(z1), args.nrep, api)
        if args.T:
            if beta != 0.0:                       # both kept accumulating: compare one fresh call of each
                z0.zero_(); z1.zero_()
                api.set_option("force_generic", 1); call(z0)
                api.set_option("force_generic", 0); call(z1)
            scale = torch.maximum(z0.abs(), z0.abs().amax(dim=1, keepdim=True)).clamp_min(1e-30)
            # the table sigmoid is a step function of s: a last-bit difference in s between two summation
            # orders can land in the neighbouring bin (bins of 10/2048), hence the wider bound for "s"
            tol = 5e-3 if args.t == "s" else (1e-4 if args.dtype == "f32" else 1e-10)
            bad = ((z1 - z0).abs() / scale) > tol
            bad |= ~torch.isfinite(z1) & torch.isfinite(z0)
            nerr = int(bad.sum().item())
            print("PASSED TEST" if nerr == 0 else f"FAILED TEST, {nerr} ELEMENTS", file=sys.stderr)
    finally:
        api.set_option("force_generic", old)
    if not args.skHd:
        print(HEADER, file=out)
    print(f"{args.input},{nnz},{m},{n},{k},{t0:e},{t1:e},{t0 / t1:f}", file=out)
    return t0, t1


def main(argv=None):
    run(parse_args(sys.argv[1:] if argv is None else argv))


if __name__ == "__main__":
    main()
