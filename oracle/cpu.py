"""ctypes loaders for the CPU checkers -- TEST INFRASTRUCTURE ONLY.

Four checkers live here, none of which the product (``fusedmm_b200``) may import:

* :class:`Oracle` -- ``oracle/fusedmm_oracle.c``, a C restatement of the general kernel of
  HipGraph/FusedMM (``fusedMM.c:698-739`` and the operator bodies ``fusedMM.c:28-333``).
* :class:`Reference` -- the reference's own ``fusedMM.c`` compiled by ``oracle/build_ref.sh`` into
  ``oracle/_ref/``; present only where that recipe has run (it needs the reference sources).
* :class:`ReferenceOpt` -- the reference's optimised OpenMP path (generated SIMD kernels behind
  ``{s,d}gfusedMM_csr``, ``kernels/src/kernels.c:456-631``) built by ``oracle/build_ref_opt.sh``; it is
  what the benchmark times as the CPU baseline.
* :func:`numpy_fusedmm` -- an independent float64 NumPy restatement for hand-sized cases.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
BUILD = HERE / "_build"
REF = HERE / "_ref"

_C = ctypes
_I32, _I64, _F32, _F64 = _C.c_int32, _C.c_int64, _C.c_float, _C.c_double


def build_oracle(force: bool = False) -> Path:
    """Compile ``fusedmm_oracle.c`` into ``oracle/_build/libfusedmm_oracle.so`` (gcc, a second or two)."""
    out = BUILD / "libfusedmm_oracle.so"
    srcs = [HERE / "fusedmm_oracle.c", HERE / "fusedmm_oracle_body.inc", HERE / "sop_bodies.h"]
    if not force and out.exists() and all(out.stat().st_mtime >= s.stat().st_mtime for s in srcs):
        return out
    BUILD.mkdir(exist_ok=True)
    tmp = out.with_suffix(f".{os.getpid()}.tmp")
    cmd = ["gcc", "-O2", "-mavx2", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared",
           str(HERE / "fusedmm_oracle.c"), "-lm", "-o", str(tmp)]
    subprocess.run(cmd, check=True)
    os.replace(tmp, out)
    return out


def build_reference(reference_dir: str = os.environ.get("FUSEDMM_REFERENCE_DIR", "/root/reference")) -> bool:
    """Run ``oracle/build_ref.sh`` when the reference sources are present; True if the libraries exist."""
    if Path(reference_dir, "fusedMM.c").exists():
        subprocess.run([str(HERE / "build_ref.sh"), reference_dir], check=True,
                       stdout=subprocess.DEVNULL)
    return reference_available()


def reference_available() -> bool:
    return all((REF / f"libfusedmm_ref_{p}_i{b}.so").exists() for p in "sd" for b in (32, 64))


def host_simd_level() -> str | None:
    """SIMD level of this host's CPU the way the reference's ``configure:150-225`` decides it:
    "avxz" with avx512f and avx512dq, else "avx2", else None (the reference supports nothing less on x86)."""
    try:
        flags = set()
        for line in Path("/proc/cpuinfo").read_text().splitlines():
            if line.startswith("flags"):
                flags = set(line.split(":", 1)[1].split())
                break
    except OSError:
        return None
    if {"avx512f", "avx512dq"} <= flags:
        return "avxz"
    if {"avx2", "fma"} <= flags:
        return "avx2"
    return None


def build_reference_opt(reference_dir: str = os.environ.get("FUSEDMM_REFERENCE_DIR", "/root/reference")) -> bool:
    """Run ``oracle/build_ref_opt.sh`` when the reference sources are present (a few minutes the first
    time, nothing when the libraries are up to date); True if the libraries for this host exist."""
    if Path(reference_dir, "kernels", "codegen", "genkern.base").exists():
        subprocess.run([str(HERE / "build_ref_opt.sh"), reference_dir], check=True, stdout=subprocess.DEVNULL)
    return reference_opt_available()


def reference_opt_available() -> bool:
    lvl = host_simd_level()
    return lvl is not None and all((REF / f"libfusedmm_refopt_{p}_i64_{lvl}.so").exists() for p in "sd")


def _ptr(a):
    return None if a is None else a.ctypes.data_as(_C.c_void_p)


def _types(val_dtype, ptr_dtype, idx_dtype):
    pre = {np.dtype(np.float32): "s", np.dtype(np.float64): "d"}[np.dtype(val_dtype)]
    pb, ib = np.dtype(ptr_dtype).itemsize * 8, np.dtype(idx_dtype).itemsize * 8
    if pb == ib:
        suffix = f"i{ib}"
    elif (pb, ib) == (64, 32):
        suffix = "p64i32"
    else:
        raise ValueError("row pointers narrower than column ids are not a supported combination")
    return pre, suffix, (_F32 if pre == "s" else _F64), (_I32 if pb == 32 else _I64)


def _check_arrays(val, indx, pntrb, pntre, x, y, z):
    for a in (val, indx, pntrb, pntre, x, y, z):
        if a is not None and not a.flags["C_CONTIGUOUS"]:
            raise ValueError("arrays must be C-contiguous")


class Oracle:
    """The C restatement.  ``csr`` mirrors ``fusedMM_csr`` (fusedMM.h:76-97) with the SOP made explicit."""

    def __init__(self):
        self.lib = _C.CDLL(str(build_oracle()))
        self.lib.oracle_sop_f32.restype = _F32
        self.lib.oracle_sop_f32.argtypes = [_F32, _C.c_int, _F64, _F64, _F64]
        self.lib.oracle_sop_f64.restype = _F64
        self.lib.oracle_sop_f64.argtypes = [_F64, _C.c_int, _F64, _F64, _F64]

    def sop(self, s, kind, p=(0.0, 0.0, 0.0), dtype=np.float32):
        f = self.lib.oracle_sop_f32 if np.dtype(dtype) == np.float32 else self.lib.oracle_sop_f64
        return f(s, kind, *p)

    def csr(self, imessage, m, n, k, val, indx, pntrb, pntre, x, ldx, y, ldy, beta, z, ldz,
            sop_kind=1, sop_params=(0.0, 0.0, 0.0), zero_first=True, alpha=1.0, nnz=0):
        """Runs the oracle in place on ``z``.  ``zero_first`` gives the optimised kernels' beta==0
        behaviour (Z overwritten); ``False`` is the general kernel, which always accumulates."""
        _check_arrays(val, indx, pntrb, pntre, x, y, z)
        pre, suffix, VT, PT = _types(z.dtype, pntrb.dtype, indx.dtype)
        fn = getattr(self.lib, f"oracle_{pre}fusedMM_csr_{suffix}")
        fn.restype = _C.c_int
        fn.argtypes = ([_I32, PT, PT, PT, VT, PT, PT, PT] + [_C.c_void_p] * 4 +
                       [_C.c_void_p, PT, _C.c_void_p, PT, VT, _C.c_void_p, PT] +
                       [_I32, _F64, _F64, _F64, _I32])
        return fn(imessage, m, n, k, alpha, nnz, m, n, _ptr(val), _ptr(indx), _ptr(pntrb),
                  _ptr(pntre), _ptr(x), ldx, _ptr(y), ldy, beta, _ptr(z), ldz, sop_kind,
                  *sop_params, int(bool(zero_first)))


class Reference:
    """The reference's own general kernel (its ``fusedMM_csr``), one library per type combination."""

    def __init__(self):
        if not reference_available():
            raise FileNotFoundError("oracle/_ref is not built (run oracle/build_ref.sh where the "
                                    "reference sources are available)")
        self.libs = {}
        for p in "sd":
            for b in (32, 64):
                self.libs[(p, b)] = _C.CDLL(str(REF / f"libfusedmm_ref_{p}_i{b}.so"))

    def threads(self, n=None):
        lib = self.libs[("s", 64)]
        if n is not None:
            for l in self.libs.values():
                l.ref_set_threads(int(n))
        return lib.ref_get_threads()

    def csr(self, imessage, m, n, k, val, indx, pntrb, pntre, x, ldx, y, ldy, beta, z, ldz,
            sop_kind=1, sop_params=(0.0, 0.0, 0.0), alpha=1.0, nnz=0):
        """Calls the reference in place on ``z``; it always accumulates into ``z`` (fusedMM.c:737)."""
        _check_arrays(val, indx, pntrb, pntre, x, y, z)
        pre, suffix, VT, PT = _types(z.dtype, pntrb.dtype, indx.dtype)
        if suffix == "p64i32":
            raise ValueError("the reference has a single INDEXTYPE (fusedMM.h:79-96)")
        lib = self.libs[(pre, 32 if PT is _I32 else 64)]
        lib.ref_set_sop.argtypes = [_C.c_int, _F64, _F64, _F64]
        lib.ref_set_sop.restype = None
        lib.ref_set_sop(sop_kind, *sop_params)
        fn = lib.ref_fusedMM_csr
        fn.restype = _C.c_int
        fn.argtypes = ([_I32, PT, PT, PT, VT, PT, PT, PT] + [_C.c_void_p] * 4 +
                       [_C.c_void_p, PT, _C.c_void_p, PT, VT, _C.c_void_p, PT])
        return fn(imessage, m, n, k, alpha, nnz, m, n, _ptr(val), _ptr(indx), _ptr(pntrb),
                  _ptr(pntre), _ptr(x), ldx, _ptr(y), ldy, beta, _ptr(z), ldz)


class ReferenceOpt:
    """The reference's ``fusedMM_csr`` compiled with ``ENABLE_OPT_FUSEDMM`` and linked with its generated
    kernels (int64 indices).  The four optimised messages run the generated SIMD kernels when ``ld* == k``
    and ``k`` is a multiple of the vector length (16/8 floats, 8/4 doubles for AVX-512/AVX2); with
    ``beta == 0`` they overwrite ``z``.  Everything else falls through to the general kernel."""

    def __init__(self):
        self.simd = host_simd_level()
        if not reference_opt_available():
            raise FileNotFoundError("oracle/_ref holds no optimised reference build for this host "
                                    "(run oracle/build_ref_opt.sh where the reference sources are available)")
        self.libs = {p: _C.CDLL(str(REF / f"libfusedmm_refopt_{p}_i64_{self.simd}.so")) for p in "sd"}
        # the general kernel alone with the same optimising flags (the second timed figure)
        self.general_libs = {p: _C.CDLL(str(REF / f"libfusedmm_refgen_{p}_i64_{self.simd}.so")) for p in "sd"
                             if (REF / f"libfusedmm_refgen_{p}_i64_{self.simd}.so").exists()}

    def vlen(self, dtype) -> int:
        return {("avxz", 4): 16, ("avxz", 8): 8, ("avx2", 4): 8, ("avx2", 8): 4}[(self.simd, np.dtype(dtype).itemsize)]

    def threads(self, n=None):
        if n is not None:
            for l in list(self.libs.values()) + list(self.general_libs.values()):
                l.ref_set_threads(int(n))
        return self.libs["s"].ref_get_threads()

    def csr(self, imessage, m, n, k, val, indx, pntrb, pntre, x, ldx, y, ldy, beta, z, ldz,
            sop_kind=1, sop_params=(0.0, 0.0, 0.0), alpha=1.0, nnz=0, general=False):
        """``general=True`` runs the general kernel alone (always accumulates into ``z``)."""
        _check_arrays(val, indx, pntrb, pntre, x, y, z)
        pre, suffix, VT, PT = _types(z.dtype, pntrb.dtype, indx.dtype)
        if suffix != "i64":
            raise ValueError("the optimised reference build takes int64 indices only")
        lib = (self.general_libs if general else self.libs)[pre]
        lib.ref_set_sop.argtypes = [_C.c_int, _F64, _F64, _F64]
        lib.ref_set_sop.restype = None
        lib.ref_set_sop(sop_kind, *sop_params)
        fn = lib.ref_fusedMM_csr
        fn.restype = _C.c_int
        fn.argtypes = ([_I32, PT, PT, PT, VT, PT, PT, PT] + [_C.c_void_p] * 4 +
                       [_C.c_void_p, PT, _C.c_void_p, PT, VT, _C.c_void_p, PT])
        return fn(imessage, m, n, k, alpha, nnz, m, n, _ptr(val), _ptr(indx), _ptr(pntrb),
                  _ptr(pntre), _ptr(x), ldx, _ptr(y), ldy, beta, _ptr(z), ldz)


def numpy_sop(s, kind, p=(0.0, 0.0, 0.0), dtype=np.float64):
    """Scalar functions in ``dtype`` (same catalogue as ``include/fusedmm_b200.h``), without the table."""
    s = dtype(s)
    with np.errstate(all="ignore"):
        if kind == 0:
            return s
        if kind in (1,):
            return 1.0 / (1.0 + np.exp(-s))
        if kind == 3:
            return 1.0 + 1.0 / s
        if kind == 4:
            return 1.0 / (1.0 + s)
        if kind == 5:
            return np.clip(-2.0 / (1.0 + s), -5.0, 5.0)
        if kind == 6:
            return np.log2(1.0 + np.sqrt(s))
        if kind == 7:
            return np.sqrt(s) + 1.0 / s
        if kind == 8:
            v = p[0] / (p[1] + s)
            return np.clip(v, -p[2], p[2]) if p[2] > 0 else v
    raise ValueError(f"no closed form for SOP kind {kind}")


def numpy_fusedmm(imessage, m, k, val, indx, pntrb, pntre, x, y, z0, sop_kind=1,
                  sop_params=(0.0, 0.0, 0.0), dtype=np.float64):
    """Independent restatement in ``dtype`` (float64, or ``np.longdouble`` as the higher-precision evaluation
    that float64 results are judged against), vectorised over K with a Python loop over edges: small cases only.
    Follows the stage order of ``fusedMM.c:706-738``; returns a new array of ``dtype``."""
    vop, rop, sop = imessage & 0xF, (imessage >> 4) & 0xF, (imessage >> 8) & 0xF
    vsc, aop = (imessage >> 12) & 0xF, (imessage >> 16) & 0xF
    X = np.asarray(x, dtype=dtype)[:, :k]
    Y = np.asarray(y, dtype=dtype)[:, :k]
    Z = np.array(z0, dtype=dtype)
    for i in range(m):
        for j in range(int(pntrb[i]), int(pntre[i])):
            xi, yv = X[i], Y[int(indx[j])]
            T = {1: xi, 2: yv, 3: xi + yv, 4: yv - xi, 5: xi - yv, 6: np.maximum(xi, yv),
                 7: np.minimum(xi, yv)}[vop].copy()
            s = {0: lambda: dtype(val[j]), 1: lambda: xi @ T, 2: lambda: xi.sum(),
                 3: lambda: T.sum(), 4: lambda: xi @ xi, 5: lambda: T @ T}[rop]()
            out = numpy_sop(s, sop_kind, sop_params, dtype) if sop == 0xF else s
            if vsc == 1:
                T = out * T
            elif vsc == 2:
                T = out + T
            if aop == 1:
                Z[i, :k] += T
            elif aop == 2:
                Z[i, :k] = np.maximum(Z[i, :k], T)
            elif aop == 3:
                Z[i, :k] = np.minimum(Z[i, :k], T)
    return Z
