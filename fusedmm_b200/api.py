"""Python mirror of the C ABI in ``include/fusedmm_b200.h`` (ctypes; no torch types cross the boundary).

:func:`fusedMM_csr` has the reference's argument list (HipGraph/FusedMM ``fusedMM.h:76-97``) and return
codes.  Arrays may be NumPy arrays (host memory: the library stages them to the GPU and copies Z back) or
torch tensors (CPU or CUDA; CUDA tensors are used in place).  The typed symbol
(``sfusedMM_csr_i32`` ... ``dfusedMM_csr_p64i32``) is picked from the arrays' dtypes, which is what the
reference does at compile time with its VALUETYPE / INDEXTYPE macros.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libfusedmm_b200.so"
_lib = None


class FusedMMError(RuntimeError):
    pass


class SopSpec(C.Structure):
    """``fusedmm_b200_sop`` of include/fusedmm_b200.h."""
    _fields_ = [("kind", C.c_int32), ("reserved", C.c_int32), ("p0", C.c_double), ("p1", C.c_double),
                ("p2", C.c_double)]


class CallInfo(C.Structure):
    """``fusedmm_b200_call_info`` of include/fusedmm_b200.h."""
    _fields_ = [("kernel_launches", C.c_int32), ("pattern", C.c_int32), ("lanes_per_edge", C.c_int32),
                ("vectors_per_lane", C.c_int32), ("h2d_bytes", C.c_int64), ("d2h_bytes", C.c_int64),
                ("hub_rows", C.c_int64), ("hub_chunks", C.c_int64), ("device_ms", C.c_float),
                ("sop_kind", C.c_int32), ("ms_scan", C.c_float), ("ms_rows", C.c_float),
                ("ms_chunks", C.c_float), ("ms_fixup", C.c_float), ("engine", C.c_int32), ("ms_main", C.c_float),
                ("jit_kernel", C.c_int32)]


def lib() -> C.CDLL:
    """Loads ``libfusedmm_b200.so``.  Raises if it is not built: there is no other implementation."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise FusedMMError(f"{LIB_PATH} is missing: build it with `python -m fusedmm_b200.build` "
                               "(nvcc, sm_100a). There is no CPU or PyTorch fallback.")
        _lib = C.CDLL(str(LIB_PATH))
        _lib.fusedmm_b200_status_string.restype = C.c_char_p
        _lib.fusedmm_b200_version.restype = C.c_char_p
        _lib.fusedmm_b200_set_sop.argtypes = [C.c_int32, C.c_double, C.c_double, C.c_double]
        _lib.fusedmm_b200_set_option.argtypes = [C.c_char_p, C.c_int64]
        _lib.fusedmm_b200_get_option.argtypes = [C.c_char_p, C.POINTER(C.c_int64)]
        _lib.fusedmm_b200_last_call_info.argtypes = [C.POINTER(CallInfo)]
        _lib.fusedmm_b200_csr.restype = C.c_int
        _lib.fusedmm_b200_csr.argtypes = (
            [C.c_int32] * 4 + [C.c_int64] * 3 + [C.c_double] + [C.c_int64] * 3 + [C.c_void_p] * 5 +
            [C.c_int64, C.c_void_p, C.c_int64, C.c_double, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p])
    return _lib


def status_string(status: int) -> str:
    return lib().fusedmm_b200_status_string(int(status)).decode()


def set_sop(kind: int, p0: float = 0.0, p1: float = 0.0, p2: float = 0.0) -> int:
    """Process-wide meaning of SOP_UDEF (``fusedmm_b200_set_sop``)."""
    return lib().fusedmm_b200_set_sop(kind, p0, p1, p2)


def set_option(name: str, value: int) -> int:
    return lib().fusedmm_b200_set_option(name.encode(), int(value))


def get_option(name: str) -> int:
    v = C.c_int64(0)
    st = lib().fusedmm_b200_get_option(name.encode(), C.byref(v))
    if st:
        raise FusedMMError(f"unknown option {name!r}")
    return v.value


def jit_prepare(imessage: int, k: int, dtype=np.float32) -> int:
    """``fusedmm_b200_jit_prepare``: build the kernel specialised for a message ahead of its first call."""
    fn = lib().fusedmm_b200_jit_prepare
    fn.argtypes = [C.c_int32, C.c_int32, C.c_int64]
    return fn(0 if np.dtype(dtype) == np.float32 else 1, int(imessage), int(k))


def jit_stats() -> dict:
    out = (C.c_int64 * 5)()
    lib().fusedmm_b200_jit_stats(out)
    return dict(zip(("compiled", "disk_hits", "launches", "failures", "nvrtc_found"), (int(v) for v in out)))


def call_info() -> CallInfo:
    """What the most recent call on this thread did (``fusedmm_b200_last_call_info``)."""
    info = CallInfo()
    lib().fusedmm_b200_last_call_info(C.byref(info))
    return info


_NP = {"float32": np.float32, "float64": np.float64, "int32": np.int32, "int64": np.int64}


def _describe(a):
    """-> (address, numpy dtype) of a NumPy array, a torch tensor or None."""
    if a is None:
        return None, None
    if isinstance(a, np.ndarray):
        if not a.flags["C_CONTIGUOUS"]:
            raise ValueError("arrays must be C-contiguous; use ldx/ldy/ldz for padded rows")
        return a.ctypes.data, a.dtype
    if hasattr(a, "data_ptr"):  # torch tensor, without importing torch here
        if not a.is_contiguous():
            raise ValueError("tensors must be contiguous; use ldx/ldy/ldz for padded rows")
        return a.data_ptr(), np.dtype(_NP[str(a.dtype).replace("torch.", "")])
    raise TypeError(f"unsupported array type {type(a)!r}")


def _symbol(vt, pt, it):
    pre = {np.dtype(np.float32): "s", np.dtype(np.float64): "d"}.get(np.dtype(vt))
    if pre is None:
        raise TypeError("values must be float32 or float64")
    pb, ib = np.dtype(pt).itemsize * 8, np.dtype(it).itemsize * 8
    if np.dtype(pt).kind != "i" or np.dtype(it).kind != "i" or pb not in (32, 64) or ib not in (32, 64):
        raise TypeError("indices must be int32 or int64")
    if pb == ib:
        return pre, f"i{pb}", pb
    if (pb, ib) == (64, 32):
        return pre, "p64i32", 64
    raise TypeError("32-bit row pointers with 64-bit column ids are not supported")


def fusedMM_csr(imessage, m, n, k, alpha, nnz, rows, cols, val, indx, pntrb, pntre, x, ldx, y, ldy, beta,
                z, ldz, sop=None, stream=None, z_peers=None, z_multicast=None):
    """``fusedMM_csr`` with the reference's argument order and return codes.

    ``sop``: ``None`` (process default, see :func:`set_sop`), an ``int`` kind, or ``(kind, p0, p1, p2)``.
    ``stream``: ``None`` for a synchronous call, or a CUDA stream handle (``int``) to enqueue on; every
    array must then be on the device.  With ``sop`` and ``stream`` both ``None`` the call goes through
    the typed symbol (``sfusedMM_csr_i64`` ...), otherwise through ``fusedmm_b200_csr``.
    ``z_peers``: device addresses (``int``) of other GPUs' Z buffers at this call's first row; finished
    rows are then also stored there (``fusedmm_b200_csr_multi``); ``z_multicast``: instead, the NVSwitch
    multicast address of Z at this call's first row (one ``multimem.st`` per row reaches every GPU).
    """
    L = lib()
    ptrs, dts = zip(*[_describe(a) for a in (val, indx, pntrb, pntre, x, y, z)])
    vt = dts[6]
    for d in (dts[0], dts[4], dts[5]):
        if d is not None and d != vt:
            raise TypeError("val, x, y and z must share one floating-point type")
    if dts[3] != dts[2]:
        raise TypeError("pntrb and pntre must share one integer type")
    pre, suffix, size_bits = _symbol(vt, dts[2], dts[1] if dts[1] is not None else dts[2])
    if sop is None and stream is None and not z_peers and not z_multicast:
        VT = C.c_float if pre == "s" else C.c_double
        IT = C.c_int32 if size_bits == 32 else C.c_int64
        fn = getattr(L, f"{pre}fusedMM_csr_{suffix}")
        fn.restype = C.c_int
        fn.argtypes = ([C.c_int32, IT, IT, IT, VT, IT, IT, IT] + [C.c_void_p] * 4 +
                       [C.c_void_p, IT, C.c_void_p, IT, VT, C.c_void_p, IT])
        return fn(imessage, m, n, k, alpha, nnz, rows, cols, ptrs[0], ptrs[1], ptrs[2], ptrs[3], ptrs[4],
                  ldx, ptrs[5], ldy, beta, ptrs[6], ldz)
    spec = None
    if sop is not None:
        kind, *params = (sop,) if isinstance(sop, int) else tuple(sop)
        params = list(params) + [0.0] * (3 - len(params))
        spec = C.byref(SopSpec(int(kind), 0, *map(float, params)))
    pb = np.dtype(dts[2]).itemsize * 8
    ib = np.dtype(dts[1]).itemsize * 8 if dts[1] is not None else pb
    if z_peers or z_multicast:
        z_peers = list(z_peers or [])
        arr = (C.c_void_p * max(1, len(z_peers)))(*[int(q) for q in z_peers])
        fn = L.fusedmm_b200_csr_multi
        fn.restype = C.c_int
        fn.argtypes = list(L.fusedmm_b200_csr.argtypes) + [C.c_int32, C.c_void_p, C.c_void_p]
        return fn(0 if pre == "s" else 1, pb, ib, imessage, m, n, k, alpha, nnz, rows, cols, ptrs[0], ptrs[1],
                  ptrs[2], ptrs[3], ptrs[4], ldx, ptrs[5], ldy, beta, ptrs[6], ldz, spec, stream, len(z_peers), arr,
                  int(z_multicast) if z_multicast else None)
    return L.fusedmm_b200_csr(0 if pre == "s" else 1, pb, ib, imessage, m, n, k, alpha, nnz, rows, cols,
                              ptrs[0], ptrs[1], ptrs[2], ptrs[3], ptrs[4], ldx, ptrs[5], ldy, beta, ptrs[6],
                              ldz, spec, stream)


def gfusedMM_csr(tkern, m, n, k, alpha, nnz, rows, cols, val, indx, pntrb, pntre, a, lda, b, ldb, beta, c,
                 ldc):
    """``sgfusedMM_csr`` / ``dgfusedMM_csr`` (kernels/include/kernels.h:17-37): dispatch by kernel letter."""
    L = lib()
    ptrs, dts = zip(*[_describe(t) for t in (val, indx, pntrb, pntre, a, b, c)])
    pre, suffix, size_bits = _symbol(dts[6], dts[2], dts[1] if dts[1] is not None else dts[2])
    if suffix == "p64i32":
        raise TypeError("the letter dispatcher has a single INDEXTYPE")
    VT = C.c_float if pre == "s" else C.c_double
    IT = C.c_int32 if size_bits == 32 else C.c_int64
    fn = getattr(L, f"{pre}gfusedMM_csr_{suffix}")
    fn.restype = None
    fn.argtypes = ([C.c_char, IT, IT, IT, VT, IT, IT, IT] + [C.c_void_p] * 4 +
                   [C.c_void_p, IT, C.c_void_p, IT, VT, C.c_void_p, IT])
    fn(tkern.encode() if isinstance(tkern, str) else tkern, m, n, k, alpha, nnz, rows, cols, ptrs[0],
       ptrs[1], ptrs[2], ptrs[3], ptrs[4], lda, ptrs[5], ldb, beta, ptrs[6], ldc)


def zero_empty_rows(pntrb, pntre, z, k, ldz, stream=None):
    """``fusedmm_b200_zero_empty_rows``: Z_u = 0 for the rows without edges among the ``len(pntrb)`` rows that
    ``pntrb``/``pntre``/``z`` start at (device tensors); returns the status code."""
    L = lib()
    ptrs, dts = zip(*[_describe(a) for a in (pntrb, pntre, z)])
    if dts[0] != dts[1]:
        raise TypeError("pntrb and pntre must share one integer type")
    fn = L.fusedmm_b200_zero_empty_rows
    fn.restype = C.c_int
    fn.argtypes = [C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
    return fn(0 if np.dtype(dts[2]) == np.float32 else 1, np.dtype(dts[0]).itemsize * 8, len(pntrb), k, ptrs[0], ptrs[1],
              ptrs[2], ldz, stream)


def shard_rows(pntrb, pntre, nshards, row_weight=0):
    """Contiguous row ranges of equal cost, a row costing its edges plus ``row_weight``
    (``fusedmm_b200_shard_rows_weighted_*``; 0 = balanced by edges alone); host NumPy row pointers."""
    L = lib()
    pntrb = np.ascontiguousarray(pntrb)
    pntre = np.ascontiguousarray(pntre)
    m = len(pntrb)
    bounds = np.zeros(nshards + 1, dtype=np.int64)
    fn = L.fusedmm_b200_shard_rows_weighted_i32 if pntrb.dtype == np.int32 else L.fusedmm_b200_shard_rows_weighted_i64
    fn.argtypes = [C.c_int64, C.c_int32, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
    st = fn(m, nshards, pntrb.ctypes.data, pntre.ctypes.data, int(row_weight), bounds.ctypes.data)
    if st:
        raise FusedMMError(status_string(st))
    return bounds


class Plan:
    """``fusedmm_b200_plan_*``: the CSR kept on the device together with its split-row list, for many calls over
    one graph.  ``indx``, ``pntrb``, ``pntre`` (and optionally ``val``) are NumPy arrays or torch tensors; device
    tensors are borrowed and must outlive the plan."""

    def __init__(self, indx, pntrb, pntre, val=None):
        L = lib()
        ptrs, dts = zip(*[_describe(a) for a in (val, indx, pntrb, pntre)])
        self._keep = (val, indx, pntrb, pntre)
        self.m = len(pntrb)
        pb, ib = np.dtype(dts[2]).itemsize * 8, np.dtype(dts[1]).itemsize * 8
        vd = -1 if val is None else (0 if np.dtype(dts[0]) == np.float32 else 1)
        self._h = C.c_void_p()
        fn = L.fusedmm_b200_plan_create
        fn.restype = C.c_int
        fn.argtypes = [C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                       C.c_void_p, C.POINTER(C.c_void_p)]
        st = fn(pb, ib, self.m, 0, ptrs[1], ptrs[2], ptrs[3], vd, ptrs[0], C.byref(self._h))
        if st:
            raise FusedMMError(status_string(st))

    def csr(self, imessage, n, k, x, ldx, y, ldy, beta, z, ldz, sop=None, stream=None):
        """``fusedmm_b200_plan_csr``: the call without the CSR arguments; returns the status code."""
        L = lib()
        ptrs, dts = zip(*[_describe(a) for a in (x, y, z)])
        dtype = 0 if np.dtype(dts[2]) == np.float32 else 1
        spec = None
        if sop is not None:
            kind, *params = (sop,) if isinstance(sop, int) else tuple(sop)
            params = list(params) + [0.0] * (3 - len(params))
            spec = C.byref(SopSpec(int(kind), 0, *map(float, params)))
        fn = L.fusedmm_b200_plan_csr
        fn.restype = C.c_int
        fn.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p,
                       C.c_int64, C.c_double, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
        return fn(self._h, dtype, imessage, n, k, ptrs[0], ldx, ptrs[1], ldy, beta, ptrs[2], ldz, spec, stream)

    def close(self):
        if self._h:
            lib().fusedmm_b200_plan_destroy.argtypes = [C.c_void_p]
            lib().fusedmm_b200_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
