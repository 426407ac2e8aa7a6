"""Parity of the CUDA path with the reference, through the C ABI, on a GPU.

Every comparison is against the CPU oracle (pinned to the reference in test_oracle_pin.py), against the
golden outputs of the reference itself, or -- at full benchmark size -- against properties that do not
need a CPU pass.  Tolerances: 1e-4 (float32) and 1e-10 (float64) in the metric of cases.rel_err.
"""
import ctypes
from pathlib import Path

import numpy as np
import pytest

from cases import within_tolerance, MESSAGES, RTOL, dense, random_csr, rel_err
from fusedmm_b200 import api, messages as M, synth

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden" / "reference_general_kernel.npz"


def dev(a, device):
    import torch
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(device)


def as_rowptr(pntrb, pntre):
    """(pntrb, pntre) -> one rowptr array when row r+1 starts where row r ends, else None."""
    if len(pntrb) and (pntre[:-1] == pntrb[1:]).all():
        return np.concatenate([pntrb, pntre[-1:]])
    return None


def run_gpu(device, msg, m, n, k, val, indx, pntrb, pntre, x, ldx, y, ldy, beta, z, ldz, sop=None):
    """device-resident call; returns (status, Z as numpy).  With pntre=None, pntrb is a rowptr array of
    m+1 entries, the call gets the two views (rowptr, rowptr+1) of it, as callers of the reference pass
    them, and the edge-stream scheduler (which needs that layout) is selected."""
    import torch
    t = [dev(a, device) for a in (val, indx, pntrb, pntre, x, y, z)]
    if pntre is None:
        t[2], t[3] = t[2][:-1], t[2][1:]
        api.set_option("engine", 2)
    try:
        return _run_gpu(t, msg, m, n, k, ldx, ldy, beta, ldz, sop)
    finally:
        api.set_option("engine", 0)


def _run_gpu(t, msg, m, n, k, ldx, ldy, beta, ldz, sop):
    import torch
    st = api.fusedMM_csr(msg, m, n, k, 1.0, 0, m, n, t[0], t[1], t[2], t[3], t[4], ldx, t[5], ldy, beta,
                         t[6], ldz, sop=sop)
    torch.cuda.synchronize()
    return st, t[6].cpu().numpy()


def sop_for(name):
    return {"sigmoid": M.SOP_SIGMOID, "tdist": M.SOP_TDIST, "subl_norml_udef_mul_max": M.SOP_TDIST,
            "copyrhs_dot_udef_mul_add_fr": M.SOP_SIGMOID_TABLE_C}.get(name, M.SOP_IDENTITY)


def test_library_is_loaded_and_reports_itself(cuda_device):
    assert b"sm_100a" in api.lib().fusedmm_b200_version()


def test_golden_outputs_of_the_reference(cuda_device):
    data = np.load(GOLDEN)
    keys = sorted({k.split("_")[0] for k in data.files})
    assert len(keys) == 44
    engines, schedulers = set(), set()
    for key in keys:
        msg, m, n, k, ld, sop = (int(v) for v in data[key + "_meta"])
        want = data[key + "_z"]
        rowptr = as_rowptr(data[key + "_pntrb"], data[key + "_pntre"])
        st, z = run_gpu(cuda_device, msg, m, n, k, data[key + "_val"], data[key + "_indx"],
                        data[key + "_pntrb"] if rowptr is None else rowptr,
                        data[key + "_pntre"] if rowptr is None else None, data[key + "_x"], ld, data[key + "_y"],
                        ld, 0.0, np.zeros_like(want), ld, sop=sop)
        assert st == 0
        engines.add(api.call_info().lanes_per_edge)
        schedulers.add(api.call_info().engine)
        assert rel_err(z, want, k) <= RTOL[want.dtype], (key, str(data[key + "_name"]))
        assert (z[:, k:] == 0).all()  # padding columns are not written
    assert 0 in engines and len(engines) > 1  # both the vector engine and the element-strided one ran
    assert schedulers == {1, 2}               # and both the row and the edge-stream scheduler


@pytest.mark.parametrize("scheduler", ["rows", "stream"])
@pytest.mark.parametrize("vt", [np.float32, np.float64])
@pytest.mark.parametrize("name", list(MESSAGES))
def test_every_message_against_the_oracle(cuda_device, oracle, vt, name, scheduler):
    """Every message, both schedulers: "rows" gets a CSR with unused slots between rows (pntre[i] <
    pntrb[i+1]), which only the row scheduler can take; "stream" gets (rowptr, rowptr+1)."""
    msg = MESSAGES[name]
    rng = np.random.default_rng(sum(map(ord, name + vt.__name__ + scheduler)))
    m, n = 1500, 1100
    generic = msg not in (M.MSG_SIGMOID, M.MSG_TDIST, M.MSG_SPMM, M.MSG_GCN)
    lo, hi = -0.5, 0.5  # signed inputs for every message
    for k, it, pt in ((4, np.int32, np.int32), (32, np.int64, np.int64), (64, np.int32, np.int64),
                      (96, np.int32, np.int32), (128, np.int64, np.int64), (200, np.int32, np.int32),
                      (256, np.int32, np.int64), (30, np.int32, np.int32)):
        pntrb, pntre, indx, val = random_csr(rng, m, n, 9, pt, it, hub=1700, gaps=(scheduler == "rows"))
        val = val.astype(vt)
        x, y = np.nan_to_num(dense(rng, m, k, k, vt, lo, hi)), np.nan_to_num(dense(rng, n, k, k, vt, lo, hi))
        sop = sop_for(name)
        z0 = rng.uniform(-1, 1, size=(m, k)).astype(vt) if generic else np.zeros((m, k), vt)
        want = z0.copy()
        assert oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k, sop_kind=sop,
                          zero_first=not generic) == 0
        if scheduler == "stream":
            st, z = run_gpu(cuda_device, msg, m, n, k, val, indx, as_rowptr(pntrb, pntre), None, x, k, y, k,
                            0.0, z0, k, sop=sop)
        else:
            st, z = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, z0, k, sop=sop)
        assert st == 0
        info = api.call_info()
        if scheduler == "rows":
            assert info.engine == 1 and info.hub_rows >= 1 and info.kernel_launches >= 4
        elif info.lanes_per_edge:
            assert info.engine == 2 and info.kernel_launches == 3 and info.hub_chunks >= m * 9 * 0.7 / 256
        # the table sigmoid is a step function of s (bins of 10/2048): a last-bit difference in s from
        # the order of summation can move an edge to the neighbouring bin, a step of up to 2.5e-3
        tol = 5e-3 if sop == M.SOP_SIGMOID_TABLE_C else RTOL[np.dtype(vt)]

        def exact():  # the same inputs one precision up: float64 oracle for float, long double NumPy for double
            if vt == np.float32:
                ex = z0.astype(np.float64)
                oracle.csr(msg, m, n, k, val.astype(np.float64), indx, pntrb, pntre, x.astype(np.float64), k,
                           y.astype(np.float64), k, 0.0, ex, k, sop_kind=sop, zero_first=not generic)
                return ex
            from oracle.cpu import numpy_fusedmm
            return numpy_fusedmm(msg, m, k, val, indx, pntrb, pntre, x, y, z0, sop_kind=sop, dtype=np.longdouble)

        ok, e, e_gpu, e_or = within_tolerance(z, want, tol, exact)
        assert ok, (name, k, it, pt, e, e_gpu, e_or)


@pytest.mark.parametrize("vt", [np.float32, np.float64])
def test_wide_rows_and_every_tiling(cuda_device, oracle, vt):
    rng = np.random.default_rng(11)
    m, n = 300, 257
    pntrb, pntre, indx, val = random_csr(rng, m, n, 6, np.int64, np.int32, hub=900)
    val = val.astype(vt)
    w = 4 if vt == np.float32 else 2
    tilings = [(4, 1), (8, 1), (8, 2), (8, 4), (16, 1), (16, 2), (16, 4), (32, 1), (32, 2), (32, 4), (32, 8), (32, 16)]
    try:
        for g, nv in tilings:
            for k in (g * nv * w, g * nv * w - w):
                if k <= 0:
                    continue
                x, y = np.nan_to_num(dense(rng, m, k, k, vt)), np.nan_to_num(dense(rng, n, k, k, vt))
                for msg, sop in ((M.MSG_SIGMOID, M.SOP_SIGMOID), (M.MSG_TDIST, M.SOP_FR), (M.MSG_SPMM, 0)):
                    want = np.zeros((m, k), vt)
                    oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k, sop_kind=sop)
                    assert api.set_option("force_tiling", (g << 8) | nv) == 0
                    for rp, pe, eng in ((pntrb, pntre, 1), (as_rowptr(pntrb, pntre), None, 2 if nv <= 8 else 1)):
                        st, z = run_gpu(cuda_device, msg, m, n, k, val, indx, rp, pe, x, k, y, k, 0.0,
                                        np.zeros((m, k), vt), k, sop=sop)
                        info = api.call_info()
                        assert st == 0 and (info.lanes_per_edge, info.vectors_per_lane, info.engine) == (g, nv, eng)
                        assert rel_err(z, want) <= RTOL[np.dtype(vt)], (g, nv, k, hex(msg), eng)
    finally:
        api.set_option("force_tiling", 0)
    # wider than any tiling: element-strided engine
    k = 2056 if vt == np.float32 else 1032
    x, y = np.nan_to_num(dense(rng, m, k, k, vt)), np.nan_to_num(dense(rng, n, k, k, vt))
    want = np.zeros((m, k), vt)
    oracle.csr(M.MSG_SIGMOID, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k, sop_kind=1)
    st, z = run_gpu(cuda_device, M.MSG_SIGMOID, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0,
                    np.zeros((m, k), vt), k, sop=1)
    assert st == 0 and rel_err(z, want) <= RTOL[np.dtype(vt)]


def test_generic_kernel_equals_specialised_kernels(cuda_device):
    rng = np.random.default_rng(5)
    m, n, k = 800, 800, 128
    pntrb, pntre, indx, val = random_csr(rng, m, n, 12, np.int32, np.int32, hub=1200)
    val = val.astype(np.float32)
    x = np.nan_to_num(dense(rng, m, k, k, np.float32))
    for msg, sop in ((M.MSG_SIGMOID, M.SOP_SIGMOID), (M.MSG_TDIST, M.SOP_FR), (M.MSG_SPMM, 0), (M.MSG_GCN, 0)):
        _, a = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, k, x, k, 0.0,
                       np.zeros((m, k), np.float32), k, sop=sop)
        api.set_option("force_generic", 1)
        try:
            _, b = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, k, x, k, 0.0,
                           np.zeros((m, k), np.float32), k, sop=sop)
            assert api.call_info().pattern == 0
        finally:
            api.set_option("force_generic", 0)
        assert rel_err(a, b) <= 1e-5, hex(msg)  # same order of operations; only FMA contraction may differ


def test_host_pointers_padding_and_beta(cuda_device, oracle):
    """NumPy (host) arrays: staged in, Z copied back; ld > k padding is neither read nor written;
    beta == 0 overwrites, beta != 0 accumulates (kernels/src/kernels.c:501-520)."""
    rng = np.random.default_rng(21)
    m, n, k, ld = 700, 650, 64, 72
    pntrb, pntre, indx, val = random_csr(rng, m, n, 8, np.int64, np.int64, hub=800)
    val = val.astype(np.float32)
    x, y = dense(rng, m, k, ld, np.float32), dense(rng, n, k, ld, np.float32)  # NaN in the padding
    for beta in (0.0, 1.0):
        z = np.full((m, ld), 3.0, np.float32)
        want = z.copy()
        oracle.csr(M.MSG_SIGMOID, m, n, k, val, indx, pntrb, pntre, np.nan_to_num(x), ld, np.nan_to_num(y), ld,
                   beta, want, ld, sop_kind=1, zero_first=True)
        st = api.fusedMM_csr(M.MSG_SIGMOID, m, n, k, 1.0, 0, m, n, val, indx, pntrb, pntre, x, ld, y, ld, beta,
                             z, ld)
        info = api.call_info()
        assert st == 0 and info.h2d_bytes > 0 and info.d2h_bytes == m * k * 4
        assert rel_err(z, want, k) <= 1e-4
        assert (z[:, k:] == 3.0).all()
    # the general kernel's behaviour (always accumulate) on request
    api.set_option("beta_mode", 1)
    try:
        z = np.full((m, ld), 3.0, np.float32)
        want = z.copy()
        oracle.csr(M.MSG_GCN, m, n, k, val, indx, pntrb, pntre, np.nan_to_num(x), ld, np.nan_to_num(y), ld, 0.0,
                   want, ld, zero_first=False)
        assert api.fusedMM_csr(M.MSG_GCN, m, n, k, 1.0, 0, m, n, val, indx, pntrb, pntre, x, ld, y, ld, 0.0, z,
                               ld) == 0
        assert rel_err(z, want, k) <= 1e-4
    finally:
        api.set_option("beta_mode", 0)
    # X aliasing Y on the host is staged once
    z = np.zeros((m, ld), np.float32)
    xx = dense(rng, max(m, n), k, ld, np.float32)
    assert api.fusedMM_csr(M.MSG_TDIST, m, max(m, n), k, 1.0, 0, m, n, val, indx, pntrb, pntre, xx, ld, xx, ld,
                           0.0, z, ld, sop=M.SOP_FR) == 0
    want = np.zeros((m, ld), np.float32)
    oracle.csr(M.MSG_TDIST, m, n, k, val, indx, pntrb, pntre, np.nan_to_num(xx), ld, np.nan_to_num(xx), ld, 0.0,
               want, ld, sop_kind=M.SOP_FR)
    assert rel_err(z, want, k) <= 1e-4


def test_m_smaller_than_rows_and_unaligned_views(cuda_device, oracle):
    import torch
    rng = np.random.default_rng(8)
    rows, n, k = 400, 300, 32
    pntrb, pntre, indx, val = random_csr(rng, rows, n, 5, np.int32, np.int32)
    val = val.astype(np.float32)
    x, y = np.nan_to_num(dense(rng, rows, k, k, np.float32)), np.nan_to_num(dense(rng, n, k, k, np.float32))
    # only rows [r0, r0+m) -- the way one shard of a row-partitioned matrix is computed
    r0, m = 37, 123
    want = np.zeros((rows, k), np.float32)
    oracle.csr(M.MSG_SPMM, m, n, k, val, indx, pntrb[r0:], pntre[r0:], x[r0:], k, y, k, 0.0, want[r0:], k)
    t = {nm: dev(a, cuda_device) for nm, a in dict(val=val, indx=indx, pb=pntrb, pe=pntre, x=x, y=y).items()}
    z = torch.full((rows, k), 9.0, device=cuda_device)
    st = api.fusedMM_csr(M.MSG_SPMM, m, n, k, 1.0, 0, rows, n, t["val"], t["indx"], t["pb"][r0:], t["pe"][r0:],
                         t["x"][r0:], k, t["y"], k, 0.0, z[r0:], k)
    assert st == 0
    zc = z.cpu().numpy()
    assert rel_err(zc[r0:r0 + m], want[r0:r0 + m]) <= 1e-4
    assert (zc[:r0] == 9.0).all() and (zc[r0 + m:] == 9.0).all()
    # a Y that starts 4 bytes off a 16-byte boundary cannot use 16-byte loads: the vector engine with one-element
    # vectors, or (option element_vectors = 0) the element-strided engine
    ybig = torch.zeros(n * k + 1, device=cuda_device)
    yoff = ybig[1:].view(n, k)
    yoff.copy_(t["y"])
    for element_vectors in (1, 0):
        api.set_option("element_vectors", element_vectors)
        try:
            z2 = torch.zeros((rows, k), device=cuda_device)
            assert api.fusedMM_csr(M.MSG_SPMM, m, n, k, 1.0, 0, rows, n, t["val"], t["indx"], t["pb"][r0:], t["pe"][r0:],
                                   t["x"][r0:], k, yoff, k, 0.0, z2[r0:], k) == 0
            assert (api.call_info().lanes_per_edge > 0) == bool(element_vectors)
        finally:
            api.set_option("element_vectors", 1)
        assert rel_err(z2.cpu().numpy()[r0:r0 + m], want[r0:r0 + m]) <= 1e-4


def test_caller_supplied_sop_udef_func_is_recognised(cuda_device, oracle):
    """A host SOP_UDEF_FUNC (fusedMM.h:139) is matched against the device catalogue by sampling it."""
    L = api.lib()
    rng = np.random.default_rng(4)
    m, n, k = 200, 200, 16
    pntrb, pntre, indx, val = random_csr(rng, m, n, 6, np.int64, np.int64)
    val = val.astype(np.float32)
    x = np.nan_to_num(dense(rng, m, k, k, np.float32))
    HOOK = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_float, ctypes.POINTER(ctypes.c_float))
    fn = L.sfusedMM_csr_i64_udef
    I, F, P = ctypes.c_int64, ctypes.c_float, ctypes.c_void_p
    fn.argtypes = [ctypes.c_int32, I, I, I, F, I, I, I, P, P, P, P, P, I, P, I, F, P, I, HOOK]
    fn.restype = ctypes.c_int

    def call(body):
        def hook(v, out):
            out[0] = body(v)
            return 0
        z = np.zeros((m, k), np.float32)
        st = fn(M.MSG_TDIST, m, n, k, 1.0, 0, m, n, val.ctypes.data, indx.ctypes.data, pntrb.ctypes.data,
                pntre.ctypes.data, x.ctypes.data, k, x.ctypes.data, k, 0.0, z.ctypes.data, k, HOOK(hook))
        return st, z, api.call_info().sop_kind

    for body, kind, params in ((lambda v: 1.0 + 1.0 / v if v != 0 else np.inf, M.SOP_FR, (0, 0, 0)),
                               (lambda v: 1.0 / (1.0 + v), M.SOP_TDIST, (0, 0, 0)),
                               (lambda v: float(np.clip(-2.0 / (1.0 + v), -5, 5)) if v != -1 else -5.0,
                                M.SOP_TDIST_CLAMPED, (0, 0, 0)),
                               (lambda v: 3.0 / (2.0 + v) if v != -2 else np.inf, M.SOP_AFFINE_RECIP, (3.0, 2.0, 0.0))):
        with np.errstate(all="ignore"):
            st, z, got_kind = call(body)
        assert st == 0 and got_kind == kind
        want = np.zeros((m, k), np.float32)
        oracle.csr(M.MSG_TDIST, m, n, k, val, indx, pntrb, pntre, x, k, x, k, 0.0, want, k, sop_kind=kind,
                   sop_params=params)
        assert rel_err(z, want) <= 1e-4
    st, _, _ = call(lambda v: float(np.tanh(v)))  # not in the catalogue
    assert st == M.ERR_UDEF


def test_letter_dispatcher(cuda_device, oracle):
    rng = np.random.default_rng(6)
    m, n, k = 300, 300, 32
    pntrb, pntre, indx, val = random_csr(rng, m, n, 6, np.int32, np.int32)
    for vt in (np.float32, np.float64):
        x = np.nan_to_num(dense(rng, m, k, k, vt))
        v = val.astype(vt)
        for letter, msg in (("s", M.MSG_SIGMOID), ("t", M.MSG_TDIST), ("m", M.MSG_SPMM), ("g", M.MSG_GCN)):
            api.set_sop(M.SOP_SIGMOID if letter == "s" else M.SOP_FR)
            z = np.zeros((m, k), vt)
            api.gfusedMM_csr(letter, m, n, k, 1.0, 0, m, n, v, indx, pntrb, pntre, x, k, x, k, 0.0, z, k)
            want = np.zeros((m, k), vt)
            oracle.csr(msg, m, n, k, v, indx, pntrb, pntre, x, k, x, k, 0.0, want, k,
                       sop_kind=M.SOP_SIGMOID if letter == "s" else M.SOP_FR)
            assert rel_err(z, want) <= RTOL[np.dtype(vt)], letter
    api.set_sop(M.SOP_SIGMOID)


def test_scratch_grows_when_there_are_many_split_rows(cuda_device, oracle):
    """More split rows than the initial hub list holds: the chunk passes report the overflow, the host
    enlarges the scratch and reruns them; whole rows are not recomputed."""
    m, n, k, deg = 70000, 64, 4, 33
    rng = np.random.default_rng(9)
    pntrb = (np.arange(m) * deg).astype(np.int32)
    pntre = pntrb + deg
    indx = rng.integers(0, n, size=m * deg).astype(np.int32)
    val = rng.uniform(0.5, 1.0, size=m * deg).astype(np.float32)
    y = np.nan_to_num(dense(rng, n, k, k, np.float32))
    api.set_option("hub_chunk", 32)
    try:
        z0 = np.ones((m, k), np.float32)
        st, z = run_gpu(cuda_device, M.MSG_SPMM, m, n, k, val, indx, pntrb, pntre, None, k, y, k, 1.0, z0, k)
        info = api.call_info()
    finally:
        api.set_option("hub_chunk", 256)
    assert st == 0 and info.hub_rows == m and info.hub_chunks == 2 * m
    want = np.ones((m, k), np.float32)
    oracle.csr(M.MSG_SPMM, m, n, k, val, indx, pntrb, pntre, y, k, y, k, 1.0, want, k)
    assert rel_err(z, want) <= 1e-4
    # the edge-stream scheduler: more quanta than its partition array holds at first
    api.lib().fusedmm_b200_release()
    api.set_option("edge_quantum", 32)
    try:
        st, z = run_gpu(cuda_device, M.MSG_SPMM, m, n, k, val, indx, as_rowptr(pntrb, pntre), None, None, k, y, k,
                        1.0, np.ones((m, k), np.float32), k)
        info = api.call_info()
    finally:
        api.set_option("edge_quantum", 256)
    assert st == 0 and info.engine == 2 and info.hub_chunks == (m * deg + 31) // 32 > 65536
    assert info.kernel_launches == 6  # one rerun
    assert rel_err(z, want) <= 1e-4


def test_scratch_growth_in_the_blocked_copy_back_does_not_accumulate_twice(cuda_device, oracle):
    """A host Z of 32 MB or more is computed and copied back in 8 blocks of rows.  With nnz = 0 (the reference never
    reads nnz) nothing sizes the split-row scratch beforehand; when a block then finds it too small, only that
    block's split rows are redone.  With beta = 1 every contribution must still be added exactly once."""
    rng = np.random.default_rng(97)
    m, n, k = 70_000, 5_000, 128          # Z: 35.8 MB
    deg = rng.poisson(4, size=m)
    hubs = rng.choice(m, size=2400, replace=False)
    deg[hubs] = rng.integers(300, 700, size=hubs.size)   # 300 split rows per block of rows
    rowptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    nnz = int(rowptr[-1])
    indx = rng.integers(0, n, size=nnz).astype(np.int32)
    val = rng.uniform(0.25, 1.5, size=nnz).astype(np.float32)
    y = rng.uniform(-0.5, 0.5, size=(n, k)).astype(np.float32)
    z0 = rng.uniform(-1, 1, size=(m, k)).astype(np.float32)
    want = z0.copy()
    assert oracle.csr(M.MSG_SPMM, m, n, k, val, indx, rowptr[:-1].copy(), rowptr[1:].copy(), y, k, y, k, 1.0, want, k,
                      zero_first=False) == 0
    api.lib().fusedmm_b200_release()
    api.set_option("hub_cap_initial", 64)
    try:
        z = z0.copy()
        st = api.fusedMM_csr(M.MSG_SPMM, m, n, k, 1.0, 0, m, n, val, indx, rowptr[:-1], rowptr[1:], None, k, y, k, 1.0, z, k)
        info = api.call_info()
    finally:
        api.set_option("hub_cap_initial", 1 << 16)
        api.lib().fusedmm_b200_release()
    assert st == 0 and info.hub_rows == hubs.size
    assert info.kernel_launches > 8 * 4          # 8 blocks, and the split rows of the blocks that overflowed again
    assert rel_err(z, want) <= 1e-4
    # column ids and edge values came in block by block behind Y (the default); all inputs first gives the same Z
    # and moves the same bytes
    api.set_option("blocked_inputs", 0)
    try:
        z2 = z0.copy()
        st2 = api.fusedMM_csr(M.MSG_SPMM, m, n, k, 1.0, 0, m, n, val, indx, rowptr[:-1], rowptr[1:], None, k, y, k, 1.0, z2, k)
        info2 = api.call_info()
    finally:
        api.set_option("blocked_inputs", 1)
    assert st2 == 0 and np.array_equal(z, z2)
    assert info.h2d_bytes == info2.h2d_bytes == rowptr.nbytes + indx.nbytes + val.nbytes + y.nbytes + z0.nbytes


def test_one_process_drives_several_gpus_from_threads(cuda_device, oracle):
    """The single-process form of the multi-GPU run: one host thread per GPU, each with its own device current and its
    row shard (Y replicated); calls on different devices do not serialise on a library-wide lock.  The shards put
    together must equal one GPU's result bit for bit."""
    import threading
    import torch
    ndev = torch.cuda.device_count()
    if ndev < 2:
        pytest.skip("needs at least two GPUs")
    ndev = min(ndev, 4)
    cfg, csr, x = synth.make_config("c2_fr_rmat20_k256", device="cpu", scale=16)
    n, k, nnz = csr.n, cfg["k"], csr.nnz
    rp = csr.rowptr.numpy()
    bounds = api.shard_rows(rp[:-1].copy(), rp[1:].copy(), ndev, row_weight=8)
    parts, errors = [None] * ndev, []

    def work(g):
        try:
            torch.cuda.set_device(g)
            d = torch.device("cuda", g)
            t = [a.to(d) for a in (csr.val, csr.indx, csr.rowptr, x)]
            r0, r1 = int(bounds[g]), int(bounds[g + 1])
            z = torch.zeros((r1 - r0, k), device=d)
            for _ in range(5):
                st = api.fusedMM_csr(cfg["msg"], r1 - r0, n, k, 1.0, nnz, n, n, t[0], t[1], t[2][r0:-1], t[2][r0 + 1:], t[3][r0:], k,
                                     t[3], k, 0.0, z, k, sop=cfg["sop"])
                assert st == 0, api.status_string(st)
            parts[g] = z.cpu()
        except Exception as exc:  # noqa: BLE001
            errors.append((g, repr(exc)))

    threads = [threading.Thread(target=work, args=(g,)) for g in range(ndev)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    torch.cuda.set_device(0)
    assert not errors, errors
    t = [a.to(cuda_device) for a in (csr.val, csr.indx, csr.rowptr, x)]
    whole = torch.zeros((n, k), device=cuda_device)
    assert api.fusedMM_csr(cfg["msg"], n, n, k, 1.0, nnz, n, n, t[0], t[1], t[2][:-1], t[2][1:], t[3], k, t[3], k, 0.0, whole, k,
                           sop=cfg["sop"]) == 0
    assert torch.equal(torch.cat(parts), whole.cpu())


def test_peer_stores_replicate_finished_rows(cuda_device, oracle):
    """fusedmm_b200_csr_multi: finished rows also go to the peers' Z buffers.  Two more buffers on the same
    GPU stand in for the peers (on several GPUs the addresses come from peer-mapped memory); vector engine
    with split rows, and the element-strided engine."""
    import torch
    rng = np.random.default_rng(31)
    m, n = 900, 700
    for k in (64, 30):
        pntrb, pntre, indx, val = random_csr(rng, m, n, 7, np.int64, np.int32, hub=1300)
        val = val.astype(np.float32)
        x, y = np.nan_to_num(dense(rng, m, k, k, np.float32)), np.nan_to_num(dense(rng, n, k, k, np.float32))
        r0 = 100  # a row shard: rows [r0, m)
        t = [dev(a, cuda_device) for a in (val, indx, pntrb, pntre, x, y)]
        zs = [torch.full((m, k), 5.0, device=cuda_device) for _ in range(3)]
        st = api.fusedMM_csr(M.MSG_TDIST, m - r0, n, k, 1.0, 0, m, n, t[0], t[1], t[2][r0:], t[3][r0:], t[4][r0:],
                             k, t[5], k, 0.0, zs[0][r0:], k, sop=M.SOP_TDIST,
                             z_peers=[zs[1][r0:].data_ptr(), zs[2][r0:].data_ptr()])
        torch.cuda.synchronize()
        assert st == 0 and api.call_info().hub_rows >= 1
        want = np.full((m, k), 5.0, np.float32)
        oracle.csr(M.MSG_TDIST, m - r0, n, k, val, indx, pntrb[r0:].copy(), pntre[r0:].copy(), x[r0:], k, y, k, 0.0,
                   want[r0:], k, sop_kind=M.SOP_TDIST)
        assert rel_err(zs[0].cpu().numpy(), want) <= 1e-4
        # rows without edges are not sent: a peer zeroes them in its own copy from the row pointers
        empty = torch.from_numpy(pntre[r0:] <= pntrb[r0:]).to(cuda_device)
        assert bool(empty.any()) and bool((zs[1][r0:][empty] == 5.0).all()) and bool((zs[0][r0:][empty] == 0.0).all())
        assert torch.equal(zs[0][r0:][~empty], zs[1][r0:][~empty])
        for peer in zs[1:]:
            assert api.zero_empty_rows(t[2][r0:], t[3][r0:], peer[r0:], k, k) == 0
        torch.cuda.synchronize()
        assert torch.equal(zs[0], zs[1]) and torch.equal(zs[0], zs[2])
        # option multi_skip_empty_rows = 0: every row of the shard is sent
        zs = [torch.full((m, k), 5.0, device=cuda_device) for _ in range(2)]
        api.set_option("multi_skip_empty_rows", 0)
        try:
            st = api.fusedMM_csr(M.MSG_TDIST, m - r0, n, k, 1.0, 0, m, n, t[0], t[1], t[2][r0:], t[3][r0:], t[4][r0:],
                                 k, t[5], k, 0.0, zs[0][r0:], k, sop=M.SOP_TDIST, z_peers=[zs[1][r0:].data_ptr()])
        finally:
            api.set_option("multi_skip_empty_rows", 1)
        torch.cuda.synchronize()
        assert st == 0 and torch.equal(zs[0], zs[1]) and rel_err(zs[0].cpu().numpy(), want) <= 1e-4


def test_run_time_built_kernels_for_messages_without_a_built_in_one(cuda_device, oracle, tmp_path, monkeypatch):
    """Messages outside the four optimised patterns get a kernel specialised for them, built at run time with NVRTC
    (option jit = 2: on first use).  Its result must agree with the flag-interpreting kernel's and with the oracle
    within the tolerance; the cubin is found in the file cache afterwards."""
    import torch
    monkeypatch.setenv("FUSEDMM_B200_JIT_CACHE", str(tmp_path / "jit"))
    before = api.jit_stats()
    rng = np.random.default_rng(123)
    m, n = 1200, 1000
    names = ["subl_norml_udef_mul_max", "add_addrhs_vscadd_add", "max_dot_copy_mul_min", "min_noop_copy_vscadd_max",
             "copylhs_addlhs_mul_add", "subr_normr_noopsop_noopvsc_add"]
    try:
        for vt in (np.float32, np.float64):
            for k in (32, 128, 256):
                pntrb, pntre, indx, val = random_csr(rng, m, n, 9, np.int64, np.int32, hub=1500)
                val = val.astype(vt)
                x, y = np.nan_to_num(dense(rng, m, k, k, vt)), np.nan_to_num(dense(rng, n, k, k, vt))
                for name in names[:3] if k != 128 else names:
                    msg, sop = MESSAGES[name], sop_for(name)
                    z0 = rng.uniform(-1, 1, size=(m, k)).astype(vt)
                    want = z0.copy()
                    assert oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k, sop_kind=sop,
                                      zero_first=False) == 0
                    api.set_option("jit", 0)
                    st0, z_rt = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, z0.copy(), k, sop=sop)
                    assert st0 == 0 and api.call_info().jit_kernel == 0
                    api.set_option("jit", 2)
                    st1, z_jit = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, z0.copy(), k, sop=sop)
                    info = api.call_info()
                    assert st1 == 0 and info.jit_kernel == 1 and info.hub_rows >= 1, (name, k, vt)

                    def exact():
                        if vt == np.float32:
                            ex = z0.astype(np.float64)
                            oracle.csr(msg, m, n, k, val.astype(np.float64), indx, pntrb, pntre, x.astype(np.float64), k,
                                       y.astype(np.float64), k, 0.0, ex, k, sop_kind=sop, zero_first=False)
                            return ex
                        from oracle.cpu import numpy_fusedmm
                        return numpy_fusedmm(msg, m, k, val, indx, pntrb, pntre, x, y, z0, sop_kind=sop, dtype=np.longdouble)

                    ok, e, e_gpu, e_or = within_tolerance(z_jit, want, RTOL[np.dtype(vt)], exact)
                    assert ok, (name, k, vt, e, e_gpu, e_or)
                    assert rel_err(z_jit, z_rt) <= RTOL[np.dtype(vt)]
    finally:
        api.set_option("jit", 1)
    after = api.jit_stats()
    assert after["nvrtc_found"] == 1 and after["failures"] == before["failures"]
    assert after["compiled"] - before["compiled"] >= 18 and after["launches"] > before["launches"]
    assert len(list((tmp_path / "jit").glob("sm100a_*.cubin"))) == after["compiled"] - before["compiled"]
    # policy 1 (the default): a small call does not compile anything ...
    msg = MESSAGES["add_addrhs_vscadd_add"] ^ M.AOP_ADD ^ M.AOP_MAX   # a tuple not used above
    st, _ = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, z0.copy(), k)
    assert st == 0 and api.call_info().jit_kernel == 0 and api.jit_stats()["compiled"] == after["compiled"]
    # ... until the same message has come 8 times
    for _ in range(8):
        st, _ = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, z0.copy(), k)
    assert st == 0 and api.call_info().jit_kernel == 1 and api.jit_stats()["compiled"] == after["compiled"] + 1


@pytest.mark.parametrize("vt", [np.float32, np.float64])
def test_kernels_built_for_the_shape_of_a_call(cuda_device, oracle, tmp_path, monkeypatch, vt):
    """Kernels for the shape of a call.  K filling the tiling exactly selects the instantiation without bounds
    predicates (option exact_k, the default; compiled in).  Option jit_call_shape = 2 additionally runs every call whose Y
    lies within 2^32 elements behind 32-bit column ids on a kernel built at run time with 32-bit row offsets.  The four
    optimised messages and a generic one, K exact and ragged, int32 and int64 column ids, against the oracle; all
    variants must give the same bits (same arithmetic, same order)."""
    monkeypatch.setenv("FUSEDMM_B200_JIT_CACHE", str(tmp_path / "jit"))
    rng = np.random.default_rng(321)
    m, n = 1500, 1300
    w = 4 if vt == np.float32 else 2
    seen = 0
    try:
        for k, it in ((32 * w, np.int32), (64 * w, np.int32), (64 * w - w, np.int32), (16 * w, np.int64), (8 * w, np.int32)):
            pntrb, pntre, indx, val = random_csr(rng, m, n, 9, np.int64, it, hub=1700)
            val = val.astype(vt)
            x, y = np.nan_to_num(dense(rng, m, k, k, vt)), np.nan_to_num(dense(rng, n, k, k, vt))
            for name in ("sigmoid", "tdist", "spmm", "gcn", "max_dot_copy_mul_min"):
                msg, sop = MESSAGES[name], sop_for(name)
                generic = name == "max_dot_copy_mul_min"
                z0 = rng.uniform(-1, 1, size=(m, k)).astype(vt) if generic else np.zeros((m, k), vt)
                want = z0.copy()
                assert oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k, sop_kind=sop,
                                  zero_first=not generic) == 0
                api.set_option("jit_call_shape", 0)
                api.set_option("jit", 2)
                api.set_option("exact_k", 0)
                st2, z_general = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, z0.copy(), k, sop=sop)
                api.set_option("exact_k", 1)
                st0, z_plain = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, z0.copy(), k, sop=sop)
                assert api.call_info().jit_kernel == int(generic)
                api.set_option("jit_call_shape", 2)
                st1, z_shape = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, z0.copy(), k, sop=sop)
                info = api.call_info()
                expect_jit = generic or it == np.int32
                assert st0 == st1 == st2 == 0 and info.jit_kernel == int(expect_jit), (name, k, it)
                seen += info.jit_kernel
                assert np.array_equal(z_plain, z_shape) and np.array_equal(z_plain, z_general), (name, k, it)
                tol = RTOL[np.dtype(vt)]
                assert rel_err(z_shape, want) <= tol or generic, (name, k, it)
    finally:
        api.set_option("jit_call_shape", 0)
        api.set_option("jit", 1)
        api.set_option("exact_k", 1)
    assert seen >= 20


@pytest.mark.parametrize("vt", [np.float32, np.float64])
def test_rows_that_are_not_16_byte_granular(cuda_device, oracle, vt):
    """K, leading dimensions or bases that are not multiples of 16 bytes (K = 2 and 3 are graph layouts in the plane
    and in space): the vector engine with one-element vectors for K <= 512, every message kind, split rows, padded
    leading dimensions, against the oracle."""
    rng = np.random.default_rng(55)
    m, n = 1300, 1100
    for k, ldpad in ((1, 0), (2, 0), (3, 1), (7, 0), (30, 3), (67, 0), (250, 1), (511, 0), (512, 1)):
        ld = k + ldpad
        pntrb, pntre, indx, val = random_csr(rng, m, n, 8, np.int64, np.int32, hub=1500)
        val = val.astype(vt)
        x, y = np.nan_to_num(dense(rng, m, k, ld, vt)), np.nan_to_num(dense(rng, n, k, ld, vt))
        for name in ("sigmoid", "tdist", "spmm", "gcn", "add_addrhs_vscadd_add", "max_dot_copy_mul_min"):
            msg, sop = MESSAGES[name], sop_for(name)
            generic = msg not in (M.MSG_SIGMOID, M.MSG_TDIST, M.MSG_SPMM, M.MSG_GCN)
            z0 = rng.uniform(-1, 1, size=(m, ld)).astype(vt) if generic else np.zeros((m, ld), vt)
            want = z0.copy()
            assert oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, ld, y, ld, 0.0, want, ld, sop_kind=sop,
                              zero_first=not generic) == 0
            st, z = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, ld, y, ld, 0.0, z0.copy(), ld, sop=sop)
            info = api.call_info()
            granular = k % (16 // np.dtype(vt).itemsize) == 0 and ld % (16 // np.dtype(vt).itemsize) == 0
            assert st == 0 and info.lanes_per_edge > 0 and info.hub_rows >= 1, (name, k, ld)
            assert granular or info.lanes_per_edge * info.vectors_per_lane >= k   # one element per vector
            assert np.array_equal(z[:, k:], z0[:, k:])                                # padding columns untouched

            def exact():
                if vt == np.float32:
                    ex = z0.astype(np.float64)
                    oracle.csr(msg, m, n, k, val.astype(np.float64), indx, pntrb, pntre, x.astype(np.float64), ld,
                               y.astype(np.float64), ld, 0.0, ex, ld, sop_kind=sop, zero_first=not generic)
                    return ex
                from oracle.cpu import numpy_fusedmm
                return numpy_fusedmm(msg, m, k, val, indx, pntrb, pntre, x, y, z0, sop_kind=sop, dtype=np.longdouble)

            ok, e, e_gpu, e_or = within_tolerance(z, want, RTOL[np.dtype(vt)], exact, k)
            assert ok, (name, k, ld, e, e_gpu, e_or)
    # longer rows than the widest tiling of one-element vectors: the element-strided engine
    k = 515
    x, y = np.nan_to_num(dense(rng, m, k, k, vt)), np.nan_to_num(dense(rng, n, k, k, vt))
    want = np.zeros((m, k), vt)
    oracle.csr(M.MSG_TDIST, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k, sop_kind=M.SOP_TDIST)
    st, z = run_gpu(cuda_device, M.MSG_TDIST, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, np.zeros((m, k), vt), k, sop=M.SOP_TDIST)
    assert st == 0 and api.call_info().lanes_per_edge == 0 and rel_err(z, want) <= RTOL[np.dtype(vt)]


@pytest.mark.parametrize("vt", [np.float32, np.float64])
def test_chunk_launch_through_bulk_copies(cuda_device, oracle, vt):
    """Option bulk_chunks: the chunks of split rows gather their neighbour rows with bulk asynchronous copies into a
    shared-memory ring (fusedmm_bulk.cuh) instead of per-lane loads.  Same result as the default path bit for bit
    (same lane tiling, same order of additions) and within the tolerance of the oracle; ring of 16 and of 32 rows,
    blocks of 4 and 8 warps, K filling the tiling and ragged, chunks shorter and longer than the ring."""
    rng = np.random.default_rng(77)
    m, n = 900, 800
    w = 4 if vt == np.float32 else 2
    try:
        for k in (16 * w, 32 * w, 64 * w, 128 * w, 64 * w - w):
            pntrb, pntre, indx, val = random_csr(rng, m, n, 6, np.int64, np.int32, hub=2300)
            deg = pntre - pntrb
            deg_extra = np.where(deg > 0)[0][:6]
            val = val.astype(vt)
            x, y = np.nan_to_num(dense(rng, m, k, k, vt)), np.nan_to_num(dense(rng, n, k, k, vt))
            for msg, sop in ((M.MSG_SIGMOID, M.SOP_SIGMOID), (M.MSG_TDIST, M.SOP_FR), (M.MSG_SPMM, 0), (M.MSG_GCN, 0)):
                want = np.zeros((m, k), vt)
                assert oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k, sop_kind=sop) == 0
                api.set_option("bulk_chunks", 0)
                st0, z_ref = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, np.zeros((m, k), vt), k, sop=sop)
                assert st0 == 0
                for d, warps, chunk in ((16, 8, 256), (32, 4, 256), (32, 8, 40), (16, 2, 70)):
                    api.set_option("bulk_chunks", d)
                    api.set_option("bulk_warps", warps)
                    api.set_option("hub_chunk", chunk)
                    st, z = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, np.zeros((m, k), vt), k, sop=sop)
                    assert st == 0 and api.call_info().hub_rows >= 1, (hex(msg), k, d, warps, chunk)
                    assert rel_err(z, want) <= RTOL[np.dtype(vt)], (hex(msg), k, d, warps, chunk)
                    if chunk == 256:
                        assert rel_err(z, z_ref) <= RTOL[np.dtype(vt)] * 0.1
                api.set_option("hub_chunk", 256)
    finally:
        api.set_option("bulk_chunks", 0)
        api.set_option("bulk_warps", 8)
        api.set_option("hub_chunk", 256)


@pytest.mark.parametrize("vt", [np.float32, np.float64])
def test_chunks_visited_in_the_order_of_their_first_column(cuda_device, oracle, vt):
    """Option chunk_order (on by itself for graphs of 16 M edges and more, forced here): the chunks of split rows are
    visited sorted by the column id of their first edge (a counting sort on the device) instead of row by row.  Every
    chunk still writes its own partial sum and the fix-up adds them in the same order, so the result is the unsorted
    path's bit for bit; device arrays, host arrays and a plan (which sorts once, when it is made); vector and
    element-strided engine."""
    import torch
    rng = np.random.default_rng(78)
    m, n = 1500, 1300
    try:
        for k in (128, 37):
            pntrb, pntre, indx, val = random_csr(rng, m, n, 5, np.int64, np.int32, hub=2300)
            val = val.astype(vt)
            x, y = np.nan_to_num(dense(rng, m, k, k, vt)), np.nan_to_num(dense(rng, n, k, k, vt))
            for msg, sop, chunk in ((M.MSG_SIGMOID, M.SOP_SIGMOID, 64), (M.MSG_TDIST, M.SOP_FR, 256), (M.MSG_SPMM, 0, 32)):
                api.set_option("hub_chunk", chunk)
                want = np.zeros((m, k), vt)
                assert oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k, sop_kind=sop) == 0
                api.set_option("chunk_order", 0)
                for _ in range(2):  # the second call finds the scratch large enough: its launch count is the plain one
                    st0, z_ref = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, np.zeros((m, k), vt), k, sop=sop)
                n0 = api.call_info().kernel_launches
                api.set_option("chunk_order", 2)
                st, z = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, np.zeros((m, k), vt), k, sop=sop)
                assert st0 == 0 and st == 0 and api.call_info().hub_rows >= 1
                assert api.call_info().kernel_launches == n0 + 3, (api.call_info().kernel_launches, n0)
                assert np.array_equal(z, z_ref), (hex(msg), k, chunk)
                assert rel_err(z, want) <= RTOL[np.dtype(vt)]
                zh = np.zeros((m, k), vt)
                assert api.fusedMM_csr(msg, m, n, k, 1.0, 0, m, n, val, indx, pntrb, pntre, x, k, y, k, 0.0, zh, k, sop=sop) == 0
                assert np.array_equal(zh, z_ref), (hex(msg), k, chunk)
            api.set_option("hub_chunk", 256)
            for order in (0, 2):
                api.set_option("chunk_order", order)
                plan = api.Plan(indx, pntrb, pntre, val)
                zp = np.zeros((m, k), vt)
                assert plan.csr(M.MSG_SIGMOID, n, k, x, k, y, k, 0.0, zp, k, sop=M.SOP_SIGMOID) == 0
                assert api.call_info().hub_rows >= 1
                plan.close()
                if order == 0:
                    zp0 = zp
            assert np.array_equal(zp, zp0), k
            want = np.zeros((m, k), vt)
            assert oracle.csr(M.MSG_SIGMOID, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k, sop_kind=M.SOP_SIGMOID) == 0
            assert rel_err(zp, want) <= RTOL[np.dtype(vt)]
    finally:
        api.set_option("chunk_order", 1)
        api.set_option("hub_chunk", 256)


def test_one_multiply_add_row_addresses_with_32_bit_column_ids(cuda_device, oracle):
    """Option offset32 (on by default): with 32-bit column ids the whole-row launch of the 16-lane tiling forms the
    address of a neighbour row with one multiply-add.  Same bits as the 64-bit form (option off, or 64-bit column
    ids), K filling the tiling and ragged, Y more than 2^32 bytes long in total."""
    import torch
    rng = np.random.default_rng(79)
    m = 700
    try:
        for vt, k, n in ((np.float32, 128, 900), (np.float32, 100, 900), (np.float64, 64, 900), (np.float64, 50, 900),
                         (np.float32, 128, (1 << 23) + 4096)):
            free_b, _ = torch.cuda.mem_get_info()
            if n * k * np.dtype(vt).itemsize * 3 > free_b:
                continue
            pntrb, pntre, indx, val = random_csr(rng, m, n, 9, np.int64, np.int32, hub=600)
            assert 0 <= indx.min() and indx.max() < n   # with the long Y: neighbours on both sides of byte 2^32
            val = val.astype(vt)
            x = np.nan_to_num(dense(rng, m, k, k, vt))
            y = dev(np.nan_to_num(dense(rng, 900, k, k, vt)), cuda_device).repeat((n + 899) // 900, 1)[:n].contiguous()
            tx, tv = dev(x, cuda_device), dev(val, cuda_device)
            tb, te = dev(pntrb, cuda_device), dev(pntre, cuda_device)
            for msg, sop in ((M.MSG_SIGMOID, M.SOP_SIGMOID), (M.MSG_SPMM, 0)):
                outs = []
                for off32, it in ((1, np.int32), (0, np.int32), (1, np.int64)):
                    api.set_option("offset32", off32)
                    z = torch.zeros((m, k), dtype=y.dtype, device=cuda_device)
                    ti = dev(indx.astype(it), cuda_device)
                    assert api.fusedMM_csr(msg, m, n, k, 1.0, 0, m, n, tv, ti, tb, te, tx, k, y, k, 0.0, z, k, sop=sop) == 0
                    torch.cuda.synchronize()
                    assert api.call_info().lanes_per_edge in (16, 32)
                    outs.append(z.cpu().numpy())
                assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2]), (vt, k, n, hex(msg))
                # Y repeats with period 900: the oracle works on the first 900 rows and the column ids modulo 900
                want = np.zeros((m, k), vt)
                assert oracle.csr(msg, m, 900, k, val, (indx % 900).astype(np.int32), pntrb, pntre, x, k, y[:900].cpu().numpy(), k, 0.0,
                                  want, k, sop_kind=sop) == 0
                assert rel_err(outs[0], want) <= RTOL[np.dtype(vt)]
            del y
    finally:
        api.set_option("offset32", 1)


@pytest.mark.parametrize("vt", [np.float32, np.float64])
def test_whole_rows_sorted_by_length_inside_windows(cuda_device, oracle, vt):
    """Option row_bins (on by itself for graphs of 4 M edges and more, forced here): the whole-row launch takes its rows
    from a permutation that sorts every window of 2048 consecutive rows by length, so that the rows sharing a warp are
    about equally long.  Every row is still computed by one group of lanes over its edges in order: same bits as the
    unsorted launch; several windows and a ragged last one, 2 / 4 / 8 rows per warp, direct call, host arrays, plan."""
    rng = np.random.default_rng(80)
    m, n = 2048 * 3 + 777, 3000
    w = 4 if vt == np.float32 else 2
    try:
        for k in (32 * w, 16 * w - w, 8 * w, 3, 64 * w, 50 * w):
            pntrb, pntre, indx, val = random_csr(rng, m, n, 7, np.int64, np.int32, hub=700, gaps=True)
            val = val.astype(vt)
            x, y = np.nan_to_num(dense(rng, m, k, k, vt)), np.nan_to_num(dense(rng, n, k, k, vt))
            for msg, sop in ((M.MSG_SIGMOID, M.SOP_SIGMOID), (M.MSG_GCN, 0)):
                want = np.zeros((m, k), vt)
                assert oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k, sop_kind=sop) == 0
                outs = []
                for bins in (0, 2):
                    api.set_option("row_bins", bins)
                    st, z = run_gpu(cuda_device, msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, np.zeros((m, k), vt), k, sop=sop)
                    assert st == 0 and (api.call_info().lanes_per_edge < 32 or k > 32 * w)
                    launches = api.call_info().kernel_launches
                    zh = np.zeros((m, k), vt)
                    assert api.fusedMM_csr(msg, m, n, k, 1.0, 0, m, n, val, indx, pntrb, pntre, x, k, y, k, 0.0, zh, k, sop=sop) == 0
                    plan = api.Plan(indx, pntrb, pntre, val)
                    zp = np.zeros((m, k), vt)
                    assert plan.csr(msg, n, k, x, k, y, k, 0.0, zp, k, sop=sop) == 0
                    plan.close()
                    outs.append((z, zh, zp, launches))
                assert outs[1][3] == outs[0][3] + 1
                if k <= 32 * w:   # longer rows: sorted, two rows share a warp; unsorted, a row has the warp to itself
                    for i in range(3):
                        assert np.array_equal(outs[0][i], outs[1][i]), (k, hex(msg), i)
                assert np.array_equal(outs[1][0], outs[1][1])
                for i in range(3):
                    assert rel_err(outs[1][i], want) <= RTOL[np.dtype(vt)] and rel_err(outs[0][i], want) <= RTOL[np.dtype(vt)]
    finally:
        api.set_option("row_bins", 1)


def test_host_arrays_step_on_one_gpu(cuda_device, oracle, tmp_path):
    """fusedmm_b200.dist.HostStep with a group of one rank: pinned host arrays in, the rank's slice of Y and of the graph
    to the GPU, re-based row pointers, the library's call on device arrays, Z back to the host array; same bits as the
    plain host-array call (the multi-rank parts are covered on CPU by tests/test_dist_gloo.py and on GPUs by bench.py)."""
    import torch
    import torch.distributed as dist
    from fusedmm_b200 import dist as fdist
    own_group = not dist.is_initialized()
    if own_group:
        dist.init_process_group("gloo", init_method=f"file://{tmp_path}/rendezvous", rank=0, world_size=1)
    try:
        rng = np.random.default_rng(81)
        m = n = 1500
        k = 128
        pntrb, pntre, indx, val = random_csr(rng, m, n, 8, np.int64, np.int32, hub=900)
        rowptr = np.concatenate([pntrb, pntre[-1:]])
        val = val.astype(np.float32)
        y = np.nan_to_num(dense(rng, n, k, k, np.float32))
        x_other = np.nan_to_num(dense(rng, m, k, k, np.float32))
        bounds = fdist.shard_bounds(rowptr, 1)
        for msg, sop, same, with_val in ((M.MSG_SIGMOID, M.SOP_SIGMOID, True, False), (M.MSG_SPMM, 0, False, True),
                                        (M.MSG_TDIST, M.SOP_FR, True, False)):
            hs = fdist.HostStep(n, k, torch.float32, cuda_device, dist, bounds, with_val=with_val)
            ty = torch.from_numpy(y).pin_memory()
            tx = ty if same else torch.from_numpy(x_other).pin_memory()
            z_host = torch.full((m, k), -777.0).pin_memory()
            with torch.cuda.device(cuda_device):
                st = hs.step(msg, torch.from_numpy(rowptr), torch.from_numpy(indx), torch.from_numpy(val) if with_val else None,
                             tx, ty, z_host, sop=sop)
            assert st == 0 and hs.out_rows() == (0, m)
            assert hs.d2h_bytes == m * k * 4 and hs.h2d_bytes >= n * k * 4 + (m + 1) * 8 + indx.nbytes
            zd = np.zeros((m, k), np.float32)
            assert api.fusedMM_csr(msg, m, n, k, 1.0, int(rowptr[-1]), m, n, val, indx, rowptr[:-1], rowptr[1:],
                                   y if same else x_other, k, y, k, 0.0, zd, k, sop=sop) == 0
            assert np.array_equal(z_host.numpy(), zd), hex(msg)
            want = np.zeros((m, k), np.float32)
            assert oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, y if same else x_other, k, y, k, 0.0, want, k, sop_kind=sop) == 0
            assert rel_err(zd, want) <= 1e-4
    finally:
        if own_group:
            dist.destroy_process_group()


def test_async_stream_entry(cuda_device, oracle):
    import torch
    rng = np.random.default_rng(10)
    m, n, k = 500, 500, 128
    pntrb, pntre, indx, val = random_csr(rng, m, n, 10, np.int64, np.int32, hub=700)
    val = val.astype(np.float32)
    x = np.nan_to_num(dense(rng, m, k, k, np.float32))
    t = [dev(a, cuda_device) for a in (val, indx, pntrb, pntre, x)]
    z = torch.zeros((m, k), device=cuda_device)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        st = api.fusedMM_csr(M.MSG_SIGMOID, m, n, k, 1.0, 0, m, n, t[0], t[1], t[2], t[3], t[4], k, t[4], k, 0.0,
                             z, k, sop=M.SOP_SIGMOID, stream=s.cuda_stream)
    assert st == 0
    s.synchronize()
    assert api.lib().fusedmm_b200_stream_status() == 0
    want = np.zeros((m, k), np.float32)
    oracle.csr(M.MSG_SIGMOID, m, n, k, val, indx, pntrb, pntre, x, k, x, k, 0.0, want, k, sop_kind=1)
    assert rel_err(z.cpu().numpy(), want) <= 1e-4
    # host arrays are refused on a caller's stream
    assert api.fusedMM_csr(M.MSG_SIGMOID, m, n, k, 1.0, 0, m, n, val, indx, pntrb, pntre, x, k, x, k, 0.0,
                           np.zeros((m, k), np.float32), k, stream=s.cuda_stream) == M.ERR_ARG


@pytest.mark.parametrize("name", ["c1_sigmoid_rmat14_k128"])
def test_benchmark_config_1_full_size(cuda_device, oracle, name):
    """The configuration the reference can run on a CPU, at full size, float32 and float64."""
    import torch
    for dtype, vt in ((torch.float32, np.float32), (torch.float64, np.float64)):
        cfg, csr, x = synth.make_config(name, device="cpu", dtype=dtype, ptr_dtype=torch.int64,
                                        idx_dtype=torch.int32)
        n, k = csr.n, cfg["k"]
        rp, ix, vl, xs = csr.rowptr.numpy(), csr.indx.numpy(), csr.val.numpy(), x.numpy()
        want = np.zeros((n, k), vt)
        assert oracle.csr(cfg["msg"], n, n, k, vl, ix, rp[:-1].copy(), rp[1:].copy(), xs, k, xs, k, 0.0, want,
                          k, sop_kind=cfg["sop"]) == 0
        st, z = run_gpu(cuda_device, cfg["msg"], n, n, k, vl, ix, rp[:-1].copy(), rp[1:].copy(), xs, k, xs, k,
                        0.0, np.zeros((n, k), vt), k, sop=cfg["sop"])
        assert st == 0 and api.call_info().hub_rows > 0
        assert rel_err(z, want) <= RTOL[np.dtype(vt)]


def test_properties_at_benchmark_size(cuda_device):
    """Size-independent checks on the headline workload (R-MAT scale 20, K=256) without a CPU pass:
    GCN of an all-ones Y counts neighbours exactly; SpMM is linear in Y; a run is reproducible bit for
    bit; computing row shards separately gives the same bits as one call."""
    import torch
    cfg, csr, x = synth.make_config("c2_fr_rmat20_k256", device=cuda_device)
    n, k = csr.n, cfg["k"]
    pb, pe = csr.pntrb.contiguous(), csr.pntre.contiguous()

    def call(msg, y, z, sop=None, rows=(0, n)):
        r0, r1 = rows
        return api.fusedMM_csr(msg, r1 - r0, n, k, 1.0, csr.nnz, n, n, csr.val, csr.indx, pb[r0:], pe[r0:],
                               x[r0:], k, y, k, 0.0, z[r0:], k, sop=sop)

    ones = torch.ones((n, k), device=cuda_device)
    z = torch.empty((n, k), device=cuda_device)
    assert call(M.MSG_GCN, ones, z) == 0
    info = api.call_info()
    assert info.hub_rows > 0 and info.engine == 1 and info.lanes_per_edge == 32, (info.hub_rows, info.engine, info.lanes_per_edge, info.vectors_per_lane)
    deg = csr.degrees().to(torch.float32)
    bad = (z != deg[:, None]).any(dim=1).nonzero().flatten()
    assert bad.numel() == 0, (bad[:10].tolist(), deg[bad[:10]].tolist(), z[bad[:10], 0].tolist())

    y2 = synth.dense_uniform(n, k, -1.0, 1.0, 7, device=cuda_device)
    za, zb, zc = (torch.empty((n, k), device=cuda_device) for _ in range(3))
    assert call(M.MSG_SPMM, x, za) == 0 and call(M.MSG_SPMM, y2, zb) == 0
    assert call(M.MSG_SPMM, 2.0 * x - 0.5 * y2, zc) == 0
    lin = 2.0 * za - 0.5 * zb
    scale = torch.maximum(lin.abs().amax(dim=1, keepdim=True), torch.tensor(1e-20, device=cuda_device))
    assert float(((zc - lin).abs() / scale).max()) <= 1e-4

    z1, z2 = torch.empty((n, k), device=cuda_device), torch.empty((n, k), device=cuda_device)
    assert call(cfg["msg"], x, z1, sop=cfg["sop"]) == 0 and call(cfg["msg"], x, z2, sop=cfg["sop"]) == 0
    assert torch.equal(z1, z2) and bool(torch.isfinite(z1).all())
    bounds = api.shard_rows(pb.cpu().numpy(), pe.cpu().numpy(), 4)
    z3 = torch.zeros((n, k), device=cuda_device)
    for g in range(4):
        assert call(cfg["msg"], x, z3, sop=cfg["sop"], rows=(int(bounds[g]), int(bounds[g + 1]))) == 0
    assert torch.equal(z1, z3)


@pytest.mark.parametrize("name,scale,vt", [("c2_fr_rmat20_k256", 13, np.float32), ("c3_tdist_er4m_k64", 17, np.float32),
                                           ("c4_spmm_rmat22_k512", 12, np.float32),
                                           ("c5_sigmoid_rmat24_k128", 16, np.float32),
                                           ("c5_sigmoid_rmat24_k128", 13, np.float64)])
def test_benchmark_configs_scaled_down_against_the_oracle(cuda_device, oracle, name, scale, vt):
    """Configurations 2-5 (same generator, message, SOP, K, value distribution and index widths as the full
    size, smaller graph) against the CPU oracle, device arrays and host arrays."""
    import torch
    dtype = torch.float32 if vt == np.float32 else torch.float64
    cfg, csr, x = synth.make_config(name, device="cpu", dtype=dtype, scale=scale, ptr_dtype=torch.int64,
                                    idx_dtype=torch.int32)
    n, k, sop = csr.n, cfg["k"], cfg["sop"] if cfg["sop"] is not None else 0
    rp, ix, vl, xs = csr.rowptr.numpy(), csr.indx.numpy(), csr.val.numpy(), x.numpy()
    want = np.zeros((n, k), vt)
    assert oracle.csr(cfg["msg"], n, n, k, vl, ix, rp[:-1].copy(), rp[1:].copy(), xs, k, xs, k, 0.0, want, k,
                      sop_kind=sop) == 0
    st, z = run_gpu(cuda_device, cfg["msg"], n, n, k, vl, ix, rp[:-1].copy(), rp[1:].copy(), xs, k, xs, k, 0.0,
                    np.zeros((n, k), vt), k, sop=sop)
    assert st == 0 and rel_err(z, want) <= RTOL[np.dtype(vt)]
    zh = np.zeros((n, k), vt)  # the same through host arrays (staged copies, X and Y aliased)
    assert api.fusedMM_csr(cfg["msg"], n, n, k, 1.0, csr.nnz, n, n, vl, ix, rp[:-1].copy(), rp[1:].copy(), xs, k, xs,
                           k, 0.0, zh, k, sop=sop) == 0
    assert rel_err(zh, want) <= RTOL[np.dtype(vt)]
    assert rel_err(zh, z) <= RTOL[np.dtype(vt)]  # not bit-equal: the nnz hint of this call splits long rows finer
    if n * k * np.dtype(vt).itemsize >= 32 << 20:
        # a large host Z is computed and copied back in 8 blocks of rows (4 launches each), overlapped
        assert api.call_info().kernel_launches >= 24 and api.call_info().d2h_bytes == n * k * np.dtype(vt).itemsize


def test_properties_at_full_size_of_config_3(cuda_device):
    """Erdos-Renyi, 4 194 304 vertices, K = 64 (short rows, several per warp): neighbour counts are exact, the
    t-distribution result is reproducible, finite, and independent of how the rows are sharded."""
    import torch
    cfg, csr, x = synth.make_config("c3_tdist_er4m_k64", device=cuda_device)
    n, k = csr.n, cfg["k"]
    pb, pe = csr.pntrb.contiguous(), csr.pntre.contiguous()
    ones = torch.ones((n, k), device=cuda_device)
    z = torch.empty((n, k), device=cuda_device)
    assert api.fusedMM_csr(M.MSG_GCN, n, n, k, 1.0, csr.nnz, n, n, csr.val, csr.indx, pb, pe, x, k, ones, k, 0.0, z,
                           k) == 0
    assert torch.equal(z, csr.degrees().to(torch.float32)[:, None].expand(n, k))
    z1, z2 = torch.empty((n, k), device=cuda_device), torch.zeros((n, k), device=cuda_device)
    assert api.fusedMM_csr(cfg["msg"], n, n, k, 1.0, csr.nnz, n, n, csr.val, csr.indx, pb, pe, x, k, x, k, 0.0, z1, k,
                           sop=cfg["sop"]) == 0
    bounds = api.shard_rows(pb.cpu().numpy(), pe.cpu().numpy(), 3)
    for g in range(3):
        r0, r1 = int(bounds[g]), int(bounds[g + 1])
        assert api.fusedMM_csr(cfg["msg"], r1 - r0, n, k, 1.0, csr.nnz, n, n, csr.val, csr.indx, pb[r0:], pe[r0:],
                               x[r0:], k, x, k, 0.0, z2[r0:], k, sop=cfg["sop"]) == 0
    assert torch.equal(z1, z2) and bool(torch.isfinite(z1).all())


@pytest.mark.parametrize("vt", ["f32", "f64"])
def test_properties_at_full_size_of_config_5(cuda_device, vt):
    """R-MAT scale 24 (16 777 216 vertices, about 520 million edges: int64 row pointers, int32 column ids, edge
    positions beyond 2^29 and n*ldy = 2^31), K = 128, float and double: neighbour counts are exact, the sigmoid
    message is finite, reproducible bit for bit and independent of how the rows are sharded, and a seeded sample of
    rows equals a float64 evaluation with torch on the device within the tolerance."""
    import torch
    free, _ = torch.cuda.mem_get_info()
    if free < (90 << 30):
        pytest.skip("needs about 90 GB of free device memory")
    dtype = torch.float32 if vt == "f32" else torch.float64
    cfg, csr, x = synth.make_config("c5_sigmoid_rmat24_k128", device=cuda_device, dtype=dtype)
    n, k = csr.n, cfg["k"]
    assert n == 1 << 24 and csr.nnz > (1 << 28) and csr.rowptr.dtype == torch.int64 and csr.indx.dtype == torch.int32
    pb, pe = csr.pntrb.contiguous(), csr.pntre.contiguous()
    deg = csr.degrees()
    z = torch.empty((n, k), dtype=dtype, device=cuda_device)
    ones = torch.ones((n, k), dtype=dtype, device=cuda_device)
    assert api.fusedMM_csr(M.MSG_GCN, n, n, k, 1.0, csr.nnz, n, n, csr.val, csr.indx, pb, pe, x, k, ones, k, 0.0, z, k) == 0
    assert api.call_info().hub_rows > 0
    for col in (0, k // 2, k - 1):
        assert torch.equal(z[:, col], deg.to(dtype))
    del ones
    z1 = torch.empty((n, k), dtype=dtype, device=cuda_device)
    assert api.fusedMM_csr(cfg["msg"], n, n, k, 1.0, csr.nnz, n, n, csr.val, csr.indx, pb, pe, x, k, x, k, 0.0, z1, k,
                           sop=cfg["sop"]) == 0
    assert api.fusedMM_csr(cfg["msg"], n, n, k, 1.0, csr.nnz, n, n, csr.val, csr.indx, pb, pe, x, k, x, k, 0.0, z, k,
                           sop=cfg["sop"]) == 0
    assert torch.equal(z, z1) and bool(torch.isfinite(z1).all())
    z.fill_(-1.0)
    bounds = api.shard_rows(pb.cpu().numpy(), pe.cpu().numpy(), 8)
    for g in range(8):
        r0, r1 = int(bounds[g]), int(bounds[g + 1])
        assert api.fusedMM_csr(cfg["msg"], r1 - r0, n, k, 1.0, csr.nnz, n, n, csr.val, csr.indx, pb[r0:], pe[r0:],
                               x[r0:], k, x, k, 0.0, z[r0:], k, sop=cfg["sop"]) == 0
    assert torch.equal(z, z1)
    # a sample of rows (the longest row, the last row with edges, 64 seeded ones) in float64 with torch
    rows = torch.cat([deg.argmax().reshape(1), (deg > 0).nonzero().flatten()[-1:],
                      torch.randint(0, n, (64,), generator=torch.Generator().manual_seed(5)).to(cuda_device)])
    worst = 0.0
    for r in rows.tolist():
        cols = csr.indx[int(csr.rowptr[r]):int(csr.rowptr[r + 1])].to(torch.int64)
        xr, yr = x[r].double(), x[cols].double()
        want = (torch.sigmoid(yr @ xr)[:, None] * yr).sum(dim=0)
        scale = torch.maximum(want.abs(), want.abs().max()).clamp_min(1e-30)
        worst = max(worst, float(((z1[r].double() - want).abs() / scale).max()))
    assert worst <= (1e-4 if vt == "f32" else 1e-10), worst


def test_32_bit_indices_with_more_than_2_31_elements_of_y(cuda_device):
    """Configuration 4 at full size (4 194 304 vertices, K = 512) with every index array int32: n*ldy = 2^31,
    so `cid*ldy` must be computed in 64 bits (an int32 build of the reference overflows here).  SpMM with the
    configuration's 1/deg(u) edge values and an all-ones Y must give exactly... 1 for every row that has edges
    (up to rounding of the sum of deg copies of 1/deg) and 0 for the others; GCN gives the degree exactly."""
    import torch
    cfg, csr, _ = synth.make_config("c4_spmm_rmat22_k512", device=cuda_device, ptr_dtype=torch.int32,
                                    idx_dtype=torch.int32)
    n, k = csr.n, cfg["k"]
    assert n * k == 2 ** 31 and csr.rowptr.dtype == torch.int32 and csr.indx.dtype == torch.int32
    pb, pe = csr.pntrb.contiguous(), csr.pntre.contiguous()
    ones = torch.ones((n, k), device=cuda_device)
    z = torch.empty((n, k), device=cuda_device)
    deg = csr.degrees().to(torch.float32)
    assert api.fusedMM_csr(M.MSG_GCN, n, n, k, 1.0, csr.nnz, n, n, csr.val, csr.indx, pb, pe, ones, k, ones, k, 0.0,
                           z, k) == 0
    assert torch.equal(z[:, 0], deg) and torch.equal(z[:, k - 1], deg) and torch.equal(z[-1], deg[-1].expand(k))
    assert api.fusedMM_csr(cfg["msg"], n, n, k, 1.0, csr.nnz, n, n, csr.val, csr.indx, pb, pe, ones, k, ones, k, 0.0,
                           z, k) == 0
    want = (deg > 0).to(torch.float32)
    assert float((z[:, 0] - want).abs().max()) <= 1e-4 and float((z[:, k // 2] - want).abs().max()) <= 1e-4
    # the last rows of Y (element offsets just below 2^31) are really read: make them distinctive
    y = torch.ones((n, k), device=cuda_device)
    y[n - 4096:] = 3.0
    assert api.fusedMM_csr(M.MSG_GCN, n, n, k, 1.0, csr.nnz, n, n, csr.val, csr.indx, pb, pe, y, k, y, k, 0.0, z,
                           k) == 0
    hi = torch.zeros(n, device=cuda_device)
    rows = torch.repeat_interleave(torch.arange(n, device=cuda_device), csr.degrees().to(torch.int64))
    hi.index_add_(0, rows, (csr.indx >= n - 4096).to(torch.float32))
    assert torch.equal(z[:, 7], deg + 2.0 * hi)


def test_check_csr_and_injected_allocation_failure(cuda_device, oracle):
    """fusedmm_b200_check_csr finds what the kernels would not (they do not bounds-check, like the reference);
    a device allocation that fails (injected on the host, nothing is done to the GPU) comes back as
    FUSEDMM_NOT_ENOUGH_MEM (-1, fusedMM.h:110) and leaves the library usable."""
    L = api.lib()
    fn = L.fusedmm_b200_check_csr
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64] + [ctypes.c_void_p] * 4
    rng = np.random.default_rng(12)
    m, n, k = 500, 400, 32
    pntrb, pntre, indx, val = random_csr(rng, m, n, 6, np.int64, np.int32, hub=900)
    rep = np.zeros(4, np.int64)
    assert fn(64, 32, m, n, indx.ctypes.data, pntrb.ctypes.data, pntre.ctypes.data, rep.ctypes.data) == 0
    deg = pntre - pntrb
    assert list(rep) == [0, 0, int(deg.sum()), int(deg.max())]
    bad = indx.copy()
    bad[int(pntrb[3])] = n + 5
    bad[int(pntrb[m // 3]) + 7] = -1
    t = dev(bad, cuda_device)
    assert fn(64, 32, m, n, t.data_ptr(), pntrb.ctypes.data, pntre.ctypes.data, rep.ctypes.data) == M.ERR_ARG
    assert rep[0] == 0 and rep[1] == 2
    swapped = pntre.copy()
    swapped[10] = pntrb[10] - 1
    assert fn(64, 32, m, n, indx.ctypes.data, pntrb.ctypes.data, swapped.ctypes.data, rep.ctypes.data) == M.ERR_ARG
    assert rep[0] == 1

    x = np.nan_to_num(dense(rng, max(m, n), k, k, np.float32))
    val = val.astype(np.float32)
    L.fusedmm_b200_release()  # so that the next call has to allocate its staging buffers and scratch
    z = np.zeros((m, k), np.float32)
    for nth in (1, 3):
        assert api.set_option("inject_alloc_failure", nth) == 0
        assert api.fusedMM_csr(M.MSG_SIGMOID, m, n, k, 1.0, 0, m, n, val, indx, pntrb, pntre, x, k, x, k, 0.0, z,
                               k) == M.ERR_NOMEM
        assert api.get_option("inject_alloc_failure") == 0
    assert api.fusedMM_csr(M.MSG_SIGMOID, m, n, k, 1.0, 0, m, n, val, indx, pntrb, pntre, x, k, x, k, 0.0, z, k) == 0
    want = np.zeros((m, k), np.float32)
    oracle.csr(M.MSG_SIGMOID, m, n, k, val, indx, pntrb, pntre, x, k, x, k, 0.0, want, k, sop_kind=M.SOP_SIGMOID)
    assert rel_err(z, want) <= 1e-4


C_CALLER = r"""
/* A caller of the reference, unchanged: VALUETYPE / INDEXTYPE, the flag macros, its own SOP_UDEF_FUNC. */
#include <stdio.h>
#include <stdlib.h>
#include <stdint.h>
#include <math.h>
#define VALUETYPE @VT@
#define INDEXTYPE @IT@
#include "fusedMM.h"

int SOP_UDEF_FUNC(VALUETYPE val, VALUETYPE *out) { *out = @SOP@; return FUSEDMM_SUCCESS_RETURN; }

static void *slurp(const char *name, size_t bytes) {
   void *p = malloc(bytes ? bytes : 1); FILE *f = fopen(name, "rb");
   if (!f || fread(p, 1, bytes, f) != bytes) { fprintf(stderr, "cannot read %s\n", name); exit(2); }
   fclose(f); return p;
}
int main(int argc, char **argv) {
   INDEXTYPE m = atol(argv[1]), n = atol(argv[2]), k = atol(argv[3]), nnz = atol(argv[4]);
   INDEXTYPE *rowptr = slurp("rowptr.bin", (m + 1) * sizeof(INDEXTYPE)), *indx = slurp("indx.bin", nnz * sizeof(INDEXTYPE));
   VALUETYPE *val = slurp("val.bin", nnz * sizeof(VALUETYPE)), *x = slurp("x.bin", m * k * sizeof(VALUETYPE));
   VALUETYPE *y = slurp("y.bin", n * k * sizeof(VALUETYPE)), *z = calloc(m * k, sizeof(VALUETYPE));
   int32_t imsg = 0;
   SET_VOP_FLAG(imsg, @VOP@); SET_ROP_FLAG(imsg, @ROP@); SET_SOP_FLAG(imsg, SOP_UDEF);
   SET_VSC_FLAG(imsg, VSC_MUL); SET_AOP_FLAG(imsg, AOP_ADD);
   int st = fusedMM_csr(imsg, m, n, k, 1.0, nnz, m, n, val, indx, rowptr, rowptr + 1, x, k, y, k, 0.0, z, k);
   FILE *o = fopen("z.bin", "wb"); fwrite(z, sizeof(VALUETYPE), m * k, o); fclose(o);
   printf("status %d message %#x\n", st, imsg);
   return st;
}
"""


@pytest.mark.parametrize("vt,it,vop,rop,sop_c,sop_kind", [
    ("float", "int64_t", "VOP_COPY_RHS", "ROP_DOT", "1.0 / (1.0 + exp(-val))", M.SOP_SIGMOID),
    ("double", "int32_t", "VOP_SUBR", "ROP_NORMR", "1.0 + 1.0 / val", M.SOP_FR)])
def test_unmodified_c_caller_of_the_reference(cuda_device, oracle, tmp_path, vt, it, vop, rop, sop_c, sop_kind):
    """The drop-in claim end to end: a C program written against the reference's header (its macros, its own
    SOP_UDEF_FUNC, host arrays) is compiled against include/fusedMM.h, linked with libfusedmm_b200.so and run."""
    import subprocess
    root = Path(__file__).resolve().parents[1]
    nvt = np.float32 if vt == "float" else np.float64
    nit = np.int64 if it == "int64_t" else np.int32
    rng = np.random.default_rng(77)
    m, n, k = 600, 500, 48
    pntrb, pntre, indx, val = random_csr(rng, m, n, 9, nit, nit, hub=1500)
    rowptr = as_rowptr(pntrb, pntre)
    nnz = int(rowptr[-1])
    indx, val = indx[:nnz].copy(), val[:nnz].astype(nvt)
    x, y = np.nan_to_num(dense(rng, m, k, k, nvt)), np.nan_to_num(dense(rng, n, k, k, nvt))
    for name, a in (("rowptr", rowptr), ("indx", indx), ("val", val), ("x", x), ("y", y)):
        a.tofile(tmp_path / f"{name}.bin")
    src = C_CALLER
    for key, rep in (("@VT@", vt), ("@IT@", it), ("@SOP@", sop_c), ("@VOP@", vop), ("@ROP@", rop)):
        src = src.replace(key, rep)
    (tmp_path / "caller.c").write_text(src)
    libdir = api.LIB_PATH.parent
    subprocess.run(["gcc", "-O1", "caller.c", f"-I{root / 'include'}", f"-L{libdir}", "-lfusedmm_b200",
                    f"-Wl,-rpath,{libdir}", "-lm", "-o", "caller"], cwd=tmp_path, check=True)
    run = subprocess.run(["./caller", str(m), str(n), str(k), str(nnz)], cwd=tmp_path, capture_output=True, text=True)
    assert run.returncode == 0, run.stdout + run.stderr
    msg = M.MSG_SIGMOID if rop == "ROP_DOT" else M.MSG_TDIST
    assert f"message {msg:#x}" in run.stdout
    z = np.fromfile(tmp_path / "z.bin", dtype=nvt).reshape(m, k)
    want = np.zeros((m, k), nvt)
    oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k, sop_kind=sop_kind)
    assert rel_err(z, want) <= RTOL[np.dtype(nvt)]


C_CALLER_LETTER = r"""
/* A caller of the reference's second public entry (kernels/include/kernels.h:17-43), unchanged: the typed
   dispatcher by kernel letter, INDEXTYPE from the caller, its own SOP_UDEF_FUNC as the generated kernels expect. */
#include <stdio.h>
#include <stdlib.h>
#include <stdint.h>
#include <math.h>
#define VALUETYPE @VT@
#define INDEXTYPE @IT@
#include "kernels.h"

int SOP_UDEF_FUNC(VALUETYPE val, VALUETYPE *out) { *out = @SOP@; return 0; }

static void *slurp(const char *name, size_t bytes) {
   void *p = malloc(bytes ? bytes : 1); FILE *f = fopen(name, "rb");
   if (!f || fread(p, 1, bytes, f) != bytes) { fprintf(stderr, "cannot read %s\n", name); exit(2); }
   fclose(f); return p;
}
int main(int argc, char **argv) {
   INDEXTYPE m = atol(argv[1]), n = atol(argv[2]), k = atol(argv[3]), nnz = atol(argv[4]);
   INDEXTYPE *rowptr = slurp("rowptr.bin", (m + 1) * sizeof(INDEXTYPE)), *indx = slurp("indx.bin", nnz * sizeof(INDEXTYPE));
   VALUETYPE *val = slurp("val.bin", nnz * sizeof(VALUETYPE)), *x = slurp("x.bin", m * k * sizeof(VALUETYPE));
   VALUETYPE *y = slurp("y.bin", n * k * sizeof(VALUETYPE)), *z = calloc(m * k, sizeof(VALUETYPE));
   @PRE@gfusedMM_csr('@LETTER@', m, n, k, 1.0, nnz, m, n, val, indx, rowptr, rowptr + 1, x, k, y, k, 0.0, z, k);
   trusted_@PRE@gfusedMM_csr('g', m, n, k, 1.0, nnz, m, n, val, indx, rowptr, rowptr + 1, x, k, y, k, 1.0, z, k);
   FILE *o = fopen("z.bin", "wb"); fwrite(z, sizeof(VALUETYPE), m * k, o); fclose(o);
   return 0;
}
"""


@pytest.mark.parametrize("vt,it,letter,sop_c,sop_kind", [
    ("float", "int32_t", "t", "1.0 / (1.0 + val)", M.SOP_TDIST),
    ("double", "int64_t", "s", "1.0 / (1.0 + exp(-val))", M.SOP_SIGMOID),
    ("float", "int64_t", "m", "val", M.SOP_IDENTITY)])
def test_unmodified_c_caller_of_the_letter_dispatcher(cuda_device, oracle, tmp_path, vt, it, letter, sop_c, sop_kind):
    """A C program written against the reference's kernels.h ({s,d}gfusedMM_csr and the trusted_ names, INDEXTYPE
    from the caller, its own SOP_UDEF_FUNC) is compiled against include/kernels.h, linked and run: the lettered
    message with beta = 0 followed by the GCN message with beta = 1 on the same Z."""
    import subprocess
    root = Path(__file__).resolve().parents[1]
    nvt = np.float32 if vt == "float" else np.float64
    nit = np.int64 if it == "int64_t" else np.int32
    rng = np.random.default_rng(78)
    m, n, k = 500, 400, 64
    pntrb, pntre, indx, val = random_csr(rng, m, n, 9, nit, nit, hub=1200)
    rowptr = as_rowptr(pntrb, pntre)
    nnz = int(rowptr[-1])
    indx, val = indx[:nnz].copy(), val[:nnz].astype(nvt)
    x, y = np.nan_to_num(dense(rng, m, k, k, nvt)), np.nan_to_num(dense(rng, n, k, k, nvt))
    for name, a in (("rowptr", rowptr), ("indx", indx), ("val", val), ("x", x), ("y", y)):
        a.tofile(tmp_path / f"{name}.bin")
    src = C_CALLER_LETTER
    for key, rep in (("@VT@", vt), ("@IT@", it), ("@SOP@", sop_c), ("@LETTER@", letter), ("@PRE@", "s" if vt == "float" else "d")):
        src = src.replace(key, rep)
    (tmp_path / "caller.c").write_text(src)
    libdir = api.LIB_PATH.parent
    subprocess.run(["gcc", "-O1", "-Wall", "-Werror", "caller.c", f"-I{root / 'include'}", f"-L{libdir}", "-lfusedmm_b200",
                    f"-Wl,-rpath,{libdir}", "-lm", "-o", "caller"], cwd=tmp_path, check=True)
    run = subprocess.run(["./caller", str(m), str(n), str(k), str(nnz)], cwd=tmp_path, capture_output=True, text=True)
    assert run.returncode == 0, run.stdout + run.stderr
    z = np.fromfile(tmp_path / "z.bin", dtype=nvt).reshape(m, k)
    msg = {"t": M.MSG_TDIST, "s": M.MSG_SIGMOID, "m": M.MSG_SPMM}[letter]
    want = np.zeros((m, k), nvt)
    oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k, sop_kind=sop_kind)
    oracle.csr(M.MSG_GCN, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 1.0, want, k, sop_kind=0, zero_first=False)
    assert rel_err(z, want) <= RTOL[np.dtype(nvt)]


def test_generators_give_the_same_graph_on_cpu_and_gpu(cuda_device):
    cpu = synth.rmat_edges(12, 16, seed=9)
    gpu = synth.rmat_edges(12, 16, seed=9, device=cuda_device)
    assert all(torch_equal(a, b.cpu()) for a, b in zip(cpu, gpu))
    a = synth.dense_uniform(300, 64, -1.0, 1.0, seed=4)
    b = synth.dense_uniform(300, 64, -1.0, 1.0, seed=4, device=cuda_device)
    assert torch_equal(a, b.cpu())


def torch_equal(a, b):
    import torch
    return torch.equal(a, b)


def test_plan_gives_the_same_bits_as_the_direct_call(cuda_device, oracle):
    """Inspector/executor split: the CSR staged once, the split-row list kept; every call through the plan
    equals the direct call bit for bit (same kernels, same chunking), for device and host arrays, with and
    without edge values, synchronous and on a stream."""
    import torch
    rng = np.random.default_rng(41)
    m, n, k = 2500, 2000, 128
    pntrb, pntre, indx, val = random_csr(rng, m, n, 11, np.int64, np.int32, hub=4000)
    rowptr = as_rowptr(pntrb, pntre)
    nnz = int(rowptr[-1])
    val = val[:nnz].astype(np.float32)
    indx = indx[:nnz].copy()
    x, y = np.nan_to_num(dense(rng, m, k, k, np.float32)), np.nan_to_num(dense(rng, n, k, k, np.float32))
    plan = api.Plan(indx, rowptr[:-1], rowptr[1:], val)          # host CSR: copied to the device once
    for msg, sop in ((M.MSG_SIGMOID, M.SOP_SIGMOID), (M.MSG_TDIST, M.SOP_FR), (M.MSG_SPMM, 0), (M.MSG_GCN, 0)):
        want = np.zeros((m, k), np.float32)
        oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k, sop_kind=sop)
        zd = np.zeros((m, k), np.float32)
        assert api.fusedMM_csr(msg, m, n, k, 1.0, nnz, m, n, val, indx, rowptr[:-1], rowptr[1:], x, k, y, k, 0.0, zd, k,
                               sop=sop) == 0
        direct_launches = api.call_info().kernel_launches
        zp = np.zeros((m, k), np.float32)
        assert plan.csr(msg, n, k, x, k, y, k, 0.0, zp, k, sop=sop) == 0
        info = api.call_info()
        assert info.kernel_launches == direct_launches - 1 and info.hub_rows >= 1   # no scan launch
        assert info.h2d_bytes == (x.nbytes if msg in (M.MSG_SIGMOID, M.MSG_TDIST) else 0) + y.nbytes  # no CSR copy
        assert np.array_equal(zp, zd) and rel_err(zp, want) <= 1e-4
        # device arrays, enqueued on a stream
        tx, ty, tz = dev(x, cuda_device), dev(y, cuda_device), torch.zeros((m, k), device=cuda_device)
        s = torch.cuda.Stream()
        torch.cuda.synchronize()
        with torch.cuda.stream(s):
            assert plan.csr(msg, n, k, tx, k, ty, k, 0.0, tz, k, sop=sop, stream=s.cuda_stream) == 0
        s.synchronize()
        assert np.array_equal(tz.cpu().numpy(), zd)
    plan.close()
    # a plan without edge values refuses a message that needs them
    plan2 = api.Plan(dev(indx, cuda_device), dev(rowptr, cuda_device)[:-1], dev(rowptr, cuda_device)[1:])
    z = np.zeros((m, k), np.float32)
    assert plan2.csr(M.MSG_SPMM, n, k, x, k, y, k, 0.0, z, k) == M.ERR_ARG
    assert plan2.csr(M.MSG_GCN, n, k, x, k, y, k, 0.0, z, k) == 0
    want = np.zeros((m, k), np.float32)
    oracle.csr(M.MSG_GCN, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k)
    assert rel_err(z, want) <= 1e-4


def test_torch_custom_operator(cuda_device, oracle):
    import torch
    import fusedmm_b200.torch_op  # noqa: F401  (registers torch.ops.fusedmm_b200.csr)
    rng = np.random.default_rng(17)
    m, n, k = 1200, 900, 64
    pntrb, pntre, indx, val = random_csr(rng, m, n, 8, np.int64, np.int32, hub=1800)
    rowptr = as_rowptr(pntrb, pntre)
    val = val.astype(np.float32)
    x, y = np.nan_to_num(dense(rng, m, k, k, np.float32)), np.nan_to_num(dense(rng, n, k, k, np.float32))
    t = {nm: dev(a, cuda_device) for nm, a in dict(rp=rowptr, ix=indx, val=val, x=x, y=y).items()}
    for msg, sop in ((M.MSG_SIGMOID, M.SOP_SIGMOID), (M.MSG_SPMM, 0)):
        want = np.zeros((m, k), np.float32)
        oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k, sop_kind=sop)
        z = torch.ops.fusedmm_b200.csr(t["rp"], t["ix"], t["val"], t["x"], t["y"], msg, sop, 0.0, None)
        s = torch.cuda.Stream()
        torch.cuda.synchronize()
        with torch.cuda.stream(s):
            z2 = torch.ops.fusedmm_b200.csr(t["rp"], t["ix"], t["val"], t["x"], t["y"], msg, sop, 0.0, None)
        s.synchronize()
        assert rel_err(z.cpu().numpy(), want) <= 1e-4 and torch.equal(z, z2)
    with pytest.raises(Exception):
        torch.ops.fusedmm_b200.csr(t["rp"], t["ix"], t["val"], t["x"], t["y"], 0x11F18, 0, 0.0, None)  # unknown VOP


def test_mtx_run_prints_the_testers_csv_line(cuda_device, tmp_path, capsys):
    import io
    from fusedmm_b200 import mtx_run
    rng = np.random.default_rng(23)
    n, e = 3000, 20000
    r, c = rng.integers(1, n + 1, e), rng.integers(1, n + 1, e)
    r[:4000] = 7                                               # one heavy row, so rows get split
    path = tmp_path / "g.mtx"
    with open(path, "w") as f:
        f.write("%%%%MatrixMarket matrix coordinate pattern general\n%d %d %d\n" % (n, n, e))
        f.writelines("%d %d\n" % (a, b) for a, b in zip(r, c))
    for kern in "stfmg":
        out = io.StringIO()
        t0, t1 = mtx_run.run(mtx_run.parse_args(["-input", str(path), "-K", "48", "-nrep", "2", "-T", "1", "-t", kern]),
                             out=out)
        head, line = out.getvalue().strip().split("\n")
        assert head == mtx_run.HEADER
        fields = line.split(",")
        assert fields[0] == str(path) and int(fields[2]) == n and int(fields[4]) == 48 and int(fields[1]) > e
        assert t0 > 0 and t1 > 0 and abs(float(fields[7]) - t0 / t1) < 1e-3 * t0 / t1 + 1e-6
        assert "PASSED TEST" in capsys.readouterr().err
