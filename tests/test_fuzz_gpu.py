"""Seeded fuzzing of the C ABI against the CPU oracle: random messages (every valid stage code), shapes down to
one row / one column / no edges at all, padded leading dimensions, all index-width combinations, both value
types, both schedulers, all engines, host and device arrays, beta 0 and 1, the sorted work orders of large graphs
forced on and off."""
import numpy as np
import pytest

from cases import RTOL, dense, random_csr, rel_err, within_tolerance
from fusedmm_b200 import api, messages as M

pytestmark = pytest.mark.gpu

VOPS = [M.VOP_COPY_LHS, M.VOP_COPY_RHS, M.VOP_ADD, M.VOP_SUBL, M.VOP_SUBR, M.VOP_MAX, M.VOP_MIN]
ROPS = [M.ROP_NOOP, M.ROP_DOT, M.ROP_ADD_LHS, M.ROP_ADD_RHS, M.ROP_NORML, M.ROP_NORMR]
SOPS = [M.SOP_NOOP, M.SOP_COPY, M.SOP_UDEF]
VSCS = [M.VSC_NOOP, M.VSC_MUL, M.VSC_ADD]
AOPS = [M.AOP_ADD, M.AOP_MAX, M.AOP_MIN]
OPT = (M.MSG_SIGMOID, M.MSG_TDIST, M.MSG_SPMM, M.MSG_GCN)


def one_case(rng, device, oracle, case):
    import torch
    vt = np.float32 if rng.random() < 0.6 else np.float64
    pt, it = [(np.int32, np.int32), (np.int64, np.int64), (np.int64, np.int32)][rng.integers(3)]
    m = int(rng.choice([1, 2, 7, 33, 150, 600, 2500]))
    n = int(rng.choice([1, 3, 40, 500]))
    k = int(rng.choice([1, 2, 3, 4, 8, 12, 16, 20, 32, 48, 64, 100, 128, 132, 256, 260]))
    pad = int(rng.choice([0, 0, 4, 5]))
    ldx, ldy, ldz = k + pad, k + int(rng.choice([0, 0, 8])), k + int(rng.choice([0, 0, 4, 3]))
    if rng.random() < 0.5:
        msg = int(rng.choice(OPT))
    else:
        msg = int(rng.choice(VOPS)) | int(rng.choice(ROPS)) | int(rng.choice(SOPS)) | int(rng.choice(VSCS)) | int(rng.choice(AOPS))
    sop = int(rng.choice([M.SOP_IDENTITY, M.SOP_SIGMOID, M.SOP_FR, M.SOP_TDIST, M.SOP_TDIST_CLAMPED, M.SOP_LL, M.SOP_FA]))
    hub = int(rng.choice([0, 0, 700, 1300])) or None
    contiguous = rng.random() < 0.5
    pntrb, pntre, indx, val = random_csr(rng, m, n, float(rng.choice([0.0, 1.5, 6.0])), pt, it, hub=hub,
                                         empty_frac=float(rng.choice([0.0, 0.3, 1.0])), gaps=not contiguous)
    val = val.astype(vt)
    # signed inputs for every message; sqrt and log need s >= 0, which only the two norms guarantee
    lo, hi = -0.5, 0.5
    uses_sop = (msg & 0xF00) == M.SOP_UDEF
    if uses_sop and sop in (M.SOP_LL, M.SOP_FA) and (msg & 0xF0) not in (M.ROP_NORML, M.ROP_NORMR):
        lo, hi = 0.1, 1.0
    x = np.nan_to_num(dense(rng, max(m, 1), k, ldx, vt, lo, hi))
    y = np.nan_to_num(dense(rng, n, k, ldy, vt, lo, hi))
    beta = float(rng.choice([0.0, 1.0]))
    z0 = rng.uniform(0.5, 1.5, size=(m, ldz)).astype(vt)
    generic = msg not in OPT
    want = z0.copy()
    st_o = oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, ldx, y, ldy, beta, want, ldz, sop_kind=sop,
                      zero_first=not generic)
    use_stream_engine = contiguous and rng.random() < 0.5
    host = rng.random() < 0.35
    element_vectors = int(rng.random() < 0.6)   # rows that are not 16-byte granular: one-element vectors, or the element-strided engine
    sorts = 2 * (case % 2)   # chunks in column order and whole rows sorted by length: forced on every other case, else off
    api.set_option("engine", 2 if use_stream_engine else 0)
    api.set_option("element_vectors", element_vectors)
    api.set_option("chunk_order", sorts)
    api.set_option("row_bins", sorts)
    try:
        if host:
            z = z0.copy()
            if contiguous:
                rp = np.concatenate([pntrb, pntre[-1:]])
                st = api.fusedMM_csr(msg, m, n, k, 1.0, 0, m, n, val, indx, rp[:-1], rp[1:], x, ldx, y, ldy, beta, z, ldz, sop=sop)
            else:
                st = api.fusedMM_csr(msg, m, n, k, 1.0, 0, m, n, val, indx, pntrb, pntre, x, ldx, y, ldy, beta, z, ldz, sop=sop)
        else:
            t = {nm: torch.from_numpy(a).to(device) for nm, a in dict(val=val, indx=indx, x=x, y=y, z=z0.copy()).items()}
            if contiguous:
                rp = torch.from_numpy(np.concatenate([pntrb, pntre[-1:]])).to(device)
                pb, pe = rp[:-1], rp[1:]
            else:
                pb, pe = torch.from_numpy(pntrb).to(device), torch.from_numpy(pntre).to(device)
            st = api.fusedMM_csr(msg, m, n, k, 1.0, 0, m, n, t["val"], t["indx"], pb, pe, t["x"], ldx, t["y"], ldy, beta,
                                 t["z"], ldz, sop=sop)
            torch.cuda.synchronize()
            z = t["z"].cpu().numpy()
    finally:
        api.set_option("engine", 0)
        api.set_option("element_vectors", 1)
        api.set_option("chunk_order", 1)
        api.set_option("row_bins", 1)
    tag = (case, hex(msg), m, n, k, (ldx, ldy, ldz), vt.__name__, pt.__name__, it.__name__, sop, beta, hub, contiguous,
           use_stream_engine, host, sorts)
    assert st == st_o == 0, tag
    assert np.array_equal(z[:, k:], z0[:, k:]), tag   # padding columns untouched
    if np.isfinite(want[:, :k]).all():
        info = api.call_info()

        def exact():  # the same inputs evaluated one precision up
            if vt == np.float32:
                ex = z0.astype(np.float64)
                oracle.csr(msg, m, n, k, val.astype(np.float64), indx, pntrb, pntre, x.astype(np.float64), ldx,
                           y.astype(np.float64), ldy, beta, ex, ldz, sop_kind=sop, zero_first=not generic)
                return ex
            from oracle.cpu import numpy_fusedmm
            start = z0 if generic or beta != 0.0 else np.zeros_like(z0)
            return numpy_fusedmm(msg, m, k, val, indx, pntrb, pntre, x, y, start, sop_kind=sop, dtype=np.longdouble)

        ok, e, e_gpu, e_or = within_tolerance(z, want, RTOL[np.dtype(vt)], exact, k)
        assert ok, (tag, e, e_gpu, e_or)
        w = 16 // np.dtype(vt).itemsize
        granular = k % w == 0 and ldx % w == 0 and ldy % w == 0 and ldz % w == 0
        return 1, int(info.engine == 2), int(info.lanes_per_edge == 0), int(info.lanes_per_edge > 0 and not granular)
    return 0, 0, 0, 0


@pytest.mark.parametrize("seed", [20240607, 7, 99])
def test_fuzz_against_the_oracle(cuda_device, oracle, seed):
    rng = np.random.default_rng(seed)
    compared = stream = strided = element = 0
    for case in range(1500):
        c, s, a, e = one_case(rng, cuda_device, oracle, case)
        compared, stream, strided, element = compared + c, stream + s, strided + a, element + e
    # nearly every case has a finite reference result, and all engines were exercised many times
    assert compared >= 1350 and stream >= 100 and strided >= 150 and element >= 150, (compared, stream, strided, element)
