"""Small seeded inputs shared by the CPU and GPU tests (NumPy only)."""
import numpy as np

from fusedmm_b200 import messages as M

# every message the tests run: the reference's four optimised patterns first, then generic 5-tuples
# that between them use every VOP, ROP, VSC and AOP code
MESSAGES = {
    "sigmoid": M.MSG_SIGMOID,
    "tdist": M.MSG_TDIST,
    "spmm": M.MSG_SPMM,
    "gcn": M.MSG_GCN,
    "copylhs_addlhs_mul_add": M.VOP_COPY_LHS | M.ROP_ADD_LHS | M.SOP_COPY | M.VSC_MUL | M.AOP_ADD,
    "add_addrhs_vscadd_add": M.VOP_ADD | M.ROP_ADD_RHS | M.SOP_COPY | M.VSC_ADD | M.AOP_ADD,
    "subl_norml_udef_mul_max": M.VOP_SUBL | M.ROP_NORML | M.SOP_UDEF | M.VSC_MUL | M.AOP_MAX,
    "max_dot_copy_mul_min": M.VOP_MAX | M.ROP_DOT | M.SOP_COPY | M.VSC_MUL | M.AOP_MIN,
    "min_noop_copy_vscadd_max": M.VOP_MIN | M.ROP_NOOP | M.SOP_COPY | M.VSC_ADD | M.AOP_MAX,
    "subr_normr_noopsop_noopvsc_add": M.VOP_SUBR | M.ROP_NORMR | M.SOP_NOOP | M.VSC_NOOP | M.AOP_ADD,
    "copyrhs_dot_udef_mul_add_fr": M.VOP_COPY_RHS | M.ROP_DOT | M.SOP_UDEF | M.VSC_MUL | M.AOP_ADD,
}


def random_csr(rng, m, n, avg_deg, ptr_dtype=np.int64, idx_dtype=np.int64, hub=None, empty_frac=0.2,
               gaps=False):
    """Random CSR with empty rows, optionally one long row (`hub` edges) and unused slots between rows
    (pntre[i] < pntrb[i+1]), which the four-array form allows (fusedMM.h:86-87)."""
    degs = rng.poisson(avg_deg, size=m)
    degs[rng.random(m) < empty_frac] = 0
    if hub is not None and m > 2:
        degs[m // 3] = hub
    pad = rng.integers(0, 3, size=m) if gaps else np.zeros(m, dtype=np.int64)
    starts = np.zeros(m, dtype=np.int64)
    pos = 0
    for i in range(m):
        starts[i] = pos
        pos += int(degs[i]) + int(pad[i])
    total = max(pos, 1)
    indx = rng.integers(0, n, size=total).astype(idx_dtype)
    for i in range(m):  # no self-loops: with X = Y they give a zero distance, and 1/0 in the FR / t-dist SOPs
        seg = indx[starts[i]:starts[i] + degs[i]]
        seg[seg == i] = (i + 1) % n
    val = rng.uniform(0.25, 1.5, size=total)
    pntrb = starts.astype(ptr_dtype)
    pntre = (starts + degs).astype(ptr_dtype)
    return pntrb, pntre, indx, val


def dense(rng, rows, k, ld, dtype, lo=-0.5, hi=0.5):
    a = np.full((rows, ld), np.nan, dtype=dtype)  # padding columns must never be read or written
    a[:, :k] = rng.uniform(lo, hi, size=(rows, k)).astype(dtype)
    return a


def rel_err(z, zref, k=None):
    """max |z - zref| / max(|zref|, row-wise max |zref|, tiny): the metric the tolerances are stated in.
    Element-wise relative error is not usable: the reference's own two code paths differ by more than
    1e-4 on near-cancelling elements while agreeing to 1e-6 in this metric."""
    z = np.asarray(z, dtype=np.float64)
    zref = np.asarray(zref, dtype=np.float64)
    if k is not None:
        z, zref = z[:, :k], zref[:, :k]
    if not np.isfinite(z).all() or not np.isfinite(zref).all():
        return np.inf
    scale = np.maximum(np.abs(zref), np.abs(zref).max(axis=1, keepdims=True))
    scale = np.maximum(scale, 1e-30)
    return float((np.abs(z - zref) / scale).max()) if z.size else 0.0


RTOL = {np.dtype(np.float32): 1e-4, np.dtype(np.float64): 1e-10}


def within_tolerance(z, want, tol, exact_fn, k=None, slack=4.0):
    """Acceptance of a GPU result `z` against the oracle's `want` (same precision).  Passes when they agree within
    `tol` in the metric of rel_err.  Messages that feed a cancelling reduction into a product or a reciprocal
    (signed inputs, s near 0 or near a pole of the scalar function) amplify the rounding of s in the oracle as much
    as in the GPU kernel; for those the arbiter is a higher-precision evaluation of the same inputs, `exact_fn()`
    (called only when needed): the GPU result must be no further from it than `slack` times the oracle is, or
    `tol`.  Returns (ok, error vs the oracle, error vs exact or None, the oracle's error vs exact or None)."""
    e = rel_err(z, want, k)
    if e <= tol:
        return True, e, None, None
    exact = exact_fn()
    e_gpu, e_or = rel_err(z, exact, k), rel_err(want, exact, k)
    return e_gpu <= max(tol, slack * e_or), e, e_gpu, e_or
