"""fusedmm_b200_csr_static_scratch: the entry point for callers that may not allocate.

It exists for hosts that cannot call cudaMalloc while they run (a server whose own pool owns all device
memory, a loop that cannot afford the device-wide stalls of the CUDA allocator, a sandbox that may only launch
kernels): the split-row scratch lives in a fixed array inside the library instead.  The check: through the C ABI,
on calls in a row that all need the scratch (graphs with rows long enough to be split), its Z must equal the Z of
the ordinary entry point fusedmm_b200_csr and of the CPU oracle within the tolerance of the parity tests; later
calls also show that what earlier ones left in the shared array does no harm.  Collected last so that
a run that stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from cases import RTOL, dense, random_csr, rel_err
from fusedmm_b200 import api, messages as M

pytestmark = pytest.mark.gpu


def _entry(name):
    fn = getattr(api.lib(), name)
    fn.restype = C.c_int
    fn.argtypes = ([C.c_int32] * 4 + [C.c_int64] * 3 + [C.c_double] + [C.c_int64] * 3 + [C.c_void_p] * 5 +
                   [C.c_int64, C.c_void_p, C.c_int64, C.c_double, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p])
    return fn


def _call(fn, dtype, msg, m, n, k, nnz, t, z, sop_kind, stream=None):
    spec = api.SopSpec(sop_kind, 0, 0.0, 0.0, 0.0)
    return fn(dtype, 64, 32, msg, m, n, k, 1.0, nnz, m, n, t["val"].data_ptr(), t["indx"].data_ptr(),
              t["pntrb"].data_ptr(), t["pntre"].data_ptr(), t["x"].data_ptr(), k, t["y"].data_ptr(), k, 0.0,
              z.data_ptr(), k, C.byref(spec), stream)


# (seed, rows, K, value type, message, SOP, edges of the long row, on a caller's stream?)
CASES = [
    (1, 3000, 128, np.float32, M.MSG_SIGMOID, M.SOP_SIGMOID, 5000, False),
    (2, 1200, 64, np.float64, M.MSG_TDIST, M.SOP_FR, 2100, False),
    (3, 900, 67, np.float32, M.MSG_TDIST, M.SOP_TDIST, 1800, False),            # odd K: the element-strided kernels
    (4, 1500, 128, np.float32, M.MSG_SIGMOID, M.SOP_SIGMOID_TABLE_C, 2600, False),  # the table kept inside the array
    (5, 1500, 32, np.float64, M.MSG_SIGMOID, M.SOP_SIGMOID_TABLE_C, 2600, True),
    (6, 2000, 256, np.float32, M.MSG_SPMM, 0, 3000, True),
]


def test_static_scratch_entry_matches_the_allocating_one_and_the_oracle(cuda_device, oracle):
    """Two rounds over all cases (so every case runs after other calls have left their data in the shared
    array): the Z of the entry point that allocates nothing equals the ordinary entry point's and the CPU
    oracle's within the parity tolerance."""
    import torch
    ordinary, no_alloc = _entry("fusedmm_b200_csr"), _entry("fusedmm_b200_csr_static_scratch")
    stream = torch.cuda.Stream()
    for round_ in range(2):
        for seed, m, k, vt, msg, sop, hub, on_stream in CASES:
            rng = np.random.default_rng(seed)
            n = m
            pntrb, pntre, indx, val = random_csr(rng, m, n, 10, np.int64, np.int32, hub=hub)
            nnz = int((pntre - pntrb).sum())
            host = dict(val=val.astype(vt), indx=indx, pntrb=pntrb, pntre=pntre,
                        x=np.nan_to_num(dense(rng, m, k, k, vt)), y=np.nan_to_num(dense(rng, n, k, k, vt)))
            t = {name: torch.from_numpy(a).to(cuda_device) for name, a in host.items()}
            tdt = torch.float32 if vt == np.float32 else torch.float64
            z_ref = torch.full((m, k), 3.0, dtype=tdt, device=cuda_device)
            z_new = torch.full((m, k), -3.0, dtype=tdt, device=cuda_device)
            torch.cuda.synchronize()
            dt = 0 if vt == np.float32 else 1
            assert _call(ordinary, dt, msg, m, n, k, nnz, t, z_ref, sop) == 0
            assert api.call_info().hub_rows >= 1  # the ordinary call needed its (allocated) scratch too
            if on_stream:
                assert _call(no_alloc, dt, msg, m, n, k, nnz, t, z_new, sop, stream=stream.cuda_stream) == 0
                stream.synchronize()
                assert api.lib().fusedmm_b200_stream_status() == 0
            else:
                assert _call(no_alloc, dt, msg, m, n, k, nnz, t, z_new, sop) == 0
                info = api.call_info()
                assert info.hub_rows >= 1 and info.hub_chunks >= hub // 512
                assert (info.lanes_per_edge == 0) == (k % 4 != 0)
            torch.cuda.synchronize()
            want = np.zeros((m, k), vt)
            assert oracle.csr(msg, m, n, k, host["val"], indx, pntrb, pntre, host["x"], k, host["y"], k, 0.0, want, k,
                              sop_kind=sop) == 0
            # the table sigmoid is a step function of s: a last-bit difference in s can move an edge to the next bin
            tol = 5e-3 if sop == M.SOP_SIGMOID_TABLE_C else RTOL[np.dtype(vt)]
            got = z_new.cpu().numpy()
            assert rel_err(got, z_ref.cpu().numpy()) <= tol, (round_, seed)
            assert rel_err(got, want) <= tol, (round_, seed)


def test_static_scratch_entry_reports_an_understated_nnz_on_a_stream(cuda_device):
    """On a caller's stream nothing is read back by the call; an nnz that understates the graph (so that the
    capacity check up front passes although the split rows do not fit) is reported by fusedmm_b200_stream_status."""
    import torch
    no_alloc = _entry("fusedmm_b200_csr_static_scratch")
    m = n = 40_000
    k = 4
    # every row is longer than the chunk length: 40 000 split rows, more than the 32 768 the array lists
    deg = 520
    rowptr = (np.arange(m + 1, dtype=np.int64) * deg)
    rng = np.random.default_rng(9)
    indx = rng.integers(0, n, size=m * deg, dtype=np.int32)
    host = dict(val=np.ones(m * deg, np.float32), indx=indx, pntrb=rowptr[:-1].copy(), pntre=rowptr[1:].copy(),
                x=rng.random((m, k), dtype=np.float32))
    t = {name: torch.from_numpy(a).to(cuda_device) for name, a in host.items()}
    t["y"] = t["x"]
    z = torch.zeros((m, k), device=cuda_device)
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()
    assert _call(no_alloc, 0, M.MSG_GCN, m, n, k, 1000, t, z, 0, stream=stream.cuda_stream) == 0   # nnz = 1000 is a lie
    stream.synchronize()
    assert api.lib().fusedmm_b200_stream_status() == M.ERR_LIMIT
    assert api.lib().fusedmm_b200_stream_status() == 0   # reported once
    # the synchronous form reports it itself
    assert _call(no_alloc, 0, M.MSG_GCN, m, n, k, 1000, t, z, 0) == M.ERR_LIMIT


def test_static_scratch_entry_refuses_what_it_cannot_hold(cuda_device):
    import torch
    no_alloc = _entry("fusedmm_b200_csr_static_scratch")
    m = n = 64
    k = 128
    rng = np.random.default_rng(3)
    pntrb, pntre, indx, val = random_csr(rng, m, n, 4, np.int64, np.int32)
    host = dict(val=val.astype(np.float32), indx=indx, pntrb=pntrb, pntre=pntre,
                x=np.nan_to_num(dense(rng, m, k, k, np.float32)))
    t = {name: torch.from_numpy(a).to(cuda_device) for name, a in host.items()}
    t["y"] = t["x"]
    z = torch.zeros((m, k), device=cuda_device)
    # an edge count whose worst case does not fit the fixed array: refused up front, Z untouched
    assert _call(no_alloc, 0, M.MSG_SIGMOID, m, n, k, 40_000_000, t, z, M.SOP_SIGMOID) == M.ERR_LIMIT
    assert float(z.abs().sum()) == 0.0
    # a host array would need a staging buffer
    spec = api.SopSpec(M.SOP_SIGMOID, 0, 0.0, 0.0, 0.0)
    zh = np.zeros((m, k), np.float32)
    st = no_alloc(0, 64, 32, M.MSG_SIGMOID, m, n, k, 1.0, 100, m, n, t["val"].data_ptr(), t["indx"].data_ptr(),
                  t["pntrb"].data_ptr(), t["pntre"].data_ptr(), t["x"].data_ptr(), k, t["y"].data_ptr(), k, 0.0,
                  zh.ctypes.data, k, C.byref(spec), None)
    assert st == M.ERR_ARG
