"""fusedmm_b200_csr_static_scratch: the entry point for callers that may not allocate.

It exists for hosts that cannot call cudaMalloc while they run (a server whose own pool owns all device
memory, a loop that cannot afford the device-wide stalls of the CUDA allocator, a sandbox that may only launch
kernels): the split-row scratch lives in a fixed array inside the library instead.  The check is simple: through
the C ABI, on two calls in a row that both need the scratch (graphs with rows long enough to be split), its Z
must equal the Z of the ordinary entry point fusedmm_b200_csr within the tolerance of the parity tests; the
second call also shows that what the first one left in the shared array does no harm.  Collected last so that
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


def _call(fn, dtype, msg, m, n, k, nnz, t, z, sop_kind):
    spec = api.SopSpec(sop_kind, 0, 0.0, 0.0, 0.0)
    return fn(dtype, 64, 32, msg, m, n, k, 1.0, nnz, m, n, t["val"].data_ptr(), t["indx"].data_ptr(),
              t["pntrb"].data_ptr(), t["pntre"].data_ptr(), t["x"].data_ptr(), k, t["y"].data_ptr(), k, 0.0,
              z.data_ptr(), k, C.byref(spec), None)


def test_static_scratch_entry_matches_the_allocating_one(cuda_device):
    import torch
    ordinary, no_alloc = _entry("fusedmm_b200_csr"), _entry("fusedmm_b200_csr_static_scratch")
    cases = [  # (seed, rows, K, value type, message, SOP, edges of the long row)
        (1, 3000, 128, np.float32, M.MSG_SIGMOID, M.SOP_SIGMOID, 5000),
        (2, 1200, 64, np.float64, M.MSG_TDIST, M.SOP_FR, 2100),
    ]
    for seed, m, k, vt, msg, sop, hub in cases:
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
        assert _call(no_alloc, dt, msg, m, n, k, nnz, t, z_new, sop) == 0
        info = api.call_info()
        assert info.hub_rows >= 1 and info.hub_chunks >= hub // 512
        torch.cuda.synchronize()
        assert rel_err(z_new.cpu().numpy(), z_ref.cpu().numpy()) <= RTOL[np.dtype(vt)]


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
