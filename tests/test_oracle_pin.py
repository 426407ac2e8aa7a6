"""Pins the CPU oracle (oracle/fusedmm_oracle.c) before anything else trusts it:
  * bit-for-bit against outputs of the reference's own fusedMM_csr stored in tests/golden/;
  * bit-for-bit against the reference itself where oracle/_ref is built;
  * within rounding of an independent float64 NumPy restatement.
"""
from pathlib import Path

import numpy as np
import pytest

from cases import MESSAGES, RTOL, dense, random_csr, rel_err
from fusedmm_b200 import messages as M
from oracle.cpu import numpy_fusedmm

GOLDEN = Path(__file__).parent / "golden" / "reference_general_kernel.npz"


def golden_cases():
    data = np.load(GOLDEN)
    keys = sorted({k.split("_")[0] for k in data.files})
    for key in keys:
        yield key, data


def test_golden_file_has_all_messages():
    data = np.load(GOLDEN)
    names = {str(data[k]) for k in data.files if k.endswith("_name")}
    assert names == set(MESSAGES)


def test_oracle_equals_golden_bit_for_bit(oracle):
    n_cases = 0
    for key, data in golden_cases():
        msg, m, n, k, ld, sop = (int(v) for v in data[key + "_meta"])
        z = np.zeros_like(data[key + "_z"])
        st = oracle.csr(msg, m, n, k, data[key + "_val"], data[key + "_indx"], data[key + "_pntrb"],
                        data[key + "_pntre"], data[key + "_x"], ld, data[key + "_y"], ld, 0.0, z, ld,
                        sop_kind=sop, zero_first=False)
        assert st == 0
        assert np.array_equal(z, data[key + "_z"]), f"case {key} ({data[key + '_name']})"
        n_cases += 1
    assert n_cases == 44


@pytest.mark.parametrize("vt", [np.float32, np.float64])
@pytest.mark.parametrize("it", [np.int32, np.int64])
def test_oracle_equals_reference_bit_for_bit(oracle, reference, vt, it):
    reference.threads(3)  # the reference's row partition must not change the result
    for case, (name, msg) in enumerate(MESSAGES.items()):
        rng = np.random.default_rng(77 + case)
        m, n, k = 101, 83, 36
        pntrb, pntre, indx, val = random_csr(rng, m, n, 7, it, it, hub=300)
        val = val.astype(vt)
        x, y = np.nan_to_num(dense(rng, m, k, k, vt)), np.nan_to_num(dense(rng, n, k, k, vt))
        for sop in (M.SOP_SIGMOID, M.SOP_FR, M.SOP_SIGMOID_TABLE_C, M.SOP_TDIST_CLAMPED):
            z0 = rng.uniform(-1, 1, size=(m, k)).astype(vt)  # the general kernel accumulates into Z
            zr, zo = z0.copy(), z0.copy()
            assert reference.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 1.0, zr, k, sop_kind=sop) == 0
            assert oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 1.0, zo, k, sop_kind=sop,
                              zero_first=False) == 0
            assert np.array_equal(zr, zo, equal_nan=True), (name, sop)


def test_oracle_status_codes_match_reference(oracle, reference):
    rng = np.random.default_rng(5)
    pntrb, pntre, indx, val = random_csr(rng, 4, 4, 2, np.int64, np.int64)
    val = val.astype(np.float32)
    x = np.zeros((4, 8), np.float32)
    for msg in (0x11F10, 0x11F18, 0x11F62, 0x11212, 0x13F12, 0x41F12, 0x11F12):
        z1, z2 = np.zeros((4, 8), np.float32), np.zeros((4, 8), np.float32)
        a = reference.csr(msg, 4, 4, 8, val, indx, pntrb, pntre, x, 8, x, 8, 0.0, z1, 8)
        b = oracle.csr(msg, 4, 4, 8, val, indx, pntrb, pntre, x, 8, x, 8, 0.0, z2, 8, zero_first=False)
        assert a == b, hex(msg)


@pytest.mark.parametrize("name", list(MESSAGES))
def test_oracle_close_to_numpy_float64(oracle, name):
    msg = MESSAGES[name]
    rng = np.random.default_rng(hash(name) % 1000)
    m, n, k = 23, 19, 12
    pntrb, pntre, indx, val = random_csr(rng, m, n, 4, np.int32, np.int32)
    for vt in (np.float32, np.float64):
        x, y = np.nan_to_num(dense(rng, m, k, k, vt)), np.nan_to_num(dense(rng, n, k, k, vt))
        sop = M.SOP_FR if "norm" in name or name == "tdist" else M.SOP_SIGMOID
        z = np.zeros((m, k), vt)
        assert oracle.csr(msg, m, n, k, val.astype(vt), indx, pntrb, pntre, x, k, y, k, 0.0, z, k,
                          sop_kind=sop, zero_first=False) == 0
        want = numpy_fusedmm(msg, m, k, val.astype(vt), indx, pntrb, pntre, x, y, np.zeros((m, k)), sop)
        assert rel_err(z, want) <= (2e-5 if vt == np.float32 else 1e-12), name


def test_oracle_sop_bodies(oracle):
    # closed forms of test/fusedMMtime.cpp:625-674
    for s in (-6.0, -2.5, -0.1, 0.2, 1.0, 3.3, 7.0):
        assert oracle.sop(s, M.SOP_SIGMOID) == pytest.approx(1 / (1 + np.exp(-s)), rel=1e-6)
        assert abs(oracle.sop(s, M.SOP_SIGMOID_TABLE_C) - (1 - 1 / (1 + np.exp(-s)))) < 3e-3
        assert oracle.sop(s, M.SOP_TDIST_CLAMPED) == pytest.approx(np.clip(-2 / (1 + s), -5, 5), rel=1e-6)
    assert oracle.sop(4.0, M.SOP_FR) == pytest.approx(1.25)
    assert oracle.sop(4.0, M.SOP_TDIST) == pytest.approx(0.2)
    assert oracle.sop(4.0, M.SOP_LL) == pytest.approx(np.log2(3.0), rel=1e-6)
    assert oracle.sop(4.0, M.SOP_FA) == pytest.approx(2.25)
    assert oracle.sop(1.0, M.SOP_AFFINE_RECIP, (3.0, 2.0, 0.5)) == pytest.approx(0.5)
    assert oracle.sop(6.0, M.SOP_SIGMOID_TABLE_C) == 0.0 and oracle.sop(-6.0, M.SOP_SIGMOID_TABLE_C) == 1.0


def test_zero_first_matches_optimised_kernel_semantics(oracle):
    # beta == 0 overwrites Z, rows without edges become 0 (kernels/codegen/genkern.base:287-295)
    rng = np.random.default_rng(3)
    m, n, k = 9, 9, 8
    pntrb, pntre, indx, val = random_csr(rng, m, n, 3, np.int64, np.int64, empty_frac=0.4)
    x = np.nan_to_num(dense(rng, m, k, k, np.float32))
    z = np.full((m, k), 7.0, np.float32)
    oracle.csr(M.MSG_GCN, m, n, k, val.astype(np.float32), indx, pntrb, pntre, x, k, x, k, 0.0, z, k)
    empty = (pntre - pntrb) == 0
    assert empty.any() and (z[empty] == 0).all()
    z2 = np.zeros((m, k), np.float32)
    oracle.csr(M.MSG_GCN, m, n, k, val.astype(np.float32), indx, pntrb, pntre, x, k, x, k, 0.0, z2, k,
               zero_first=False)
    assert np.array_equal(z, z2)


@pytest.mark.parametrize("vt", [np.float32, np.float64])
def test_optimised_reference_build_agrees_with_the_oracle(oracle, vt):
    """The timed CPU baseline (the reference's generated OpenMP kernels, oracle/build_ref_opt.sh) computes what the
    oracle computes: the four optimised messages within the tolerance the GPU is held to (the vector kernels sum in
    another order than the general kernel), beta = 0 overwriting Z and beta = 1 accumulating, and a message without
    an optimised kernel falling through to the general kernel bit for bit."""
    from oracle.cpu import ReferenceOpt, reference_opt_available
    if not reference_opt_available():
        pytest.skip("oracle/_ref holds no optimised reference build (needs the reference sources; run oracle/build_ref_opt.sh)")
    opt = ReferenceOpt()
    opt.threads(3)
    rng = np.random.default_rng(5)
    m, n = 700, 600
    pntrb, pntre, indx, val = random_csr(rng, m, n, 8, np.int64, np.int64, hub=900)
    val = val.astype(vt)
    for k in (opt.vlen(vt), 64, 128, 512 + 2 * opt.vlen(vt)):   # one vector, unrolled kernels, beyond bestK (rolled tail)
        x, y = np.nan_to_num(dense(rng, m, k, k, vt)), np.nan_to_num(dense(rng, n, k, k, vt))
        for msg, sop in ((M.MSG_SIGMOID, M.SOP_SIGMOID), (M.MSG_TDIST, M.SOP_FR), (M.MSG_TDIST, M.SOP_TDIST),
                         (M.MSG_SPMM, 0), (M.MSG_GCN, 0)):
            for beta in (0.0, 1.0):
                if beta == 0.0 and k > 512:
                    continue  # the reference's rolled tail accumulates onto stale Z when beta == 0 (genkern.base:392-393)
                z0 = rng.uniform(-1, 1, size=(m, k)).astype(vt)
                want, got = z0.copy(), z0.copy()
                assert oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, beta, want, k, sop_kind=sop,
                                  zero_first=(beta == 0.0)) == 0
                assert opt.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, beta, got, k, sop_kind=sop) == 0
                assert rel_err(got, want) <= RTOL[np.dtype(vt)], (hex(msg), k, beta)
    k = 32
    x, y = np.nan_to_num(dense(rng, m, k, k, vt)), np.nan_to_num(dense(rng, n, k, k, vt))
    msg = MESSAGES["add_addrhs_vscadd_add"]
    z0 = rng.uniform(-1, 1, size=(m, k)).astype(vt)
    got = z0.copy()
    assert opt.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, got, k) == 0
    gen = z0.copy()
    assert opt.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, gen, k, general=True) == 0
    assert np.array_equal(got, gen)
    want = z0.copy()
    assert oracle.csr(msg, m, n, k, val, indx, pntrb, pntre, x, k, y, k, 0.0, want, k, zero_first=False) == 0
    assert rel_err(got, want) <= RTOL[np.dtype(vt)]
