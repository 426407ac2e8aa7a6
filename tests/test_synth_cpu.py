"""The seeded generators: deterministic, independent of chunking, and with the clean-up the configurations
describe (symmetrised, deduplicated, no self-loops, columns sorted within a row)."""
import numpy as np
import torch

from fusedmm_b200 import messages as M, synth


def test_rmat_is_deterministic_and_chunk_independent():
    a = synth.rmat_edges(10, 16, seed=5)
    b = synth.rmat_edges(10, 16, seed=5, chunk=1000)
    c = synth.rmat_edges(10, 16, seed=6)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    assert not torch.equal(a[0], c[0])
    assert a[0].numel() == 16 << 10 and int(a[0].max()) < 1 << 10 and int(a[0].min()) >= 0
    # the skew of R-MAT(0.57, 0.19, 0.19): low vertex ids are far more frequent than high ones
    assert (a[0] < 512).float().mean() > 0.7


def test_csr_cleanup():
    src, dst = synth.rmat_edges(9, 8, seed=3)
    csr = synth.build_csr(src, dst, 1 << 9)
    rp, ix = csr.rowptr.numpy(), csr.indx.numpy()
    assert rp[0] == 0 and rp[-1] == csr.nnz and (np.diff(rp) >= 0).all()
    dense = np.zeros((512, 512), np.int32)
    for r in range(512):
        cols = ix[rp[r]:rp[r + 1]]
        assert (np.diff(cols) > 0).all()          # sorted, no duplicates
        assert not (cols == r).any()              # no self-loops
        dense[r, cols] = 1
    assert (dense == dense.T).all()               # symmetric
    inv = synth.build_csr(src, dst, 1 << 9, values="inv_degree")
    deg = np.diff(rp)
    row_of = np.repeat(np.arange(512), deg)
    assert np.allclose(inv.val.numpy(), 1.0 / deg[row_of])


def test_dense_generators_and_configs():
    u = synth.dense_uniform(100, 8, -0.5, 0.5, seed=1)
    v = synth.dense_uniform(100, 8, -0.5, 0.5, seed=1, chunk_rows=7)
    assert torch.equal(u, v) and float(u.min()) >= -0.5 and float(u.max()) < 0.5
    g = synth.dense_normal(4000, 8, 0.1, seed=2)
    assert abs(float(g.std()) - 0.1) < 0.005 and abs(float(g.mean())) < 0.005
    cfg, csr, x = synth.make_config("c3_tdist_er4m_k64", scale=10)
    assert cfg["msg"] == M.MSG_TDIST and x.shape == (1024, 64) and 6 < csr.nnz / 1024 < 9
    assert set(synth.CONFIGS) == {"c1_sigmoid_rmat14_k128", "c2_fr_rmat20_k256", "c3_tdist_er4m_k64",
                                  "c4_spmm_rmat22_k512", "c5_sigmoid_rmat24_k128"}


def test_algorithmic_bytes_formula():
    # nnz*(K*4 + 4) + m*(2*K*4 + 16) for a message that reads X and writes Z
    assert synth.algorithmic_bytes(M.MSG_SIGMOID, 10, 3, 8, 4, 4, 8) == 10 * 36 + 3 * (64 + 16)
    assert synth.algorithmic_bytes(M.MSG_SPMM, 10, 3, 8, 4, 4, 8) == 10 * 40 + 3 * (32 + 16)
    assert synth.algorithmic_bytes(M.MSG_GCN, 10, 3, 8, 4, 4, 8, beta_nonzero=True) == 10 * 36 + 3 * (64 + 16)
