"""MatrixMarket ingest (fusedmm_b200.mtx): symmetrised, self-loops dropped, duplicates removed, sorted rows --
what the reference's reader does to its inputs (test/include/IO.h:62-162)."""
import numpy as np
import pytest

from fusedmm_b200.mtx import read_mtx


def test_general_real_file(tmp_path):
    p = tmp_path / "g.mtx"
    p.write_text("%%MatrixMarket matrix coordinate real general\n% a comment\n5 5 7\n"
                 "1 2 0.5\n2 1 0.25\n3 3 9.0\n4 1 2.0\n1 4 7.0\n5 2 1.5\n1 2 4.0\n")
    csr = read_mtx(p)
    rp, ix, vl = csr.rowptr.numpy(), csr.indx.numpy(), csr.val.numpy()
    assert csr.n == 5 and list(rp) == [0, 2, 4, 4, 5, 6]
    assert list(ix) == [1, 3, 0, 4, 0, 1]            # (0,1) (0,3) | (1,0) (1,4) | - | (3,0) | (4,1)
    assert np.allclose(vl, [0.5, 7.0, 0.25, 1.5, 2.0, 1.5])   # first occurrence in file order wins; (3,3) dropped
    dense = np.zeros((5, 5))
    for r in range(5):
        dense[r, ix[rp[r]:rp[r + 1]]] = 1
    assert (dense == dense.T).all() and np.trace(dense) == 0


def test_pattern_symmetric_file_and_errors(tmp_path):
    p = tmp_path / "p.mtx"
    p.write_text("%%MatrixMarket matrix coordinate pattern symmetric\n4 4 3\n2 1\n3 1\n4 3\n")
    csr = read_mtx(p, symmetrize=False)  # the file's own symmetry still expands it
    assert csr.nnz == 6 and np.allclose(csr.val.numpy(), 1.0) and list(csr.rowptr.numpy()) == [0, 2, 3, 5, 6]
    bad = tmp_path / "b.mtx"
    bad.write_text("%%MatrixMarket matrix array real general\n2 2\n1\n2\n3\n4\n")
    with pytest.raises(ValueError):
        read_mtx(bad)
    short = tmp_path / "s.mtx"
    short.write_text("%%MatrixMarket matrix coordinate real general\n3 3 2\n1 2 1.0\n")
    with pytest.raises(ValueError):
        read_mtx(short)


def test_mtx_run_command_line_matches_the_reference_tester_flags():
    from fusedmm_b200 import mtx_run
    a = mtx_run.parse_args(["-input", "g.mtx", "-K", "64", "-nrep", "3", "-skHd", "1", "-t", "s", "-C", "1024"])
    assert (a.input, a.K, a.nrep, a.skHd, a.t, a.T) == ("g.mtx", 64, 3, 1, "s", 0)
    assert mtx_run.HEADER.split(",")[:5] == ["Filename", "NNZ", "M", "N", "K"]
    assert set(mtx_run.KERNELS) == {"s", "t", "f", "m", "g"}
