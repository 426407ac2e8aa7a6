"""MatrixMarket ingest: a coordinate ``.mtx`` file -> the CSR arrays ``fusedMM_csr`` takes.

Follows what the reference's tester does to its inputs (``test/include/IO.h:62-162``: the graph is made
symmetric, self-loops are dropped; ``CSC.h:147-190`` / ``CSR.h:154-186``: entries sorted by row and column), plus
removal of duplicate entries.  Values: ``pattern`` files get 1.0; for symmetrised duplicates the first value in
file order wins.  The reference parses values with ``atoi`` and its tester then overwrites them with random numbers
(``IO.h:118``, ``fusedMMtime.cpp:948-951``), so no caller of the reference depends on them.
"""
from __future__ import annotations

import numpy as np

from .synth import CSR


def read_mtx(path, symmetrize: bool = True, drop_self_loops: bool = True, ptr_dtype=np.int64, idx_dtype=np.int32,
             val_dtype=np.float32):
    """Returns a :class:`fusedmm_b200.synth.CSR` of CPU torch tensors (square: max(rows, cols) vertices)."""
    import torch
    with open(path, "r") as f:
        header = f.readline().strip().lower().split()
        if len(header) < 5 or header[0] != "%%matrixmarket" or header[1] != "matrix" or header[2] != "coordinate":
            raise ValueError(f"{path}: only MatrixMarket coordinate matrices are supported")
        field, symmetry = header[3], header[4]
        line = f.readline()
        while line.startswith("%") or not line.strip():
            line = f.readline()
        rows, cols, entries = (int(t) for t in line.split()[:3])
        data = np.loadtxt(f, ndmin=2) if entries else np.zeros((0, 3))
    if data.shape[0] != entries:
        raise ValueError(f"{path}: header announces {entries} entries, file has {data.shape[0]}")
    r = data[:, 0].astype(np.int64) - 1
    c = data[:, 1].astype(np.int64) - 1
    v = data[:, 2].astype(np.float64) if (field != "pattern" and data.shape[1] > 2) else np.ones(entries)
    n = max(rows, cols)
    if drop_self_loops:
        keep = r != c
        r, c, v = r[keep], c[keep], v[keep]
    if symmetrize or symmetry in ("symmetric", "skew-symmetric", "hermitian"):
        r, c, v = np.concatenate([r, c]), np.concatenate([c, r]), np.concatenate([v, v])
    key = r * n + c
    _, first = np.unique(key, return_index=True)  # sorted by (row, col); first occurrence of a duplicate wins
    r, c, v = r[first], c[first], v[first]
    rowptr = np.zeros(n + 1, dtype=np.int64)
    np.add.at(rowptr, r + 1, 1)
    rowptr = np.cumsum(rowptr)
    return CSR(n, torch.from_numpy(rowptr.astype(ptr_dtype)), torch.from_numpy(c.astype(idx_dtype)),
               torch.from_numpy(v.astype(val_dtype)))
