"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

The graphs the reference's scripts name (``runtime.sh:42-43``, ``README.md:35``) are not available, so
R-MAT and Erdos-Renyi graphs stand in for them.  Everything is a pure function of (seed, index) through a
counter-based 64-bit hash evaluated with integer tensor ops, so the same call gives bit-identical graphs
and uniform matrices on the CPU and on a GPU, in any chunking.

Clean-up of the edge list follows what the reference's MatrixMarket reader does to its inputs
(``test/include/IO.h:62-162``): self-loops dropped, both directions stored, duplicates removed; columns
are sorted within a row.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

_M1 = 0xBF58476D1CE4E5B9 - (1 << 64)
_M2 = 0x94D049BB133111EB - (1 << 64)
_GOLD = 0x9E3779B97F4A7C15 - (1 << 64)


def _lsr(z, s):
    return (z >> s) & ((1 << (64 - s)) - 1)


def hash64(counter: torch.Tensor, seed: int) -> torch.Tensor:
    """splitmix64 finaliser of ``counter + seed * golden`` (int64 tensors, wrap-around arithmetic)."""
    mask = (1 << 64) - 1
    s = (seed * 0x9E3779B97F4A7C15 + 0x632BE59BD9B4E019) & mask
    s = s - (1 << 64) if s >= (1 << 63) else s
    z = counter * _GOLD + s
    z = (z ^ _lsr(z, 30)) * _M1
    z = (z ^ _lsr(z, 27)) * _M2
    return z ^ _lsr(z, 31)


def uniform01(counter: torch.Tensor, seed: int) -> torch.Tensor:
    """24-bit uniform in [0, 1) as float32 (exact, identical on every device)."""
    return _lsr(hash64(counter, seed), 40).to(torch.float32) * (1.0 / (1 << 24))


def rmat_edges(scale: int, edge_factor: int, seed: int, a=0.57, b=0.19, c=0.19, device="cpu",
               chunk: int = 1 << 24):
    """Raw R-MAT edge list: ``edge_factor * 2**scale`` (src, dst) pairs, one quadrant draw per level."""
    n_edges = edge_factor << scale
    ta, tb, tc = (int(round(v * (1 << 24))) for v in (a, a + b, a + b + c))
    srcs, dsts = [], []
    for e0 in range(0, n_edges, chunk):
        e = torch.arange(e0, min(e0 + chunk, n_edges), dtype=torch.int64, device=device)
        src = torch.zeros_like(e)
        dst = torch.zeros_like(e)
        for lvl in range(scale):
            r = _lsr(hash64(e * scale + lvl, seed), 40)  # 24-bit integer draw
            # quadrants: [0,a) -> (0,0); [a,a+b) -> (0,1); [a+b,a+b+c) -> (1,0); rest -> (1,1)
            sb = (r >= tb).to(torch.int64)
            db = (((r >= ta) & (r < tb)) | (r >= tc)).to(torch.int64)
            src = (src << 1) | sb
            dst = (dst << 1) | db
        srcs.append(src)
        dsts.append(dst)
    return torch.cat(srcs), torch.cat(dsts)


def er_edges(n: int, avg_degree: int, seed: int, device="cpu", chunk: int = 1 << 24):
    """``n * avg_degree / 2`` uniform vertex pairs (average directed degree ~ avg_degree after symmetrising)."""
    n_edges = n * avg_degree // 2
    srcs, dsts = [], []
    for e0 in range(0, n_edges, chunk):
        e = torch.arange(e0, min(e0 + chunk, n_edges), dtype=torch.int64, device=device)
        srcs.append(_lsr(hash64(2 * e, seed), 1) % n)
        dsts.append(_lsr(hash64(2 * e + 1, seed), 1) % n)
    return torch.cat(srcs), torch.cat(dsts)


@dataclass
class CSR:
    """Zero-based CSR in the four-array form ``fusedMM_csr`` takes (``pntrb = rowptr[:-1]``, ``pntre = rowptr[1:]``)."""
    n: int
    rowptr: torch.Tensor   # n+1 entries
    indx: torch.Tensor     # column ids, sorted within each row
    val: torch.Tensor      # edge values

    @property
    def nnz(self) -> int:
        return int(self.indx.numel())

    @property
    def pntrb(self):
        return self.rowptr[:-1]

    @property
    def pntre(self):
        return self.rowptr[1:]

    def degrees(self):
        return self.rowptr[1:] - self.rowptr[:-1]


def build_csr(src, dst, n, ptr_dtype=torch.int64, idx_dtype=torch.int32, val_dtype=torch.float32,
              values="ones") -> CSR:
    """Symmetrise, drop self-loops, deduplicate, sort by (row, col).  ``values``: "ones" or "inv_degree"."""
    keep = src != dst
    src, dst = src[keep], dst[keep]
    key = torch.cat([src * n + dst, dst * n + src])
    del src, dst
    key = torch.unique(key)  # sorted
    rows = torch.div(key, n, rounding_mode="floor")
    cols = key - rows * n
    del key
    deg = torch.bincount(rows, minlength=n)
    rowptr = torch.zeros(n + 1, dtype=torch.int64, device=cols.device)
    torch.cumsum(deg, 0, out=rowptr[1:])
    if values == "ones":
        val = torch.ones(cols.numel(), dtype=val_dtype, device=cols.device)
    elif values == "inv_degree":
        val = (1.0 / deg.to(torch.float64))[rows].to(val_dtype)
    else:
        raise ValueError(values)
    del rows
    return CSR(n, rowptr.to(ptr_dtype), cols.to(idx_dtype), val)


def dense_uniform(n, k, lo, hi, seed, device="cpu", dtype=torch.float32, chunk_rows: int = 1 << 18):
    """n x k matrix of lo + (hi-lo)*u, u a 24-bit uniform of (seed, element index)."""
    out = torch.empty((n, k), dtype=dtype, device=device)
    for r0 in range(0, n, chunk_rows):
        r1 = min(n, r0 + chunk_rows)
        ctr = torch.arange(r0 * k, r1 * k, dtype=torch.int64, device=device)
        u = uniform01(ctr, seed).to(dtype)
        out[r0:r1] = (lo + (hi - lo) * u).view(r1 - r0, k)
    return out


def dense_normal(n, k, std, seed, device="cpu", dtype=torch.float32, chunk_rows: int = 1 << 18):
    """n x k matrix of N(0, std) by Box-Muller over two hashed uniforms (last-bit differences between
    devices are possible because log/cos are library functions)."""
    out = torch.empty((n, k), dtype=dtype, device=device)
    for r0 in range(0, n, chunk_rows):
        r1 = min(n, r0 + chunk_rows)
        ctr = torch.arange(r0 * k, r1 * k, dtype=torch.int64, device=device)
        u1 = (uniform01(2 * ctr, seed).to(torch.float64) + 2.0 ** -25)
        u2 = uniform01(2 * ctr + 1, seed).to(torch.float64)
        g = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(2.0 * math.pi * u2)
        out[r0:r1] = (std * g).to(dtype).view(r1 - r0, k)
    return out


# ---------------------------------------------------------------------------------------------------
# The benchmark configurations.  name -> (graph, message, SOP kind, K, dense distribution, value type)
# ---------------------------------------------------------------------------------------------------
from . import messages as M  # noqa: E402

CONFIGS = {
    # sigmoid / Force2Vec on R-MAT scale 14, K=128
    "c1_sigmoid_rmat14_k128": dict(graph=("rmat", 14, 16), msg=M.MSG_SIGMOID, sop=M.SOP_SIGMOID, k=128,
                                   dense=("uniform", -0.5, 0.5), values="ones", seed=43),
    # Fruchterman-Reingold on R-MAT scale 20, K=256
    "c2_fr_rmat20_k256": dict(graph=("rmat", 20, 16), msg=M.MSG_TDIST, sop=M.SOP_FR, k=256,
                              dense=("uniform", -1.0, 1.0), values="ones", seed=44),
    # t-distribution on Erdos-Renyi, 4M vertices, average degree 8, K=64
    "c3_tdist_er4m_k64": dict(graph=("er", 1 << 22, 8), msg=M.MSG_TDIST, sop=M.SOP_TDIST, k=64,
                              dense=("normal", 0.1), values="ones", seed=45),
    # GCN aggregation = SpMM with 1/deg edge values on R-MAT scale 22, K=512
    "c4_spmm_rmat22_k512": dict(graph=("rmat", 22, 16), msg=M.MSG_SPMM, sop=None, k=512,
                                dense=("uniform", -1.0, 1.0), values="inv_degree", seed=46),
    # sigmoid at scale: R-MAT scale 24, K=128, 64-bit row pointers with 32-bit column ids
    "c5_sigmoid_rmat24_k128": dict(graph=("rmat", 24, 16), msg=M.MSG_SIGMOID, sop=M.SOP_SIGMOID, k=128,
                                   dense=("uniform", -0.5, 0.5), values="ones", seed=47),
}


def make_config(name, device="cpu", dtype=torch.float32, scale=None, ptr_dtype=torch.int64,
                idx_dtype=torch.int32):
    """Builds (CSR, X) for a named configuration; X doubles as Y, as in every benchmark configuration.
    ``scale`` overrides the R-MAT scale (or log2 of the vertex count for ER) to get a smaller instance of
    the same family."""
    cfg = dict(CONFIGS[name])
    kind, size, factor = cfg["graph"]
    if kind == "rmat":
        sc = scale if scale is not None else size
        n = 1 << sc
        src, dst = rmat_edges(sc, factor, cfg["seed"], device=device)
    else:
        n = (1 << scale) if scale is not None else size
        src, dst = er_edges(n, factor, cfg["seed"], device=device)
    csr = build_csr(src, dst, n, ptr_dtype=ptr_dtype, idx_dtype=idx_dtype, val_dtype=dtype,
                    values=cfg["values"])
    d = cfg["dense"]
    if d[0] == "uniform":
        x = dense_uniform(n, cfg["k"], d[1], d[2], cfg["seed"] + 1000, device=device, dtype=dtype)
    else:
        x = dense_normal(n, cfg["k"], d[1], cfg["seed"] + 1000, device=device, dtype=dtype)
    cfg["n"] = n
    return cfg, csr, x


def algorithmic_bytes(msg, nnz, m, k, val_bytes, idx_bytes, ptr_bytes, beta_nonzero=False):
    """Bytes one call must move: every gathered Y row in full, one column id (and one edge value when the
    message consumes it: ROP_NOOP with a VSC stage, e.g. SpMM) per edge, X_u read (messages whose VOP or ROP uses
    X) and Z_u written once per row (and read when the call accumulates: beta != 0, or any message outside the
    four optimised patterns), two row pointers per row."""
    vop, rop, vsc = msg & 0xF, msg & 0xF0, msg & 0xF000
    reads_x = vop not in (M.VOP_COPY_RHS, M.VOP_NOOP) or rop in (M.ROP_DOT, M.ROP_ADD_LHS, M.ROP_NORML)
    reads_y = vop != M.VOP_COPY_LHS
    uses_val = rop == M.ROP_NOOP and vsc != M.VSC_NOOP
    accumulates = beta_nonzero or msg not in (M.MSG_SIGMOID, M.MSG_TDIST, M.MSG_SPMM, M.MSG_GCN)
    per_edge = (k * val_bytes + idx_bytes if reads_y else 0) + (val_bytes if uses_val else 0)
    r = (2 if reads_x else 1) + (1 if accumulates else 0)
    return nnz * per_edge + m * (r * k * val_bytes + 2 * ptr_bytes)
