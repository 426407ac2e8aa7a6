"""The multi-GPU path on CPU: two gloo ranks shard the rows by edge count, each fills its shard of Z (the
CPU oracle stands in for the GPU kernel, on exactly the pointer-offset call a GPU rank makes) and the shards
are exchanged with fusedmm_b200.dist.exchange_row_shards.  Every rank must end up with the full result."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import torch
    import torch.distributed as dist
    from cases import dense, random_csr
    from fusedmm_b200 import dist as fdist, messages as M
    from oracle.cpu import Oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(123)  # same inputs on every rank
        m = n = 900
        k = 24
        pntrb, pntre, indx, val = random_csr(rng, m, n, 6, np.int64, np.int32, hub=2500)
        rowptr = np.concatenate([pntrb, pntre[-1:]])
        val = val.astype(np.float32)
        x = np.nan_to_num(dense(rng, m, k, k, np.float32))
        bounds = fdist.shard_bounds(rowptr, world)
        assert bounds[0] == 0 and bounds[-1] == m
        r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
        orc = Oracle()
        z = np.full((m, k), -777.0, np.float32)  # rows of other ranks start as garbage
        if r1 > r0:
            st = orc.csr(M.MSG_SIGMOID, r1 - r0, n, k, val, indx, rowptr[r0:-1].copy(), rowptr[r0 + 1:].copy(),
                         x[r0:], k, x, k, 0.0, z[r0:], k, sop_kind=M.SOP_SIGMOID)
            assert st == 0
        zt = torch.from_numpy(z)
        fdist.exchange_row_shards(zt, bounds, dist)
        want = np.zeros((m, k), np.float32)
        orc.csr(M.MSG_SIGMOID, m, n, k, val, indx, rowptr[:-1].copy(), rowptr[1:].copy(), x, k, x, k, 0.0, want, k,
                sop_kind=M.SOP_SIGMOID)
        assert np.array_equal(zt.numpy(), want), f"rank {rank}"
        # edge balance: no shard is heavier than an equal share plus one row
        deg = np.diff(rowptr)
        per = [int(deg[bounds[g]:bounds[g + 1]].sum()) for g in range(world)]
        assert max(per) <= deg.sum() / world + deg.max()
        Path(tmp, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def _host_step_worker(rank, world, port, tmp):
    """fusedmm_b200.dist.HostStep on CPU tensors: every rank brings its slice of Y and of the graph, the all-gather
    completes Y, a stand-in for the GPU call (the CPU oracle on the very arguments the GPU call would get) computes
    the row shard, and the rank's rows land in the shared result."""
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import torch
    import torch.distributed as dist
    from cases import dense, random_csr
    from fusedmm_b200 import dist as fdist, messages as M
    from oracle.cpu import Oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(321)  # same inputs on every rank
        m = n = 701                        # not a multiple of the world size: the last slice of Y is ragged
        k = 12
        pntrb, pntre, indx, val = random_csr(rng, m, n, 5, np.int64, np.int32, hub=900)
        rowptr = np.concatenate([pntrb, pntre[-1:]])
        val = val.astype(np.float32)
        y = np.nan_to_num(dense(rng, n, k, k, np.float32))
        x_other = np.nan_to_num(dense(rng, m, k, k, np.float32))
        bounds = fdist.shard_bounds(rowptr, world)
        r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
        orc = Oracle()
        calls = []

        def compute(msg, mm, nn, kk, alpha, nnz, rows, cols, v, ix, pb, pe, xx, ldx, yy, ldy, beta, z, ldz, sop=None):
            calls.append((mm, nnz, int(pb[0]), int(pe[-1])))
            zz = np.zeros((mm, kk), np.float32)
            st = orc.csr(msg, mm, nn, kk, None if v is None else v.numpy(), ix.numpy(), pb.numpy().copy(), pe.numpy().copy(),
                         np.ascontiguousarray(xx.numpy()[:mm]), ldx, yy.numpy()[:nn], ldy, beta, zz, kk, sop_kind=sop)
            z[:mm] = torch.from_numpy(zz)
            return st

        for msg, sop, same, with_val in ((M.MSG_SIGMOID, M.SOP_SIGMOID, True, False), (M.MSG_SPMM, 0, False, True)):
            hs = fdist.HostStep(n, k, torch.float32, "cpu", dist, bounds, with_val=with_val, compute=compute)
            ty = torch.from_numpy(y)
            tx = ty if same else torch.from_numpy(x_other)
            z_host = torch.full((m, k), -777.0)
            st = hs.step(msg, torch.from_numpy(rowptr), torch.from_numpy(indx), torch.from_numpy(val) if with_val else None,
                         tx, ty, z_host, sop=sop)
            assert st == 0
            # the stand-in saw re-based row pointers (first edge 0) and exactly this shard's edges
            assert calls[-1] == (r1 - r0, int(rowptr[-1]), 0, int(rowptr[r1] - rowptr[r0]))   # nnz: the whole graph's, a hint
            assert torch.equal(hs.y[:n], ty)                      # all of Y arrived through the all-gather
            want = np.zeros((m, k), np.float32)
            orc.csr(msg, m, n, k, val, indx, rowptr[:-1].copy(), rowptr[1:].copy(), y if same else x_other, k, y, k, 0.0,
                    want, k, sop_kind=sop)
            assert np.array_equal(z_host.numpy()[r0:r1], want[r0:r1]), f"rank {rank}"
            assert (z_host.numpy()[:r0] == -777.0).all() and (z_host.numpy()[r1:] == -777.0).all()
            per_rank_y = ((n + world - 1) // world) * k * 4
            assert hs.d2h_bytes == (r1 - r0) * k * 4 and hs.h2d_bytes <= per_rank_y + (r1 - r0 + 1) * 8 + \
                int(rowptr[r1] - rowptr[r0]) * (8 if with_val else 4) + (0 if same else (r1 - r0) * k * 4)
        Path(tmp, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_host_arrays_step_over_gloo(tmp_path, world):
    import torch.multiprocessing as mp
    from fusedmm_b200.build import build
    build()
    port = 29700 + (os.getpid() % 200) + world
    mp.spawn(_host_step_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


@pytest.mark.parametrize("world", [2, 3])
def test_row_shards_exchange_over_gloo(tmp_path, world):
    import torch.multiprocessing as mp
    from fusedmm_b200.build import build
    build()
    port = 29500 + (os.getpid() % 1000) + world
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
