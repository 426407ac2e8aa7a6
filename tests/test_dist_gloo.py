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


@pytest.mark.parametrize("world", [2, 3])
def test_row_shards_exchange_over_gloo(tmp_path, world):
    import torch.multiprocessing as mp
    from fusedmm_b200.build import build
    build()
    port = 29500 + (os.getpid() % 1000) + world
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
