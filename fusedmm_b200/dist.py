"""Multi-GPU row sharding: one process per GPU, rows cut into cost-balanced contiguous shards, Y
replicated, Z shards exchanged over NCCL (NVLink 5 / NVSwitch).

The compute of a shard is an ordinary ``fusedMM_csr`` call on a row range (the four-array CSR needs no
re-basing), so only the exchange lives here.  The shards are ragged (equal edges, not equal rows), so the
exchange is one broadcast per owner, all in flight together; with the ``gloo`` backend the same code runs
on CPU tensors, which is how the host logic is tested without GPUs.
"""
from __future__ import annotations

import numpy as np

from . import api


# Cost of a row, in edges, beside its edges: X_u read, Z_u written (and sent to the peers) and the latency of a
# short row.  On a B200 the whole-row launch spends about as long on a row as on 9 of its edges, and with two
# GPUs on the FR benchmark graph a weight of 8 gave 2.32 ms per step against 2.62 ms for shards of equal edges
# (3: 2.49, 5: 2.41, 12: 2.34, 24: 2.61).
ROW_WEIGHT = 8


def shard_bounds(rowptr_host: np.ndarray, world: int, row_weight: int = ROW_WEIGHT) -> np.ndarray:
    """Row bounds of ``world`` shards of (nearly) equal cost, a row costing its edges plus ``row_weight``
    (0: equal edge counts, the reference's thread partition); ``rowptr_host`` has m+1 entries."""
    rp = np.ascontiguousarray(rowptr_host)
    return api.shard_rows(rp[:-1].copy(), rp[1:].copy(), world, row_weight=row_weight)


def exchange_row_shards(z, bounds, dist, group=None):
    """Every rank owns rows [bounds[r], bounds[r+1]) of ``z`` (same shape on all ranks); afterwards every
    rank holds all rows.  Enqueued on the current stream; returns when the work is enqueued (NCCL) or
    done (gloo)."""
    world = dist.get_world_size(group)
    works = []
    for g in range(world):
        r0, r1 = int(bounds[g]), int(bounds[g + 1])
        if r1 > r0:
            works.append(dist.broadcast(z[r0:r1], src=dist.get_global_rank(group, g) if group else g,
                                        group=group, async_op=True))
    for w in works:
        w.wait()


def fusedMM_csr_sharded(imessage, n, k, val, indx, rowptr, x, y, z, bounds, dist, sop=None, stream=None,
                        group=None):
    """The multi-GPU step: this rank computes its row shard of ``z`` on its GPU and the shards are
    exchanged.  ``rowptr``, ``indx``, ``val``, ``x`` (all rows) and ``y`` are this rank's device copies."""
    rank = dist.get_rank(group)
    r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
    st = 0
    if r1 > r0:
        st = api.fusedMM_csr(imessage, r1 - r0, n, k, 1.0, int(indx.numel()), n, n, val, indx, rowptr[r0:-1],
                             rowptr[r0 + 1:], x[r0:], k, y, k, 0.0, z[r0:], k, sop=sop, stream=stream)
    exchange_row_shards(z, bounds, dist, group)
    return st


class PeerZ:
    """A Z matrix that every rank of the group can write into on every other rank (torch symmetric memory:
    one allocation per GPU, peer-mapped over NVLink).  With it the exchange of the Z row shards is fused into
    the compute kernels: ``fusedmm_b200_csr_multi`` stores each finished row into the local Z and into the
    peers' Z, and a step ends with one small collective that orders the ranks."""

    def __init__(self, n, k, dtype, device, dist, group=None):
        import torch
        import torch.distributed._symmetric_memory as symm_mem
        self.dist, self.group = dist, group
        self.z = symm_mem.empty((n, k), dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.z, group if group is not None else dist.group.WORLD)
        self.rank, self.world = self.handle.rank, self.handle.world_size
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        assert self.ptrs[self.rank] == self.z.data_ptr()
        # NVSwitch multicast mapping of the same buffers (0 when the fabric has none)
        self.multicast = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.row_bytes = k * self.z.element_size()
        self._token = torch.zeros(1, dtype=torch.float32, device=device)
        self._torch = torch
        self._side = torch.cuda.Stream(device=device)  # the local fill of rows without edges runs beside the kernels
        self._fill_pending = False

    def peers_at_row(self, r0):
        """Addresses of row ``r0`` in the other ranks' copies of Z."""
        return [p + r0 * self.row_bytes for i, p in enumerate(self.ptrs) if i != self.rank]

    def multicast_at_row(self, r0):
        """Multicast address of row ``r0`` (None without NVSwitch multicast)."""
        return self.multicast + r0 * self.row_bytes if self.multicast else None

    def use_multicast(self):
        """Multicast stores pay from three GPUs on: every GPU then receives all of Z once whatever the number
        of ranks, while per-peer stores make the rank with the most rows send them N-1 times.  Between two GPUs
        a multicast store also loops this rank's own rows back through the switch, and plain peer stores measured
        7 % faster."""
        return bool(self.multicast) and self.world > 2

    def zero_foreign_empty_rows(self, rowptr, r0, r1, stream=None):
        """The fused exchange does not send rows without edges (a quarter to half of the rows of an R-MAT graph):
        with beta == 0 every rank zeroes those rows of the OTHER ranks' shards in its own copy of Z, from the row
        pointers it holds anyway.  ``rowptr``: device tensor of n+1 entries; [r0, r1) is this rank's shard.
        The fill is pure store bandwidth on rows nobody else writes in this step, so it is enqueued on a side stream
        (after the work already on torch's current stream) and runs beside the step's kernels; ``finish_step`` joins
        it.  ``stream`` is ignored (kept for callers that passed the current stream's handle)."""
        n, k = self.z.shape
        torch = self._torch
        self._side.wait_stream(torch.cuda.current_stream())
        st = 0
        if r0 > 0:
            st = st or api.zero_empty_rows(rowptr[:r0], rowptr[1:r0 + 1], self.z, k, k, stream=self._side.cuda_stream)
        if r1 < n:
            st = st or api.zero_empty_rows(rowptr[r1:n], rowptr[r1 + 1:n + 1], self.z[r1:], k, k, stream=self._side.cuda_stream)
        self._fill_pending = True
        return st

    def finish_step(self):
        """Enqueue the collective that follows this rank's kernels in stream order; when it completes on a
        rank, every rank's kernels of the step (and with them their stores into this rank's Z) are done."""
        if self._fill_pending:
            self._torch.cuda.current_stream().wait_stream(self._side)
            self._fill_pending = False
        self.dist.all_reduce(self._token, group=self.group)


def fusedMM_csr_fused_exchange(imessage, n, k, val, indx, rowptr, x, y, pz: PeerZ, bounds, sop=None,
                               stream=None):
    """The multi-GPU step with the exchange fused into the kernels: this rank computes its row shard and
    the kernels write the finished rows into every rank's Z (``pz``).  ``stream`` must be the stream the
    following collective is enqueued on (torch's current stream)."""
    r0, r1 = int(bounds[pz.rank]), int(bounds[pz.rank + 1])
    st = pz.zero_foreign_empty_rows(rowptr, r0, r1, stream=stream)  # beta == 0: rows without edges become 0 everywhere
    if r1 > r0 and st == 0:
        st = api.fusedMM_csr(imessage, r1 - r0, n, k, 1.0, int(indx.numel()), n, n, val, indx, rowptr[r0:-1],
                             rowptr[r0 + 1:], x[r0:], k, y, k, 0.0, pz.z[r0:], k, sop=sop, stream=stream,
                             z_peers=None if pz.use_multicast() else pz.peers_at_row(r0),
                             z_multicast=pz.multicast_at_row(r0) if pz.use_multicast() else None)
    pz.finish_step()
    return st
