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


class HostStep:
    """The step for callers whose arrays live in HOST memory while N GPUs share the work (every rank sees the same
    host arrays, or its own copy of them).  A rank that called ``fusedMM_csr`` with host arrays would bring all of Y
    over its own PCIe link, N times the same bytes per node and per step.  Here the links work side by side and
    NVLink does the rest:

    1. rank r copies rows ``[r*n/N, (r+1)*n/N)`` of Y, and of the graph only the row pointers and column ids
       (edge values) of its own row shard, to its GPU;
    2. one all-gather (in place, over NVLink) completes Y on every GPU;
    3. the rank's kernels compute its row shard of Z (shards of equal COST, ``bounds``) from device arrays;
    4. the rank copies rows of Z back to the host array: without ``pz`` its own shard; with ``pz`` (a ``PeerZ``) the
       rows ``[r*m/N, (r+1)*m/N)``, equal BYTES per link: the kernels store every finished row that has edges
       straight into the Z of the one rank that will copy it out (a row crosses NVLink at most once; rows without
       edges are zeroed by the receiver from the row pointers of its range).

    ``compute`` is the call that does step 3 (``api.fusedMM_csr`` with device tensors); the CPU tests pass a stand-in,
    so that slicing, re-basing and the all-gather are covered with the ``gloo`` backend."""

    def __init__(self, n, k, dtype, device, dist, bounds, nnz_max=None, with_val=False, idx_dtype=None, group=None,
                 compute=None, pz=None, m=None):
        import torch
        self._torch, self.dist, self.group = torch, dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.n, self.k = int(n), int(k)
        self.m = int(m) if m is not None else int(n)
        self.r0, self.r1 = int(bounds[self.rank]), int(bounds[self.rank + 1])
        self.rows_per = (self.n + self.world - 1) // self.world
        self.zrows_per = (self.m + self.world - 1) // self.world
        self.y = torch.empty((self.rows_per * self.world, self.k), dtype=dtype, device=device)
        self.pz = pz if (pz is not None and self.world > 1) else None
        self.z = None if self.pz is not None else torch.zeros((max(self.r1 - self.r0, 1), self.k), dtype=dtype, device=device)
        self.rowptr = torch.empty(self.r1 - self.r0 + 1, dtype=torch.int64, device=device)
        self.rowptr_out = torch.empty(self.zrows_per + 1, dtype=torch.int64, device=device) if self.pz is not None else None
        self.idx_dtype = idx_dtype or torch.int32
        self.indx = self.val = None
        self._nnz_cap = 0
        self._with_val = with_val
        self._dtype, self._device = dtype, device
        if nnz_max:
            self._reserve(int(nnz_max))
        self.compute = compute or api.fusedMM_csr
        self.h2d_bytes = self.d2h_bytes = 0

    def out_rows(self):
        """Rows of Z this rank copies to the host in a step."""
        if self.pz is None:
            return self.r0, self.r1
        a = min(self.m, self.rank * self.zrows_per)
        return a, min(self.m, a + self.zrows_per)

    def _reserve(self, edges):
        if edges > self._nnz_cap:
            torch = self._torch
            self.indx = torch.empty(edges, dtype=self.idx_dtype, device=self._device)
            self.val = torch.empty(edges, dtype=self._dtype, device=self._device) if self._with_val else None
            self._nnz_cap = edges

    def step(self, imessage, rowptr_host, indx_host, val_host, x_host, y_host, z_host, sop=None, stream=None,
             z_rows_only=False):
        """One call: ``rowptr_host`` (m+1 int64 entries), ``indx_host``, ``val_host`` (or None), ``x_host``
        (``y_host`` itself when X and Y are the same matrix), ``y_host`` and ``z_host`` are host tensors (pinned for
        speed).  Returns the status of the compute calls; the rows ``out_rows()`` of ``z_host`` are complete on return
        (``z_rows_only``: ``z_host`` holds just those rows).  Every rank of the group must call it."""
        torch = self._torch
        r0, r1, k, n = self.r0, self.r1, self.k, self.n
        cuda = self.y.is_cuda
        esz = self.y.element_size()
        kw = {"stream": stream} if stream is not None else {}
        h2d = 0
        # 1. this rank's slice of Y, and its slice of the graph
        a = self.rank * self.rows_per
        b = min(n, a + self.rows_per)
        if b > a:
            self.y[a:b].copy_(y_host[a:b], non_blocking=True)
            h2d += (b - a) * k * esz
        e0, e1 = int(rowptr_host[r0]), int(rowptr_host[r1])
        self._reserve(max(e1 - e0, 1))
        self.rowptr.copy_(rowptr_host[r0:r1 + 1], non_blocking=True)
        self.rowptr.sub_(e0)  # the slice of column ids starts at 0 on the device
        h2d += (r1 - r0 + 1) * 8
        if e1 > e0:
            self.indx[:e1 - e0].copy_(indx_host[e0:e1], non_blocking=True)
            h2d += (e1 - e0) * self.indx.element_size()
            if self._with_val and val_host is not None:
                self.val[:e1 - e0].copy_(val_host[e0:e1], non_blocking=True)
                h2d += (e1 - e0) * self.val.element_size()
        za, zb = self.out_rows()
        if self.pz is not None and zb > za:  # the row pointers of the rows this rank copies out: their empty rows become 0 here
            self.rowptr_out[:zb - za + 1].copy_(rowptr_host[za:zb + 1], non_blocking=True)
            h2d += (zb - za + 1) * 8
        # 2. all ranks' slices of Y, in place
        if self.world > 1:
            mine = self.y[a:a + self.rows_per].reshape(-1)
            # NCCL gathers in place (the input is this rank's slot of the output); other backends get a copy
            self.dist.all_gather_into_tensor(self.y.view(-1), mine if cuda else mine.clone(), group=self.group)
        # 3. the row shard
        if x_host is y_host:
            x_dev = self.y[r0:]
        else:
            x_dev = torch.empty((max(r1 - r0, 1), k), dtype=self.y.dtype, device=self.y.device)
            if r1 > r0:
                x_dev[:r1 - r0].copy_(x_host[r0:r1], non_blocking=True)
                h2d += (r1 - r0) * k * esz
        st = 0
        # nnz is the library's hint for scratch sizes and for the length at which rows are split: the whole graph's
        # count everywhere, so that a row is cut (and its pieces added) the same way whatever the sharding
        nnz_hint = int(rowptr_host[self.m]) - int(rowptr_host[0])
        if self.pz is None:
            if r1 > r0:
                st = self.compute(imessage, r1 - r0, n, k, 1.0, nnz_hint, n, n, self.val, self.indx, self.rowptr[:-1],
                                  self.rowptr[1:], x_dev, k, self.y, k, 0.0, self.z, k, sop=sop, **kw)
                # 4. its rows of Z back to the host
                (z_host[:r1 - r0] if z_rows_only else z_host[r0:r1]).copy_(self.z[:r1 - r0], non_blocking=True)
        else:
            pz = self.pz
            if zb > za:
                st = api.zero_empty_rows(self.rowptr_out[:zb - za], self.rowptr_out[1:zb - za + 1], pz.z[za:], k, k,
                                         stream=stream)
            # one call per rank whose output range this shard reaches into: rows [lo, hi) go to rank d's Z
            for d in range(self.world):
                lo, hi = max(r0, d * self.zrows_per), min(r1, (d + 1) * self.zrows_per, self.m)
                if hi <= lo or st != 0:
                    continue
                st = self.compute(imessage, hi - lo, n, k, 1.0, nnz_hint, n, n, self.val, self.indx,
                                  self.rowptr[lo - r0:-1], self.rowptr[lo - r0 + 1:], x_dev[lo - r0:], k, self.y, k, 0.0,
                                  pz.z[lo:], k, sop=sop,
                                  z_peers=None if d == self.rank else [pz.ptrs[d] + lo * pz.row_bytes], **kw)
            pz.finish_step()  # every rank's kernels, and with them their stores into this rank's Z, are done
            if zb > za:
                (z_host[:zb - za] if z_rows_only else z_host[za:zb]).copy_(pz.z[za:zb], non_blocking=True)
            pz.finish_step()  # nobody stores into a Z that is still being copied out
        if cuda:
            torch.cuda.current_stream().synchronize()
        self.h2d_bytes, self.d2h_bytes = h2d, (zb - za) * k * esz
        return st
