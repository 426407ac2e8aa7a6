"""``torch.ops.fusedmm_b200.csr``: the C ABI as a PyTorch custom operator (CUDA tensors, zero copy, enqueued on
torch's current stream).  This is the binding a GNN framework built on PyTorch would call (the reference ships a
CMake file "for DGL integration", ``CMakeLists.txt:1``); autograd is not defined for it.

    import fusedmm_b200.torch_op            # registers the operator
    z = torch.ops.fusedmm_b200.csr(rowptr, colidx, val, x, y, imessage, sop_kind, beta, z_in)
"""
from __future__ import annotations

from typing import Optional

import torch

from . import api


@torch.library.custom_op("fusedmm_b200::csr", mutates_args=(), device_types="cuda")
def csr(rowptr: torch.Tensor, colidx: torch.Tensor, val: Optional[torch.Tensor], x: torch.Tensor, y: torch.Tensor,
        imessage: int, sop_kind: int, beta: float, z_in: Optional[torch.Tensor]) -> torch.Tensor:
    """Z = fusedMM_csr(imessage; CSR(rowptr, colidx, val); X, Y), rows of Z = rows of X.  ``z_in`` is the Z the
    message accumulates into (messages the reference has no optimised kernel for always accumulate; the four
    optimised ones only when beta != 0); ``None`` means zeros."""
    m, k = x.shape
    n = y.shape[0]
    z = torch.zeros((m, k), dtype=x.dtype, device=x.device) if z_in is None else z_in.clone()
    stream = torch.cuda.current_stream(x.device)
    handle = stream.cuda_stream
    if handle == 0:  # the legacy default stream is the C ABI's "synchronous" value: run synchronously
        handle = None
    # nnz = colidx.numel() bounds the edges of the rows, so the library sizes its split-row scratch before it
    # enqueues anything and the call needs no later status check
    with torch.cuda.device(x.device):
        st = api.fusedMM_csr(imessage, m, n, k, 1.0, int(colidx.numel()), m, n, val, colidx, rowptr[:-1], rowptr[1:],
                             x.contiguous(), k, y.contiguous(), k, float(beta), z, k, sop=int(sop_kind), stream=handle)
    if st != 0:
        raise api.FusedMMError(f"fusedMM_csr failed: {api.status_string(st)} ({st})")
    return z


@csr.register_fake
def _(rowptr, colidx, val, x, y, imessage, sop_kind, beta, z_in):
    return torch.empty_like(x)
