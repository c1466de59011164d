"""Large-m linears (prefill, big verify batches): dequantised weights x activations on the tensor cores."""
from __future__ import annotations

import torch

from . import linear as L


def wq_linear(lin: L.WqLinear, x: torch.Tensor, owner=None) -> torch.Tensor:
    """``bf16 [T, n] = x @ dequant(W)^T``.  The weight is dequantised FM -> bf16 into a reusable buffer first."""
    tmp = None
    if owner is not None:
        need = lin.n * lin.k
        if getattr(owner, "_deq_tmp", None) is None or owner._deq_tmp.numel() < need:
            owner._deq_tmp = torch.empty(need, dtype=torch.bfloat16, device=x.device)
        tmp = owner._deq_tmp[:need].view(lin.n, lin.k)
    w = lin.dequant(out=tmp)
    return torch.matmul(x, w.t())
