"""Large-m linears (prefill, big verify batches) on the tcgen05 tensor cores (``csrc/kernels/sm100/gemm_tc.cu``)."""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import _lib
from .._lib import check, current_stream, ptr
from . import linear as L


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, resid: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
              out_f32: bool = False, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a[M,K] @ b[N,K]^T (+ resid)`` with bf16 operands, fp32 accumulation in TMEM; bf16 (or fp32) result."""
    lib = _lib.cuda_lib()
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.stride(1) == 1 and b.stride(1) == 1
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=a.device)
    d_bf, d_f32 = (None, out) if out.dtype == torch.float32 else (out, None)
    with torch.cuda.device(a.device):
        check(lib.b2_gemm_bf16(ptr(a), a.stride(0), ptr(b), b.stride(0), M, N, K, ptr(d_bf), ptr(d_f32), out.stride(0),
                               ptr(resid), resid.stride(0) if resid is not None else 0, ptr(status), current_stream()),
              "b2_gemm_bf16")
    return out


def dequant_bf16(lin, owner=None) -> torch.Tensor:
    """The linear's weights as bf16 [n, k]: a bf16 linear's own tensor, else the quantised weights expanded into a
    buffer that ``owner`` keeps and reuses."""
    if isinstance(lin, L.Bf16Linear):
        return lin.w
    tmp = None
    if owner is not None:
        need = lin.n * lin.k
        if getattr(owner, "_deq_tmp", None) is None or owner._deq_tmp.numel() < need:
            owner._deq_tmp = torch.empty(need, dtype=torch.bfloat16, device=lin.wq.device)
        tmp = owner._deq_tmp[:need].view(lin.n, lin.k)
    return lin.dequant(out=tmp)


def wq_linear(lin: L.WqLinear, x: torch.Tensor, owner=None, resid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``bf16 [T, n] = x @ dequant(W)^T (+ resid)``.  The weight is dequantised FM -> bf16 into a reusable buffer, then
    multiplied by the tcgen05 GEMM.  ``B200E_PLAIN_GEMM=1`` selects the library GEMM instead (same-box baseline)."""
    if isinstance(lin, L.Bf16Linear):
        return gemm_bf16(x, lin.w, resid=resid, status=getattr(owner, "status", None))
    tmp = None
    if owner is not None:
        need = lin.n * lin.k
        if getattr(owner, "_deq_tmp", None) is None or owner._deq_tmp.numel() < need:
            owner._deq_tmp = torch.empty(need, dtype=torch.bfloat16, device=x.device)
        tmp = owner._deq_tmp[:need].view(lin.n, lin.k)
    w = lin.dequant(out=tmp)
    if os.environ.get("B200E_PLAIN_GEMM") == "1":
        y = torch.matmul(x, w.t())
        return y if resid is None else (y.float() + resid.float()).to(torch.bfloat16)
    return gemm_bf16(x, w, resid=resid, status=getattr(owner, "status", None))
