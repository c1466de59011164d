"""Quantised linears on the GPU: FM weight holder + GEMV launcher (decode / verify / small batch).

Python here only assembles argument blocks; the arithmetic is in ``csrc/kernels/sm100/wq_gemv.cu``.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import os
from typing import Optional

import torch

from .. import _lib
from .._lib import (EPI_ARGMAX, EPI_F32, EPI_RESID, EPI_STORE, EPI_SWIGLU, EPI_TP_RESID, PRO_NORM, PRO_PLAIN, WqGemvArgs,
                    check, current_stream, ptr)
from ..utils import quant

SS_LD = 128  # token stride of partial-sum-of-squares / argmax-partial buffers = most token rows of one step


def fm_bytes(n: int, k: int, bits: int, group: int) -> int:
    return (n // 32) * (k // 128) * quant.block_bytes(bits, group)


def choose_rb(n: int) -> int:
    """Row blocks per warp item: 64-row items when the matrix has enough rows to keep every warp busy."""
    if os.environ.get("B200E_GEMV_RB"):
        return int(os.environ["B200E_GEMV_RB"])
    return 4 if n >= 16384 else 2


def choose_ks(n: int, k: int, slice_k: int = 2560) -> int:
    """Number of k slices of a linear: a function of the shape only (never of the token count), so per-row
    arithmetic stays batch invariant.  Slices of about ``slice_k`` inputs keep the staged activations small and give
    the persistent GEMV thousands of (panel, slice) work items to balance over the SMs."""
    slice_k = int(os.environ.get("B200E_SLICE_K", slice_k))
    nu = k // 128
    want = max(1, round(k / slice_k))
    best = 1
    for ks in range(1, min(nu, _lib.K_MAX_KS) + 1):
        if nu % ks == 0 and abs(ks - want) < abs(best - want):
            best = ks
    return best


@dataclasses.dataclass
class WqLinear:
    """One quantised linear in kernel (FM) layout on a CUDA device."""
    n: int
    k: int
    bits: int
    group: int
    wq: torch.Tensor            # uint8 [fm_bytes]: (32-row panel, 128-k batch) blocks, scales inside
    ks: int = 1
    rb: int = 2

    @staticmethod
    def from_quant(ql: quant.QuantLinear, device, ks: Optional[int] = None) -> "WqLinear":
        wq = quant.pack_fm(ql)
        ks = ks or choose_ks(ql.n, ql.k)
        return WqLinear(ql.n, ql.k, ql.bits, ql.group, wq.reshape(-1).to(device), ks, choose_rb(ql.n))

    @staticmethod
    def random(n: int, k: int, bits: int, group: int, device, seed: int, stddev: float = 0.02,
               ks: Optional[int] = None) -> "WqLinear":
        """Random-init N(0, stddev) weights quantised on the device directly into FM form."""
        lib = _lib.cuda_lib()
        wq = torch.empty(fm_bytes(n, k, bits, group), dtype=torch.uint8, device=device)
        with torch.cuda.device(device):
            check(lib.b2_wq_random(ptr(wq), n, k, bits, group, stddev, seed, current_stream()), "b2_wq_random")
        ks = ks or choose_ks(n, k)
        return WqLinear(n, k, bits, group, wq, ks, choose_rb(n))

    @staticmethod
    def from_checkpoint(packed: torch.Tensor, scale: torch.Tensor, zero: Optional[torch.Tensor], n: int, k: int,
                        bits: int, group: int, device, ks: Optional[int] = None) -> "WqLinear":
        """Checkpoint container (bit stream + scales [+ zero points]) -> FM, repacked on the device."""
        lib = _lib.cuda_lib()
        packed = packed.to(device).contiguous()
        scale = scale.to(device).contiguous()
        zero = None if zero is None else zero.to(device=device, dtype=torch.float16).contiguous()
        wq = torch.empty(fm_bytes(n, k, bits, group), dtype=torch.uint8, device=device)
        is_bf16 = 1 if scale.dtype == torch.bfloat16 else 0
        if not is_bf16 and scale.dtype != torch.float16:
            scale = scale.to(torch.float16)
        with torch.cuda.device(device):
            check(lib.b2_wq_repack(ptr(packed), ptr(scale), is_bf16, ptr(zero), n, k, bits, group, ptr(wq),
                                   current_stream()), "b2_wq_repack")
        ks = ks or choose_ks(n, k)
        return WqLinear(n, k, bits, group, wq, ks, choose_rb(n))

    def n_panels(self) -> int:
        return self.n // 32

    def nbytes(self) -> int:
        return self.wq.numel()

    def dequant(self, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """bf16 [n, k] on the device (kernel path)."""
        lib = _lib.cuda_lib()
        if out is None:
            out = torch.empty(self.n, self.k, dtype=torch.bfloat16, device=self.wq.device)
        with torch.cuda.device(out.device):
            check(lib.b2_wq_dequant(ptr(self.wq), self.n, self.k, self.bits, self.group, ptr(out), self.k,
                                    current_stream()), "b2_wq_dequant")
        return out

    def dequant_cpu(self) -> torch.Tensor:
        """fp32 [n, k] computed on the CPU from the FM bytes (independent of every kernel)."""
        ql = quant.unpack_fm(self.wq.cpu(), self.bits, self.n, self.k, self.group)
        return ql.dequant()


@dataclasses.dataclass
class Bf16Linear:
    """A linear kept in bf16 (checkpoint format ``bf16``, reference: crates/agens-core/src/weights.rs:176-187
    ``LinearFormat::Bf16``; the bf16 drafter): ``w`` is bf16 ``[n, k]`` on the device.  :func:`gemv` and :func:`mm` take
    it like a quantised linear; up to eight rows run the bf16 GEMV (``csrc/kernels/sm100/bf16_gemv.cu``), more rows the
    tcgen05 GEMM.  Norm prologue, SwiGLU and the next norm's statistics are separate small kernels on this path."""
    n: int
    k: int
    w: torch.Tensor
    bits: int = 16
    group: int = 0
    ks: int = 1
    rb: int = 2

    @staticmethod
    def from_tensor(w: torch.Tensor, device) -> "Bf16Linear":
        w = w.to(device=device, dtype=torch.bfloat16).contiguous()
        return Bf16Linear(w.shape[0], w.shape[1], w)

    def n_panels(self) -> int:
        return 1                 # parts of the sum of squares a residual epilogue leaves (one: a separate pass computes it)

    def nbytes(self) -> int:
        return self.w.numel() * 2

    def dequant(self, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.w

    def dequant_cpu(self) -> torch.Tensor:
        return self.w.float().cpu()


BF16_GEMV_ROWS = 8


def _bf16_linear(lin: Bf16Linear, x: torch.Tensor, *, epi: int, pro: int, norm_w, eps: float, resid, out, ss_out, gemv_rows: int = BF16_GEMV_ROWS):
    """The contract of :func:`gemv` for a bf16 linear, as separate kernels: RMSNorm (when asked), the product, then
    SwiGLU or the residual's sum of squares."""
    from . import basic
    from . import gemm as G
    lib = _lib.cuda_lib()
    m = x.shape[0]
    assert x.dtype == torch.bfloat16 and x.shape[1] == lin.k and x.stride(1) == 1
    xin = basic.rmsnorm(x, norm_w, eps) if pro == PRO_NORM else x
    dev = x.device

    def product(dst_bf16, dst_f32, r):
        if m <= gemv_rows:
            d = dst_bf16 if dst_bf16 is not None else dst_f32
            with torch.cuda.device(dev):
                check(lib.b2_bf16_gemv(ptr(xin), xin.stride(0), ptr(lin.w), lin.w.stride(0), m, lin.n, lin.k, ptr(dst_bf16), ptr(dst_f32),
                                       d.stride(0), ptr(r), r.stride(0) if r is not None else 0, current_stream()), "b2_bf16_gemv")
        else:
            G.gemm_bf16(xin, lin.w, resid=r, out=dst_bf16 if dst_bf16 is not None else dst_f32)

    if epi in (EPI_STORE, EPI_RESID):
        if out is None:
            out = torch.empty(m, lin.n, dtype=torch.bfloat16, device=dev)
        product(out, None, resid if epi == EPI_RESID else None)
        if epi == EPI_RESID and ss_out is not None:
            basic.sumsq(out, ss_out)
        return out
    if epi == EPI_SWIGLU:
        gu = torch.empty(m, lin.n, dtype=torch.bfloat16, device=dev)
        product(gu, None, None)
        act = basic.swiglu_interleaved(gu)
        if out is None:
            return act
        out.copy_(act)
        return out
    if epi == EPI_F32:
        if out is None:
            out = torch.empty(m, lin.n, dtype=torch.float32, device=dev)
        product(None, out, None)
        return out
    raise ValueError("this epilogue is not available for a bf16 linear (the lm_head is quantised at load)")


class GemvWorkspace:
    """Split-k scratch, self-resetting item counters and the status word shared by the GEMV / GEMM launches of one
    stream, plus the fp16 activation staging buffer of the tensor-core path (grown on first use)."""

    def __init__(self, device, floats: int = 4 << 20, panels: int = 1 << 16, status: Optional[torch.Tensor] = None):
        self.scratch = torch.empty(floats, dtype=torch.float32, device=device)
        self.counters = torch.zeros(panels, dtype=torch.int32, device=device)
        # the status word may live inside a block of status words that the owner reads with one copy
        self.status = status if status is not None else torch.zeros(1, dtype=torch.int32, device=device)
        self.x16 = None
        self.mm_min_rows = None      # overrides MM_MIN_ROWS for the launches that use this workspace

    def x16_buffer(self, n_pad: int, k: int) -> torch.Tensor:
        """fp16 activation staging of the tensor-core path.  Sized once for 256 rows x 32768 inputs so that its address
        stays valid inside captured CUDA graphs; only a wider linear makes it grow (which invalidates such graphs)."""
        if self.x16 is None or self.x16.numel() < n_pad * k:
            self.x16 = torch.empty(max(n_pad * k, 256 * 32768), dtype=torch.float16, device=self.scratch.device)
        return self.x16

    def ensure_scratch(self, floats: int):
        if floats > self.scratch.numel():
            self.scratch = torch.empty(floats, dtype=torch.float32, device=self.scratch.device)


MM_MIN_ROWS = int(os.environ.get("B200E_MM_MIN_ROWS", "9"))     # token rows from which the tcgen05 GEMM takes over
# Measurement aids.  Only a library built with B200E_NVCC_DEFS=-DB2_MEASURE reads these fields; the production kernels
# have the modes compiled out, so a stray environment variable cannot change results.
TRACE_BUFFER = None      # int64 CUDA tensor [CTAs * 8 warps * 8] that receives the GEMV's phase stamps
GEMV_DEBUG = int(os.environ.get("B200E_GEMV_DEBUG", "0"))
MM_DBG = int(os.environ.get("B200E_MM_DBG", "0"))


def gemv(lin: WqLinear, x: torch.Tensor, ws: GemvWorkspace, *, epi: int = EPI_STORE,
         pro: int = PRO_PLAIN, ss_in: Optional[torch.Tensor] = None, ss_parts: int = 0,
         norm_w: Optional[torch.Tensor] = None, eps: float = 1e-6, resid: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None, ss_out: Optional[torch.Tensor] = None,
         amax_val: Optional[torch.Tensor] = None, amax_idx: Optional[torch.Tensor] = None, n_valid: Optional[int] = None,
         yf: Optional[torch.Tensor] = None, tp: Optional[_lib.TpPush] = None):
    """Launch one GEMV on the current stream.  ``x``: bf16 ``[m, k]`` (``h`` when ``pro == PRO_NORM``).  More than
    ``MM_MIN_ROWS - 1`` rows go to the tensor-core GEMM (:func:`mm`), which takes the same arguments."""
    if isinstance(lin, Bf16Linear):
        if tp is not None:
            raise ValueError("bf16 linears are not sharded: tensor-parallel models quantise them at load")
        # a workspace pinned to the tensor-core path (one kernel family for every step) pins bf16 linears to the GEMM too
        rows = BF16_GEMV_ROWS if ws.mm_min_rows is None else min(BF16_GEMV_ROWS, ws.mm_min_rows - 1)
        return _bf16_linear(lin, x, epi=epi, pro=pro, norm_w=norm_w, eps=eps, resid=resid, out=out, ss_out=ss_out, gemv_rows=rows)
    lib = _lib.cuda_lib()
    m = x.shape[0]
    if m >= (ws.mm_min_rows or MM_MIN_ROWS) and tp is None:
        return mm(lin, x, ws, epi=epi, pro=pro, ss_in=ss_in, ss_parts=ss_parts, norm_w=norm_w, eps=eps, resid=resid, out=out,
                  ss_out=ss_out, amax_val=amax_val, amax_idx=amax_idx, n_valid=n_valid, yf=yf)
    assert x.dtype == torch.bfloat16 and x.shape[1] == lin.k and x.stride(1) == 1
    dev = x.device
    a = WqGemvArgs()
    a.wq = ptr(lin.wq)
    a.n, a.k, a.m = lin.n, lin.k, m
    a.bits, a.group, a.ks, a.rb = lin.bits, lin.group, lin.ks, (lin.rb if m <= 16 else 2)
    a.pro = pro
    a.x, a.ldx = ptr(x), x.stride(0)
    a.ss_in, a.ss_parts, a.ss_ld = ptr(ss_in), ss_parts, SS_LD
    a.norm_w, a.eps = ptr(norm_w), eps
    a.epi = epi
    if epi in (EPI_STORE, EPI_RESID, EPI_TP_RESID):
        if out is None:
            out = torch.empty(m, lin.n, dtype=torch.bfloat16, device=dev)
        a.y, a.ldy = ptr(out), out.stride(0)
    elif epi == EPI_SWIGLU:
        if out is None:
            out = torch.empty(m, lin.n // 2, dtype=torch.bfloat16, device=dev)
        a.y, a.ldy = ptr(out), out.stride(0)
    elif epi == EPI_F32:
        if out is None:
            out = torch.empty(m, lin.n, dtype=torch.float32, device=dev)
        a.yf, a.ldy = ptr(out), out.stride(0)
    elif epi == EPI_ARGMAX:
        a.amax_val, a.amax_idx = ptr(amax_val), ptr(amax_idx)
        a.n_valid = lin.n if n_valid is None else n_valid
        if yf is not None:
            a.yf, a.ldy = ptr(yf), yf.stride(0)
    if resid is not None:
        a.resid, a.ldr = ptr(resid), resid.stride(0)
    a.ss_out = ptr(ss_out)
    a.vworkers = lib.b2_wq_gemv_vworkers(lin.n, lin.k, lin.ks, a.rb)
    a.fmax = lib.b2_wq_gemv_fmax(lin.n, lin.k, lin.ks, a.rb)
    need = lib.b2_wq_gemv_scratch_floats(lin.n, lin.k, lin.ks, a.rb, m)
    if need > ws.scratch.numel() or lin.n_panels() > ws.counters.numel():
        raise RuntimeError(f"GEMV workspace too small: need {need} floats, {lin.n_panels()} counters")
    a.scratch, a.counters = ptr(ws.scratch), ptr(ws.counters)
    a.status = ptr(ws.status)
    a.debug = GEMV_DEBUG
    a.trace = ptr(TRACE_BUFFER)
    if tp is not None:
        a.tp = tp
    with torch.cuda.device(dev):
        check(lib.b2_wq_gemv(C.byref(a), current_stream()), "b2_wq_gemv")
    return out


def mm(lin: WqLinear, x: torch.Tensor, ws: GemvWorkspace, *, epi: int = EPI_STORE, pro: int = PRO_PLAIN,
       ss_in: Optional[torch.Tensor] = None, ss_parts: int = 0, norm_w: Optional[torch.Tensor] = None, eps: float = 1e-6,
       resid: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, ss_out: Optional[torch.Tensor] = None,
       amax_val: Optional[torch.Tensor] = None, amax_idx: Optional[torch.Tensor] = None, n_valid: Optional[int] = None,
       yf: Optional[torch.Tensor] = None):
    """Same contract as :func:`gemv` for 1 .. 256 rows on the tcgen05 tensor cores (``csrc/kernels/sm100/wq_mm.cu``):
    the weights are dequantised to fp16 tiles inside the kernel, the activations are staged as fp16 by a small prologue
    kernel that also applies the RMSNorm of ``pro == PRO_NORM``."""
    if isinstance(lin, Bf16Linear):
        return _bf16_linear(lin, x, epi=epi, pro=pro, norm_w=norm_w, eps=eps, resid=resid, out=out, ss_out=ss_out, gemv_rows=0)
    lib = _lib.cuda_lib()
    m = x.shape[0]
    assert x.dtype == torch.bfloat16 and x.shape[1] == lin.k and x.stride(1) == 1 and 1 <= m <= 256
    dev = x.device
    a = _lib.WqMmArgs()
    a.wq, a.n, a.k, a.m, a.bits, a.group = ptr(lin.wq), lin.n, lin.k, m, lin.bits, lin.group
    a.epi = epi
    if epi in (EPI_STORE, EPI_RESID):
        out = torch.empty(m, lin.n, dtype=torch.bfloat16, device=dev) if out is None else out
        a.y, a.ldy = ptr(out), out.stride(0)
    elif epi == EPI_SWIGLU:
        out = torch.empty(m, lin.n // 2, dtype=torch.bfloat16, device=dev) if out is None else out
        a.y, a.ldy = ptr(out), out.stride(0)
    elif epi == EPI_F32:
        out = torch.empty(m, lin.n, dtype=torch.float32, device=dev) if out is None else out
        a.yf, a.ldy = ptr(out), out.stride(0)
    elif epi == EPI_ARGMAX:
        a.amax_val, a.amax_idx = ptr(amax_val), ptr(amax_idx)
        a.n_valid = lin.n if n_valid is None else n_valid
        if yf is not None:
            a.yf, a.ldy = ptr(yf), yf.stride(0)
    else:
        raise ValueError("epilogue not available on the tensor-core path")
    if resid is not None:
        a.resid, a.ldr = ptr(resid), resid.stride(0)
    a.ss_out, a.ss_ld = ptr(ss_out), SS_LD
    n_pad = lib.b2_wq_mm_npad(m)
    ws.ensure_scratch(lib.b2_wq_mm_scratch_floats(lin.n, lin.k, n_pad))
    if (lin.n + 127) // 128 > ws.counters.numel():
        raise RuntimeError("workspace has too few counters")
    a.scratch, a.counters, a.status = ptr(ws.scratch), ptr(ws.counters), ptr(ws.status)
    x16 = ws.x16_buffer(n_pad, lin.k)
    a.dbg = MM_DBG
    norm = pro == PRO_NORM
    with torch.cuda.device(dev):
        check(lib.b2_wq_mm(C.byref(a), ptr(x), x.stride(0), ptr(ss_in) if norm else 0, ss_parts if norm else 0, SS_LD,
                           ptr(norm_w) if norm else 0, eps, ptr(x16), current_stream()), "b2_wq_mm")
    return out
