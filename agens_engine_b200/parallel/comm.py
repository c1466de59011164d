"""Collectives: the engine's own bounded push kernels over symmetric memory, and the NCCL baseline with the same
interface (the same-box baseline the fused paths are compared against)."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from .. import _lib
from .._lib import check, current_stream, ptr
from .symm import SymmetricInbox


class PushComm:
    """Standalone collectives on a :class:`SymmetricInbox`.  Slots rotate over three indices per communicator, the
    rotation the reference's push all-reduce uses (``tp_push.cuh:135-148``): a call re-arms the slot of the call
    before it.  Not graph-safe by itself (the rotation is host state); graph-captured steps use fixed call-site slots."""

    def __init__(self, inbox: SymmetricInbox, first_slot: int = 0):
        self.inbox, self.first, self.calls, self.prev_n = inbox, first_slot, 0, 0

    def _args(self, n: int, skip_push=False):
        cur = self.first + self.calls % 3
        prev = self.first + (self.calls - 1) % 3
        self.calls += 1
        a = self.inbox.comm_args(cur, prev, skip_push, clear_n=self.prev_n)
        self.prev_n = n
        return a

    def all_reduce(self, x: torch.Tensor, out_dtype=None, skip_push: bool = False) -> torch.Tensor:
        lib = _lib.cuda_lib()
        n = x.numel()
        assert x.is_contiguous() and n % 4 == 0 and n <= self.inbox.slot_stride
        out = torch.empty_like(x, dtype=out_dtype or x.dtype)
        a = self._args(n, skip_push)
        f32 = x.dtype == torch.float32
        with torch.cuda.device(x.device):
            check(lib.b2_comm_all_reduce(C.byref(a), ptr(x) if f32 else 0, 0 if f32 else ptr(x), n,
                                         ptr(out) if out.dtype == torch.float32 else 0,
                                         ptr(out) if out.dtype == torch.bfloat16 else 0, current_stream()), "all_reduce")
        return out

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        lib = _lib.cuda_lib()
        n = x.numel()
        assert x.dtype == torch.float32 and x.is_contiguous() and n % 4 == 0 and n <= self.inbox.slot_stride
        out = torch.empty(self.inbox.world, *x.shape, dtype=torch.float32, device=x.device)
        a = self._args(n)
        with torch.cuda.device(x.device):
            check(lib.b2_comm_all_gather(C.byref(a), ptr(x), n, ptr(out), current_stream()), "all_gather")
        return out

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        lib = _lib.cuda_lib()
        w = self.inbox.world
        assert x.dtype == torch.float32 and x.is_contiguous() and x.shape[0] == w
        n = x.numel() // w
        assert n % 4 == 0 and n <= self.inbox.slot_stride
        out = torch.empty(x.shape[1:], dtype=torch.float32, device=x.device)
        a = self._args(n)
        with torch.cuda.device(x.device):
            check(lib.b2_comm_reduce_scatter(C.byref(a), ptr(x), n, ptr(out), current_stream()), "reduce_scatter")
        return out

    def barrier(self):
        lib = _lib.cuda_lib()
        a = self._args(4)
        with torch.cuda.device(self.inbox.device):
            check(lib.b2_comm_barrier(C.byref(a), current_stream()), "barrier")


class NcclComm:
    """Same interface on NCCL through ``torch.distributed`` (baseline and bring-up)."""

    def __init__(self, group=None):
        self.group = group

    def all_reduce(self, x: torch.Tensor, out_dtype=None, skip_push: bool = False) -> torch.Tensor:
        y = x.float().clone()
        dist.all_reduce(y, group=self.group)
        return y.to(out_dtype or x.dtype)

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        w = dist.get_world_size(self.group)
        out = torch.empty(w, *x.shape, dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty(x.shape[1:], dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=self.group)
        return out

    def barrier(self):
        dist.barrier(group=self.group)
