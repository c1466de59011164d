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

    def gemm_reduce_scatter(self, a: torch.Tensor, b: torch.Tensor, status: Optional[torch.Tensor] = None):
        """Row-parallel linear with the reduce-scatter fused into the GEMM: ``a`` [T, K] and ``b`` [N, K] are this
        rank's bf16 activation and weight shards; every rank ends with the rank-ordered fp32 sum of its
        ``ceil(T / world)`` rows (flat, zero padded), without a separate push pass: the tcgen05 GEMM's epilogue stores
        each partial tile into the owner's inbox slot over NVLink while the other tiles are still being computed
        (``b2_gemm_bf16_push``), and the wait-and-combine half of the reduce-scatter kernel sums the slots.  Returns
        ``(shard, rows_per_rank)``."""
        lib = _lib.cuda_lib()
        ib = self.inbox
        w, rank = ib.world, ib.rank
        T, K = a.shape
        N = b.shape[0]
        assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and b.shape[1] == K and T >= w
        rows_per = (T + w - 1) // w
        n = rows_per * N
        assert n % 4 == 0 and n <= ib.slot_stride, "the inbox slot is too small for this chunk"
        args = self._args(n, skip_push=True)
        arr = (C.c_void_p * 8)(*([ib.ptrs[r] for r in range(w)] + [None] * (8 - w)))
        shard = torch.zeros(n, dtype=torch.float32, device=a.device)
        n_valid = max(0, min(rows_per, T - rank * rows_per)) * N
        with torch.cuda.device(a.device):
            check(lib.b2_gemm_bf16_push(ptr(a), a.stride(0), ptr(b), b.stride(0), T, N, K, arr, w, rank, args.slot_off,
                                        args.slot_stride, rows_per, ptr(status if status is not None else ib.status), current_stream()),
                  "b2_gemm_bf16_push")
            if n_valid:
                check(lib.b2_comm_reduce_scatter(C.byref(args), 0, n_valid, ptr(shard), current_stream()), "reduce_scatter (collect)")
        return shard, rows_per

    def gemm_reduce_gather(self, a: torch.Tensor, b: torch.Tensor, status: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The whole row-parallel linear of a prefill chunk in two launches: the tcgen05 GEMM whose epilogue stores its
        fp32 partial tiles into the owners' inboxes (slot A), then ONE kernel that sums each rank's rows in rank order,
        writes them as bf16, pushes the sums to the peers (slot B) and collects the peers' rows as they arrive
        (``b2_comm_collect_gather``).  Returns the summed bf16 ``[T, N]`` (the same bits on every rank).  The inbox must
        have six slots: calls rotate over three slot pairs, and every unit is re-armed by the thread that read it, so
        there is no clearing pass.  Do not mix with the rotating calls above on the same inbox."""
        lib = _lib.cuda_lib()
        ib = self.inbox
        w, rank = ib.world, ib.rank
        T, K = a.shape
        N = b.shape[0]
        assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and b.shape[1] == K and ib.n_slots >= 6
        rows_per = (T + w - 1) // w
        assert N % 4 == 0 and rows_per * N <= ib.slot_stride, "the inbox slot is too small for this chunk"
        slot_a = 2 * (self.calls % 3)
        self.calls += 1
        args = ib.comm_args(slot_a, None, skip_push=True, clear_n=0)
        slot_b_off = (slot_a + 1) * ib.slot_floats
        arr = (C.c_void_p * 8)(*([ib.ptrs[r] for r in range(w)] + [None] * (8 - w)))
        out = torch.empty(T, N, dtype=torch.bfloat16, device=a.device)
        st = ptr(status if status is not None else ib.status)
        with torch.cuda.device(a.device):
            check(lib.b2_gemm_bf16_push(ptr(a), a.stride(0), ptr(b), b.stride(0), T, N, K, arr, w, rank, args.slot_off,
                                        args.slot_stride, rows_per, st, current_stream()), "b2_gemm_bf16_push")
            check(lib.b2_comm_collect_gather(C.byref(args), slot_b_off, rows_per, N, T, ptr(out), current_stream()), "collect_gather")
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
