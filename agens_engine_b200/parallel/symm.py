"""Symmetric peer memory and the slotted inbox used by every in-kernel collective.

Each tensor-parallel rank (one process per GPU, ``torch.distributed`` for the bootstrap) allocates one inbox region,
exports its CUDA IPC handle and maps all peers' regions.  A region is a sequence of *slots*; a slot holds one fp32
contribution per source rank.  Call sites own slots statically (slot index = position of the call in the step), and a
call re-arms the slot of the call before it, which no rank writes again before its next use -- so a step needs no
host-side bookkeeping and can live in a CUDA graph.  Reference: ``crates/agens-cli/src/tp.rs:94-175`` (region
exchange through files) and ``kernels/src/tp_push.cuh:17-39`` (three rotating Lamport buffers).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _lib
from .._lib import CommArgs, TpPush, check, ptr

SENTINEL = 0x80000000   # -0.0f: "not written yet"


class SymmetricInbox:
    def __init__(self, rank: int, world: int, slot_floats: int, n_slots: int, device, group=None,
                 timeout_s: float = 2.0, status: Optional[torch.Tensor] = None):
        """``slot_floats``: floats per source rank in one slot (multiple of 4); the region holds
        ``n_slots * world * slot_floats`` floats."""
        assert slot_floats % 4 == 0 and world <= _lib.K_MAX_TP
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.slot_stride = slot_floats
        self.slot_floats = slot_floats * world
        self.n_slots = n_slots
        self.timeout_ns = int(timeout_s * 1e9)
        lib = _lib.cuda_lib()
        nbytes = self.slot_floats * n_slots * 4
        self._own = C.c_void_p()
        handle = C.create_string_buffer(64)
        with torch.cuda.device(self.device):
            check(lib.b2_ipc_alloc(nbytes, C.byref(self._own), handle), "b2_ipc_alloc")
            check(lib.b2_fill_u32(self._own.value, SENTINEL, nbytes // 4, _lib.current_stream()), "b2_fill_u32")
            torch.cuda.synchronize(self.device)
        handles: List[Optional[bytes]] = [None] * world
        if world > 1:
            dist.all_gather_object(handles, handle.raw, group=group)
        else:
            handles[0] = handle.raw
        self.ptrs: List[int] = []
        self._opened = []
        for r in range(world):
            if r == rank:
                self.ptrs.append(self._own.value)
            else:
                p = C.c_void_p()
                with torch.cuda.device(self.device):
                    check(lib.b2_ipc_open(handles[r], C.byref(p)), "b2_ipc_open")
                self.ptrs.append(p.value)
                self._opened.append(p.value)
        self.status = status if status is not None else torch.zeros(1, dtype=torch.int32, device=self.device)
        if world > 1:
            dist.barrier(group=group)   # every region is armed before anyone pushes

    def _fill(self, a, slot: int, clear_slot: Optional[int], skip_push: bool):
        for r in range(self.world):
            a.inbox[r] = self.ptrs[r]
        a.rank, a.size = self.rank, self.world
        a.slot_off = slot * self.slot_floats
        a.clear_off = -1 if clear_slot is None else clear_slot * self.slot_floats
        a.slot_stride = self.slot_stride
        a.status = ptr(self.status)
        a.timeout_ns = self.timeout_ns
        a.skip_push = 1 if skip_push else 0
        return a

    def comm_args(self, slot: int, clear_slot: Optional[int] = None, skip_push: bool = False,
                  clear_n: Optional[int] = None) -> CommArgs:
        """``clear_n``: floats per source rank that the earlier user of ``clear_slot`` wrote (default: whole slot)."""
        assert 0 <= slot < self.n_slots
        a = self._fill(CommArgs(), slot, clear_slot, skip_push)
        a.clear_n = self.slot_stride if clear_n is None else (clear_n + 3) // 4 * 4
        return a

    def tp_push(self, slot: int, clear_slot: Optional[int] = None, skip_push: bool = False) -> TpPush:
        assert 0 <= slot < self.n_slots
        return self._fill(TpPush(), slot, clear_slot, skip_push)

    def check_status(self, what: str = "collective"):
        st = int(self.status.item())
        if st != 0:
            self.status.zero_()
            raise _lib.B2Error(what, st)

    def rearm_all(self):
        """Host-side recovery after a failed step: put every slot of the own region back to the sentinel."""
        lib = _lib.cuda_lib()
        with torch.cuda.device(self.device):
            check(lib.b2_fill_u32(self._own.value, SENTINEL, self.slot_floats * self.n_slots, _lib.current_stream()),
                  "b2_fill_u32")

    def close(self, group=None):
        """Unmap the peers' regions, wait until every rank has done so, then free the own region (an exporter must
        not free memory that an importer still maps)."""
        lib = _lib.cuda_lib()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for p in self._opened:
                lib.b2_ipc_close(p)
            self._opened = []
            if self.world > 1 and dist.is_initialized():
                dist.barrier(group=group)
            if self._own:
                lib.b2_ipc_free(self._own)
                self._own = None
