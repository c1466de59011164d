"""Launchers of the paged attention kernels (``csrc/kernels/sm100/attn_decode.cu``: decode, verify and chunked prefill)."""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Optional

import torch

from .. import _lib
from .._lib import AttnDecodeArgs, check, current_stream, ptr

PAGE = 16


def attn_decode(q: torch.Tensor, kv_pool: torch.Tensor, block_table: torch.Tensor, grp_tok0: torch.Tensor,
                grp_cnt: torch.Tensor, tok_pos: torch.Tensor, tok_seq: torch.Tensor, hq: int, hkv: int, hd: int,
                split_keys: int, max_splits: int, part_o: Optional[torch.Tensor] = None,
                part_ml: Optional[torch.Tensor] = None, tree_mask: Optional[torch.Tensor] = None,
                status: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                split_range: Optional[tuple] = None, phase: int = 0, shared_kv: bool = False) -> torch.Tensor:
    """q: bf16 [n_tok, hq*hd] (RoPE applied); kv_pool: bf16 [pages, 2, hkv, 16, hd].  Returns bf16 [n_tok, hq*hd].
    ``split_range=(lo, hi)`` restricts the launch to those KV splits and ``phase`` selects the split kernel (1), the
    merge (2) or both (0): the pieces of a tiered-KV step."""
    lib = _lib.cuda_lib()
    n_tok = q.shape[0]
    dev = q.device
    if part_o is None:
        part_o = torch.empty(n_tok, hq, max_splits, hd, dtype=torch.float32, device=dev)
        part_ml = torch.empty(n_tok, hq, max_splits, 2, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev) if status is None else status
    if out is None:
        out = torch.empty(n_tok, hq * hd, dtype=torch.bfloat16, device=dev)
    a = AttnDecodeArgs()
    a.q, a.ldq = ptr(q), q.stride(0)
    a.kv_pool, a.n_pages = ptr(kv_pool), kv_pool.shape[0]
    a.block_table, a.bt_ld = ptr(block_table), block_table.stride(0)
    a.grp_tok0, a.grp_cnt, a.n_groups = ptr(grp_tok0), ptr(grp_cnt), grp_tok0.numel()
    a.tok_pos, a.tok_seq = ptr(tok_pos), ptr(tok_seq)
    a.tree_mask = ptr(tree_mask)
    a.hq, a.hkv = hq, hkv
    a.split_keys, a.max_splits = split_keys, max_splits
    a.scale_log2 = (1.0 / math.sqrt(hd)) * math.log2(math.e)
    a.part_o, a.part_ml = ptr(part_o), ptr(part_ml)
    a.out, a.ldo = ptr(out), out.stride(0)
    a.n_tok = n_tok
    a.status = ptr(status)
    a.split_lo, a.split_hi = split_range if split_range else (0, 0)
    a.phase = phase
    a.shared_kv = 1 if shared_kv else 0     # CTA-shared K/V ring: same arithmetic per row, fewer loads for many-row groups
    with torch.cuda.device(dev):
        check(lib.b2_attn_decode(C.byref(a), hd, current_stream()), "b2_attn_decode")
    return out


def prefill_groups(T: int, pos0: int, seq: int, dev):
    """Row groups of a prefill chunk for the split-KV kernel: 8 consecutive rows per group."""
    pos = torch.arange(pos0, pos0 + T, dtype=torch.int32, device=dev)
    seqv = torch.full((T,), seq, dtype=torch.int32, device=dev)
    g0 = torch.arange(0, T, 8, dtype=torch.int32, device=dev)
    gc = torch.clamp(T - g0, max=8).to(torch.int32)
    return g0, gc, pos, seqv


PREFILL_TC_MIN_TOKENS = 64          # chunks from this size run the tcgen05 kernel (head_dim 128, group size dividing 128)


def attn_prefill_tc(q: torch.Tensor, kv_pool: torch.Tensor, block_table: torch.Tensor, seq: int, pos0: int, hq: int,
                    hkv: int, status: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of a prefill chunk on the tcgen05 tensor cores (``csrc/kernels/sm100/attn_prefill_tc.cu``):
    128-row query tiles (128 / group-size tokens x the heads of one KV group), S and the per-block output in TMEM."""
    lib = _lib.cuda_lib()
    if not getattr(lib, "_pf_tc_declared", False):
        vp, i = C.c_void_p, C.c_int
        lib.b2_attn_prefill_tc.argtypes = [vp, vp, vp, i, vp, i, i, i, i, i, C.c_float, vp, vp]
        lib.b2_attn_prefill_tc.restype = i
        lib._pf_tc_declared = True
    T = q.shape[0]
    assert q.is_contiguous() and q.shape[1] == hq * 128
    status = torch.zeros(1, dtype=torch.int32, device=q.device) if status is None else status
    if out is None:
        out = torch.empty(T, hq * 128, dtype=torch.bfloat16, device=q.device)
    row = block_table[seq]
    with torch.cuda.device(q.device):
        check(lib.b2_attn_prefill_tc(ptr(q), ptr(kv_pool), ptr(row), row.numel(), ptr(out), T, pos0, hq, hkv, kv_pool.shape[0],
                                     1.0 / math.sqrt(128.0), ptr(status), current_stream()), "b2_attn_prefill_tc")
    return out


def attn_prefill(q: torch.Tensor, kv_pool: torch.Tensor, block_table: torch.Tensor, seq: int, pos0: int, hq: int,
                 hkv: int, hd: int, status: Optional[torch.Tensor] = None, split_keys: int = 256,
                 tensor_core: Optional[bool] = None) -> torch.Tensor:
    """Causal attention of a prefill chunk (``q``: bf16 ``[T, hq*hd]`` at positions ``pos0 .. pos0+T-1`` of ``seq``)
    over the paged KV cache, which already holds the chunk's own K/V.  Chunks of at least PREFILL_TC_MIN_TOKENS rows
    with head_dim 128 run the tcgen05 kernel (``tensor_core`` forces the choice), the rest the split-KV kernel."""
    T = q.shape[0]
    gq = hq // hkv
    can_tc = hd == 128 and 128 % gq == 0 and q.is_contiguous() and block_table.stride(1) == 1
    if tensor_core is None:
        tensor_core = T >= PREFILL_TC_MIN_TOKENS and os.environ.get("B200E_PREFILL_ATTN_TC", "1") == "1"
    if tensor_core and can_tc:
        return attn_prefill_tc(q, kv_pool, block_table, seq, pos0, hq, hkv, status=status)
    g0, gc, pos, seqv = prefill_groups(T, pos0, seq, q.device)
    max_splits = (pos0 + T + split_keys - 1) // split_keys
    return attn_decode(q, kv_pool, block_table, g0, gc, pos, seqv, hq, hkv, hd, split_keys, max_splits, status=status,
                       shared_kv=True)
