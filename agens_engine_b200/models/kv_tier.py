"""Host tier of the paged KV cache: pages older than a resident window live in pinned host memory and are streamed
back, batch by batch, on a side stream while attention runs on the batches already staged.

Replaces the reference's tiered KV (``kernels/m1/m1_kv.cu`` ring/stage kernels, ``kernels/src/kv_tier.cu``,
``m1_dense8.cu:95-125`` partial (o, lse) merge).  Here every batch of host pages is one more set of KV splits of the
same split-KV attention kernel: the resident launch skips splits marked as host resident, staged launches fill exactly
those split slots from a double-buffered device staging area, and one merge pass combines all slots in split order,
so a tiered step is bit-identical to an all-resident one.  Copies are plain pinned ``cudaMemcpyAsync`` (one per batch
and layer) ordered against the attention launches with events.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..ops import attention as A

HOST_PAGE = -2


class HostKvTier:
    def __init__(self, model, window_tokens: int, batch_pages: int = 256):
        cfg = model.cfg
        assert batch_pages % 16 == 0, "a batch must cover whole KV splits of both the decode and the prefill split size"
        self.m, self.B = model, batch_pages
        self.window_pages = max(batch_pages, (window_tokens + cfg.page_size - 1) // cfg.page_size)
        shape = (batch_pages,) + tuple(model.kv[0].shape[1:])
        self.stage = [torch.empty(shape, dtype=torch.bfloat16, device=model.dev) for _ in range(2)]
        self.copy_stream = torch.cuda.Stream(device=model.dev)
        self.ev_copied = [torch.cuda.Event() for _ in range(2)]
        self.ev_used = [torch.cuda.Event() for _ in range(2)]
        for e in self.ev_used:
            e.record(torch.cuda.current_stream(model.dev))
        # every logical page p of a staged batch sits in staging slot p % B (batches start at multiples of B)
        self.bt_stage = (torch.arange(model.pages_per_seq, dtype=torch.int32, device=model.dev) % batch_pages)[None, :] \
            .expand(model.max_seqs, -1)
        self.blocks: Dict[int, List[torch.Tensor]] = {}        # seq -> pinned [layers, B, 2, hkv, 16, hd] per batch
        self.ready: Dict[int, List[torch.cuda.Event]] = {}     # seq -> per batch: its device-to-host copies are complete
        self._free: List[torch.Tensor] = []                    # pinned blocks of ended sequences, reused (no allocation per batch)
        self.bytes_h2d = 0
        self.bytes_d2h = 0

    # ------------------------------------------------------------------------------------------------ offload
    def n_host_pages(self, seq: int) -> int:
        return len(self.blocks.get(seq, ())) * self.B

    def maybe_offload(self, seq: int):
        """Moves whole batches of the oldest resident pages to the host while more than window + one batch is resident."""
        m = self.m
        full_pages = m.seq_len_host[seq] // m.cfg.page_size
        while full_pages - self.n_host_pages(seq) >= self.window_pages + self.B:
            self._offload_batch(seq)

    def _offload_batch(self, seq: int):
        m = self.m
        b = len(self.blocks.setdefault(seq, []))
        lo = b * self.B
        idx = torch.tensor(m.seq_pages[seq][lo:lo + self.B], dtype=torch.long, device=m.dev)
        blk = self._free.pop() if self._free else \
            torch.empty((m.cfg.n_layers, self.B) + tuple(m.kv[0].shape[1:]), dtype=torch.bfloat16, pin_memory=True)
        main = torch.cuda.current_stream(m.dev)
        for l, kv in enumerate(m.kv):
            blk[l].copy_(kv.index_select(0, idx), non_blocking=True)
        # No host wait: whatever writes the freed pages next is ordered behind these copies on the same stream, and the
        # side stream that brings the block back waits for this event before it reads the pinned memory.
        ev = torch.cuda.Event()
        ev.record(main)
        self.bytes_d2h += blk.numel() * 2
        self.blocks[seq].append(blk)
        self.ready.setdefault(seq, []).append(ev)
        for i in range(lo, lo + self.B):
            m.pool.evict_page(m._aid[seq], i)
            m.seq_pages[seq][i] = HOST_PAGE
        m.block_table[seq, lo:lo + self.B] = HOST_PAGE

    def drop(self, seq: int):
        blks, evs = self.blocks.pop(seq, None), self.ready.pop(seq, None)
        if blks:
            for e in evs or ():
                e.synchronize()                                 # a block is only reused once its copies have landed
            self.copy_stream.synchronize()                      # ... and nothing is still reading it back
            self._free.extend(blks)

    # ------------------------------------------------------------------------------------------------ attention
    def attend(self, layer: int, q, grp_tok0, grp_cnt, tok_pos, tok_seq, tiered_groups: Dict[int, tuple], split_keys: int,
               max_splits: int, part_o, part_ml, out, tree_mask=None, shared_kv: bool = False):
        """Attention of one layer for a step in which the sequences of ``tiered_groups`` (seq -> (first group, number
        of groups)) have pages on the host.  Resident splits first, then the staged batches, then one merge."""
        m, cfg = self.m, self.m.cfg
        common = dict(hq=cfg.n_heads, hkv=cfg.n_kv_heads, hd=cfg.head_dim, split_keys=split_keys, max_splits=max_splits,
                      part_o=part_o, part_ml=part_ml, status=m.status, out=out, tree_mask=tree_mask, shared_kv=shared_kv)
        main = torch.cuda.current_stream(m.dev)
        A.attn_decode(q, m.kv[layer], m.block_table, grp_tok0, grp_cnt, tok_pos, tok_seq, phase=1, **common)
        spb = self.B * cfg.page_size // split_keys               # splits per batch
        k = 0
        for seq, (g_first, g_n) in tiered_groups.items():
            blocks = self.blocks[seq]
            for b, blk in enumerate(blocks):
                buf = k % 2
                with torch.cuda.stream(self.copy_stream):
                    self.copy_stream.wait_event(self.ev_used[buf])           # the launch that last read this buffer
                    self.copy_stream.wait_event(self.ready[seq][b])          # the block's own device-to-host copies
                    self.stage[buf].copy_(blk[layer], non_blocking=True)
                    self.ev_copied[buf].record(self.copy_stream)
                self.bytes_h2d += blk[layer].numel() * 2
                main.wait_event(self.ev_copied[buf])
                A.attn_decode(q, self.stage[buf], self.bt_stage, grp_tok0[g_first:g_first + g_n], grp_cnt[g_first:g_first + g_n],
                              tok_pos, tok_seq, split_range=(b * spb, (b + 1) * spb), phase=1, **common)
                self.ev_used[buf].record(main)
                k += 1
        A.attn_decode(q, m.kv[layer], m.block_table, grp_tok0, grp_cnt, tok_pos, tok_seq, phase=2, **common)
        return out
