"""Multi-token-prediction (MTP) head: one extra decoder layer of the target's shape that shares its embedding and
lm_head and drafts from the target's own hidden state.

Input of MTP position ``i`` is ``fc([norm_e(E[t_{i+1}]) ; norm_h(h_i)])`` where ``h_i`` is the target's last-layer
residual stream at position ``i`` and ``t_{i+1}`` the token that follows; the layer's output goes through the shared
final norm and lm_head and predicts ``t_{i+2}``.  Deeper drafts feed the layer's own output back as ``h``.
Reference: ``kernels/m1/m1_mtp.cu`` (head forward :565-687, context entries :11, :768) and the MTP checkpoint reader
``crates/agens-cli/src/spec.rs:306-370`` (``upload_mtp``, ``mtp.*`` tensor names).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..ops import basic
from ..ops import linear as L
from .._lib import EPI_STORE
from .config import ModelConfig, scaled
from .dense import DenseModel, M_GEMV


class MtpHead(DenseModel):
    """One-layer model with its own paged KV; ``embed``, ``final_norm`` weights for the head and ``lm_head`` are the
    target's tensors (shared, not copied).  Beside a tensor-parallel target the head runs unsharded on the leader's GPU
    (the target's hidden rows are replicated on every rank); the target's lm_head is a vocabulary shard there, so the
    head carries its own full one (``own_lm_head``; reference: the MTP head under TP, kernels/m1/m1_mtp.cu:503-524)."""

    def __init__(self, target: DenseModel, **kw):
        full = getattr(target, "full_cfg", None)
        cfg = scaled(full or target.cfg, 1)
        self.own_lm_head = full is not None
        kw.setdefault("max_seqs", target.max_seqs)
        kw.setdefault("max_ctx", target.max_ctx)
        kw.setdefault("split_keys", target.split_keys)
        lm_rows = (cfg.vocab + 31) // 32 * 32 if self.own_lm_head else target.lm_rows
        super().__init__(cfg, target.dev, lm_rows=lm_rows, **kw)
        self.embed = target.embed
        self.lm_head = None if self.own_lm_head else target.lm_head
        self.final_norm = target.final_norm
        self.fc: Optional[L.WqLinear] = None
        self.norm_e = self.norm_h = None
        self.cat = torch.zeros(M_GEMV, 2 * cfg.d_model, dtype=torch.bfloat16, device=self.dev)
        self.hid_in = torch.zeros(M_GEMV, cfg.d_model, dtype=torch.bfloat16, device=self.dev)
        self._pair_hidden = None
        self.shortlist = None          # int32 [rows of the shortlist lm_head]: token id of every row (use_shortlist)
        self._short_n = 0

    @staticmethod
    def random_init_for(target: DenseModel, seed: int = 7, **kw) -> "MtpHead":
        m = MtpHead(target, **kw)
        cfg, dev = m.cfg, m.dev
        g = torch.Generator(device=dev).manual_seed(seed)
        shapes = cfg.linear_shapes()
        d = {}
        for i, (lin, (n, k)) in enumerate(shapes.items()):
            d[lin] = L.WqLinear.random(n, k, 4, cfg.group, dev, seed=seed * 7919 + i)
        d["ln1"] = (1.0 + 0.05 * torch.randn(cfg.d_model, device=dev, generator=g)).to(torch.bfloat16)
        d["ln2"] = (1.0 + 0.05 * torch.randn(cfg.d_model, device=dev, generator=g)).to(torch.bfloat16)
        m.layers.append(d)
        m.fc = L.WqLinear.random(cfg.d_model, 2 * cfg.d_model, 4, cfg.group, dev, seed=seed * 7919 + 100)
        m.norm_e = (1.0 + 0.05 * torch.randn(cfg.d_model, device=dev, generator=g)).to(torch.bfloat16)
        m.norm_h = (1.0 + 0.05 * torch.randn(cfg.d_model, device=dev, generator=g)).to(torch.bfloat16)
        if m.own_lm_head:
            m.lm_head = L.WqLinear.random(m.lm_rows, cfg.d_model, cfg.lm_head_bits, cfg.group, dev, seed=seed * 7919 + 200)
        return m.finalize()

    def use_shortlist(self, ids):
        """Restricts the head's lm_head to the token ids of ``ids`` (the reference's draft shortlist, by default the
        32768 most frequent ids of its own generations: crates/agens-cli/src/spec.rs:372-386): a chain step then reads
        that many rows of the head instead of the whole vocabulary.  The rows are taken from the current lm_head,
        quantised again in its format; a drafted token is always one of ``ids``."""
        from ..utils import quant
        full = self.lm_head
        idx = torch.as_tensor(list(ids), dtype=torch.long, device=self.dev)
        assert idx.numel() > 0 and int(idx.max()) < (self.cfg.vocab_valid or self.cfg.vocab) and int(idx.min()) >= 0
        rows = full.dequant().index_select(0, idx).float().cpu()
        n = int(idx.numel())
        pad = (-n) % 32
        if pad:
            rows = torch.cat([rows, torch.zeros(pad, rows.shape[1])])
        self.lm_head = L.WqLinear.from_quant(quant.quantize(rows, full.bits, full.group), self.dev)
        self.lm_rows = n + pad
        self._short_n = n
        self.shortlist = torch.cat([idx, torch.zeros(pad, dtype=torch.long, device=self.dev)]).to(torch.int32)
        return self.finalize()

    def _lm_valid(self) -> int:
        return self._short_n if self.shortlist is not None else super()._lm_valid()

    def _combine_argmax(self, m: int, standalone: bool = False):
        if self.shortlist is not None:                   # position in the shortlist -> token id
            self.out_ids[:m].copy_(self.shortlist.index_select(0, self.out_ids[:m].long()))

    def finalize(self):
        super().finalize()
        if self.fc is not None:
            from .. import _lib
            need = _lib.cuda_lib().b2_wq_gemv_scratch_floats(self.fc.n, self.fc.k, self.fc.ks, 2, M_GEMV)
            if need > self.ws.scratch.numel():
                self.ws = L.GemvWorkspace(self.dev, floats=need, panels=max(self.ws.counters.numel(), 1 << 10))
        return self

    def _rows_body(self, m: int, n_groups: int, want_logits: bool):
        cfg = self.cfg
        d = cfg.d_model
        e = basic.embed(self.ids[:m], self.embed, None, status=self.status)
        self.cat[:m, :d] = basic.rmsnorm(e, self.norm_e, cfg.rms_eps)
        self.cat[:m, d:] = basic.rmsnorm(self.hid_in[:m], self.norm_h, cfg.rms_eps)
        L.gemv(self.fc, self.cat[:m], self.ws, epi=EPI_STORE, out=self.h_a[:m])
        basic.sumsq(self.h_a[:m], self.ss_a)
        parts = self._layers_small(m, n_groups)
        self._head_small(m, parts, want_logits)

    # -------------------------------------------------------------------------------------------- prompt positions
    def _chunk_input(self, ids: torch.Tensor, sub_i) -> torch.Tensor:
        cfg = self.cfg
        c0, c1 = self._sub_slice
        e = basic.embed(ids, self.embed, None, status=self.status)
        cat = torch.cat([basic.rmsnorm(e, self.norm_e, cfg.rms_eps),
                         basic.rmsnorm(self._pair_hidden[c0:c1].contiguous(), self.norm_h, cfg.rms_eps)], dim=1)
        return self._linear_big(self.fc, cat)

    def _prefill_chunk(self, seq: int, ids: torch.Tensor, pos0: int, final: bool, want_logits: bool):
        if ids.numel() <= M_GEMV:                      # short tail: the row path reads its hidden rows from hid_in
            c0, c1 = self._sub_slice
            self.hid_in[:c1 - c0].copy_(self._pair_hidden[c0:c1])
        return super()._prefill_chunk(seq, ids, pos0, final, want_logits)

    def prefill_pairs(self, seq: int, tokens_after: torch.Tensor, hidden: torch.Tensor):
        """Context entries for ``T`` committed positions at once (a prefill chunk of the target): ``hidden[i]`` is the
        target's last-layer residual row of a position and ``tokens_after[i]`` the token that follows it.  Runs the
        layer through the large-m path (tensor-core linears, prefill attention) and appends T entries to the head's
        own KV of ``seq``; nothing is drafted.  Reference: kernels/m1/m1_mtp.cu:768 (``materialize`` after every
        prefill chunk)."""
        T = int(tokens_after.numel())
        assert hidden.shape[0] == T
        self._pair_hidden = hidden
        try:
            self.prefill(seq, tokens_after)
        finally:
            self._pair_hidden = None

    def forward_mtp(self, ids: List[int], hidden: torch.Tensor, seqs: List[int]):
        """Rows ``(ids[i], hidden[i])`` appended to ``seqs[i]``; returns the drafted token of every row.  The layer's
        output hidden state of every row stays in ``self.h_a``."""
        m = len(ids)
        self.hid_in[:m].copy_(hidden[:m])
        out, _ = self.forward_rows(ids, seqs)
        return out
