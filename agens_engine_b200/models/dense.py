"""Engine-backed dense GQA decoder: weights in kernel layout, paged KV, chunked prefill, graph-captured decode.

This is the model-runtime layer (reference: ``kernels/m1/m1_model.cu`` ``run_model`` :2815-2967 and ``layer``
:2544-2596, the page allocator :1694-1716 and the decode graphs :3071-3140) restated for the dense family.
A decode step is five fused launches per layer -- qkv GEMV (RMSNorm folded into its prologue), RoPE + KV store,
paged attention (+ merge), o_proj GEMV (residual add + next norm statistic in its epilogue), gate/up GEMV (norm
prologue, SwiGLU epilogue), down GEMV (residual epilogue) -- captured once per batch size into a CUDA graph whose
only per-step input is the token produced by the previous step, handled on the device.
"""
from __future__ import annotations

import math
import os
from typing import Dict, List, Optional

import torch

from .. import _lib
from .._lib import EPI_ARGMAX, EPI_F32, EPI_RESID, EPI_STORE, EPI_SWIGLU, PRO_NORM, PRO_PLAIN, check, current_stream, ptr
from ..ops import attention as A
from ..ops import basic
from ..ops import linear as L
from .config import LINEARS, ModelConfig

M_GEMV = 32          # most token rows the GEMV family takes in one launch
STEP_ROWS = 16       # most token rows the persistent step kernel takes (ops/step.py)
M_ROWS = 128         # most token rows of one step (64 decode rows or 128 verify rows, as the reference's batched engine,
                     # kernels/m1/m1_model.cu:203-212); beyond M_GEMV rows the linears run on the tensor-core GEMM


class DenseModel:
    def __init__(self, cfg: ModelConfig, device="cuda:0", max_seqs: int = 1, max_ctx: int = 4096,
                 n_pages: Optional[int] = None, split_keys: int = 64, prefill_chunk: int = 256,
                 lm_rows: Optional[int] = None):
        self.cfg, self.dev = cfg, torch.device(device)
        self.lm_rows = lm_rows or cfg.vocab          # rows of the (possibly vocab-sharded, padded) lm_head
        self.max_seqs, self.max_ctx, self.split_keys = max_seqs, max_ctx, split_keys
        self.prefill_chunk = prefill_chunk
        self.pages_per_seq = (max_ctx + cfg.page_size - 1) // cfg.page_size
        self.n_pages = n_pages or self.pages_per_seq * max_seqs
        self.max_splits = (max_ctx + split_keys - 1) // split_keys
        self.layers: List[Dict[str, object]] = []
        self.embed = None
        self.final_norm = None
        self.lm_head: Optional[L.WqLinear] = None
        from ..serve import host as _host
        self.pool = _host.PageAllocator(self.n_pages, cfg.page_size)     # C++ allocator: refcounted pages, fork
        self._aid: Dict[int, int] = {}                                   # sequence slot -> allocator sequence id
        self.seq_pages: Dict[int, List[int]] = {}                        # host mirror of each slot's block-table row
        self.seq_len_host: Dict[int, int] = {}
        self._graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.row_graphs = False                        # forward_rows replays a per-shape CUDA graph when set
        self.tier = None                               # HostKvTier once enable_host_tier() was called
        self._tiered_groups: Dict[int, tuple] = {}     # this step's sequences with pages on the host
        self.prefill_split = 256                       # KV split size of prefill attention
        self.prefill_mm = os.environ.get("B200E_PREFILL_MM", "1") == "1"
        # Steps of up to sixteen rows can run as ONE persistent kernel (ops/step.py).  Measured on the 32B model (one
        # GPU, ms per step, step kernel against per-op path): sixteen rows 14.6 / 21.1, twelve 13.9 / 20.0, eight
        # 11.8 / 30.9, four 10.5 / 12.1, one 9.9 / 7.8.  Mode "auto" (default) therefore uses it for three to sixteen
        # rows, "on" (B200E_STEP=1, or a serving loop that pins one kernel family) for every step of up to sixteen rows,
        # "off" never.  It keeps a second copy of the quantised weights in its own layout, built on first use.
        env = os.environ.get("B200E_STEP", "auto")
        self.step_mode = {"1": "on", "0": "off"}.get(env, "auto")
        self.use_step = self.step_mode != "off"
        self.step_uniform = False      # every step (1..16 rows) on the work split of the 9..16-row class: rows comparable bit for bit
        self.step = None
        # prefill hands every chunk's last-layer residual rows to this callable: hidden_sink(first position, bf16 [T, d_model])
        self.hidden_sink = None
        self._alloc_buffers()

    # ------------------------------------------------------------------------------------------------ weights
    @staticmethod
    def from_oracle(ow, device="cuda:0", **kw) -> "DenseModel":
        m = DenseModel(ow.cfg, device, **kw)
        for l, lay in enumerate(ow.layers):
            d = {lin: L.WqLinear.from_quant(ow.quant[f"{l}.{lin}"], m.dev) for lin in LINEARS}
            d["ln1"], d["ln2"] = lay["ln1"].to(m.dev), lay["ln2"].to(m.dev)
            m.layers.append(d)
        m.embed = ow.embed.to(m.dev)
        m.final_norm = ow.final_norm.to(m.dev)
        m.lm_head = L.WqLinear.from_quant(ow.quant["lm_head"], m.dev)
        return m.finalize()

    @staticmethod
    def random_init(cfg: ModelConfig, device="cuda:0", seed: int = 0, **kw) -> "DenseModel":
        """Random-init weights of the named architecture, quantised on the device (no host copy of 32B weights).
        ``bf16_linears=True``: the layers' linears are bf16 instead (the benchmark drafter of the reference is bf16)."""
        bf16_linears = bool(kw.pop("bf16_linears", False))
        m = DenseModel(cfg, device, **kw)
        shapes = cfg.linear_shapes()
        g = torch.Generator(device=m.dev).manual_seed(seed)
        for l in range(cfg.n_layers):
            d = {}
            for i, lin in enumerate(LINEARS):
                n, k = shapes[lin]
                if bf16_linears:
                    d[lin] = L.Bf16Linear(n, k, (torch.randn(n, k, device=m.dev, generator=g) * 0.02).to(torch.bfloat16))
                    continue
                d[lin] = L.WqLinear.random(n, k, cfg.bits_of(l, lin), cfg.group, m.dev, seed=seed * 1000003 + l * 8 + i)
            d["ln1"] = (1.0 + 0.05 * torch.randn(cfg.d_model, device=m.dev, generator=g)).to(torch.bfloat16)
            d["ln2"] = (1.0 + 0.05 * torch.randn(cfg.d_model, device=m.dev, generator=g)).to(torch.bfloat16)
            m.layers.append(d)
        # in row chunks: the fp32 intermediate of the whole table would be a 3 GB transient on the 32B vocabulary
        m.embed = torch.empty(cfg.vocab, cfg.d_model, dtype=torch.bfloat16, device=m.dev)
        for r0 in range(0, cfg.vocab, 16384):
            r1 = min(cfg.vocab, r0 + 16384)
            m.embed[r0:r1] = (torch.randn(r1 - r0, cfg.d_model, device=m.dev, generator=g) * 0.02).to(torch.bfloat16)
        m.final_norm = (1.0 + 0.05 * torch.randn(cfg.d_model, device=m.dev, generator=g)).to(torch.bfloat16)
        m.lm_head = L.WqLinear.random(cfg.vocab, cfg.d_model, cfg.lm_head_bits, cfg.group, m.dev, seed=seed * 1000003 + 999983)
        return m.finalize()

    def weight_bytes(self) -> int:
        t = self.embed.numel() * 2 + self.lm_head.nbytes()
        for d in self.layers:
            for lin in LINEARS:
                t += d[lin].nbytes()
        return t

    # ------------------------------------------------------------------------------------------------ buffers
    def _alloc_buffers(self):
        cfg, dev = self.cfg, self.dev
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
        bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)
        # rows of one step: eight per sequence slot (a verify group), at least M_GEMV, at most M_ROWS
        M = self.max_rows = min(M_ROWS, max(M_GEMV, 8 * self.max_seqs))
        self.kv = [torch.zeros(self.n_pages, 2, cfg.n_kv_heads, cfg.page_size, cfg.head_dim, dtype=torch.bfloat16, device=dev)
                   for _ in range(cfg.n_layers)]
        self.block_table = torch.full((self.max_seqs, self.pages_per_seq), -1, dtype=torch.int32, device=dev)
        self.seq_len = i32(self.max_seqs)
        # the per-step row description lives in one buffer so that an eager step uploads it with a single copy
        self._rowbuf = i32(6, M)
        self._rowbuf_host = torch.zeros(6, M, dtype=torch.int32).pin_memory() if dev.type == "cuda" else torch.zeros(6, M, dtype=torch.int32)
        self.ids, self.tok_pos, self.tok_seq, self.grp_tok0, self.grp_cnt, self.rope_pos = (self._rowbuf[i] for i in range(6))
        # rotary position = KV position + delta: after an image the text positions run behind the token count
        self.rope_delta: Dict[int, int] = {}
        self._use_rope_pos = False
        self.last_ids, self.out_ids = i32(M), i32(M)
        self._slot_seq = i32(M)              # decode slots -> sequence ids (fixed address: captured graphs read it)
        self.h_a, self.h_b = bf(M, cfg.d_model), bf(M, cfg.d_model)
        parts = max(cfg.d_model // 32, 1)
        self.ss_a = torch.zeros(parts, L.SS_LD, dtype=torch.float32, device=dev)
        self.ss_b = torch.zeros(parts, L.SS_LD, dtype=torch.float32, device=dev)
        self.qkv = bf(M, cfg.q_dim + 2 * cfg.kv_dim)
        self.q = bf(M, cfg.q_dim)
        self.attn = bf(M, cfg.q_dim)
        self.act = bf(M, cfg.ffn)
        self.part_o = torch.empty(M, cfg.n_heads, self.max_splits, cfg.head_dim, dtype=torch.float32, device=dev)
        self.part_ml = torch.empty(M, cfg.n_heads, self.max_splits, 2, dtype=torch.float32, device=dev)
        lm_panels = (self.lm_rows + 31) // 32
        self.amax_val = torch.empty(lm_panels, L.SS_LD, dtype=torch.float32, device=dev)
        self.amax_idx = torch.empty(lm_panels, L.SS_LD, dtype=torch.int32, device=dev)
        self.logits = torch.empty(M, self.lm_rows, dtype=torch.float32, device=dev)
        self.out_val = torch.empty(M, dtype=torch.float32, device=dev)
        # status words of every kernel family this model launches, side by side so that one small copy reads them all:
        # [0] model kernels (bounds checks, step kernel waits), [1] GEMV / GEMM waits, [2], [3] tensor-parallel inboxes
        self._status_all = i32(4)
        self.status = self._status_all[0:1]
        self.inv_freq = basic.rope_inv_freq(cfg.head_dim, cfg.rope_theta, dev)
        self.ws = L.GemvWorkspace(dev, floats=max(4 << 20, 2 * cfg.d_model * 64 * M), panels=max(1 << 16, lm_panels),
                                  status=self._status_all[1:2])
        self._deq_tmp = None

    def finalize(self):
        """Size the split-k workspace from the loaded linears (call once after the weights are in place)."""
        lib = _lib.cuda_lib()
        lins = [x for x in [self.lm_head] + [d[lin] for d in self.layers for lin in LINEARS] if isinstance(x, L.WqLinear)]
        need = max(lib.b2_wq_gemv_scratch_floats(x.n, x.k, x.ks, r, M_GEMV) for x in lins for r in (2, x.rb))
        # the tensor-core path's split-k partials at its largest row count, so that the scratch never moves afterwards
        need = max(need, max(lib.b2_wq_mm_scratch_floats(x.n, x.k, 256) for x in lins))
        panels = max(x.n_panels() for x in lins)
        keep = self.ws.mm_min_rows
        self.ws = L.GemvWorkspace(self.dev, floats=max(need, 1 << 16), panels=max(panels, 1 << 10), status=self._status_all[1:2])
        self.ws.mm_min_rows = keep
        self.ws.x16_buffer(32, 128)          # allocate the staging buffer now, outside any graph capture
        self._open_step()
        return self

    def _open_step(self):
        """Build the descriptor table of the persistent step kernel (head_dim 128, 16-token pages, CUDA device)."""
        if self.step is not None:
            self.step.close()
            self.step = None
        if self.step_mode != "on" or not self._step_possible():
            return                       # "auto" builds on first use (see _step_ok)
        from ..ops.step import StepRunner
        self.step = StepRunner(self, uniform=self.step_uniform)

    def _step_possible(self) -> bool:
        # (the step kernel reads quantised weights only: a model with bf16 linears stays on the per-op kernels)
        return self.dev.type == "cuda" and self.cfg.head_dim == 128 and self.cfg.page_size == 16 and bool(self.layers) \
            and all(isinstance(d[lin], L.WqLinear) for d in self.layers for lin in LINEARS)

    def enable_step(self, on=True, uniform: Optional[bool] = None):
        """``True`` / "on": every step of up to sixteen rows runs on the persistent step kernel (its weight copies are
        built now); "auto": three to sixteen rows; ``False`` / "off": never.  ``uniform``: steps of one to eight rows use
        the work split of the nine-to-sixteen-row class too, so that a row gives the same bits in a step of any size
        (batch-invariant serving with up to sixteen rows per step); otherwise rows are bit-comparable within 1..8 and
        within 9..16.  Under tensor parallelism every rank calls it (it opens the exchange region collectively).
        Returns whether the kernel is available."""
        mode = {True: "on", False: "off"}.get(on, on)
        assert mode in ("on", "off", "auto")
        self.step_mode = mode
        self.use_step = mode != "off"
        if uniform is not None and bool(uniform) != self.step_uniform:
            self.step_uniform = bool(uniform)
            if self.step is not None:
                self.step.close()
                self.step = None
        if mode == "on" and self.step is None and self._step_possible():
            from ..ops.step import StepRunner
            self.step = StepRunner(self, uniform=self.step_uniform)
        self._graphs.clear()
        return self.step is not None or (mode == "auto" and self._step_possible())

    def _step_ok(self, m: int) -> bool:
        """The persistent kernel takes this step: the mode wants it for this many rows, the deployment has not pinned
        the tensor-core family for small steps, no KV is tiered, and the kernel is (or can now be) built."""
        if self.step_mode == "off" or m > STEP_ROWS or (self.step_mode == "auto" and m < 3):
            return False
        if (self.ws.mm_min_rows and m >= self.ws.mm_min_rows) or self._tiered_groups:
            return False
        if self.step is None:
            # "auto" on one GPU builds lazily; tensor-parallel models build through enable_step (a collective)
            if getattr(self, "world", 1) > 1 or not self._step_possible() or torch.cuda.is_current_stream_capturing():
                return False
            from ..ops.step import StepRunner
            try:
                self.step = StepRunner(self, uniform=self.step_uniform)
            except (RuntimeError, MemoryError) as e:
                # the second weight layout did not fit (a capped allocator, a nearly full GPU): stay on the per-op kernels
                self.step = None
                self.step_mode = "off"
                self.use_step = False
                import warnings
                warnings.warn(f"persistent step kernel disabled: {e}")
                return False
        return True

    def set_linear_path(self, mm_min_rows: Optional[int]):
        """Token rows from which the small-m linears run on the tcgen05 GEMM instead of the GEMV (None: the default of
        ops.linear).  The two kernels round differently, so a deployment that wants every row to be independent of the
        batch it travels in pins one path: 1 = tensor-core GEMM for every step, 33 = GEMV for every step."""
        self.ws.mm_min_rows = mm_min_rows
        self._graphs.clear()

    # ------------------------------------------------------------------------------------------------ sessions
    def new_seq(self, seq: int):
        assert 0 <= seq < self.max_seqs and seq not in self.seq_pages
        self._aid[seq] = self.pool.new_seq()
        self.seq_pages[seq] = []
        self.seq_len_host[seq] = 0
        self.seq_len[seq] = 0

    def enable_host_tier(self, window_tokens: int, batch_pages: int = 256):
        """KV pages older than ``window_tokens`` (rounded up to batches of ``batch_pages`` pages) move to pinned host
        memory; attention streams them back on a side stream.  Eager steps only (graph replays need resident KV)."""
        from .kv_tier import HostKvTier
        self.tier = HostKvTier(self, window_tokens, batch_pages)
        return self.tier

    def free_seq(self, seq: int):
        if self.tier is not None:
            self.tier.drop(seq)
        self.pool.free_seq(self._aid.pop(seq))
        self.rope_delta.pop(seq, None)
        self.seq_pages.pop(seq)
        self.seq_len_host.pop(seq)
        self.block_table[seq].fill_(-1)

    def free_pages(self) -> int:
        return self.pool.free_pages

    def reserve(self, seq: int, n_tokens: int):
        """Make sure pages exist for the first ``n_tokens`` positions of ``seq`` (rows grow lazily, as in the
        reference's KV admission, serve.rs:343-410)."""
        pages = self.seq_pages[seq]
        need = (n_tokens + self.cfg.page_size - 1) // self.cfg.page_size
        if need > self.pages_per_seq:
            raise RuntimeError("context length exceeds max_ctx")
        if need > len(pages):
            if self.pool.reserve(self._aid[seq], n_tokens) < 0:
                raise RuntimeError("KV pool exhausted")
            new = self.pool.pages(self._aid[seq])[len(pages):]
            self.block_table[seq, len(pages):need] = torch.tensor(new, dtype=torch.int32, device=self.dev)
            pages.extend(new)

    def truncate(self, seq: int, n_tokens: int):
        """Roll a sequence back to ``n_tokens`` (rejected speculative rows); pages past the end are released.  A forked
        sequence must not be rolled back below its fork point (its earlier pages are shared)."""
        if n_tokens == self.seq_len_host[seq]:
            return
        if self.tier is not None and n_tokens < self.tier.n_host_pages(seq) * self.cfg.page_size:
            raise RuntimeError(f"truncate: sequence {seq} cannot be rolled back into pages that moved to the host tier")
        self.seq_len_host[seq] = n_tokens
        self.seq_len[seq] = n_tokens
        keep = (n_tokens + self.cfg.page_size - 1) // self.cfg.page_size
        pages = self.seq_pages[seq]
        if keep < len(pages):
            self.pool.truncate(self._aid[seq], n_tokens)
            self.block_table[seq, keep:len(pages)] = -1
            del pages[keep:]

    def fork(self, src: int, dst: int):
        """``dst`` becomes a copy of ``src`` that shares its full KV pages; only a partial last page is copied
        (reference: fork_row / COW pages, m1_model.cu:1638-1716)."""
        assert dst not in self.seq_pages and 0 <= dst < self.max_seqs
        self.pool.set_len(self._aid[src], self.seq_len_host[src])
        child, cs, cd = self.pool.fork(self._aid[src])
        if child < 0:
            raise RuntimeError("KV pool exhausted")
        if cs >= 0:
            for kv in self.kv:
                kv[cd].copy_(kv[cs])
        self._aid[dst] = child
        pages = self.pool.pages(child)
        self.seq_pages[dst] = list(pages)
        self.block_table[dst].fill_(-1)
        if pages:
            self.block_table[dst, :len(pages)] = torch.tensor(pages, dtype=torch.int32, device=self.dev)
        self.seq_len_host[dst] = self.seq_len_host[src]
        self.seq_len[dst] = self.seq_len_host[src]

    def _resident_or_raise(self, seq: int, used: int, what: str):
        """Pages that live in the host tier carry a negative marker in the page list; gathering them by index would be
        an out-of-range access on the device, so such calls are refused on the host."""
        if any(p < 0 for p in self.seq_pages[seq][:used]):
            raise RuntimeError(f"{what}: sequence {seq} has KV pages in the host tier; bring them back or drop the sequence")

    def park(self, seq: int) -> Dict[str, object]:
        """Moves a sequence's KV rows to pinned host memory and frees its slot and pages.  :meth:`unpark` brings it
        back bit for bit, so a preempted or idle conversation resumes without recomputation (reference: park/unpark of
        conversations, serve.rs:616-760, and the host KV tier of m1_model.cu:1818-1905)."""
        n = self.seq_len_host[seq]
        used = (n + self.cfg.page_size - 1) // self.cfg.page_size
        self._resident_or_raise(seq, used, "park")
        idx = torch.tensor(self.seq_pages[seq][:used], dtype=torch.long, device=self.dev)
        shape = (self.cfg.n_layers, used) + tuple(self.kv[0].shape[1:])
        host_kv = torch.empty(shape, dtype=torch.bfloat16, pin_memory=True)
        for l, kv in enumerate(self.kv):
            host_kv[l].copy_(kv.index_select(0, idx), non_blocking=True)
        torch.cuda.current_stream(self.dev).synchronize()
        delta = self.rope_delta.get(seq, 0)
        self.free_seq(seq)
        return {"len": n, "kv": host_kv, "rope_delta": delta}

    def unpark(self, seq: int, blob: Dict[str, object]):
        """Restores a parked sequence into the (free) slot ``seq``."""
        self.new_seq(seq)
        n = int(blob["len"])
        if blob.get("rope_delta"):
            self.rope_delta[seq] = int(blob["rope_delta"])
        self.reserve(seq, n)
        used = (n + self.cfg.page_size - 1) // self.cfg.page_size
        idx = torch.tensor(self.seq_pages[seq][:used], dtype=torch.long, device=self.dev)
        host_kv = blob["kv"]
        for l, kv in enumerate(self.kv):
            kv.index_copy_(0, idx, host_kv[l].to(self.dev, non_blocking=True))
        self.seq_len_host[seq] = n
        self.seq_len[seq] = n

    def save_session(self, seq: int, path: str, tokens: Optional[List[int]] = None):
        """Writes the KV rows (and optionally the token history) of ``seq`` to a safetensors file so that a conversation
        survives a restart of the engine (reference: session blob, m1_model.cu snapshot / restore, serve.rs:616-760).
        The sequence stays where it is."""
        from ..utils import checkpoint as K
        n = self.seq_len_host[seq]
        used = (n + self.cfg.page_size - 1) // self.cfg.page_size
        self._resident_or_raise(seq, used, "save_session")
        idx = torch.tensor(self.seq_pages[seq][:used], dtype=torch.long, device=self.dev)
        kv = torch.stack([layer.index_select(0, idx) for layer in self.kv]).cpu()
        meta = {"format": "b200e-session-1", "len": str(n), "n_layers": str(self.cfg.n_layers), "n_kv_heads": str(self.cfg.n_kv_heads),
                "head_dim": str(self.cfg.head_dim), "page_size": str(self.cfg.page_size)}
        t = {"kv": kv, "len": torch.tensor([n], dtype=torch.int32)}
        if tokens is not None:
            t["tokens"] = torch.tensor(list(tokens), dtype=torch.int32)
        K.write_safetensors(path, t, metadata=meta)

    def load_session(self, seq: int, path: str) -> List[int]:
        """Restores a file written by :meth:`save_session` into the free slot ``seq``; returns the stored tokens."""
        from ..utils import checkpoint as K
        f = K.SafeTensorsFile(path)
        kv = f.tensor("kv").clone()
        toks = f.tensor("tokens").tolist() if "tokens" in f.keys() else []
        n = int(f.tensor("len")[0])
        f.close()
        want = (self.cfg.n_layers, (n + self.cfg.page_size - 1) // self.cfg.page_size, 2, self.cfg.n_kv_heads, self.cfg.page_size, self.cfg.head_dim)
        if tuple(kv.shape) != want:
            raise ValueError(f"session file does not match this model: {tuple(kv.shape)} vs {want}")
        self.unpark(seq, {"len": n, "kv": kv.pin_memory()})
        return toks

    def device_status(self) -> int:
        """First non-zero status word of the kernels this model launched since the last clear (0: all fine).  One
        16-byte device-to-host copy; the serving loop calls it once per step before it delivers tokens."""
        st = self._status_all.cpu().tolist()
        return next((x for x in st if x), 0)

    def recover(self):
        """After a device-side error status (bounded wait expired, bounds check): drop every sequence, clear the status
        words and the self-resetting counters, forget captured graphs.  Weights stay loaded (reference: ak_m1_recover)."""
        torch.cuda.synchronize(self.dev)
        for s in list(self.seq_pages):
            self.free_seq(s)
        self._status_all.zero_()
        self.ws.counters.zero_()
        if self.step is not None:
            self.step.reset_sync()
        self._graphs.clear()

    # ------------------------------------------------------------------------------------------------ small-m forward
    def _layers_small(self, m: int, n_groups: int):
        """Layers of one step for m <= 32 token rows already described by tok_pos / tok_seq / grp_*; h_a and ss_a
        hold the embedded tokens.  Every launch goes to the current stream (capturable)."""
        cfg, ws = self.cfg, self.ws
        h_a, h_b = self.h_a[:m], self.h_b[:m]
        parts_a = 1
        for li, d in enumerate(self.layers):
            L.gemv(d["qkv"], h_a, ws, pro=PRO_NORM, ss_in=self.ss_a, ss_parts=parts_a, norm_w=d["ln1"], eps=cfg.rms_eps,
                   out=self.qkv[:m])
            basic.rope_kvstore(self.qkv[:m], cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, self.inv_freq, self.tok_pos,
                               self.tok_seq, self.block_table, self.kv[li], self.q[:m], status=self.status,
                               rope_pos=self.rope_pos if self._use_rope_pos else None)
            if self._tiered_groups:
                self.tier.attend(li, self.q[:m], self.grp_tok0[:n_groups], self.grp_cnt[:n_groups], self.tok_pos, self.tok_seq,
                                 self._tiered_groups, self.split_keys, self.max_splits, self.part_o, self.part_ml, self.attn[:m])
            else:
                A.attn_decode(self.q[:m], self.kv[li], self.block_table, self.grp_tok0[:n_groups], self.grp_cnt[:n_groups],
                              self.tok_pos, self.tok_seq, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, self.split_keys,
                              self.max_splits, part_o=self.part_o, part_ml=self.part_ml, status=self.status, out=self.attn[:m])
            parts_b = self._row_parallel(d["o"], self.attn[:m], h_a, h_b, self.ss_b, 2 * li)
            L.gemv(d["gate_up"], h_b, ws, pro=PRO_NORM, ss_in=self.ss_b, ss_parts=parts_b, norm_w=d["ln2"],
                   eps=cfg.rms_eps, epi=EPI_SWIGLU, out=self.act[:m])
            parts_a = self._row_parallel(d["down"], self.act[:m], h_b, h_a, self.ss_a, 2 * li + 1)
        return parts_a

    def _row_parallel(self, lin, x, resid, out, ss_out, site: int):
        """Row-parallel linear + residual add + next-norm statistics (one GPU: nothing to reduce).  Returns the
        number of partial sums of squares it left in ``ss_out``."""
        L.gemv(lin, x, self.ws, epi=EPI_RESID, resid=resid, out=out, ss_out=ss_out)
        return lin.n_panels()

    def _reduce_rows(self, x: torch.Tensor) -> torch.Tensor:
        """Sum of a row-parallel partial over the tensor-parallel ranks (prefill path); identity on one GPU."""
        return x

    def _head_small(self, m: int, parts_a: int, want_logits: bool, standalone: bool = False):
        """lm_head + argmax of the rows in h_a.  ``standalone``: the call does not follow a pass through the small-m
        layers (prefill tail); vocab-parallel models then must not rely on the layers' slot re-arming."""
        cfg = self.cfg
        L.gemv(self.lm_head, self.h_a[:m], self.ws, pro=PRO_NORM, ss_in=self.ss_a, ss_parts=parts_a, norm_w=self.final_norm,
               eps=cfg.rms_eps, epi=EPI_ARGMAX, amax_val=self.amax_val, amax_idx=self.amax_idx,
               n_valid=self._lm_valid(), yf=self.logits[:m] if want_logits else None)
        lib = _lib.cuda_lib()
        check(lib.b2_argmax_final(ptr(self.amax_val), ptr(self.amax_idx), self.lm_head.n_panels(), L.SS_LD, m,
                                  ptr(self.out_ids), ptr(self.out_val), current_stream()), "b2_argmax_final")
        self._combine_argmax(m, standalone)

    def _lm_valid(self) -> int:
        return self.cfg.vocab_valid or self.cfg.vocab

    def _combine_argmax(self, m: int, standalone: bool = False):
        """Vocab-parallel models merge the per-rank winners here; nothing to do on one GPU."""

    def _full_logits(self, m: int) -> torch.Tensor:
        """fp32 logits of the last step's first ``m`` rows over the whole vocabulary (vocab-parallel models gather)."""
        return self.logits[:m].clone()

    def vocab_valid_full(self) -> int:
        return self.cfg.vocab_valid or self.cfg.vocab

    def forward_rows(self, ids: List[int], seqs: List[int], want_logits: bool = False):
        """Eager step over explicit rows: ``ids[i]`` is appended to sequence ``seqs[i]`` (rows of one sequence must be
        adjacent: they form a verify group).  Returns the argmax token of every row (and fp32 logits on request)."""
        m = len(ids)
        assert 1 <= m <= self.max_rows
        pos, g0, gc = [], [], []
        nxt = dict(self.seq_len_host)
        for i, s in enumerate(seqs):
            if i == 0 or seqs[i - 1] != s:
                g0.append(i); gc.append(0)
            gc[-1] += 1
            assert gc[-1] <= 8
            pos.append(nxt[s]); nxt[s] += 1
        for s, n in nxt.items():
            self.reserve(s, n)
        hb = self._rowbuf_host
        hb[0, :m] = torch.tensor(ids, dtype=torch.int32); hb[1, :m] = torch.tensor(pos, dtype=torch.int32)
        hb[2, :m] = torch.tensor(seqs, dtype=torch.int32)
        hb[3, :len(g0)] = torch.tensor(g0, dtype=torch.int32); hb[4, :len(g0)] = torch.tensor(gc, dtype=torch.int32)
        self._use_rope_pos = any(self.rope_delta.get(s, 0) for s in seqs)
        if self._use_rope_pos:
            hb[5, :m] = torch.tensor([p + self.rope_delta.get(s, 0) for p, s in zip(pos, seqs)], dtype=torch.int32)
        self._rowbuf.copy_(hb)                     # blocking copy from pinned memory: the host buffer is reused next step
        self._tiered_groups = {}
        if self.tier is not None:
            for gi, i in enumerate(g0):
                s = seqs[i]
                if self.tier.n_host_pages(s):
                    first, cnt = self._tiered_groups.get(s, (gi, 0))
                    self._tiered_groups[s] = (first, cnt + 1)
        if self.row_graphs and not self._tiered_groups and not self._use_rope_pos:
            self._rows_graph(m, len(g0), want_logits).replay()
        else:
            self._rows_body(m, len(g0), want_logits)
        self._tiered_groups = {}
        touched = sorted(set(seqs))
        for s in touched:
            self.seq_len_host[s] = nxt[s]
        self.seq_len[torch.tensor(touched, dtype=torch.long, device=self.dev)] = \
            torch.tensor([nxt[s] for s in touched], dtype=torch.int32, device=self.dev)
        if self.tier is not None:
            for s in set(seqs):
                self.tier.maybe_offload(s)
        return self.out_ids[:m].clone(), (self._full_logits(m) if want_logits else None)

    def _rows_body(self, m: int, n_groups: int, want_logits: bool):
        if self._step_ok(m):
            self.step.launch(m, n_groups, want_logits)
            return
        basic.embed(self.ids[:m], self.embed, self.ss_a, status=self.status, out=self.h_a[:m])
        parts = self._layers_small(m, n_groups)
        self._head_small(m, parts, want_logits)

    def _rows_graph(self, m: int, n_groups: int, want_logits: bool) -> torch.cuda.CUDAGraph:
        """CUDA graph of one eager-shaped step (rows, groups and positions are read from device buffers, so one graph
        serves every step of the same shape: verify blocks, drafter steps, mixed batches)."""
        key = ("rows", m, n_groups, want_logits)
        g = self._graphs.get(key)
        if g is None:
            st = torch.cuda.Stream(device=self.dev)
            st.wait_stream(torch.cuda.current_stream(self.dev))
            with torch.cuda.stream(st):
                self._rows_body(m, n_groups, want_logits)          # warm-up: the step is idempotent on its buffers
            torch.cuda.current_stream(self.dev).wait_stream(st)
            torch.cuda.synchronize(self.dev)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                self._rows_body(m, n_groups, want_logits)
            self._graphs[key] = g
        return g

    # ------------------------------------------------------------------------------------------------ prefill
    def _linear_big(self, lin: L.WqLinear, x: torch.Tensor) -> torch.Tensor:
        """bf16 [T, n] = x @ dequant(W)^T for a prefill chunk.  Up to 256 rows run on the mixed-bit tensor-core GEMM
        (weights dequantised inside the kernel, one pass over the packed weights); longer chunks dequantise to a bf16
        buffer first and use the plain bf16 GEMM."""
        if x.shape[0] <= 256 and self.prefill_mm:
            return L.mm(lin, x.contiguous(), self.ws)
        from ..ops import gemm as G
        return G.wq_linear(lin, x, self)

    def _row_linear_big(self, lin, x: torch.Tensor) -> torch.Tensor:
        """A row-parallel linear of a prefill chunk, summed over the tensor-parallel ranks (one GPU: the plain linear)."""
        return self._reduce_rows(self._linear_big(lin, x))

    def _prefill_split_for(self, kv_len: int) -> int:
        """KV split size of a prefill chunk: the base size, doubled until at most 64 splits cover the context (keeps the
        partial-result buffers bounded at long context)."""
        s = self.prefill_split
        while (kv_len + s - 1) // s > 64:
            s *= 2
        return s

    def prefill(self, seq: int, ids: torch.Tensor, want_logits: bool = False, image_rows: Optional[torch.Tensor] = None,
                image_pad_id: Optional[int] = None, rope_pos3: Optional[torch.Tensor] = None,
                pair_axis: Optional[torch.Tensor] = None, rope_next: Optional[int] = None):
        """Chunked prefill of ``ids`` (1-D int tensor) appended to ``seq``; returns the greedy next token (int).
        ``image_rows`` (bf16 [n, d_model], from the vision encoder) replace the embedding rows of the ``image_pad_id``
        tokens, in order (reference: m1_model.cu:2821-2834)."""
        cfg = self.cfg
        ids = ids.to(device=self.dev, dtype=torch.int32)
        T = ids.numel()
        # multi-axis rotary positions (int32 [3, T], serve.vision.mrope_positions) with the axis of every frequency pair;
        # rope_next = the running position after the prompt: later tokens rotate by KV position + (rope_next - length)
        self._rope3 = None
        if rope_pos3 is not None:
            assert self.seq_len_host[seq] == 0 and pair_axis is not None and tuple(rope_pos3.shape) == (3, T)
            self._rope3 = (rope_pos3.to(self.dev, torch.int32).contiguous(), pair_axis.to(self.dev))
            if rope_next is not None:
                self.rope_delta[seq] = int(rope_next) - T
        self._sub_rows = self._sub_index = None
        if image_rows is not None:
            is_img = ids == image_pad_id
            assert int(is_img.sum()) == image_rows.shape[0], "image rows do not match the placeholders"
            self._sub_rows = image_rows.to(self.dev, torch.bfloat16).contiguous()
            self._sub_index = torch.where(is_img, torch.cumsum(is_img.to(torch.int32), 0, dtype=torch.int32) - 1,
                                          torch.full_like(ids, -1)).contiguous()
        start = self.seq_len_host[seq]
        self.reserve(seq, start + T)
        last = None
        cuts = list(range(0, T, self.prefill_chunk)) + [T]
        if self._rope3 is not None or self._sub_rows is not None:
            # image rows and multi-axis positions exist in the large-m path only (more than 8 rows per chunk): a short
            # tail borrows 16 rows from the chunk before it
            assert T > 8 and self.prefill_chunk > 24, "prompts with images need more than 8 tokens"
            if len(cuts) > 2 and T - cuts[-2] <= 8:
                cuts[-2] -= 16
        for c0, c1 in zip(cuts[:-1], cuts[1:]):
            self._sub_slice = (c0, c1)
            last = self._prefill_chunk(seq, ids[c0:c1], start + c0, final=(c1 == T), want_logits=want_logits)
            self.seq_len_host[seq] = start + c1
            self.seq_len[seq] = start + c1
            if self.tier is not None:
                self.tier.maybe_offload(seq)
        self._sub_rows = self._sub_index = None
        self._rope3 = None
        return last

    def _chunk_input(self, ids: torch.Tensor, sub_i: Optional[torch.Tensor]) -> torch.Tensor:
        """Input rows of the first layer for a prefill chunk of more than eight tokens (bf16 [T, d_model])."""
        return basic.embed(ids, self.embed, None, sub_rows=self._sub_rows if sub_i is not None else None, sub_index=sub_i,
                           status=self.status)

    def _prefill_chunk(self, seq: int, ids: torch.Tensor, pos0: int, final: bool, want_logits: bool):
        cfg, dev = self.cfg, self.dev
        T = ids.numel()
        if T <= 8:
            out, logits = self.forward_rows(ids.tolist(), [seq] * T, want_logits)
            if self.hidden_sink is not None:
                self.hidden_sink(pos0, self.h_a[:T])
            # forward_rows advanced the host length itself; undo so prefill() owns the bookkeeping
            return (int(out[-1]), logits[-1] if logits is not None else None) if final else None
        from ..ops import gemm as G
        pos = torch.arange(pos0, pos0 + T, dtype=torch.int32, device=dev)
        seqv = torch.full((T,), seq, dtype=torch.int32, device=dev)
        sub_i = None
        if getattr(self, "_sub_index", None) is not None:
            sub_i = self._sub_index[self._sub_slice[0]:self._sub_slice[1]].contiguous()
        h = self._chunk_input(ids, sub_i)
        q = torch.empty(T, cfg.q_dim, dtype=torch.bfloat16, device=dev)
        delta = None
        tiered = self.tier is not None and self.tier.n_host_pages(seq) > 0
        if tiered:
            pg0, pgc, _, _ = A.prefill_groups(T, pos0, seq, dev)
            p_splits = (pos0 + T + self.prefill_split - 1) // self.prefill_split
            p_o = torch.empty(T, cfg.n_heads, p_splits, cfg.head_dim, dtype=torch.float32, device=dev)
            p_ml = torch.empty(T, cfg.n_heads, p_splits, 2, dtype=torch.float32, device=dev)
            p_out = torch.empty(T, cfg.q_dim, dtype=torch.bfloat16, device=dev)
        for li, d in enumerate(self.layers):
            if delta is None:
                x = basic.rmsnorm(h, d["ln1"], cfg.rms_eps)
            else:
                x, h = basic.rmsnorm(delta, d["ln1"], cfg.rms_eps, resid=h)
            qkv = self._linear_big(d["qkv"], x)
            if getattr(self, "_rope3", None) is not None:
                r3 = self._rope3[0][:, self._sub_slice[0]:self._sub_slice[1]].contiguous()
                basic.rope_kvstore_m(qkv, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, self.inv_freq, pos, r3, self._rope3[1], seqv,
                                     self.block_table, self.kv[li], q, status=self.status)
            else:
                rp = pos + self.rope_delta[seq] if self.rope_delta.get(seq, 0) else None
                basic.rope_kvstore(qkv, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, self.inv_freq, pos, seqv, self.block_table,
                                   self.kv[li], q, status=self.status, rope_pos=rp)
            if tiered:
                a = self.tier.attend(li, q, pg0, pgc, pos, seqv, {seq: (0, pg0.numel())}, self.prefill_split, p_splits, p_o, p_ml, p_out,
                                     shared_kv=True)
            else:
                a = A.attn_prefill(q, self.kv[li], self.block_table, seq, pos0, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim,
                                   status=self.status, split_keys=self._prefill_split_for(pos0 + T))
            o = self._row_linear_big(d["o"], a)
            x, h = basic.rmsnorm(o, d["ln2"], cfg.rms_eps, resid=h)
            gu = self._linear_big(d["gate_up"], x)
            act = basic.swiglu_interleaved(gu)
            delta = self._row_linear_big(d["down"], act)
        if self.hidden_sink is not None:
            # the residual stream after the last layer, every row of the chunk (what an MTP head reads as its context)
            self.hidden_sink(pos0, (h.float() + delta.float()).to(torch.bfloat16))
        if not final:
            return None
        hl = (h[-1:].float() + delta[-1:].float()).to(torch.bfloat16)
        self.h_a[:1] = hl
        basic.sumsq(self.h_a[:1], self.ss_a)
        self._head_small(1, 1, want_logits, standalone=True)
        return int(self.out_ids[0]), (self._full_logits(1)[0] if want_logits else None)

    # ------------------------------------------------------------------------------------------------ decode
    def _decode_body(self, seqs: List[int]):
        """One decode step for ``seqs`` (one row each): the token of the previous step is the input."""
        m = len(seqs)
        if self._step_ok(m):
            self.step.launch(m, m, False, decode=True)
            return
        lib = _lib.cuda_lib()
        check(lib.b2_decode_step_prep(m, ptr(self.last_ids), ptr(self.ids), ptr(self.seq_len), ptr(self.tok_pos),
                                      ptr(self.tok_seq), ptr(self._slot_seq), current_stream()), "b2_decode_step_prep")
        basic.embed(self.ids[:m], self.embed, self.ss_a, status=self.status, out=self.h_a[:m])
        parts = self._layers_small(m, m)
        self._head_small(m, parts, False)
        self.last_ids[:m].copy_(self.out_ids[:m])

    def decode_setup(self, seqs: List[int], first_tokens: List[int], n_steps: int):
        """Prepare device state for ``n_steps`` graph-replayed decode steps of ``seqs``."""
        m = len(seqs)
        t = lambda x: torch.tensor(x, dtype=torch.int32, device=self.dev)
        self._slot_seq[:m] = t(seqs)
        self.last_ids[:m] = t(first_tokens)
        self.grp_tok0[:m] = torch.arange(m, dtype=torch.int32, device=self.dev)
        self.grp_cnt[:m] = 1
        for s in seqs:
            self.reserve(s, self.seq_len_host[s] + n_steps)
        self._decode_seqs = list(seqs)

    def decode_graph(self) -> torch.cuda.CUDAGraph:
        key = tuple(self._decode_seqs)
        g = self._graphs.get(key)
        if g is None:
            # warm-up on a side stream (lazy module loads, attribute calls), restoring the state it advanced
            saved = (self.seq_len.clone(), self.last_ids.clone())
            st = torch.cuda.Stream(device=self.dev)
            st.wait_stream(torch.cuda.current_stream(self.dev))
            with torch.cuda.stream(st):
                self._decode_body(self._decode_seqs)
            torch.cuda.current_stream(self.dev).wait_stream(st)
            torch.cuda.synchronize(self.dev)
            self.seq_len.copy_(saved[0]); self.last_ids.copy_(saved[1])
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                self._decode_body(self._decode_seqs)
            self.seq_len.copy_(saved[0]); self.last_ids.copy_(saved[1])
            self._graphs[key] = g
        return g

    def decode_steps(self, n_steps: int, collect: bool = True) -> Optional[torch.Tensor]:
        """Replay the decode graph ``n_steps`` times; returns the produced tokens ``[n_steps, batch]``."""
        g = self.decode_graph()
        m = len(self._decode_seqs)
        outs = torch.empty(n_steps, m, dtype=torch.int32, device=self.dev) if collect else None
        for i in range(n_steps):
            g.replay()
            if collect:
                outs[i].copy_(self.out_ids[:m])
        for s in self._decode_seqs:
            self.seq_len_host[s] += n_steps
        return outs

    def generate_greedy(self, seq: int, prompt: torch.Tensor, n_new: int) -> torch.Tensor:
        """Prefill ``prompt`` into ``seq`` and decode ``n_new`` tokens greedily; returns them as a CPU tensor."""
        first, _ = self.prefill(seq, prompt)
        if n_new == 1:
            return torch.tensor([first])
        self.decode_setup([seq], [first], n_new - 1)
        outs = self.decode_steps(n_new - 1)
        torch.cuda.synchronize(self.dev)
        st = int(self.status.item())
        if st != 0 or int(self.ws.status.item()) != 0:
            raise _lib.B2Error("decode", st or int(self.ws.status.item()))
        return torch.cat([torch.tensor([first]), outs[:, 0].cpu().long()])

    def step_host(self, tok_in: torch.Tensor, tok_out: torch.Tensor):
        """Public step API: feed this step's input tokens from pinned host memory, run one decode step for the
        sequences given to :meth:`decode_setup`, read the produced tokens back to pinned host memory."""
        m = len(self._decode_seqs)
        self.last_ids[:m].copy_(tok_in, non_blocking=True)
        self.decode_graph().replay()
        tok_out.copy_(self.out_ids[:m], non_blocking=True)
        torch.cuda.current_stream(self.dev).synchronize()
        for s in self._decode_seqs:
            self.seq_len_host[s] += 1

    def launches_per_step(self, batch: int = 1) -> int:
        """Kernels of this package launched by one decode step: one persistent kernel, or (per-op path) prep, embed,
        7 per layer, lm_head, argmax."""
        if self._step_ok(batch):
            return 1
        return 2 + 7 * self.cfg.n_layers + 2
