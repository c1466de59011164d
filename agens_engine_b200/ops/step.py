"""Launcher of the persistent decode-step kernel (``csrc/kernels/sm100/step_kernel.cu``).

One cooperative launch runs a whole decode or verify step (up to sixteen token rows) of a dense model: every layer,
the lm_head and the argmax, on one GPU or as one rank of a tensor-parallel group.  Python only assembles the argument
block; the table of per-layer weight descriptors lives in device memory and is built once.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _lib
from .._lib import check, current_stream, ptr

MAX_ROWS = 16          # rows of one step
SMALL_ROWS = 8         # steps of up to this many rows stage k slices of SLICE_K inputs, larger steps half of that
SLICE_K = 5120
MAX_TP = 8
N_WARPS = 15


class StepLinear(C.Structure):
    _fields_ = [
        ("wq", C.c_void_p),
        ("n", C.c_int), ("k", C.c_int), ("bits", C.c_int), ("group", C.c_int),
        ("npan", C.c_int), ("nbat", C.c_int),
        ("wbatch", C.c_int), ("szb", C.c_int), ("blk", C.c_int),
        ("ks", C.c_int), ("cps", C.c_int), ("fmax", C.c_int), ("pad", C.c_int),
    ]


class StepLayer(C.Structure):
    _fields_ = [
        ("qkv", StepLinear), ("o", StepLinear), ("gate_up", StepLinear), ("down", StepLinear),
        ("ln1", C.c_void_p), ("ln2", C.c_void_p), ("kv_pool", C.c_void_p), ("pad", C.c_void_p),
    ]


class StepArgs(C.Structure):
    _fields_ = [
        ("layers", C.c_void_p), ("n_layers", C.c_int),
        ("lm_head", StepLinear),
        ("final_norm", C.c_void_p), ("embed", C.c_void_p),
        ("vocab", C.c_int), ("d_model", C.c_int), ("hq", C.c_int), ("hkv", C.c_int), ("ffn", C.c_int),
        ("eps", C.c_float), ("lm_valid", C.c_int), ("lm_offset", C.c_int),
        ("n_rows", C.c_int), ("slice_k", C.c_int),
        ("ids", C.c_void_p), ("tok_pos", C.c_void_p), ("tok_seq", C.c_void_p),
        ("rope_pos", C.c_void_p),
        ("grp_tok0", C.c_void_p), ("grp_cnt", C.c_void_p), ("n_groups", C.c_int),
        ("tree_mask", C.c_void_p),
        ("block_table", C.c_void_p), ("bt_ld", C.c_int), ("n_pages", C.c_int),
        ("inv_freq", C.c_void_p),
        ("split_keys", C.c_int), ("max_splits", C.c_int), ("scale_log2", C.c_float),
        ("slot_seq", C.c_void_p), ("last_ids", C.c_void_p), ("seq_len", C.c_void_p),
        ("part", C.c_void_p), ("tile_scratch", C.c_void_p), ("xq", C.c_void_p), ("xg", C.c_void_p), ("psq", C.c_void_p), ("attn_ctr", C.c_void_p),
        ("h", C.c_void_p), ("q", C.c_void_p), ("attn", C.c_void_p), ("act", C.c_void_p),
        ("part_o", C.c_void_p), ("part_ml", C.c_void_p),
        ("amax_val", C.c_void_p), ("amax_idx", C.c_void_p),
        ("logits", C.c_void_p), ("ld_logits", C.c_long),
        ("out_ids", C.c_void_p), ("out_val", C.c_void_p),
        ("sync", C.c_void_p), ("status", C.c_void_p),
        ("timeout_ns", C.c_ulonglong),
        ("tp_rank", C.c_int), ("tp_size", C.c_int),
        ("xreg", C.c_void_p * MAX_TP),
        ("x_off", C.c_long * 2), ("x_amax", C.c_long),
        ("skip_push", C.c_int),
        ("trace", C.c_void_p),
    ]


_declared = False


def _lib_step():
    global _declared
    lib = _lib.cuda_lib()
    if not _declared:
        vp, i = C.c_void_p, C.c_int
        _lib.declare_optional(lib, "b2_step_linear", [vp, i, i, i, i, i, i, C.POINTER(StepLinear)], i)
        _lib.declare_optional(lib, "b2_step_part_floats", [C.POINTER(StepLinear), i], C.c_long)
        _lib.declare_optional(lib, "b2_step_smem_bytes", [], i)
        _lib.declare_optional(lib, "b2_step_grid", [C.POINTER(i)], i)
        _lib.declare_optional(lib, "b2_step_launch", [C.POINTER(StepArgs), i, vp], i)
        _lib.declare_optional(lib, "b2_wq_fm_to_fi", [vp, i, i, i, i, vp, vp], i)
        if lib.b2_step_args_bytes() != C.sizeof(StepArgs) or lib.b2_step_layer_bytes() != C.sizeof(StepLayer):
            raise RuntimeError("ops/step.py and step_kernel.cuh disagree about the argument structures")
        _declared = True
    return lib


def to_fi(lin) -> torch.Tensor:
    """The linear's weights in the integer-MMA layout of the step kernel (``wq_tools.cu``: FI), converted on the
    device from the FM buffer.  Same size as the FM buffer: a model that runs both the step kernel and the per-op /
    prefill kernels holds its quantised weights twice (the reference's dual-layout mode does the same for its W4H
    copies, kernels/src/w4h.cu:957-968)."""
    lib = _lib_step()
    fi = torch.empty_like(lin.wq)
    with torch.cuda.device(lin.wq.device):
        check(lib.b2_wq_fm_to_fi(ptr(lin.wq), lin.n, lin.k, lin.bits, lin.group, ptr(fi), current_stream()), "b2_wq_fm_to_fi")
    return fi


def step_linear(lin, ncta: int, wq: Optional[torch.Tensor] = None, slice_k: int = SLICE_K) -> StepLinear:
    lib = _lib_step()
    out = StepLinear()
    check(lib.b2_step_linear(ptr(lin.wq if wq is None else wq), lin.n, lin.k, lin.bits, lin.group, ncta, slice_k, C.byref(out)),
          "b2_step_linear")
    return out


class _Geometry:
    """Descriptor table of every linear for one k slice: steps of up to SMALL_ROWS rows use the table cut for SLICE_K,
    larger steps the one cut for half of it.  Both tables point at the same weights."""

    def __init__(self, runner, slice_k: int, rows: int):
        lib = _lib_step()
        model = runner.model
        L = len(model.layers)
        self.slice_k, self.rows = slice_k, rows
        table = (StepLayer * max(L, 1))()
        need = 0
        i = 0
        for l, d in enumerate(model.layers):
            for name in ("qkv", "o", "gate_up", "down"):
                sl = step_linear(d[name], runner.ncta, runner._fi[i], slice_k)
                i += 1
                setattr(table[l], name, sl)
                need = max(need, lib.b2_step_part_floats(C.byref(sl), rows))
            table[l].ln1, table[l].ln2 = ptr(d["ln1"]), ptr(d["ln2"])
            table[l].kv_pool = ptr(model.kv[l])
        self.lm = step_linear(model.lm_head, runner.ncta, runner._fi[i], slice_k)
        self.part_floats = max(need, lib.b2_step_part_floats(C.byref(self.lm), rows))
        self.table = torch.frombuffer(bytearray(bytes(table)), dtype=torch.uint8).to(model.dev)
        self.host = table                 # geometry of the row-parallel linears (exchange-region sizing)

    def exchange_floats(self, world: int, d_model: int):
        if not len(self.host) or not self.table.numel():
            return 0, 0
        so, sd = self.host[0].o, self.host[0].down
        return world * so.ks * so.fmax * self.rows * d_model, world * sd.ks * sd.fmax * self.rows * d_model


class StepRunner:
    """Owns the descriptor table and the workspaces of the step kernel for one model instance."""

    def __init__(self, model, timeout_s: float = 2.0, max_rows: int = MAX_ROWS, uniform: bool = False):
        lib = _lib_step()
        self.model = model
        cfg, dev = model.cfg, model.dev
        if cfg.head_dim != 128 or cfg.page_size != 16:
            raise ValueError("the step kernel is built for head_dim 128 and 16-token pages")
        if not 1 <= max_rows <= MAX_ROWS:
            raise ValueError(f"the step kernel runs 1..{MAX_ROWS} rows")
        n = C.c_int(0)
        with torch.cuda.device(dev):
            check(lib.b2_step_grid(C.byref(n)), "b2_step_grid")
        self.ncta = n.value
        self.max_rows = max_rows
        self.world = getattr(model, "world", 1)
        self.rank = getattr(model, "rank", 0)
        # FI copies of every linear (kept alive here), in table order
        self._fi = [to_fi(d[name]) for d in model.layers for name in ("qkv", "o", "gate_up", "down")]
        self._fi.append(to_fi(model.lm_head))
        # uniform: one work split (that of the large class) for every step, so that rows are bit-comparable across sizes
        self.uniform = uniform and max_rows > SMALL_ROWS
        if self.uniform:
            self.geo = [_Geometry(self, SLICE_K // 2, max_rows)] * 2
        else:
            self.geo = [_Geometry(self, SLICE_K, min(max_rows, SMALL_ROWS))]
            if max_rows > SMALL_ROWS:
                self.geo.append(_Geometry(self, SLICE_K // 2, max_rows))
        f32 = lambda *s: torch.empty(*s, dtype=torch.float32, device=dev)
        self.part = f32(max(max(g.part_floats for g in self.geo), 1024))
        self.tile_scratch = f32(self.ncta * N_WARPS * 2 * MAX_ROWS * 32) if max_rows > SMALL_ROWS else None
        # staged activations of the widest linear input (fixed-point limbs, group scalars) and the rows' sums of squares
        kmax = max([cfg.d_model, cfg.q_dim, cfg.ffn] + [d[name].k for d in model.layers[:1] for name in ("qkv", "o", "gate_up", "down")])
        self.xq = torch.zeros((kmax // 128) * 4096, dtype=torch.uint8, device=dev)
        self.xg = f32((kmax // 64) * 16 * 2).zero_()
        self.psq = f32(MAX_ROWS * (cfg.d_model // 128)).zero_()
        self.attn_ctr = torch.zeros(max(len(model.layers), 1), dtype=torch.int32, device=dev)
        self.amax_val = f32(self.ncta, MAX_ROWS)
        self.amax_idx = torch.empty(self.ncta, MAX_ROWS, dtype=torch.int32, device=dev)
        self.sync = torch.zeros(64, dtype=torch.int32, device=dev)
        self.status = model.status
        self.timeout_ns = int(timeout_s * 1e9)
        self.skip_push = False
        self.region = None
        self.x_off = (0, 0)
        self.x_amax = 0
        if self.world > 1:
            self._open_region()
        self.launches = 0
        self.trace = None            # int64 CUDA tensor; only a library built with -DB2_STEP_TRACE writes to it

    def _open_region(self):
        """Exchange region of this rank, mapped by every peer: [counter | o_proj partials | down partials | argmax]."""
        import torch.distributed as dist
        from ..parallel.symm import SymmetricInbox
        m, w = self.model, self.world
        d = m.cfg.d_model
        n_o = max(g.exchange_floats(w, d)[0] for g in self.geo) if len(m.layers) else 0
        n_d = max(g.exchange_floats(w, d)[1] for g in self.geo) if len(m.layers) else 0
        head = 64
        self.x_off = (head, head + n_o)
        self.x_amax = head + n_o + n_d
        total = self.x_amax + w * MAX_ROWS * 2
        per = (total + w - 1) // w
        per = (per + 3) // 4 * 4
        self.region = SymmetricInbox(self.rank, w, per, 1, m.dev)
        lib = _lib.cuda_lib()
        with torch.cuda.device(m.dev):
            check(lib.b2_fill_u32(self.region.ptrs[self.rank], 0, per * w, current_stream()), "b2_fill_u32")
            torch.cuda.synchronize(m.dev)
        dist.barrier()

    def _args(self, m: int, n_groups: int, want_logits: bool, decode: bool) -> StepArgs:
        md, cfg = self.model, self.model.cfg
        a = StepArgs()
        geo = self.geo[1 if m > SMALL_ROWS else 0]
        a.layers, a.n_layers = ptr(geo.table), len(md.layers)
        a.lm_head = geo.lm
        a.slice_k = geo.slice_k
        a.tile_scratch = ptr(self.tile_scratch)
        a.xq, a.xg, a.psq = ptr(self.xq), ptr(self.xg), ptr(self.psq)
        a.attn_ctr = ptr(self.attn_ctr)
        a.final_norm, a.embed = ptr(md.final_norm), ptr(md.embed)
        a.vocab, a.d_model, a.hq, a.hkv, a.ffn = md.embed.shape[0], cfg.d_model, cfg.n_heads, cfg.n_kv_heads, cfg.ffn
        a.eps = cfg.rms_eps
        a.lm_valid = md._lm_valid()
        a.lm_offset = self.rank * getattr(md, "vocab_shard", 0) if self.world > 1 else 0
        a.n_rows = m
        a.ids, a.tok_pos, a.tok_seq = ptr(md.ids), ptr(md.tok_pos), ptr(md.tok_seq)
        a.rope_pos = ptr(md.rope_pos) if (md._use_rope_pos and not decode) else 0
        a.grp_tok0, a.grp_cnt, a.n_groups = ptr(md.grp_tok0), ptr(md.grp_cnt), n_groups
        a.tree_mask = 0
        a.block_table, a.bt_ld, a.n_pages = ptr(md.block_table), md.block_table.stride(0), md.n_pages
        a.inv_freq = ptr(md.inv_freq)
        a.split_keys, a.max_splits = md.split_keys, md.max_splits
        a.scale_log2 = (cfg.head_dim ** -0.5) * 1.4426950408889634
        if decode:
            a.slot_seq, a.last_ids, a.seq_len = ptr(md._slot_seq), ptr(md.last_ids), ptr(md.seq_len)
        a.part, a.h, a.q, a.attn, a.act = ptr(self.part), ptr(md.h_a), ptr(md.q), ptr(md.attn), ptr(md.act)
        a.part_o, a.part_ml = ptr(md.part_o), ptr(md.part_ml)
        a.amax_val, a.amax_idx = ptr(self.amax_val), ptr(self.amax_idx)
        if want_logits:
            a.logits, a.ld_logits = ptr(md.logits), md.logits.stride(0)
        a.out_ids, a.out_val = ptr(md.out_ids), ptr(md.out_val)
        a.sync, a.status = ptr(self.sync), ptr(self.status)
        a.timeout_ns = self.timeout_ns
        a.tp_rank, a.tp_size = self.rank, self.world
        if self.region is not None:
            for r in range(self.world):
                a.xreg[r] = self.region.ptrs[r]
            a.x_off[0], a.x_off[1] = self.x_off
            a.x_amax = self.x_amax
        a.skip_push = 1 if self.skip_push else 0
        a.trace = ptr(self.trace)
        return a

    def launch(self, m: int, n_groups: int, want_logits: bool = False, decode: bool = False):
        """One step on the current stream (capturable).  ``decode``: rows come from ``last_ids`` / ``seq_len`` of the
        model's decode slots and both advance on the device."""
        assert 1 <= m <= self.max_rows
        lib = _lib_step()
        a = self._args(m, n_groups, want_logits, decode)
        with torch.cuda.device(self.model.dev):
            check(lib.b2_step_launch(C.byref(a), self.ncta, current_stream()), "b2_step_launch")
        self.launches += 1

    def reset_sync(self):
        """After a failed step (status word set): put the barrier counters back to zero on this rank."""
        self.sync.zero_()
        self.attn_ctr.zero_()
        if self.region is not None:
            lib = _lib.cuda_lib()
            with torch.cuda.device(self.model.dev):
                check(lib.b2_fill_u32(self.region.ptrs[self.rank], 0, 64, current_stream()), "b2_fill_u32")

    def close(self):
        if self.region is not None:
            self.region.close()
            self.region = None
