"""Tensor-parallel dense decoder: one process per GPU, weights sharded, collectives fused into the kernels.

Sharding (reference rules: ``crates/agens-cli/src/m1.rs:41-98``): q/k/v and gate/up are column parallel (heads and FFN
features split), o_proj and down_proj are row parallel, the lm_head is vocab parallel, embeddings and norms are
replicated.  On the decode path the two row-parallel linears of a layer run as ONE kernel each: the GEMV epilogue
pushes its partial into every rank's inbox over NVLink, sums all ranks in rank order, adds the residual and leaves the
next norm's statistics (``EPI_TP_RESID`` in ``wq_gemv.cu``) -- no NCCL call and no separate all-reduce launch.  The
lm_head produces per-rank (value, index) winners that are exchanged and merged by ``b2_comm_argmax_combine``.
Prefill chunks reduce their row-parallel outputs with the two-shot push kernels (reduce-scatter + all-gather over the
same symmetric memory); NCCL is used by the ``use_nccl_decode`` baseline only.
"""
from __future__ import annotations

import ctypes as C
import os
import dataclasses
from typing import Optional

import torch
import torch.distributed as dist

from .. import _lib
from .._lib import EPI_TP_RESID, check, current_stream, ptr
from ..models.config import LINEARS, ModelConfig
from ..models.dense import M_GEMV, M_ROWS, DenseModel
from ..ops import linear as L
from ..utils import quant
from .symm import SymmetricInbox


def local_config(cfg: ModelConfig, world: int) -> ModelConfig:
    assert cfg.n_heads % world == 0 and cfg.n_kv_heads % world == 0 and cfg.ffn % (world * 128) == 0
    return dataclasses.replace(cfg, name=f"{cfg.name}/tp{world}", n_heads=cfg.n_heads // world,
                               n_kv_heads=cfg.n_kv_heads // world, ffn=cfg.ffn // world)


def _pad32(n: int) -> int:
    return (n + 31) // 32 * 32


class TpDenseModel(DenseModel):
    def __init__(self, cfg: ModelConfig, device, rank: int, world: int, use_nccl_decode: bool = False, **kw):
        self.full_cfg, self.rank, self.world = cfg, rank, world
        self.vocab_shard = (cfg.vocab + world - 1) // world
        self.use_nccl_decode = use_nccl_decode
        super().__init__(local_config(cfg, world), device, lm_rows=_pad32(self.vocab_shard), **kw)
        n_sites = 2 * cfg.n_layers + 1
        self.inbox = SymmetricInbox(rank, world, M_GEMV * cfg.d_model, n_sites, self.dev, status=self._status_all[2:3])
        self.n_sites = n_sites
        self.idx_off = torch.full((self.max_rows,), rank * self.vocab_shard, dtype=torch.int32, device=self.dev)
        self.skip_push_site = -1     # test hook: the call site whose push this rank drops
        from .comm import PushComm
        self._gather_inbox = SymmetricInbox(rank, world, 8 * self.lm_rows, 3, self.dev,
                                            status=self._status_all[3:4])                       # logits / winners exchange
        self._gather = PushComm(self._gather_inbox)
        self._prefill_inbox = self._prefill_comm = None      # opened by the first prefill chunk (collective)
        self._fused_inbox = self._fused_comm = None          # inbox of the fused GEMM + reduce-scatter (first long chunk)
        self.fused_prefill = os.environ.get("B200E_TP_FUSED_PREFILL", "1") == "1"

    # ------------------------------------------------------------------------------------------------ weights
    @staticmethod
    def random_init(cfg: ModelConfig, device, seed: int, rank: int, world: int, **kw) -> "TpDenseModel":
        m = TpDenseModel(cfg, device, rank, world, **kw)
        lc = m.cfg
        shapes = lc.linear_shapes()
        g = torch.Generator(device=m.dev).manual_seed(seed)     # replicated tensors: same seed on every rank
        for l in range(cfg.n_layers):
            d = {}
            for i, lin in enumerate(LINEARS):
                n, k = shapes[lin]
                d[lin] = L.WqLinear.random(n, k, cfg.bits_of(l, lin), cfg.group, m.dev,
                                           seed=(seed * 1000003 + l * 8 + i) * 64 + rank)
            d["ln1"] = (1.0 + 0.05 * torch.randn(cfg.d_model, device=m.dev, generator=g)).to(torch.bfloat16)
            d["ln2"] = (1.0 + 0.05 * torch.randn(cfg.d_model, device=m.dev, generator=g)).to(torch.bfloat16)
            m.layers.append(d)
        m.embed = (torch.randn(cfg.vocab, cfg.d_model, device=m.dev, generator=g) * 0.02).to(torch.bfloat16)
        m.final_norm = (1.0 + 0.05 * torch.randn(cfg.d_model, device=m.dev, generator=g)).to(torch.bfloat16)
        m.lm_head = L.WqLinear.random(m.lm_rows, cfg.d_model, cfg.lm_head_bits, cfg.group, m.dev,
                                      seed=(seed * 1000003 + 999983) * 64 + rank)
        return m.finalize()

    @staticmethod
    def from_oracle(ow, device, rank: int, world: int, **kw) -> "TpDenseModel":
        """Shard a full set of oracle weights (tests: TP-N logits against TP1)."""
        cfg = ow.cfg
        m = TpDenseModel(cfg, device, rank, world, **kw)
        hd = cfg.head_dim
        hq, hkv, f = cfg.n_heads // world, cfg.n_kv_heads // world, cfg.ffn // world

        def rows(ql, idx):
            return quant.QuantLinear(len(idx), ql.k, ql.bits, ql.group, ql.codes[idx], ql.scale[idx], ql.zero[idx])

        def cols(ql, k0, k1):
            g0, g1 = k0 // ql.group, k1 // ql.group
            return quant.QuantLinear(ql.n, k1 - k0, ql.bits, ql.group, ql.codes[:, k0:k1].contiguous(),
                                     ql.scale[:, g0:g1].contiguous(), ql.zero[:, g0:g1].contiguous())

        for l, lay in enumerate(ow.layers):
            q = ow.quant
            qi = torch.arange(rank * hq * hd, (rank + 1) * hq * hd)
            ki = cfg.q_dim + torch.arange(rank * hkv * hd, (rank + 1) * hkv * hd)
            vi = cfg.q_dim + cfg.kv_dim + torch.arange(rank * hkv * hd, (rank + 1) * hkv * hd)
            d = {"qkv": L.WqLinear.from_quant(rows(q[f"{l}.qkv"], torch.cat([qi, ki, vi])), m.dev),
                 "o": L.WqLinear.from_quant(cols(q[f"{l}.o"], rank * hq * hd, (rank + 1) * hq * hd), m.dev),
                 # merged gate_up rows come in blocks of 16 (8 gate + 8 up) per 8 features
                 "gate_up": L.WqLinear.from_quant(rows(q[f"{l}.gate_up"], torch.arange(rank * 2 * f, (rank + 1) * 2 * f)), m.dev),
                 "down": L.WqLinear.from_quant(cols(q[f"{l}.down"], rank * f, (rank + 1) * f), m.dev),
                 "ln1": lay["ln1"].to(m.dev), "ln2": lay["ln2"].to(m.dev)}
            m.layers.append(d)
        m.embed = ow.embed.to(m.dev)
        m.final_norm = ow.final_norm.to(m.dev)
        ql = ow.quant["lm_head"]
        lo, hi = rank * m.vocab_shard, min(cfg.vocab, (rank + 1) * m.vocab_shard)
        idx = torch.arange(lo, hi)
        pad = m.lm_rows - (hi - lo)
        sh = rows(ql, idx)
        if pad:
            sh = quant.QuantLinear(m.lm_rows, ql.k, ql.bits, ql.group,
                                   torch.cat([sh.codes, torch.zeros(pad, ql.k, dtype=torch.uint8)]),
                                   torch.cat([sh.scale, torch.zeros(pad, ql.k // ql.group, dtype=torch.float16)]),
                                   torch.cat([sh.zero, torch.zeros(pad, ql.k // ql.group, dtype=torch.float16)]))
        m.lm_head = L.WqLinear.from_quant(sh, m.dev)
        return m.finalize()

    # ------------------------------------------------------------------------------------------------ collectives
    def _row_parallel(self, lin, x, resid, out, ss_out, site: int):
        if self.use_nccl_decode:
            # baseline: library all-reduce between an unfused GEMV and a separate add + statistics pass
            part = L.gemv(lin, x, self.ws, epi=_lib.EPI_F32)
            dist.all_reduce(part)
            out.copy_((part + resid.float()).to(torch.bfloat16))
            from ..ops import basic
            basic.sumsq(out, ss_out)
            return 1
        m = x.shape[0]
        if m >= (self.ws.mm_min_rows or L.MM_MIN_ROWS):
            # More rows than the GEMV family serves well: partial rows from the tensor-core GEMM, summed over the ranks by
            # the push all-reduce kernel (rank order, bounded waits), then residual add and the next norm's statistic.
            part = L.mm(lin, x, self.ws, epi=_lib.EPI_F32)
            rows_per = max(1, self._gather_inbox.slot_stride // lin.n)
            for r0 in range(0, m, rows_per):
                r1 = min(m, r0 + rows_per)
                part[r0:r1] = self._gather.all_reduce(part[r0:r1].reshape(-1)).view(r1 - r0, lin.n)
            out.copy_((part + resid.float()).to(torch.bfloat16))
            from ..ops import basic
            basic.sumsq(out, ss_out)
            return 1
        prev = (site - 1) % self.n_sites
        tp = self.inbox.tp_push(site, prev, skip_push=(site == self.skip_push_site))
        L.gemv(lin, x, self.ws, epi=EPI_TP_RESID, resid=resid, out=out, ss_out=ss_out, tp=tp)
        return lin.n_panels()

    def _reduce_rows(self, x: torch.Tensor) -> torch.Tensor:
        """Sum of a row-parallel partial [rows, n] over the ranks for prefill-size chunks, with the engine's own bounded
        push kernels and no library collective: two-shot (reduce-scatter, then all-gather) so that every rank moves
        2 (N - 1) / N of the chunk over NVLink instead of (N - 1) times the chunk.  Sums are taken in rank order, so
        every rank holds the same bits.  ``use_nccl_decode`` keeps the library all-reduce as the baseline."""
        if self.use_nccl_decode:
            y = x.float()
            dist.all_reduce(y)
            return y.to(torch.bfloat16)
        w = self.world
        if self._prefill_comm is None:
            from .comm import PushComm
            self._prefill_inbox = SymmetricInbox(self.rank, w, 1 << 20, 3, self.dev, status=self._status_all[3:4])
            self._prefill_comm = PushComm(self._prefill_inbox)
        pc, per = self._prefill_comm, self._prefill_inbox.slot_stride
        flat = x.float().reshape(-1)
        n = flat.numel()
        out = torch.empty_like(flat)
        step = w * per
        for o in range(0, n, step):
            m = min(step, n - o)
            shard = (m + w - 1) // w
            shard = (shard + 3) // 4 * 4
            buf = torch.zeros(w * shard, dtype=torch.float32, device=self.dev)
            buf[:m] = flat[o:o + m]
            mine = pc.reduce_scatter(buf.view(w, shard))
            full = pc.all_gather(mine)
            out[o:o + m] = full.reshape(-1)[:m]
        return out.view_as(x).to(torch.bfloat16)

    def _row_linear_big(self, lin, x: torch.Tensor) -> torch.Tensor:
        """Prefill-size row-parallel linear with the reduce-scatter fused into the GEMM (fused path 1 beyond decode
        rows): the tcgen05 GEMM's epilogue stores every fp32 partial tile into the inbox of the rank that owns its rows,
        over NVLink, while the remaining tiles are computed; one more kernel sums each rank's rows in rank order, hands the
        sums to the peers and collects theirs (``PushComm.gemm_reduce_gather``).  No library collective and no separate
        pass over the partial product.  Chunks that run on the in-kernel-dequant
        GEMM (up to 256 rows) and the NCCL baseline keep the unfused route."""
        T = x.shape[0]
        w = self.world
        if self.use_nccl_decode or not self.fused_prefill or (T <= 256 and self.prefill_mm) or T < 32 * w:
            return self._reduce_rows(self._linear_big(lin, x))
        if self._fused_comm is None:
            from .comm import PushComm
            rows = (self.prefill_chunk + 32 + w - 1) // w
            self._fused_inbox = SymmetricInbox(self.rank, w, (rows * self.cfg.d_model + 3) // 4 * 4, 6, self.dev, status=self._status_all[3:4])
            self._fused_comm = PushComm(self._fused_inbox)
        pc = self._fused_comm
        if ((T + w - 1) // w) * lin.n > self._fused_inbox.slot_stride:
            return self._reduce_rows(self._linear_big(lin, x))
        from ..ops import gemm as G
        return pc.gemm_reduce_gather(x.contiguous(), G.dequant_bf16(lin, self), status=self.status)

    def _lm_valid(self) -> int:
        valid = self.full_cfg.vocab_valid or self.full_cfg.vocab
        lo = self.rank * self.vocab_shard
        return max(0, min(self.vocab_shard, valid - lo))

    def _combine_argmax(self, m: int, standalone: bool = False):
        lib = _lib.cuda_lib()
        self.out_ids[:m].add_(self.idx_off[:m])
        if (standalone or m >= (self.ws.mm_min_rows or L.MM_MIN_ROWS)) and not self.use_nccl_decode:
            # The static argmax slot is re-armed by the first fused row-parallel site of the next small-m pass; a prefill
            # tail, and steps on the tensor-core path (whose row-parallel linears do not use the static sites), are not
            # followed by one, so they exchange the winners through the rotating gather inbox instead.
            n = (2 * m + 3) // 4 * 4
            x = torch.zeros(n, dtype=torch.float32, device=self.dev)
            x[:m] = self.out_val[:m]
            x[m:2 * m] = self.out_ids[:m].float()                    # ids < 2^24: exact in fp32
            g = self._gather.all_gather(x)
            vals, ids = g[:, :m], g[:, m:2 * m].to(torch.int32)
            best = vals.max(dim=0, keepdim=True).values
            cand = torch.where(vals == best, ids, torch.full_like(ids, 0x7fffffff))
            self.out_ids[:m].copy_(cand.min(dim=0).values)
            return
        if self.use_nccl_decode:
            # baseline: library all-gather of the per-rank winners, merged with framework ops
            vals = torch.empty(self.world, m, dtype=torch.float32, device=self.dev)
            ids = torch.empty(self.world, m, dtype=torch.int32, device=self.dev)
            dist.all_gather_into_tensor(vals, self.out_val[:m].contiguous())
            dist.all_gather_into_tensor(ids, self.out_ids[:m].contiguous())
            best = vals.max(dim=0, keepdim=True).values
            cand = torch.where(vals == best, ids, torch.full_like(ids, 0x7fffffff))
            self.out_ids[:m].copy_(cand.min(dim=0).values)
            return
        site = self.n_sites - 1
        a = self.inbox.comm_args(site, site - 1, skip_push=(site == self.skip_push_site), clear_n=m * self.cfg.d_model)
        check(lib.b2_comm_argmax_combine(C.byref(a), ptr(self.out_val), ptr(self.out_ids), m, ptr(self.out_ids), 0,
                                         current_stream()), "b2_comm_argmax_combine")

    def _full_logits(self, m: int) -> torch.Tensor:
        """All-gather of the vocab shards through the push inbox (own kernel, no library collective): every rank ends
        up with the same [m, vocab] fp32 logits, so that sampling is replicated and needs no further exchange."""
        outs = []
        for r0 in range(0, m, 8):
            r1 = min(m, r0 + 8)
            g = self._gather.all_gather(self.logits[r0:r1].contiguous().view(-1))          # [world, rows * lm_rows]
            g = g.view(self.world, r1 - r0, self.lm_rows)[:, :, :self.vocab_shard]
            outs.append(g.permute(1, 0, 2).reshape(r1 - r0, self.world * self.vocab_shard)[:, :self.full_cfg.vocab])
        return torch.cat(outs).contiguous()

    def vocab_valid_full(self) -> int:
        return self.full_cfg.vocab_valid or self.full_cfg.vocab

    def recover(self):
        """As the single-GPU recovery, plus re-arming this rank's collective inboxes.  Every rank calls it (the driver
        forwards the call), with a host-side barrier before anyone launches again."""
        super().recover()
        self.inbox.rearm_all()
        for ib, pc in ((self._gather_inbox, self._gather), (self._prefill_inbox, self._prefill_comm), (self._fused_inbox, self._fused_comm)):
            if ib is not None:
                ib.rearm_all()
                pc.calls, pc.prev_n = 0, 0
        torch.cuda.synchronize(self.dev)

    def close(self):
        """Releases the peer mappings (collective: every rank calls it, with nothing in flight)."""
        self._graphs.clear()
        if self.step is not None:
            self.step.close()
            self.step = None
        if self._gather_inbox is not None:
            self._gather_inbox.close()
            self._gather = self._gather_inbox = None
        if self._prefill_inbox is not None:
            self._prefill_inbox.close()
            self._prefill_inbox = self._prefill_comm = None
        if self._fused_inbox is not None:
            self._fused_inbox.close()
            self._fused_inbox = self._fused_comm = None
        self.inbox.close()

    def weight_bytes(self) -> int:
        return super().weight_bytes()

    def _step_ok(self, m: int) -> bool:
        return not self.use_nccl_decode and super()._step_ok(m)

    def launches_per_step(self, batch: int = 1) -> int:
        n = super().launches_per_step(batch)
        return n if n == 1 else n + 1
