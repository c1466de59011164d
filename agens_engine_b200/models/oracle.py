"""Plain PyTorch reference of the dense GQA decoder on dequantised weights (the "CPU oracle").

Two precisions: ``mirror=False`` keeps every intermediate in fp32 (the fp32 dequantised reference the logits are
compared against); ``mirror=True`` rounds to bf16 at the places where the engine's kernels store bf16 (residual
stream, normalised activations, projections, SwiGLU output), which makes greedy token sequences comparable one to one.
The reference engine has no such model-level oracle in its repository (its parity tooling is
``tools/compare_logits.py`` against dumps of a Python stack); this module is that stack for the dense family.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Dict, List, Optional

import torch

from ..utils import quant
from .config import LINEARS, ModelConfig


@dataclasses.dataclass
class OracleWeights:
    cfg: ModelConfig
    embed: torch.Tensor                       # bf16 [vocab, d]
    layers: List[Dict[str, torch.Tensor]]     # fp32 dequantised "qkv", "o", "gate", "up", "down", bf16 "ln1", "ln2"
    final_norm: torch.Tensor                  # bf16 [d]
    lm_head: torch.Tensor                     # fp32 dequantised [vocab, d]
    quant: Dict[str, quant.QuantLinear]       # quantised forms keyed "l.linear" and "lm_head"


def random_weights(cfg: ModelConfig, seed: int = 0, symmetric: bool = False) -> OracleWeights:
    """Random-init N(0, 0.02) weights, quantised per the config (asymmetric fp16 scale + zero by default)."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g) * 0.02
    embed = rn(cfg.vocab, cfg.d_model).to(torch.bfloat16)
    layers, qd = [], {}
    for l in range(cfg.n_layers):
        wq, wk, wv = rn(cfg.q_dim, cfg.d_model), rn(cfg.kv_dim, cfg.d_model), rn(cfg.kv_dim, cfg.d_model)
        wo = rn(cfg.d_model, cfg.q_dim)
        wg, wu, wd = rn(cfg.ffn, cfg.d_model), rn(cfg.ffn, cfg.d_model), rn(cfg.d_model, cfg.ffn)
        raw = {"qkv": torch.cat([wq, wk, wv], 0), "o": wo, "gate_up": quant.interleave_gate_up(wg, wu), "down": wd}
        lay = {}
        for lin in LINEARS:
            ql = quant.quantize(raw[lin], cfg.bits_of(l, lin), cfg.group, symmetric=symmetric)
            qd[f"{l}.{lin}"] = ql
            lay[lin] = ql.dequant()
        gu = lay.pop("gate_up").reshape(cfg.ffn // 8, 16, cfg.d_model)
        lay["gate"] = gu[:, :8].reshape(cfg.ffn, cfg.d_model).contiguous()
        lay["up"] = gu[:, 8:].reshape(cfg.ffn, cfg.d_model).contiguous()
        lay["ln1"] = (1.0 + 0.05 * torch.randn(cfg.d_model, generator=g)).to(torch.bfloat16)
        lay["ln2"] = (1.0 + 0.05 * torch.randn(cfg.d_model, generator=g)).to(torch.bfloat16)
        layers.append(lay)
    final_norm = (1.0 + 0.05 * torch.randn(cfg.d_model, generator=g)).to(torch.bfloat16)
    ql = quant.quantize(rn(cfg.vocab, cfg.d_model), cfg.lm_head_bits, cfg.group, symmetric=symmetric)
    qd["lm_head"] = ql
    return OracleWeights(cfg, embed, layers, final_norm, ql.dequant(), qd)


def _r(x: torch.Tensor, mirror: bool) -> torch.Tensor:
    return x.to(torch.bfloat16).float() if mirror else x


def rmsnorm(h: torch.Tensor, w: torch.Tensor, eps: float, mirror: bool) -> torch.Tensor:
    return _r(h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps) * w.float(), mirror)


def rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """x [T, heads, hd] fp32, NeoX pairing (i, i + hd/2); angles in fp32 as the kernel computes them."""
    hd = x.shape[-1]
    inv = (theta ** (-2.0 * torch.arange(0, hd // 2, dtype=torch.float64) / hd)).float()
    ang = pos.float()[:, None] * inv[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., : hd // 2], x[..., hd // 2:]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


class OracleModel:
    """Stateful reference: keeps the K/V of one sequence, so prefill-then-decode can be replayed token by token."""

    def __init__(self, w: OracleWeights, mirror: bool = False):
        self.w, self.cfg, self.mirror = w, w.cfg, mirror
        self.k: List[torch.Tensor] = [torch.zeros(0, w.cfg.n_kv_heads, w.cfg.head_dim) for _ in range(w.cfg.n_layers)]
        self.v: List[torch.Tensor] = [torch.zeros(0, w.cfg.n_kv_heads, w.cfg.head_dim) for _ in range(w.cfg.n_layers)]

    @property
    def seq_len(self) -> int:
        return self.k[0].shape[0]

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        """Append ``ids`` (1-D) to the sequence; returns fp32 logits ``[len(ids), vocab]``."""
        cfg, m = self.cfg, self.mirror
        T = ids.numel()
        pos = torch.arange(self.seq_len, self.seq_len + T)
        h = self.w.embed[ids.long()].float()
        gq = cfg.n_heads // cfg.n_kv_heads
        for l, lay in enumerate(self.w.layers):
            x = rmsnorm(h, lay["ln1"], cfg.rms_eps, m)
            qkv = _r(x @ lay["qkv"].t(), m)
            q = qkv[:, : cfg.q_dim].reshape(T, cfg.n_heads, cfg.head_dim)
            k = qkv[:, cfg.q_dim: cfg.q_dim + cfg.kv_dim].reshape(T, cfg.n_kv_heads, cfg.head_dim)
            v = qkv[:, cfg.q_dim + cfg.kv_dim:].reshape(T, cfg.n_kv_heads, cfg.head_dim)
            q, k = _r(rope(q, pos, cfg.rope_theta), m), _r(rope(k, pos, cfg.rope_theta), m)
            self.k[l] = torch.cat([self.k[l], k], 0)
            self.v[l] = torch.cat([self.v[l], v], 0)
            K = self.k[l].repeat_interleave(gq, dim=1)        # [L, hq, hd]
            V = self.v[l].repeat_interleave(gq, dim=1)
            s = torch.einsum("thd,lhd->htl", q, K) / math.sqrt(cfg.head_dim)
            mask = torch.arange(K.shape[0])[None, :] > pos[:, None]
            s = s.masked_fill(mask[None], float("-inf"))
            p = torch.softmax(s, dim=-1)
            a = _r(torch.einsum("htl,lhd->thd", p, V).reshape(T, cfg.q_dim), m)
            h = _r(a @ lay["o"].t() + h, m)
            x = rmsnorm(h, lay["ln2"], cfg.rms_eps, m)
            gate, up = _r(x @ lay["gate"].t(), m), _r(x @ lay["up"].t(), m)
            act = _r(torch.nn.functional.silu(gate) * up, m)
            h = _r(act @ lay["down"].t() + h, m)
        x = rmsnorm(h, self.w.final_norm, cfg.rms_eps, m)
        return x @ self.w.lm_head.t()

    def generate_greedy(self, prompt: torch.Tensor, n_new: int):
        """Returns (token ids [n_new], logits of every generated position [n_new, vocab])."""
        logits = self.forward(prompt)[-1:]
        toks, outs = [], []
        for _ in range(n_new):
            outs.append(logits[0])
            t = int(torch.argmax(logits[0, : self.cfg.vocab_valid or self.cfg.vocab]))
            toks.append(t)
            logits = self.forward(torch.tensor([t]))
        return torch.tensor(toks), torch.stack(outs)
