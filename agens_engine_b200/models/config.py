"""Model configuration: dense GQA decoder family (target, companion drafter, MTP layer).

Plays the role of the reference's ``VolundrConfig`` (``crates/agens-core/src/config.rs:165-243``): parse a Hugging Face
``config.json``, expose per-token KV bytes and the per-linear quantisation plan.
"""
from __future__ import annotations

import dataclasses
import json
from typing import Dict, Optional

LINEARS = ("qkv", "o", "gate_up", "down")


@dataclasses.dataclass
class ModelConfig:
    name: str
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    group: int = 128
    lm_head_bits: int = 4
    # bits[(layer, linear)] -> 2 | 3 | 4 ; missing entries use default_bits
    bits: Dict[str, int] = dataclasses.field(default_factory=dict)
    default_bits: int = 4
    vocab_valid: Optional[int] = None      # ids >= vocab_valid are never produced (reference: VOCAB_VALID)
    page_size: int = 16

    def bits_of(self, layer: int, linear: str) -> int:
        return self.bits.get(f"{layer}.{linear}", self.default_bits)

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    def kv_bytes_per_token(self, tp: int = 1) -> int:
        """bf16 K and V of every layer for one token on one rank (reference: config.rs:236-243)."""
        return self.n_layers * 2 * (self.n_kv_heads // tp) * self.head_dim * 2

    def n_params_linear(self) -> int:
        per = self.d_model * (self.q_dim + 2 * self.kv_dim) + self.q_dim * self.d_model + 3 * self.d_model * self.ffn
        return self.n_layers * per

    def weight_bytes(self, tp: int = 1) -> int:
        """Bytes of quantised weights (codes + fp16 scale/zero pairs) plus bf16 embedding and quantised lm_head."""
        total = 0
        for l in range(self.n_layers):
            for lin, (n, k) in self.linear_shapes().items():
                b = self.bits_of(l, lin)
                total += n * k * b // 8 + (n * k // self.group) * 4
        total //= tp
        total += self.vocab * self.d_model * 2
        total += (self.vocab * self.d_model * self.lm_head_bits // 8 + self.vocab * self.d_model // self.group * 4) // tp
        return total

    def linear_shapes(self) -> Dict[str, tuple]:
        return {"qkv": (self.q_dim + 2 * self.kv_dim, self.d_model), "o": (self.d_model, self.q_dim),
                "gate_up": (2 * self.ffn, self.d_model), "down": (self.d_model, self.ffn)}

    @staticmethod
    def from_hf(cfg: dict, name: str = "hf") -> "ModelConfig":
        hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
        return ModelConfig(name=name, n_layers=cfg["num_hidden_layers"], d_model=cfg["hidden_size"],
                           n_heads=cfg["num_attention_heads"], n_kv_heads=cfg.get("num_key_value_heads", cfg["num_attention_heads"]),
                           head_dim=hd, ffn=cfg["intermediate_size"], vocab=cfg["vocab_size"],
                           rope_theta=float(cfg.get("rope_theta", 1e6)), rms_eps=float(cfg.get("rms_norm_eps", 1e-6)))

    @staticmethod
    def from_json(path: str) -> "ModelConfig":
        return ModelConfig.from_hf(json.load(open(path)), name=path)


def oracle_tiny() -> ModelConfig:
    """CPU-oracle plumbing config: 2 layers, d 256, 4 q / 2 kv heads x 64, FFN 512, vocab 1024, group 64;
    layer 0 at 4 bits, layer 1 at 2 bits (attention) and 3 bits (MLP)."""
    bits = {"0.qkv": 4, "0.o": 4, "0.gate_up": 4, "0.down": 4, "1.qkv": 2, "1.o": 2, "1.gate_up": 3, "1.down": 3}
    return ModelConfig("oracle-tiny", 2, 256, 4, 2, 64, 512, 1024, rope_theta=1e6, group=64, bits=bits, lm_head_bits=4)


def dense_32b(seed: int = 0) -> ModelConfig:
    """32B dense GQA decoder: 64 layers, d 5120, 64 q / 8 kv heads x 128, FFN 25600, vocab 151936, group 128, each
    linear at 2, 3 or 4 bits from a seeded assignment."""
    from ..utils.quant import seeded_bit_assignment
    names = [f"{l}.{lin}" for l in range(64) for lin in LINEARS]
    return ModelConfig("dense-32b", 64, 5120, 64, 8, 128, 25600, 151936, group=128,
                       bits=seeded_bit_assignment(names, seed), lm_head_bits=4)


def drafter_0p6b() -> ModelConfig:
    """Companion drafter: 28 layers, d 1024, 16 q / 8 kv heads x 128, FFN 3072, shared vocab 151936 (4-bit)."""
    return ModelConfig("drafter-0.6b", 28, 1024, 16, 8, 128, 3072, 151936, group=128, default_bits=4)


def scaled(cfg: ModelConfig, n_layers: int) -> ModelConfig:
    """Same architecture with fewer layers (tests, smoke runs)."""
    bits = {k: v for k, v in cfg.bits.items() if int(k.split(".")[0]) < n_layers}
    return dataclasses.replace(cfg, name=f"{cfg.name}-{n_layers}l", n_layers=n_layers, bits=bits)
