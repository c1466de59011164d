"""MTP head checkpoints: the ``mtp.*`` tensor layout is read and validated on the host (reference reader:
crates/agens-cli/src/spec.rs:306-370)."""
import pytest
import torch

from agens_engine_b200.models.config import ModelConfig
from agens_engine_b200.utils import checkpoint as K


def _cfg():
    return ModelConfig(name="t", n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=128, ffn=512, vocab=512)


def _tensors(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    d, f = cfg.d_model, cfg.ffn
    shapes = {"fc.weight": (d, 2 * d), "layers.0.self_attn.q_proj.weight": (cfg.q_dim, d),
              "layers.0.self_attn.k_proj.weight": (cfg.kv_dim, d), "layers.0.self_attn.v_proj.weight": (cfg.kv_dim, d),
              "layers.0.self_attn.o_proj.weight": (d, cfg.q_dim), "layers.0.mlp.gate_proj.weight": (f, d),
              "layers.0.mlp.up_proj.weight": (f, d), "layers.0.mlp.down_proj.weight": (d, f)}
    shapes.update({n: (d,) for n in K.MTP_NORMS})
    return {"mtp." + n: (torch.randn(*s, generator=g) * 0.05).to(torch.bfloat16) for n, s in shapes.items()}


def test_read_mtp_round_trip(tmp_path):
    cfg = _cfg()
    t = _tensors(cfg)
    t["mtp.layers.0.self_attn.q_norm.weight"] = torch.ones(cfg.head_dim, dtype=torch.bfloat16)      # another head design's tensor
    t["model.norm.weight"] = torch.ones(cfg.d_model, dtype=torch.bfloat16)                           # not an mtp tensor: skipped
    half = len(t) // 2
    items = list(t.items())
    K.write_safetensors(str(tmp_path / "a.safetensors"), dict(items[:half]))
    K.write_safetensors(str(tmp_path / "b.safetensors"), dict(items[half:]))
    got = K.read_mtp(str(tmp_path), cfg)
    assert got.pop("_unexpected") == ["mtp.layers.0.self_attn.q_norm.weight"]
    assert set(got) == set(K.MTP_NORMS) | set(K.MTP_LINEARS)
    for n, v in got.items():
        assert torch.equal(v, t["mtp." + n])


def test_read_mtp_refuses_bad_checkpoints(tmp_path):
    cfg = _cfg()
    t = _tensors(cfg)
    with pytest.raises(FileNotFoundError):
        K.read_mtp(str(tmp_path), cfg)
    miss = dict(t); miss.pop("mtp.fc.weight")
    K.write_safetensors(str(tmp_path / "m.safetensors"), miss)
    with pytest.raises(ValueError, match="missing"):
        K.read_mtp(str(tmp_path), cfg)
    bad = dict(t); bad["mtp.fc.weight"] = bad["mtp.fc.weight"].float()
    K.write_safetensors(str(tmp_path / "m.safetensors"), bad)
    with pytest.raises(ValueError, match="bf16 expected"):
        K.read_mtp(str(tmp_path), cfg)
    bad = dict(t); bad["mtp.fc.weight"] = bad["mtp.fc.weight"][:, :cfg.d_model].contiguous()
    K.write_safetensors(str(tmp_path / "m.safetensors"), bad)
    with pytest.raises(ValueError, match="shape"):
        K.read_mtp(str(tmp_path), cfg)
