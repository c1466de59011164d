"""Checkpoint directories in the public format: write, inspect, validate, verify, load.

Format (the reference's container, ``crates/agens-core/src/weights.rs:133-251``, extended): Hugging Face directory with
``config.json``, ``model.safetensors`` (or shards + ``model.safetensors.index.json``), optional ``SHA256SUMS``.  A
quantised linear stores ``<name>.weight_packed`` (int32 bit stream along k), ``<name>.weight_scale`` (bf16 or fp16,
``[n, k/group]``) and, when asymmetric, ``<name>.weight_zero_point`` (fp16).  Reading, hashing and validation run in the
C++ core (``csrc/core/checkpoint.cpp``); this module writes files and turns tensors into engine weights.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import dataclasses
import json
import os
import struct
from typing import Dict, Optional

import torch

from .. import _lib
from . import quant

_ST_DTYPES = {torch.bfloat16: "BF16", torch.float16: "F16", torch.float32: "F32", torch.int32: "I32", torch.int64: "I64",
              torch.uint8: "U8", torch.int8: "I8"}
_TORCH_OF = {v: k for k, v in _ST_DTYPES.items()}


def _host():
    h = _lib.host_lib()
    if not getattr(h, "_ckpt_sig", False):
        vp, i = C.c_void_p, C.c_int
        h.b2h_st_open.argtypes, h.b2h_st_open.restype = [C.c_char_p, C.c_char_p, i], vp
        h.b2h_st_close.argtypes, h.b2h_st_close.restype = [vp], None
        h.b2h_st_count.argtypes, h.b2h_st_count.restype = [vp], i
        h.b2h_st_info.argtypes, h.b2h_st_info.restype = [vp, i], vp
        h.b2h_st_data.argtypes, h.b2h_st_data.restype = [vp, C.c_char_p, C.POINTER(C.c_longlong)], vp
        h.b2h_st_advise_sequential.argtypes, h.b2h_st_advise_sequential.restype = [vp], None
        h.b2h_sha256_file.argtypes, h.b2h_sha256_file.restype = [C.c_char_p], vp
        h.b2h_verify_sha256sums.argtypes, h.b2h_verify_sha256sums.restype = [C.c_char_p, i], vp
        h.b2h_validate_checkpoint.argtypes, h.b2h_validate_checkpoint.restype = [C.c_char_p], vp
        h.b2h_free_str.argtypes, h.b2h_free_str.restype = [vp], None
        h._ckpt_sig = True
    return h


def _take(p) -> str:
    s = C.cast(p, C.c_char_p).value.decode()
    _host().b2h_free_str(p)
    return s


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[dict] = None):
    header, off, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _ST_DTYPES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


class SafeTensorsFile:
    """mmap reader of the C++ core; tensors are zero-copy views valid while the file object lives."""

    def __init__(self, path: str):
        err = C.create_string_buffer(512)
        self._h = _host().b2h_st_open(path.encode(), err, 512)
        if not self._h:
            raise IOError(err.value.decode())
        _host().b2h_st_advise_sequential(self._h)
        self.info = {}
        for i in range(_host().b2h_st_count(self._h)):
            d = json.loads(_take(_host().b2h_st_info(self._h, i)))
            self.info[d["name"]] = d

    def keys(self):
        return list(self.info)

    def tensor(self, name: str) -> torch.Tensor:
        d = self.info[name]
        n = C.c_longlong()
        p = _host().b2h_st_data(self._h, name.encode(), C.byref(n))
        if n.value == 0:
            return torch.empty(d["shape"], dtype=_TORCH_OF[d["dtype"]])
        buf = (C.c_uint8 * n.value).from_address(p)
        return torch.frombuffer(buf, dtype=_TORCH_OF[d["dtype"]]).reshape(d["shape"])

    def close(self):
        if self._h:
            _host().b2h_st_close(self._h)
            self._h = None

    def __del__(self):
        self.close()


def sha256_file(path: str) -> str:
    return _take(_host().b2h_sha256_file(path.encode()))


def verify(dir_: str, threads: int = 8) -> dict:
    return json.loads(_take(_host().b2h_verify_sha256sums(dir_.encode(), threads)))


def validate(dir_: str) -> dict:
    return json.loads(_take(_host().b2h_validate_checkpoint(dir_.encode())))


def inspect(dir_: str) -> dict:
    rep = validate(dir_)
    cfg = json.load(open(os.path.join(dir_, "config.json")))
    hist: Dict[str, int] = {}
    for fmt in rep.get("linears", {}).values():
        k = fmt["format"] if fmt["format"] == "bf16" else f"w{fmt['bits']}g{fmt['group']}{'a' if fmt['asymmetric'] else 's'}"
        hist[k] = hist.get(k, 0) + 1
    return {"config": cfg, "ok": rep["ok"], "errors": rep["errors"], "tensors": rep.get("tensors"), "bytes": rep.get("bytes"),
            "linear_formats": hist}


# ---------------------------------------------------------------------------------------------------------------
# writing a model / loading it into the engine
# ---------------------------------------------------------------------------------------------------------------

def _put_linear(out: dict, name: str, ql: quant.QuantLinear, symmetric: bool):
    out[name + ".weight_packed"] = quant.pack_stream(ql.codes, ql.bits)
    out[name + ".weight_scale"] = ql.scale.to(torch.bfloat16) if symmetric else ql.scale
    if not symmetric:
        out[name + ".weight_zero_point"] = ql.zero


def _rows(ql: quant.QuantLinear, lo: int, hi: int) -> quant.QuantLinear:
    return quant.QuantLinear(hi - lo, ql.k, ql.bits, ql.group, ql.codes[lo:hi], ql.scale[lo:hi], ql.zero[lo:hi])


def save_oracle(dir_: str, ow, shards: int = 1, symmetric: bool = False, sums: bool = True):
    """Writes oracle weights (``models/oracle.py``) as a checkpoint directory with separate q/k/v and gate/up tensors."""
    cfg = ow.cfg
    os.makedirs(dir_, exist_ok=True)
    hf = {"architectures": ["DenseGQAForCausalLM"], "num_hidden_layers": cfg.n_layers, "hidden_size": cfg.d_model,
          "num_attention_heads": cfg.n_heads, "num_key_value_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim,
          "intermediate_size": cfg.ffn, "vocab_size": cfg.vocab, "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_eps,
          "tie_word_embeddings": False, "torch_dtype": "bfloat16",
          "quantization_config": {"format": "pack-quantized", "group_size": cfg.group, "symmetric": symmetric}}
    json.dump(hf, open(os.path.join(dir_, "config.json"), "w"), indent=1)
    t: Dict[str, torch.Tensor] = {"model.embed_tokens.weight": ow.embed, "model.norm.weight": ow.final_norm}
    for l, lay in enumerate(ow.layers):
        p = f"model.layers.{l}."
        t[p + "input_layernorm.weight"], t[p + "post_attention_layernorm.weight"] = lay["ln1"], lay["ln2"]
        qkv = ow.quant[f"{l}.qkv"]
        _put_linear(t, p + "self_attn.q_proj", _rows(qkv, 0, cfg.q_dim), symmetric)
        _put_linear(t, p + "self_attn.k_proj", _rows(qkv, cfg.q_dim, cfg.q_dim + cfg.kv_dim), symmetric)
        _put_linear(t, p + "self_attn.v_proj", _rows(qkv, cfg.q_dim + cfg.kv_dim, cfg.q_dim + 2 * cfg.kv_dim), symmetric)
        _put_linear(t, p + "self_attn.o_proj", ow.quant[f"{l}.o"], symmetric)
        gu = ow.quant[f"{l}.gate_up"]
        gi = torch.arange(cfg.ffn * 2).reshape(cfg.ffn // 8, 2, 8)
        g_rows, u_rows = gi[:, 0].reshape(-1), gi[:, 1].reshape(-1)
        sel = lambda idx: quant.QuantLinear(len(idx), gu.k, gu.bits, gu.group, gu.codes[idx], gu.scale[idx], gu.zero[idx])
        _put_linear(t, p + "mlp.gate_proj", sel(g_rows), symmetric)
        _put_linear(t, p + "mlp.up_proj", sel(u_rows), symmetric)
        _put_linear(t, p + "mlp.down_proj", ow.quant[f"{l}.down"], symmetric)
    _put_linear(t, "lm_head", ow.quant["lm_head"], symmetric)
    names = list(t)
    if shards <= 1:
        write_safetensors(os.path.join(dir_, "model.safetensors"), t, {"format": "pt"})
        files = ["model.safetensors"]
    else:
        per = (len(names) + shards - 1) // shards
        wm, files = {}, []
        for s in range(shards):
            fn = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
            part = {n: t[n] for n in names[s * per:(s + 1) * per]}
            if not part:
                continue
            write_safetensors(os.path.join(dir_, fn), part, {"format": "pt"})
            files.append(fn)
            wm.update({n: fn for n in part})
        json.dump({"metadata": {}, "weight_map": wm}, open(os.path.join(dir_, "model.safetensors.index.json"), "w"))
    if sums:
        with open(os.path.join(dir_, "SHA256SUMS"), "w") as f:
            for fn in files + ["config.json"]:
                f.write(f"{hashlib.sha256(open(os.path.join(dir_, fn), 'rb').read()).hexdigest()}  {fn}\n")


def _get_linear(files, wm, name: str, n: int, k: int, fmt: dict) -> quant.QuantLinear:
    def T(suffix):
        full = name + suffix
        return files[wm[full]].tensor(full)
    if fmt["format"] == "bf16":
        raise NotImplementedError("bf16 linears are quantised at load by the caller")
    bits, group = fmt["bits"], fmt["group"]
    codes = quant.unpack_stream(T(".weight_packed"), bits, k)
    # copies: the mapped file may be closed before the weights are packed for the device
    scale = T(".weight_scale").to(torch.float16).clone()
    zero = T(".weight_zero_point").clone() if fmt["asymmetric"] else torch.full_like(scale, float(1 << (bits - 1)))
    return quant.QuantLinear(n, k, bits, group, codes, scale, zero)


@dataclasses.dataclass
class CheckpointWeights:
    """Quantised weights of a checkpoint in the merged form the models take (q/k/v as one ``qkv`` linear, gate/up
    interleaved), all on the CPU; the same fields :class:`models.oracle.OracleWeights` offers to ``from_oracle``."""
    cfg: object
    embed: torch.Tensor
    layers: list
    final_norm: torch.Tensor
    quant: dict


def read_weights(dir_: str) -> CheckpointWeights:
    """Validates the directory and reads every tensor (reference: m1::load weight loop with gate+up merge,
    crates/agens-cli/src/m1.rs:452-1066)."""
    from ..models.config import ModelConfig
    rep = validate(dir_)
    if not rep["ok"]:
        raise ValueError("invalid checkpoint: " + "; ".join(rep["errors"][:5]))
    cfg = ModelConfig.from_json(os.path.join(dir_, "config.json"))
    idx = os.path.join(dir_, "model.safetensors.index.json")
    if os.path.exists(idx):
        wm = json.load(open(idx))["weight_map"]
    else:
        f0 = SafeTensorsFile(os.path.join(dir_, "model.safetensors"))
        wm = {k: "model.safetensors" for k in f0.keys()}
    files = {fn: SafeTensorsFile(os.path.join(dir_, fn)) for fn in set(wm.values())}
    fm = rep["linears"]
    cfg.group = next(iter(fm.values())).get("group", 128)
    cat = lambda qs: quant.QuantLinear(sum(q.n for q in qs), qs[0].k, qs[0].bits, qs[0].group, torch.cat([q.codes for q in qs]),
                                       torch.cat([q.scale for q in qs]), torch.cat([q.zero for q in qs]))
    layers, qd = [], {}
    for l in range(cfg.n_layers):
        p = f"model.layers.{l}."
        g = lambda nm, n, k: _get_linear(files, wm, p + nm, n, k, fm[p + nm])
        q, kk, v = g("self_attn.q_proj", cfg.q_dim, cfg.d_model), g("self_attn.k_proj", cfg.kv_dim, cfg.d_model), g("self_attn.v_proj", cfg.kv_dim, cfg.d_model)
        if not (q.bits == kk.bits == v.bits):
            raise ValueError(f"layer {l}: q/k/v use different bit widths; they share one fused kernel launch")
        gate, up = g("mlp.gate_proj", cfg.ffn, cfg.d_model), g("mlp.up_proj", cfg.ffn, cfg.d_model)
        if gate.bits != up.bits:
            raise ValueError(f"layer {l}: gate/up use different bit widths")
        qd[f"{l}.qkv"] = cat([q, kk, v])
        qd[f"{l}.o"] = g("self_attn.o_proj", cfg.d_model, cfg.q_dim)
        qd[f"{l}.gate_up"] = quant.QuantLinear(2 * cfg.ffn, cfg.d_model, gate.bits, gate.group,
                                               quant.interleave_gate_up(gate.codes, up.codes),
                                               quant.interleave_gate_up(gate.scale, up.scale),
                                               quant.interleave_gate_up(gate.zero, up.zero))
        qd[f"{l}.down"] = g("mlp.down_proj", cfg.d_model, cfg.ffn)
        T = lambda nm: files[wm[p + nm]].tensor(p + nm).clone()
        layers.append({"ln1": T("input_layernorm.weight"), "ln2": T("post_attention_layernorm.weight")})
        for lin in ("qkv", "o", "gate_up", "down"):
            cfg.bits[f"{l}.{lin}"] = qd[f"{l}.{lin}"].bits
    embed = files[wm["model.embed_tokens.weight"]].tensor("model.embed_tokens.weight").clone()
    final_norm = files[wm["model.norm.weight"]].tensor("model.norm.weight").clone()
    qd["lm_head"] = _get_linear(files, wm, "lm_head", cfg.vocab, cfg.d_model, fm["lm_head"])
    cfg.lm_head_bits = qd["lm_head"].bits
    for f in files.values():
        f.close()
    return CheckpointWeights(cfg, embed, layers, final_norm, qd)


def load_model(dir_: str, device="cuda:0", rank: int = 0, world: int = 1, **kw):
    """Builds a :class:`DenseModel` (or this rank's :class:`TpDenseModel` shard) from a checkpoint directory."""
    w = read_weights(dir_)
    if world > 1:
        from ..parallel.tp_model import TpDenseModel
        return TpDenseModel.from_oracle(w, device, rank, world, **kw)
    from ..models.dense import DenseModel
    return DenseModel.from_oracle(w, device, **kw)
