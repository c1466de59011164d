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


def save_oracle(dir_: str, ow, shards: int = 1, symmetric: bool = False, sums: bool = True, root: str = "model.",
                bf16_linears: tuple = (), tied: bool = False, extra: Optional[Dict[str, torch.Tensor]] = None):
    """Writes oracle weights (``models/oracle.py``) as a checkpoint directory with separate q/k/v and gate/up tensors.
    ``root``: name prefix of the text model (``model.`` or ``model.language_model.``); ``bf16_linears``: suffixes such
    as ``"self_attn.o_proj"`` written as dequantised bf16 ``weight`` tensors; ``tied``: no lm_head tensor and
    ``tie_word_embeddings`` set; ``extra``: further tensors stored as they are."""
    cfg = ow.cfg
    os.makedirs(dir_, exist_ok=True)
    hf = {"architectures": ["DenseGQAForCausalLM"], "num_hidden_layers": cfg.n_layers, "hidden_size": cfg.d_model,
          "num_attention_heads": cfg.n_heads, "num_key_value_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim,
          "intermediate_size": cfg.ffn, "vocab_size": cfg.vocab, "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_eps,
          "tie_word_embeddings": bool(tied), "torch_dtype": "bfloat16",
          "quantization_config": {"format": "pack-quantized", "group_size": cfg.group, "symmetric": symmetric}}
    json.dump(hf, open(os.path.join(dir_, "config.json"), "w"), indent=1)
    t: Dict[str, torch.Tensor] = {root + "embed_tokens.weight": ow.embed, root + "norm.weight": ow.final_norm}
    def put(out, name, ql, symmetric):
        if any(name.endswith(sfx) for sfx in bf16_linears):
            out[name + ".weight"] = ql.dequant().to(torch.bfloat16)
        else:
            _put_linear(out, name, ql, symmetric)
    for l, lay in enumerate(ow.layers):
        p = f"{root}layers.{l}."
        t[p + "input_layernorm.weight"], t[p + "post_attention_layernorm.weight"] = lay["ln1"], lay["ln2"]
        qkv = ow.quant[f"{l}.qkv"]
        put(t, p + "self_attn.q_proj", _rows(qkv, 0, cfg.q_dim), symmetric)
        put(t, p + "self_attn.k_proj", _rows(qkv, cfg.q_dim, cfg.q_dim + cfg.kv_dim), symmetric)
        put(t, p + "self_attn.v_proj", _rows(qkv, cfg.q_dim + cfg.kv_dim, cfg.q_dim + 2 * cfg.kv_dim), symmetric)
        put(t, p + "self_attn.o_proj", ow.quant[f"{l}.o"], symmetric)
        gu = ow.quant[f"{l}.gate_up"]
        gi = torch.arange(cfg.ffn * 2).reshape(cfg.ffn // 8, 2, 8)
        g_rows, u_rows = gi[:, 0].reshape(-1), gi[:, 1].reshape(-1)
        sel = lambda idx: quant.QuantLinear(len(idx), gu.k, gu.bits, gu.group, gu.codes[idx], gu.scale[idx], gu.zero[idx])
        put(t, p + "mlp.gate_proj", sel(g_rows), symmetric)
        put(t, p + "mlp.up_proj", sel(u_rows), symmetric)
        put(t, p + "mlp.down_proj", ow.quant[f"{l}.down"], symmetric)
    if not tied:
        put(t, "lm_head", ow.quant["lm_head"], symmetric)
    t.update(extra or {})
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


BF16_LOAD_BITS = 4     # bf16 linears (and a tied lm_head) are quantised at load: asymmetric, group 128, this many bits


def _get_linear(files, wm, name: str, n: int, k: int, fmt: dict) -> quant.QuantLinear:
    def T(suffix):
        full = name + suffix
        return files[wm[full]].tensor(full)
    if fmt["format"] == "bf16":
        # the kernels of this engine take quantised linears only: a bf16 linear is quantised here, once, at load
        return quant.quantize(T(".weight").float(), BF16_LOAD_BITS, 128)
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
    unexpected: list = dataclasses.field(default_factory=list)     # text-model tensors the loader had no use for


def _open(dir_: str):
    """Validates the directory; returns (report, config, weight map, open shard files)."""
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
    groups = [f.get("group", 128) for f in rep["linears"].values()]
    cfg.group = max(set(groups), key=groups.count) if groups else 128      # linears carry their own group size
    hf = json.load(open(os.path.join(dir_, "config.json")))
    return rep, cfg, wm, files, bool(hf.get("tie_word_embeddings", False))


def read_weights(dir_: str) -> CheckpointWeights:
    """Validates the directory and reads every tensor to the CPU in expanded form (reference: m1::load weight loop with
    gate+up merge, crates/agens-cli/src/m1.rs:452-1066).  Meant for tests and small models: :func:`load_model` streams
    the packed tensors to the device instead."""
    rep, cfg, wm, files, tied = _open(dir_)
    fm, root = rep["linears"], rep.get("root", "model.")
    cat = lambda qs: quant.QuantLinear(sum(q.n for q in qs), qs[0].k, qs[0].bits, qs[0].group, torch.cat([q.codes for q in qs]),
                                       torch.cat([q.scale for q in qs]), torch.cat([q.zero for q in qs]))
    layers, qd = [], {}
    for l in range(cfg.n_layers):
        p = f"{root}layers.{l}."
        g = lambda nm, n, k: _get_linear(files, wm, p + nm, n, k, fm[p + nm])
        q, kk, v = g("self_attn.q_proj", cfg.q_dim, cfg.d_model), g("self_attn.k_proj", cfg.kv_dim, cfg.d_model), g("self_attn.v_proj", cfg.kv_dim, cfg.d_model)
        if not (q.bits == kk.bits == v.bits and q.group == kk.group == v.group):
            raise ValueError(f"layer {l}: q/k/v use different bit widths or group sizes; they share one fused kernel launch")
        gate, up = g("mlp.gate_proj", cfg.ffn, cfg.d_model), g("mlp.up_proj", cfg.ffn, cfg.d_model)
        if gate.bits != up.bits or gate.group != up.group:
            raise ValueError(f"layer {l}: gate/up use different bit widths or group sizes")
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
    embed = files[wm[root + "embed_tokens.weight"]].tensor(root + "embed_tokens.weight").clone()
    final_norm = files[wm[root + "norm.weight"]].tensor(root + "norm.weight").clone()
    if tied:
        qd["lm_head"] = quant.quantize(embed.float(), BF16_LOAD_BITS, 128)       # tied head: the embedding, quantised once
    else:
        qd["lm_head"] = _get_linear(files, wm, "lm_head", cfg.vocab, cfg.d_model, fm["lm_head"])
    cfg.lm_head_bits = qd["lm_head"].bits
    for f in files.values():
        f.close()
    return CheckpointWeights(cfg, embed, layers, final_norm, qd, list(rep.get("unexpected", [])))


# ---- streaming load: packed tensors go to the device as they are and are repacked there ------------------------------

def _device_linear(parts, device, rows=None, kcut=None, interleave=False):
    """One engine linear from checkpoint linears that share k, bits and group.  ``parts``: list of (packed int32 [n, w],
    scale [n, g], zero or None, n, k, bits, group) views into the mapped files.  ``rows``: per-part row ranges (a
    column-parallel shard), ``kcut``: (k0, k1) input range (a row-parallel shard; word- and group-aligned).  The bit
    streams are only sliced and concatenated; the device kernel ``b2_wq_repack`` turns them into the kernel layout, so no
    code is ever expanded on the host (reference: crates/agens-cuda/src/lib.rs:163-214, kernels/src/w4_gemv.cu:441)."""
    from ..ops import linear as L
    _, _, _, _, k, bits, group = parts[0]
    packs, scales, zeros = [], [], []
    for i, (pk, sc, zp, n, _k, _b, _g) in enumerate(parts):
        lo, hi = rows[i] if rows is not None else (0, n)
        pk, sc = pk[lo:hi], sc[lo:hi]
        zp = None if zp is None else zp[lo:hi]
        if kcut is not None:
            k0, k1 = kcut
            assert (k0 * bits) % 32 == 0 and (k1 * bits) % 32 == 0 and k0 % group == 0 and k1 % group == 0
            pk = pk[:, k0 * bits // 32:k1 * bits // 32]
            sc = sc[:, k0 // group:k1 // group]
            zp = None if zp is None else zp[:, k0 // group:k1 // group]
        packs.append(pk.to(device)); scales.append(sc.to(device)); zeros.append(None if zp is None else zp.to(device))
    if any(z is None for z in zeros) and not all(z is None for z in zeros):
        zeros = [z if z is not None else torch.full_like(s_, float(1 << (bits - 1)), dtype=torch.float16) for z, s_ in zip(zeros, scales)]
    pk = torch.cat(packs) if len(packs) > 1 else packs[0]
    sc = torch.cat(scales) if len(scales) > 1 else scales[0]
    zp = None if zeros[0] is None else (torch.cat(zeros) if len(zeros) > 1 else zeros[0])
    if interleave:                      # gate rows and up rows in blocks of eight (see quant.interleave_gate_up)
        f = pk.shape[0] // 2
        idx = torch.arange(2 * f, device=device).reshape(2, f // 8, 8).permute(1, 0, 2).reshape(-1)
        pk, sc = pk[idx], sc[idx]
        zp = None if zp is None else zp[idx]
    kk = k if kcut is None else kcut[1] - kcut[0]
    return L.WqLinear.from_checkpoint(pk.contiguous(), sc.contiguous(), None if zp is None else zp.contiguous(),
                                      pk.shape[0], kk, bits, group, device)


def load_model(dir_: str, device="cuda:0", rank: int = 0, world: int = 1, **kw):
    """Builds a :class:`DenseModel` (or this rank's :class:`TpDenseModel` shard) from a checkpoint directory.

    Quantised linears stream from the memory-mapped shards to the device in their packed form and are repacked there;
    peak host memory is the page cache of one tensor.  bf16 linears stay bf16 on one GPU (see ``keep_bf16`` below);
    a tied lm_head, and bf16 linears of a tensor-parallel load, are quantised at load (asymmetric 4 bits, group 128)."""
    from ..models.config import LINEARS
    from ..models.dense import DenseModel
    from ..ops import linear as L
    rep, cfg, wm, files, tied = _open(dir_)
    fm, root = rep["linears"], rep.get("root", "model.")
    dev = torch.device(device)
    if world > 1:
        from ..parallel.tp_model import TpDenseModel
        m = TpDenseModel(cfg, dev, rank, world, **kw)
        lc = m.cfg
    else:
        m = DenseModel(cfg, dev, **kw)
        lc = cfg
    hd = cfg.head_dim
    hq, hkv, f = lc.n_heads, lc.n_kv_heads, lc.ffn

    def part(name, n, k):
        fmt = fm[name]
        if fmt["format"] == "bf16":
            ql = quant.quantize(files[wm[name + ".weight"]].tensor(name + ".weight").float(), BF16_LOAD_BITS, 128)
            return (quant.pack_stream(ql.codes, ql.bits), ql.scale, ql.zero, n, k, ql.bits, ql.group)
        T = lambda suf: files[wm[name + suf]].tensor(name + suf)
        zp = T(".weight_zero_point") if fmt["asymmetric"] else None
        return (T(".weight_packed"), T(".weight_scale"), zp, n, k, fmt["bits"], fmt["group"])

    # Linears stored as bf16 stay bf16 on one GPU (Bf16Linear: bf16 GEMV / tcgen05 GEMM) when every tensor of the fused
    # launch is bf16; B200E_BF16_LINEARS=quant, a tensor-parallel load or a mixed group quantises them at load instead.
    keep_bf16 = world == 1 and os.environ.get("B200E_BF16_LINEARS", "bf16") != "quant"

    def all_bf16(*names):
        return keep_bf16 and all(fm[n_]["format"] == "bf16" for n_ in names)

    def raw(name):
        return files[wm[name + ".weight"]].tensor(name + ".weight")

    for l in range(cfg.n_layers):
        p = f"{root}layers.{l}."
        groups = {"qkv": [p + "self_attn.q_proj", p + "self_attn.k_proj", p + "self_attn.v_proj"], "o": [p + "self_attn.o_proj"],
                  "gate_up": [p + "mlp.gate_proj", p + "mlp.up_proj"], "down": [p + "mlp.down_proj"]}
        if any(all_bf16(*grp) for grp in groups.values()):
            d = {}
            shapes = {"qkv": [(cfg.q_dim, cfg.d_model), (cfg.kv_dim, cfg.d_model), (cfg.kv_dim, cfg.d_model)], "o": [(cfg.d_model, cfg.q_dim)],
                      "gate_up": [(cfg.ffn, cfg.d_model)] * 2, "down": [(cfg.d_model, cfg.ffn)]}
            for lin, names in groups.items():
                if all_bf16(*names):
                    if lin == "gate_up":
                        w = quant.interleave_gate_up(raw(names[0]), raw(names[1]))
                    else:
                        w = torch.cat([raw(n_) for n_ in names]) if len(names) > 1 else raw(names[0])
                    d[lin] = L.Bf16Linear.from_tensor(w, dev)
                else:
                    parts_ = [part(n_, *shp) for n_, shp in zip(names, shapes[lin])]
                    if len({(x[5], x[6]) for x in parts_}) != 1:
                        raise ValueError(f"layer {l}: the tensors of {lin} use different bit widths or group sizes; they share one launch")
                    d[lin] = _device_linear(parts_, dev, interleave=(lin == "gate_up"))
            T = lambda nm: files[wm[p + nm]].tensor(p + nm).to(dev)
            d["ln1"], d["ln2"] = T("input_layernorm.weight"), T("post_attention_layernorm.weight")
            m.layers.append(d)
            for lin in LINEARS:
                cfg.bits[f"{l}.{lin}"] = d[lin].bits
            continue
        q, kk, v = part(p + "self_attn.q_proj", cfg.q_dim, cfg.d_model), part(p + "self_attn.k_proj", cfg.kv_dim, cfg.d_model), \
            part(p + "self_attn.v_proj", cfg.kv_dim, cfg.d_model)
        if not (q[5] == kk[5] == v[5] and q[6] == kk[6] == v[6]):
            raise ValueError(f"layer {l}: q/k/v use different bit widths or group sizes; they share one fused kernel launch")
        gate, up = part(p + "mlp.gate_proj", cfg.ffn, cfg.d_model), part(p + "mlp.up_proj", cfg.ffn, cfg.d_model)
        if gate[5] != up[5] or gate[6] != up[6]:
            raise ValueError(f"layer {l}: gate/up use different bit widths or group sizes")
        d = {
            "qkv": _device_linear([q, kk, v], dev, rows=[(rank * hq * hd, (rank + 1) * hq * hd), (rank * hkv * hd, (rank + 1) * hkv * hd),
                                                        (rank * hkv * hd, (rank + 1) * hkv * hd)]),
            "o": _device_linear([part(p + "self_attn.o_proj", cfg.d_model, cfg.q_dim)], dev, kcut=(rank * hq * hd, (rank + 1) * hq * hd)),
            "gate_up": _device_linear([gate, up], dev, rows=[(rank * f, (rank + 1) * f)] * 2, interleave=True),
            "down": _device_linear([part(p + "mlp.down_proj", cfg.d_model, cfg.ffn)], dev, kcut=(rank * f, (rank + 1) * f)),
        }
        T = lambda nm: files[wm[p + nm]].tensor(p + nm).to(dev)
        d["ln1"], d["ln2"] = T("input_layernorm.weight"), T("post_attention_layernorm.weight")
        m.layers.append(d)
        for lin in LINEARS:
            cfg.bits[f"{l}.{lin}"] = d[lin].bits
    embed_cpu = files[wm[root + "embed_tokens.weight"]].tensor(root + "embed_tokens.weight")
    m.embed = embed_cpu.to(dev)
    m.final_norm = files[wm[root + "norm.weight"]].tensor(root + "norm.weight").to(dev)
    # lm_head: vocabulary shard of this rank, padded with zero rows to whole panels
    if tied:
        ql = quant.quantize(embed_cpu.float(), BF16_LOAD_BITS, 128)
        lm = (quant.pack_stream(ql.codes, ql.bits), ql.scale, ql.zero, cfg.vocab, cfg.d_model, ql.bits, ql.group)
    else:
        lm = part("lm_head", cfg.vocab, cfg.d_model)
    if world > 1:
        lo, hi = rank * m.vocab_shard, min(cfg.vocab, (rank + 1) * m.vocab_shard)
    else:
        lo, hi = 0, cfg.vocab
    head = _device_linear([lm], dev, rows=[(lo, hi)])
    pad = m.lm_rows - (hi - lo)
    if pad:
        zq = quant.QuantLinear(pad, cfg.d_model, head.bits, head.group, torch.zeros(pad, cfg.d_model, dtype=torch.uint8),
                               torch.zeros(pad, cfg.d_model // head.group, dtype=torch.float16),
                               torch.zeros(pad, cfg.d_model // head.group, dtype=torch.float16))
        padl = L.WqLinear.from_quant(zq, dev)
        head = L.WqLinear(m.lm_rows, cfg.d_model, head.bits, head.group, torch.cat([head.wq, padl.wq]), head.ks, L.choose_rb(m.lm_rows))
    m.lm_head = head
    cfg.lm_head_bits = head.bits
    m.unexpected_tensors = list(rep.get("unexpected", []))
    for fl in files.values():
        fl.close()
    return m.finalize()


# ---------------------------------------------------------------------------------------------------- MTP head
MTP_NORMS = ("pre_fc_norm_embedding.weight", "pre_fc_norm_hidden.weight", "norm.weight", "layers.0.input_layernorm.weight",
             "layers.0.post_attention_layernorm.weight")
MTP_LINEARS = ("fc.weight", "layers.0.self_attn.q_proj.weight", "layers.0.self_attn.k_proj.weight",
               "layers.0.self_attn.v_proj.weight", "layers.0.self_attn.o_proj.weight", "layers.0.mlp.gate_proj.weight",
               "layers.0.mlp.up_proj.weight", "layers.0.mlp.down_proj.weight")


def read_mtp(dir_: str, cfg) -> Dict[str, torch.Tensor]:
    """Reads an MTP head checkpoint: bf16 tensors named ``mtp.*`` in the ``*.safetensors`` files of ``dir_`` (the
    layout of the reference's exporter; reader: crates/agens-cli/src/spec.rs:306-370).  Returns the tensors by their
    name without the prefix, on the host, after checking that every tensor the dense-shaped head needs is there, is
    bf16 and has the shape ``cfg`` implies.  Tensors of other head designs (``q_norm`` / ``k_norm``) are listed under
    the key ``"_unexpected"`` and ignored."""
    d, f = cfg.d_model, cfg.ffn
    want = {"fc.weight": (d, 2 * d), "layers.0.self_attn.q_proj.weight": (cfg.q_dim, d),
            "layers.0.self_attn.k_proj.weight": (cfg.kv_dim, d), "layers.0.self_attn.v_proj.weight": (cfg.kv_dim, d),
            "layers.0.self_attn.o_proj.weight": (d, cfg.q_dim), "layers.0.mlp.gate_proj.weight": (f, d),
            "layers.0.mlp.up_proj.weight": (f, d), "layers.0.mlp.down_proj.weight": (d, f)}
    want.update({n: (d,) for n in MTP_NORMS})
    out: Dict[str, torch.Tensor] = {}
    extra = []
    names = sorted(x for x in os.listdir(dir_) if x.endswith(".safetensors"))
    if not names:
        raise FileNotFoundError(f"mtp {dir_}: no .safetensors file")
    for fn in names:
        st = SafeTensorsFile(os.path.join(dir_, fn))
        for full in st.keys():
            if not full.startswith("mtp."):
                continue
            name = full[4:]
            if name not in want:
                extra.append(full)
                continue
            info = st.info[full]
            if info["dtype"] != "BF16":
                raise ValueError(f"mtp {full}: {info['dtype']} (bf16 expected)")
            if tuple(info["shape"]) != want[name]:
                raise ValueError(f"mtp {full}: shape {tuple(info['shape'])}, expected {want[name]}")
            out[name] = st.tensor(full).clone()
        st.close()
    missing = [n for n in want if n not in out]
    if missing:
        raise ValueError(f"mtp {dir_}: missing tensors {missing}")
    out["_unexpected"] = extra
    return out


def load_lm_head(dir_: str, device, rows: Optional[int] = None):
    """The whole (unsharded) lm_head of the model checkpoint ``dir_`` as an engine linear, padded with zero rows to
    ``rows``: what a head beside a tensor-parallel target needs (the target itself holds a vocabulary shard)."""
    from ..ops import linear as L
    rep, cfg, wm, files, tied = _open(dir_)
    fm, root = rep["linears"], rep.get("root", "model.")
    if tied or fm["lm_head"]["format"] == "bf16":
        name = root + "embed_tokens.weight" if tied else "lm_head.weight"
        ql = quant.quantize(files[wm[name]].tensor(name).float(), BF16_LOAD_BITS, 128)
        lm = (quant.pack_stream(ql.codes, ql.bits), ql.scale, ql.zero, cfg.vocab, cfg.d_model, ql.bits, ql.group)
    else:
        fmt = fm["lm_head"]
        T = lambda suf: files[wm["lm_head" + suf]].tensor("lm_head" + suf)
        lm = (T(".weight_packed"), T(".weight_scale"), T(".weight_zero_point") if fmt["asymmetric"] else None, cfg.vocab, cfg.d_model,
              fmt["bits"], fmt["group"])
    head = _device_linear([lm], torch.device(device))
    rows = rows or (cfg.vocab + 31) // 32 * 32
    pad = rows - cfg.vocab
    if pad:
        zq = quant.QuantLinear(pad, cfg.d_model, head.bits, head.group, torch.zeros(pad, cfg.d_model, dtype=torch.uint8),
                               torch.zeros(pad, cfg.d_model // head.group, dtype=torch.float16),
                               torch.zeros(pad, cfg.d_model // head.group, dtype=torch.float16))
        padl = L.WqLinear.from_quant(zq, device)
        head = L.WqLinear(rows, cfg.d_model, head.bits, head.group, torch.cat([head.wq, padl.wq]), head.ks, L.choose_rb(rows))
    for fl in files.values():
        fl.close()
    return head


def load_mtp(dir_: str, target, bits: int = BF16_LOAD_BITS, lm_head_dir: Optional[str] = None, **kw):
    """An :class:`~agens_engine_b200.models.mtp.MtpHead` for ``target`` from the ``mtp.*`` tensors of ``dir_``.  The
    linears are quantised at load (asymmetric, ``bits`` bits, group 128 or the model's group when that is smaller; the
    reference quantises its head to 4-bit group 128 at load as well, spec.rs:318-340); gate and up are merged row-interleaved as in the main model; embedding and
    lm_head stay the target's."""
    from ..models.mtp import MtpHead
    from ..ops import linear as L
    t = read_mtp(dir_, getattr(target, "full_cfg", None) or target.cfg)
    dev = target.dev
    h = MtpHead(target, **kw)
    if h.own_lm_head:          # beside a tensor-parallel target: the whole lm_head comes from the model's checkpoint
        if not lm_head_dir:
            raise ValueError("an MTP head beside a tensor-parallel model needs the model checkpoint for its lm_head (lm_head_dir)")
        h.lm_head = load_lm_head(lm_head_dir, dev, rows=h.lm_rows)

    def lin(*names, interleave=False):
        if interleave:
            w = quant.interleave_gate_up(t[names[0]].float(), t[names[1]].float())
        else:
            w = torch.cat([t[n].float() for n in names])
        return L.WqLinear.from_quant(quant.quantize(w, bits, min(128, h.cfg.group)), dev)

    p = "layers.0."
    h.layers.append({
        "qkv": lin(p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight", p + "self_attn.v_proj.weight"),
        "o": lin(p + "self_attn.o_proj.weight"),
        "gate_up": lin(p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight", interleave=True),
        "down": lin(p + "mlp.down_proj.weight"),
        "ln1": t[p + "input_layernorm.weight"].to(dev), "ln2": t[p + "post_attention_layernorm.weight"].to(dev)})
    h.fc = lin("fc.weight")
    h.norm_e, h.norm_h = t["pre_fc_norm_embedding.weight"].to(dev), t["pre_fc_norm_hidden.weight"].to(dev)
    h.final_norm = t["norm.weight"].to(dev)
    h.unexpected_tensors = t["_unexpected"]
    return h.finalize()
