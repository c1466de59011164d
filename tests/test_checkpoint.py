"""Checkpoint container tests on the CPU (model: the reference's toy 4-layer checkpoint tests,
crates/agens-core/src/weights.rs:311-453: format detection, bad shapes, SHA sums, shard index cross-check)."""
import json
import os

import pytest
import torch

from agens_engine_b200.models import config as C
from agens_engine_b200.models import oracle as O
from agens_engine_b200.utils import checkpoint as K
from agens_engine_b200.utils import quant


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("ckpt"))
    ow = O.random_weights(C.oracle_tiny(), seed=1)
    K.save_oracle(d, ow, shards=3)
    return d, ow


def test_safetensors_roundtrip(tmp_path):
    p = str(tmp_path / "x.safetensors")
    t = {"a": torch.arange(12, dtype=torch.int32).reshape(3, 4), "b": torch.randn(5).to(torch.bfloat16), "e": torch.zeros(0, 3)}
    K.write_safetensors(p, t)
    f = K.SafeTensorsFile(p)
    assert set(f.keys()) == {"a", "b", "e"}
    assert torch.equal(f.tensor("a"), t["a"]) and torch.equal(f.tensor("b"), t["b"]) and f.tensor("e").shape == (0, 3)
    with pytest.raises(IOError):
        K.SafeTensorsFile(str(tmp_path / "missing.safetensors"))
    open(p, "r+b").write(b"\xff" * 8)
    with pytest.raises(IOError):
        K.SafeTensorsFile(p)


def test_validate_detects_formats(ckpt):
    d, ow = ckpt
    rep = K.validate(d)
    assert rep["ok"], rep["errors"]
    assert rep["shards"] == 3
    f = rep["linears"]
    assert f["model.layers.0.self_attn.q_proj"] == {"format": "wq", "bits": 4, "group": 64, "asymmetric": True, "scale_dtype": "F16"}
    assert f["model.layers.1.self_attn.o_proj"]["bits"] == 2 and f["model.layers.1.mlp.down_proj"]["bits"] == 3
    info = K.inspect(d)
    assert info["linear_formats"] == {"w4g64a": 8, "w2g64a": 4, "w3g64a": 3}


def test_sha256_verify_and_tamper(ckpt, tmp_path):
    d, _ = ckpt
    r = K.verify(d)
    assert r["files"] == 4 and r["ok"] == 4 and r["bad"] == []
    import hashlib
    fn = os.path.join(d, "config.json")
    assert K.sha256_file(fn) == hashlib.sha256(open(fn, "rb").read()).hexdigest()
    import shutil
    d2 = str(tmp_path / "t")
    shutil.copytree(d, d2)
    with open(os.path.join(d2, "config.json"), "a") as f:
        f.write(" ")
    r2 = K.verify(d2)
    assert r2["ok"] == 3 and r2["bad"][0]["file"] == "config.json"


def test_validate_reports_bad_shapes_and_index(ckpt, tmp_path):
    d, ow = ckpt
    import shutil
    d2 = str(tmp_path / "bad")
    shutil.copytree(d, d2)
    cfg = json.load(open(os.path.join(d2, "config.json")))
    cfg["intermediate_size"] = 640
    json.dump(cfg, open(os.path.join(d2, "config.json"), "w"))
    rep = K.validate(d2)
    assert not rep["ok"] and any("mlp.gate_proj" in e for e in rep["errors"])
    d3 = str(tmp_path / "idx")
    shutil.copytree(d, d3)
    idx = json.load(open(os.path.join(d3, "model.safetensors.index.json")))
    idx["weight_map"]["model.layers.9.ghost.weight"] = "model-00001-of-00003.safetensors"
    json.dump(idx, open(os.path.join(d3, "model.safetensors.index.json"), "w"))
    rep3 = K.validate(d3)
    assert not rep3["ok"] and any("ghost" in e for e in rep3["errors"])


def test_symmetric_reference_container(tmp_path):
    """The reference's own container: int4 nibbles (code = q + 8), bf16 scales, symmetric, no zero-point tensor."""
    cfg = C.oracle_tiny()
    cfg.bits = {}
    ow = O.random_weights(cfg, seed=2, symmetric=True)
    d = str(tmp_path / "sym")
    K.save_oracle(d, ow, symmetric=True)
    rep = K.validate(d)
    assert rep["ok"], rep["errors"]
    assert rep["linears"]["lm_head"] == {"format": "wq", "bits": 4, "group": 64, "asymmetric": False, "scale_dtype": "BF16"}
    f = K.SafeTensorsFile(os.path.join(d, "model.safetensors"))
    packed = f.tensor("model.layers.0.self_attn.o_proj.weight_packed")
    codes = quant.unpack_stream(packed, 4, cfg.q_dim)
    assert torch.equal(codes, ow.quant["0.o"].codes)


def test_reference_tensor_names_and_leftover_report(tmp_path):
    """Checkpoints that carry a vision tower name the text model ``model.language_model.*``; tensors of the text model
    that the loader has no use for (here: q_norm) are reported, not fatal."""
    d = str(tmp_path / "lm")
    cfg = C.oracle_tiny()
    ow = O.random_weights(cfg, seed=2)
    extra = {"model.language_model.layers.0.self_attn.q_norm.weight": torch.ones(cfg.head_dim, dtype=torch.bfloat16),
             "model.visual.patch_embed.proj.weight": torch.zeros(4, 4, dtype=torch.bfloat16)}
    K.save_oracle(d, ow, root="model.language_model.", extra=extra)
    rep = K.validate(d)
    assert rep["ok"], rep["errors"]
    assert rep["root"] == "model.language_model."
    assert rep["unexpected"] == ["model.language_model.layers.0.self_attn.q_norm.weight"]     # the vision tensor is not text
    w = K.read_weights(d)
    assert w.unexpected == rep["unexpected"]
    for k, ql in ow.quant.items():
        assert torch.equal(w.quant[k].codes, ql.codes), k
    assert torch.equal(w.embed, ow.embed)


def test_bf16_linears_and_tied_head_are_quantised_at_load(tmp_path):
    d = str(tmp_path / "bf")
    cfg = C.oracle_tiny()
    ow = O.random_weights(cfg, seed=3)
    K.save_oracle(d, ow, bf16_linears=("self_attn.o_proj",), tied=True)
    rep = K.validate(d)
    assert rep["ok"], rep["errors"]
    assert rep["linears"]["model.layers.0.self_attn.o_proj"]["format"] == "bf16" and "lm_head" not in rep["linears"]
    w = K.read_weights(d)
    o = w.quant["0.o"]
    assert o.bits == K.BF16_LOAD_BITS and o.group == 128
    ref = ow.quant["0.o"].dequant().to(torch.bfloat16).float()
    err = (o.dequant() - ref).abs().max().item()
    assert err <= 0.6 * float(o.scale.float().max())                       # within half a quantisation step
    head = w.quant["lm_head"]
    assert head.n == cfg.vocab and head.bits == K.BF16_LOAD_BITS
    assert (head.dequant() - ow.embed.float()).abs().max().item() <= 0.6 * float(head.scale.float().max())


def test_gated_q_proj_is_named_as_such(tmp_path):
    d = str(tmp_path / "gated")
    cfg = C.oracle_tiny()
    ow = O.random_weights(cfg, seed=4)
    K.save_oracle(d, ow, sums=False)
    f = K.SafeTensorsFile(os.path.join(d, "model.safetensors"))
    t = {k: f.tensor(k).clone() for k in f.keys()}
    f.close()
    for suf in (".weight_packed", ".weight_scale", ".weight_zero_point"):
        n = "model.layers.0.self_attn.q_proj" + suf
        t[n] = torch.cat([t[n], t[n]])
    K.write_safetensors(os.path.join(d, "model.safetensors"), t, {"format": "pt"})
    rep = K.validate(d)
    assert not rep["ok"] and any("gated attention" in e for e in rep["errors"])


def test_damaged_safetensors_headers_are_refused(tmp_path):
    """A header whose offsets, shapes or lengths do not describe the file is refused with a message; nothing is read
    past the mapping (development runs this reader on mutated files under AddressSanitizer)."""
    import json
    import struct
    from agens_engine_b200.utils.checkpoint import SafeTensorsFile
    good = {"a": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}

    def write(header, payload=bytes(16), hlen=None):
        hj = json.dumps(header).encode() if not isinstance(header, bytes) else header
        p = tmp_path / "x.safetensors"
        p.write_bytes(struct.pack("<Q", len(hj) if hlen is None else hlen) + hj + payload)
        return str(p)
    assert SafeTensorsFile(write(good)).tensor("a").shape == (2, 2)
    bad = [
        {"a": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0]}},                       # one offset only
        {"a": {"dtype": "F32", "shape": [2, 2], "data_offsets": []}},
        {"a": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 32]}},                   # past the end of the file
        {"a": {"dtype": "F32", "shape": [2, 2], "data_offsets": [-16, 0]}},
        {"a": {"dtype": "F32", "shape": [-2, -2], "data_offsets": [0, 16]}},                 # negative extents
        {"a": {"dtype": "F32", "shape": [4611686018427387904, 4, 1], "data_offsets": [0, 16]}},   # product wraps to 4
        {"a": {"dtype": "F32", "shape": [9223372036854775807, 9223372036854775807], "data_offsets": [0, 16]}},
        {"a": {"dtype": "F33", "shape": [2, 2], "data_offsets": [0, 16]}},
        {"a": {"dtype": "F32", "shape": "2x2", "data_offsets": [0, 16]}},
        {"a": [1, 2, 3]},
        b"{\"a\": ",
    ]
    for h in bad:
        with pytest.raises(IOError):
            SafeTensorsFile(write(h))
    for hlen in (2**63, 2**64 - 1, 10**6):
        with pytest.raises(IOError):
            SafeTensorsFile(write(good, hlen=hlen))


def test_sha256_portable_loop_in_a_process_of_its_own():
    """B200E_NO_SHA_NI=1 keeps the portable compression function: the same test in a fresh process."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, B200E_NO_SHA_NI="1")
    r = subprocess.run([sys.executable, "-m", "pytest", __file__, "-q", "-k", "equals_hashlib", "-p", "no:cacheprovider"], env=env,
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "1 passed" in r.stdout, r.stdout[-1500:] + r.stderr[-500:]


def test_sha256_equals_hashlib_at_every_length():
    """Both compression functions (the CPU's SHA extensions where it has them, the portable loop elsewhere) through the
    streaming interface: every length around the block and padding boundaries, and a few megabytes."""
    import ctypes as C
    import hashlib
    import os
    from agens_engine_b200 import _lib
    h = _lib.host_lib()
    h.b2h_sha256_bytes.restype = C.c_void_p
    h.b2h_sha256_bytes.argtypes = [C.c_char_p, C.c_longlong]
    h.b2h_free_str.argtypes = [C.c_void_p]
    data = os.urandom(3 * 1024 * 1024 + 17)
    for n in list(range(0, 260)) + [4095, 4096, 4097, 65536 + 55, 65536 + 56, 1 << 20, len(data)]:
        p = h.b2h_sha256_bytes(data[:n], n)
        got = C.string_at(p).decode()
        h.b2h_free_str(p)
        assert got == hashlib.sha256(data[:n]).hexdigest(), n
