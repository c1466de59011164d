"""Vision encoder (ViT with 2-D rotary attention and a 2x2 patch merger) producing the embedding rows that replace
image placeholder tokens in prefill.

Structure (reference: ``kernels/oracle/bridge/vision.cpp:105-199``): patch embed = one linear over 2x16x16x3 patches
(+bias); learned position table interpolated bilinearly (align-corners) to the image grid; ``depth`` pre-LN blocks of
LayerNorm -> fused qkv (+bias) -> rotary on q, k -> full non-causal attention -> proj (+bias) -> residual; LayerNorm ->
fc1 -> GELU(tanh) -> fc2 -> residual; merger = LayerNorm -> [N/4, 4 d] -> fc1 -> GELU(erf) -> fc2 -> [N/4, out_dim].
Rows are in merge-block order throughout.  Linears run on the tcgen05 GEMM, the rest on the kernels of
``csrc/kernels/sm100/vision.cu``; weights may stay in pinned host memory and be streamed one block ahead.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import math
from typing import Dict, List, Optional, Tuple

import torch

from .. import _lib
from .._lib import check, current_stream, ptr
from ..ops.gemm import gemm_bf16

_sig = False


def _k():
    global _sig
    lib = _lib.cuda_lib()
    if not _sig:
        vp, i, l, f = C.c_void_p, C.c_int, C.c_long, C.c_float
        for name, args in {"b2_layernorm": [vp, l, vp, vp, f, vp, l, i, i, vp],
                           "b2_bias_act": [vp, l, vp, i, vp, l, vp, l, i, i, vp],
                           "b2_rope2d": [vp, l, vp, vp, i, i, i, vp],
                           "b2_attn_full": [vp, l, vp, l, i, i, i, f, vp]}.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, i
        _sig = True
    return lib


@dataclasses.dataclass
class VisionConfig:
    depth: int = 27
    d_model: int = 1152
    n_heads: int = 16
    mlp: int = 4304
    patch_dim: int = 1536
    out_dim: int = 5120
    pos_grid: int = 48
    eps: float = 1e-6

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads


def layernorm(x, w, b, eps):
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(_k().b2_layernorm(ptr(x), x.stride(0), ptr(w), ptr(b), eps, ptr(out), out.stride(0), x.shape[0], x.shape[1], current_stream()), "b2_layernorm")
    return out


def bias_act(x, bias, act=0, resid=None):
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(_k().b2_bias_act(ptr(x), x.stride(0), ptr(bias), act, ptr(resid), resid.stride(0) if resid is not None else 0, ptr(out),
                               out.stride(0), x.shape[0], x.shape[1], current_stream()), "b2_bias_act")
    return out


def rope2d(qkv, cos, sin, n_heads, head_dim):
    with torch.cuda.device(qkv.device):
        check(_k().b2_rope2d(ptr(qkv), qkv.stride(0), ptr(cos), ptr(sin), qkv.shape[0], n_heads, head_dim, current_stream()), "b2_rope2d")


def attn_full(qkv, n_heads, head_dim):
    N = qkv.shape[0]
    out = torch.empty(N, n_heads * head_dim, dtype=torch.bfloat16, device=qkv.device)
    with torch.cuda.device(qkv.device):
        check(_k().b2_attn_full(ptr(qkv), qkv.stride(0), ptr(out), out.stride(0), N, n_heads, head_dim, 1.0 / math.sqrt(head_dim),
                                current_stream()), "b2_attn_full")
    return out


def merge_order(gh: int, gw: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(row, col) of every patch in merge-block order (gh/2, gw/2, 2, 2)."""
    r = torch.arange(gh).view(gh // 2, 2, 1, 1).expand(gh // 2, 2, gw // 2, 2).permute(0, 2, 1, 3).reshape(-1)
    c = torch.arange(gw).view(1, 1, gw // 2, 2).expand(gh // 2, 2, gw // 2, 2).permute(0, 2, 1, 3).reshape(-1)
    return r, c


def rotary_tables(cfg: VisionConfig, gh: int, gw: int):
    """fp32 cos/sin [N, head_dim]: hd/4 frequencies for the row, hd/4 for the column, the pair duplicated."""
    hd = cfg.head_dim
    nf = hd // 4
    inv = 10000.0 ** (-torch.arange(nf, dtype=torch.float32) * 2.0 / (hd // 2))
    r, c = merge_order(gh, gw)
    ang = torch.cat([r[:, None].float() * inv, c[:, None].float() * inv], 1)          # [N, hd/2]
    ang = torch.cat([ang, ang], 1)
    return torch.cos(ang).contiguous(), torch.sin(ang).contiguous()


def interp_pos(table: torch.Tensor, grid: int, gh: int, gw: int) -> torch.Tensor:
    """Bilinear interpolation (align-corners linspace) of the learned [grid*grid, d] table to gh x gw, in merge-block
    order; fp32 arithmetic on bf16 table rows."""
    ys = torch.linspace(0, grid - 1, gh, dtype=torch.float32)
    xs = torch.linspace(0, grid - 1, gw, dtype=torch.float32)
    y0, x0 = ys.floor().long(), xs.floor().long()
    y1, x1 = (y0 + 1).clamp(max=grid - 1), (x0 + 1).clamp(max=grid - 1)
    fy, fx = (ys - y0.float()), (xs - x0.float())
    r, c = merge_order(gh, gw)
    t = table.float()
    dev = table.device
    g = lambda yy, xx: t[(yy[r] * grid + xx[c]).to(dev)]
    wy, wx = fy[r].to(dev)[:, None], fx[c].to(dev)[:, None]
    return g(y0, x0) * (1 - wy) * (1 - wx) + g(y0, x1) * (1 - wy) * wx + g(y1, x0) * wy * (1 - wx) + g(y1, x1) * wy * wx


class VisionTower:
    def __init__(self, cfg: VisionConfig, device="cuda:0", resident: bool = True):
        self.cfg, self.dev, self.resident = cfg, torch.device(device), resident
        self.w: Dict[str, torch.Tensor] = {}
        self.blocks: List[Dict[str, torch.Tensor]] = []
        self.copy_stream = torch.cuda.Stream(device=self.dev) if torch.cuda.is_available() else None

    @staticmethod
    def random_init(cfg: VisionConfig, device="cuda:0", seed: int = 0, resident: bool = True) -> "VisionTower":
        t = VisionTower(cfg, device, resident)
        g = torch.Generator().manual_seed(seed)
        d = cfg.d_model
        W = lambda n, k: (torch.randn(n, k, generator=g) / math.sqrt(k)).to(torch.bfloat16)
        B = lambda n: (torch.randn(n, generator=g) * 0.02).to(torch.bfloat16)
        G = lambda n: (1 + 0.05 * torch.randn(n, generator=g)).to(torch.bfloat16)
        put = (lambda x: x.to(t.dev)) if resident else (lambda x: x.pin_memory())
        t.w = {k: v.to(t.dev) for k, v in {
            "patch_w": W(d, cfg.patch_dim), "patch_b": B(d), "pos": (torch.randn(cfg.pos_grid ** 2, d, generator=g) * 0.02).to(torch.bfloat16),
            "m_ln_w": G(d), "m_ln_b": B(d), "m_fc1_w": W(4 * d, 4 * d), "m_fc1_b": B(4 * d), "m_fc2_w": W(cfg.out_dim, 4 * d),
            "m_fc2_b": B(cfg.out_dim)}.items()}
        for _ in range(cfg.depth):
            t.blocks.append({k: put(v) for k, v in {
                "ln1_w": G(d), "ln1_b": B(d), "qkv_w": W(3 * d, d), "qkv_b": B(3 * d), "proj_w": W(d, d), "proj_b": B(d),
                "ln2_w": G(d), "ln2_b": B(d), "fc1_w": W(cfg.mlp, d), "fc1_b": B(cfg.mlp), "fc2_w": W(d, cfg.mlp), "fc2_b": B(d)}.items()})
        return t

    # names of the tower's tensors in a checkpoint (``model.visual.`` + ...), as the reference registers them
    # (kernels/oracle/bridge/vision.cpp:56-61, :114; loader crates/agens-cli/src/m1.rs:338-360)
    _TOP = {"patch_embed.proj.weight": "patch_w", "patch_embed.proj.bias": "patch_b", "pos_embed.weight": "pos",
            "merger.norm.weight": "m_ln_w", "merger.norm.bias": "m_ln_b", "merger.linear_fc1.weight": "m_fc1_w",
            "merger.linear_fc1.bias": "m_fc1_b", "merger.linear_fc2.weight": "m_fc2_w", "merger.linear_fc2.bias": "m_fc2_b"}
    _BLOCK = {"norm1.weight": "ln1_w", "norm1.bias": "ln1_b", "attn.qkv.weight": "qkv_w", "attn.qkv.bias": "qkv_b",
              "attn.proj.weight": "proj_w", "attn.proj.bias": "proj_b", "norm2.weight": "ln2_w", "norm2.bias": "ln2_b",
              "mlp.linear_fc1.weight": "fc1_w", "mlp.linear_fc1.bias": "fc1_b", "mlp.linear_fc2.weight": "fc2_w",
              "mlp.linear_fc2.bias": "fc2_b"}

    @staticmethod
    def has_tower(dir_: str, prefix: str = "model.visual.") -> bool:
        """Whether the checkpoint directory carries vision tower tensors."""
        import json
        import os
        idx = os.path.join(dir_, "model.safetensors.index.json")
        if os.path.exists(idx):
            return any(k.startswith(prefix) for k in json.load(open(idx))["weight_map"])
        from ..utils.checkpoint import SafeTensorsFile
        one = os.path.join(dir_, "model.safetensors")
        return os.path.exists(one) and any(k.startswith(prefix) for k in SafeTensorsFile(one).keys())

    @staticmethod
    def from_checkpoint(dir_: str, device="cuda:0", n_heads: int = 16, resident: bool = True, prefix: str = "model.visual.",
                        eps: float = 1e-6) -> "VisionTower":
        """The checkpoint's own tower: bf16 tensors ``model.visual.*`` of the safetensors shards in ``dir_``.  Sizes come
        from the tensors (depth = number of blocks, width, MLP width, patch size, position grid, output width); only the
        head count is not in them.  ``resident=False`` keeps the blocks in pinned host memory and streams them per layer
        at encode time, as the reference does."""
        import json
        import os
        from ..utils.checkpoint import SafeTensorsFile
        idx = os.path.join(dir_, "model.safetensors.index.json")
        if os.path.exists(idx):
            wm = {k: v for k, v in json.load(open(idx))["weight_map"].items() if k.startswith(prefix)}
        else:
            wm = {k: "model.safetensors" for k in SafeTensorsFile(os.path.join(dir_, "model.safetensors")).keys() if k.startswith(prefix)}
        if not wm:
            raise ValueError(f"{dir_}: no {prefix}* tensors")
        files = {fn: SafeTensorsFile(os.path.join(dir_, fn)) for fn in set(wm.values())}

        def get(name):
            full = prefix + name
            if full not in wm:
                raise ValueError(f"vision tower: missing tensor {full}")
            f = files[wm[full]]
            if f.info[full]["dtype"] != "BF16":
                raise ValueError(f"{full}: vision tensors must be bf16 (got {f.info[full]['dtype']})")
            return f.tensor(full).clone()

        depth = 1 + max(int(k[len(prefix) + 7:].split(".")[0]) for k in wm if k.startswith(prefix + "blocks."))
        top = {mine: get(name) for name, mine in VisionTower._TOP.items()}
        d = top["patch_w"].shape[0]
        top["patch_w"] = top["patch_w"].reshape(d, -1).contiguous()              # [d, channels x (frames x) patch x patch]
        grid = int(round(math.sqrt(top["pos"].shape[0])))
        blocks = [{mine: get(f"blocks.{i}.{name}") for name, mine in VisionTower._BLOCK.items()} for i in range(depth)]
        cfg = VisionConfig(depth=depth, d_model=d, n_heads=n_heads, mlp=blocks[0]["fc1_w"].shape[0], patch_dim=top["patch_w"].shape[1],
                           out_dim=top["m_fc2_w"].shape[0], pos_grid=grid, eps=eps)
        if grid * grid != top["pos"].shape[0] or d % n_heads or tuple(top["m_fc1_w"].shape) != (4 * d, 4 * d) or \
                tuple(blocks[0]["qkv_w"].shape) != (3 * d, d):
            raise ValueError("vision tower: tensor shapes do not fit together")
        t = VisionTower(cfg, device, resident)
        put = (lambda x: x.to(t.dev)) if resident or t.dev.type != "cuda" else (lambda x: x.pin_memory())
        t.w = {k: v.to(t.dev) for k, v in top.items()}
        t.blocks = [{k: put(v) for k, v in b.items()} for b in blocks]
        for f in files.values():
            f.close()
        return t

    def weight_bytes(self) -> int:
        return sum(v.numel() * 2 for v in self.w.values()) + sum(v.numel() * 2 for b in self.blocks for v in b.values())

    def _fetch(self, i: int):
        """Block weights on the device: resident ones as they are, host ones copied on the side stream."""
        if self.resident:
            return self.blocks[i], None
        with torch.cuda.stream(self.copy_stream):
            blk = {k: v.to(self.dev, non_blocking=True) for k, v in self.blocks[i].items()}
            ev = torch.cuda.Event()
            ev.record(self.copy_stream)
        return blk, ev

    def encode(self, patches: torch.Tensor, grid: Tuple[int, int]) -> torch.Tensor:
        """patches: [gh*gw, patch_dim] (merge-block order); returns bf16 [gh*gw/4, out_dim]."""
        cfg, dev = self.cfg, self.dev
        gh, gw = grid
        N, d, H, hd = gh * gw, cfg.d_model, cfg.n_heads, cfg.head_dim
        main = torch.cuda.current_stream(dev)
        x = patches.to(dev, torch.bfloat16).contiguous()
        pos = interp_pos(self.w["pos"], cfg.pos_grid, gh, gw).to(torch.bfloat16)
        h = bias_act(gemm_bf16(x, self.w["patch_w"]), self.w["patch_b"], 0, resid=pos)
        cos, sin = (t.to(dev) for t in rotary_tables(cfg, gh, gw))
        nxt = self._fetch(0)
        for i in range(cfg.depth):
            blk, ev = nxt
            if ev is not None:
                main.wait_event(ev)
            if i + 1 < cfg.depth:
                nxt = self._fetch(i + 1)                     # one block ahead, overlapping this block's compute
            y = layernorm(h, blk["ln1_w"], blk["ln1_b"], cfg.eps)
            qkv = bias_act(gemm_bf16(y, blk["qkv_w"]), blk["qkv_b"])
            rope2d(qkv, cos, sin, H, hd)
            a = attn_full(qkv, H, hd)
            h = bias_act(gemm_bf16(a, blk["proj_w"]), blk["proj_b"], 0, resid=h)
            y = layernorm(h, blk["ln2_w"], blk["ln2_b"], cfg.eps)
            y = bias_act(gemm_bf16(y, blk["fc1_w"]), blk["fc1_b"], 1)
            h = bias_act(gemm_bf16(y, blk["fc2_w"]), blk["fc2_b"], 0, resid=h)
            if ev is not None:
                for v in blk.values():
                    v.record_stream(main)
        y = layernorm(h, self.w["m_ln_w"], self.w["m_ln_b"], cfg.eps).view(N // 4, 4 * d)
        y = bias_act(gemm_bf16(y, self.w["m_fc1_w"]), self.w["m_fc1_b"], 2)
        return bias_act(gemm_bf16(y, self.w["m_fc2_w"]), self.w["m_fc2_b"])

    # ------------------------------------------------------------------------------------------------ fp32 restatement
    def encode_ref(self, patches: torch.Tensor, grid: Tuple[int, int]) -> torch.Tensor:
        """The same computation with plain fp32 tensor operations (oracle)."""
        import torch.nn.functional as F
        cfg = self.cfg
        gh, gw = grid
        N, d, H, hd = gh * gw, cfg.d_model, cfg.n_heads, cfg.head_dim
        f = lambda v: v.to(self.dev).float()
        x = patches.to(self.dev, torch.bfloat16).float()
        h = x @ f(self.w["patch_w"]).T + f(self.w["patch_b"]) + interp_pos(self.w["pos"], cfg.pos_grid, gh, gw)
        cos, sin = (t.to(self.dev) for t in rotary_tables(cfg, gh, gw))

        def rope(v):                                         # [N, H, hd]
            half = hd // 2
            rot = torch.cat([-v[..., half:], v[..., :half]], -1)
            return v * cos[:, None, :] + rot * sin[:, None, :]

        for blk in self.blocks:
            y = F.layer_norm(h, (d,), f(blk["ln1_w"]), f(blk["ln1_b"]), cfg.eps)
            qkv = (y @ f(blk["qkv_w"]).T + f(blk["qkv_b"])).view(N, 3, H, hd)
            q, k, v = rope(qkv[:, 0]), rope(qkv[:, 1]), qkv[:, 2]
            s = torch.einsum("nhd,mhd->hnm", q, k) / math.sqrt(hd)
            a = torch.einsum("hnm,mhd->nhd", torch.softmax(s, -1), v).reshape(N, d)
            h = h + a @ f(blk["proj_w"]).T + f(blk["proj_b"])
            y = F.layer_norm(h, (d,), f(blk["ln2_w"]), f(blk["ln2_b"]), cfg.eps)
            y = F.gelu(y @ f(blk["fc1_w"]).T + f(blk["fc1_b"]), approximate="tanh")
            h = h + y @ f(blk["fc2_w"]).T + f(blk["fc2_b"])
        y = F.layer_norm(h, (d,), f(self.w["m_ln_w"]), f(self.w["m_ln_b"]), cfg.eps).view(N // 4, 4 * d)
        y = F.gelu(y @ f(self.w["m_fc1_w"]).T + f(self.w["m_fc1_b"]))
        return y @ f(self.w["m_fc2_w"]).T + f(self.w["m_fc2_b"])
