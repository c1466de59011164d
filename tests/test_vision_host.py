"""Host image pipeline against torch's antialiased bicubic and hand-worked cases (reference: vision.rs tests :223 and
the preprocess contract of kernels/oracle/bridge/vision.cpp:234-256)."""
import base64
import json
import struct
import zlib

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from agens_engine_b200.serve import vision as V


def test_smart_resize_rules():
    assert V.smart_resize(480, 640) == (480, 640)
    assert V.smart_resize(100, 100) == (96, 96)
    assert V.smart_resize(50, 50) == (64, 64)                 # 48 x 48 would fall below min_pixels: scaled up
    assert V.smart_resize(16, 16) == (64, 64)
    h, w = V.smart_resize(4000, 6000)
    assert h % 32 == 0 and w % 32 == 0 and h * w <= V.MAX_PIXELS and abs(h / w - 4000 / 6000) < 0.02
    assert V.smart_resize(48, 80) == (64, 64)                 # 1.5 -> 2 and 2.5 -> 2: halves round to even
    with pytest.raises(ValueError):
        V.smart_resize(10, 4000)


@pytest.mark.parametrize("hw,size", [((97, 131), (64, 96)), ((40, 52), (96, 128)), ((300, 200), (160, 96)), ((64, 64), (64, 64))])
def test_bicubic_aa_matches_torch_and_patch_layout(hw, size):
    rng = np.random.default_rng(0)
    img = rng.integers(0, 256, size=(hw[0], hw[1], 3), dtype=np.uint8)
    patches, (gh, gw), resized = V.preprocess(img, size, want_resized=True)
    ref = F.interpolate(torch.from_numpy(img).permute(2, 0, 1)[None].float(), size=size, mode="bicubic", antialias=True,
                        align_corners=False)[0].numpy()
    assert np.abs(resized - ref).max() < 2e-3
    q = (np.rint(np.clip(resized, 0, 255)) - 127.5) / 127.5
    P = V.PATCH
    assert patches.shape == (gh * gw, 1536)
    # row order (gh/2, gw/2, 2, 2); columns (channel, time, py, px) with the frame duplicated in time
    row = 0
    for by in range(gh // 2):
        for bx in range(gw // 2):
            for iy in range(2):
                for ix in range(2):
                    gy, gx = by * 2 + iy, bx * 2 + ix
                    blk = q[:, gy * P:(gy + 1) * P, gx * P:(gx + 1) * P]
                    exp = np.stack([blk, blk], 1).reshape(-1)
                    assert np.array_equal(patches[row], exp.astype(np.float32)), row
                    row += 1


def test_placeholders_positions_and_decoders():
    PAD = 900
    ids = [1, 2, PAD, 3, PAD, 4]
    out = V.expand_placeholders(ids, PAD, [6, 2])
    assert out == [1, 2] + [PAD] * 6 + [3] + [PAD] * 2 + [4]
    with pytest.raises(ValueError):
        V.expand_placeholders(ids, PAD, [6])
    pos, nxt = V.mrope_positions(out, PAD, [(2, 3), (1, 2)])
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:8].tolist() == [2] * 6 and pos[1, 2:8].tolist() == [2, 2, 2, 3, 3, 3] and pos[2, 2:8].tolist() == [2, 3, 4, 2, 3, 4]
    assert pos[:, 8].tolist() == [5, 5, 5]                     # text resumes at 2 + max(2, 3)
    assert pos[0, 9:11].tolist() == [6, 6] and pos[2, 9:11].tolist() == [6, 7]
    assert pos[:, 11].tolist() == [8, 8, 8] and nxt == 9
    rng = np.random.default_rng(1)
    img = rng.integers(0, 256, size=(5, 7, 3), dtype=np.uint8)
    ppm = b"P6\n# comment\n7 5\n255\n" + img.tobytes()
    assert np.array_equal(V.decode_image(ppm), img)
    # PNG with every filter type
    raw = b""
    prev = np.zeros(21, dtype=np.int32)
    for y in range(5):
        line = img[y].reshape(-1).astype(np.int32)
        f = y % 5
        enc = np.zeros(21, dtype=np.int32)
        for x in range(21):
            a = line[x - 3] if x >= 3 else 0
            b, c = prev[x], (prev[x - 3] if x >= 3 else 0)
            pa, pb, pc = abs(b - c), abs(a - c), abs(a + b - 2 * c)
            pr = [0, a, b, (a + b) >> 1, a if pa <= pb and pa <= pc else (b if pb <= pc else c)][f]
            enc[x] = (line[x] - pr) & 255
        raw += bytes([f]) + enc.astype(np.uint8).tobytes()
        prev = line

    def chunk(kind, body):
        return struct.pack(">I", len(body)) + kind + body + struct.pack(">I", zlib.crc32(kind + body))

    png = b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", 7, 5, 8, 2, 0, 0, 0)) + chunk(b"IDAT", zlib.compress(raw)) + chunk(b"IEND", b"")
    assert np.array_equal(V.decode_image(png), img)
    url = "data:image/png;base64," + base64.b64encode(png).decode()
    assert V.load_url(url) == png and V.image_key(png) == V.image_key(png)
    with pytest.raises(ValueError):
        V.decode_image(b"\xff\xd8\xff\xe0")


def test_front_end_expands_placeholders_and_positions_with_a_stub_tower():
    """VisionFrontEnd.prepare on the CPU with a stand-in encoder: one placeholder per image becomes one token per merged
    patch, rows and multi-axis positions line up, bad inputs raise ValueError (reference: crates/agens-cli/src/mm.rs)."""
    import base64
    import torch

    class StubTower:
        def encode(self, patches, grid):
            gh, gw = grid
            assert patches.shape == (gh * gw, 1536)
            return torch.full((gh * gw // 4, 32), float(gh * 100 + gw), dtype=torch.bfloat16)

    PAD = 9
    fe = V.VisionFrontEnd(StubTower(), PAD, head_dim=64)
    assert fe.pair_axis.numel() == 32

    def ppm(w, h):
        return "data:image/x-portable-pixmap;base64," + base64.b64encode(b"P6\n%d %d\n255\n" % (w, h) + bytes(w * h * 3)).decode()

    prompt = [1, 2, PAD, 3, PAD, 4]
    mm = fe.prepare(prompt, [ppm(96, 64), ppm(64, 128)])          # merged grids 2 x 3 and 4 x 2
    assert mm["ids"] == [1, 2] + [PAD] * 6 + [3] + [PAD] * 8 + [4]
    assert mm["rows"].shape == (14, 32) and float(mm["rows"][0, 0]) == 406.0 and float(mm["rows"][6, 0]) == 804.0
    assert tuple(mm["pos3"].shape) == (3, len(mm["ids"])) and len(mm["keys"]) == 2 and mm["keys"][0] != mm["keys"][1]
    # text advances all axes together; an image advances the running position by max(grid)
    assert mm["pos3"][:, 1].tolist() == [1, 1, 1] and mm["rope_next"] == len(mm["ids"]) - 6 - 8 + 3 + 4
    with pytest.raises(ValueError):
        fe.prepare(prompt, [ppm(96, 64)])                            # two placeholders, one image
    with pytest.raises(ValueError):
        fe.prepare([1, PAD], ["http://example.com/a.png"])
    with pytest.raises(ValueError):
        fe.prepare([1, PAD], ["data:image/jpeg;base64," + base64.b64encode(b"\xff\xd8\xff\xe0").decode()])


def test_vision_tower_loads_from_checkpoint_tensors(tmp_path):
    """The tower of a checkpoint (``model.visual.*`` tensors, the reference's names): sizes are read off the tensors and
    the loaded tower computes what the tower that wrote them computes (fp32 restatement, on the CPU)."""
    import torch
    from agens_engine_b200.models.vision import VisionConfig, VisionTower
    from agens_engine_b200.utils import checkpoint as K
    cfg = VisionConfig(depth=3, d_model=64, n_heads=4, mlp=160, patch_dim=3 * 2 * 8 * 8, out_dim=96, pos_grid=6)
    a = VisionTower.random_init(cfg, "cpu", seed=4)
    back = {v: k for k, v in VisionTower._TOP.items()}
    tensors = {"model.visual." + back[k]: v.clone() for k, v in a.w.items()}
    tensors["model.visual.patch_embed.proj.weight"] = a.w["patch_w"].reshape(64, 3, 2, 8, 8).contiguous()     # conv-shaped in the file
    bback = {v: k for k, v in VisionTower._BLOCK.items()}
    for i, blk in enumerate(a.blocks):
        for k, v in blk.items():
            tensors[f"model.visual.blocks.{i}.{bback[k]}"] = v.clone()
    tensors["model.norm.weight"] = torch.ones(8, dtype=torch.bfloat16)                    # not a tower tensor
    items = list(tensors.items())
    K.write_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), dict(items[:20]))
    K.write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), dict(items[20:]))
    wm = {k: "model-00001-of-00002.safetensors" for k, _ in items[:20]}
    wm.update({k: "model-00002-of-00002.safetensors" for k, _ in items[20:]})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    assert VisionTower.has_tower(str(tmp_path))
    b = VisionTower.from_checkpoint(str(tmp_path), "cpu", n_heads=4)
    assert (b.cfg.depth, b.cfg.d_model, b.cfg.mlp, b.cfg.patch_dim, b.cfg.out_dim, b.cfg.pos_grid) == (3, 64, 160, 384, 96, 6)
    patches = torch.randn(4 * 6, cfg.patch_dim)
    assert torch.equal(a.encode_ref(patches, (4, 6)), b.encode_ref(patches, (4, 6)))
    # an incomplete tower is refused by name
    wm.pop("model.visual.merger.linear_fc2.bias")
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    with pytest.raises(ValueError, match="merger.linear_fc2.bias"):
        VisionTower.from_checkpoint(str(tmp_path), "cpu", n_heads=4)
