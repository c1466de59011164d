"""Vision tower on the GPU against its fp32 restatement, with resident and host-streamed weights, and image rows
replacing placeholder embeddings in prefill (reference: kernels/oracle/bridge/vision.cpp, m1_model.cu:2821-2834)."""
import numpy as np
import pytest
import torch

from agens_engine_b200.models import config as C
from agens_engine_b200.models import oracle as O
from agens_engine_b200.models.dense import DenseModel
from agens_engine_b200.models.vision import VisionConfig, VisionTower
from agens_engine_b200.serve import vision as V

pytestmark = pytest.mark.gpu


def test_tower_matches_fp32_and_streams_weights():
    cfg = VisionConfig(depth=3, d_model=288, n_heads=4, mlp=608, out_dim=256, pos_grid=12)      # head_dim 72, as the full tower
    rng = np.random.default_rng(0)
    img = rng.integers(0, 256, size=(150, 210, 3), dtype=np.uint8)
    patches, grid = V.preprocess(img, (128, 192))
    t = VisionTower.random_init(cfg, seed=1)
    out = t.encode(torch.from_numpy(patches), grid)
    ref = t.encode_ref(torch.from_numpy(patches), grid)
    assert out.shape == (grid[0] * grid[1] // 4, cfg.out_dim)
    err = (out.float() - ref).abs().max().item()
    assert err < 0.05 * ref.abs().max().item() + 0.02, err
    t2 = VisionTower.random_init(cfg, seed=1, resident=False)
    assert not t2.blocks[0]["qkv_w"].is_cuda and t2.blocks[0]["qkv_w"].is_pinned()
    assert torch.equal(t2.encode(torch.from_numpy(patches), grid), out)


def test_image_rows_replace_placeholder_embeddings():
    cfg = C.oracle_tiny()
    ow = O.random_weights(cfg, seed=0)
    m = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=256, prefill_chunk=64)
    torch.manual_seed(0)
    PAD = 7
    ids = torch.randint(8, cfg.vocab, (40,))
    ids[5:17] = PAD
    rows = (torch.randn(12, cfg.d_model) * 0.02).to(torch.bfloat16)
    m.new_seq(0)
    _, a = m.prefill(0, ids, want_logits=True, image_rows=rows, image_pad_id=PAD)
    # the same result when the rows are planted in the embedding table at fresh ids
    m2 = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=256, prefill_chunk=64)
    m2.embed = m2.embed.clone()
    m2.embed[100:112] = rows.to(m2.dev)
    ids2 = ids.clone()
    ids2[5:17] = torch.arange(100, 112)
    m2.new_seq(0)
    _, b = m2.prefill(0, ids2, want_logits=True)
    assert torch.equal(a, b)
    m.new_seq(1)
    _, c = m.prefill(1, ids, want_logits=True)
    assert not torch.equal(a, c)


def test_prefill_with_multi_axis_positions_and_rope_delta():
    from agens_engine_b200.ops import basic
    cfg = C.oracle_tiny()
    ow = O.random_weights(cfg, seed=0)
    torch.manual_seed(1)
    PAD = 7
    ids = torch.randint(8, cfg.vocab, (40,))
    ids[4:16] = PAD                                               # one image: merged grid 3 x 4
    rows = (torch.randn(12, cfg.d_model) * 0.02).to(torch.bfloat16)
    axis = basic.mrope_pair_axis(cfg.head_dim, [11, 11, 10], True)
    pos3, nxt = V.mrope_positions(ids.tolist(), PAD, [(3, 4)])
    assert nxt == 40 - 12 + 4                                     # the image advances the running position by max(3, 4)

    def run(p3, nx):
        m = DenseModel.from_oracle(ow, max_seqs=1, max_ctx=256, prefill_chunk=64)
        m.new_seq(0)
        tok, lg = m.prefill(0, ids, want_logits=True, image_rows=rows, image_pad_id=PAD,
                            rope_pos3=None if p3 is None else torch.from_numpy(p3), pair_axis=axis, rope_next=nx)
        out, lg2 = m.forward_rows([tok], [0], want_logits=True)
        return lg, lg2[0], m

    plain, plain2, _ = run(None, None)
    import numpy as np
    same_axes = np.tile(np.arange(40, dtype=np.int32), (3, 1))
    a, a2, _ = run(same_axes, 40)                                 # every axis = token index: identical to plain RoPE
    assert torch.equal(a, plain) and torch.equal(a2, plain2)
    b, b2, m = run(pos3, nxt)
    assert not torch.equal(b, plain) and m.rope_delta[0] == nxt - 40
    assert not torch.equal(b2, plain2)                            # the decode row rotates by its KV position + delta
