"""Linears kept in bf16: the bf16 GEMV against an fp32 PyTorch product, and a checkpoint whose linears are stored as
bf16 loaded and run without quantising them (reference: LinearFormat::Bf16, crates/agens-core/src/weights.rs:176-187;
kernels/src/bf16_gemv.cu, bi_gemv.cu)."""
import pytest
import torch

from agens_engine_b200 import _lib
from agens_engine_b200._lib import check, current_stream, ptr
from agens_engine_b200.models import config as C
from agens_engine_b200.models import oracle as O
from agens_engine_b200.ops import linear as L
from agens_engine_b200.utils import checkpoint as K

pytestmark = pytest.mark.gpu
ALL7 = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")


def _gemv(x, w, resid=None, f32=False):
    m, n = x.shape[0], w.shape[0]
    y = torch.empty(m, n, dtype=torch.float32 if f32 else torch.bfloat16, device=x.device)
    lib = _lib.cuda_lib()
    check(lib.b2_bf16_gemv(ptr(x), x.stride(0), ptr(w), w.stride(0), m, n, x.shape[1], None if f32 else ptr(y), ptr(y) if f32 else None,
                           y.stride(0), ptr(resid), resid.stride(0) if resid is not None else 0, current_stream()), "b2_bf16_gemv")
    return y


def test_bf16_gemv_matches_fp32_and_is_batch_invariant():
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)
    for n, k in ((1024, 512), (520, 2056), (5120, 8192), (37, 64)):
        w = (torch.randn(n, k, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        x8 = torch.randn(8, k, device=dev, generator=g).to(torch.bfloat16)
        r8 = torch.randn(8, n, device=dev, generator=g).to(torch.bfloat16)
        ref = x8.float() @ w.float().t()
        for m in (1, 3, 8):
            y = _gemv(x8[:m], w, f32=True)
            assert torch.allclose(y, ref[:m], rtol=2e-3, atol=2e-3 * ref.abs().max().item()), (n, k, m)
            yb = _gemv(x8[:m], w, resid=r8[:m])
            want = (ref[:m] + r8[:m].float()).to(torch.bfloat16)
            assert (yb.float() - want.float()).abs().max().item() <= 0.02 * want.float().abs().max().item(), (n, k, m)
        # a row gives the same bits alone and as the last of eight
        assert torch.equal(_gemv(x8[7:8], w, f32=True)[0], _gemv(x8, w, f32=True)[7])
    torch.cuda.synchronize()


@pytest.mark.parametrize("which", [ALL7, ("self_attn.o_proj",)])
def test_checkpoint_with_bf16_linears_runs_in_bf16(tmp_path, which, monkeypatch):
    cfg = C.oracle_tiny()
    ow = O.random_weights(cfg, seed=3)
    d = str(tmp_path / "bf")
    K.save_oracle(d, ow, bf16_linears=which)
    m = K.load_model(d, "cuda:0", max_seqs=2, max_ctx=256)
    kinds = {lin: type(m.layers[0][lin]).__name__ for lin in ("qkv", "o", "gate_up", "down")}
    if which is ALL7:
        assert set(kinds.values()) == {"Bf16Linear"} and m.cfg.bits["0.qkv"] == 16
    else:
        assert kinds == {"qkv": "WqLinear", "o": "Bf16Linear", "gate_up": "WqLinear", "down": "WqLinear"}
    assert not m._step_possible()
    torch.manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (48,))
    ref_tok, ref_logits = O.OracleModel(ow, mirror=False).generate_greedy(prompt, 24)
    # prefill (large-m path), then one-row decode steps
    m.new_seq(0)
    toks = m.generate_greedy(0, prompt, 24)
    agree = sum(int(a == b) for a, b in zip(toks.tolist(), ref_tok.tolist()))
    assert agree >= 18, (agree, toks.tolist(), ref_tok.tolist())
    m.new_seq(1)
    _, lg = m.prefill(1, prompt, want_logits=True)
    err = (lg.cpu() - ref_logits[0]).abs().max().item()
    assert err < 0.05 * ref_logits[0].abs().max().item(), err
    # verify rows (four rows of one sequence) give the decode tokens again: the bf16 path is batch invariant
    m.truncate(0, prompt.numel())
    out, _ = m.forward_rows(toks[:4].tolist(), [0] * 4)
    assert out.tolist() == toks[1:5].tolist()
    # the switch that quantises them at load instead
    monkeypatch.setenv("B200E_BF16_LINEARS", "quant")
    q = K.load_model(d, "cuda:0", max_seqs=1, max_ctx=256)
    assert all(isinstance(q.layers[0][lin], L.WqLinear) for lin in ("qkv", "o", "gate_up", "down"))


def test_bf16_drafter_with_row_graphs_keeps_speculation_exact():
    """A random-init bf16 model as companion drafter, its steps replayed as CUDA graphs: the emitted tokens are those of
    plain decoding, and a drafter with the target's own weights in bf16 gets most of its drafts accepted."""
    from agens_engine_b200.models.dense import DenseModel
    from agens_engine_b200.spec import ModelSource, SpecDecoder
    cfg = C.oracle_tiny()
    ow = O.random_weights(cfg, seed=0)
    torch.manual_seed(4)
    prompt = torch.randint(0, cfg.vocab, (30,)).tolist()
    plain = SpecDecoder(DenseModel.from_oracle(ow, max_seqs=2, max_ctx=512), [], max_drafts=0).generate(0, prompt, 24)
    target = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=512)
    drafter = DenseModel.random_init(cfg, "cuda:0", seed=9, max_seqs=2, max_ctx=512, bf16_linears=True)
    assert all(isinstance(drafter.layers[0][lin], L.Bf16Linear) for lin in ("qkv", "o", "gate_up", "down"))
    drafter.row_graphs = True
    dec = SpecDecoder(target, [ModelSource(drafter, depth=3)], max_drafts=3)
    assert dec.generate(0, prompt, 24) == plain and dec.stats.proposed > 0
    # the target's weights, dequantised to bf16 linears, as the drafter: nearly every draft is right
    same = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=512)
    for l, d in enumerate(same.layers):
        for lin in ("qkv", "o", "gate_up", "down"):
            d[lin] = L.Bf16Linear.from_tensor(ow.quant[f"{l}.{lin}"].dequant(), same.dev)
    same.finalize()
    same.row_graphs = True
    dec = SpecDecoder(target, [ModelSource(same, depth=3)], max_drafts=3)
    assert dec.generate(0, prompt, 24) == plain
    assert dec.stats.accepted >= 0.7 * dec.stats.proposed, (dec.stats.accepted, dec.stats.proposed)
