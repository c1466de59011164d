"""End-to-end gates on the GPU: the engine on the CPU-oracle plumbing config reproduces the oracle's greedy tokens
and logits; decode rows are batch invariant (reference gates: m1 x2 identical, m1-batch, m1-spec;
crates/agens-cli/src/m1.rs:159-289, batch.rs)."""
import pytest
import torch

from agens_engine_b200.models import config as C
from agens_engine_b200.models import oracle as O
from agens_engine_b200.models.dense import DenseModel

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny():
    cfg = C.oracle_tiny()
    ow = O.random_weights(cfg, seed=0)
    return cfg, ow


def test_tiny_greedy_matches_oracle(tiny):
    cfg, ow = tiny
    torch.manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (64,))
    ref_tok, ref_logits = O.OracleModel(ow, mirror=True).generate_greedy(prompt, 32)
    f32_tok, f32_logits = O.OracleModel(ow, mirror=False).generate_greedy(prompt, 32)
    m = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=256)
    m.new_seq(0)
    toks = m.generate_greedy(0, prompt, 32)
    assert toks.tolist() == ref_tok.tolist()
    # teacher-forced logits vs the fp32 dequantised reference
    m.new_seq(1)
    _, lg = m.prefill(1, prompt, want_logits=True)
    err = (lg.cpu() - f32_logits[0]).abs().max().item()
    assert err < 0.05 * f32_logits[0].abs().max().item(), err
    agree = sum(int(a == b) for a, b in zip(toks.tolist(), f32_tok.tolist()))
    assert agree >= 24, agree


def test_rows_batch_invariant_and_verify_equals_decode(tiny):
    cfg, ow = tiny
    torch.manual_seed(1)
    m = DenseModel.from_oracle(ow, max_seqs=3, max_ctx=256)
    p0 = torch.randint(0, cfg.vocab, (40,))
    p1 = torch.randint(0, cfg.vocab, (23,))
    for s, p in ((0, p0), (1, p1), (2, p0)):
        m.new_seq(s)
        m.prefill(s, p)
    cont = torch.randint(0, cfg.vocab, (6,)).tolist()
    # sequence 0: six tokens one by one; sequence 2 (same prompt): the same six tokens as one verify block
    singles = []
    for t in cont:
        _, lg = m.forward_rows([t], [0], want_logits=True)
        singles.append(lg[0])
    _, lg_block = m.forward_rows(cont, [2] * 6, want_logits=True)
    for i in range(6):
        assert torch.equal(lg_block[i], singles[i]), i
    # batched rows of different sequences equal their single-row runs
    m.truncate(0, 40); m.truncate(2, 40)
    _, a = m.forward_rows([cont[0]], [0], want_logits=True)
    m.truncate(0, 40)
    _, b = m.forward_rows([cont[0], 5, cont[0]], [0, 1, 2], want_logits=True)
    assert torch.equal(a[0], b[0]) and torch.equal(a[0], b[2])


def test_decode_graph_matches_eager(tiny):
    cfg, ow = tiny
    torch.manual_seed(2)
    prompt = torch.randint(0, cfg.vocab, (30,))
    m = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=256)
    m.new_seq(0); m.new_seq(1)
    g = m.generate_greedy(0, prompt, 12).tolist()
    first, _ = m.prefill(1, prompt)
    toks = [first]
    for _ in range(11):
        out, _ = m.forward_rows([toks[-1]], [1])
        toks.append(int(out[0]))
    assert toks == g


def test_checkpoint_round_trip_on_gpu(tiny, tmp_path):
    """save -> validate -> load gives a model whose greedy tokens equal the one built from the same weights in memory."""
    from agens_engine_b200.utils import checkpoint as K
    cfg, ow = tiny
    d = str(tmp_path / "ckpt")
    K.save_oracle(d, ow, shards=2)
    torch.manual_seed(2)
    prompt = torch.randint(0, cfg.vocab, (40,))
    a = DenseModel.from_oracle(ow, max_seqs=1, max_ctx=256)
    a.new_seq(0)
    ta = a.generate_greedy(0, prompt, 16)
    b = K.load_model(d, "cuda:0", max_seqs=1, max_ctx=256)
    b.new_seq(0)
    tb = b.generate_greedy(0, prompt, 16)
    assert ta.tolist() == tb.tolist()
    assert b.cfg.bits == a.cfg.bits and b.cfg.group == a.cfg.group
