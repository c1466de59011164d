"""Host KV tier: with most of a long sequence's pages in pinned host memory, prefill and decode produce bit-identical
logits and tokens to an all-resident run, the GPU pool holds only the window, and copies run on the side stream
(reference gate: m1-session tiers gpu/host, crates/agens-cli/src/m1.rs:1217-1330; m1_kv.cu)."""
import pytest
import torch

from agens_engine_b200.models import config as C
from agens_engine_b200.models import oracle as O
from agens_engine_b200.models.dense import DenseModel

pytestmark = pytest.mark.gpu


def test_tiered_kv_is_bit_identical():
    cfg = C.oracle_tiny()
    ow = O.random_weights(cfg, seed=0)
    torch.manual_seed(21)
    prompt = torch.randint(0, cfg.vocab, (1500,))
    n_new = 40

    def run(tiered):
        m = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=2048, prefill_chunk=256)
        tier = m.enable_host_tier(window_tokens=256, batch_pages=16) if tiered else None
        m.new_seq(0)
        tok, lg = m.prefill(0, prompt, want_logits=True)
        toks, logits = [tok], [lg]
        for _ in range(n_new):
            out, l2 = m.forward_rows([toks[-1]], [0], want_logits=True)
            toks.append(int(out[0])); logits.append(l2[0])
        torch.cuda.synchronize()
        assert int(m.status.item()) == 0
        return m, tier, toks, torch.stack(logits)

    m0, _, t0, l0 = run(False)
    m1, tier, t1, l1 = run(True)
    assert t0 == t1
    assert torch.equal(l0, l1)
    assert len(tier.blocks[0]) >= 4 and tier.bytes_h2d > 0 and tier.bytes_d2h > 0
    used0 = m0.n_pages - m0.free_pages()
    used1 = m1.n_pages - m1.free_pages()
    assert used1 <= used0 - 16 * len(tier.blocks[0]) + 1
    # a verify block over the tiered sequence equals single steps
    m1.truncate(0, 1500 + 10)
    m0.truncate(0, 1500 + 10)
    blk = t0[10:16]
    _, a = m0.forward_rows(blk, [0] * 6, want_logits=True)
    _, b = m1.forward_rows(blk, [0] * 6, want_logits=True)
    assert torch.equal(a, b)
    m1.free_seq(0)
    assert m1.free_pages() == m1.n_pages and 0 not in tier.blocks


def test_session_file_round_trip_and_recover(tmp_path):
    cfg = C.oracle_tiny()
    ow = O.random_weights(cfg, seed=0)
    torch.manual_seed(22)
    prompt = torch.randint(0, cfg.vocab, (50,))
    m = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=256)
    m.new_seq(0)
    first, _ = m.prefill(0, prompt)
    path = str(tmp_path / "session.safetensors")
    m.save_session(0, path, tokens=prompt.tolist() + [first])
    ref, tok = [], first
    for _ in range(10):
        out, _ = m.forward_rows([tok], [0]); tok = int(out[0]); ref.append(tok)
    # a fresh engine instance resumes the conversation from the file
    m2 = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=256)
    toks = m2.load_session(1, path)
    assert toks == prompt.tolist() + [first] and m2.seq_len_host[1] == 50
    got, tok = [], toks[-1]
    for _ in range(10):
        out, _ = m2.forward_rows([tok], [1]); tok = int(out[0]); got.append(tok)
    assert got == ref
    m2.status.fill_(3)
    m2.recover()
    assert int(m2.status.item()) == 0 and m2.free_pages() == m2.n_pages and not m2.seq_pages
    m2.new_seq(0)
    assert m2.prefill(0, prompt)[0] == first
