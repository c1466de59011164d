"""The persistent decode-step kernel (one launch per step) against the per-op path and the fp32 oracle: logits within
tolerance, greedy tokens equal, rows of a verify block bit-identical to single decode rows, batched rows bit-identical
to solo rows (reference gates: m1-spec / m1-batch equality, crates/agens-cli/src/m1.rs:159-289)."""
import dataclasses

import pytest
import torch

from agens_engine_b200.models import config as C
from agens_engine_b200.models import oracle as O
from agens_engine_b200.models.dense import DenseModel

pytestmark = pytest.mark.gpu


def small_cfg(group: int) -> C.ModelConfig:
    bits = {"0.qkv": 4, "0.o": 3, "0.gate_up": 2, "0.down": 4, "1.qkv": 2, "1.o": 4, "1.gate_up": 3, "1.down": 2,
            "2.qkv": 3, "2.o": 2, "2.gate_up": 4, "2.down": 3}
    return C.ModelConfig(f"step-small-g{group}", 3, 512, 8, 2, 128, 1024, 2048, rope_theta=1e6, group=group, bits=bits,
                         lm_head_bits=4)


@pytest.fixture(scope="module", params=[64, 128])
def pair(request):
    cfg = small_cfg(request.param)
    ow = O.random_weights(cfg, seed=3)
    fused = DenseModel.from_oracle(ow, max_seqs=4, max_ctx=512)
    assert fused.enable_step(), "the step kernel must be available on a CUDA device"
    plain = DenseModel.from_oracle(ow, max_seqs=4, max_ctx=512)
    plain.enable_step(False)
    return cfg, ow, fused, plain


def _reset(m):
    for s in list(m.seq_pages):
        m.free_seq(s)


def test_logits_match_per_op_path_and_oracle(pair):
    cfg, ow, fused, plain = pair
    torch.manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (70,))
    cont = torch.randint(0, cfg.vocab, (5,)).tolist()
    outs = []
    for m in (fused, plain):
        _reset(m)
        m.new_seq(0)
        m.prefill(0, prompt)
        rows = []
        for t in cont:
            _, lg = m.forward_rows([t], [0], want_logits=True)
            rows.append(lg[0].cpu())
        outs.append(torch.stack(rows))
        assert int(m.status.item()) == 0
    scale = outs[1].abs().max().item()
    err = (outs[0] - outs[1]).abs().max().item()
    assert err < 0.02 * scale, (err, scale)
    assert (outs[0].argmax(-1) == outs[1].argmax(-1)).float().mean().item() >= 0.8
    assert fused.step.launches >= 5


def test_greedy_tokens_match_per_op_path(pair):
    cfg, ow, fused, plain = pair
    torch.manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (33,))
    toks = []
    for m in (fused, plain):
        _reset(m)
        m.new_seq(0)
        toks.append(m.generate_greedy(0, prompt, 24).tolist())
    # free-running greedy decoding of a random-weight model forks at the first near tie: the start must agree
    assert toks[0][:4] == toks[1][:4], toks


def test_verify_block_equals_single_rows_and_batch_invariance(pair):
    cfg, ow, fused, _ = pair
    m = fused
    _reset(m)
    torch.manual_seed(2)
    p0 = torch.randint(0, cfg.vocab, (40,))
    p1 = torch.randint(0, cfg.vocab, (23,))
    for s, p in ((0, p0), (1, p1), (2, p0)):
        m.new_seq(s)
        m.prefill(s, p)
    cont = torch.randint(0, cfg.vocab, (6,)).tolist()
    singles = []
    for t in cont:
        _, lg = m.forward_rows([t], [0], want_logits=True)
        singles.append(lg[0])
    _, lg_block = m.forward_rows(cont, [2] * 6, want_logits=True)
    for i in range(6):
        assert torch.equal(lg_block[i], singles[i]), i
    m.truncate(0, 40); m.truncate(2, 40)
    _, a = m.forward_rows([cont[0]], [0], want_logits=True)
    _, b = m.forward_rows([cont[1]], [1], want_logits=True)
    m.truncate(0, 40); m.truncate(1, 23)
    _, ab = m.forward_rows([cont[0], cont[1], cont[2]], [0, 1, 2], want_logits=True)
    assert torch.equal(ab[0], a[0]) and torch.equal(ab[1], b[0])
    assert int(m.status.item()) == 0


@pytest.mark.parametrize("per_seq", [3, 4])
def test_nine_to_sixteen_rows_match_per_op_path(pair, per_seq):
    """Steps of 12 and 16 rows (four conversations, verify blocks of 3 or 4 rows each): the large-step instance of the
    kernel (four token sets, half k slices, partial tiles in global memory) against the per-op path."""
    cfg, ow, fused, plain = pair
    torch.manual_seed(6)
    prompts = [torch.randint(0, cfg.vocab, (17 + 9 * i,)) for i in range(4)]
    toks = torch.randint(0, cfg.vocab, (4 * per_seq,)).tolist()
    seqs = [s for s in range(4) for _ in range(per_seq)]
    outs = []
    for m in (fused, plain):
        _reset(m)
        for s, p in enumerate(prompts):
            m.new_seq(s)
            m.prefill(s, p)
        before = m.step.launches if m.step is not None else 0
        ids, lg = m.forward_rows(toks, seqs, want_logits=True)
        outs.append(lg.cpu())
        assert int(m.status.item()) == 0
        if m is fused:
            assert m.step.launches == before + 1
    scale = outs[1].abs().max().item()
    err = (outs[0] - outs[1]).abs().max().item()
    assert err < 0.02 * scale, (err, scale)
    assert (outs[0].argmax(-1) == outs[1].argmax(-1)).float().mean().item() >= 0.8


def test_uniform_split_makes_rows_bit_identical_across_step_sizes():
    """With the uniform work split a row of a 12-row step equals the same row run alone (and in a 3-row step)."""
    cfg = small_cfg(128)
    ow = O.random_weights(cfg, seed=3)
    m = DenseModel.from_oracle(ow, max_seqs=4, max_ctx=512)
    assert m.enable_step("on", uniform=True)
    torch.manual_seed(7)
    prompts = [torch.randint(0, cfg.vocab, (21 + 5 * i,)) for i in range(3)]
    for s, p in enumerate(prompts):
        m.new_seq(s)
        m.prefill(s, p)
    toks = torch.randint(0, cfg.vocab, (12,)).tolist()
    seqs = [s for s in range(3) for _ in range(4)]
    _, big = m.forward_rows(toks, seqs, want_logits=True)
    big = big.clone()
    for s, p in enumerate(prompts):
        m.truncate(s, len(p))
    _, small = m.forward_rows(toks[:3], [0, 0, 0], want_logits=True)
    assert torch.equal(small[:3], big[:3])
    m.truncate(0, len(prompts[0]))
    _, one = m.forward_rows([toks[4]], [1], want_logits=True)
    assert torch.equal(one[0], big[4])
    assert int(m.status.item()) == 0


def test_decode_graph_replays_and_advances_on_device(pair):
    cfg, ow, fused, _ = pair
    m = fused
    _reset(m)
    torch.manual_seed(4)
    prompts = [torch.randint(0, cfg.vocab, (20 + 7 * i,)) for i in range(3)]
    firsts = []
    for s, p in enumerate(prompts):
        m.new_seq(s)
        firsts.append(m.prefill(s, p)[0])
    m.decode_setup([0, 1, 2], firsts, 12)
    outs = m.decode_steps(12).cpu()
    torch.cuda.synchronize()
    assert int(m.status.item()) == 0
    # the same three conversations one at a time
    for s, p in enumerate(prompts):
        _reset(m)
        m.new_seq(0)
        solo = m.generate_greedy(0, p, 13)
        assert solo[1:].tolist() == outs[:, s].tolist(), s


def test_32b_width_two_layers():
    cfg = C.scaled(C.dense_32b(seed=0), 2)
    torch.manual_seed(5)
    prompt = torch.randint(0, cfg.vocab, (96,))
    toks = []
    for use in (True, False):
        m = DenseModel.random_init(cfg, "cuda:0", seed=0, max_seqs=1, max_ctx=512, prefill_chunk=64)
        m.enable_step(use)
        m.new_seq(0)
        toks.append(m.generate_greedy(0, prompt, 10).tolist())
        assert int(m.status.item()) == 0
        del m
    assert toks[0][:3] == toks[1][:3], toks
