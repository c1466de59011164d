"""Device sampler and speculative decoding gates: the sampler follows its one positional rule (checked against an
fp64 restatement), is batch invariant and draws from the softmax; speculative decoding emits exactly the tokens of
plain decoding, greedy and sampled, whatever the drafts (reference gates: m1-spec, drafter, mtp; crates/agens-cli/src/
m1.rs, drafter.rs, mtp.rs)."""
import math

import pytest
import torch

from agens_engine_b200.models import config as C
from agens_engine_b200.models import oracle as O
from agens_engine_b200.models.dense import DenseModel
from agens_engine_b200.models.mtp import MtpHead
from agens_engine_b200.ops import basic
from agens_engine_b200.spec import CopyLookupSource, ModelSource, MtpSource, SamplingState, SpecDecoder

pytestmark = pytest.mark.gpu
M32 = 0xFFFFFFFF


def philox_first(seed: int, ctr: int) -> int:
    c = [ctr & M32, (ctr >> 32) & M32, 0, 0]
    k = [seed & M32, (seed >> 32) & M32]
    for _ in range(10):
        p0, p1 = 0xD2511F53 * c[0], 0xCD9E8D57 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & M32, p1 & M32, ((p0 >> 32) ^ c[3] ^ k[1]) & M32, p0 & M32]
        k = [(k[0] + 0x9E3779B9) & M32, (k[1] + 0xBB67AE85) & M32]
    return c[0]


def ref_sample(x: torch.Tensor, T, top_k, top_p, min_p, seed, pos) -> int:
    x = x.double()
    if T <= 0 or top_k == 1:
        return int(torch.argmax(x))
    order = sorted(range(x.numel()), key=lambda i: (-float(x[i]), i))
    xs = torch.tensor([float(x[i]) for i in order], dtype=torch.float64)
    p = torch.exp((xs - xs[0]) / T)
    keep = torch.ones_like(p, dtype=torch.bool)
    if min_p > 0:
        keep &= xs >= float(torch.tensor(float(xs[0]), dtype=torch.float32) + torch.tensor(T * math.log(min_p), dtype=torch.float32)) - 1e-6
    if 1 < top_k < x.numel():
        keep &= xs >= xs[top_k - 1]
    if top_p < 1:
        pk = p * keep
        cum = torch.cumsum(pk, 0)
        tgt = top_p * float(pk.sum())
        cut = int(torch.searchsorted(cum, torch.tensor(tgt, dtype=torch.float64), right=True))
        cut = min(cut, x.numel() - 1)
        keep &= xs >= xs[cut]
    pk = p * keep
    u = ((philox_first(seed, pos) >> 8) + 0.5) / 16777216.0
    cum = torch.cumsum(pk, 0)
    j = int(torch.searchsorted(cum, torch.tensor(u * float(pk.sum()), dtype=torch.float64), right=True))
    return order[min(j, x.numel() - 1)]


def _params(dev, rows, T, k, p, mp, seeds, pos):
    f = lambda v: torch.tensor(v, dtype=torch.float32, device=dev)
    return (f(T), torch.tensor(k, dtype=torch.int32, device=dev), f(p), f(mp),
            torch.tensor(seeds, dtype=torch.int64, device=dev), torch.tensor(pos, dtype=torch.int32, device=dev))


def test_sampler_matches_rule_and_is_batch_invariant():
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    rows, vocab = 24, 5000
    logits = (torch.randn(rows, vocab) * 3).to(dev)
    T = [0.0, 1.0, 0.7, 1.3] * 6
    k = [0, 0, 50, 0, 0, 7] * 4
    p = [1.0, 1.0, 1.0, 0.9, 0.5, 1.0] * 4
    mp = [0.0] * 12 + [0.05] * 12
    seeds = [1234 + 17 * i for i in range(rows)]
    pos = [3 * i + 1 for i in range(rows)]
    out = basic.sample_rows(logits, *_params(dev, rows, T, k, p, mp, seeds, pos)).cpu().tolist()
    ref = [ref_sample(logits[i].cpu(), T[i], k[i], p[i], mp[i], seeds[i], pos[i]) for i in range(rows)]
    assert out == ref
    # a row alone gives the same token as inside the batch
    for i in (1, 5, 17):
        one = basic.sample_rows(logits[i:i + 1], *_params(dev, 1, T[i:i + 1], k[i:i + 1], p[i:i + 1], mp[i:i + 1], seeds[i:i + 1],
                                                          pos[i:i + 1]))
        assert int(one[0]) == out[i]


def test_sampler_ties_and_distribution():
    dev = torch.device("cuda:0")
    # all-equal logits: uniform over indices by the index rule
    rows = 512
    logits = torch.zeros(rows, 64, device=dev)
    prm = _params(dev, rows, [1.0] * rows, [0] * rows, [1.0] * rows, [0.0] * rows, [9] * rows, list(range(rows)))
    out = basic.sample_rows(logits, *prm).cpu()
    ref = [min(int((((philox_first(9, i) >> 8) + 0.5) / 16777216.0) * 64), 63) for i in range(rows)]
    assert out.tolist() == ref
    # empirical frequencies follow the softmax
    x = torch.tensor([2.0, 1.0, 0.0, -1.0, 0.5, 0.5, -3.0, 1.5], device=dev)
    rows = 8192
    logits = x[None, :].repeat(rows, 1).contiguous()
    prm = _params(dev, rows, [1.0] * rows, [0] * rows, [1.0] * rows, [0.0] * rows, [77] * rows, list(range(rows)))
    out = basic.sample_rows(logits, *prm).cpu()
    freq = torch.bincount(out.long(), minlength=8).double() / rows
    prob = torch.softmax(x.double().cpu(), 0)
    assert (freq - prob).abs().max() < 0.02, (freq, prob)


def test_spec_accept_kernel():
    dev = torch.device("cuda:0")
    ti = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    ids = ti([10, 11, 12, 13, 20, 21, 22, 30])
    tgt = ti([11, 12, 99, 14, 77, 0, 0, 31])
    n, em = basic.spec_accept(ids, tgt, ti([0, 4, 7]), ti([4, 3, 1]), 8)
    assert n.tolist() == [3, 1, 1]
    assert em[0, :3].tolist() == [11, 12, 99] and em[1, 0].item() == 77 and em[2, 0].item() == 31


@pytest.fixture(scope="module")
def tiny():
    cfg = C.oracle_tiny()
    return cfg, O.random_weights(cfg, seed=0)


def _plain(ow, prompt, n_new, sampling=None):
    m = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=512)
    return SpecDecoder(m, [], max_drafts=0).generate(0, prompt, n_new, sampling)


def test_spec_greedy_equals_plain(tiny):
    cfg, ow = tiny
    torch.manual_seed(3)
    prompt = torch.randint(0, cfg.vocab, (37,)).tolist()
    n_new = 40
    plain = _plain(ow, prompt, n_new)
    m = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=512)
    m.new_seq(1)
    assert plain == m.generate_greedy(1, torch.tensor(prompt), n_new).tolist()      # graph decode == rows decode
    m.free_seq(1)
    # perfect, corrupted and garbage drafts
    for mode in ("perfect", "corrupt", "garbage"):
        dec = SpecDecoder(m, [], max_drafts=5)
        out = [dec.begin(0, prompt)]
        while len(out) < n_new:
            nxt = plain[len(out):len(out) + 5]
            if mode == "corrupt" and len(nxt) > 2:
                nxt = nxt[:2] + [(nxt[2] + 1) % cfg.vocab] + nxt[3:]
            if mode == "garbage":
                nxt = [(t + 5) % cfg.vocab for t in nxt]
            got = dec.step([0], forced_drafts={0: nxt})[0]
            if mode == "perfect" and len(nxt) == 5:
                assert len(got) == 6
            if mode == "garbage":
                assert len(got) == 1
            out += got
        dec.end(0)
        assert out[:n_new] == plain, mode
    # the row-graph path gives the same tokens
    m.row_graphs = True
    dec = SpecDecoder(m, [], max_drafts=3)
    out = [dec.begin(0, prompt)]
    while len(out) < n_new:
        out += dec.step([0], forced_drafts={0: plain[len(out):len(out) + 3]})[0]
    dec.end(0)
    assert out[:n_new] == plain


def test_spec_sources_and_sampling(tiny):
    cfg, ow = tiny
    torch.manual_seed(4)
    base = torch.randint(0, cfg.vocab, (12,)).tolist()
    prompt = base * 4                                      # repetitive: copy-lookup finds drafts
    n_new = 36
    plain = _plain(ow, prompt, n_new)
    m = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=512)
    drafter = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=512)            # same weights: every draft is right
    dec = SpecDecoder(m, [ModelSource(drafter, depth=4)], max_drafts=4)
    assert dec.generate(0, prompt, n_new) == plain
    assert dec.stats.accepted == dec.stats.proposed and dec.stats.tokens_per_step() > 4.0
    other = DenseModel.from_oracle(O.random_weights(cfg, seed=5), max_seqs=2, max_ctx=512)   # unrelated drafter
    dec = SpecDecoder(m, [CopyLookupSource(), ModelSource(other, depth=3)], max_drafts=4)
    assert dec.generate(0, prompt, n_new) == plain
    head = MtpHead.random_init_for(m)
    dec = SpecDecoder(m, [MtpSource(head, depth=2)], max_drafts=4)
    assert dec.generate(0, prompt, n_new) == plain
    assert dec.stats.by_source.get("mtp", [0, 0])[0] > 0
    # seeded sampling: the same tokens with and without speculation
    samp = SamplingState(temperature=0.8, top_k=40, top_p=0.95, seed=4242)
    plain_s = _plain(ow, prompt, n_new, samp)
    assert plain_s != plain
    dec = SpecDecoder(m, [ModelSource(drafter, depth=4)], max_drafts=4)
    assert dec.generate(0, prompt, n_new, samp) == plain_s
    dec = SpecDecoder(m, [CopyLookupSource()], max_drafts=4)
    out = [dec.begin(0, prompt, samp)]
    while len(out) < n_new:
        out += dec.step([0], forced_drafts={0: plain_s[len(out):len(out) + 4]})[0]
    dec.end(0)
    assert out[:n_new] == plain_s and dec.stats.accepted > 0


def _seq_kv(model, seq, n):
    """K and V rows of ``seq`` (layer 0) as [2, kv_heads, n, head_dim] fp32."""
    ps = model.cfg.page_size
    pages = model.seq_pages[seq][:(n + ps - 1) // ps]
    kv = model.kv[0][torch.tensor(pages, device=model.dev)]              # [pages, 2, heads, page, hd]
    return kv.permute(1, 2, 0, 3, 4).reshape(2, model.cfg.n_kv_heads, -1, model.cfg.head_dim)[:, :, :n].float()


def test_mtp_prompt_context_entries(tiny):
    """The MTP head gets one context entry per prompt position while the target prefills (reference:
    kernels/m1/m1_mtp.cu:11, :768): the entries written through the large-m path equal those of the row path fed with
    the same (hidden, next token) pairs, the first draft attends to them, and the decoded tokens stay those of plain
    decoding."""
    cfg, ow = tiny
    torch.manual_seed(11)
    prompt = torch.randint(0, cfg.vocab, (77,)).tolist()              # chunks of 32, 32 and a 13-row tail
    n_new = 24
    plain = _plain(ow, prompt, n_new)
    m = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=512, prefill_chunk=32)
    head = MtpHead.random_init_for(m)
    src = MtpSource(head, depth=2)
    dec = SpecDecoder(m, [src], max_drafts=4)
    captured = []
    first_sink = src.prefill_sink

    def spy(seq, p):                                                   # keeps the hidden rows the sink was given
        f = first_sink(seq, p)
        def g(pos0, hid):
            captured.append((pos0, hid.clone()))
            f(pos0, hid)
        return g
    src.prefill_sink = spy
    first = dec.begin(0, prompt)
    P = len(prompt)
    assert first == plain[0]
    assert [c[0] for c in captured] == [0, 32, 64] and sum(c[1].shape[0] for c in captured) == P
    assert head.seq_len_host[0] == P and src.first[0] == 1 and 0 in src.pending
    big = _seq_kv(head, 0, P)
    # the same pairs through the row path (eight rows per call) on a second head with the same weights
    hidden = torch.cat([c[1] for c in captured])
    toks = prompt[1:] + [first]
    head2 = MtpHead.random_init_for(m)
    head2.new_seq(0)
    for c in range(0, P, 8):
        e = min(P, c + 8)
        head2.forward_mtp(toks[c:e], hidden[c:e], [0] * (e - c))
    small = _seq_kv(head2, 0, P)
    err = (big - small).abs().max().item()
    ref = small.abs().max().item()
    assert err <= 0.03 * ref + 1e-3, (err, ref)
    # decoding goes on from there and stays exact; the head keeps one entry per committed position
    out = [first]
    while len(out) < n_new:
        out += dec.step([0])[0]
    assert out[:n_new] == plain
    assert head.seq_len_host[0] == len(dec.hist[0]) - 1
    assert dec.stats.by_source.get("mtp", [0, 0])[0] > 0
    dec.end(0)
    # without prompt entries (the switch off) the head starts at the first generated token
    dec = SpecDecoder(m, [MtpSource(MtpHead.random_init_for(m), depth=2)], max_drafts=4)
    dec.mtp_prompt = False
    assert dec.generate(0, prompt, n_new) == plain


def test_mtp_head_from_checkpoint(tiny, tmp_path):
    """An MTP head loaded from ``mtp.*`` tensors drafts; speculative output equals plain decoding."""
    from agens_engine_b200.utils import checkpoint as K
    cfg, ow = tiny
    g = torch.Generator().manual_seed(3)
    d, f = cfg.d_model, cfg.ffn
    shapes = {"fc.weight": (d, 2 * d), "layers.0.self_attn.q_proj.weight": (cfg.q_dim, d),
              "layers.0.self_attn.k_proj.weight": (cfg.kv_dim, d), "layers.0.self_attn.v_proj.weight": (cfg.kv_dim, d),
              "layers.0.self_attn.o_proj.weight": (d, cfg.q_dim), "layers.0.mlp.gate_proj.weight": (f, d),
              "layers.0.mlp.up_proj.weight": (f, d), "layers.0.mlp.down_proj.weight": (d, f)}
    t = {"mtp." + n: (torch.randn(*s, generator=g) * 0.05).to(torch.bfloat16) for n, s in shapes.items()}
    t.update({"mtp." + n: (1.0 + 0.05 * torch.randn(d, generator=g)).to(torch.bfloat16) for n in K.MTP_NORMS})
    K.write_safetensors(str(tmp_path / "mtp.safetensors"), t)
    torch.manual_seed(5)
    prompt = torch.randint(0, cfg.vocab, (40,)).tolist()
    plain = _plain(ow, prompt, 20)
    m = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=512)
    head = K.load_mtp(str(tmp_path), m)
    assert head.final_norm is not m.final_norm and head.embed is m.embed and head.lm_head is m.lm_head
    dec = SpecDecoder(m, [MtpSource(head, depth=2)], max_drafts=4)
    assert dec.generate(0, prompt, 20) == plain
    assert dec.stats.by_source.get("mtp", [0, 0])[0] > 0


def test_mtp_shortlist_head(tiny):
    """The MTP head with a shortlist lm_head (reference: the draft shortlist, crates/agens-cli/src/spec.rs:372-386):
    it reads only the shortlist's rows, every draft is one of the shortlist's ids, the output stays exact."""
    cfg, ow = tiny
    torch.manual_seed(21)
    prompt = torch.randint(0, cfg.vocab, (40,)).tolist()
    plain = _plain(ow, prompt, 20)
    m = DenseModel.from_oracle(ow, max_seqs=2, max_ctx=512)
    head = MtpHead.random_init_for(m)
    ids = list(range(3, cfg.vocab, 4))[:200]                       # 200 ids, not a multiple of 32
    head.use_shortlist(ids)
    assert head.lm_head.n == 224 and head._lm_valid() == 200 and head.lm_head is not m.lm_head
    seen = []
    src = MtpSource(head, depth=2)
    many0 = src.propose_many

    def spy(seqs, hist, max_n):
        out = many0(seqs, hist, max_n)
        seen.extend(t for d in out.values() for t in d)
        return out
    src.propose_many = spy
    dec = SpecDecoder(m, [src], max_drafts=4)
    assert dec.generate(0, prompt, 20) == plain
    assert seen and set(seen) <= set(ids)
    # the shortlist rows are the full head's rows: the winner among them is the full head's best shortlist id
    full = MtpHead.random_init_for(m)
    h = torch.randn(1, cfg.d_model, device=m.dev).to(torch.bfloat16)
    for hd in (head, full):
        hd.new_seq(0)
    tok = int(prompt[5])
    a = int(head.forward_mtp([tok], h, [0])[0])
    full.hid_in[:1].copy_(h)                               # (same weights: random_init_for is seeded)
    _, logits = full.forward_rows([tok], [0], want_logits=True)
    best = max(ids, key=lambda t: float(logits[0, t]))
    assert a == best or abs(float(logits[0, a]) - float(logits[0, best])) < 0.05 * float(logits[0].abs().max())
