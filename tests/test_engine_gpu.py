"""Engine loop on the GPU: continuous batching gives every request the tokens it gets alone (greedy and seeded
sampling, with and without speculation), stops at stop ids and length limits, survives KV pressure by preempting, and
serves the OpenAI front end end to end (reference gates: serve-smoke, batch-e2e; crates/agens-cli/src/serve.rs)."""
import dataclasses
import json
import threading

import pytest
import torch

from agens_engine_b200.models import config as C
from agens_engine_b200.models import oracle as O
from agens_engine_b200.models.dense import DenseModel
from agens_engine_b200.serve.engine import Engine, attach_to_server
from agens_engine_b200.spec import CopyLookupSource, ModelSource, SamplingState, SpecDecoder

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny():
    cfg = C.oracle_tiny()
    return cfg, O.random_weights(cfg, seed=0)


class Collector:
    def __init__(self):
        self.toks, self.done, self.err = {}, {}, {}

    def __call__(self, rid, toks, finished, error):
        self.toks.setdefault(rid, []).extend(toks)
        if finished:
            self.done[rid] = True
        if error:
            self.err[rid] = error
        return False


def _alone(ow, prompt, n_new, sampling=None, path=None, uniform=False):
    m = DenseModel.from_oracle(ow, max_seqs=1, max_ctx=512, prefill_chunk=128)
    m.set_linear_path(path)         # the engine pins the tensor-core path when a step can exceed sixteen rows,
    m.enable_step("on", uniform=uniform)   # and the persistent step kernel (one work split beyond eight rows) up to there
    return SpecDecoder(m, [], max_drafts=0).generate(0, prompt, n_new, sampling)


def test_engine_batches_match_single_runs(tiny):
    cfg, ow = tiny
    torch.manual_seed(11)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (5, 300, 47, 130, 9, 64)]
    samp = {"temperature": 0.9, "top_k": 50, "top_p": 0.9, "seed": 99, "max_new_tokens": 24}
    for spec in (False, True):
        # 4 sequences x (1 + 3 drafts) = 16 rows: the step kernel with the uniform work split for every step where the
        # model allows it (head_dim 128), else the tensor-core path for every step
        path = 1 if (spec and cfg.head_dim != 128) else None
        want = [_alone(ow, p, 24, path=path, uniform=spec) for p in prompts]
        want_s = _alone(ow, prompts[2], 24, SamplingState(0.9, 50, 0.9, 0.0, 99), path=path, uniform=spec)
        m = DenseModel.from_oracle(ow, max_seqs=4, max_ctx=512, prefill_chunk=128)
        col = Collector()
        drafter = DenseModel.from_oracle(ow, max_seqs=4, max_ctx=512) if spec else None
        eng = Engine(m, col, sources_factory=(lambda: [CopyLookupSource(), ModelSource(drafter, 3)]) if spec else None,
                     max_drafts=3 if spec else 0)
        rids = [eng.submit(p, {"max_new_tokens": 24}) for p in prompts]
        rs = eng.submit(prompts[2], samp)
        eng.run_until_idle(10000)
        assert eng.idle() and not col.err
        for rid, w in zip(rids, want):
            assert col.toks[rid] == w, (spec, rid)
        assert col.toks[rs] == want_s
        assert eng.stats.peak_batch == 4 and m.free_pages() == m.n_pages
        if spec:
            assert eng.spec.stats.accepted > 0


def test_engine_feeds_prompt_positions_to_the_mtp_head(tiny):
    """With an MTP head as draft source the engine hands every prefill chunk's hidden rows to the head: a request leaves
    prefill with one head entry per prompt position, and the tokens stay those of a run alone."""
    from agens_engine_b200.models.mtp import MtpHead
    from agens_engine_b200.spec import MtpSource
    cfg, ow = tiny
    torch.manual_seed(13)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (150, 6, 40)]
    path = 1 if cfg.head_dim != 128 else None
    want = [_alone(ow, p, 16, path=path, uniform=True) for p in prompts]
    m = DenseModel.from_oracle(ow, max_seqs=4, max_ctx=512, prefill_chunk=64)
    head = MtpHead.random_init_for(m)
    src = MtpSource(head, depth=2)
    seen = {}
    begin0 = src.begin

    def begin(seq, hist):                                  # entries of the head when the request enters decoding
        begin0(seq, hist)
        seen[len(hist) - 1] = (head.seq_len_host[seq], src.first[seq])
    src.begin = begin
    col = Collector()
    eng = Engine(m, col, sources_factory=lambda: [src], max_drafts=3)
    rids = [eng.submit(p, {"max_new_tokens": 16}) for p in prompts]
    eng.run_until_idle(10000)
    assert eng.idle() and not col.err
    for rid, w in zip(rids, want):
        assert col.toks[rid] == w, rid
    assert seen == {150: (150, 1), 6: (6, 1), 40: (40, 1)}
    assert eng.spec.stats.by_source.get("mtp", [0, 0])[0] > 0
    assert m.free_pages() == m.n_pages and head.free_pages() == head.n_pages


def test_engine_stops_limits_and_pressure(tiny):
    cfg, ow = tiny
    torch.manual_seed(12)
    p = torch.randint(0, cfg.vocab, (40,)).tolist()
    ref = _alone(ow, p, 48)
    m = DenseModel.from_oracle(ow, max_seqs=4, max_ctx=256, n_pages=14, prefill_chunk=128)          # 224 token rows for everybody
    col = Collector()
    eng = Engine(m, col)
    stop_tok = ref[10]
    first_stop = ref.index(stop_tok)
    r1 = eng.submit(p, {"max_new_tokens": 48, "stop_token_ids": [stop_tok]})
    r2 = eng.submit(p, {"max_new_tokens": 48})
    r3 = eng.submit(p, {"max_new_tokens": 48})
    r4 = eng.submit(p + p, {"max_new_tokens": 30})
    r5 = eng.submit(list(range(300)), {"max_new_tokens": 4})                      # longer than the context window
    eng.run_until_idle(20000)
    assert eng.idle()
    assert col.toks[r1] == ref[:first_stop + 1]
    assert col.toks[r2] == ref and col.toks[r3] == ref
    assert col.toks[r4] == _alone(ow, p + p, 30)
    assert r5 in col.err and col.toks[r5] == []
    assert m.free_pages() == m.n_pages


def test_engine_behind_openai_server(tiny, tmp_path):
    from agens_engine_b200.serve.server import Server
    from tests.fixtures import tiny_tokenizer_json
    cfg, ow = tiny
    tj = str(tmp_path / "tokenizer.json")
    open(tj, "w").write(tiny_tokenizer_json())
    srv = Server(tj, model_name="tiny", eos_token_ids=[])
    m = DenseModel.from_oracle(ow, max_seqs=4, max_ctx=512)
    m.cfg = dataclasses.replace(m.cfg, vocab_valid=256)           # ids the test tokenizer knows
    eng = Engine(m, lambda *a: False)
    attach_to_server(eng, srv)
    eng.start()
    try:
        body = {"model": "tiny", "prompt": "hello world and the thing", "max_tokens": 12, "temperature": 0}
        st, text = srv.handle("POST", "/v1/completions", body)
        assert st == 200, text
        a = json.loads(text)
        assert a["usage"]["completion_tokens"] == 12
        # the same request concurrently with others gives the same text
        res = {}
        def call(i):
            res[i] = srv.handle("POST", "/v1/completions", dict(body, prompt=body["prompt"] if i == 0 else "in the " * (i + 1)))
        th = [threading.Thread(target=call, args=(i,)) for i in range(4)]
        [t.start() for t in th]; [t.join(60) for t in th]
        assert all(res[i][0] == 200 for i in range(4))
        assert json.loads(res[0][1])["choices"][0]["text"] == a["choices"][0]["text"]
        st, text = srv.handle("POST", "/v1/chat/completions", {"model": "tiny", "messages": [{"role": "user", "content": "hello"}],
                                                              "max_tokens": 8, "temperature": 0.7, "seed": 5})
        assert st == 200 and json.loads(text)["usage"]["completion_tokens"] == 8
    finally:
        eng.stop()


def test_engine_keeps_sequences_for_conversations_and_prefix_reuse(tiny):
    cfg, ow = tiny
    torch.manual_seed(13)
    m = DenseModel.from_oracle(ow, max_seqs=4, max_ctx=512, prefill_chunk=128)
    col = Collector()
    eng = Engine(m, col, max_batch=2, keep_sequences=True, prefix_chunk=64)
    q = torch.randint(0, cfg.vocab, (100,)).tolist()
    solo = _alone(ow, q, 16)
    a = eng.submit(q, {"max_new_tokens": 16})
    eng.run_until_idle(5000)
    assert col.toks[a] == solo and eng.stats.tokens_reused == 0 and len(eng.kept) == 1
    # the same prompt again: forked from the kept sequence at a chunk boundary, same tokens, less prefill
    b = eng.submit(q, {"max_new_tokens": 16})
    eng.run_until_idle(5000)
    assert eng.stats.tokens_reused == 64 and col.toks[b] == solo
    # a conversation: the second turn extends the first turn's tokens and takes its sequence over
    c = eng.submit(q[:70], {"max_new_tokens": 10}, session="conv")
    eng.run_until_idle(5000)
    turn2 = q[:70] + col.toks[c] + torch.randint(0, cfg.vocab, (25,)).tolist()
    before = eng.stats.tokens_reused
    d = eng.submit(turn2, {"max_new_tokens": 10}, session="conv")
    eng.run_until_idle(5000)
    assert eng.stats.tokens_reused - before >= 64 and len(col.toks[d]) == 10 and not col.err
    # slots run out: kept sequences are given up (conversations parked on the host) and everything still completes
    rs = [eng.submit(torch.randint(0, cfg.vocab, (40 + i,)).tolist(), {"max_new_tokens": 6}) for i in range(6)]
    eng.run_until_idle(20000)
    assert eng.idle() and all(len(col.toks[r]) == 6 for r in rs) and not col.err
    e = eng.submit(turn2 + col.toks[d] + [5, 6, 7, 8, 9, 10, 11, 12, 13], {"max_new_tokens": 4}, session="conv")
    eng.run_until_idle(5000)
    assert len(col.toks[e]) == 4 and not col.err


def test_engine_serves_a_request_with_images(tiny):
    """A request with an image part: the engine decodes the data URL, runs the vision tower, expands the placeholder,
    prefills with the encoder rows and multi-axis positions and decodes with the rotary delta; its tokens equal the
    direct model calls, also while a text request shares the batch (reference: crates/agens-cli/src/mm.rs)."""
    import base64
    import numpy as np
    from agens_engine_b200.models.vision import VisionConfig, VisionTower
    from agens_engine_b200.serve import vision as V
    cfg, ow = tiny
    tower = VisionTower.random_init(VisionConfig(depth=2, d_model=288, n_heads=4, mlp=608, out_dim=cfg.d_model, pos_grid=12), seed=1)
    PAD = 7
    fe = V.VisionFrontEnd(tower, PAD, cfg.head_dim)
    img = np.random.default_rng(0).integers(0, 256, size=(70, 100, 3), dtype=np.uint8)
    url = "data:image/x-portable-pixmap;base64," + base64.b64encode(b"P6\n100 70\n255\n" + img.tobytes()).decode()
    prompt = [20, 21, 22, PAD, 30, 31, 32, 33, 34]
    mm = fe.prepare(prompt, [url])
    assert len(mm["ids"]) == len(prompt) - 1 + 6 and mm["rows"].shape == (6, cfg.d_model)      # 64 x 96 pixels: merged grid 2 x 3
    m = DenseModel.from_oracle(ow, max_seqs=1, max_ctx=512, prefill_chunk=128)
    m.new_seq(0)
    tok, _ = m.prefill(0, torch.tensor(mm["ids"]), image_rows=mm["rows"], image_pad_id=PAD, rope_pos3=mm["pos3"],
                       pair_axis=mm["pair_axis"], rope_next=mm["rope_next"])
    ref = [tok]
    for _ in range(7):
        out, _ = m.forward_rows([ref[-1]], [0])
        ref.append(int(out[0]))
    assert m.rope_delta[0] == mm["rope_next"] - len(mm["ids"]) != 0

    col = Collector()
    eng = Engine(DenseModel.from_oracle(ow, max_seqs=2, max_ctx=512, prefill_chunk=128), col, max_batch=2, vision=fe)
    a = eng.submit(prompt, {"max_new_tokens": 8, "ignore_eos": True}, images=[url])
    b = eng.submit(list(range(40, 60)), {"max_new_tokens": 8, "ignore_eos": True})
    eng.run_until_idle()
    assert col.toks[a] == ref and len(col.toks[b]) == 8 and not col.err
    assert col.toks[b] == _alone(ow, list(range(40, 60)), 8)
    assert eng.stats.images_encoded == 1

    col2 = Collector()
    eng2 = Engine(DenseModel.from_oracle(ow, max_seqs=1, max_ctx=512, prefill_chunk=128), col2)
    c = eng2.submit(prompt, {"max_new_tokens": 4}, images=[url])
    d = eng2.submit(prompt, {"max_new_tokens": 4}, images=["data:image/png;base64,AAAA"])
    eng2.run_until_idle()
    assert "images" in col2.err[c] and col2.done[c] and col2.done[d]


_BUDGET_SCRIPT = r"""
import json, torch
from agens_engine_b200 import cli
cfg = cli.EngineConfig(random="dense-32b-2l", budget_gib=8.0, wctx=262144, max_batch=2, prefill_chunk=256)
m, rank, world, ctrl = cli.build_model(cfg)
out = {"fits": bool(m.deployment.fits), "max_ctx": m.max_ctx, "allocated": torch.cuda.memory_allocated(0),
       "budget": m.deployment.budget_bytes, "booked": m.budget.used, "n_pages": m.n_pages, "plan_pages": m.deployment.n_pages,
       "split_keys": m.split_keys, "peak": torch.cuda.max_memory_allocated(0)}
m.new_seq(0)
first, _ = m.prefill(0, torch.randint(0, m.cfg.vocab, (300,)))
out["first_ok"] = 0 <= int(first) < m.cfg.vocab
try:
    m.reserve(0, m.max_ctx + 64)
    out["over_context"] = "accepted"
except RuntimeError as e:
    out["over_context"] = str(e)
try:
    torch.empty(int(m.deployment.budget_bytes), dtype=torch.uint8, device="cuda:0")
    out["over_cap"] = "accepted"
except Exception as e:
    out["over_cap"] = type(e).__name__
out["status"] = int(m.status.item())
print("RESULT " + json.dumps(out))
"""


def test_budgeted_build_stays_under_the_cap_and_clamps_the_context():
    """`build_model` with a per-GPU budget, in a process of its own (the cap is per process): the KV pool comes from the
    plan, what the load took stays under the budget, a conversation past the planned context is refused on the host and
    an allocation past the cap is refused by the allocator."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", _BUDGET_SCRIPT], capture_output=True, text=True, timeout=300, cwd=root,
                       env=dict(os.environ, PYTHONPATH=root))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    out = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert out["fits"] and out["first_ok"] and out["status"] == 0
    assert out["allocated"] <= out["budget"] and out["booked"] <= out["budget"]
    assert out["n_pages"] == out["plan_pages"] < 2 * 262144 // 16 + 2      # the plan's pool, not max_ctx x max_seqs
    assert out["split_keys"] == 256 and out["peak"] <= out["budget"]
    assert "max_ctx" in out["over_context"]
    assert out["over_cap"] != "accepted"
