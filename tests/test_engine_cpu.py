"""The serving loop on the CPU with a stand-in model (no kernels): the scheduler, the speculative decoder's bookkeeping and
the KV policy run exactly as on a GPU, the "model" is a fixed function of everything a sequence was fed.  Any slip in the
bookkeeping (a token fed twice or not at all, a sequence resumed with the wrong rows, drafts accepted wrongly) changes
the tokens.  Reference gates: serve-smoke, batch-e2e, session and eviction behaviour of crates/agens-cli/src/serve.rs."""
import types

import torch

from agens_engine_b200.serve.engine import Engine
from agens_engine_b200.spec import CopyLookupSource, ModelSource


def _next(tokens):
    return (sum((j % 97 + 1) * v for j, v in enumerate(tokens)) * 31 + 7 * len(tokens)) % 500


class FakeModel:
    def __init__(self, max_seqs=4, max_ctx=256, n_pages=None, page=16, chunk=32, wrong_every=0):
        self.cfg = types.SimpleNamespace(page_size=page, vocab=500, vocab_valid=0, d_model=8, kv_bytes_per_token=lambda tp=1: 64)
        self.dev = torch.device("cpu")
        self.max_seqs, self.max_ctx, self.prefill_chunk, self.max_rows = max_seqs, max_ctx, chunk, 32
        self.n_pages = n_pages or max_seqs * ((max_ctx + page - 1) // page)
        self.tokens, self.seq_len_host, self.seq_pages = {}, {}, {}
        self.hidden_sink = None
        self.h_a = torch.zeros(32, 8)
        self.calls = 0

    # ---- pages ----
    def free_pages(self):
        return self.n_pages - sum(len(p) for p in self.seq_pages.values())

    def _fit(self, s, n):
        if n > self.max_ctx:
            raise RuntimeError("context length exceeds max_ctx")
        need = (n + self.cfg.page_size - 1) // self.cfg.page_size - len(self.seq_pages[s])
        if need > self.free_pages():
            raise RuntimeError("KV pool exhausted")
        self.seq_pages[s] += [0] * max(need, 0)

    def reserve(self, s, n):
        self._fit(s, n)

    def new_seq(self, s):
        assert s not in self.tokens and 0 <= s < self.max_seqs
        self.tokens[s], self.seq_len_host[s], self.seq_pages[s] = [], 0, []

    def free_seq(self, s):
        self.tokens.pop(s); self.seq_len_host.pop(s); self.seq_pages.pop(s)

    def truncate(self, s, n):
        assert n <= len(self.tokens[s])
        del self.tokens[s][n:]
        self.seq_len_host[s] = n
        del self.seq_pages[s][(n + self.cfg.page_size - 1) // self.cfg.page_size:]

    def fork(self, src, dst):
        self.new_seq(dst)
        self._fit(dst, len(self.tokens[src]))
        self.tokens[dst] = list(self.tokens[src])
        self.seq_len_host[dst] = len(self.tokens[dst])

    def park(self, s):
        blob = {"len": len(self.tokens[s]), "tokens": list(self.tokens[s])}
        self.free_seq(s)
        return blob

    def unpark(self, s, blob):
        self.new_seq(s)
        try:
            self._fit(s, blob["len"])
        except RuntimeError:
            self.free_seq(s)
            raise
        self.tokens[s] = list(blob["tokens"])
        self.seq_len_host[s] = blob["len"]

    # ---- forward ----
    def prefill(self, s, ids, want_logits=False, **kw):
        ids = ids.tolist()
        self._fit(s, len(self.tokens[s]) + len(ids))
        self.tokens[s] += ids
        self.seq_len_host[s] = len(self.tokens[s])
        self.calls += 1
        return _next(self.tokens[s]), None

    def forward_rows(self, ids, seqs, want_logits=False):
        assert 1 <= len(ids) <= self.max_rows
        grow = {}
        for s in seqs:
            grow[s] = grow.get(s, 0) + 1
        for s, g in grow.items():
            self._fit(s, len(self.tokens[s]) + g)
        out = []
        for t, s in zip(ids, seqs):
            self.tokens[s].append(int(t))
            out.append(_next(self.tokens[s]))
        for s in grow:
            self.seq_len_host[s] = len(self.tokens[s])
        self.calls += 1
        return torch.tensor(out, dtype=torch.int32), None

    def set_linear_path(self, x): pass
    def device_status(self): return 0
    def recover(self): pass
    def vocab_valid_full(self): return 500


def _alone(prompt, n_new, stop=()):
    toks, out = list(prompt), []
    while len(out) < n_new:
        t = _next(toks)
        if t in stop:
            break
        out.append(t); toks.append(t)
    return out


def _serve(model, reqs, **kw):
    got, done = {}, {}

    def emit(rid, toks, finished, err):
        got.setdefault(rid, []).extend(toks)
        if finished:
            done[rid] = err
        return False
    eng = Engine(model, emit, **kw)
    rids = [eng.submit(p, s) for p, s in reqs]
    eng.run_until_idle(20000)
    assert eng.idle()
    return eng, [got.get(r, []) for r in rids], [done.get(r) for r in rids]


def _prompts(n, lo=5, hi=120, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 500, (int(torch.randint(lo, hi, (1,), generator=g)),), generator=g).tolist() for _ in range(n)]


def test_batched_requests_get_the_tokens_of_a_run_alone():
    prompts = _prompts(9)
    m = FakeModel(max_seqs=4, max_ctx=256)
    eng, outs, errs = _serve(m, [(p, {"max_new_tokens": 20}) for p in prompts])
    assert outs == [_alone(p, 20) for p in prompts] and errs == [None] * 9
    assert eng.stats.peak_batch == 4 and m.free_pages() == m.n_pages and not m.tokens


def test_speculation_with_right_wrong_and_copied_drafts():
    prompts = [p * 3 for p in _prompts(5, lo=6, hi=20, seed=2)]            # repetitive prompts: copy-lookup finds drafts
    want = [_alone(p, 30) for p in prompts]
    # a drafter that computes the same function drafts perfectly; one with another page size of history does not
    class Drafter(FakeModel):
        pass
    good = Drafter(max_seqs=4, max_ctx=256)
    m = FakeModel(max_seqs=4, max_ctx=256)
    eng, outs, _ = _serve(m, [(p, {"max_new_tokens": 30}) for p in prompts], sources_factory=lambda: [ModelSource(good, 3)], max_drafts=3)
    assert outs == want and eng.spec.stats.accepted == eng.spec.stats.proposed > 0
    assert eng.spec.stats.tokens_per_step() > 3.0 and not good.tokens and not m.tokens
    bad = Drafter(max_seqs=4, max_ctx=256)
    bad.forward_rows = lambda ids, seqs, want_logits=False, f=bad.forward_rows: ((f(ids, seqs)[0] + (torch.arange(len(ids)) % 2)).to(torch.int32), None)
    m = FakeModel(max_seqs=4, max_ctx=256)
    eng, outs, _ = _serve(m, [(p, {"max_new_tokens": 30}) for p in prompts], sources_factory=lambda: [CopyLookupSource(), ModelSource(bad, 3)],
                          max_drafts=3)
    assert outs == want and 0 < eng.spec.stats.accepted < eng.spec.stats.proposed


def test_stop_ids_limits_and_context_overflow():
    p = _prompts(1, seed=5)[0]
    full = _alone(p, 40)
    stop = full[7]
    m = FakeModel(max_seqs=2, max_ctx=256)
    eng, outs, errs = _serve(m, [(p, {"max_new_tokens": 40, "stop_token_ids": [stop]}), (p, {"max_new_tokens": 3}),
                                 (list(range(300)), {"max_new_tokens": 4})])
    assert outs[0] == full[:full.index(stop) + 1] and outs[1] == full[:3]        # the stop token itself is delivered (the server drops it)
    assert outs[2] == [] and errs[2] and not m.tokens


def test_kv_pressure_preempts_and_resumes_exactly():
    prompts = _prompts(6, lo=40, hi=100, seed=7)
    m = FakeModel(max_seqs=4, max_ctx=256, n_pages=22)                        # far fewer pages than four full sequences need
    eng, outs, errs = _serve(m, [(p, {"max_new_tokens": 60}) for p in prompts])
    assert outs == [_alone(p, 60) for p in prompts] and errs == [None] * 6
    assert eng.stats.evictions > 0 and m.free_pages() == m.n_pages


def test_kept_sequences_reuse_a_conversation_prefix():
    p1 = _prompts(1, lo=60, hi=61, seed=9)[0]
    m = FakeModel(max_seqs=4, max_ctx=512)
    got = {}
    eng = Engine(m, lambda rid, t, f, e: got.setdefault(rid, []).extend(t) or False, keep_sequences=True)
    r1 = eng.submit(p1, {"max_new_tokens": 10}, session="conv")
    eng.run_until_idle(5000)
    a1 = got[r1]
    assert a1 == _alone(p1, 10)
    calls_before = m.calls
    p2 = p1 + a1 + [11, 12, 13]                                              # the next turn of the same conversation
    r2 = eng.submit(p2, {"max_new_tokens": 10}, session="conv")
    eng.run_until_idle(5000)
    assert got[r2] == _alone(p2, 10)
    fed = m.calls - calls_before
    assert fed <= 1 + 10 + 1, fed                                            # the old turn was not prefilled again (one short chunk + decode)


def test_engine_thread_behind_the_http_front_end(tmp_path):
    """The OpenAI front end (C++) on top of the engine thread on top of the stand-in model: requests in parallel, plain and
    streamed, get the text of the tokens a run alone produces; usage counts them."""
    import json
    import threading
    from agens_engine_b200.serve.engine import attach_to_server
    from agens_engine_b200.serve.server import Server, Tokenizer
    from tests.fixtures import tiny_tokenizer_json
    tok = tmp_path / "tokenizer.json"
    tok.write_text(tiny_tokenizer_json())
    tk = Tokenizer(tiny_tokenizer_json())
    srv = Server(str(tok), model_name="fake", eos_token_ids=[])

    class Bytes(FakeModel):                                  # ids the byte-level test tokenizer can print
        def prefill(self, s, ids, want_logits=False, **kw):
            t, lg = super().prefill(s, ids, want_logits, **kw)
            return 65 + t % 26, lg

        def forward_rows(self, ids, seqs, want_logits=False):
            out, lg = super().forward_rows(ids, seqs, want_logits)
            return 65 + out % 26, lg

    m = Bytes(max_seqs=4, max_ctx=512)
    eng = Engine(m, lambda *a: False)
    attach_to_server(eng, srv)
    eng.start()
    try:
        prompts = ["count to three", "the quick brown fox", "hello", "a b c d e f g"]
        res = {}

        def call(i, stream):
            res[(i, stream)] = srv.handle("POST", "/v1/completions", {"prompt": prompts[i], "max_tokens": 9, "temperature": 0, "stream": stream})
        th = [threading.Thread(target=call, args=(i, st)) for i in range(4) for st in (False, True)]
        [t.start() for t in th]
        [t.join(60) for t in th]
        for i, p in enumerate(prompts):
            toks, want = tk.encode(p), []
            while len(want) < 9:
                want.append(65 + _next(toks) % 26)
                toks.append(want[-1])
            text = tk.decode(want, skip_special=False)
            st, body = res[(i, False)]
            r = json.loads(body)
            assert st == 200 and r["choices"][0]["text"] == text and r["usage"]["completion_tokens"] == 9, (i, body)
            st, body = res[(i, True)]
            ev = [json.loads(x[6:]) for x in body.split("\n\n") if x.startswith("data: {")]
            assert st == 200 and "".join(e["choices"][0]["text"] for e in ev if e["choices"]) == text
        assert "b200e_requests_total 8" in srv.handle("GET", "/metrics")[1]
    finally:
        eng.stop()
    assert not m.tokens


def test_a_failed_step_ends_open_requests_and_the_engine_keeps_serving():
    """A step that raises (a device error status, a bounds check) ends every running request with an error, the model is
    put back into a clean state and the engine thread keeps serving: later requests get exact tokens.  A failure marked
    fatal (a tensor-parallel follower is gone) ends the engine instead, and waiting requests are told."""
    import time

    class Flaky(FakeModel):
        fail_at, fatal = -1, False

        def forward_rows(self, ids, seqs, want_logits=False):
            if self.calls == self.fail_at:
                self.fail_at = -1
                e = (RuntimeError if self.fatal else ValueError)("the step went wrong")
                e.fatal = self.fatal
                raise e
            return super().forward_rows(ids, seqs, want_logits)

        def device_status(self):
            st, self.status_once = getattr(self, "status_once", 0), 0
            return st

        def recover(self):
            for s in list(self.tokens):
                self.free_seq(s)

    got, done = {}, {}

    def emit(rid, toks, finished, err):
        got.setdefault(rid, []).extend(toks)
        if finished:
            done[rid] = err
        return False
    m = Flaky(max_seqs=4, max_ctx=256)
    eng = Engine(m, emit)
    eng.start()
    try:
        prompts = _prompts(6, lo=10, hi=40, seed=3)
        m.fail_at = 12                                             # somewhere in the decode steps of the first batch
        first = [eng.submit(p, {"max_new_tokens": 30}) for p in prompts[:3]]
        t0 = time.time()
        while len(done) < 3 and time.time() - t0 < 30:
            time.sleep(0.01)
        assert all(done.get(r) and "engine step failed" in done[r] for r in first), done
        assert not m.tokens and m.free_pages() == m.n_pages
        later = [eng.submit(p, {"max_new_tokens": 12}) for p in prompts[3:]]
        t0 = time.time()
        while len(done) < 6 and time.time() - t0 < 30:
            time.sleep(0.01)
        assert [got[r] for r in later] == [_alone(p, 12) for p in prompts[3:]] and all(done[r] is None for r in later)
        # a device status word (a bounded wait that ran out) is found after the step: same recovery
        m.status_once = 3
        more = [eng.submit(p, {"max_new_tokens": 8}) for p in prompts[:2]]
        t0 = time.time()
        while len(done) < 8 and time.time() - t0 < 30:
            time.sleep(0.01)
        assert any("device reported" in (done.get(r) or "") for r in more) and not m.tokens, done
        done.pop(more[0]); done.pop(more[1])
        # a fatal failure: the engine thread ends, open and waiting requests are told why
        m.fail_at, m.fatal = m.calls + 3, True
        last = [eng.submit(p, {"max_new_tokens": 30}) for p in prompts[:5]]
        t0 = time.time()
        while len(done) < 11 and time.time() - t0 < 30:
            time.sleep(0.01)
        assert eng.fatal is not None and all("engine stopped" in (done.get(r) or "") for r in last), done
    finally:
        eng.stop()


def test_random_workloads_keep_every_request_exact_and_leak_nothing():
    """Seeded random deployments: pool sizes from ample to tight, batch widths, draft sources that are right, wrong or
    copied, stop ids, clients that go away, kept conversations.  Every request that ends without an error has exactly
    the tokens of a run alone (up to its stop or limit), and when the engine is idle no page or slot is held."""
    import random
    seen = {"evictions": 0, "accepted": 0, "rejected_drafts": 0, "left": 0, "errors": 0}
    for seed in range(40):
        rng = random.Random(seed)
        max_seqs = rng.choice([2, 3, 4, 6])
        max_ctx = rng.choice([128, 256])
        page = rng.choice([8, 16])
        full = max_seqs * ((max_ctx + page - 1) // page)
        n_pages = rng.choice([full, full // 2, max(full // 3, (max_ctx + page - 1) // page + 2)])
        m = FakeModel(max_seqs=max_seqs, max_ctx=max_ctx, n_pages=n_pages, page=page, chunk=rng.choice([16, 32, 64]))
        kw = {}
        mode = rng.choice(["plain", "good", "bad", "copy"])
        if mode != "plain":
            d = FakeModel(max_seqs=max_seqs, max_ctx=max_ctx, page=page)
            if mode == "bad":
                d.forward_rows = lambda ids, seqs, want_logits=False, f=d.forward_rows: ((f(ids, seqs)[0] + (torch.arange(len(ids)) % 3 == 1)).to(torch.int32), None)
            srcs = [CopyLookupSource()] if mode == "copy" else [CopyLookupSource(), ModelSource(d, rng.choice([2, 3]))]
            kw = dict(sources_factory=lambda srcs=srcs: srcs, max_drafts=rng.choice([2, 3]))
        keep = rng.random() < 0.4
        got, done, gone = {}, {}, {}

        def emit(rid, toks, finished, err):
            got.setdefault(rid, []).extend(toks)
            if finished:
                done[rid] = err
            return rid in gone and len(got[rid]) >= gone[rid]          # True: the client went away
        eng = Engine(m, emit, keep_sequences=keep, max_batch=rng.choice([2, 4, 8]), **kw)
        reqs = {}
        for wave in range(3):
            for _ in range(rng.randint(1, 5)):
                base = [rng.randrange(500) for _ in range(rng.randint(3, 12))]
                prompt = (base * rng.randint(1, 6))[:max_ctx - 40] if rng.random() < 0.5 else [rng.randrange(500) for _ in range(rng.randint(4, max_ctx - 60))]
                n_new = rng.randint(1, 30)
                samp = {"max_new_tokens": n_new}
                alone = _alone(prompt, n_new)
                stop = None
                if rng.random() < 0.3 and len(alone) > 2:
                    stop = alone[rng.randrange(1, len(alone))]
                    samp["stop_token_ids"] = [stop]
                rid = eng.submit(prompt, samp, session=f"s{rng.randrange(3)}" if keep and rng.random() < 0.5 else "")
                if rng.random() < 0.15:
                    gone[rid] = rng.randint(1, max(1, n_new // 2))
                want = alone if stop is None else alone[:alone.index(stop) + 1]
                reqs[rid] = want
            for _ in range(rng.randint(0, 40)):
                eng.step()
        eng.run_until_idle(50000)
        assert eng.idle(), seed
        for rid, want in reqs.items():
            assert rid in done or rid in gone, (seed, rid)              # nobody is told about a request whose client left
            if rid in done and done[rid] is None and rid not in gone:
                assert got.get(rid, []) == want, (seed, rid, mode)
            else:
                assert got.get(rid, []) == want[:len(got.get(rid, []))], (seed, rid, mode)
        if not keep:
            assert not m.tokens and m.free_pages() == m.n_pages, seed
        seen["evictions"] += eng.stats.evictions
        seen["accepted"] += eng.spec.stats.accepted
        seen["rejected_drafts"] += eng.spec.stats.proposed - eng.spec.stats.accepted
        seen["left"] += len(gone)
        seen["errors"] += sum(1 for e in done.values() if e)
    assert seen["evictions"] > 0 and seen["accepted"] > 0 and seen["rejected_drafts"] > 0 and seen["left"] > 0, seen


def test_the_scheduler_itself_is_cheap_at_128k_tokens():
    """A 128K-token conversation through the engine with a stand-in model that costs nothing: admission, chunking, the
    prefix cache, the copy-lookup index and keeping the sequence for the next turn take well under a second (keeping it
    alone took 18 s when every chunk boundary was hashed from the start of the prompt)."""
    import time

    class Free(FakeModel):
        def prefill(self, s, ids, want_logits=False, **kw):
            self._fit(s, len(self.tokens[s]) + len(ids))
            self.tokens[s] += ids.tolist()
            self.seq_len_host[s] = len(self.tokens[s])
            return 5, None

        def forward_rows(self, ids, seqs, want_logits=False):
            for t, s in zip(ids, seqs):
                self.tokens[s].append(int(t))
                self.seq_len_host[s] = len(self.tokens[s])
            for s in set(seqs):
                self._fit(s, len(self.tokens[s]))
            return torch.tensor([7] * len(ids), dtype=torch.int32), None
    m = Free(max_seqs=2, max_ctx=140000, page=16, chunk=8192)
    got = {}
    eng = Engine(m, lambda rid, t, f, e: got.setdefault(rid, []).extend(t) or False, sources_factory=lambda: [CopyLookupSource()],
                 max_drafts=3, keep_sequences=True)
    prompt = torch.randint(0, 500, (131072,)).tolist()
    t0 = time.time()
    r1 = eng.submit(prompt, {"max_new_tokens": 16}, session="a")
    eng.run_until_idle(100000)
    t1 = time.time()
    r2 = eng.submit(prompt + got[r1] + [3, 4, 5], {"max_new_tokens": 16}, session="a")     # the next turn takes the kept sequence over
    eng.run_until_idle(100000)
    t2 = time.time()
    assert len(got[r1]) == 16 and len(got[r2]) == 16 and t1 - t0 < 5.0 and t2 - t1 < 5.0, (t1 - t0, t2 - t1)
