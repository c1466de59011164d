"""CPU tests of the host-side C++ runtime (sampler, budget, guard, pages, admission, lookup, prefix cache, planner).
Modelled on the reference's unit tests (sampler.rs:286-365, profile.rs:90-144) plus the pieces it leaves untested
(lookup.rs, prefix.rs, plan.rs, kv_safe)."""
import numpy as np
import pytest

from agens_engine_b200.serve import host as H


def test_sampler_greedy_first_max_and_bias_suppress():
    s = H.Sampler({"temperature": 0.0})
    x = np.zeros(100, np.float32); x[7] = 3; x[50] = 3
    assert s.sample(x) == 7                          # first index of the maximum
    s = H.Sampler({"temperature": 0.0, "logit_bias": {"50": 1.0}})
    assert s.sample(x) == 50
    s = H.Sampler({"temperature": 0.0, "suppress_tokens": [7, 50]})
    assert s.sample(x) not in (7, 50)
    assert s.needs_logits(100) and not H.Sampler({"temperature": 0.0}).needs_logits(100)


def test_sampler_seed_determinism_and_filters():
    x = np.random.RandomState(0).randn(1000).astype(np.float32) * 3
    a = [H.Sampler({"temperature": 1.0, "seed": 5}).sample(x) for _ in range(3)]
    assert len(set(a)) == 1
    s1, s2 = H.Sampler({"temperature": 1.0, "seed": 5}), H.Sampler({"temperature": 1.0, "seed": 6})
    assert [s1.sample(x) for _ in range(20)] != [s2.sample(x) for _ in range(20)]
    top = set(np.argsort(-x)[:5].tolist())
    s = H.Sampler({"temperature": 1.0, "top_k": 5, "seed": 1})
    assert all(s.sample(x) in top for _ in range(200))
    s = H.Sampler({"temperature": 1.0, "top_p": 1e-9, "seed": 1})
    assert all(s.sample(x) == int(np.argmax(x)) for _ in range(50))
    s = H.Sampler({"temperature": 1.0, "min_p": 0.9999, "seed": 2})
    assert all(s.sample(x) == int(np.argmax(x)) for _ in range(50))


def test_sampler_matches_softmax_distribution():
    x = np.array([2.0, 1.0, 0.0, -1.0], np.float32)
    p = np.exp(x / 0.7); p /= p.sum()
    s = H.Sampler({"temperature": 0.7, "seed": 123})
    n = 20000
    cnt = np.bincount([s.sample(x) for _ in range(n)], minlength=4) / n
    assert np.abs(cnt - p).max() < 0.015


def test_sampler_penalties_and_min_new_tokens():
    x = np.zeros(10, np.float32); x[3] = 2.0; x[4] = 1.9
    s = H.Sampler({"temperature": 0.0, "repetition_penalty": 2.0})
    assert s.sample(x) == 3
    s.accept(3)
    assert s.sample(x) == 4                          # 2.0 / 2 < 1.9
    s = H.Sampler({"temperature": 0.0, "presence_penalty": 0.5})
    s.accept(3)
    assert s.sample(x) == 4
    s = H.Sampler({"temperature": 0.0, "min_new_tokens": 2, "stop_token_ids": [3]})
    assert s.sample(x) == 4
    s.accept(4); s.accept(4)
    assert s.sample(x) == 3


def test_reasoning_budget_forces_close():
    S, E = 90, 91
    b = H.ReasoningBudget(3, 0.0, [1, 2, S], S, E)           # block open in the prompt tail
    acts = []
    for j in range(5):
        a = b.act(j)
        acts.append(a[0])
        tok = E if a[0] == "force" else 5
        b.accept(j, tok)
    assert acts[:4] == ["none", "none", "none", "force"]
    assert b.act(5) == ("bias", S, float("-inf"))            # reopening is masked after a forced close
    soft = H.ReasoningBudget(10, 2.5, [S], S, E)
    assert soft.act(7) == ("none",) and soft.act(8) == ("bias", E, 2.5)


def test_think_guard_fires_on_repetition():
    S, E = 90, 91
    g = H.ThinkGuard(3, 3, 64, [S], S, E)
    out = [g.filter(t) for t in [1, 2, 3, 1, 2, 3, 1, 2, 3]]
    assert g.fired is not None and out[-1] == 3
    assert g.filter(7) == E                                  # next replaceable token becomes the closing tag
    g2 = H.ThinkGuard(3, 3, 64, [5], S, E)                   # no open block: never fires
    for t in [1, 2, 3] * 5:
        g2.filter(t)
    assert g2.fired is None


def test_page_allocator_fork_truncate_refcounts():
    a = H.PageAllocator(8, 16)
    s = a.new_seq()
    assert a.reserve(s, 40) == 3 and a.free_pages == 5
    a.set_len(s, 40)
    c, src, dst = a.fork(s)
    assert c >= 0 and src == a.pages(s)[2] and dst == a.pages(c)[2] and a.free_pages == 4
    assert a.pages(c)[:2] == a.pages(s)[:2] and a.refcount(a.pages(s)[0]) == 2
    assert a.exclusive(s) == 1
    a.set_len(s, 32)
    c2, src2, dst2 = a.fork(s)                               # page-aligned fork copies nothing
    assert src2 == -1 and dst2 == -1
    assert a.reserve(c, 16 * 9) == -1                        # does not fit: nothing changes
    assert a.free_seq(s) == 1                                # only its exclusive partial page comes back
    assert a.truncate(c, 16) == 1                            # c's own partial page; shared page 1 stays (c2 holds it)
    a.free_seq(c); a.free_seq(c2)
    assert a.free_pages == 8


def test_bankers_check_and_victims_and_prefill_order():
    assert H.kv_safe(10, [(4, 6), (12, 1), (9, 3)])          # 4 -> 16 -> 9 -> 19 -> 12
    assert not H.kv_safe(3, [(4, 6), (2, 0)])
    cands = [(1, 10, 50.0, 0), (0, 77, 5.0, 0), (1, 11, 2.0, 0), (1, 12, 100.0, 1)]
    assert H.pick_victim(cands) == 1                         # unreferenced snapshot first
    assert H.pick_victim(cands[:1] + cands[2:]) == 0         # then the conversation idle past the hold window
    assert H.pick_victim(cands[2:]) == -1                    # the rest is protected ...
    assert H.pick_victim(cands[2:], allow_protected=True) == 0   # ... unless the waiting request has waited long enough
    assert H.pick_prefill([500, 100, 300], [3.0, 1.0, 2.0], 0) == 1      # shortest remaining prompt
    assert H.pick_prefill([500, 100, 300], [3.0, 1.0, 2.0], 3) == 0      # every 4th chunk: the oldest
    assert H.pick_prefill([500, 100, 300], [3.0, 1.0, 2.0], 0, srpt=False) == 0


def test_copy_lookup_proposes_continuation():
    lk = H.CopyLookup()
    text = [5, 6, 7, 8, 9, 10, 11, 12, 1, 2, 3, 5, 6, 7]
    lk.extend(text)
    toks, m = lk.propose(copy_only=True)
    assert toks == [8, 9, 10, 11, 12, 1, 2] and m == 3
    toks2, _ = lk.propose(copy_only=False)                   # bucket prior 1.0 < drafter prior 2.0: defer to the drafter
    assert toks2 == []
    for _ in range(60):                                      # copying keeps paying off -> its bucket overtakes
        lk.propose(copy_only=True); lk.record(7)
    assert lk.mean(1) > lk.mean(-1)
    assert lk.propose(copy_only=False)[0] == toks


def test_prefix_cache_longest_prefix_and_lru():
    pc = H.PrefixCache(300, 4)
    toks = list(range(12))
    assert pc.lookup(toks) == (0, -1)
    assert pc.insert(toks[:4], 100, 100)[0] == 0 and pc.insert(toks[:8], 101, 100)[0] == 0
    assert pc.lookup(toks) == (8, 101)
    assert pc.lookup(toks[:7]) == (4, 100)
    assert pc.lookup([9] + toks[1:]) == (0, -1)
    other = [50, 51, 52, 53]
    assert pc.insert(other, 102, 100)[0] == 0 and pc.used == 300
    pc.lookup(toks[:4])                                      # touch 100 -> 101 is now least recently used
    n, ev = pc.insert([60, 61, 62, 63], 103, 100)
    assert n == 1 and ev == [101]
    pc.ref(100, +1)
    assert pc.insert(toks[:5], 104, 100)[0] == -1            # not on a chunk boundary
    assert pc.lookup(toks, salt=7) == (0, -1)                # image keys change the chain


def test_planner_gpu_and_host_tier_and_profiles():
    base = dict(weights_bytes=15 * 2**30, kv_bytes_per_token=262144, page_size=16, max_batch=16, sessions=1,
                prefill_chunk=8192, wctx=258052)
    p = H.plan(budget_gib=160, **base)
    assert p["fits"] and p["tier"] == "gpu" and p["context"] == 258052 and p["pool_tokens"] >= 258052
    p16 = H.plan(budget_gib=24, host_avail_gib=200, **base)
    assert p16["tier"] == "host" and p16["host_pages"] > 0 and p16["context"] == 258052
    assert any("tiered" in l for l in p16["lines"])
    clamp = H.plan(budget_gib=24, host_avail_gib=20, **base)
    assert clamp["context"] < 258052 and any("clamped" in l for l in clamp["lines"])
    none = H.plan(budget_gib=24, allow_host_tier=False, **base)
    assert none["tier"] == "gpu" and none["context"] == none["pool_tokens"]
    pr = H.profile("16gb")
    assert pr["flags"]["budget_gib"] == 16 and pr["flags"]["wctx"] == 262148 and pr["flags"]["mode"] == "personal"
    assert H.profile("48gb", 8)["flags"]["tp"] == 8
    assert "error" in H.profile("16gb", 3) and "error" in H.profile("nope")


def test_page_allocator_against_a_model_under_random_operations():
    """Reserve / truncate / fork / free / evict in seeded random order against a plain Python restatement: the same page
    counts, reference counts that equal the number of holders, free + held = total at every step; unknown ids come back
    as an error code instead of ending the process."""
    import random
    for seed in range(20):
        rng = random.Random(seed)
        n_pages, page = rng.choice([8, 24, 64]), rng.choice([4, 16])
        a = H.PageAllocator(n_pages, page)
        model = {}                                             # id -> [pages (or -2), len]
        for _ in range(400):
            op = rng.random()
            ids = list(model)
            if op < 0.2 or not ids:
                s = a.new_seq()
                assert s not in model
                model[s] = [[], 0]
            elif op < 0.5:
                s = rng.choice(ids)
                n = rng.randint(0, page * 10)
                need = max(0, (n + page - 1) // page - len(model[s][0]))
                got = a.reserve(s, n)
                if need > a_free(model, n_pages):
                    assert got == -1
                else:
                    assert got == need
                    model[s][0] = a.pages(s)
                    if n > model[s][1] and got >= 0:
                        model[s][1] = min(n, len(model[s][0]) * page)
                        a.set_len(s, model[s][1])
            elif op < 0.65:
                s = rng.choice(ids)
                n = rng.randint(0, max(model[s][1], 1))
                a.truncate(s, n)
                model[s][1] = min(model[s][1], n)
                del model[s][0][(n + page - 1) // page:]
            elif op < 0.8:
                s = rng.choice(ids)
                c, src, dst = a.fork(s)
                partial = model[s][1] % page != 0
                if any(p < 0 for p in model[s][0]) or (partial and a_free(model, n_pages) == 0):
                    assert c == -1
                else:
                    assert c >= 0 and (src >= 0) == partial
                    model[c] = [a.pages(c), model[s][1]]
                    used = (model[s][1] + page - 1) // page
                    assert len(model[c][0]) == used and model[c][0][:used - (1 if partial else 0)] == model[s][0][:used - (1 if partial else 0)]
            elif op < 0.9:
                s = rng.choice(ids)
                a.free_seq(s)
                del model[s]
            else:
                s = rng.choice(ids)
                if model[s][0]:
                    i = rng.randrange(len(model[s][0]))
                    a.evict_page(s, i)
                    model[s][0][i] = -2
            # invariants
            held = {}
            for s, (pages, n) in model.items():
                assert a.pages(s) == pages and a.seq_len(s) == n, (seed, s)
                for p in pages:
                    if p >= 0:
                        held[p] = held.get(p, 0) + 1
            assert a.free_pages == n_pages - len(held)
            assert all(a.refcount(p) == c for p, c in held.items())
        assert a.reserve(10**6, 5) == -1000 and a.seq_len(10**6) == -1000 and a.refcount(-1) == -1000 and a.pages(10**6) == []
        assert a.fork(10**6)[0] == -1000 and a.truncate(10**6, 0) == -1000 and a.free_seq(10**6) == 0


def a_free(model, n_pages):
    return n_pages - len({p for pages, _ in model.values() for p in pages if p >= 0})


def test_prefix_chain_insert_equals_one_insert_per_boundary():
    """insert_chain registers every chunk boundary of a token list in one pass; lookups and evictions behave as after one
    insert() per boundary (which hashed every prefix from its start: 18 s for a 128K-token conversation)."""
    import random
    import time
    rng = random.Random(3)
    toks = [rng.randrange(50000) for _ in range(1000)]
    a, b = H.PrefixCache(10_000, 64), H.PrefixCache(10_000, 64)
    for cache, chained in ((a, False), (b, True)):
        cache.insert([1] * 128, 7, 6000)                       # an older snapshot that the new one pushes out
        if chained:
            n, ev = cache.insert_chain(toks, 9, 5000)
        else:
            ev = []
            top = len(toks) // 64 * 64
            for c in range(64, top + 1, 64):
                _, e = cache.insert(toks[:c], 9, 5000 if c == top else 0)
                ev += e
        assert ev == [7] and cache.used == 5000
    for probe in (toks, toks[:700], toks[:64] + [0] * 200, toks[:63], [5] * 300):
        assert a.lookup(probe) == b.lookup(probe)
    assert b.lookup(toks) == (960, 9) and b.lookup(toks[:700]) == (640, 9)
    big = [rng.randrange(50000) for _ in range(131072)]
    c = H.PrefixCache(1 << 40, 64)
    t0 = time.time()
    c.insert_chain(big, 1, 1 << 30)
    assert c.lookup(big) == (131072, 1) and time.time() - t0 < 2.0
