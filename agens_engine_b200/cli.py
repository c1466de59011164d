"""Command line: ``python -m agens_engine_b200 <command>``.

Commands mirror the reference's ``agens`` binary (``crates/agens-cli/src/main.rs:31-126``): ``--version``, ``inspect``,
``validate``, ``verify``, ``load``, ``devices``, ``plan`` (m1-plan dry run), ``profile``, the offline gates ``run`` (m1),
``kv`` (m1-kv), ``spec`` (m1-spec), ``batch`` (m1-batch), ``session`` (m1-session) and ``serve``.  A model comes from
``--model-dir`` (checkpoint directory) or ``--random NAME`` (random-init weights of a named architecture:
``oracle-tiny``, ``dense-32b``, ``dense-32b-<L>l``, ``drafter-0.6b``).  Settings resolve in the order model config ->
profile -> flags -> ``B200E_*`` environment, and the resolved set is printed at start-up.
"""
from __future__ import annotations

import argparse
import dataclasses
import hashlib
import json
import os
import sys
import time
from typing import List, Optional

VERSION = "0.1.0"


@dataclasses.dataclass
class EngineConfig:
    """Every knob of a run in one typed record (flags override profile values, ``B200E_<NAME>`` overrides flags)."""
    model_dir: Optional[str] = None
    random: Optional[str] = None
    seed: int = 0
    tp: int = 1
    device: int = 0
    budget_gib: float = 0.0
    wctx: int = 8192
    max_batch: int = 8
    max_convs: int = 64
    mode: str = "server"
    prefill_chunk: int = 256
    split_keys: int = 64
    spec_copy: int = 0
    spec_drafter: Optional[str] = None
    mtp: Optional[str] = None
    mtp_vocab: Optional[str] = None       # shortlist of the MTP head's lm_head: a count (first N ids) or a file of uint32 ids
    draft_depth: int = 4
    host: str = "127.0.0.1"
    port: int = 30000
    served_model_name: str = "b200-engine"
    max_tokens_default: int = 32768
    think_guard: str = "off"
    tokenizer: Optional[str] = None
    profile: Optional[str] = None
    row_graphs: int = 1
    vision: int = 0

    @staticmethod
    def resolve(ns: argparse.Namespace) -> "EngineConfig":
        from .serve import host as H
        cfg = EngineConfig()
        if getattr(ns, "profile", None):
            prof = H.profile(ns.profile, getattr(ns, "tp", None) or 1)
            for k, v in prof.get("flags", {}).items():
                k = k.replace("-", "_")
                if hasattr(cfg, k):
                    setattr(cfg, k, type(getattr(cfg, k))(v) if getattr(cfg, k) is not None else v)
            for k, v in prof.get("env", {}).items():
                os.environ.setdefault(k, str(v))
        for f in dataclasses.fields(cfg):
            v = getattr(ns, f.name, None)
            if v is not None:
                setattr(cfg, f.name, v)
            e = os.environ.get("B200E_" + f.name.upper())
            if e is not None:
                cur = getattr(cfg, f.name)
                setattr(cfg, f.name, type(cur)(e) if cur is not None else e)
        return cfg


def _named_config(name: str):
    from .models import config as C
    if name == "oracle-tiny":
        return C.oracle_tiny()
    if name == "drafter-0.6b":
        return C.drafter_0p6b()
    if name.startswith("dense-32b"):
        base = C.dense_32b()
        rest = name[len("dense-32b"):]
        return C.scaled(base, int(rest.strip("-l"))) if rest else base
    raise SystemExit(f"unknown architecture {name!r}")


def _model_config(cfg: EngineConfig):
    if cfg.model_dir:
        from .models.config import ModelConfig
        return ModelConfig.from_json(os.path.join(cfg.model_dir, "config.json"))
    if cfg.random:
        return _named_config(cfg.random)
    raise SystemExit("give --model-dir DIR or --random NAME")


def build_model(cfg: EngineConfig, **kw):
    """Builds the (possibly tensor-parallel) model of this rank.  Returns ``(model, rank, world, ctrl_group)``.

    With ``--budget-gib`` the load is planned first (``serve/budget.py``): the KV pool gets the pages the plan grants,
    the context is clamped to what the pool plus the host tier can hold, the host tier is switched on when the plan
    says so, every rank takes the minimum, the process's allocator is capped at the budget, and the plan is printed.
    Reference: crates/agens-cli/src/m1.rs:905-974, plan.rs:182-241, tp.rs:77-90."""
    import torch
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    kw.setdefault("max_seqs", max(cfg.max_batch, 1))
    kw.setdefault("max_ctx", cfg.wctx)
    kw.setdefault("prefill_chunk", cfg.prefill_chunk)
    kw.setdefault("split_keys", cfg.split_keys)
    # long contexts: at most 1024 attention splits per (row, head), so that the split partials stay near 1 GB at 256K
    want = (kw["max_ctx"] + 1023) // 1024
    while kw["split_keys"] < want:
        kw["split_keys"] *= 2
    ctrl = None
    local = int(os.environ.get("LOCAL_RANK", rank)) if world > 1 else cfg.device
    dev = f"cuda:{local}"
    if world > 1:
        import torch.distributed as dist
        from .parallel import driver as D
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device(dev))
        ctrl = D.control_group()
    dep = ledger = None
    if cfg.budget_gib > 0:
        from .serve import budget as B
        mc = _model_config(cfg)
        free, _total = torch.cuda.mem_get_info(local)
        dep = B.plan_deployment(mc, cfg.budget_gib, kw["max_ctx"], cfg.max_batch, kw["max_seqs"], kw["prefill_chunk"], tp=world,
                                gpu_free_gib=free / B.GiB, dual_layout=os.environ.get("B200E_STEP", "auto") != "0",
                                split_keys=kw["split_keys"])
        if world > 1:
            import torch.distributed as dist

            def all_min(v):
                t = torch.tensor(v, dtype=torch.int64)
                dist.all_reduce(t, op=dist.ReduceOp.MIN, group=ctrl)
                return t.tolist()
            dep = B.agree_min(dep, all_min)
        if rank == 0:
            for line in dep.lines:
                print(line, flush=True)
        if not dep.fits or dep.n_pages <= 0:
            raise SystemExit(f"plan: weights and scratch do not fit {cfg.budget_gib} GiB per GPU")
        kw["n_pages"] = dep.n_pages
        kw["max_ctx"] = max(dep.max_ctx, mc.page_size)
        B.cap_process(dep.budget_bytes, local)
        ledger = B.BudgetLedger(dep.budget_bytes)
    if world > 1:
        from .parallel.tp_model import TpDenseModel
        if cfg.random is None:
            from .utils import checkpoint as K
            m = K.load_model(cfg.model_dir, dev, rank=rank, world=world, **kw)
        else:
            m = TpDenseModel.random_init(_named_config(cfg.random), dev, cfg.seed, rank, world, **kw)
    elif cfg.model_dir:
        from .utils import checkpoint as K
        m = K.load_model(cfg.model_dir, dev, **kw)
    elif cfg.random:
        from .models.dense import DenseModel
        m = DenseModel.random_init(_named_config(cfg.random), dev, seed=cfg.seed, **kw)
    else:
        raise SystemExit("give --model-dir DIR or --random NAME")
    if dep is not None:
        # book what the load took and hold the deployment to it from here on
        torch.cuda.synchronize(m.dev)
        ledger.book("weights, KV pool and buffers (allocator)", torch.cuda.memory_allocated(m.dev))
        m.budget, m.deployment = ledger, dep
        tier_on = dep.host_tier and os.environ.get("B200E_KV_TIER", "host") != "off" and world == 1
        if tier_on:
            m.enable_host_tier(max(dep.resident_window_tokens, 16 * 256))
        if rank == 0:
            for line in ledger.report():
                print(line, flush=True)
            print(f"plan: context per conversation {kw['max_ctx']} tokens, host tier {'on' if tier_on else 'off'}", flush=True)
    return m, rank, world, ctrl


def _hash(tokens: List[int]) -> str:
    return hashlib.sha256(json.dumps(list(map(int, tokens))).encode()).hexdigest()[:16]


def _prompt(cfg_model, n: int, seed: int) -> List[int]:
    import torch
    g = torch.Generator().manual_seed(seed)
    hi = cfg_model.vocab_valid or cfg_model.vocab
    return torch.randint(0, hi, (n,), generator=g).tolist()


# ---------------------------------------------------------------------------------------------------------------------
def cmd_inspect(ns):
    from .utils import checkpoint as K
    print(json.dumps(K.inspect(ns.dir), indent=1))


def cmd_validate(ns):
    from .utils import checkpoint as K
    rep = K.validate(ns.dir)
    print(json.dumps(rep, indent=1))
    return 0 if rep["ok"] else 1


def cmd_verify(ns):
    from .utils import checkpoint as K
    rep = K.verify(ns.dir, threads=ns.threads)
    print(json.dumps(rep, indent=1))
    return 0 if rep.get("ok") else 1


def cmd_devices(ns):
    import torch
    out = []
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        free, total = torch.cuda.mem_get_info(i)
        peers = [j for j in range(torch.cuda.device_count()) if j != i and torch.cuda.can_device_access_peer(i, j)]
        out.append({"index": i, "name": p.name, "cc": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                    "total_gib": round(total / 2**30, 2), "free_gib": round(free / 2**30, 2), "peers": peers})
    print(json.dumps(out, indent=1))


def cmd_plan(ns):
    from .serve import host as H
    cfg = EngineConfig.resolve(ns)
    mc = _named_config(cfg.random) if cfg.random else None
    if cfg.model_dir:
        from .models.config import ModelConfig
        mc = ModelConfig.from_json(os.path.join(cfg.model_dir, "config.json"))
    if mc is None:
        raise SystemExit("give --model-dir DIR or --random NAME")
    rep = H.plan(budget_gib=cfg.budget_gib, gpu_free_gib=ns.gpu_free_gib, weights_bytes=mc.weight_bytes(cfg.tp),
                 kv_bytes_per_token=mc.kv_bytes_per_token(cfg.tp), page_size=mc.page_size, max_batch=cfg.max_batch,
                 sessions=cfg.max_convs, prefill_chunk=ns.plan_prefill_chunk, d_model=mc.d_model, ffn=mc.ffn, q_dim=mc.q_dim,
                 kv_dim=mc.kv_dim, vocab=mc.vocab, n_heads=mc.n_heads, head_dim=mc.head_dim, tp=cfg.tp, wctx=cfg.wctx,
                 host_avail_gib=ns.host_avail_gib)
    for line in rep.get("lines", []):
        print(line)
    print(json.dumps({k: v for k, v in rep.items() if k != "lines"}, indent=1))


def cmd_profile(ns):
    from .serve import host as H
    print(json.dumps(H.profile(ns.name, ns.tp or 1), indent=1))


def cmd_load(ns):
    import torch
    cfg = EngineConfig.resolve(ns)
    t0 = time.time()
    m, rank, world, _ = build_model(cfg)
    torch.cuda.synchronize()
    if rank == 0:
        print(json.dumps({"loaded": cfg.model_dir or cfg.random, "seconds": round(time.time() - t0, 2), "tp": world,
                          "weight_gib": round(m.weight_bytes() / 2**30, 3), "kv_pages": m.n_pages,
                          "device_gib_in_use": round(torch.cuda.memory_allocated() / 2**30, 3)}))


def cmd_run(ns):
    """Greedy generation gate: prints the tokens' hash; two runs must print the same line."""
    import torch
    cfg = EngineConfig.resolve(ns)
    m, rank, world, ctrl = build_model(cfg, max_seqs=1, max_ctx=max(cfg.wctx, ns.prompt_len + ns.new_tokens + 16))
    prompt = _prompt(m.cfg if world == 1 else m.full_cfg, ns.prompt_len, cfg.seed)
    m.new_seq(0)
    t0 = time.time()
    toks = m.generate_greedy(0, torch.tensor(prompt), ns.new_tokens).tolist()
    dt = time.time() - t0
    if rank == 0:
        print(json.dumps({"tokens_hash": _hash(toks), "first": toks[:8], "n": len(toks), "seconds": round(dt, 3)}))
    _finish(m, world)


def cmd_kv(ns):
    """Teacher-forced logits determinism: the same prompt twice must give bitwise equal last-token logits."""
    import torch
    cfg = EngineConfig.resolve(ns)
    m, rank, world, _ = build_model(cfg, max_seqs=2, max_ctx=max(cfg.wctx, ns.prompt_len + 16))
    prompt = torch.tensor(_prompt(m.cfg, ns.prompt_len, cfg.seed))
    outs = []
    for s in (0, 1):
        m.new_seq(s)
        _, lg = m.prefill(s, prompt, want_logits=True)
        outs.append(lg)
    same = bool(torch.equal(outs[0], outs[1]))
    if ns.save_logits:
        torch.save(outs[0].cpu(), ns.save_logits)
    rep = {"bitwise_equal": same, "logits_hash": hashlib.sha256(outs[0].cpu().numpy().tobytes()).hexdigest()[:16]}
    if ns.cmp_logits:
        ref = torch.load(ns.cmp_logits)
        p, q = torch.log_softmax(ref.double(), -1), torch.log_softmax(outs[0].cpu().double(), -1)
        rep["kl"] = float((p.exp() * (p - q)).sum())
        rep["argmax_equal"] = bool(ref.argmax() == outs[0].cpu().argmax())
    print(json.dumps(rep))
    return 0 if same else 1


def cmd_spec(ns):
    """Speculation gate: with perfect, corrupted and garbage drafts the output equals plain greedy decoding."""
    from .spec import SpecDecoder
    cfg = EngineConfig.resolve(ns)
    m, rank, world, _ = build_model(cfg, max_seqs=2, max_ctx=max(cfg.wctx, ns.prompt_len + ns.new_tokens + 16))
    m.row_graphs = bool(cfg.row_graphs)
    prompt = _prompt(m.cfg, ns.prompt_len, cfg.seed)
    plain = SpecDecoder(m, [], max_drafts=0).generate(0, prompt, ns.new_tokens)
    ok = True
    rep = {"plain_hash": _hash(plain)}
    for mode in ("perfect", "corrupt", "garbage"):
        dec = SpecDecoder(m, [], max_drafts=cfg.draft_depth)
        out = [dec.begin(0, prompt)]
        while len(out) < ns.new_tokens:
            d = plain[len(out):len(out) + cfg.draft_depth]
            if mode == "corrupt" and len(d) > ns.corrupt:
                d = d[:ns.corrupt] + [(d[ns.corrupt] + 1) % m.cfg.vocab] + d[ns.corrupt + 1:]
            if mode == "garbage":
                d = [(t + 7) % m.cfg.vocab for t in d]
            out += dec.step([0], forced_drafts={0: d})[0]
        dec.end(0)
        rep[mode] = {"equal": out[:ns.new_tokens] == plain, "tokens_per_step": round(dec.stats.tokens_per_step(), 2)}
        ok &= rep[mode]["equal"]
    print(json.dumps(rep))
    return 0 if ok else 1


def cmd_batch(ns):
    """Batch gate: every row of a batch equals its single-sequence run (reference: m1-batch)."""
    from .serve.engine import Engine
    from .spec import SpecDecoder
    cfg = EngineConfig.resolve(ns)
    sizes = [int(x) for x in ns.batch.split(",")]
    m, rank, world, _ = build_model(cfg, max_seqs=max(sizes), max_ctx=max(cfg.wctx, ns.prompt_len + ns.new_tokens + 16))
    prompts = [_prompt(m.cfg, max(4, ns.prompt_len - 3 * i), cfg.seed + i) for i in range(max(sizes))]
    singles = [SpecDecoder(m, [], max_drafts=0).generate(0, p, ns.new_tokens) for p in prompts]
    ok, rep = True, {}
    for b in sizes:
        got = {}
        eng = Engine(m, lambda rid, t, f, e: got.setdefault(rid, []).extend(t) or False, max_batch=b)
        rids = [eng.submit(p, {"max_new_tokens": ns.new_tokens}) for p in prompts[:b]]
        eng.run_until_idle()
        rep[str(b)] = all(got[r] == s for r, s in zip(rids, singles))
        ok &= rep[str(b)]
    print(json.dumps({"batch_equals_single": rep}))
    return 0 if ok else 1


def cmd_spec_batch(ns):
    """Batched speculation gate (reference: m1-spec-batch, crates/agens-cli/src/spec.rs ``run_batch``): several
    sequences verify their draft blocks in one step; with perfect, corrupted and garbage drafts every sequence emits
    exactly its plain greedy tokens."""
    from .spec import SpecDecoder
    cfg = EngineConfig.resolve(ns)
    nb = max(2, int(ns.sequences))
    depth = max(1, min(cfg.draft_depth, 7))
    m, rank, world, _ = build_model(cfg, max_seqs=nb, max_ctx=max(cfg.wctx, ns.prompt_len + ns.new_tokens + 16))
    m.row_graphs = bool(cfg.row_graphs)
    prompts = [_prompt(m.cfg, max(4, ns.prompt_len - 5 * i), cfg.seed + i) for i in range(nb)]
    plain = [SpecDecoder(m, [], max_drafts=0).generate(0, p, ns.new_tokens) for p in prompts]
    ok, rep = True, {"plain_hash": _hash([t for p in plain for t in p])}
    for mode in ("perfect", "corrupt", "garbage"):
        dec = SpecDecoder(m, [], max_drafts=depth)
        outs = [[dec.begin(i, p)] for i, p in enumerate(prompts)]
        while any(len(o) < ns.new_tokens for o in outs):
            live = [i for i, o in enumerate(outs) if len(o) < ns.new_tokens]
            forced = {}
            for i in live:
                d = plain[i][len(outs[i]):len(outs[i]) + depth]
                if mode == "corrupt" and len(d) > ns.corrupt:
                    d = d[:ns.corrupt] + [(d[ns.corrupt] + 1) % m.cfg.vocab] + d[ns.corrupt + 1:]
                if mode == "garbage":
                    d = [(t + 7) % m.cfg.vocab for t in d]
                forced[i] = d
            for i, toks in dec.step(live, forced_drafts=forced).items():
                outs[i] += toks
        for i in range(nb):
            dec.end(i)
        same = all(o[:ns.new_tokens] == p for o, p in zip(outs, plain))
        rep[mode] = {"equal": same, "tokens_per_step": round(dec.stats.tokens_per_step(), 2)}
        ok &= same
    print(json.dumps(rep))
    return 0 if ok else 1


def cmd_agent_replay(ns):
    """Agent-session replay (reference: m2a-demo, crates/agens-cli/src/m1.rs:1417-1514).  ``transcripts`` is a JSON
    list of sessions, each a list of turns, each turn the full prompt ids of that turn (consecutive turns share a
    growing prefix).  Mode ``session`` keeps one resident sequence per transcript holding the prefix common to
    consecutive turns: a turn advances it by the new tokens only, forks it, prefills the rest of the turn's prompt on
    the fork, generates greedily and frees the fork; nothing is prefilled twice.  Mode ``reprefill`` prefills every
    turn from scratch.  Both write per turn the time to the first token and the generated tokens to ``out``; ``--check``
    runs both and reports how far their tokens agree."""
    import time
    import torch
    cfg = EngineConfig.resolve(ns)
    sessions = json.load(open(ns.transcripts))
    if ns.max_sessions:
        sessions = sessions[:ns.max_sessions]
    longest = max(len(t) for s_ in sessions for t in s_)
    m, rank, world, _ = build_model(cfg, max_seqs=2, max_ctx=max(cfg.wctx, longest + ns.new_tokens + 16))
    m.set_linear_path(1)          # one linear kernel family whatever the chunk size, so that both modes see the same numerics

    def generate(seq, first):
        out, tok = [first], first
        while len(out) < ns.new_tokens and tok != ns.eos:
            o, _ = m.forward_rows([tok], [seq]); tok = int(o[0]); out.append(tok)
        return out

    def run(mode):
        rows = []
        for si, turns in enumerate(sessions):
            if mode == "session":
                m.new_seq(0)
            kept: List[int] = []
            for ti, ids in enumerate(turns):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                if mode == "session":
                    nxt = turns[ti + 1] if ti + 1 < len(turns) else ids
                    keep = 0
                    while keep < min(len(ids), len(nxt)) and ids[keep] == nxt[keep]:
                        keep += 1
                    keep = max(len(kept), min(keep, len(ids) - 1))        # the resident prefix only grows; one token stays for the fork
                    common = 0
                    while common < min(len(kept), len(ids)) and kept[common] == ids[common]:
                        common += 1
                    if common < len(kept):                                  # the conversation was edited: drop what differs
                        m.truncate(0, common); kept = kept[:common]; keep = max(keep, common)
                    if keep > len(kept):
                        m.prefill(0, torch.tensor(ids[len(kept):keep], dtype=torch.int32)); kept = list(ids[:keep])
                    m.fork(0, 1)
                    first, _ = m.prefill(1, torch.tensor(ids[len(kept):], dtype=torch.int32))
                else:
                    m.new_seq(1)
                    first, _ = m.prefill(1, torch.tensor(ids, dtype=torch.int32))
                torch.cuda.synchronize()
                ttft = time.perf_counter() - t0
                toks = generate(1, first)
                m.free_seq(1)
                rows.append({"session": si, "turn": ti, "prompt_tokens": len(ids), "ttft_s": round(ttft, 4), "tokens": toks})
            if mode == "session":
                m.free_seq(0)
        return rows

    modes = ["session", "reprefill"] if ns.check else [ns.replay_mode]
    res = {md: run(md) for md in modes}
    json.dump(res, open(ns.out, "w"))
    rep = {md: {"turns": len(r), "mean_ttft_s": round(sum(x["ttft_s"] for x in r) / max(len(r), 1), 4)} for md, r in res.items()}
    ok = True
    if ns.check:
        a_, b_ = [x["tokens"] for x in res["session"]], [x["tokens"] for x in res["reprefill"]]
        # The two modes cut the prompt into different chunks, and chunks of different sizes take different kernels (their
        # sums run in different orders), so the comparison is an agreement rate, not bit equality: the first generated
        # token of every turn, and all positions up to the first difference of a turn.
        first = sum(int(x[0] == y[0]) for x, y in zip(a_, b_)) / max(len(a_), 1)
        same = sum(next((i for i, (p, q) in enumerate(zip(x, y)) if p != q), min(len(x), len(y))) for x, y in zip(a_, b_))
        rep["tokens_equal"] = a_ == b_
        rep["first_token_agreement"] = round(first, 3)
        rep["agreement_until_first_difference"] = round(same / max(sum(len(x) for x in a_), 1), 3)
        ok = first >= ns.min_agreement
    print(json.dumps(rep))
    return 0 if ok else 1


def cmd_session(ns):
    """Session gate: park -> clobber -> unpark restores exactly; a fork continues like its parent."""
    import torch
    cfg = EngineConfig.resolve(ns)
    m, rank, world, _ = build_model(cfg, max_seqs=3, max_ctx=max(cfg.wctx, ns.prompt_len + ns.new_tokens + 16))
    prompt = torch.tensor(_prompt(m.cfg, ns.prompt_len, cfg.seed))
    m.new_seq(0)
    first, _ = m.prefill(0, prompt)
    ref = []
    m.fork(0, 1)
    tok = first
    for _ in range(ns.new_tokens):
        out, _ = m.forward_rows([tok], [0]); tok = int(out[0]); ref.append(tok)
    blob = m.park(1)
    m.new_seq(2)
    m.prefill(2, torch.tensor(_prompt(m.cfg, ns.prompt_len, cfg.seed + 1)))      # clobber freed pages
    m.free_seq(2)
    m.unpark(2, blob)
    got, tok = [], first
    for _ in range(ns.new_tokens):
        out, _ = m.forward_rows([tok], [2]); tok = int(out[0]); got.append(tok)
    print(json.dumps({"fork_park_unpark_equal": got == ref, "hash": _hash(got)}))
    return 0 if got == ref else 1


def _finish(m, world):
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        m.close()
        dist.destroy_process_group()


def cmd_serve(ns):
    import torch
    from .serve.engine import Engine, attach_to_server
    from .serve.server import Server
    from .spec import CopyLookupSource, ModelSource, MtpSource
    cfg = EngineConfig.resolve(ns)
    children = []
    if cfg.tp > 1 and "RANK" not in os.environ:
        from .parallel import driver as D
        children = D.launch(["-m", "agens_engine_b200"] + sys.argv[1:], cfg.tp)   # the other ranks run the same command line
    import signal

    def _on_term(signum, frame):           # a plain kill still releases the followers and the peer mappings
        raise KeyboardInterrupt
    signal.signal(signal.SIGTERM, _on_term)
    if cfg.mode == "personal":
        cfg.max_batch = 1
    # slots beyond the running batch hold finished conversations and prompt-prefix snapshots
    m, rank, world, ctrl = build_model(cfg, max_seqs=max(cfg.max_batch, 1) + max(0, min(cfg.max_convs, 64)))
    if rank == 0:
        print("config: " + json.dumps(dataclasses.asdict(cfg)), flush=True)
    if world > 1 and rank > 0:
        from .parallel import driver as D
        D.follow(m, ctrl)
        _finish(m, world)
        return 0
    model = m
    if world > 1:
        from .parallel import driver as D
        model = D.TpDriver(m, ctrl, children=children)
    m.row_graphs = bool(cfg.row_graphs) and world == 1
    sources = []
    if cfg.spec_copy:
        sources.append(CopyLookupSource())
    if cfg.mtp:                                           # under --tp the head runs beside the leader, unsharded
        from .models.mtp import MtpHead
        if os.path.isdir(cfg.mtp):                        # a head checkpoint (mtp.* tensors); anything else: a random-init head
            from .utils import checkpoint as K
            head = K.load_mtp(cfg.mtp, m, lm_head_dir=cfg.model_dir)
        else:
            head = MtpHead.random_init_for(m)
        if cfg.mtp_vocab:                                 # the head's shortlist: the first N ids, or a file of little-endian uint32 ids
            if os.path.isfile(cfg.mtp_vocab):
                import numpy as np
                head.use_shortlist(np.fromfile(cfg.mtp_vocab, dtype="<u4").astype(np.int64).tolist())
            else:
                head.use_shortlist(range(min(int(cfg.mtp_vocab), head.cfg.vocab_valid or head.cfg.vocab)))
        sources.append(MtpSource(head, depth=min(cfg.draft_depth, 2)))
    if cfg.spec_drafter:                                  # under --tp the drafter lives beside the leader, unsharded
        from .models.dense import DenseModel
        dcfg = _named_config(cfg.spec_drafter) if not os.path.isdir(cfg.spec_drafter) else None
        if dcfg is None:
            from .utils import checkpoint as K
            drafter = K.load_model(cfg.spec_drafter, m.dev, max_seqs=m.max_seqs, max_ctx=m.max_ctx)
        else:
            drafter = DenseModel.random_init(dcfg, m.dev, seed=cfg.seed + 1, max_seqs=m.max_seqs, max_ctx=m.max_ctx)
        drafter.row_graphs = True
        sources.append(ModelSource(drafter, depth=cfg.draft_depth))
    tok_path = cfg.tokenizer or (os.path.join(cfg.model_dir, "tokenizer.json") if cfg.model_dir else None)
    if not tok_path or not os.path.exists(tok_path):
        raise SystemExit("serve needs a tokenizer.json (--tokenizer PATH or inside --model-dir)")
    gen_cfg = {}
    if cfg.model_dir and os.path.exists(os.path.join(cfg.model_dir, "generation_config.json")):
        gen_cfg = json.load(open(os.path.join(cfg.model_dir, "generation_config.json")))
    eos = gen_cfg.get("eos_token_id", [])
    # the checkpoint's own chat template, when it ships one (else the built-in ChatML renderer)
    tcfg_path = os.path.join(os.path.dirname(tok_path), "tokenizer_config.json")
    tcfg = json.load(open(tcfg_path)) if os.path.exists(tcfg_path) else {}
    special = lambda v: v.get("content", "") if isinstance(v, dict) else (v or "")
    template = tcfg.get("chat_template") or ""
    if isinstance(template, list):                       # named templates: take the default one
        template = next((t.get("template", "") for t in template if t.get("name") == "default"), "")
    srv = Server(tok_path, model_name=cfg.served_model_name, generation_config=gen_cfg,
                 eos_token_ids=eos if isinstance(eos, list) else [eos], max_tokens_default=cfg.max_tokens_default,
                 chat_template=template, bos_token=special(tcfg.get("bos_token")), eos_token=special(tcfg.get("eos_token")))
    # ids the tokenizer does not know (padding rows of the embedding) are never produced
    tj = json.load(open(tok_path))
    n_tok = 1 + max([max(tj["model"]["vocab"].values(), default=0)] + [int(t["id"]) for t in tj.get("added_tokens", [])])
    full = m.full_cfg if world > 1 else m.cfg
    full.vocab_valid = min(full.vocab_valid or full.vocab, n_tok)
    front = None
    if cfg.vision:                                        # under --tp the tower runs on the leader; the driver hands the
        # encoder rows and position tables to the followers with the prefill call (every rank substitutes the same rows)
        # image input: the checkpoint's own tower (model.visual.* tensors) when it has one, else random-init weights of
        # the reference tower's shape; the placeholder id comes from the tokenizer's added tokens
        from .models.vision import VisionConfig, VisionTower
        from .serve.vision import VisionFrontEnd
        pad = [int(t["id"]) for t in tj.get("added_tokens", []) if t.get("content") == "<|image_pad|>"]
        if not pad:
            raise SystemExit("--vision 1 needs an <|image_pad|> token in the tokenizer")
        vc = VisionConfig(out_dim=full.d_model) if full.d_model >= 2048 else \
            VisionConfig(depth=2, d_model=288, n_heads=4, mlp=608, out_dim=full.d_model, pos_grid=12)
        if cfg.model_dir and VisionTower.has_tower(cfg.model_dir):
            tower = VisionTower.from_checkpoint(cfg.model_dir, m.dev)
            if tower.cfg.out_dim != full.d_model:
                raise SystemExit(f"the checkpoint's vision tower feeds {tower.cfg.out_dim}-wide rows into a {full.d_model}-wide model")
        else:
            tower = VisionTower.random_init(vc, m.dev, seed=cfg.seed + 2)
        front = VisionFrontEnd(tower, pad[0], full.head_dim)
    eng = Engine(model, lambda *a: False, sources_factory=(lambda: sources) if sources else None,
                 max_drafts=cfg.draft_depth if sources else 0, max_batch=cfg.max_batch, keep_sequences=world == 1, vision=front)
    attach_to_server(eng, srv, context_length=m.max_ctx)
    eng.start()
    port = srv.start(cfg.host, cfg.port)
    print(f"serving {cfg.served_model_name} on http://{cfg.host}:{port} (tp {world}, max batch {eng.max_batch})", flush=True)
    rc = 0

    def _terminate(signum, frame):           # `docker stop` sends SIGTERM: leave through the same path as Ctrl-C
        raise KeyboardInterrupt
    try:
        import signal
        signal.signal(signal.SIGTERM, _terminate)
    except ValueError:                       # not the main thread (embedded use): the caller owns signal handling
        pass
    try:
        while eng.fatal is None:
            time.sleep(0.5)
        print(f"serve: {eng.fatal}", flush=True)
        rc = 3                           # a follower is gone: same exit code as the reference's leader
    except KeyboardInterrupt:
        pass
    finally:
        srv.stop()
        eng.stop()
        if world > 1:
            model.shutdown()
            _finish(m, world)
        for c in children:                 # the ranks this process started: wait, then stop exactly those processes
            try:
                c.wait(timeout=20)
            except Exception:
                c.terminate()
    return rc


# ---------------------------------------------------------------------------------------------------------------------
def _engine_flags(p):
    p.add_argument("--model-dir"); p.add_argument("--random"); p.add_argument("--seed", type=int)
    p.add_argument("--tp", type=int); p.add_argument("--device", type=int); p.add_argument("--budget-gib", type=float)
    p.add_argument("--wctx", type=int); p.add_argument("--max-batch", type=int); p.add_argument("--max-convs", type=int)
    p.add_argument("--mode", choices=["personal", "server"]); p.add_argument("--prefill-chunk", type=int)
    p.add_argument("--profile"); p.add_argument("--draft-depth", type=int); p.add_argument("--row-graphs", type=int)
    p.add_argument("--prompt-len", type=int, default=64); p.add_argument("--new-tokens", type=int, default=32)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="agens_engine_b200", description=__doc__.split("\n\n")[0])
    ap.add_argument("--version", action="version", version=VERSION)
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name, fn in (("inspect", cmd_inspect), ("validate", cmd_validate), ("verify", cmd_verify)):
        p = sub.add_parser(name); p.add_argument("dir"); p.add_argument("--threads", type=int, default=8); p.set_defaults(fn=fn)
    sub.add_parser("devices").set_defaults(fn=cmd_devices)
    p = sub.add_parser("plan"); _engine_flags(p); p.add_argument("--gpu-free-gib", type=float, default=170.0)
    p.add_argument("--host-avail-gib", type=float, default=-1.0); p.add_argument("--plan-prefill-chunk", type=int, default=8192)
    p.set_defaults(fn=cmd_plan)
    p = sub.add_parser("profile"); p.add_argument("name"); p.add_argument("--tp", type=int); p.set_defaults(fn=cmd_profile)
    for name, fn in (("load", cmd_load), ("run", cmd_run), ("session", cmd_session)):
        p = sub.add_parser(name); _engine_flags(p); p.set_defaults(fn=fn)
    p = sub.add_parser("kv"); _engine_flags(p); p.add_argument("--save-logits"); p.add_argument("--cmp-logits"); p.set_defaults(fn=cmd_kv)
    p = sub.add_parser("spec"); _engine_flags(p); p.add_argument("--corrupt", type=int, default=2); p.set_defaults(fn=cmd_spec)
    p = sub.add_parser("batch"); _engine_flags(p); p.add_argument("--batch", default="2,4,8"); p.set_defaults(fn=cmd_batch)
    p = sub.add_parser("spec-batch"); _engine_flags(p); p.add_argument("--corrupt", type=int, default=2)
    p.add_argument("--sequences", type=int, default=4); p.set_defaults(fn=cmd_spec_batch)
    p = sub.add_parser("agent-replay"); _engine_flags(p); p.add_argument("transcripts"); p.add_argument("out")
    p.add_argument("--replay-mode", choices=["session", "reprefill"], default="session"); p.add_argument("--check", action="store_true")
    p.add_argument("--max-sessions", type=int, default=0); p.add_argument("--eos", type=int, default=-1)
    p.add_argument("--min-agreement", type=float, default=0.75); p.set_defaults(fn=cmd_agent_replay)
    p = sub.add_parser("serve"); _engine_flags(p)
    p.add_argument("--host"); p.add_argument("--port", type=int); p.add_argument("--served-model-name")
    p.add_argument("--spec-copy", type=int); p.add_argument("--spec-drafter"); p.add_argument("--mtp"); p.add_argument("--mtp-vocab")
    p.add_argument("--max-tokens-default", type=int); p.add_argument("--think-guard"); p.add_argument("--tokenizer")
    p.add_argument("--vision", type=int)
    p.set_defaults(fn=cmd_serve)
    ns = ap.parse_args(argv)
    return int(ns.fn(ns) or 0)


if __name__ == "__main__":
    sys.exit(main())
