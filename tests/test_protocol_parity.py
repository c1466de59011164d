"""Replays the reference's protocol parity corpus against the C++ server's parsers, when a checkout of the reference's
fixtures is available: B200E_REF_FIXTURES names its ``crates/agens-server/tests/fixtures`` directory, or the checkout
sits next to this repository as ``../reference`` (the tests are skipped otherwise).  The corpus holds raw model outputs (real generations, re-rendered agent transcripts, synthetic edge
cases) with the reasoning / content / tool-call split its parsers produce (reference test:
crates/agens-server/tests/parser_parity.rs).  Compared here, non-streaming and streamed in 7-byte chunks: the reasoning
text, the content outside calls, and every call's name and arguments."""
import ctypes as C
import json
import os

import pytest

from agens_engine_b200.serve import host as H

def _fixtures_dir() -> str:
    """B200E_REF_FIXTURES, else a checkout of the reference next to this repository (``../reference``) if there is one."""
    env = os.environ.get("B200E_REF_FIXTURES", "")
    if env:
        return env
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    guess = os.path.join(os.path.dirname(here), "reference", "crates", "agens-server", "tests", "fixtures")
    return guess if os.path.isfile(os.path.join(guess, "parser_corpus.json")) else ""


FIX = _fixtures_dir()
pytestmark = pytest.mark.skipif(not os.path.isfile(os.path.join(FIX, "parser_corpus.json")),
                                reason="the reference's fixtures are not available (B200E_REF_FIXTURES)")
TAGS = (b"<|think|>", b"<|/think|>", b"<|call|>", b"<|/call|>")


def _parse(text, tools, starts_in_reasoning, chunk):
    lib = H.lib()
    fn = lib.b2h_parse_output_tags
    fn.restype = C.c_void_p
    fn.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.c_int, C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p]
    p = fn(text.encode(), json.dumps(tools).encode(), 1 if starts_in_reasoning else 0, chunk, *TAGS)
    out = json.loads(C.string_at(p).decode())
    lib.b2h_free_str(C.c_void_p(p))
    return out


def _norm_calls(calls):
    return [(c["name"], json.loads(c.get("parameters", c.get("arguments", "{}")) or "{}")) for c in (calls or [])]


def test_parser_corpus_replay():
    corpus = json.load(open(os.path.join(FIX, "parser_corpus.json")))
    sets = corpus["tool_sets"]
    total = same = 0
    diffs = []
    for case in corpus["cases"]:
        tools = sets[case["tools"]] if case.get("tools") else None
        for mode in case["modes"]:
            want = mode["nonstream"]
            if tools and want.get("calls") is None:
                continue                          # tool_choice "none": the request layer skips the call parser
            for chunk in (0, 7):
                got = _parse(case["text"], tools, mode["force_reasoning"], chunk)
                content_want = want["tool_normal"] if want.get("calls") is not None else want["normal"]
                ok = (got["reasoning"].strip() == want["reasoning"].strip()
                      and got["content"].strip() == (content_want or "").strip()
                      and _norm_calls(got["tool_calls"]) == _norm_calls(want.get("calls")))
                total += 1
                same += int(ok)
                if not ok and len(diffs) < 8:
                    diffs.append((case["name"], mode["force_reasoning"], chunk))
    rate = same / max(total, 1)
    print(f"parser corpus: {same} of {total} checks agree ({rate:.1%}); first differences: {diffs}")
    assert rate >= float(os.environ.get("B200E_PARITY_MIN", "0.9")), diffs


def test_template_cases_replay():
    """The reference's chat template (fixtures/model/chat_template.jinja) rendered by the C++ Jinja interpreter on the
    51 cases of its template parity test (crates/agens-server/tests/template_parity.rs): every expected prompt must
    come out byte for byte, and the cases that expect a template error must raise one."""
    from agens_engine_b200.serve import server as S
    path = os.path.join(FIX, "template_cases.json")
    tpl_path = os.path.join(FIX, "model", "chat_template.jinja")
    if not (os.path.isfile(path) and os.path.isfile(tpl_path)):
        pytest.skip("template fixtures not present")
    tpl = open(tpl_path).read()
    cases = json.load(open(path))["cases"]
    bad = []
    for x in cases:
        ctx = {"messages": x["messages"], "add_generation_prompt": True}
        if x.get("tools") is not None:
            ctx["tools"] = x["tools"]
        ctx.update(x.get("kwargs") or {})
        try:
            out, err = S.render_template(tpl, **ctx), None
        except Exception as e:          # a template that calls raise_exception
            out, err = None, str(e)
        ok = (err is not None) if x.get("error") is not None else (out == x["expected"])
        if not ok:
            bad.append(x["name"])
    print(f"template cases: {len(cases) - len(bad)} of {len(cases)} agree; differences: {bad}")
    assert not bad, bad


def test_request_cases_replay(tmp_path):
    """The reference's request corpus (fixtures/request_cases.json, test crates/agens-server/tests/request_parity.rs):
    chat-completion bodies with the prompt text and the sampling parameters the engine must receive, or the 400 error
    the request must get.  Each body goes through the C++ server's chat handler with the reference's template and
    generation_config and a byte-level tokenizer that carries the template's marker tokens; the mock engine records
    the prompt ids and the sampling record.  Prompts are compared byte for byte.  Sampling fields are compared with
    four representation differences allowed: no token cap (null) is this server's default cap, an absent
    stop-token list is an empty one, the end-of-sequence ids of generation_config travel inside the stop-token list, and
    greedy is recorded as top_k 1 rather than temperature 0."""
    from agens_engine_b200.serve import server as S
    from tests import fixtures as F
    path = os.path.join(FIX, "request_cases.json")
    tpl_path = os.path.join(FIX, "model", "chat_template.jinja")
    gen_path = os.path.join(FIX, "model", "generation_config.json")
    if not all(os.path.isfile(p) for p in (path, tpl_path, gen_path)):
        pytest.skip("request fixtures not present")
    tj = json.loads(F.tiny_tokenizer_json())
    nid = max(a["id"] for a in tj["added_tokens"]) + 1
    for s in ("<|agens_start|>", "<|agens_end|>", "<|think|>", "<|/think|>", "<|call|>", "<|/call|>"):
        tj["added_tokens"].append({"id": nid, "content": s, "single_word": False, "lstrip": False, "rstrip": False,
                                   "normalized": False, "special": True})
        nid += 1
    tok_json = json.dumps(tj)
    tok_path = tmp_path / "tokenizer.json"
    tok_path.write_text(tok_json)
    srv = S.Server(str(tok_path), model_name="volundr", generation_config=json.load(open(gen_path)),
                   chat_template=open(tpl_path).read())
    srv.use_mock([65, 66], step=1, supports_images=True)
    tk = S.Tokenizer(tok_json)
    eos = json.load(open(gen_path)).get("eos_token_id", [])
    eos = eos if isinstance(eos, list) else [eos]
    keys = ("temperature", "top_p", "top_k", "min_p", "max_new_tokens", "presence_penalty", "frequency_penalty",
            "repetition_penalty", "min_new_tokens", "ignore_eos", "stop_token_ids")
    cases = json.load(open(path))["cases"]
    bad = []
    for x in cases:
        n0 = len(srv.mock_calls())
        status, body = srv.handle("POST", "/v1/chat/completions", x["body"])
        calls = srv.mock_calls()
        if "error" in x:
            if not (status == 400 and x["error"] in body):
                bad.append((x["name"], "error", status))
            continue
        if len(calls) == n0:
            bad.append((x["name"], "no engine call", status))
            continue
        c = calls[-1]
        if tk.decode(c["prompt"], skip_special=False) != x["prompt"]:
            bad.append((x["name"], "prompt"))
        want, got = dict(x["sampling"]), dict(c["sampling"])
        if want.get("max_new_tokens") is None:
            want.pop("max_new_tokens", None), got.pop("max_new_tokens", None)
        if want.get("stop_token_ids") is None:
            want["stop_token_ids"] = []
        got["stop_token_ids"] = [t for t in got.get("stop_token_ids", []) if t not in eos or t in want["stop_token_ids"]]
        if want.get("temperature") == 0.0 and got.get("top_k") == 1:
            for d in (want, got):
                d.pop("temperature", None), d.pop("top_k", None)
        diff = {k: (want.get(k), got.get(k)) for k in keys if want.get(k) != got.get(k)}
        if diff:
            bad.append((x["name"], "sampling", diff))
    print(f"request cases: {len(cases) - len({b[0] for b in bad})} of {len(cases)} agree; differences: {bad}")
    assert not bad, bad


# ---- end-to-end cases: recorded token ids through the HTTP layer ------------------------------------------------------
# The reference's e2e cases carry token ids of its own 248K-entry tokenizer, which is not part of its test files.  The
# replay builds a stand-in tokenizer that decodes exactly the ids the cases use: the first 256 ids are the byte tokens
# (byte-level BPE order), the markers keep their ids, and every other id gets the text the case's recorded per-step
# output shows for it.  Prompt token counts therefore differ and are left out of the comparison; everything else
# (bodies and event streams) is compared byte for byte.
def _byte_alphabet():
    bs = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b); cs.append(256 + n); n += 1
    return bs, {b: chr(c) for b, c in zip(bs, cs)}


def _stand_in_tokenizer(cases, completion_cases, tok_cases):
    from tests import fixtures as F
    bs, b2u = _byte_alphabet()
    piece = {i: bytes([b]) for i, b in enumerate(bs)}
    marker, special = {}, set()
    for c in tok_cases["decode"]:
        if len(c["ids"]) == 1 and c["skip"] == "" and c["keep"]:
            marker[c["ids"][0]] = c["keep"]; special.add(c["ids"][0])
    for t in special:
        piece[t] = b""
    # where the recorded outputs do not align one to one with the ids (a stop string cuts inside a token) the pieces
    # follow from the case's text
    piece.update({44020: b" STOP", 3786: b".</", 8944: b"answer", 1021: b"line", 357: b" A", 13962: b"###", 6918: b"alpha"})

    def give_prev(ids, i, rest):                     # the token before carried the first bytes of this character
        if i > 0 and ids[i - 1] >= 256 and ids[i - 1] not in special and not piece.get(ids[i - 1], b"").endswith(rest):
            piece[ids[i - 1]] = piece.get(ids[i - 1], b"") + rest

    def learn(ids, deltas):
        i = 0
        while i < len(deltas):
            j = i
            while j < len(deltas) and deltas[j] == "":
                j += 1
            if j >= len(deltas):
                break
            run, text = ids[i:j + 1], deltas[j].encode()
            if len(run) == 1:
                t = run[0]
                if t in marker:
                    pass
                elif deltas[j].startswith("<|") and deltas[j].endswith("|>"):
                    marker[t] = deltas[j]
                elif t in piece and piece[t] != text and text.endswith(piece[t]):
                    give_prev(ids, i, text[:len(text) - len(piece[t])])
                else:
                    piece.setdefault(t, text)
            else:
                lo, hi, rest = 0, len(run), text
                while lo < hi and run[lo] in piece and rest.startswith(piece[run[lo]]):
                    rest = rest[len(piece[run[lo]]):]; lo += 1
                while hi > lo and run[hi - 1] in piece and rest.endswith(piece[run[hi - 1]]):
                    rest = rest[:len(rest) - len(piece[run[hi - 1]])]; hi -= 1
                unk = run[lo:hi]
                if not unk and rest:
                    give_prev(ids, i, rest)
                for k, t in enumerate(unk):
                    if k == len(unk) - 1:
                        piece[t] = rest; rest = b""
                    else:
                        n = 1
                        while n < len(rest) and rest[n - 1] < 0x80:
                            n += 1
                        piece[t] = rest[:n]; rest = rest[n:]
            i = j + 1

    for c in cases:
        if (c.get("step") or 1) == 1 and "deltas" in c and len(c["deltas"]) == len(c["output_ids"]):
            learn(c["output_ids"], c["deltas"])
    for c in cases:
        if (c.get("step") or 1) == 1 and "deltas" in c and len(c["deltas"]) < len(c["output_ids"]) and "max_tokens" in c["body"]:
            learn(c["output_ids"][:len(c["deltas"])], c["deltas"])
    for c in completion_cases:
        texts = [json.loads(e[6:])["choices"][0]["text"] for e in c["sse"] if e.startswith("data: {") and json.loads(e[6:])["choices"]]
        for t, x in zip(c["output_ids"], texts):
            if x and t >= 256 and t not in piece:
                piece[t] = x.encode()
    tj = json.loads(F.tiny_tokenizer_json())
    vocab = {b2u[b]: i for i, b in enumerate(bs)}
    for t, bts in sorted(piece.items()):
        st = "".join(b2u[b] for b in bts)
        if t >= 256 and t not in special and st not in vocab:
            vocab[st] = t
    tj["model"]["vocab"], tj["model"]["merges"] = vocab, []
    tj["added_tokens"] = [{"id": i, "content": c, "single_word": False, "lstrip": False, "rstrip": False, "normalized": False,
                           "special": i in special} for i, c in sorted(marker.items())]
    return json.dumps(tj)


def _norm_wire(s):
    import re
    s = re.sub(r'"created":\d+', '"created":0', s)
    s = re.sub(r'"id":"call_[0-9a-f]{24}', '"id":"call_X', s)
    return re.sub(r'"(prompt_tokens|total_tokens)":\d+', r'"\1":N', s)


def _events(body):
    import re
    return [_norm_wire(x) for x in re.findall(r'.*?\n\n', body, flags=re.S)]


def test_e2e_cases_replay(tmp_path):
    """The reference's end-to-end corpus (fixtures/e2e_cases.json and completion_cases.json, test
    crates/agens-server/tests/e2e_parity.rs): a mock engine replays recorded token ids, one to seven per step, and the
    complete response body and the event stream of every case are compared with what the reference's serving code
    produced: ids, field order, null fields, finish reasons and matched stops, usage with reasoning tokens, reasoning /
    content / tool-call deltas (call header, then the arguments parameter by parameter), stop strings and stop ids,
    error bodies.  One known difference in event boundaries: a lone "<" at the end of a reasoning piece is held until
    the next piece arrives (the parsers here accept markers cut anywhere; the reference expects them in one piece)."""
    from agens_engine_b200.serve import server as S
    need = ["e2e_cases.json", "completion_cases.json", "tokenizer_cases.json", "model/chat_template.jinja", "model/generation_config.json"]
    if not all(os.path.isfile(os.path.join(FIX, n)) for n in need):
        pytest.skip("e2e fixtures not present")
    d = json.load(open(os.path.join(FIX, "e2e_cases.json")))
    cases, tool_sets = d["cases"], d["tool_sets"]
    comp = json.load(open(os.path.join(FIX, "completion_cases.json")))["cases"]
    tok_json = _stand_in_tokenizer(cases, comp, json.load(open(os.path.join(FIX, "tokenizer_cases.json"))))
    tok_path = tmp_path / "tokenizer.json"
    tok_path.write_text(tok_json)
    tpl = open(os.path.join(FIX, "model", "chat_template.jinja")).read()
    gen = json.load(open(os.path.join(FIX, "model", "generation_config.json")))

    def post(path, body, ids, step, stream):
        srv = S.Server(str(tok_path), model_name="volundr", generation_config=gen, chat_template=tpl)
        srv.use_mock(ids, step=step)
        return srv.handle("POST", path, dict(body, stream=stream))

    bad_ns, bad_st = [], []
    for c in cases:
        body = dict(c["body"], rid="RID")
        if c.get("tools"):
            body["tools"] = tool_sets[c["tools"]]
        ids, step = c["output_ids"], c.get("step") or 1
        if c.get("error"):
            e = c["error"]
            for stream in (False, True):
                st, got = post("/v1/chat/completions", body, ids, step, stream)
                if not (st == e["status"] and (e.get("body") is None or e["body"] == got)):
                    (bad_st if stream else bad_ns).append(c["name"])
            continue
        st, got = post("/v1/chat/completions", body, ids, step, False)
        if not (st == 200 and _norm_wire(got) == _norm_wire(c["nonstream"]["body"])):
            bad_ns.append(c["name"])
        st, got = post("/v1/chat/completions", body, ids, step, True)
        if not (st == 200 and _events(got) == [_norm_wire(x) for x in c["sse"]]):
            bad_st.append(c["name"])
    for c in comp:
        body = dict(c["body"], rid="RID")
        st, got = post("/v1/completions", body, c["output_ids"], 1, False)
        if not (st == 200 and _norm_wire(got) == _norm_wire(c["nonstream"])):
            bad_ns.append("completion/" + c["name"])
        st, got = post("/v1/completions", body, c["output_ids"], 1, True)
        if not (st == 200 and _events(got) == [_norm_wire(x) for x in c["sse"]]):
            bad_st.append("completion/" + c["name"])
    n = len(cases) + len(comp)
    print(f"e2e cases: complete responses {n - len(bad_ns)} of {n}, event streams {n - len(bad_st)} of {n}; differences: {bad_ns} {bad_st}")
    assert not bad_ns, bad_ns
    assert set(bad_st) <= {"syn/lt_in_text_and_value"}, bad_st
