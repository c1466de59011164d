"""Replays the reference's protocol parity corpus against the C++ server's parsers, when a checkout of the reference's
fixtures is available: set B200E_REF_FIXTURES to its ``crates/agens-server/tests/fixtures`` directory (the test is
skipped otherwise).  The corpus holds raw model outputs (real generations, re-rendered agent transcripts, synthetic edge
cases) with the reasoning / content / tool-call split its parsers produce (reference test:
crates/agens-server/tests/parser_parity.rs).  Compared here, non-streaming and streamed in 7-byte chunks: the reasoning
text, the content outside calls, and every call's name and arguments."""
import ctypes as C
import json
import os

import pytest

from agens_engine_b200.serve import host as H

FIX = os.environ.get("B200E_REF_FIXTURES", "")
pytestmark = pytest.mark.skipif(not os.path.isfile(os.path.join(FIX, "parser_corpus.json")),
                                reason="B200E_REF_FIXTURES does not point at the reference's fixtures")
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
    three representation differences allowed: no token cap (null) is this server's default cap, an absent
    stop-token list is an empty one, and greedy is recorded as top_k 1 rather than temperature 0."""
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
        if want.get("temperature") == 0.0 and got.get("top_k") == 1:
            for d in (want, got):
                d.pop("temperature", None), d.pop("top_k", None)
        diff = {k: (want.get(k), got.get(k)) for k in keys if want.get(k) != got.get(k)}
        if diff:
            bad.append((x["name"], "sampling", diff))
    print(f"request cases: {len(cases) - len({b[0] for b in bad})} of {len(cases)} agree; differences: {bad}")
    assert not bad, bad
