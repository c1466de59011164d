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
