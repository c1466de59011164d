"""CPU tests of the server stack with the mock backend (model: crates/agens-server/tests: tokenizer / template /
parser / request / e2e parity suites and server_basics.rs)."""
import json
import socket
import threading

import pytest

from agens_engine_b200.serve import server as S
from tests.fixtures import tiny_tokenizer_json

SAMPLES = ["hello world", "the thing and the other thing", "Hello,  world!\n\nNew   paragraph's text isn't  here ",
           "x=12*345;\n\ty = 'it''s'", "naïve café — ünïcödé 漢字かな 한국어", "tabs\t\tand\r\nCRLF  \n  trailing   ", "   lead",
           "emoji 🙂 ok", "a" * 50 + " " * 7 + "b", "<|im_start|>user\nhi<|im_end|>\n<think>x</think>", "12 1234 12th"]


@pytest.fixture(scope="module")
def tok_text():
    return tiny_tokenizer_json()


@pytest.fixture(scope="module")
def tok_path(tmp_path_factory, tok_text):
    p = tmp_path_factory.mktemp("tok") / "tokenizer.json"
    p.write_text(tok_text)
    return str(p)


def test_tokenizer_matches_hf_tokenizers(tok_text):
    tokenizers = pytest.importorskip("tokenizers")
    ref = tokenizers.Tokenizer.from_str(tok_text)
    mine = S.Tokenizer(tok_text)
    for s in SAMPLES:
        want = ref.encode(s, add_special_tokens=False).ids
        assert mine.encode(s) == want, s
        assert mine.decode(want, skip_special=False) == s
    ids = mine.encode("<|im_start|>the<|im_end|>")
    assert mine.decode(ids, skip_special=True) == "the"


def test_stream_detok_never_splits_utf8(tok_text):
    mine = S.Tokenizer(tok_text)
    s = "漢字 🙂 ünï"
    ids = mine.encode(s)
    parts = mine.stream_decode(ids, step=1)
    assert "".join(parts) == s
    for p in parts:
        p.encode("utf-8").decode("utf-8")          # every piece is valid on its own
    cut = mine.stream_decode(ids[:2], step=1)       # ends inside a multi-byte character
    assert cut[-1] == "�"


def test_chat_template():
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}]
    t = S.render_chat(msgs)
    assert t == "<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    assert S.render_chat(msgs, enable_thinking=False).endswith("<|im_start|>assistant\n<think>\n\n</think>\n\n")
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object", "properties": {"x": {"type": "integer"}}}}}]
    tt = S.render_chat(msgs, tools=tools)
    assert "# Tools" in tt and '"name": "f"' in tt and tt.index("be brief") < tt.index("# Tools")
    conv = msgs + [{"role": "assistant", "content": "", "tool_calls": [{"function": {"name": "f", "arguments": "{\"x\": 1}"}}]},
                   {"role": "tool", "content": "42"}]
    tc = S.render_chat(conv, tools=tools)
    assert '<tool_call>\n{"name": "f", "arguments": {"x": 1}}\n</tool_call><|im_end|>' in tc
    assert "<|im_start|>user\n<tool_response>\n42\n</tool_response><|im_end|>" in tc
    cont = S.render_chat(msgs + [{"role": "assistant", "content": "par"}], add_generation_prompt=False, continue_final=True)
    assert cont.endswith("<|im_start|>assistant\npar")


@pytest.mark.parametrize("chunk", [0, 1, 3, 7])
def test_reasoning_and_tool_parsers(chunk):
    tools = [{"type": "function", "function": {"name": "get", "parameters": {"type": "object", "properties": {
        "n": {"type": "integer"}, "q": {"type": "string"}, "flag": {"type": "boolean"}}}}}]
    text = '<think>\nlet me see\n</think>\n\nAnswer first.\n<tool_call>\n{"name": "get", "arguments": {"n": 3, "q": "a b"}}\n</tool_call>'
    r = S.parse_output(text, tools, chunk=chunk)
    assert r["reasoning"].strip() == "let me see" and r["content"].strip() == "Answer first."
    assert r["tool_calls"] == [{"name": "get", "arguments": '{"n": 3, "q": "a b"}'}]
    xml = "ok<function=get>\n<parameter=n>\n5\n</parameter>\n<parameter=q>\nhello\n</parameter>\n<parameter=flag>\ntrue\n</parameter>\n</function>"
    r2 = S.parse_output(xml, tools, chunk=chunk)
    assert r2["content"] == "ok" and json.loads(r2["tool_calls"][0]["arguments"]) == {"n": 5, "q": "hello", "flag": True}
    r3 = S.parse_output("still thinking", starts_in_reasoning=True, chunk=chunk)
    assert r3 == {"content": "", "reasoning": "still thinking", "tool_calls": []}
    r4 = S.parse_output("a < b and <thin air", chunk=chunk)
    assert r4["content"] == "a < b and <thin air" and r4["reasoning"] == ""


def _server(tok_path, tok_text, script_text, step=2, **kw):
    tk = S.Tokenizer(tok_text)
    sv = S.Server(tok_path, model_name="m", generation_config={"temperature": 1.0, "top_k": 20, "top_p": 0.95},
                  eos_token_ids=[tk.encode("<|im_end|>")[0]], **kw)
    sv.use_mock(tk.encode(script_text), step=step)
    return sv, tk


def test_chat_completion_non_stream_defaults_and_usage(tok_path, tok_text):
    sv, tk = _server(tok_path, tok_text, "<think>hm</think>\n\nhello world<|im_end|>ignored")
    st, body = sv.handle("POST", "/v1/chat/completions", {"model": "m", "messages": [{"role": "user", "content": "hi"}]}, session_id="abc")
    assert st == 200, body
    r = json.loads(body)
    msg = r["choices"][0]["message"]
    assert msg["content"] == "hello world" and msg["reasoning_content"] == "hm" and r["choices"][0]["finish_reason"] == "stop"
    assert r["usage"]["prompt_tokens"] == len(tk.encode(S.render_chat([{"role": "user", "content": "hi"}])))
    assert r["usage"]["completion_tokens"] == len(tk.encode("<think>hm</think>\n\nhello world")) + 1
    assert r["usage"]["reasoning_tokens"] == len(tk.encode("<think>hm")) + len(tk.encode("</think>"))
    call = sv.mock_calls()[0]
    assert call["session_id"] == "abc"                                 # header wins / is forwarded
    s = call["sampling"]
    assert s["temperature"] == 1.0 and s["top_k"] == 20 and s["top_p"] == 0.95 and s["max_new_tokens"] == 32768
    st, body = sv.handle("POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "temperature": 0})
    assert sv.mock_calls()[-1]["sampling"]["top_k"] == 1              # greedy is top_k = 1


def test_streaming_sse_stop_string_and_max_tokens(tok_path, tok_text):
    sv, tk = _server(tok_path, tok_text, "the thing and the other thing", step=3)
    st, body = sv.handle("POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "stream": True,
                                                           "stop": ["other"], "stream_options": {"include_usage": True}})
    events = [json.loads(l[6:]) for l in body.split("\n\n") if l.startswith("data: {")]
    assert body.endswith("data: [DONE]\n\n") and events[0]["choices"][0]["delta"]["role"] == "assistant"
    text = "".join(e["choices"][0]["delta"].get("content", "") for e in events if e["choices"])
    assert text == "the thing and the "
    assert [e for e in events if e["choices"]][-1]["choices"][0]["finish_reason"] == "stop"
    assert events[-1]["usage"]["completion_tokens"] > 0 and events[-1]["choices"] == []
    st, body = sv.handle("POST", "/v1/completions", {"prompt": "the", "max_tokens": 2})
    r = json.loads(body)
    assert r["choices"][0]["finish_reason"] == "length" and r["usage"]["completion_tokens"] == 2
    assert r["choices"][0]["text"] == tk.decode(tk.encode("the thing and the other thing")[:2])
    st, body = sv.handle("POST", "/v1/completions", {"prompt": [1, 2, 3], "max_tokens": 1})
    assert st == 200 and sv.mock_calls()[-1]["prompt"] == [1, 2, 3]


def test_tool_call_response(tok_path, tok_text):
    sv, _ = _server(tok_path, tok_text, '<tool_call>\n{"name": "f", "arguments": {"x": 1}}\n</tool_call><|im_end|>')
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object", "properties": {"x": {"type": "integer"}}}}}]
    st, body = sv.handle("POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "tools": tools})
    r = json.loads(body)["choices"][0]
    assert r["finish_reason"] == "tool_calls" and r["message"]["content"] == "" and r["matched_stop"] is None
    tc = r["message"]["tool_calls"][0]
    assert tc["function"] == {"name": "f", "arguments": '{"x": 1}'} and tc["id"].startswith("call_") and len(tc["id"]) == 29


def test_validation_errors_and_routes(tok_path, tok_text):
    sv, _ = _server(tok_path, tok_text, "hello")
    bad = [({"messages": []}, "non-empty"), ({"messages": [{"role": "user", "content": "x"}], "n": 2}, "n > 1"),
           ({"messages": [{"role": "user", "content": "x"}], "response_format": {"type": "json_object"}}, "response_format"),
           ({"messages": [{"role": "user", "content": "x"}], "logprobs": True}, "logprobs"),
           ({"messages": [{"role": "user", "content": "x"}], "temperature": -1}, "temperature"),
           ({"messages": [{"role": "user", "content": "x"}], "top_p": 0}, "top_p"),
           ({"messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "data:image/png;base64,AA"}}]}]}, "images")]
    for body, frag in bad:
        st, text = sv.handle("POST", "/v1/chat/completions", body)
        assert st == 400 and frag in json.loads(text)["message"], (body, text)
    assert sv.handle("POST", "/v1/completions", {"prompt": ["a", "b"]})[0] == 400
    assert sv.handle("POST", "/v1/completions", {"prompt": "a", "echo": True})[0] == 400
    assert sv.handle("GET", "/health")[0] == 200 and sv.handle("GET", "/health_generate") == (200, "")
    st, text = sv.handle("GET", "/v1/models")
    assert json.loads(text)["data"][0]["id"] == "m"
    assert sv.handle("GET", "/v1/models/m")[0] == 200 and sv.handle("GET", "/v1/models/zzz")[0] == 404
    assert "b200e_requests_total" in sv.handle("GET", "/metrics")[1]


def test_engine_callback_backend_and_socket(tok_path, tok_text):
    tk = S.Tokenizer(tok_text)
    sv = S.Server(tok_path, model_name="m", eos_token_ids=[tk.encode("<|im_end|>")[0]])
    out = tk.encode("hello world<|im_end|>")
    seen = {}

    def generate(req_id, prompt, sampling, session):
        seen["prompt"], seen["sampling"] = prompt, sampling
        def run():
            for i in range(0, len(out), 2):
                if sv.push(req_id, out[i:i + 2]):
                    break
            sv.push(req_id, [], finished=True)
        threading.Thread(target=run).start()

    sv.use_engine(generate, context_length=4096)
    port = sv.start()
    body = json.dumps({"messages": [{"role": "user", "content": "hi"}], "stream": True}).encode()
    s = socket.create_connection(("127.0.0.1", port))
    s.sendall(b"POST /v1/chat/completions HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nContent-Length: %d\r\n\r\n" % len(body) + body)
    data = b""
    while True:
        chunk = s.recv(65536)
        if not chunk:
            break
        data += chunk
    s.close()
    sv.stop()
    head, _, payload = data.partition(b"\r\n\r\n")
    assert b"200 OK" in head and b"text/event-stream" in head
    events = [json.loads(l[6:]) for l in payload.decode().split("\n\n") if l.startswith("data: {")]
    text = "".join(e["choices"][0]["delta"].get("content", "") for e in events if e["choices"])
    assert text == "hello world" and payload.decode().endswith("data: [DONE]\n\n")
    assert seen["prompt"] == tk.encode(S.render_chat([{"role": "user", "content": "hi"}]))


def test_detokenizer_never_emits_invalid_utf8():
    """Byte tokens in an order that is not UTF-8 (a model may produce them) come out as U+FFFD, never as raw bytes."""
    import json as _json
    from tests.fixtures import bytes_to_unicode, tiny_tokenizer_json
    tj = tiny_tokenizer_json()
    vocab, b2u = _json.loads(tj)["model"]["vocab"], bytes_to_unicode()
    tk = S.Tokenizer(tj)
    ids = [vocab[b2u[b]] for b in (0xB5, ord("a"), 0xE2, ord("b"), 0xC3, 0xA9, 0xF0, 0x9F)]
    pieces = tk.stream_decode(ids, 1)
    text = "".join(pieces)
    assert text == "�a�bé�"
    assert tk.stream_decode(tk.encode("héllo ✓ wörld"), 2)[-1] == "" and "".join(tk.stream_decode(tk.encode("héllo ✓ wörld"), 2)) == "héllo ✓ wörld"


def test_image_parts_reach_the_engine_callback(tok_path, tok_text):
    """image_url parts: refused unless the backend takes images; otherwise one placeholder in the prompt per image and
    the URLs, in order, under sampling["images"] (reference: crates/agens-server/src/openai.rs content-part handling)."""
    sv = S.Server(tok_path, model_name="m")
    seen = {}

    def generate(req_id, prompt, sampling, session):
        seen["sampling"] = sampling
        sv.push(req_id, [], finished=True)

    url = "data:image/png;base64,AAAA"
    body = {"messages": [{"role": "user", "content": [{"type": "text", "text": "what is "}, {"type": "image_url", "image_url": {"url": url}},
                                                     {"type": "image_url", "image_url": {"url": url + "BB"}}]}], "max_tokens": 4}
    sv.use_engine(generate, context_length=4096)
    status, resp = sv.handle("POST", "/v1/chat/completions", body)
    assert status == 400 and "images" in json.loads(resp)["message"]
    sv.use_engine(generate, context_length=4096, supports_images=True)
    status, resp = sv.handle("POST", "/v1/chat/completions", body)
    assert status == 200
    assert seen["sampling"]["images"] == [url, url + "BB"]
    body["messages"][0]["content"][1]["image_url"]["url"] = "http://example.com/x.png"
    status, resp = sv.handle("POST", "/v1/chat/completions", body)
    assert status == 400


# ---- the other marker family (<|think|> ... <|/think|>, <|call|> ... <|/call|>) and the wire format, without fixtures ----
FAMILY_TEMPLATE = (
    "{% for m in messages %}<|agens_start|>{{ m.role }}\n{{ m.content }}<|agens_end|>\n{% endfor %}"
    "{% if tools %}<tools>{% for t in tools %}{{ t | tojson }}{% endfor %}</tools> calls look like <|call|>...<|/call|>\n{% endif %}"
    "<|agens_start|>assistant\n{% if enable_thinking is defined and not enable_thinking %}{% else %}<|think|>\n{% endif %}")
WEATHER = [{"type": "function", "function": {"name": "get_weather", "description": "weather", "parameters": {
    "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "int"}}}}}]


def _family_server(tok_path, tok_text, reply, step=1, **kw):
    tk = S.Tokenizer(tok_text)
    sv = S.Server(tok_path, model_name="m", chat_template=FAMILY_TEMPLATE, eos_token_ids=[tk.encode("<|im_end|>")[0]], **kw)
    sv.use_mock(tk.encode(reply) + tk.encode("<|im_end|>"), step=step)
    return sv, tk


def _events(body):
    out = []
    for line in body.split("\n\n"):
        if line.startswith("data: {"):
            out.append(json.loads(line[6:]))
    return out


def test_marker_family_comes_from_the_template_and_generation_starts_in_reasoning(tok_path, tok_text):
    reply = "plan it\n<|/think|>\n\nThe answer."
    sv, tk = _family_server(tok_path, tok_text, reply)
    st, body = sv.handle("POST", "/v1/chat/completions", {"rid": "R1", "messages": [{"role": "user", "content": "hi"}]})
    r = json.loads(body)
    assert st == 200 and r["id"] == "R1" and list(r) == ["id", "object", "created", "model", "choices", "usage", "metadata"]
    ch = r["choices"][0]
    assert list(ch) == ["index", "message", "logprobs", "finish_reason", "matched_stop"]
    assert ch["message"] == {"role": "assistant", "content": "\n\nThe answer.", "reasoning_content": "plan it\n", "tool_calls": None}
    eos = tk.encode("<|im_end|>")[0]
    assert ch["finish_reason"] == "stop" and ch["matched_stop"] == eos
    n_out = len(tk.encode(reply)) + 1
    n_reason = len(tk.encode("plan it\n<|/think|>"))             # tokens through the closing marker (several byte tokens here)
    assert r["usage"]["completion_tokens"] == n_out and r["usage"]["reasoning_tokens"] == n_reason
    assert r["usage"]["prompt_tokens_details"] is None and r["metadata"] == {"weight_version": "default"}
    # thinking off: the template leaves the block closed, nothing is reasoning and no reasoning tokens are counted
    sv, _ = _family_server(tok_path, tok_text, "Just text.")
    st, body = sv.handle("POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}],
                                                          "chat_template_kwargs": {"enable_thinking": False}})
    r = json.loads(body)
    assert r["choices"][0]["message"]["content"] == "Just text." and r["choices"][0]["message"]["reasoning_content"] is None
    assert r["usage"]["reasoning_tokens"] == 0
    # reasoning alone, with force_nonempty_content: it becomes the content
    sv, _ = _family_server(tok_path, tok_text, "only thoughts")
    st, body = sv.handle("POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}],
                                                          "chat_template_kwargs": {"force_nonempty_content": True}})
    msg = json.loads(body)["choices"][0]["message"]
    assert msg["content"] == "only thoughts" and msg["reasoning_content"] is None


def test_streamed_tool_call_goes_out_piece_by_piece(tok_path, tok_text):
    reply = ("think\n<|/think|>\n\nFirst.\n\n<|call|>\n<function=get_weather>\n<parameter=city>\nHong Kong\n</parameter>\n"
             "<parameter=days>\n2\n</parameter>\n</function>\n<|/call|>")
    for step in (1, 5):
        sv, tk = _family_server(tok_path, tok_text, reply, step=step)
        body = {"rid": "R2", "messages": [{"role": "user", "content": "weather?"}], "tools": WEATHER, "stream": True,
                "stream_options": {"include_usage": True}}
        st, text = sv.handle("POST", "/v1/chat/completions", body)
        assert st == 200 and text.endswith("data: [DONE]\n\n")
        ev = _events(text)
        first = ev[0]["choices"][0]
        assert first["delta"] == {"reasoning_content": None, "role": "assistant", "content": ""} and "usage" not in ev[0]
        reasoning = "".join(e["choices"][0]["delta"].get("reasoning_content") or "" for e in ev if e["choices"])
        content = "".join(e["choices"][0]["delta"].get("content") or "" for e in ev if e["choices"])
        assert reasoning == "think\n" and content == "\n\nFirst.\n\n"
        calls = [e["choices"][0]["delta"]["tool_calls"][0] for e in ev if e["choices"] and e["choices"][0]["delta"].get("tool_calls")]
        assert calls[0]["id"].startswith("call_") and calls[0]["function"] == {"name": "get_weather", "arguments": ""}
        assert [c["function"]["arguments"] for c in calls[1:]] == ["{", '"city": "Hong Kong"', ', "days": 2', "}"]
        assert all(c["id"] is None and c["function"]["name"] is None and c["index"] == 0 for c in calls[1:])
        # content events of a request with tools carry every delta field and a usage key
        with_content = [e for e in ev if e["choices"] and e["choices"][0]["delta"].get("content")]
        assert set(with_content[0]["choices"][0]["delta"]) == {"role", "content", "reasoning_content", "tool_calls"} and "usage" in with_content[0]
        fin = [e for e in ev if e["choices"] and e["choices"][0]["finish_reason"]][-1]["choices"][0]
        assert fin["finish_reason"] == "tool_calls" and fin["matched_stop"] == tk.encode("<|im_end|>")[0]
        assert ev[-1]["choices"] == [] and ev[-1]["usage"]["completion_tokens"] == len(tk.encode(reply)) + 1
    # the complete response of the same output: arguments typed by the (normalised) schema, no matched stop
    sv, tk = _family_server(tok_path, tok_text, reply)
    st, text = sv.handle("POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "weather?"}], "tools": WEATHER})
    ch = json.loads(text)["choices"][0]
    assert ch["finish_reason"] == "tool_calls" and ch["matched_stop"] is None and ch["message"]["content"] == "\n\nFirst.\n\n"
    tc = ch["message"]["tool_calls"][0]
    assert tc["index"] == 0 and tc["function"] == {"name": "get_weather", "arguments": '{"city": "Hong Kong", "days": 2}'}


def test_stop_strings_errors_and_completion_stream(tok_path, tok_text):
    sv, tk = _family_server(tok_path, tok_text, "r\n<|/think|>\n\nalpha beta STOP gamma")
    st, text = sv.handle("POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "stop": "STOP"})
    ch = json.loads(text)["choices"][0]
    assert ch["message"]["content"] == "\n\nalpha beta " and ch["finish_reason"] == "stop" and ch["matched_stop"] == "STOP"
    # validation errors: the reference's flat body
    st, text = sv.handle("POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "tool_choice": "required"})
    assert st == 400 and json.loads(text) == {"object": "error", "message": "Tools cannot be empty if tool choice is set to required.",
                                               "type": "BadRequestError", "param": None, "code": 400}
    st, text = sv.handle("POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "tools": WEATHER,
                                                          "tool_choice": {"type": "function", "function": {"name": "nope"}}})
    assert st == 400 and json.loads(text)["message"] == "Tool 'nope' not found in tools list."
    st, text = sv.handle("POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "max_tokens": 10 ** 7})
    assert st == 400 and "is too large" in json.loads(text)["message"]
    # /v1/completions stream: one event per step, the last step carries its text and the finish reason
    sv2 = S.Server(tok_path, model_name="m")
    sv2.use_mock(tk.encode("one two three"), step=1)
    st, text = sv2.handle("POST", "/v1/completions", {"prompt": "count", "max_tokens": 3, "stream": True, "stream_options": {"include_usage": True}})
    ev = _events(text)
    assert [e["choices"][0]["finish_reason"] for e in ev if e["choices"]] == [None, None, "length"]
    assert "".join(e["choices"][0]["text"] for e in ev if e["choices"]) == tk.decode(tk.encode("one two three")[:3], skip_special=False)
    assert ev[-1]["choices"] == [] and "prompt_tokens_details" not in ev[-1]["usage"]


def test_tools_reach_the_template_in_normal_form(tok_path, tok_text):
    """Tools as the template sees them: description / name / parameters / strict in that order plus defer_loading,
    database-style type names rewritten to JSON-schema ones, a named tool_choice listing that tool only."""
    tpl = "{% for t in tools %}{{ t | tojson }}\n{% endfor %}{{ messages[0].content }}"
    tk = S.Tokenizer(tok_text)
    sv = S.Server(tok_path, model_name="m", chat_template=tpl)
    sv.use_mock(tk.encode("ok"), step=1)
    tools = [{"type": "function", "function": {"name": "db", "parameters": {"type": "object", "properties": {
                 "id": {"type": "int"}, "name": {"type": "varchar(255)"}, "price": {"type": "decimal(10,2)"}, "tags": {"type": "list[str]"},
                 "meta": {"type": "map"}, "flag": {"type": ["bool", "null", "boolean"]}, "u": {"type": "uint8"}, "other": {"type": "widget"},
                 "nested": {"type": "object", "properties": {"when": {"type": "TIMESTAMP"}}, "items": {"type": "float32"}}}}}},
             {"type": "function", "function": {"name": "second", "description": "d", "parameters": {"type": "object"}, "strict": True},
              "defer_loading": True}]
    body = {"messages": [{"role": "user", "content": "END"}], "tools": tools, "max_tokens": 2}
    assert sv.handle("POST", "/v1/chat/completions", body)[0] == 200
    lines = tk.decode(sv.mock_calls()[-1]["prompt"], skip_special=False).split("\n")
    first, second = json.loads(lines[0]), json.loads(lines[1])
    assert list(first) == ["type", "function", "defer_loading"] and first["defer_loading"] is None
    assert list(first["function"]) == ["description", "name", "parameters", "strict"] and first["function"]["strict"] is False
    props = first["function"]["parameters"]["properties"]
    assert {k: v["type"] for k, v in props.items() if k != "nested"} == {
        "id": "integer", "name": "string", "price": "number", "tags": "array", "meta": "object", "flag": ["boolean", "null"],
        "u": "integer", "other": "widget"}
    assert props["nested"]["properties"]["when"]["type"] == "string" and props["nested"]["items"]["type"] == "number"
    assert second["function"]["strict"] is True and second["function"]["defer_loading"] is True and second["defer_loading"] is True
    # a named tool_choice: only that tool is shown
    assert sv.handle("POST", "/v1/chat/completions", dict(body, tool_choice={"type": "function", "function": {"name": "second"}}))[0] == 200
    text = tk.decode(sv.mock_calls()[-1]["prompt"], skip_special=False)
    assert text.count("\n") == 1 and json.loads(text.split("\n")[0])["function"]["name"] == "second"


def test_tokenizer_differential_on_a_trained_bpe():
    """A byte-level BPE trained here with the `tokenizers` library on mixed-script text (the pre-tokeniser pattern of the
    dense GQA checkpoints): the C++ tokenizer gives the same ids and the same decoded text on the corpus and on random
    strings of awkward pieces (contractions in any case, digits of other scripts, emoji, marker tokens, runs of blanks)."""
    import random
    tk_lib = pytest.importorskip("tokenizers")
    from tokenizers import Regex, decoders, models, pre_tokenizers, trainers
    rnd = random.Random(0)
    words = ["hello", "world", "the", "quick", "brown", "fox", "naïve", "café", "漢字", "かな", "한국어", "don't", "I'm", "we'll", "THEY'RE", "x=12*345;",
             "foo_bar", "CamelCase", "1234567", "3.14159", "🙂", "👍🏽", "Ünïcödé", "ß", "Ελληνικά", "русский", "עברית", "العربية", "\t", "\n", "\r\n",
             "  ", "   ", "!!!", "...", "<|im_start|>", "</s>", "a", "b", "ab", "abc"]
    corpus = ["".join(rnd.choice(words) + rnd.choice(["", " ", " ", "  ", "\n", ", ", ". "]) for _ in range(rnd.randint(1, 12))) for _ in range(1500)]
    tok = tk_lib.Tokenizer(models.BPE())
    pat = "(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\\r\\n\\p{L}\\p{N}]?\\p{L}+|\\p{N}| ?[^\\s\\p{L}\\p{N}]+[\\r\\n]*|\\s*[\\r\\n]+|\\s+(?!\\S)|\\s+"
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pat), behavior="isolated", invert=False),
                                                 pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=900, special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"],
                                                        initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False))
    mine = S.Tokenizer(tok.to_str())
    pieces = ["a", "b", " ", "  ", "\n", "'", "'s", "'S", "'Re", "1", "22", "é", "漢", "🙂", "\t", "!", "?", "_", "x", "The", " the", "<|im_start|>",
              "<|im_end|>", "\r\n", " ", "Ⅷ", "²", "٣"]
    tests = corpus[:200] + ["".join(rnd.choice(pieces) for _ in range(rnd.randint(0, 40))) for _ in range(600)]
    for t in tests:
        want = tok.encode(t, add_special_tokens=False).ids
        assert mine.encode(t) == want, t
        assert mine.decode(want, skip_special=False) == tok.decode(want, skip_special_tokens=False), t


def _raw(port, payload: bytes, half_close: bool = False) -> bytes:
    s = socket.create_connection(("127.0.0.1", port))
    s.settimeout(20)
    s.sendall(payload)
    if half_close:
        s.shutdown(socket.SHUT_WR)
    data = b""
    while True:
        chunk = s.recv(65536)
        if not chunk:
            break
        data += chunk
    s.close()
    return data


def test_socket_layer_limits_and_framing(tok_path, tok_text):
    """The listener's own framing rules: Content-Length must be a plain number within the body limit, a chunked body is
    reassembled, ``Expect: 100-continue`` is answered before the body is read, a body that ends early is an error, and
    none of it disturbs the next request."""
    tk = S.Tokenizer(tok_text)
    sv = S.Server(tok_path, model_name="m", eos_token_ids=[])
    sv.use_mock(tk.encode("ok then"), step=2)
    port = sv.start()
    try:
        body = json.dumps({"prompt": "hi", "max_tokens": 3}).encode()
        head = b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\n"
        ok = _raw(port, head + b"Content-Length: %d\r\n\r\n" % len(body) + body)
        want = json.loads(ok.partition(b"\r\n\r\n")[2])["choices"][0]["text"]
        assert ok.startswith(b"HTTP/1.1 200") and want
        # a body limit and a syntax check on the length
        big = _raw(port, head + b"Content-Length: 99999999999999\r\n\r\n")
        assert big.startswith(b"HTTP/1.1 413") and json.loads(big.partition(b"\r\n\r\n")[2])["object"] == "error"
        for bad in (b"-5", b"12abc", b"", b"1" * 30):
            r = _raw(port, head + b"Content-Length: " + bad + b"\r\n\r\n" + body)
            assert r.startswith(b"HTTP/1.1 400"), (bad, r[:80])
        # chunked transfer encoding, with a chunk extension and the pieces cut mid-token
        cut = [body[:5], body[5:6], body[6:]]
        chunked = b"".join(b"%x;ext=1\r\n" % len(c) + c + b"\r\n" for c in cut) + b"0\r\n\r\n"
        r = _raw(port, head + b"Transfer-Encoding: chunked\r\n\r\n" + chunked)
        assert r.startswith(b"HTTP/1.1 200") and json.loads(r.partition(b"\r\n\r\n")[2])["choices"][0]["text"] == want
        r = _raw(port, head + b"Transfer-Encoding: chunked\r\n\r\nzz\r\n")
        assert r.startswith(b"HTTP/1.1 400")
        # Expect: 100-continue
        s = socket.create_connection(("127.0.0.1", port))
        s.settimeout(20)
        s.sendall(head + b"Expect: 100-continue\r\nContent-Length: %d\r\n\r\n" % len(body))
        assert s.recv(64).startswith(b"HTTP/1.1 100 Continue")
        s.sendall(body)
        data = b""
        while True:
            chunk = s.recv(65536)
            if not chunk:
                break
            data += chunk
        s.close()
        assert b"200 OK" in data and want.encode() in data
        # the client goes away in the middle of the body; extra bytes after the body are not part of it
        r = _raw(port, head + b"Content-Length: %d\r\n\r\n" % (len(body) + 10) + body, half_close=True)
        assert r.startswith(b"HTTP/1.1 408")
        r = _raw(port, head + b"Content-Length: %d\r\n\r\n" % len(body) + body + b"GARBAGE")
        assert r.startswith(b"HTTP/1.1 200")
        assert _raw(port, b"\r\n\r\n").startswith(b"HTTP/1.1 404") and _raw(port, b"GET /health HTTP/1.1\r\n\r\n").startswith(b"HTTP/1.1 200")
    finally:
        sv.stop()


def test_first_requests_of_a_process_may_arrive_together(tok_text, tmp_path):
    """The tokenizer's byte tables are built on first use; many threads may be the first at once (connection threads
    of the listener).  Fresh processes, sixteen threads released together, every decode checked."""
    import subprocess
    import sys
    (tmp_path / "tok.json").write_text(tok_text)
    prog = (
        "import sys, threading\n"
        "from agens_engine_b200.serve import server as S\n"
        "tk = S.Tokenizer(open(sys.argv[1]).read())\n"
        "ids = list(range(40, 256)) * 4\n"
        "go, out = threading.Barrier(16), [None] * 16\n"
        "def run(i):\n"
        "    go.wait()\n"
        "    out[i] = (tk.decode(ids, skip_special=False), tk.encode('héllo wörld ✓ ' * 20))\n"
        "th = [threading.Thread(target=run, args=(i,)) for i in range(16)]\n"
        "[t.start() for t in th]; [t.join() for t in th]\n"
        "assert all(o == out[0] for o in out) and out[0][0] and tk.decode(out[0][1], skip_special=False) == 'héllo wörld ✓ ' * 20\n"
        "print('same')\n")
    for _ in range(3):
        r = subprocess.run([sys.executable, "-c", prog, str(tmp_path / "tok.json")], capture_output=True, text=True, timeout=120)
        assert r.returncode == 0 and r.stdout.strip() == "same", r.stderr[-2000:]


def test_long_unbroken_runs_tokenize_in_linear_time_and_like_the_library(tok_text):
    """A hundred thousand spaces, or one word repeated without a break, is one pre-token; its merges must not cost a
    scan each (that took minutes).  Same ids as the tokenizers library, within seconds."""
    import time
    tokenizers = pytest.importorskip("tokenizers")
    ref = tokenizers.Tokenizer.from_str(tok_text)
    mine = S.Tokenizer(tok_text)
    t0 = time.time()
    for text in (" " * 100000, "the" * 33000, "ab" * 20000 + " " + "thing" * 9000, "\n" * 50000, "aaaa" * 10000 + "é" * 5000):
        ids = mine.encode(text)
        assert ids == ref.encode(text, add_special_tokens=False).ids, text[:12]
    assert time.time() - t0 < 30


def test_deeply_nested_tool_arguments_fall_back_to_text():
    """Model output decides how deep a parameter's literal nests: beyond the parser's depth the value is kept as text
    (a hundred thousand brackets used to overflow the stack)."""
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object", "properties": {"a": {"type": "array"}, "o": {"type": "object"}}}}}]
    for lit, key in (("[" * 100000 + "]" * 100000, "a"), ("{'k': " * 100000 + "1" + "}" * 100000, "o"), ("(" * 100000 + "1," + ")" * 100000, "a")):
        out = S.parse_output(f"<tool_call>\n<function=f>\n<parameter={key}>\n{lit}\n</parameter>\n</function>\n</tool_call>", tools)
        assert json.loads(out["tool_calls"][0]["arguments"])[key] == lit
    out = S.parse_output("<tool_call>\n<function=f>\n<parameter=a>\n" + "[" * 40 + "(1, 'x')" + "]" * 40 + "\n</parameter>\n</function>\n</tool_call>", tools)
    v = json.loads(out["tool_calls"][0]["arguments"])["a"]
    for _ in range(40):
        v = v[0]
    assert v == [1, "x"]
