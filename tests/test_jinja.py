"""The C++ Jinja subset against jinja2 (the renderer Hugging Face chat templates are written for: trim_blocks,
lstrip_blocks, tojson = json.dumps(ensure_ascii=False), raise_exception, loop controls) on chat templates of the
families the reference serves (reference: crates/agens-server/src/template.rs and its parity tests)."""
import json

import pytest

from agens_engine_b200.serve import server as S

jinja2 = pytest.importorskip("jinja2")


def oracle(source, **ctx):
    from jinja2.sandbox import ImmutableSandboxedEnvironment
    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, extensions=["jinja2.ext.loopcontrols"])

    def tojson(x, ensure_ascii=False, indent=None, separators=None, sort_keys=False):
        return json.dumps(x, ensure_ascii=ensure_ascii, indent=indent, separators=separators, sort_keys=sort_keys)

    def raise_exception(msg):
        raise jinja2.exceptions.TemplateError(msg)

    env.filters["tojson"] = tojson
    env.globals["raise_exception"] = raise_exception
    return env.from_string(source).render(**ctx)


CHATML_TOOLS = """{%- if tools %}
    {{- '<|im_start|>system\\n' }}
    {%- if messages[0]['role'] == 'system' %}
        {{- messages[0]['content'] }}
    {%- else %}
        {{- 'You are a helpful assistant.' }}
    {%- endif %}
    {{- "\\n\\n# Tools\\n\\nYou may call one or more functions.\\n<tools>" }}
    {%- for tool in tools %}
        {{- "\\n" }}
        {{- tool | tojson }}
    {%- endfor %}
    {{- "\\n</tools><|im_end|>\\n" }}
{%- else %}
    {%- if messages[0]['role'] == 'system' %}
        {{- '<|im_start|>system\\n' + messages[0]['content'] + '<|im_end|>\\n' }}
    {%- endif %}
{%- endif %}
{%- for message in messages %}
    {%- if (message.role == "user") or (message.role == "system" and not loop.first) or (message.role == "assistant" and not message.tool_calls) %}
        {{- '<|im_start|>' + message.role + '\\n' + message.content + '<|im_end|>' + '\\n' }}
    {%- elif message.role == "assistant" %}
        {{- '<|im_start|>' + message.role }}
        {%- if message.content %}
            {{- '\\n' + message.content }}
        {%- endif %}
        {%- for tool_call in message.tool_calls %}
            {%- if tool_call.function is defined %}
                {%- set tool_call = tool_call.function %}
            {%- endif %}
            {{- '\\n<tool_call>\\n{"name": "' }}
            {{- tool_call.name }}
            {{- '", "arguments": ' }}
            {{- tool_call.arguments | tojson }}
            {{- '}\\n</tool_call>' }}
        {%- endfor %}
        {{- '<|im_end|>\\n' }}
    {%- elif message.role == "tool" %}
        {%- if (loop.index0 == 0) or (messages[loop.index0 - 1].role != "tool") %}
            {{- '<|im_start|>user' }}
        {%- endif %}
        {{- '\\n<tool_response>\\n' }}
        {{- message.content }}
        {{- '\\n</tool_response>' }}
        {%- if loop.last or (messages[loop.index0 + 1].role != "tool") %}
            {{- '<|im_end|>\\n' }}
        {%- endif %}
    {%- endif %}
{%- endfor %}
{%- if add_generation_prompt %}
    {{- '<|im_start|>assistant\\n' }}
{%- endif %}
"""

THINKING = """{%- set ns = namespace(multi_step_tool=true, last_query_index=messages|length - 1) %}
{%- for message in messages[::-1] %}
    {%- set index = (messages|length - 1) - loop.index0 %}
    {%- if ns.multi_step_tool and message.role == "user" and message.content is string and not(message.content.startswith('<tool_response>') and message.content.endswith('</tool_response>')) %}
        {%- set ns.multi_step_tool = false %}
        {%- set ns.last_query_index = index %}
    {%- endif %}
{%- endfor %}
{%- for message in messages %}
    {%- if message.content is string %}
        {%- set content = message.content %}
    {%- else %}
        {%- set content = '' %}
    {%- endif %}
    {%- if message.role == "assistant" %}
        {%- set reasoning_content = '' %}
        {%- if message.reasoning_content is string %}
            {%- set reasoning_content = message.reasoning_content %}
        {%- else %}
            {%- if '</think>' in content %}
                {%- set reasoning_content = content.split('</think>')[0].rstrip('\\n').split('<think>')[-1].lstrip('\\n') %}
                {%- set content = content.split('</think>')[-1].lstrip('\\n') %}
            {%- endif %}
        {%- endif %}
        {%- if loop.index0 > ns.last_query_index %}
            {%- if loop.last or (not loop.last and reasoning_content) %}
                {{- '<|im_start|>' + message.role + '\\n<think>\\n' + reasoning_content.strip('\\n') + '\\n</think>\\n\\n' + content.lstrip('\\n') }}
            {%- else %}
                {{- '<|im_start|>' + message.role + '\\n' + content }}
            {%- endif %}
        {%- else %}
            {{- '<|im_start|>' + message.role + '\\n' + content }}
        {%- endif %}
        {{- '<|im_end|>\\n' }}
    {%- else %}
        {{- '<|im_start|>' + message.role + '\\n' + content + '<|im_end|>' + '\\n' }}
    {%- endif %}
{%- endfor %}
{%- if add_generation_prompt %}
    {{- '<|im_start|>assistant\\n' }}
    {%- if enable_thinking is defined and enable_thinking is false %}
        {{- '<think>\\n\\n</think>\\n\\n' }}
    {%- endif %}
{%- endif %}
"""

HEADER_STYLE = """{{ bos_token }}
{% for message in messages %}
{% set content = '<|start_header_id|>' ~ message['role'] ~ '<|end_header_id|>\\n\\n' ~ message['content'] | trim ~ '<|eot_id|>' %}
{% if loop.index0 == 0 %}{% set content = bos_token + content %}{% endif %}
{{ content }}
{% endfor %}
{% if add_generation_prompt %}{{ '<|start_header_id|>assistant<|end_header_id|>\\n\\n' }}{% endif %}
"""

FEATURES = """{# a comment #}
{% macro tag(name, body='x') %}<{{ name }}>{{ body }}</{{ name }}>{% endmacro %}
{{ tag('a') }}|{{ tag('b', body=items|length) }}
{% for k, v in table.items() %}{{ k }}={{ v }}{% if not loop.last %}, {% endif %}{% endfor %}

{% for x in items if x % 2 == 1 %}[{{ loop.index }}/{{ loop.length }}:{{ x }}]{% else %}none{% endfor %}

{% for x in [] %}never{% else %}empty{% endfor %}

{% for x in items %}{% if x == 3 %}{% continue %}{% endif %}{% if x == 5 %}{% break %}{% endif %}{{ x }}{% endfor %}

{{ items | join('-') }} {{ items[1:3] }} {{ items[-1] }} {{ name | upper }} {{ name[::-1] }} {{ missing | default('dflt') }}
{{ 7 // 2 }} {{ 7 % 3 }} {{ 7 / 2 }} {{ 2 * 3 + 1 }} {{ -items[0] }} {{ 'ab' * 2 }} {{ 1 if items else 2 }} {{ none }} {{ true }}
{{ table | tojson }} {{ table | tojson(indent=2) }} {{ nested | tojson }}
{{ 'é' | length }} {{ name is string }} {{ table is mapping }} {{ missing is defined }} {{ items is iterable }} {{ 3 is odd }}
{{ 'x' in name }} {{ 'a' in table }} {{ 9 not in items }} {{ name.startswith('ex') }} {{ "a,b,c".split(',') }} {{ "  pad ".strip() ~ '|' }}
{{ people | selectattr('age', 'gt', 30) | map(attribute='name') | join(', ') }} {{ people | rejectattr('vip') | list | length }}
{% set total = namespace(v=0) %}{% for p in people %}{% set total.v = total.v + p.age %}{% endfor %}{{ total.v }}
{%+ if true %}kept{% endif +%}
    {% if true %}
  indented
    {% endif %}
{{- ' tight ' -}}
   end
"""

MESSAGES = [
    {"role": "system", "content": "be brief"},
    {"role": "user", "content": "what is 2+2?"},
    {"role": "assistant", "content": "<think>\nadd\n</think>\n\n4"},
    {"role": "user", "content": "weather in Zürich?"},
    {"role": "assistant", "content": "", "tool_calls": [{"type": "function", "function": {"name": "get_weather", "arguments": {"city": "Zürich", "days": 2}}}]},
    {"role": "tool", "content": "{\"temp\": 21.5}"},
    {"role": "tool", "content": "sunny"},
    {"role": "assistant", "content": "21.5 °C and sunny", "reasoning_content": "two results"},
    {"role": "user", "content": "thanks  "},
]
TOOLS = [{"type": "function", "function": {"name": "get_weather", "description": "Weather \"now\"", "parameters": {
    "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer", "default": 1}}, "required": ["city"]}}}]


@pytest.mark.parametrize("tools", [None, TOOLS])
@pytest.mark.parametrize("gen", [True, False])
def test_chatml_family_with_tools(tools, gen):
    for msgs in (MESSAGES, MESSAGES[1:], MESSAGES[:2]):
        ctx = dict(messages=msgs, tools=tools, add_generation_prompt=gen)
        assert S.render_template(CHATML_TOOLS, **ctx) == oracle(CHATML_TOOLS, **ctx)


@pytest.mark.parametrize("thinking", [None, True, False])
def test_thinking_family(thinking):
    text_only = [m for m in MESSAGES if m["role"] != "tool" and not m.get("tool_calls")]
    for msgs in (text_only, text_only[:3], text_only[:2]):
        ctx = dict(messages=msgs, add_generation_prompt=True)
        if thinking is not None:
            ctx["enable_thinking"] = thinking
        assert S.render_template(THINKING, **ctx) == oracle(THINKING, **ctx)


def test_header_family_and_feature_coverage():
    ctx = dict(messages=MESSAGES[:2], bos_token="<|begin_of_text|>", add_generation_prompt=True)
    assert S.render_template(HEADER_STYLE, **ctx) == oracle(HEADER_STYLE, **ctx)
    ctx = dict(items=[1, 2, 3, 4, 5, 6], name="example", table={"b": 1, "a": "two", "c": [1.5, None, True]},
               nested={"k": {"x": [1, {"y": "ü\n\"q\""}], "z": 1e-07}},
               people=[{"name": "Ann", "age": 41, "vip": True}, {"name": "Bo", "age": 29, "vip": False}, {"name": "Cy", "age": 35, "vip": False}])
    assert S.render_template(FEATURES, **ctx) == oracle(FEATURES, **ctx)


def test_errors_are_reported():
    with pytest.raises(ValueError, match="only user and assistant"):
        S.render_template("{% if messages[0].role == 'tool' %}{{ raise_exception('only user and assistant roles') }}{% endif %}",
                          messages=[{"role": "tool", "content": "x"}])
    for bad in ("{% if x %}open", "{{ 1 + }}", "{% frobnicate %}", "{{ x | nosuchfilter }}", "{{ 'abc' "):
        with pytest.raises(ValueError):
            S.render_template(bad, x=1)


def test_server_renders_chat_requests_with_the_checkpoint_template(tmp_path):
    from tests.fixtures import tiny_tokenizer_json
    tok = tmp_path / "tokenizer.json"
    tok.write_text(tiny_tokenizer_json())
    tk = S.Tokenizer(tiny_tokenizer_json())
    sv = S.Server(str(tok), model_name="m", chat_template=CHATML_TOOLS)
    sv.use_mock(tk.encode("ok"), step=1)
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "weather?"},
            {"role": "assistant", "content": "", "tool_calls": [{"id": "c1", "type": "function", "function": {
                "name": "get_weather", "arguments": json.dumps({"city": "Oslo"})}}]},
            {"role": "tool", "tool_call_id": "c1", "content": "rain"}]
    status, _ = sv.handle("POST", "/v1/chat/completions", {"messages": msgs, "tools": TOOLS, "max_tokens": 4})
    assert status == 200
    want_msgs = json.loads(json.dumps(msgs))
    want_msgs[2]["tool_calls"][0]["function"]["arguments"] = {"city": "Oslo"}
    # the template sees the tools in the server's normal form: description, name, parameters, strict, then defer_loading
    want_tools = [{"type": "function", "function": {"description": t["function"].get("description"), "name": t["function"]["name"],
                                                    "parameters": t["function"].get("parameters"), "strict": False},
                   "defer_loading": None} for t in TOOLS]
    want = oracle(CHATML_TOOLS, messages=want_msgs, tools=want_tools, add_generation_prompt=True)
    assert sv.mock_calls()[-1]["prompt"] == tk.encode(want)
    # a template that refuses the conversation turns into a 400 with its message
    sv2 = S.Server(str(tok), model_name="m", chat_template="{{ raise_exception('no system role') }}")
    status, resp = sv2.handle("POST", "/v1/chat/completions", {"messages": msgs[:2]})
    assert status == 400 and "no system role" in resp


def test_templates_that_nest_without_end_are_refused_not_crashed():
    """Parentheses, unary chains, blocks, operator chains and macro recursion beyond the interpreter's limits raise an
    error (in a fresh process: before the limits these overflowed the stack)."""
    import subprocess
    import sys
    prog = (
        "from agens_engine_b200.serve import server as S\n"
        "cases = ['{{ ' + '(' * 5000 + '1' + ')' * 5000 + ' }}', '{{ ' + '(' * 100000 + '1' + ')' * 100000 + ' }}',\n"
        "         '{{ ' + 'not ' * 5000 + 'true }}', '{{ ' + '-' * 5000 + '1 }}', '{{ ' + '[' * 5000 + ']' * 5000 + ' }}',\n"
        "         '{% if true %}' * 50000 + 'x' + '{% endif %}' * 50000, '{% for a in [1] %}' * 3000 + 'x' + '{% endfor %}' * 3000,\n"
        "         '{{ ' + ' + '.join(['1'] * 9990) + ' }}', '{{ ' + ' ~ '.join([\"'a'\"] * 9990) + ' }}',\n"
        "         '{% macro f(n) %}{{ f(n + 1) }}{% endmacro %}{{ f(0) }}',\n"
        "         '{{ 1 if ' * 3000 + 'true' + ' else 2 }}' * 0 + '{{ ' + 'a if b else ' * 3000 + 'c }}']\n"
        "bad = 0\n"
        "for c in cases:\n"
        "    try:\n"
        "        S.render_template(c, a=1, b=0, c=2)\n"
        "    except ValueError:\n"
        "        bad += 1\n"
        "deep = 1\n"
        "for _ in range(150):\n"
        "    deep = [deep]\n"
        "assert S.render_template('{{ v | tojson }}{{ v }}', v=deep).count('[') == 300\n"
        "assert S.render_template('{{ ' + ' + '.join(['1'] * 500) + ' }}') == '500'\n"
        "assert S.render_template('{{ ' + '(' * 100 + '7' + ')' * 100 + ' }}') == '7'\n"
        "print('refused', bad, 'of', len(cases))\n")
    r = subprocess.run([sys.executable, "-c", prog], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip() == "refused 11 of 11", (r.returncode, r.stdout, r.stderr[-1500:])


def test_long_conversations_render_in_linear_time():
    """A template that subscripts the message list inside its loop over the messages (most chat templates do) must not
    copy the conversation per access: 4000 messages took seconds, a 1000-message agent transcript a quarter of one."""
    import time
    tmpl = ("{% for m in messages %}{% if loop.index0 > 0 and messages[loop.index0 - 1].role == m.role %}!{% endif %}"
            "<|{{ m.role }}|>{{ m['content'] }}{% if messages | length > 1 and loop.last %}[{{ messages[-1].content | length }}]{% endif %}\n{% endfor %}")
    def conv(n):
        return [{"role": "user" if i % 2 == 0 else "assistant", "content": ("message %d " % i) * 40} for i in range(n)]
    jinja2 = pytest.importorskip("jinja2")
    want = jinja2.Environment(trim_blocks=True, lstrip_blocks=True).from_string(tmpl).render(messages=conv(50))
    assert S.render_template(tmpl, messages=conv(50)) == want
    S.render_template(tmpl, messages=conv(500))
    t0 = time.time(); S.render_template(tmpl, messages=conv(1000)); t1 = time.time() - t0
    t0 = time.time(); out = S.render_template(tmpl, messages=conv(8000)); t8 = time.time() - t0
    assert out.count("<|user|>") == 4000 and t8 < 2.0 and t8 < 40 * max(t1, 0.005), (t1, t8)
