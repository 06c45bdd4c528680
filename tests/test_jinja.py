"""Native Jinja subset against the jinja2 package on chat-template style sources."""
import pytest

from volta_engine_b200.loader.chat_template import ChatTemplate, TemplateError, render

QWEN_LIKE = r"""
{%- if tools %}
    {{- '<|im_start|>system\n' }}
    {%- if messages[0].role == 'system' %}
        {{- messages[0].content + '\n\n' }}
    {%- endif %}
    {{- "# Tools\n\n<tools>" }}
    {%- for tool in tools %}
        {{- "\n" }}
        {{- tool | tojson }}
    {%- endfor %}
    {{- "\n</tools><|im_end|>\n" }}
{%- else %}
    {%- if messages[0].role == 'system' %}
        {{- '<|im_start|>system\n' + messages[0].content + '<|im_end|>\n' }}
    {%- endif %}
{%- endif %}
{%- set ns = namespace(multi_step_tool=true, last_query_index=messages|length - 1) %}
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
    {%- if (message.role == "user") or (message.role == "system" and not loop.first) %}
        {{- '<|im_start|>' + message.role + '\n' + content + '<|im_end|>' + '\n' }}
    {%- elif message.role == "assistant" %}
        {%- set reasoning_content = '' %}
        {%- if '</think>' in content %}
            {%- set reasoning_content = content.split('</think>')[0].rstrip('\n').split('<think>')[-1].lstrip('\n') %}
            {%- set content = content.split('</think>')[-1].lstrip('\n') %}
        {%- endif %}
        {%- if loop.index0 > ns.last_query_index and reasoning_content %}
            {{- '<|im_start|>' + message.role + '\n<think>\n' + reasoning_content.strip('\n') + '\n</think>\n\n' + content.lstrip('\n') }}
        {%- else %}
            {{- '<|im_start|>' + message.role + '\n' + content }}
        {%- endif %}
        {%- if message.tool_calls %}
            {%- for tool_call in message.tool_calls %}
                {%- if tool_call.function %}
                    {%- set tool_call = tool_call.function %}
                {%- endif %}
                {{- '\n<tool_call>\n{"name": "' }}
                {{- tool_call.name }}
                {{- '", "arguments": ' }}
                {%- if tool_call.arguments is string %}
                    {{- tool_call.arguments }}
                {%- else %}
                    {{- tool_call.arguments | tojson }}
                {%- endif %}
                {{- '}\n</tool_call>' }}
            {%- endfor %}
        {%- endif %}
        {{- '<|im_end|>\n' }}
    {%- elif message.role == "tool" %}
        {%- if loop.first or (messages[loop.index0 - 1].role != "tool") %}
            {{- '<|im_start|>user' }}
        {%- endif %}
        {{- '\n<tool_response>\n' }}
        {{- content }}
        {{- '\n</tool_response>' }}
        {%- if loop.last or (messages[loop.index0 + 1].role != "tool") %}
            {{- '<|im_end|>\n' }}
        {%- endif %}
    {%- endif %}
{%- endfor %}
{%- if add_generation_prompt %}
    {{- '<|im_start|>assistant\n' }}
    {%- if enable_thinking is defined and enable_thinking is false %}
        {{- '<think>\n\n</think>\n\n' }}
    {%- endif %}
{%- endif %}
"""

MISC = r"""
{%- macro greet(name, punct='!') -%}Hello {{ name|upper }}{{ punct }}{%- endmacro -%}
{{ greet('bob') }} {{ greet('amy', punct='?') }}
{% for k, v in d.items() %}{{ k }}={{ v }}{% if not loop.last %}, {% endif %}{% endfor %}
{% set xs = [] %}{% for i in range(5) if i % 2 == 0 %}{% set _ = xs.append(i * 2) %}{% endfor %}{{ xs | join('-') }}
{{ 'a,b,c'.split(',') | last }} {{ (3 + 4) * 2 // 3 }} {{ 7 % 3 }} {{ 'x' ~ 1 ~ none }} {{ [1,2,3][1:] }}
{{ missing | default('dflt') }} {{ name if name is defined else 'anon' }} {{ items | selectattr('on') | map(attribute='id') | list }}
{%- if 'ell' in 'hello' and not (1 > 2) %} yes{% else %} no{% endif %}
{{ {'a': 1, 'b': [true, none]} | tojson }}
"""


def _jinja2(src, ctx):
    jinja2 = pytest.importorskip("jinja2")
    env = jinja2.Environment(trim_blocks=True, lstrip_blocks=True)
    env.policies["json.dumps_kwargs"] = {"ensure_ascii": False, "sort_keys": False}
    return env.from_string(src).render(**ctx)


CONVS = [
    [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Hi"}],
    [{"role": "user", "content": "2+2?"}, {"role": "assistant", "content": "<think>\neasy\n</think>\n\n4"},
     {"role": "user", "content": "and 3+3?"}],
    [{"role": "user", "content": "weather?"},
     {"role": "assistant", "content": "", "tool_calls": [{"type": "function", "function": {"name": "get_w", "arguments": {"city": "Oslo"}}}]},
     {"role": "tool", "content": "{\"t\": 3}"}, {"role": "tool", "content": "{\"t\": 4}"}],
]
TOOLS = [{"type": "function", "function": {"name": "get_w", "description": "Weather", "parameters": {"type": "object", "properties": {"city": {"type": "string"}}}}}]


@pytest.mark.parametrize("conv", range(len(CONVS)))
@pytest.mark.parametrize("tools", [None, TOOLS])
@pytest.mark.parametrize("think", [None, False])
def test_qwen_like_template_matches_jinja2(conv, tools, think):
    ctx = {"messages": CONVS[conv], "add_generation_prompt": True}
    if tools:
        ctx["tools"] = tools
    if think is not None:
        ctx["enable_thinking"] = think
    assert render(QWEN_LIKE, ctx) == _jinja2(QWEN_LIKE, ctx)


def test_misc_constructs_match_jinja2():
    ctx = {"d": {"x": 1, "y": "two"}, "items": [{"id": 1, "on": True}, {"id": 2, "on": False}, {"id": 3, "on": True}]}
    assert render(MISC, ctx) == _jinja2(MISC, ctx)


def test_errors_and_default_template():
    with pytest.raises(TemplateError):
        render("{{ raise_exception('bad role') }}", {})
    with pytest.raises(TemplateError):
        render("{% if x %}unclosed", {})
    t = ChatTemplate("{{ bos_token }}{% for m in messages %}[{{ m.role }}]{{ m.content }}{% endfor %}", bos_token="<s>")
    assert t.apply([{"role": "user", "content": "hey"}]) == "<s>[user]hey"
