"""Built-in DeepSeek prompt format: turn markers, thinking open/close rules, effort line, DSML tool markup, tool results
folded into user turns in call order, image placeholders, error cases. Golden strings written out by hand from the
format rules."""
import pytest

from volta_engine_b200.loader import deepseek_encoding as ds

B, E, U, A, S = ds.BOS, ds.EOS, ds.USER, ds.ASSISTANT, ds.SYSTEM


def test_plain_chat_with_and_without_thinking():
    msgs = [{"role": "user", "content": "Hi"}]
    assert ds.encode(msgs, thinking=False) == f"{B}{U}Hi{A}</think>"
    assert ds.encode(msgs, thinking=True) == (f"{B}{S}Reasoning Effort: 75 (range 1-100, the higher the value, the more "
                                             f"thorough the reasoning)\n\n{U}Hi{A}<think>")
    assert ds.encode(msgs, thinking=True, reasoning_effort="low").startswith(f"{B}{S}Reasoning Effort: 50 ")
    assert ds.encode(msgs, thinking=True, reasoning_effort="33").startswith(f"{B}{S}Reasoning Effort: 33 ")
    with pytest.raises(ds.EncodingError):
        ds.encode(msgs, thinking=True, reasoning_effort="101")


def test_multi_turn_drops_old_reasoning_but_keeps_the_latest():
    msgs = [{"role": "system", "content": "Be terse."}, {"role": "user", "content": "1+1?"},
            {"role": "assistant", "content": "2", "reasoning_content": "easy"}, {"role": "user", "content": "2+2?"}]
    out = ds.encode(msgs, thinking=False)
    assert out == f"{B}{S}Be terse.{U}1+1?{A}</think>2{E}{U}2+2?{A}</think>"
    out = ds.encode(msgs, thinking=True, reasoning_effort="max")
    eff = "Reasoning Effort: 100 (range 1-100, the higher the value, the more thorough the reasoning)\n\n"
    assert out == f"{B}{S}{eff}Be terse.{U}1+1?{A}</think>2{E}{U}2+2?{A}<think>"
    keep = ds.encode(msgs, thinking=True, drop_thinking=False, reasoning_effort="max")
    assert keep == f"{B}{S}{eff}Be terse.{U}1+1?{A}<think>easy</think>2{E}{U}2+2?{A}<think>"
    # continuing a generated assistant turn after the last user turn keeps its reasoning
    cont = msgs[:3]
    out = ds.encode(cont, thinking=True, reasoning_effort="max")
    assert out.endswith(f"{U}1+1?{A}<think>easy</think>2{E}")


def test_tools_calls_and_results():
    tools = [{"type": "function", "function": {"name": "get_weather", "description": "Weather", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}}}}}]
    msgs = [{"role": "user", "content": "Weather?"},
            {"role": "assistant", "content": "", "tool_calls": [
                {"id": "b", "function": {"name": "get_weather", "arguments": "{\"city\": \"Paris\", \"days\": 2}"}},
                {"id": "a", "function": {"name": "ns::lookup", "arguments": {"q": [1, 2.0]}}}]},
            {"role": "tool", "tool_call_id": "a", "content": "A-result"},
            {"role": "tool", "tool_call_id": "b", "content": "B-result"}]
    out = ds.encode(msgs, tools, thinking=False)
    D = ds.DSML
    assert out.startswith(f"{B}{S}\n\n## Tools\n\nYou have access to a set of tools")
    assert '{"name": "get_weather", "description": "Weather", "parameters": {"type": "object", "properties": ' \
           '{"city": {"type": "string"}, "days": {"type": "integer"}}}}' in out
    calls = (f"\n\n<{D} calls>\n<{D} invoke name=\"get_weather\">\n<{D} parameter name=\"city\" string=\"true\">Paris</{D} parameter>\n"
             f"<{D} parameter name=\"days\" string=\"false\">2</{D} parameter>\n</{D} invoke>\n"
             f"<{D} invoke name=\"ns::lookup\">\n<{D} parameter name=\"q\" string=\"false\">[1, 2.0]</{D} parameter>\n</{D} invoke>\n</{D} calls>")
    assert f"{U}Weather?{A}</think>{calls}{E}" in out
    # results are re-ordered to the order of the calls (b first), folded into one user turn
    assert out.endswith(f"{E}{U}<tool_result>B-result</tool_result>\n\n<tool_result>A-result</tool_result>{A}</think>")


def test_images_tasks_and_errors():
    msgs = [{"role": "user", "content": [{"type": "text", "text": "Look"}, {"type": "image_url", "image_url": {"url": "x"}}]}]
    assert ds.encode(msgs, thinking=False) == f"{B}{U}Look\n\n{ds.IMAGE}{A}</think>"
    with pytest.raises(ds.EncodingError):
        ds.encode([{"role": "user", "content": "bad " + ds.IMAGE}], thinking=False)
    q = ds.encode([{"role": "user", "content": "find", "task": "query"}], thinking=False)
    assert q == f"{B}{U}find<｜query｜>"
    a = ds.encode([{"role": "user", "content": "do", "task": "action"}], thinking=False)
    assert a == f"{B}{U}do{A}</think><｜action｜>"
    with pytest.raises(ds.EncodingError):
        ds.encode([{"role": "user", "content": "x", "task": "nope"}], thinking=False)
    with pytest.raises(ds.EncodingError):
        ds.encode([{"role": "narrator", "content": "x"}], thinking=False)
    with pytest.raises(ds.EncodingError):
        ds.encode([{"role": "user", "content": "x"}], [{"function": {"name": "a::b::c"}}], thinking=False)
    assert ds.py_dumps({"a": [1, 2.0, None, True], "ü": "é\n"}) == '{"a": [1, 2.0, null, true], "ü": "é\\n"}'


def test_context_continuation_omits_bos_and_earlier_turns():
    ctx = [{"role": "user", "content": "first"}, {"role": "assistant", "content": "ok"}]
    out = ds.encode([{"role": "user", "content": "second"}], thinking=False, context=ctx)
    assert out == f"{U}second{A}</think>"
