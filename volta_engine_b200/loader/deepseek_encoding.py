"""Built-in prompt format of the DeepSeek V4-style models (no Jinja template): system / user / assistant turns,
thinking mode with reasoning effort, tool schemas and tool calls in DSML markup, tool results folded into user
turns, image placeholders.

Behaviour follows the reference's statement of the model vendor's ``encoding.py`` (src/loader/deepseek_encoding.cpp:
message merging :214-246, tool-result ordering :248-274, image blocks :276-318, effort line :336-351, per-message
rendering :353-446, thinking removal :448-461, conversation assembly :463-483).
"""
from __future__ import annotations

import copy
import json

BOS = "<｜begin▁of▁sentence｜>"
EOS = "<｜end▁of▁sentence｜>"
THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
DSML = "｜DSML｜"
USER, ASSISTANT, SYSTEM = "<｜User｜>", "<｜Assistant｜>", "<｜System｜>"
REMINDER = "<｜latest_reminder｜>"
IMAGE = "<｜deepseek_image｜>"
TASK_TOKENS = {t: f"<｜{t}｜>" for t in ("action", "query", "authority", "domain", "title", "read_url")}
_CALLS, _INVOKE, _PARAM = DSML + " calls", DSML + " invoke", DSML + " parameter"


class EncodingError(ValueError):
    pass


def py_dumps(v) -> str:
    """``json.dumps(v, ensure_ascii=False)`` with Python's default separators."""
    return json.dumps(v, ensure_ascii=False)


def _truthy(m, key) -> bool:
    return isinstance(m, dict) and bool(m.get(key))


def _s(m, key, default="") -> str:
    v = m.get(key) if isinstance(m, dict) else None
    return v if isinstance(v, str) else default


def _namespace_name(ns):
    if isinstance(ns, str):
        return ns
    if isinstance(ns, dict) and isinstance(ns.get("name"), str):
        return ns["name"]
    return None


def _split_name(name: str, ns):
    if "::" in name:
        prefix, name = name.split("::", 1)
        if ns is not None and ns != prefix:
            raise EncodingError(f"Conflicting tool namespaces: {ns} != {prefix}")
        ns = prefix
    if "::" in name:
        raise EncodingError(f"Tool name must not contain '::': {name}")
    if ns is not None and "::" in ns:
        raise EncodingError(f"Tool namespace must not contain '::': {ns}")
    return ns, name


def _qualified(tool: dict) -> str:
    ns = _namespace_name(tool["namespace"]) if tool.get("namespace") is not None else None
    ns, name = _split_name(_s(tool, "name"), ns)
    return f"{ns}::{name}" if ns else name


def _functions(tools: list) -> list:
    out = []
    for tool in tools:
        fn = dict(tool["function"]) if isinstance(tool.get("function"), dict) else dict(tool)
        if tool.get("namespace") is not None:
            fn["namespace"] = tool["namespace"]
        fn["name"] = _qualified(fn)
        ns = fn.pop("namespace", None)
        if isinstance(ns, dict) and ns.get("description"):
            fn["description"] = _s(ns, "description") + "\n" + _s(fn, "description")
        out.append(fn)
    return out


def _calls(tool_calls: list) -> list:
    out = []
    for tc in tool_calls:
        fn = tc["function"] if isinstance(tc.get("function"), dict) else {}
        ns = None
        if tc.get("namespace") is not None:
            ns = _namespace_name(tc["namespace"])
        elif fn.get("namespace") is not None:
            ns = _namespace_name(fn["namespace"])
        ns, name = _split_name(_s(fn, "name"), ns)
        call = {"name": name, "arguments": fn.get("arguments")}
        if ns:
            call["namespace"] = ns
        out.append(call)
    return out


def render_tools(functions: list) -> str:
    schemas = "\n".join(py_dumps(f) for f in functions)
    return (
        "## Tools\n\nYou have access to a set of tools to help answer the user's question. You can invoke tools by "
        f"writing a \"<{_CALLS}>\" block like the following:\n\n"
        f"<{_CALLS}>\n<{_INVOKE} name=\"$TOOL_NAME\">\n<{_PARAM} name=\"$PARAMETER_NAME\" string=\"true|false\">"
        f"$PARAMETER_VALUE</{_PARAM}>\n...\n</{_INVOKE}>\n<{_INVOKE} name=\"$TOOL_NAME2\">\n...\n</{_INVOKE}>\n</{_CALLS}>\n\n"
        "String parameters should be specified as is and set `string=\"true\"`. For all other types (numbers, booleans, "
        "arrays, objects), pass the value in JSON format and set `string=\"false\"`.\n\n"
        f"If thinking_mode is enabled (triggered by {THINK_OPEN}), you MUST output your complete reasoning inside "
        f"{THINK_OPEN}...{THINK_CLOSE} BEFORE any tool calls or final response.\n\n"
        f"Otherwise, output directly after {THINK_CLOSE} with tool calls or final response.\n\n"
        f"### Available Tool Schemas\n\n{schemas}\n\n"
        "You MUST strictly follow the above defined tool name and parameter schemas to invoke tool calls.\n")


def _arguments_dsml(call: dict) -> str:
    args = call.get("arguments")
    if not isinstance(args, dict):
        for _ in range(2):                      # arguments may arrive as (doubly) encoded JSON text
            if not isinstance(args, str):
                break
            try:
                args = json.loads(args)
            except ValueError:
                break
        if not isinstance(args, dict):
            args = {"arguments": call.get("arguments")}
    parts = []
    for k, v in args.items():
        is_str = isinstance(v, str)
        parts.append(f"<{_PARAM} name=\"{k}\" string=\"{'true' if is_str else 'false'}\">{v if is_str else py_dumps(v)}</{_PARAM}>")
    return "\n".join(parts)


def merge_tool_messages(messages: list) -> list:
    """Tool messages become ``tool_result`` blocks of a user turn; adjacent user turns merge."""
    merged: list = []
    for msg in messages:
        msg = copy.deepcopy(msg)
        role = _s(msg, "role")
        last = merged[-1] if merged else None
        if role == "tool":
            content = msg.get("content", "")
            if msg.get("content_blocks") and not isinstance(msg.get("content"), str):
                content = msg["content_blocks"]
            block = {"type": "tool_result", "tool_use_id": _s(msg, "tool_call_id"), "content": content}
            if last is not None and _s(last, "role") == "user" and "content_blocks" in last:
                last["content_blocks"].append(block)
            else:
                merged.append({"role": "user", "content_blocks": [block]})
        elif role == "user":
            if msg.get("content_blocks") is not None:
                blocks = msg["content_blocks"]
            else:
                c = msg.get("content", "")
                blocks = c if isinstance(c, list) else [{"type": "text", "text": c if isinstance(c, str) else ""}]
            if last is not None and _s(last, "role") == "user" and "content_blocks" in last and "task" not in last:
                last["content_blocks"].extend(blocks)
            else:
                msg["content_blocks"] = blocks
                merged.append(msg)
        else:
            merged.append(msg)
    return merged


def order_tool_results(messages: list) -> None:
    """Inside each user turn, tool results follow the order of the calls in the assistant turn before it."""
    order: dict = {}
    for msg in messages:
        role = _s(msg, "role")
        if role == "assistant" and msg.get("tool_calls"):
            order = {}
            for i, tc in enumerate(msg["tool_calls"]):
                cid = _s(tc, "id") or _s(tc.get("function") or {}, "id")
                if cid:
                    order[cid] = i
        elif role == "user" and msg.get("content_blocks"):
            results = [b for b in msg["content_blocks"] if _s(b, "type") == "tool_result"]
            if len(results) > 1 and order:
                results.sort(key=lambda b: order.get(_s(b, "tool_use_id"), 0))
                it = iter(results)
                msg["content_blocks"] = [next(it) if _s(b, "type") == "tool_result" else b for b in msg["content_blocks"]]


def _image_blocks(blocks: list) -> list:
    out = []
    for b in blocks:
        if not isinstance(b, dict):
            out.append(b)
            continue
        t = _s(b, "type")
        if t in ("image", "image_url"):
            out.append({"type": "text", "text": IMAGE})
        elif t == "tool_result" and isinstance(b.get("content"), list):
            out.append(dict(b, content=_image_blocks(b["content"])))
        else:
            if t == "text" and IMAGE in _s(b, "text"):
                raise EncodingError("Text block contains image placeholder")
            out.append(b)
    return out


def _image_messages(messages: list) -> list:
    out = []
    for msg in messages:
        msg = dict(msg)
        if isinstance(msg.get("content"), str) and IMAGE in msg["content"]:
            raise EncodingError("Message content contains the image special token")
        if IMAGE in _s(msg, "reasoning_content"):
            raise EncodingError("reasoning_content contains the image special token")
        if isinstance(msg.get("content"), list) and "content_blocks" not in msg:
            msg["content_blocks"] = msg.pop("content")
        if msg.get("content_blocks"):
            msg["content_blocks"] = _image_blocks(msg["content_blocks"])
            if not isinstance(msg.get("content"), str):
                msg["content"] = "\n\n".join(_s(b, "text") for b in msg["content_blocks"]
                                             if isinstance(b, dict) and _s(b, "type") == "text")
        out.append(msg)
    return out


def _last_user_index(messages: list) -> int:
    for i in range(len(messages) - 1, -1, -1):
        m = messages[i]
        role = _s(m, "role")
        if role == "user" or (role == "system" and i > 0):
            if m.get("content_blocks") and not any(_s(b, "type") in ("text", "image", "image_url") for b in m["content_blocks"]):
                continue
            return i
    return -1


def _effort_line(index: int, thinking: bool, effort: str) -> str:
    effort = effort or "high"
    named = {"low": 50, "high": 75, "max": 100}
    if effort in named:
        budget = named[effort]
    else:
        try:
            budget = int(effort)
        except ValueError:
            budget = 0
        if not 1 <= budget <= 100 or str(budget) != effort.lstrip("+"):
            raise EncodingError(f"Invalid reasoning effort for deepseek_v41: {effort}, should be int within [1,100] or low / high / max")
    if index == 0 and thinking:
        return f"Reasoning Effort: {budget} (range 1-100, the higher the value, the more thorough the reasoning)\n\n"
    return ""


def _render(index: int, messages: list, thinking: bool, drop_thinking: bool, effort: str) -> str:
    msg = messages[index]
    last_user = _last_user_index(messages)
    role = _s(msg, "role")
    content = msg["content"] if isinstance(msg.get("content"), str) else ""
    tools = _functions(msg["tools"]) if msg.get("tools") else None
    calls = _calls(msg["tool_calls"]) if msg.get("tool_calls") else None
    eff = _effort_line(index, thinking, effort)
    out = SYSTEM if index == 0 and (eff or role == "system") else ""
    out += eff
    if role == "system":
        if index > 0:
            out += SYSTEM
        out += content
        if tools is not None:
            out += "\n\n" + render_tools(tools)
        if msg.get("response_format"):
            out += ("\n\n## Response Format:\n\nYou MUST strictly adhere to the following schema to reply:\n" +
                    py_dumps(msg["response_format"]))
    elif role == "user":
        out += USER
        if msg.get("content_blocks"):
            parts = []
            for b in msg["content_blocks"]:
                t = _s(b, "type")
                if t == "text":
                    parts.append(_s(b, "text"))
                elif t == "tool_result":
                    c = b.get("content")
                    if isinstance(c, list):
                        c = "\n\n".join(_s(x, "text") if _s(x, "type") == "text" else f"[Unsupported {_s(x, 'type')}]" for x in c)
                    elif not isinstance(c, str):
                        c = ""
                    parts.append(f"<tool_result>{c}</tool_result>")
                else:
                    parts.append(f"[Unsupported {t}]")
            out += "\n\n".join(parts)
        else:
            out += content
    elif role == "latest_reminder":
        out += REMINDER + content
    elif role == "assistant":
        tc = ""
        if calls is not None:
            items = "\n".join(f"<{_INVOKE} name=\"{_qualified(c)}\">\n{_arguments_dsml(c)}\n</{_INVOKE}>" for c in calls)
            tc = f"\n\n<{_CALLS}>\n{items}\n</{_CALLS}>"
        prev_task = index >= 1 and messages[index - 1].get("task") is not None
        think = ""
        if thinking and not prev_task and (not drop_thinking or index > last_user):
            think = _s(msg, "reasoning_content") + THINK_CLOSE
        out += think + content + tc
        if not msg.get("wo_eos"):
            out += EOS
    elif role == "tool":
        raise EncodingError("tool messages must be merged first")
    else:
        raise EncodingError(f"Unknown role: {role}")

    if index + 1 < len(messages) and _s(messages[index + 1], "role") not in ("assistant", "latest_reminder"):
        return out
    if msg.get("task") is not None:
        task = _s(msg, "task")
        if task not in TASK_TOKENS:
            raise EncodingError(f"Invalid task: {task}")
        out += TASK_TOKENS[task] if task != "action" else ASSISTANT + (THINK_OPEN if thinking else THINK_CLOSE) + TASK_TOKENS[task]
    elif role == "user" or (role == "system" and index > 0):
        out += ASSISTANT
        if thinking and (not drop_thinking or index >= last_user):
            out += THINK_OPEN
        else:
            out += THINK_CLOSE
    return out


def _without_old_thinking(messages: list) -> list:
    last_user = _last_user_index(messages)
    out = []
    for i, m in enumerate(messages):
        role = _s(m, "role")
        if role in ("user", "system", "tool", "latest_reminder", "direct_search_results") or i >= last_user:
            out.append(m)
        elif role == "assistant":
            out.append({k: v for k, v in m.items() if k != "reasoning_content"})
    return out


def encode(messages: list, tools: list | None = None, *, thinking: bool = True, drop_thinking: bool = True,
           add_bos: bool = True, reasoning_effort: str = "", context: list | None = None) -> str:
    """Conversation -> prompt text that ends where the model continues."""
    messages, context = copy.deepcopy(messages), copy.deepcopy(context or [])
    if tools:
        host = context if context else messages
        if not host or _s(host[0], "role") != "system":
            host.insert(0, {"role": "system", "content": ""})
        host[0]["tools"] = tools
    ctx, msgs = merge_tool_messages(context), merge_tool_messages(messages)
    both = ctx + msgs
    order_tool_results(both)
    msgs = _image_messages(both[len(ctx):])
    ctx = _image_messages(ctx) if ctx else []
    full = ctx + msgs
    prompt = BOS if add_bos and not ctx else ""
    drop = drop_thinking and not any(m.get("tools") for m in full)
    if thinking and drop:
        full = _without_old_thinking(full)
        n = len(full) - len(_without_old_thinking(ctx))
    else:
        n = len(msgs)
    start = len(full) - n
    return prompt + "".join(_render(start + i, full, thinking, drop, reasoning_effort) for i in range(n))
