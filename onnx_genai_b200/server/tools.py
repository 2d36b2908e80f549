"""Tool calling glue: prompt injection of tool schemas and parsing of ``<tool_call>`` blocks.

Behaviour of the reference's `parse_tool_calls` (crates/onnx-genai-server/src/routes/
completions.rs:1896): the model emits ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>``
(Hermes / Qwen convention); each well-formed block becomes an OpenAI ``tool_calls`` entry, and
malformed JSON is left in the text.
"""
from __future__ import annotations

import json
import re
import uuid

_BLOCK = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)


def inject_tool_prompt(messages, tools, tool_choice=None):
    desc = "\n".join(json.dumps(t.get("function", t), ensure_ascii=False) for t in tools)
    rule = ("You may call one or more functions. For each call return a JSON object with the function name and arguments "
            'inside <tool_call></tool_call> tags: <tool_call>{"name": <function-name>, "arguments": <args-json-object>}</tool_call>')
    if tool_choice == "required":
        rule += "\nYou MUST call at least one function."
    elif isinstance(tool_choice, dict) and tool_choice.get("function", {}).get("name"):
        rule += f"\nYou MUST call the function {tool_choice['function']['name']!r}."
    sys_msg = {"role": "system", "content": f"# Tools\n<tools>\n{desc}\n</tools>\n{rule}"}
    return [sys_msg] + list(messages)


def parse_tool_calls(text: str) -> list:
    calls = []
    for m in _BLOCK.finditer(text or ""):
        try:
            obj = json.loads(m.group(1))
        except json.JSONDecodeError:
            continue
        name = obj.get("name")
        if not isinstance(name, str):
            continue
        args = obj.get("arguments", {})
        calls.append({"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
                      "function": {"name": name, "arguments": args if isinstance(args, str) else json.dumps(args, ensure_ascii=False)}})
    return calls
