"""Turn tool-call text emitted by the model into OpenAI `tool_calls` objects.

Supported layouts: Hermes-2-Pro / Qwen `<tool_call>{json}</tool_call>` blocks, bare JSON objects with
`name` + `arguments`, and `[TOOL_CALLS] [...]` arrays (reference: src/v2/utils/ToolCallParser.cpp,
src/v2/utils/ToolCallTypes.h); and the tagged layout that the reference's own Qwen3.5 chat template writes for past
calls (jinja/qwen/qwen35/template.jinja), which a model trained on that template emits:
`<tool_call><function=NAME><parameter=KEY>VALUE</parameter>...</function></tool_call>`.
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field

_BLOCK = re.compile(r"<tool_call>\s*(.*?)\s*</tool_call>", re.S)
_FUNCTION = re.compile(r"<function=([^>\s]+)>\s*(.*?)\s*</function>", re.S)
_PARAMETER = re.compile(r"<parameter=([^>\s]+)>\n?(.*?)\n?</parameter>", re.S)


def _tagged_calls(payload: str) -> list[dict]:
    """`<function=name><parameter=key>value</parameter>...</function>` -> name / arguments objects.  A value that reads
    as JSON (number, boolean, null, object, array) keeps its type; anything else is a string."""
    out = []
    for m in _FUNCTION.finditer(payload):
        args = {}
        for pm in _PARAMETER.finditer(m.group(2)):
            raw = pm.group(2)
            try:
                val = json.loads(raw)
                if isinstance(val, str):
                    val = raw
            except json.JSONDecodeError:
                val = raw
            args[pm.group(1)] = val
        out.append({"name": m.group(1), "arguments": args})
    return out


@dataclass
class ToolCallParse:
    content: str
    tool_calls: list[dict] = field(default_factory=list)

    @property
    def has_tool_calls(self) -> bool:
        return bool(self.tool_calls)


def _to_openai(obj: dict) -> dict | None:
    if not isinstance(obj, dict) or "name" not in obj:
        return None
    args = obj.get("arguments", obj.get("parameters", {}))
    if not isinstance(args, str):
        args = json.dumps(args, ensure_ascii=False)
    return {"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
            "function": {"name": str(obj["name"]), "arguments": args}}


def parse_tool_calls(text: str) -> ToolCallParse:
    calls: list[dict] = []
    rest = text

    def take(payload: str) -> bool:
        try:
            obj = json.loads(payload)
        except json.JSONDecodeError:
            obj = _tagged_calls(payload)
            if not obj:
                return False
        items = obj if isinstance(obj, list) else [obj]
        got = [c for c in (_to_openai(o) for o in items) if c]
        calls.extend(got)
        return bool(got)

    if _BLOCK.search(text):
        kept = []
        pos = 0
        for m in _BLOCK.finditer(text):
            kept.append(text[pos:m.start()])
            if not take(m.group(1)):
                kept.append(m.group(0))
            pos = m.end()
        kept.append(text[pos:])
        rest = "".join(kept)
    elif "[TOOL_CALLS]" in text:
        head, _, tail = text.partition("[TOOL_CALLS]")
        if take(tail.strip()):
            rest = head
    else:
        s = text.strip()
        if s.startswith("{") and s.endswith("}") and take(s):
            rest = ""
    return ToolCallParse(rest.strip() if calls else text, calls)
