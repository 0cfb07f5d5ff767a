"""Parse the model's tool-call markup back into OpenAI ``tool_calls``.

Two markups are understood, chosen by content (reference: src/tools.rs:1-215):

* qwen: ``<tool_call><function=NAME><parameter=KEY>VALUE</parameter>...</function></tool_call>``
* hy3:  ``<tool_call:opensource>NAME<tool_sep:opensource><arg_key:opensource>K</arg_key:opensource>
  <arg_value:opensource>V</arg_value:opensource>...</tool_call:opensource>``

Every value arrives as text and is coerced to the type the tool's JSON schema declares (integer, number,
boolean, object, array), falling back to the string. A call without its closing tag (generation hit the
token budget) is dropped, never half-parsed. Call ids come from a process-wide counter so they stay
unique across the turns of an agent loop.
"""
from __future__ import annotations

import itertools
import json
import re
import threading
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

_seq = itertools.count()
_seq_lock = threading.Lock()

CALL_OPEN, CALL_CLOSE = "<tool_call>", "</tool_call>"
HY_OPEN, HY_CLOSE = "<tool_call:opensource>", "</tool_call:opensource>"
HY_WRAP_OPEN, HY_WRAP_CLOSE = "<tool_calls:opensource>", "</tool_calls:opensource>"
HY_SEP = "<tool_sep:opensource>"
_HY_ARG = re.compile(r"<arg_key:opensource>(.*?)</arg_key:opensource>\s*<arg_value:opensource>(.*?)</arg_value:opensource>",
                     re.S)
_FN = re.compile(r"<function=([^>\n]+)>(.*?)</function>", re.S)
_PARAM = re.compile(r"<parameter=([^>\n]+)>\n?(.*?)\n?</parameter>", re.S)


@dataclass
class ToolCall:
    id: str
    name: str
    arguments: str            # JSON text

    def to_openai(self, index: Optional[int] = None) -> dict:
        d = {"id": self.id, "type": "function", "function": {"name": self.name, "arguments": self.arguments}}
        if index is not None:
            d["index"] = index
        return d


@dataclass
class ParsedOutput:
    content: str
    tool_calls: List[ToolCall] = field(default_factory=list)


def next_call_id() -> str:
    with _seq_lock:
        return f"call_{next(_seq)}"


def has_tool_call(text: str) -> bool:
    """True once the text contains the start of a call (shared prefix of both markups)."""
    return "<tool_call" in text


def _schema_for(tools: Optional[List[dict]], name: str) -> Dict[str, dict]:
    for t in tools or []:
        fn = t.get("function", t)
        if fn.get("name") == name:
            return (fn.get("parameters") or {}).get("properties") or {}
    return {}


def coerce(value: str, schema: Optional[dict]) -> Any:
    ty = (schema or {}).get("type")
    if isinstance(ty, list):
        ty = next((t for t in ty if t != "null"), None)
    v = value.strip()
    try:
        if ty == "integer":
            return int(v)
        if ty == "number":
            f = float(v)
            return int(f) if f.is_integer() and "." not in v and "e" not in v.lower() else f
        if ty == "boolean":
            if v.lower() in ("true", "false"):
                return v.lower() == "true"
        if ty in ("object", "array"):
            parsed = json.loads(v)
            if (ty == "object" and isinstance(parsed, dict)) or (ty == "array" and isinstance(parsed, list)):
                return parsed
    except (ValueError, json.JSONDecodeError):
        pass
    return value


def _make_call(name: str, pairs: List[Tuple[str, str]], tools) -> ToolCall:
    props = _schema_for(tools, name)
    args = {k: coerce(v, props.get(k)) for k, v in pairs}
    return ToolCall(next_call_id(), name, json.dumps(args, ensure_ascii=False))


def parse(text: str, tools: Optional[List[dict]] = None) -> ParsedOutput:
    """Split a finished generation into prose and calls."""
    if HY_OPEN in text:
        return _parse_hy(text, tools)
    calls: List[ToolCall] = []
    prose: List[str] = []
    i = 0
    while True:
        o = text.find(CALL_OPEN, i)
        if o < 0:
            prose.append(text[i:])
            break
        prose.append(text[i:o])
        c = text.find(CALL_CLOSE, o)
        if c < 0:
            break                       # truncated call: drop it and everything after
        body = text[o + len(CALL_OPEN):c]
        m = _FN.search(body)
        if m:
            pairs = [(k.strip(), v) for k, v in _PARAM.findall(m.group(2))]
            calls.append(_make_call(m.group(1).strip(), pairs, tools))
        i = c + len(CALL_CLOSE)
    return ParsedOutput("".join(prose).strip(), calls)


def _parse_hy(text: str, tools) -> ParsedOutput:
    calls: List[ToolCall] = []
    prose: List[str] = []
    i = 0
    while True:
        o = text.find(HY_OPEN, i)
        if o < 0:
            prose.append(text[i:])
            break
        prose.append(text[i:o])
        c = text.find(HY_CLOSE, o)
        if c < 0:
            break
        body = text[o + len(HY_OPEN):c]
        name, _, rest = body.partition(HY_SEP)
        pairs = [(k.strip(), v.strip()) for k, v in _HY_ARG.findall(rest)]
        calls.append(_make_call(name.strip(), pairs, tools))
        i = c + len(HY_CLOSE)
    content = "".join(prose).replace(HY_WRAP_OPEN, "").replace(HY_WRAP_CLOSE, "").strip()
    return ParsedOutput(content, calls)
