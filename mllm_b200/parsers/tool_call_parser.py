"""Extract tool calls from model output (formats of pymllm/parsers/tool_call_parser.py:39-433):

* ``qwen25`` / ``hermes`` — ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>``
* ``llama3`` — ``<|python_tag|>{"name": ..., "parameters": {...}}`` (calls separated by ``;``)
* ``qwen3_coder`` — ``<tool_call><function=NAME><parameter=KEY>VALUE</parameter>...</function></tool_call>``

``parse_non_stream`` returns (plain text, calls).  ``parse_stream_chunk`` returns (plain text delta,
call deltas): the first delta of a call carries its name with empty arguments, later deltas carry
argument text as it arrives, in the OpenAI streaming shape.
"""

from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class ToolCallItem:
    tool_index: int
    name: Optional[str] = None
    parameters: str = ""  # JSON text (whole, or a fragment when streaming)
    call_id: str = field(default_factory=lambda: f"call_{uuid.uuid4().hex[:24]}")

    def to_openai_dict(self, streaming: bool = True) -> Dict[str, Any]:
        fn: Dict[str, Any] = {"arguments": self.parameters}
        if self.name is not None:
            fn["name"] = self.name
        d: Dict[str, Any] = {"type": "function", "function": fn}
        if streaming:
            d["index"] = self.tool_index
            if self.name is not None:
                d["id"] = self.call_id
        else:
            d["id"] = self.call_id
        return d


@dataclass(frozen=True)
class _Format:
    bot: str
    eot: str
    args_key: str
    style: str  # "json" | "xml"


FORMATS: Dict[str, _Format] = {
    "qwen25": _Format("<tool_call>", "</tool_call>", "arguments", "json"),
    "qwen": _Format("<tool_call>", "</tool_call>", "arguments", "json"),
    "hermes": _Format("<tool_call>", "</tool_call>", "arguments", "json"),
    "llama3": _Format("<|python_tag|>", "", "parameters", "json"),
    "qwen3_coder": _Format("<tool_call>", "</tool_call>", "arguments", "xml"),
}

_FN_RE = re.compile(r"<function=([^>\s]+)>(.*?)(?:</function>|$)", re.S)
_PARAM_RE = re.compile(r"<parameter=([^>\s]+)>(.*?)(?:</parameter>|(?=<parameter=)|$)", re.S)


def _coerce(v: str) -> Any:
    t = v.strip()
    try:
        return json.loads(t)
    except (ValueError, TypeError):
        return t


def _json_value_prefix(text: str) -> str:
    """The part of ``text`` that belongs to the JSON value starting at its first character: all of
    it while the value is still open, up to its closing bracket / quote once it has closed."""
    if not text:
        return ""
    depth, in_str, esc = 0, False, False
    opener = text[0]
    for i, ch in enumerate(text):
        if in_str:
            if esc:
                esc = False
            elif ch == "\\":
                esc = True
            elif ch == '"':
                in_str = False
                if depth == 0:
                    return text[: i + 1]
            continue
        if ch == '"':
            in_str = True
        elif ch in "{[":
            depth += 1
        elif ch in "}]":
            depth -= 1
            if depth == 0:
                return text[: i + 1]
            if depth < 0:  # a scalar value ended at the enclosing object's brace
                return text[:i].rstrip()
        elif ch == "," and depth == 0 and opener not in '{["':
            return text[:i].rstrip()
    return text if opener in '{["' else ""


class ToolCallParser:
    def __init__(self, model_type: str, tools: Optional[List[Any]] = None) -> None:
        if model_type not in FORMATS:
            raise ValueError(f"unknown tool-call parser {model_type!r}; have {sorted(FORMATS)}")
        self.fmt = FORMATS[model_type]
        self.tools = tools or []
        self._buf = ""
        self._in_call = False
        self._index = -1
        self._name_sent = False
        self._args_sent = 0

    def has_tool_call(self, text: str) -> bool:
        return self.fmt.bot in text

    # ------------------------------------------------------------------ whole strings
    def _parse_body(self, body: str, index: int) -> Optional[ToolCallItem]:
        body = body.strip()
        if not body:
            return None
        if self.fmt.style == "xml":
            m = _FN_RE.search(body)
            if not m:
                return None
            args = {k: _coerce(v) for k, v in _PARAM_RE.findall(m.group(2))}
            return ToolCallItem(index, m.group(1), json.dumps(args, ensure_ascii=False))
        try:
            obj = json.loads(body)
        except ValueError:
            return None
        if not isinstance(obj, dict) or "name" not in obj:
            return None
        args = obj.get(self.fmt.args_key, obj.get("arguments", obj.get("parameters", {})))
        return ToolCallItem(index, obj["name"], args if isinstance(args, str) else json.dumps(args, ensure_ascii=False))

    def parse_non_stream(self, text: str) -> Tuple[str, List[ToolCallItem]]:
        f = self.fmt
        if f.bot not in text:
            return text, []
        calls: List[ToolCallItem] = []
        plain = []
        rest = text
        while f.bot in rest:
            before, _, after = rest.partition(f.bot)
            plain.append(before)
            if f.eot:
                body, sep, rest = after.partition(f.eot)
                if not sep:
                    rest = ""
                bodies = [body]
            else:
                bodies, rest = [b for b in after.split(";")], ""
            for b in bodies:
                item = self._parse_body(b, len(calls))
                if item is not None:
                    calls.append(item)
        plain.append(rest)
        return "".join(plain).strip(), calls

    # ------------------------------------------------------------------ streams
    def parse_stream_chunk(self, delta: str) -> Tuple[str, List[ToolCallItem]]:
        f = self.fmt
        self._buf += delta
        text_out = ""
        items: List[ToolCallItem] = []
        while True:
            if not self._in_call:
                idx = self._buf.find(f.bot)
                if idx < 0:
                    keep = 0
                    for n in range(min(len(f.bot) - 1, len(self._buf)), 0, -1):
                        if f.bot.startswith(self._buf[-n:]):
                            keep = n
                            break
                    text_out += self._buf[: len(self._buf) - keep]
                    self._buf = self._buf[len(self._buf) - keep:]
                    break
                text_out += self._buf[:idx]
                self._buf = self._buf[idx + len(f.bot):]
                self._in_call, self._name_sent, self._args_sent = True, False, 0
                self._index += 1
                continue
            end = self._buf.find(f.eot) if f.eot else -1
            body = self._buf if end < 0 else self._buf[:end]
            items.extend(self._stream_body(body, closed=end >= 0))
            if end < 0:
                break
            self._buf = self._buf[end + len(f.eot):]
            self._in_call = False
        return text_out, items

    def _stream_body(self, body: str, closed: bool) -> List[ToolCallItem]:
        out: List[ToolCallItem] = []
        if self.fmt.style == "xml":
            if closed:
                item = self._parse_body(body, self._index)
                if item is not None:
                    if self._name_sent:
                        item = ToolCallItem(self._index, None, item.parameters[self._args_sent:])
                    out.append(item)
            elif not self._name_sent:
                m = re.search(r"<function=([^>\s]+)>", body)
                if m:
                    self._name_sent = True
                    out.append(ToolCallItem(self._index, m.group(1), ""))
            return out
        if not self._name_sent:
            m = re.search(r'"name"\s*:\s*"([^"]+)"', body)
            if m:
                self._name_sent = True
                out.append(ToolCallItem(self._index, m.group(1), ""))
        if self._name_sent:
            m = re.search(r'"(?:%s|arguments|parameters)"\s*:\s*' % re.escape(self.fmt.args_key), body)
            if m:
                args = _json_value_prefix(body[m.end():])
                if len(args) > self._args_sent:
                    out.append(ToolCallItem(self._index, None, args[self._args_sent:]))
                    self._args_sent = len(args)
        return out

    def flush(self) -> List[ToolCallItem]:
        """End of stream: emit what a format without a closing tag still holds."""
        if self._in_call and not self.fmt.eot:
            items = self._stream_body(self._buf, closed=True)
            self._buf, self._in_call = "", False
            return items
        return []
