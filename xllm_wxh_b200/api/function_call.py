"""Tool-call detection in generated text, one detector per model family, non-streaming and streaming.

Formats (xllm/function_call/*_detector.cpp in the reference; registry function_call_parser.cpp:60-120):
  qwen25       <tool_call>\\n{"name": ..., "arguments": {...}}\\n</tool_call>
  qwen3_coder  <tool_call><function=NAME><parameter=KEY>VALUE</parameter>...</function></tool_call>
  deepseekv3   <｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>NAME\\n```json\\n{...}\\n```<｜tool▁call▁end｜>...<｜tool▁calls▁end｜>
  kimi_k2      <|tool_calls_section_begin|><|tool_call_begin|>functions.NAME:IDX<|tool_call_argument_begin|>{...}<|tool_call_end|>...
  glm45        <tool_call>NAME\\n<arg_key>K</arg_key>\\n<arg_value>V</arg_value>...</tool_call>
  glm47        the same tags written without line breaks: <tool_call>NAME<arg_key>K</arg_key><arg_value>V</arg_value>...</tool_call>
  deepseekv32  <｜DSML｜function_calls><｜DSML｜invoke name="NAME"><｜DSML｜parameter name="K" string="true|false">V
               </｜DSML｜parameter>...</｜DSML｜invoke>...</｜DSML｜function_calls>   (or a JSON object inside the invoke block)

Streaming: `StreamingToolParser.feed(delta)` returns the text that is certainly not part of a tool call plus tool-call
deltas in OpenAI shape: the first delta of a call carries its index, id and name, later ones carry `arguments` fragments
(the raw JSON as the model writes it for the JSON formats; the assembled JSON object for the tag formats when the call
closes).  Text that may still turn out to be the start of a marker is held back.
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .partial_json import parse_partial


@dataclass
class ToolCall:
    index: int
    name: str
    arguments: str            # JSON text
    id: str = ""


@dataclass
class ToolDelta:
    index: int
    id: Optional[str] = None
    name: Optional[str] = None
    arguments: str = ""


def _call_id() -> str:
    return "call_" + uuid.uuid4().hex[:24]


def _coerce(value: str) -> Any:
    v = value.strip()
    try:
        return json.loads(v)
    except (json.JSONDecodeError, ValueError):
        return value.strip("\n")


class Detector:
    """`bot`: text that opens a tool-call section.  Subclasses parse complete calls out of a section."""
    name = ""
    bot = ""

    def has_tool_call(self, text: str) -> bool:
        return self.bot in text

    def parse(self, text: str) -> Tuple[str, List[ToolCall]]:
        """Whole-message parse: (normal text before the first tool call, calls)."""
        pos = text.find(self.bot)
        if pos < 0:
            return text, []
        calls = [ToolCall(i, n, a, _call_id()) for i, (n, a) in enumerate(self.extract(text[pos:]))]
        return (text[:pos].rstrip() if calls else text), calls

    def extract(self, section: str) -> List[Tuple[str, str]]:
        raise NotImplementedError

    # streaming hooks -------------------------------------------------------------------------------------------------
    def split_open_call(self, section: str) -> Tuple[List[Tuple[str, str]], Optional[Tuple[Optional[str], str]]]:
        """From the text after `bot`: (closed calls, open call as (name or None, raw argument text so far) or None)."""
        raise NotImplementedError


class Qwen25Detector(Detector):
    name, bot = "qwen25", "<tool_call>"
    _block = re.compile(r"<tool_call>\s*([\s\S]*?)\s*</tool_call>")

    def extract(self, section):
        out = []
        for m in self._block.finditer(section):
            try:
                obj = json.loads(m.group(1))
            except json.JSONDecodeError:
                continue
            for call in (obj if isinstance(obj, list) else [obj]):
                if isinstance(call, dict) and "name" in call:
                    args = call.get("arguments", call.get("parameters", {}))
                    out.append((call["name"], args if isinstance(args, str) else json.dumps(args, ensure_ascii=False)))
        return out

    def split_open_call(self, section):
        closed = self.extract(section)
        last_open = section.rfind("<tool_call>")
        last_close = section.rfind("</tool_call>")
        if last_open < 0 or last_close > last_open:
            return closed, None
        body = section[last_open + len("<tool_call>"):].lstrip()
        nm = re.search(r'"name"\s*:\s*"((?:[^"\\]|\\.)*)"', body)        # only a name whose string has closed
        name = json.loads('"' + nm.group(1) + '"') if nm else None
        raw = ""
        m = re.search(r'"arguments"\s*:\s*', body)
        if m and name is not None:
            raw = body[m.end():]
            end = _object_end(raw)          # drop what follows the arguments object (the outer closing brace)
            if end >= 0:
                raw = raw[:end + 1]
        return closed, (name, raw)


class KimiK2Detector(Detector):
    name, bot = "kimi_k2", "<|tool_calls_section_begin|>"
    _call = re.compile(r"<\|tool_call_begin\|>\s*([\w\.\-]+):(\d+)\s*<\|tool_call_argument_begin\|>\s*(\{[\s\S]*?\})\s*<\|tool_call_end\|>")
    _open = re.compile(r"<\|tool_call_begin\|>\s*([\w\.\-]+):(\d+)\s*<\|tool_call_argument_begin\|>\s*([\s\S]*)$")

    @staticmethod
    def _fn(name: str) -> str:
        return name.split(".", 1)[1] if name.startswith("functions.") else name

    def extract(self, section):
        return [(self._fn(m.group(1)), m.group(3)) for m in self._call.finditer(section)]

    def split_open_call(self, section):
        closed = self.extract(section)
        tail = section[section.rfind("<|tool_call_begin|>"):] if "<|tool_call_begin|>" in section else ""
        if not tail or "<|tool_call_end|>" in tail:
            return closed, None
        m = self._open.search(tail)
        if not m:
            return closed, (None, "")
        return closed, (self._fn(m.group(1)), m.group(3))


class DeepSeekV3Detector(Detector):
    name, bot = "deepseekv3", "<｜tool▁calls▁begin｜>"
    _call = re.compile(r"<｜tool▁call▁begin｜>(.*?)<｜tool▁sep｜>(.*?)\n```json\n([\s\S]*?)\n```\s*<｜tool▁call▁end｜>")
    _open = re.compile(r"<｜tool▁call▁begin｜>(.*?)<｜tool▁sep｜>(.*?)\n```json\n([\s\S]*)$")

    def extract(self, section):
        return [(m.group(2).strip(), m.group(3).strip()) for m in self._call.finditer(section)]

    def split_open_call(self, section):
        closed = self.extract(section)
        idx = section.rfind("<｜tool▁call▁begin｜>")
        if idx < 0 or "<｜tool▁call▁end｜>" in section[idx:]:
            return closed, None
        m = self._open.search(section[idx:])
        if not m:
            return closed, (None, "")
        raw = m.group(3)
        cut = raw.find("\n```")
        return closed, (m.group(2).strip(), raw[:cut] if cut >= 0 else raw)


class Glm45Detector(Detector):
    name, bot = "glm45", "<tool_call>"
    _block = re.compile(r"<tool_call>\s*([^\n<]+)\s*([\s\S]*?)</tool_call>")
    _arg = re.compile(r"<arg_key>([\s\S]*?)</arg_key>\s*<arg_value>([\s\S]*?)</arg_value>")

    def extract(self, section):
        out = []
        for m in self._block.finditer(section):
            args = {k.strip(): _coerce(v) for k, v in self._arg.findall(m.group(2))}
            out.append((m.group(1).strip(), json.dumps(args, ensure_ascii=False)))
        return out

    def split_open_call(self, section):
        closed = self.extract(section)
        idx = section.rfind("<tool_call>")
        if idx < 0 or "</tool_call>" in section[idx:]:
            return closed, None
        body = section[idx + len("<tool_call>"):]
        name = body.split("\n", 1)[0].strip() if "\n" in body else None
        return closed, (name or None, "")       # arguments are emitted when the call closes


class Qwen3CoderDetector(Detector):
    name, bot = "qwen3_coder", "<tool_call>"
    _block = re.compile(r"<tool_call>\s*<function=([^>\n]+)>([\s\S]*?)</function>\s*</tool_call>")
    _param = re.compile(r"<parameter=([^>\n]+)>([\s\S]*?)</parameter>")

    def extract(self, section):
        out = []
        for m in self._block.finditer(section):
            args = {k.strip(): _coerce(v) for k, v in self._param.findall(m.group(2))}
            out.append((m.group(1).strip(), json.dumps(args, ensure_ascii=False)))
        return out

    def split_open_call(self, section):
        closed = self.extract(section)
        idx = section.rfind("<tool_call>")
        if idx < 0 or "</tool_call>" in section[idx:]:
            return closed, None
        m = re.search(r"<function=([^>\n]+)>", section[idx:])
        return closed, (m.group(1).strip() if m else None, "")


class Glm47Detector(Detector):
    """GLM-4.7 writes the GLM-4.5 tags compactly: the function name runs up to the first `<arg_key>` (or the closing tag),
    with or without line breaks (glm47_detector.cpp:25-32).  A block without any argument is not a call."""
    name, bot = "glm47", "<tool_call>"
    _block = re.compile(r"<tool_call>([\s\S]*?)</tool_call>")
    _arg = re.compile(r"<arg_key>([\s\S]*?)</arg_key>\s*<arg_value>([\s\S]*?)</arg_value>")

    def has_tool_call(self, text: str) -> bool:
        return "<tool_call>" in text

    @staticmethod
    def _name(body: str) -> str:
        cut = body.find("<arg_key>")
        return (body if cut < 0 else body[:cut]).strip()

    def extract(self, section):
        out = []
        for m in self._block.finditer(section):
            body = m.group(1)
            pairs = self._arg.findall(body)
            name = self._name(body)
            if not pairs or not name:
                continue
            args = {k.strip(): _coerce(v) for k, v in pairs}
            out.append((name, json.dumps(args, ensure_ascii=False)))
        return out

    def split_open_call(self, section):
        closed = self.extract(section)
        idx = section.rfind("<tool_call>")
        if idx < 0 or "</tool_call>" in section[idx:]:
            return closed, None
        body = section[idx + len("<tool_call>"):]
        name = self._name(body) if "<arg_key>" in body else None     # the name is complete once an argument starts
        return closed, (name or None, "")       # arguments are emitted when the call closes


class DeepSeekV32Detector(Detector):
    """DeepSeek-V3.2 "DSML" calls (deepseekv32_detector.cpp:28-66): parameters as tags, `string="true"` keeps the value
    as text and anything else is read as JSON; an invoke block may also hold one JSON object with all arguments."""
    name, bot = "deepseekv32", "<｜DSML｜function_calls>"
    _invoke = re.compile(r'<｜DSML｜invoke\s+name="([^"]+)"\s*>([\s\S]*?)</｜DSML｜invoke>')
    _param = re.compile(r'<｜DSML｜parameter\s+name="([^"]+)"\s+string="([^"]+)"\s*>([\s\S]*?)</｜DSML｜parameter>')
    _open = re.compile(r'<｜DSML｜invoke\s+name="([^"]+)"\s*>')

    def has_tool_call(self, text: str) -> bool:
        return self.bot in text or "<｜DSML｜invoke" in text

    def parse(self, text):
        pos = text.find(self.bot)
        if pos < 0:
            pos = text.find("<｜DSML｜invoke")
        if pos < 0:
            return text, []
        calls = [ToolCall(i, n, a, _call_id()) for i, (n, a) in enumerate(self.extract(text[pos:]))]
        return text[:pos].rstrip(), calls          # an unfinished block is dropped, the text before it stays

    def _arguments(self, body: str) -> Dict[str, Any]:
        stripped = body.strip()
        if stripped.startswith("{"):
            try:
                obj = json.loads(stripped)
                if isinstance(obj, dict):
                    return obj
            except json.JSONDecodeError:
                pass
        args: Dict[str, Any] = {}
        for key, is_string, value in self._param.findall(body):
            if is_string.strip() == "true":
                args[key.strip()] = value
            else:
                v = value.strip()
                try:
                    args[key.strip()] = json.loads(v)
                except (json.JSONDecodeError, ValueError):
                    args[key.strip()] = v
        return args

    def extract(self, section):
        return [(m.group(1).strip(), json.dumps(self._arguments(m.group(2)), ensure_ascii=False))
                for m in self._invoke.finditer(section)]

    def split_open_call(self, section):
        closed = self.extract(section)
        idx = section.rfind("<｜DSML｜invoke")
        if idx < 0 or "</｜DSML｜invoke>" in section[idx:]:
            return closed, None
        m = self._open.search(section[idx:])
        return closed, (m.group(1).strip() if m else None, "")


DETECTORS = {d.name: d for d in (Qwen25Detector, KimiK2Detector, DeepSeekV3Detector, Glm45Detector, Qwen3CoderDetector,
                                 Glm47Detector, DeepSeekV32Detector)}
_ALIASES = {"qwen2": "qwen25", "qwen3": "qwen25", "qwen35": "qwen3_coder", "glm5": "glm47"}
_AUTO = {"qwen2": "qwen25", "qwen3": "qwen25", "qwen3_moe": "qwen25", "deepseek_v3": "deepseekv3", "deepseek_v32": "deepseekv32",
         "kimi_k2": "kimi_k2", "glm4_moe": "glm45"}


def resolve_parser(parser: str, model_type: str = "") -> str:
    """'' -> no parsing; 'auto' -> by model type; aliases as in the reference (function_call_parser.cpp:79-120)."""
    if not parser:
        return ""
    if parser == "auto":
        if model_type not in _AUTO:
            raise ValueError(f"no automatic tool-call parser for model type '{model_type}' (known: {sorted(_AUTO)})")
        return _AUTO[model_type]
    parser = _ALIASES.get(parser, parser)
    if parser not in DETECTORS:
        raise ValueError(f"unsupported tool-call parser '{parser}' (supported: {sorted(DETECTORS)})")
    return parser


def get_detector(parser: str) -> Detector:
    return DETECTORS[resolve_parser(parser)]()


def parse_tool_calls(text: str, parser: str) -> Tuple[str, List[ToolCall]]:
    return get_detector(parser).parse(text)


class StreamingToolParser:
    def __init__(self, parser: str):
        self.det = get_detector(parser)
        self.buf = ""               # everything received and not yet classified
        self.in_section = False
        self.section = ""
        self.n_closed = 0           # calls fully emitted
        self.open_started = False   # name of the currently open call already sent
        self.open_sent = 0          # characters of the open call's raw arguments already sent

    def _safe_prefix(self, text: str) -> int:
        """Length of `text` that cannot be the beginning of the section marker."""
        bot = self.det.bot
        for k in range(min(len(bot) - 1, len(text)), 0, -1):
            if text.endswith(bot[:k]):
                return len(text) - k
        return len(text)

    def feed(self, delta: str) -> Tuple[str, List[ToolDelta]]:
        out_text, deltas = "", []
        if not self.in_section:
            self.buf += delta
            pos = self.buf.find(self.det.bot)
            if pos < 0:
                n = self._safe_prefix(self.buf)
                out_text, self.buf = self.buf[:n], self.buf[n:]
                return out_text, deltas
            out_text = self.buf[:pos].rstrip()
            self.section, self.buf, self.in_section = self.buf[pos:], "", True
        else:
            self.section += delta
        closed, open_call = self.det.split_open_call(self.section)
        # calls that closed since the last feed
        while self.n_closed < len(closed):
            name, args = closed[self.n_closed]
            idx = self.n_closed
            if self.open_started:
                rest = args[self.open_sent:] if args.startswith(args[:self.open_sent]) else args
                if rest:
                    deltas.append(ToolDelta(idx, arguments=rest))
            else:
                deltas.append(ToolDelta(idx, _call_id(), name, ""))
                deltas.append(ToolDelta(idx, arguments=args))
            self.n_closed += 1
            self.open_started, self.open_sent = False, 0
        if open_call is not None:
            name, raw = open_call
            end = _object_end(raw)              # the arguments value is complete: what follows is closing markup
            if end >= 0:
                raw = raw[:end + 1]
            idx = self.n_closed
            if name and not self.open_started:
                deltas.append(ToolDelta(idx, _call_id(), name, ""))
                self.open_started = True
            if self.open_started and len(raw) > self.open_sent:
                # hold back a trailing fragment that could belong to the closing markers
                safe = raw.rstrip()
                safe = safe[:-1] if safe.endswith("}") and not _balanced(safe) else safe
                if len(safe) > self.open_sent:
                    deltas.append(ToolDelta(idx, arguments=safe[self.open_sent:]))
                    self.open_sent = len(safe)
        return out_text, deltas

    def flush(self) -> str:
        """End of generation: text that was held back and never became a marker."""
        t, self.buf = self.buf, ""
        return t


def _object_end(s: str) -> int:
    """Index of the brace / bracket that closes the first top-level JSON value of `s`, or -1 while it is still open."""
    depth, in_str, esc = 0, False, False
    for i, ch in enumerate(s):
        if in_str:
            if esc:
                esc = False
            elif ch == "\\":
                esc = True
            elif ch == '"':
                in_str = False
            continue
        if ch == '"':
            in_str = True
        elif ch in "{[":
            depth += 1
        elif ch in "}]":
            depth -= 1
            if depth == 0:
                return i
    return -1


def _balanced(s: str) -> bool:
    depth, in_str, esc = 0, False, False
    for ch in s:
        if in_str:
            if esc:
                esc = False
            elif ch == "\\":
                esc = True
            elif ch == '"':
                in_str = False
            continue
        if ch == '"':
            in_str = True
        elif ch in "{[":
            depth += 1
        elif ch in "}]":
            depth -= 1
    return depth == 0 and not in_str
