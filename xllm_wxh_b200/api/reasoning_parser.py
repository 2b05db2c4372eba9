"""Splits generated text into reasoning ("thinking") content and answer content.

Registry as in the reference (xllm/parser/detector_registry.cpp:45-66, reasoning_detector.cpp): per parser name a start
tag, an end tag and whether generation starts inside the reasoning block without an explicit start tag
(`force_reasoning`: deepseek-r1, qwen3-thinking).  Streaming keeps back text that may be a partial tag."""
from __future__ import annotations

from typing import Optional, Tuple

_PARSERS = {
    "deepseek-r1": ("<think>", "</think>", True),
    "deepseek-v3": ("<think>", "</think>", False),
    "glm45": ("<think>", "</think>", False),
    "glm47": ("<think>", "</think>", False),
    "kimi": ("◁think▷", "◁/think▷", False),
    "qwen3": ("<think>", "</think>", False),
    "qwen35": ("<think>", "</think>", False),
    "qwen3-thinking": ("<think>", "</think>", True),
    "step3": ("<think>", "</think>", False),
}
_AUTO = {"glm4_moe": "glm45", "deepseek_v32": "deepseek-v3", "kimi_k2": "kimi", "qwen3": "qwen3", "qwen3_moe": "qwen3",
         "deepseek_v3": "deepseek-v3"}


def resolve_reasoning_parser(name: str, model_type: str = "") -> str:
    if not name:
        return ""
    if name == "auto":
        if model_type not in _AUTO:
            raise ValueError(f"no automatic reasoning parser for model type '{model_type}'")
        return _AUTO[model_type]
    if name not in _PARSERS:
        raise ValueError(f"unsupported reasoning parser '{name}' (supported: {sorted(_PARSERS)})")
    return name


class ReasoningParser:
    def __init__(self, name: str, force_reasoning: Optional[bool] = None):
        self.start, self.end, default_force = _PARSERS[resolve_reasoning_parser(name)]
        self.in_reasoning = default_force if force_reasoning is None else (force_reasoning or default_force)
        self.done = False
        self.buf = ""

    def parse(self, text: str) -> Tuple[str, str]:
        """Whole message -> (reasoning, content)."""
        t = text
        in_r = self.in_reasoning
        if self.start in t:
            before, t = t.split(self.start, 1)
            in_r = True
            prefix = before
        else:
            prefix = ""
        if not in_r:
            return "", text
        if self.end in t:
            r, c = t.split(self.end, 1)
            return r.strip(), (prefix + c).lstrip("\n")
        return t.strip(), prefix                     # truncated inside the reasoning block

    def _hold(self, text: str, tag: str) -> int:
        for k in range(min(len(tag) - 1, len(text)), 0, -1):
            if text.endswith(tag[:k]):
                return len(text) - k
        return len(text)

    def feed(self, delta: str) -> Tuple[str, str]:
        """Streaming: returns (reasoning delta, content delta)."""
        if self.done:
            return "", delta
        self.buf += delta
        r_out, c_out = "", ""
        while True:
            if not self.in_reasoning:
                pos = self.buf.find(self.start)
                if pos >= 0:
                    c_out += self.buf[:pos]
                    self.buf = self.buf[pos + len(self.start):]
                    self.in_reasoning = True
                    continue
                n = self._hold(self.buf, self.start)
                c_out += self.buf[:n]
                self.buf = self.buf[n:]
                return r_out, c_out
            if self.buf.startswith(self.start):          # explicit start tag although reasoning was forced
                self.buf = self.buf[len(self.start):]
            pos = self.buf.find(self.end)
            if pos >= 0:
                r_out += self.buf[:pos]
                rest = self.buf[pos + len(self.end):].lstrip("\n")
                self.buf, self.in_reasoning, self.done = "", False, True
                return r_out, c_out + rest
            n = min(self._hold(self.buf, self.end), self._hold(self.buf, self.start))
            r_out += self.buf[:n]
            self.buf = self.buf[n:]
            return r_out, c_out

    def flush(self) -> Tuple[str, str]:
        t, self.buf = self.buf, ""
        return (t, "") if self.in_reasoning else ("", t)
