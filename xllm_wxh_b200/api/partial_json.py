"""Tolerant parser for JSON that is still being generated.

`parse_partial(text)` returns `(value, complete)`: the Python value of the longest well-formed reading of a JSON
prefix — open strings are closed, dangling keys / commas dropped, open arrays and objects closed — and whether the
text was already a complete JSON document.  Used by the streaming tool-call parsers to surface the function name and
the arguments while the model is still writing them (role of the reference's `xllm/function_call/partial_json_parser`).
"""
from __future__ import annotations

import json
from typing import Any, Tuple


class _Incomplete(Exception):
    pass


def parse_partial(text: str) -> Tuple[Any, bool]:
    s = text.lstrip()
    if not s:
        return None, False
    try:
        return json.loads(s), True
    except json.JSONDecodeError:
        pass
    p = _P(s)
    try:
        v = p.value()
        return v, False
    except _Incomplete:
        return None, False


class _P:
    def __init__(self, s: str):
        self.s, self.i, self.n = s, 0, len(s)

    def ws(self):
        while self.i < self.n and self.s[self.i] in " \t\r\n":
            self.i += 1

    def value(self) -> Any:
        self.ws()
        if self.i >= self.n:
            raise _Incomplete()
        c = self.s[self.i]
        if c == "{":
            return self.obj()
        if c == "[":
            return self.arr()
        if c == '"':
            return self.string()[0]
        return self.scalar()

    def string(self) -> Tuple[str, bool]:
        """Returns (text, closed)."""
        assert self.s[self.i] == '"'
        self.i += 1
        out = []
        while self.i < self.n:
            c = self.s[self.i]
            if c == '"':
                self.i += 1
                return "".join(out), True
            if c == "\\":
                if self.i + 1 >= self.n:
                    self.i = self.n
                    break
                e = self.s[self.i + 1]
                if e == "u":
                    if self.i + 6 > self.n:
                        self.i = self.n
                        break
                    try:
                        out.append(chr(int(self.s[self.i + 2:self.i + 6], 16)))
                    except ValueError:
                        pass
                    self.i += 6
                    continue
                out.append({"n": "\n", "t": "\t", "r": "\r", "b": "\b", "f": "\f"}.get(e, e))
                self.i += 2
                continue
            out.append(c)
            self.i += 1
        return "".join(out), False

    def scalar(self) -> Any:
        j = self.i
        while j < self.n and self.s[j] not in ",]} \t\r\n":
            j += 1
        tok = self.s[self.i:j]
        at_end = j >= self.n
        self.i = j
        for lit, val in (("true", True), ("false", False), ("null", None)):
            if tok == lit:
                return val
            if at_end and lit.startswith(tok) and tok:
                raise _Incomplete()
        try:
            return int(tok)
        except ValueError:
            pass
        try:
            return float(tok)
        except ValueError:
            # "-", "1e", "1." at the very end: number still being written
            t = tok.rstrip("eE+-.")
            if at_end and t:
                try:
                    return float(t) if any(ch in t for ch in ".eE") else int(t)
                except ValueError:
                    pass
            raise _Incomplete()

    def arr(self) -> list:
        self.i += 1
        out = []
        while True:
            self.ws()
            if self.i >= self.n:
                return out
            if self.s[self.i] == "]":
                self.i += 1
                return out
            if self.s[self.i] == ",":
                self.i += 1
                continue
            try:
                out.append(self.value())
            except _Incomplete:
                return out

    def obj(self) -> dict:
        self.i += 1
        out = {}
        while True:
            self.ws()
            if self.i >= self.n:
                return out
            c = self.s[self.i]
            if c == "}":
                self.i += 1
                return out
            if c == ",":
                self.i += 1
                continue
            if c != '"':
                return out
            key, closed = self.string()
            if not closed:
                return out
            self.ws()
            if self.i >= self.n or self.s[self.i] != ":":
                return out
            self.i += 1
            self.ws()
            if self.i >= self.n:
                return out
            try:
                out[key] = self.value()
            except _Incomplete:
                return out
