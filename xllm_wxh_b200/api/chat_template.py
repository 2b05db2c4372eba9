"""Jinja chat templates (reference: xllm/core/framework/chat_template/jinja_chat_template.cpp, which
embeds `minja`).  HF chat templates are Jinja2 with a few extras (`raise_exception`, `strftime_now`,
`tojson`, loop controls); rendered here with the sandboxed Jinja2 environment."""
from __future__ import annotations

import datetime
import json
from typing import Any, Dict, List, Optional

import jinja2
from jinja2.sandbox import ImmutableSandboxedEnvironment


class JinjaChatTemplate:
    def __init__(self, template: str, tokenizer=None):
        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, extensions=["jinja2.ext.loopcontrols"])

        def raise_exception(msg):
            raise jinja2.exceptions.TemplateError(msg)

        def tojson(x, ensure_ascii=False, indent=None, separators=None, sort_keys=False):
            return json.dumps(x, ensure_ascii=ensure_ascii, indent=indent, separators=separators, sort_keys=sort_keys)

        env.globals["raise_exception"] = raise_exception
        env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
        env.filters["tojson"] = tojson
        self.template = env.from_string(template)
        self.bos = self.eos = ""
        if tokenizer is not None:
            b, e = getattr(tokenizer, "bos_token_id", -1), getattr(tokenizer, "eos_token_id", -1)
            self.bos = tokenizer.id_to_token(b) if b is not None and b >= 0 else ""
            self.eos = tokenizer.id_to_token(e) if e is not None and e >= 0 else ""

    def apply(self, messages: List[Dict[str, Any]], tools: Optional[List[Dict[str, Any]]] = None,
              kwargs: Optional[Dict[str, Any]] = None, add_generation_prompt: bool = True) -> str:
        ctx = dict(messages=messages, tools=tools or None, add_generation_prompt=add_generation_prompt,
                   bos_token=self.bos, eos_token=self.eos)
        ctx.update(kwargs or {})
        return self.template.render(**ctx)
