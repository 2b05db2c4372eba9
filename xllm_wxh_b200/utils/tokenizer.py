"""Tokenizer front-end.

Factory order follows the reference (xllm/core/framework/tokenizer/tokenizer_factory.cpp:22-52):
`tokenizer.json` (HF fast tokenizer) -> `*.tiktoken` -> sentencepiece `tokenizer.model`.  Byte-level
BPE models (Qwen, DeepSeek, GPT-style) run on the C++ `BpeTokenizer`; layouts it does not cover fall
back to the HF `tokenizers` wheel at this API edge.  Architectures instantiated from a preset have no
vocabulary: `IdTokenizer` maps text made of decimal ids to those ids and back.
"""
from __future__ import annotations

import base64
import json
import os
from typing import Dict, List, Optional

from .. import _core


def _gpt2_byte_decoder() -> Dict[str, int]:
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {chr(c): b for b, c in zip(bs, cs)}


_BYTE_DECODER = _gpt2_byte_decoder()


def _unicode_to_bytes(tok: str) -> Optional[bytes]:
    try:
        return bytes(_BYTE_DECODER[c] for c in tok)
    except KeyError:
        return None


class Tokenizer:
    """Common interface (reference: tokenizer.h `Tokenizer::encode/decode/id_to_token/token_to_id/vocab_size`)."""
    eos_token_id: int = -1
    bos_token_id: int = -1
    chat_template: Optional[str] = None
    special_tokens: Dict[str, int]

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]: raise NotImplementedError
    def decode(self, ids: List[int], skip_special_tokens: bool = True) -> str: raise NotImplementedError
    def decode_bytes(self, ids: List[int], skip_special_tokens: bool = True) -> bytes:
        return self.decode(ids, skip_special_tokens).encode("utf-8", "ignore")
    def token_to_id(self, tok: str) -> int: raise NotImplementedError
    def id_to_token(self, i: int) -> str: raise NotImplementedError
    @property
    def vocab_size(self) -> int: raise NotImplementedError


class NativeBpeTokenizer(Tokenizer):
    def __init__(self, core: "_core.BpeTokenizer", specials: Dict[str, int], bos_prefix: Optional[int] = None):
        self.core = core
        self.special_tokens = specials
        self.bos_prefix = bos_prefix

    def encode(self, text, add_special_tokens=True):
        ids = list(self.core.encode(text, True))
        if add_special_tokens and self.bos_prefix is not None:
            ids = [self.bos_prefix] + ids
        return ids

    def decode_bytes(self, ids, skip_special_tokens=True):
        return self.core.decode(list(ids), skip_special_tokens)

    def decode(self, ids, skip_special_tokens=True):
        return self.decode_bytes(ids, skip_special_tokens).decode("utf-8", "replace")

    def token_to_id(self, tok):
        if tok in self.special_tokens:
            return self.special_tokens[tok]
        return self.core.token_to_id(tok.encode())

    def id_to_token(self, i):
        return self.core.id_to_token(i).decode("utf-8", "replace")

    @property
    def vocab_size(self):
        return self.core.vocab_size


class HFTokenizer(Tokenizer):
    """Fallback through the HF `tokenizers` wheel for tokenizer.json layouts the C++ BPE does not cover."""

    def __init__(self, path: str):
        import tokenizers
        self.tk = tokenizers.Tokenizer.from_file(path)
        self.special_tokens = {}

    def encode(self, text, add_special_tokens=True):
        return self.tk.encode(text, add_special_tokens=add_special_tokens).ids

    def decode(self, ids, skip_special_tokens=True):
        return self.tk.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def token_to_id(self, tok):
        r = self.tk.token_to_id(tok)
        return -1 if r is None else r

    def id_to_token(self, i):
        return self.tk.id_to_token(i) or ""

    @property
    def vocab_size(self):
        return self.tk.get_vocab_size()


class IdTokenizer(Tokenizer):
    """Text is a list of decimal token ids separated by blanks (random-initialised presets, tests)."""

    def __init__(self, vocab_size: int, eos_token_id: int = -1):
        self._v = vocab_size
        self.eos_token_id = eos_token_id
        self.special_tokens = {}

    def encode(self, text, add_special_tokens=True):
        # a word that is not a number still gets a stable id, so that scripts with ordinary prompts run on a preset
        import zlib
        return [(int(t) if t.lstrip("-").isdigit() else zlib.crc32(t.encode())) % self._v for t in text.split()]

    def decode(self, ids, skip_special_tokens=True):
        return "".join(f" {i}" for i in ids)

    def token_to_id(self, tok):
        return int(tok) if tok.strip().isdigit() else -1

    def id_to_token(self, i):
        return str(i)

    @property
    def vocab_size(self):
        return self._v


_QWEN_PATTERNS = ("(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\\r\\n\\p{L}\\p{N}]?\\p{L}+|\\p{N}| ?[^\\s\\p{L}\\p{N}]+[\\r\\n]*|\\s*[\\r\\n]+|\\s+(?!\\S)|\\s+",)
_CL100K_PATTERNS = ("(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\\r\\n\\p{L}\\p{N}]?\\p{L}+|\\p{N}{1,3}| ?[^\\s\\p{L}\\p{N}]+[\\r\\n]*|\\s*[\\r\\n]+|\\s+(?!\\S)|\\s+",)


def _native_from_tokenizer_json(path: str) -> Optional[NativeBpeTokenizer]:
    with open(path, encoding="utf-8") as f:
        tj = json.load(f)
    model = tj.get("model", {})
    if model.get("type") != "BPE":
        return None
    # which pre-tokenizer?
    pre = tj.get("pre_tokenizer") or {}
    pats = []
    def walk(p):
        if not p:
            return
        if p.get("type") == "Sequence":
            for q in p.get("pretokenizers", []):
                walk(q)
        elif p.get("type") == "Split":
            pats.append(p.get("pattern", {}).get("Regex", ""))
        elif p.get("type") == "ByteLevel":
            if p.get("use_regex", True):
                pats.append("<gpt2>")
    walk(pre)
    if len(pats) != 1:
        return None
    if pats[0] in _QWEN_PATTERNS:
        max_digits = 1
    elif pats[0] in _CL100K_PATTERNS:
        max_digits = 3
    else:
        return None
    vocab = []
    for tok, idx in model.get("vocab", {}).items():
        b = _unicode_to_bytes(tok)
        if b is None:
            return None
        vocab.append((b, idx))
    merges = []
    for m in model.get("merges", []):
        a, b = m.split(" ", 1) if isinstance(m, str) else m
        ab, bb = _unicode_to_bytes(a), _unicode_to_bytes(b)
        if ab is None or bb is None:
            return None
        merges.append((ab, bb))
    core = _core.BpeTokenizer()
    core.load_vocab(vocab, merges, max_digits)
    specials = {}
    for t in tj.get("added_tokens", []):
        core.add_special(t["content"].encode(), t["id"])
        specials[t["content"]] = t["id"]
    return NativeBpeTokenizer(core, specials)


def _native_from_tiktoken(path: str, specials: Dict[str, int]) -> NativeBpeTokenizer:
    vocab = []
    with open(path, "rb") as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            tok, rank = line.split()
            vocab.append((base64.b64decode(tok), int(rank)))
    core = _core.BpeTokenizer()
    core.load_vocab(vocab, [], 3)
    for s, i in specials.items():
        core.add_special(s.encode(), i)
    return NativeBpeTokenizer(core, dict(specials))


def load_tokenizer(model_dir: Optional[str], vocab_size: int = 0, eos_token_id: int = -1) -> Tokenizer:
    if not model_dir or not os.path.isdir(model_dir):
        return IdTokenizer(vocab_size, eos_token_id)
    cfg = {}
    cpath = os.path.join(model_dir, "tokenizer_config.json")
    if os.path.exists(cpath):
        with open(cpath, encoding="utf-8") as f:
            cfg = json.load(f)
    tok: Optional[Tokenizer] = None
    tj = os.path.join(model_dir, "tokenizer.json")
    if os.path.exists(tj):
        tok = _native_from_tokenizer_json(tj)
        if tok is None:
            tok = HFTokenizer(tj)
    else:
        tik = [f for f in os.listdir(model_dir) if f.endswith(".tiktoken")]
        if tik:
            specials = {}
            for k, v in (cfg.get("added_tokens_decoder") or {}).items():
                specials[v["content"]] = int(k)
            tok = _native_from_tiktoken(os.path.join(model_dir, tik[0]), specials)
    if tok is None:
        if os.path.exists(os.path.join(model_dir, "tokenizer.model")):
            import sentencepiece as spm

            class _SP(Tokenizer):
                def __init__(self, p):
                    self.sp = spm.SentencePieceProcessor(model_file=p)
                    self.special_tokens = {}
                def encode(self, text, add_special_tokens=True): return self.sp.encode(text)
                def decode(self, ids, skip_special_tokens=True): return self.sp.decode(list(ids))
                def token_to_id(self, t): return self.sp.piece_to_id(t)
                def id_to_token(self, i): return self.sp.id_to_piece(i)
                @property
                def vocab_size(self): return self.sp.get_piece_size()
            tok = _SP(os.path.join(model_dir, "tokenizer.model"))
        else:
            return IdTokenizer(vocab_size, eos_token_id)
    tok.chat_template = cfg.get("chat_template")
    ct = os.path.join(model_dir, "chat_template.jinja")
    if tok.chat_template is None and os.path.exists(ct):
        with open(ct, encoding="utf-8") as f:
            tok.chat_template = f.read()

    def tid(name):
        v = cfg.get(name)
        if isinstance(v, dict):
            v = v.get("content")
        return tok.token_to_id(v) if isinstance(v, str) else -1
    tok.eos_token_id = tid("eos_token") if cfg.get("eos_token") else eos_token_id
    tok.bos_token_id = tid("bos_token") if cfg.get("bos_token") else -1
    if cfg.get("add_bos_token") and isinstance(tok, NativeBpeTokenizer) and tok.bos_token_id >= 0:
        tok.bos_prefix = tok.bos_token_id
    return tok


class IncrementalDecoder:
    """Streams text for a growing token list without emitting half UTF-8 characters
    (reference: xllm/core/framework/request/incremental_decoder.cpp:41-83).

    The native BPE tokenizer gives bytes per token, so new bytes are appended and an incomplete trailing UTF-8 sequence
    is held back.  Any other tokenizer is asked for text, and only for a short window of tokens, the reference's
    two-offset scheme: the text of [prefix, read) is known to be out already; when the text of [prefix, end) has grown
    and does not end in a replacement character, the difference is emitted and the window moves on.  The cost per token
    does not grow with the length of the output (decoding the whole list every time did).  A tokenizer whose text for a
    slice of ids is not the matching slice of the whole text says so with `slice_decodable = False` and is decoded whole."""

    def __init__(self, tokenizer: Tokenizer, skip_special_tokens: bool = True):
        self.tok, self.skip = tokenizer, skip_special_tokens
        self.ids: List[int] = []
        self.emitted = 0          # bytes already returned (native path)
        self._bytes = b""
        self._native = isinstance(tokenizer, NativeBpeTokenizer)
        self._whole = not self._native and not getattr(tokenizer, "slice_decodable", True)
        self._prefix = self._read = 0          # window offsets into `ids` (text path)
        self._prefix_text: Optional[str] = ""  # text of ids[_prefix:_read]; None: not decoded yet

    def _window(self):
        if self._prefix_text is None:
            self._prefix_text = self.tok.decode(self.ids[self._prefix:self._read], self.skip)
        return self._prefix_text, self.tok.decode(self.ids[self._prefix:], self.skip)

    def add(self, new_ids: List[int]) -> str:
        if not new_ids:
            return ""
        self.ids.extend(new_ids)
        if self._whole:
            self._bytes = self.tok.decode(self.ids, self.skip).encode("utf-8")
        elif not self._native:
            prefix_text, new_text = self._window()
            if len(new_text) > len(prefix_text) and not new_text.endswith("\ufffd"):
                self._prefix, self._read, self._prefix_text = self._read, len(self.ids), None
                return new_text[len(prefix_text):]
            return ""
        else:
            self._bytes += self.tok.decode_bytes(new_ids, self.skip)
        data = self._bytes[self.emitted:]
        # hold back an incomplete trailing UTF-8 sequence
        cut = len(data)
        for back in range(1, min(4, len(data)) + 1):
            c = data[-back]
            if c & 0xC0 == 0x80:
                continue
            need = 1 if c < 0x80 else 2 if c >> 5 == 6 else 3 if c >> 4 == 14 else 4 if c >> 3 == 30 else 1
            if need > back:
                cut = len(data) - back
            break
        out = data[:cut]
        self.emitted += len(out)
        return out.decode("utf-8", "replace")

    def flush(self) -> str:
        """Whatever is still held back (an unfinished character at the end of the output)."""
        if not self._native and not self._whole:
            prefix_text, new_text = self._window()
            self._prefix = self._read = len(self.ids)
            self._prefix_text = ""
            return new_text[len(prefix_text):] if len(new_text) > len(prefix_text) else ""
        data = self._bytes[self.emitted:]
        self.emitted = len(self._bytes)
        return data.decode("utf-8", "replace")
