"""Byte-level BPE tokenizer built from GGUF metadata.

Reads ``tokenizer.ggml.{tokens,merges,token_type,bos_token_id,eos_token_id,padding_token_id}``;
CONTROL (3) and USER_DEFINED (4) tokens are matched as atomic strings before BPE runs, as the
reference does (reference: src/v2/utils/Tokenizer.cpp:52-123, :247-305, :445-491).  The merge
loop runs in the native helper when it is built (``llaminar_b200/tokenizer/csrc/bpe_merge.cpp``)
and in Python otherwise; both give identical ids.
"""
from __future__ import annotations

import functools
from typing import Iterable

try:
    import regex as _re
    _QWEN_SPLIT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*"
                   r"|\s*[\r\n]+|\s+(?!\S)|\s+")
    # the hybrid families' vocabulary was built with combining marks counted as letters
    _QWEN35_SPLIT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?[\p{L}\p{M}]+|\p{N}| ?[^\s\p{L}\p{M}\p{N}]+[\r\n]*"
                     r"|\s*[\r\n]+|\s+(?!\S)|\s+")
except ImportError:                                        # pragma: no cover
    import re as _re
    _QWEN_SPLIT = r"'s|'t|'re|'ve|'m|'ll|'d| ?[A-Za-z]+| ?[0-9]| ?[^\sA-Za-z0-9]+|\s+(?!\S)|\s+"
    _QWEN35_SPLIT = _QWEN_SPLIT

# pre-tokeniser by the name in `tokenizer.ggml.pre`; a file may also carry the expression itself
# (`tokenizer.llaminar.split_regex`, written by models/convert_hf.py from the checkpoint's tokenizer.json)
SPLIT_BY_NAME = {"qwen2": _QWEN_SPLIT, "qwen35": _QWEN35_SPLIT}

TOKEN_NORMAL, TOKEN_UNKNOWN, TOKEN_CONTROL, TOKEN_USER_DEFINED, TOKEN_UNUSED, TOKEN_BYTE = 1, 2, 3, 4, 5, 6


@functools.lru_cache(maxsize=1)
def byte_alphabet() -> tuple[str, ...]:
    """The GPT-2 printable stand-in for each of the 256 byte values."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return tuple(table[b] for b in range(256))


class BPETokenizer:
    def __init__(self, tokens: list[str], merges: Iterable[str] = (), token_types: list[int] | None = None,
                 bos_id: int | None = None, eos_id: int | None = None, pad_id: int | None = None,
                 chat_template: str | None = None, add_bos: bool = False, split_regex: str | None = None):
        self.tokens = list(tokens)
        self.vocab = {}
        for i, t in enumerate(self.tokens):
            self.vocab.setdefault(t, i)
        self.token_types = list(token_types) if token_types else [TOKEN_NORMAL] * len(self.tokens)
        self.ranks: dict[tuple[str, str], int] = {}
        for r, m in enumerate(merges):
            a, _, b = m.partition(" ")
            self.ranks[(a, b)] = r
        self.bos_id, self.eos_id, self.pad_id = bos_id, eos_id, pad_id
        self.chat_template = chat_template
        self.add_bos = add_bos
        self._alphabet = byte_alphabet()
        self._byte_of = {c: b for b, c in enumerate(self._alphabet)}
        self.special = {t: i for i, (t, ty) in enumerate(zip(self.tokens, self.token_types))
                        if ty in (TOKEN_CONTROL, TOKEN_USER_DEFINED) and t}
        self._special_re = None
        if self.special:
            alts = sorted(self.special, key=len, reverse=True)
            self._special_re = _re.compile("|".join(_re.escape(a) for a in alts))
        self._split_re = _re.compile(split_regex or _QWEN_SPLIT)
        self._cache: dict[str, list[int]] = {}
        self._native = None
        try:
            from . import native
            self._native = native.make_merger(self.tokens, self.ranks)
        except Exception:
            self._native = None

    # -- construction from a checkpoint --------------------------------------------------
    @staticmethod
    def from_metadata(md: dict) -> "BPETokenizer":
        tokens = md.get("tokenizer.ggml.tokens")
        if tokens is None:
            raise ValueError("checkpoint has no embedded tokenizer (tokenizer.ggml.tokens)")
        return BPETokenizer(tokens, md.get("tokenizer.ggml.merges") or (),
                            md.get("tokenizer.ggml.token_type"),
                            md.get("tokenizer.ggml.bos_token_id"), md.get("tokenizer.ggml.eos_token_id"),
                            md.get("tokenizer.ggml.padding_token_id"), md.get("tokenizer.chat_template"),
                            bool(md.get("tokenizer.ggml.add_bos_token", False)),
                            md.get("tokenizer.llaminar.split_regex") or SPLIT_BY_NAME.get(str(md.get("tokenizer.ggml.pre", "qwen2"))))

    @property
    def vocab_size(self) -> int:
        return len(self.tokens)

    # -- encode ----------------------------------------------------------------------------
    def _bpe_word(self, word: str) -> list[int]:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        if self._native is not None:
            ids = self._native.encode_word(word)
        else:
            parts = list(word)
            while len(parts) > 1:
                best, best_rank = -1, None
                for i in range(len(parts) - 1):
                    r = self.ranks.get((parts[i], parts[i + 1]))
                    if r is not None and (best_rank is None or r < best_rank):
                        best, best_rank = i, r
                if best < 0:
                    break
                parts[best:best + 2] = [parts[best] + parts[best + 1]]
            ids = []
            for p in parts:
                tid = self.vocab.get(p)
                if tid is not None:
                    ids.append(tid)
                else:                                    # unknown piece: fall back to its bytes
                    ids.extend(self.vocab[c] for c in p if c in self.vocab)
        if len(self._cache) < 200_000:
            self._cache[word] = ids
        return ids

    def _encode_plain(self, text: str) -> list[int]:
        out: list[int] = []
        for piece in self._split_re.findall(text):
            word = "".join(self._alphabet[b] for b in piece.encode("utf-8"))
            out.extend(self._bpe_word(word))
        return out

    def encode(self, text: str, add_special: bool = False, parse_special: bool = True) -> list[int]:
        ids: list[int] = []
        if add_special and self.add_bos and self.bos_id is not None:
            ids.append(self.bos_id)
        if parse_special and self._special_re is not None:
            pos = 0
            for m in self._special_re.finditer(text):
                if m.start() > pos:
                    ids.extend(self._encode_plain(text[pos:m.start()]))
                ids.append(self.special[m.group(0)])
                pos = m.end()
            if pos < len(text):
                ids.extend(self._encode_plain(text[pos:]))
        else:
            ids.extend(self._encode_plain(text))
        return ids

    # -- decode ----------------------------------------------------------------------------
    def token_bytes(self, tid: int) -> bytes:
        if tid < 0 or tid >= len(self.tokens):
            return b""
        t = self.tokens[tid]
        if self.token_types[tid] in (TOKEN_CONTROL, TOKEN_USER_DEFINED, TOKEN_UNUSED):
            return t.encode("utf-8")
        try:
            return bytes(self._byte_of[c] for c in t)
        except KeyError:
            return t.encode("utf-8")

    def is_special(self, tid: int) -> bool:
        return 0 <= tid < len(self.tokens) and self.token_types[tid] == TOKEN_CONTROL

    def decode(self, ids: Iterable[int], skip_special: bool = False) -> str:
        buf = b"".join(self.token_bytes(i) for i in ids if not (skip_special and self.is_special(i)))
        return buf.decode("utf-8", errors="replace")


class StreamDecoder:
    """Incremental detokeniser that never emits half of a multi-byte UTF-8 character."""

    def __init__(self, tok: BPETokenizer, skip_special: bool = True):
        self.tok, self.skip_special = tok, skip_special
        self._pending = b""

    def push(self, tid: int) -> str:
        if self.skip_special and self.tok.is_special(tid):
            return ""
        self._pending += self.tok.token_bytes(tid)
        # emit the longest valid prefix; keep at most 3 trailing bytes of an unfinished character
        for cut in range(len(self._pending), max(len(self._pending) - 4, -1), -1):
            try:
                text = self._pending[:cut].decode("utf-8")
            except UnicodeDecodeError:
                continue
            self._pending = self._pending[cut:]
            return text
        text = self._pending.decode("utf-8", errors="replace")
        self._pending = b""
        return text

    def flush(self) -> str:
        text = self._pending.decode("utf-8", errors="replace")
        self._pending = b""
        return text
