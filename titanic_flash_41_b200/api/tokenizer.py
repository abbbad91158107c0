"""Tokenizers behind one small interface.

``ByteTokenizer`` needs no files: ids 0..2 are BOS/EOS/PAD as in the reference config
(tests/fixtures/1017-config.json: bos 0, eos 1, pad 2), every special marker of the chat
template is one id, and all other text is UTF-8 bytes.  ``HFTokenizer`` wraps a tokenizer
directory when one is available (the reference loads the model's own tokenizer:
src/protocol.rs:32 Frontend).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

from . import protocol as P

SPECIALS = [P.BOS, P.EOS, "<｜pad｜>", P.USER, P.ASSISTANT, P.THINK_OPEN, P.THINK_CLOSE, "<｜tool▁output｜>",
            "<｜tool▁output▁end｜>", "<｜image｜>", f"<{P.DSML} calls>", f"</{P.DSML} calls>"]


class ByteTokenizer:
    bos_id, eos_id, pad_id = 0, 1, 2

    def __init__(self, vocab: int = 1024):
        self.base = len(SPECIALS)
        assert vocab >= self.base + 256, "vocabulary too small for byte fallback"
        self.vocab = vocab
        self.special_ids: Dict[str, int] = {s: i for i, s in enumerate(SPECIALS)}
        self.image_id = self.special_ids["<｜image｜>"]

    def encode(self, text: str) -> List[int]:
        out: List[int] = []
        i = 0
        while i < len(text):
            hit = None
            if text[i] == "<":
                for s, sid in self.special_ids.items():
                    if text.startswith(s, i):
                        hit = (s, sid)
                        break
            if hit:
                out.append(hit[1])
                i += len(hit[0])
            else:
                j = i + 1
                while j < len(text) and text[j] != "<":
                    j += 1
                out += [self.base + b for b in text[i:j].encode("utf-8")]
                i = j
        return out

    def decode(self, ids: Iterable[int]) -> str:
        parts: List[str] = []
        buf = bytearray()
        for t in ids:
            if self.base <= t < self.base + 256:
                buf.append(t - self.base)
            else:
                if buf:
                    parts.append(buf.decode("utf-8", errors="replace"))
                    buf = bytearray()
                if 0 <= t < self.base:
                    parts.append(SPECIALS[t])
        if buf:
            parts.append(buf.decode("utf-8", errors="replace"))
        return "".join(parts)


class IncrementalDecoder:
    """Streams text out of token ids without splitting a UTF-8 sequence across deltas."""

    def __init__(self, tok):
        self.tok, self.ids, self.sent = tok, [], 0

    def push(self, new_ids: Iterable[int]) -> str:
        self.ids += list(new_ids)
        text = self.tok.decode(self.ids)
        # hold back a trailing replacement character: the sequence may complete with the next token
        safe = len(text)
        while safe > self.sent and text[safe - 1] == "�":
            safe -= 1
        out = text[self.sent:safe]
        self.sent = safe
        return out

    def flush(self) -> str:
        text = self.tok.decode(self.ids)
        out = text[self.sent:]
        self.sent = len(text)
        return out


class HFTokenizer:
    def __init__(self, path: str):
        from transformers import AutoTokenizer
        self.t = AutoTokenizer.from_pretrained(path)
        self.bos_id, self.eos_id = self.t.bos_token_id or 0, self.t.eos_token_id or 1
        self.vocab = len(self.t)
        self.image_id = self.t.convert_tokens_to_ids("<｜image｜>")

    def encode(self, text: str) -> List[int]:
        return self.t.encode(text, add_special_tokens=False)

    def decode(self, ids) -> str:
        return self.t.decode(list(ids), skip_special_tokens=False)


def load_tokenizer(path: Optional[str], vocab: int):
    return HFTokenizer(path) if path else ByteTokenizer(vocab)
