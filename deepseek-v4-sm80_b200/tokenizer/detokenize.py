"""Incremental detokenisation for streaming.

Per request the manager keeps the generated ids and two offsets: ``surr`` (start of the context window that is
re-decoded each step so that byte-level merges come out right) and ``read`` (ids already turned into committed text).
New text is committed when it does not end in an incomplete UTF-8 sequence (U+FFFD); otherwise only its printable
prefix -- whole words, or whole CJK characters -- is shown provisionally.  A final EOS token is dropped.
Same algorithm as python/minisgl/tokenizer/detokenize.py:10-111 of the reference (which follows SGLang).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List

_CJK = ((0x4E00, 0x9FFF), (0x3400, 0x4DBF), (0x20000, 0x2A6DF), (0x2A700, 0x2B73F), (0x2B740, 0x2B81F),
        (0x2B820, 0x2CEAF), (0xF900, 0xFAFF), (0x2F800, 0x2FA1F))


def is_cjk(ch: str) -> bool:
    cp = ord(ch)
    return any(a <= cp <= b for a, b in _CJK)


def printable_prefix(text: str) -> str:
    """Longest prefix that will not change when more tokens arrive."""
    if not text:
        return text
    if text.endswith("\n") or is_cjk(text[-1]):
        return text
    if len(text) > 1 and is_cjk(text[-2]):
        return text[:-1]
    return text[: text.rfind(" ") + 1]


@dataclass
class DecodeStatus:
    ids: List[int] = field(default_factory=list)
    text: str = ""
    read: int = 0
    surr: int = 0
    sent: int = 0


class DetokenizeManager:
    def __init__(self, tokenizer):
        self.tokenizer = tokenizer
        self.eos_token_id = tokenizer.eos_token_id
        self.state: Dict[int, DecodeStatus] = {}

    def detokenize(self, msgs) -> List[str]:
        read_ids, surr_ids = [], []
        for m in msgs:
            s = self.state.setdefault(m.uid, DecodeStatus())
            if not (m.finished and m.next_token == self.eos_token_id):
                s.ids.append(m.next_token)
            read_ids.append(s.ids[s.surr:])
            surr_ids.append(s.ids[s.surr: s.read])
        read_txt = self.tokenizer.batch_decode(read_ids)
        surr_txt = self.tokenizer.batch_decode(surr_ids)
        out: List[str] = []
        for m, rt, st in zip(msgs, read_txt, surr_txt):
            s = self.state[m.uid]
            new = rt[len(st):]
            if new and not new.endswith("�"):
                full = s.text + new
                s.text, s.surr, s.read = full, s.read, len(s.ids)
            else:
                full = s.text + printable_prefix(new)
            out.append(full[s.sent:])
            s.sent = len(full)
            if m.finished:
                del self.state[m.uid]
        return out
