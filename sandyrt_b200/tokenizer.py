"""Byte-level BPE tokenizer for GPT-2 vocab.json + merges.txt, standard library only.

Behaviour follows the reference's driver (scripts/run_gpt2.py:195-290): bytes are mapped to
printable code points, text is cut into chunks that keep their leading space ('s, 't, 're,
've, 'm, 'll, 'd, words, numbers, punctuation runs, white space: the reference's
approximation of GPT-2's pattern with the `re` module, :239-245), and each chunk is merged
greedily by the rank of its adjacent pairs.  The engine itself works on token ids only; this
module serves the command-line entry points when a model folder ships the two files.
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, List, Tuple

_CHUNKS = re.compile(r"'s|'t|'re|'ve|'m|'ll|'d| ?[^\W\d_]+| ?\d+| ?[^\s\w]+|\s+", re.UNICODE)


def _byte_table() -> Dict[int, str]:
    """256 bytes -> 256 printable characters: the visible Latin-1 ranges stand for themselves,
    every other byte gets the next free code point from 256 on."""
    keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


class BPETokenizer:
    def __init__(self, vocab_path: str, merges_path: str):
        with open(vocab_path, "r", encoding="utf-8") as f:
            self.token_to_id: Dict[str, int] = json.load(f)
        if not self.token_to_id:
            raise ValueError(f"{vocab_path} holds no vocabulary")
        self.id_to_token = {i: t for t, i in self.token_to_id.items()}
        self.rank: Dict[Tuple[str, str], int] = {}
        with open(merges_path, "r", encoding="utf-8") as f:
            for line in f:
                parts = line.split()
                if len(parts) == 2 and not line.startswith("#"):
                    self.rank[(parts[0], parts[1])] = len(self.rank)
        self.byte_to_char = _byte_table()
        self.char_to_byte = {c: b for b, c in self.byte_to_char.items()}
        self._memo: Dict[str, List[str]] = {}

    @classmethod
    def from_dir(cls, folder: str) -> "BPETokenizer":
        return cls(os.path.join(folder, "vocab.json"), os.path.join(folder, "merges.txt"))

    @staticmethod
    def available(folder: str) -> bool:
        v, m = os.path.join(folder, "vocab.json"), os.path.join(folder, "merges.txt")
        return os.path.isfile(v) and os.path.getsize(v) > 2 and os.path.isfile(m)

    def _merge(self, chunk: str) -> List[str]:
        hit = self._memo.get(chunk)
        if hit is not None:
            return hit
        parts = list(chunk)
        while len(parts) > 1:
            best, best_rank = -1, None
            for i in range(len(parts) - 1):
                r = self.rank.get((parts[i], parts[i + 1]))
                if r is not None and (best_rank is None or r < best_rank):
                    best, best_rank = i, r
            if best < 0:
                break
            a, b = parts[best], parts[best + 1]
            merged, i = [], 0
            while i < len(parts):                      # every occurrence of the best pair, left to right
                if i < len(parts) - 1 and parts[i] == a and parts[i + 1] == b:
                    merged.append(a + b)
                    i += 2
                else:
                    merged.append(parts[i])
                    i += 1
            parts = merged
        self._memo[chunk] = parts
        return parts

    def encode(self, text: str) -> List[int]:
        ids: List[int] = []
        for m in _CHUNKS.finditer(text):
            mapped = "".join(self.byte_to_char[b] for b in m.group(0).encode("utf-8"))
            ids.extend(self.token_to_id[p] for p in self._merge(mapped))
        return ids

    def decode(self, ids) -> str:
        chars = "".join(self.id_to_token[int(i)] for i in ids)
        return bytes(self.char_to_byte[c] for c in chars).decode("utf-8", errors="replace")
