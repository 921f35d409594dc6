"""Dependency-free byte-level byte-pair encoding.

Capability parity with the reference's `tokenizer/bpe.py:29-70` (train / encode / decode on raw
UTF-8 bytes).  The merge loop here keeps pair counts incrementally instead of recounting the
whole corpus after every merge.
"""
from __future__ import annotations

from collections import Counter
from typing import Dict, List, Tuple


class BytePairEncoding:
    def __init__(self) -> None:
        self.merges: Dict[Tuple[int, int], int] = {}
        self.vocab: Dict[int, bytes] = {i: bytes([i]) for i in range(256)}

    @property
    def n_vocab(self) -> int:
        return len(self.vocab)

    @staticmethod
    def _merge(ids: List[int], pair: Tuple[int, int], new_id: int) -> List[int]:
        out, i, n = [], 0, len(ids)
        while i < n:
            if i + 1 < n and ids[i] == pair[0] and ids[i + 1] == pair[1]:
                out.append(new_id)
                i += 2
            else:
                out.append(ids[i])
                i += 1
        return out

    def train(self, text: str, vocab_size: int) -> None:
        assert vocab_size >= 256
        ids = list(text.encode("utf-8"))
        for new_id in range(256, vocab_size):
            counts = Counter(zip(ids, ids[1:]))
            if not counts:
                break
            pair, freq = max(counts.items(), key=lambda kv: (kv[1], -kv[0][0], -kv[0][1]))
            if freq < 2:
                break
            ids = self._merge(ids, pair, new_id)
            self.merges[pair] = new_id
            self.vocab[new_id] = self.vocab[pair[0]] + self.vocab[pair[1]]

    def encode(self, text: str) -> List[int]:
        ids = list(text.encode("utf-8"))
        while len(ids) >= 2:
            candidates = [(self.merges[p], p) for p in set(zip(ids, ids[1:])) if p in self.merges]
            if not candidates:
                break
            new_id, pair = min(candidates)      # earliest-learned merge first
            ids = self._merge(ids, pair, new_id)
        return ids

    def decode(self, ids: List[int]) -> str:
        return b"".join(self.vocab[i] for i in ids).decode("utf-8", errors="replace")
