"""Tokenizer resolution.

Training uses the GPT-2 vocabulary through tiktoken when its files are available
(reference `config/training.py:102`).  Without network access tiktoken cannot fetch them, so a
byte-level fallback with the same interface (`n_vocab`, `encode`, `encode_ordinary`, `decode`,
`eot_token`) keeps sampling and the evaluations runnable on synthetic or pre-tokenised data.
"""
from __future__ import annotations

from typing import List


class ByteTokenizer:
    """Bytes 0..255 map to ids 0..255; ids >= 256 decode to nothing; `eot_token` = 50256."""
    n_vocab = 50257
    eot_token = 50256
    name = "bytes"

    def encode(self, text: str, allowed_special=None) -> List[int]:
        return list(text.encode("utf-8"))

    encode_ordinary = encode

    def decode(self, ids) -> str:
        return bytes(int(i) for i in ids if 0 <= int(i) < 256).decode("utf-8", errors="replace")


def load_tokenizer(name: str = "gpt2"):
    if name != "bytes":
        try:
            import tiktoken
            return tiktoken.get_encoding(name)
        except Exception:
            pass
    return ByteTokenizer()
