"""Offline stand-in for `tiktoken`: the reference calls `tiktoken.get_encoding("gpt2")` while its config
module is imported, which needs network access.  The benchmark feeds token ids directly, so only the
attributes the reference touches at import time are provided."""
from . import core
from .core import Encoding


def get_encoding(name: str) -> Encoding:
    return Encoding(name)
