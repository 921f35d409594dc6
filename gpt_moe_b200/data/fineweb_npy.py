"""Tokenise FineWeb-Edu (sample-10BT) into 100M-token uint16 `.npy` shards.

Shard 0 is the validation shard (`edufineweb_val_000000.npy`), the rest are training shards
(`edufineweb_train_{idx:06d}.npy`) — the layout `data/loader.py` expects (reference
`data/fineweb-npy.py:21-92`).  Needs network access for the dataset and the GPT-2 vocabulary;
`--synthetic N` instead writes N shards of uniform random tokens for offline runs.
"""
from __future__ import annotations

import argparse
import multiprocessing as mp
import os

import numpy as np

SHARD_TOKENS = int(1e8)


def _shard_path(out_dir: str, index: int) -> str:
    split = "val" if index == 0 else "train"
    return os.path.join(out_dir, f"edufineweb_{split}_{index:06d}.npy")


def _tokenize(doc):
    import tiktoken
    enc = _tokenize.enc = getattr(_tokenize, "enc", None) or tiktoken.get_encoding("gpt2")
    ids = [enc.eot_token] + enc.encode_ordinary(doc["text"])
    arr = np.asarray(ids)
    assert (0 <= arr).all() and (arr < 2 ** 16).all(), "token id does not fit uint16"
    return arr.astype(np.uint16)


def write_synthetic(out_dir: str, shards: int, tokens_per_shard: int, vocab_size: int = 50304, seed: int = 0) -> None:
    os.makedirs(out_dir, exist_ok=True)
    rng = np.random.default_rng(seed)
    for i in range(shards):
        np.save(_shard_path(out_dir, i), rng.integers(0, vocab_size, tokens_per_shard, dtype=np.uint16))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(os.path.dirname(__file__), "edu_fineweb10B"))
    ap.add_argument("--synthetic", type=int, default=0, help="write this many random-token shards instead of downloading")
    ap.add_argument("--tokens-per-shard", type=int, default=SHARD_TOKENS)
    args = ap.parse_args()
    if args.synthetic:
        write_synthetic(args.out, args.synthetic, args.tokens_per_shard)
        return
    from datasets import load_dataset
    os.makedirs(args.out, exist_ok=True)
    data = load_dataset("HuggingFaceFW/fineweb-edu", name="sample-10BT", split="train")
    shard, fill, index = np.empty(args.tokens_per_shard, dtype=np.uint16), 0, 0
    with mp.Pool(max(1, os.cpu_count() // 2)) as pool:
        for tokens in pool.imap(_tokenize, data, chunksize=16):
            while len(tokens):
                take = min(len(tokens), args.tokens_per_shard - fill)
                shard[fill: fill + take] = tokens[:take]
                fill += take
                tokens = tokens[take:]
                if fill == args.tokens_per_shard:
                    np.save(_shard_path(args.out, index), shard)
                    index, fill = index + 1, 0
    if fill:
        np.save(_shard_path(args.out, index), shard[:fill])


if __name__ == "__main__":
    main()
