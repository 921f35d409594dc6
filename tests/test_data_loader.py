import os

import numpy as np
import torch

from gpt_moe_b200.data.fineweb_npy import write_synthetic
from gpt_moe_b200.data.loader import DataLoader, SyntheticLoader


def _shards(tmp_path, tokens=4 * 2 * 16 * 6 + 37, shards=3):
    write_synthetic(str(tmp_path), shards, tokens, vocab_size=1000, seed=1)
    return str(tmp_path)


def test_shard_naming_and_split(tmp_path):
    folder = _shards(tmp_path)
    names = set(os.listdir(folder))
    assert names == {"edufineweb_val_000000.npy", "edufineweb_train_000001.npy", "edufineweb_train_000002.npy"}


def test_batches_are_shifted_and_ranks_disjoint(tmp_path):
    folder = _shards(tmp_path)
    loaders = [DataLoader(2, 16, 2, r, folder, "train") for r in range(2)]
    seen = set()
    for loader in loaders:
        for _ in range(loader.grad_accum_mini_steps_per_shard):
            x, y, docs = loader.next_batch()
            assert docs is None and x.shape == (2, 16)
            assert torch.equal(x[:, 1:], y[:, :-1])
            for row in x:
                key = tuple(row.tolist())
                assert key not in seen
                seen.add(key)
    tokens = np.load(loaders[0].sorted_shards[0])
    assert len(seen) == (len(tokens) // (2 * 2 * 16)) * 4


def test_resume_continues_with_the_next_batch(tmp_path):
    folder = _shards(tmp_path)
    a = DataLoader(2, 16, 1, 0, folder, "train")
    batches = [a.next_batch()[0].clone() for _ in range(15)]          # crosses a shard boundary (12 mini-steps per shard)
    b = DataLoader(2, 16, 1, 0, folder, "train")
    for _ in range(13):
        b.next_batch()
    c = DataLoader(2, 16, 1, 0, folder, "train", epoch=b.epoch, current_shard_idx=b.current_shard_idx,
                   grad_accum_mini_steps_per_shard_counter=b.grad_accum_mini_steps_per_shard_counter)
    assert torch.equal(c.next_batch()[0], batches[13]) and torch.equal(c.next_batch()[0], batches[14])


def test_validation_walks_an_ordered_global_prefix(tmp_path):
    folder = _shards(tmp_path)
    tokens = torch.from_numpy(np.load(os.path.join(folder, "edufineweb_val_000000.npy")).astype(np.int64))
    r0 = DataLoader(2, 16, 2, 0, folder, "val", shuffle_val_tokens=False)
    r1 = DataLoader(2, 16, 2, 1, folder, "val", shuffle_val_tokens=False)
    x0, _, _ = r0.next_batch()
    x1, _, _ = r1.next_batch()
    assert torch.equal(x0.reshape(-1), tokens[:32]) and torch.equal(x1.reshape(-1), tokens[32:64])
    r0.reset()
    assert torch.equal(r0.next_batch()[0].reshape(-1), tokens[:32])


def test_document_ids_count_eos(tmp_path):
    np.save(os.path.join(str(tmp_path), "x_train_000001.npy"), np.array([5, 7, 9, 7, 7, 1, 2, 3, 4] * 8, dtype=np.uint16))
    loader = DataLoader(1, 8, 1, 0, str(tmp_path), "train", eos_token_id=7, return_document_ids=True)
    x, _, docs = loader.next_batch()
    expect = torch.cumsum((x == 7).int(), 1) - (x == 7).int()
    assert torch.equal(docs, expect)


def test_synthetic_loader_is_seeded_per_rank():
    a, b, c = SyntheticLoader(2, 8, 2, 0, 100, seed=0), SyntheticLoader(2, 8, 2, 0, 100, seed=0), SyntheticLoader(2, 8, 2, 1, 100, seed=0)
    xa, ya, _ = a.next_batch()
    xb, _, _ = b.next_batch()
    xc, _, _ = c.next_batch()
    assert torch.equal(xa, xb) and not torch.equal(xa, xc) and torch.equal(xa[:, 1:], ya[:, :-1])
    assert xa.min() >= 0 and xa.max() < 100
