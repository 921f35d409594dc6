"""Token-shard data loader.

Reads `.npy` shards of uint16 token ids named `*train*` / `*val*`, exactly the files the
reference consumes, and reproduces its batch order (`data/loader.py:12-215`):

* each shard is truncated to a whole number of mini-steps (`world * batch * seq` tokens) plus one
  token for the shifted targets;
* sequence starts (stride `seq_len`) are shuffled per shard with `torch.Generator` seeded by
  `shard_idx + epoch` (train, and val when `shuffle_val_tokens`), then split into contiguous
  per-rank slices; unshuffled validation walks an ordered global prefix instead;
* position is `(epoch, current_shard_idx, grad_accum_mini_steps_per_shard_counter)`, which is what
  checkpoints store, so resuming continues with the very next batch;
* the next shard is read by a background thread while the current one is consumed.

Batches are assembled into a reusable pinned staging buffer so the host-to-device copy that
follows is a single asynchronous DMA per tensor.
"""
from __future__ import annotations

import os
import threading
from typing import List, Optional, Tuple

import numpy as np
import torch
from torch import Tensor


def _load_tokens(path: str) -> Tensor:
    return torch.from_numpy(np.load(path).astype(np.int64))


class DataLoader:
    def __init__(self, gpu_batch_size: int, seq_len: int, world_size: int, rank: int, data_folder: str,
                 split: str = "train", epoch: int = 0, current_shard_idx: int = 0,
                 grad_accum_mini_steps_per_shard_counter: int = 0, pad_token_id: int = 50257,
                 eos_token_id: int = 50256, return_document_ids: bool = False, shuffle_val_tokens: bool = True,
                 *, master_process: bool = False, log_buffer: Optional[List[str]] = None) -> None:
        self.gpu_batch_size, self.seq_len = gpu_batch_size, seq_len
        self.world_size, self.rank, self.split, self.epoch = world_size, rank, split, epoch
        self.pad_token_id, self.eos_token_id = pad_token_id, eos_token_id
        self.return_document_ids = return_document_ids
        self.shuffle_val_tokens = shuffle_val_tokens
        self.master_process = master_process
        self.log_buffer = log_buffer if log_buffer is not None else []
        self.sorted_shards = sorted(os.path.join(data_folder, f) for f in os.listdir(data_folder) if split in f)
        assert self.sorted_shards, f"no shards found for split {split}"
        self._log(f"found {len(self.sorted_shards)} shards for split {split}")
        self.current_shard_idx = current_shard_idx
        self.grad_accum_tokens_per_mini_step = world_size * gpu_batch_size * seq_len
        self._next_tokens: Optional[Tensor] = None
        self._prefetch_thread: Optional[threading.Thread] = None
        self._pinned = None
        self._install_shard(_load_tokens(self.sorted_shards[current_shard_idx]))
        self.grad_accum_mini_steps_per_shard_counter = grad_accum_mini_steps_per_shard_counter
        self._start_prefetch()

    def _log(self, message: str) -> None:
        if self.master_process:
            print(message)
            self.log_buffer.append(message)

    # ---- shard handling -----------------------------------------------------------------------
    def _install_shard(self, tokens: Tensor) -> None:
        per = self.grad_accum_tokens_per_mini_step
        self.grad_accum_mini_steps_per_shard = len(tokens) // per
        self.tokens = tokens[: per * self.grad_accum_mini_steps_per_shard + 1]
        starts = torch.arange(0, max(len(self.tokens) - self.seq_len, 0), self.seq_len)
        if self.split == "train" or self.shuffle_val_tokens:
            g = torch.Generator()
            g.manual_seed(self.current_shard_idx + self.epoch)
            starts = starts[torch.randperm(len(starts), generator=g)]
        self.x_seq_starts = starts
        lo = len(starts) * self.rank // self.world_size
        self.gpu_x_seq_starts = starts[lo: lo + len(starts) // self.world_size]
        self._log(f"{self.split} shard {self.current_shard_idx}: {len(self.tokens):,} tokens, "
                  f"{self.grad_accum_mini_steps_per_shard:,} mini-steps of {per:,} tokens over {self.world_size} gpus")

    def _start_prefetch(self) -> None:
        if self._prefetch_thread is not None and self._prefetch_thread.is_alive():
            return
        nxt = (self.current_shard_idx + 1) % len(self.sorted_shards)

        def worker() -> None:
            self._next_tokens = _load_tokens(self.sorted_shards[nxt])

        self._prefetch_thread = threading.Thread(target=worker, daemon=True)
        self._prefetch_thread.start()

    def _advance_shard(self) -> None:
        self.current_shard_idx += 1
        self.grad_accum_mini_steps_per_shard_counter = 0
        if self.current_shard_idx >= len(self.sorted_shards):
            self.current_shard_idx = 0
            self.epoch += 1
            self._log(f"--- starting epoch {self.epoch} ---")
        if self._prefetch_thread is not None:
            self._prefetch_thread.join()
        tokens, self._next_tokens = self._next_tokens, None
        if tokens is None:
            tokens = _load_tokens(self.sorted_shards[self.current_shard_idx])
        self._install_shard(tokens)
        self._start_prefetch()

    def reset(self) -> None:
        if self._prefetch_thread is not None:
            self._prefetch_thread.join()
        self.current_shard_idx = 0
        self.grad_accum_mini_steps_per_shard_counter = 0
        self._next_tokens = None
        self._install_shard(_load_tokens(self.sorted_shards[0]))
        self._start_prefetch()

    # ---- batches ------------------------------------------------------------------------------
    def _staging(self) -> Tuple[Tensor, Tensor]:
        if self._pinned is None:
            pin = torch.cuda.is_available()
            shape = (self.gpu_batch_size, self.seq_len)
            self._pinned = (torch.empty(shape, dtype=torch.long, pin_memory=pin),
                            torch.empty(shape, dtype=torch.long, pin_memory=pin))
        return self._pinned

    def next_batch(self) -> Tuple[Tensor, Tensor, Optional[Tensor]]:
        if self.grad_accum_mini_steps_per_shard_counter == self.grad_accum_mini_steps_per_shard:
            self._advance_shard()
        c = self.grad_accum_mini_steps_per_shard_counter
        if self.split == "val" and not self.shuffle_val_tokens:
            start = c * self.world_size * self.gpu_batch_size + self.rank * self.gpu_batch_size
            batch_starts = self.x_seq_starts[start: start + self.gpu_batch_size]
        else:
            batch_starts = self.gpu_x_seq_starts[c * self.gpu_batch_size: (c + 1) * self.gpu_batch_size]
        x, y = self._staging()
        x, y = x[: len(batch_starts)], y[: len(batch_starts)]
        for row, s in enumerate(batch_starts.tolist()):
            x[row] = self.tokens[s: s + self.seq_len]
            y[row] = self.tokens[s + 1: s + self.seq_len + 1]
        doc_ids = None
        if self.return_document_ids:
            is_eos = (x == self.eos_token_id).to(torch.int32)
            doc_ids = torch.cumsum(is_eos, dim=1, dtype=torch.int32) - is_eos
        self.grad_accum_mini_steps_per_shard_counter += 1
        return x, y, doc_ids


class SyntheticLoader:
    """Uniform random token ids in [0, vocab) from a seeded CPU generator, written into pinned
    staging buffers; same `next_batch`/`reset`/position surface as `DataLoader`.  Targets are the
    inputs shifted by one."""

    def __init__(self, gpu_batch_size: int, seq_len: int, world_size: int, rank: int, vocab_size: int,
                 seed: int = 0, split: str = "train", return_document_ids: bool = False) -> None:
        self.gpu_batch_size, self.seq_len, self.vocab_size = gpu_batch_size, seq_len, vocab_size
        self.seed, self.rank, self.world_size, self.split = seed, rank, world_size, split
        self.return_document_ids = return_document_ids
        self.epoch = self.current_shard_idx = 0
        self.grad_accum_mini_steps_per_shard_counter = 0
        pin = torch.cuda.is_available()
        self._buf = [torch.empty((gpu_batch_size, seq_len + 1), dtype=torch.long, pin_memory=pin) for _ in range(2)]
        self._flip = 0
        self.reset()

    def reset(self) -> None:
        self._gen = torch.Generator()
        self._gen.manual_seed(self.seed * 1_000_003 + self.rank + (7919 if self.split == "val" else 0))
        self.grad_accum_mini_steps_per_shard_counter = 0

    def next_batch(self) -> Tuple[Tensor, Tensor, Optional[Tensor]]:
        buf = self._buf[self._flip]
        self._flip ^= 1
        torch.randint(0, self.vocab_size, buf.shape, generator=self._gen, out=buf)
        self.grad_accum_mini_steps_per_shard_counter += 1
        x, y = buf[:, :-1], buf[:, 1:]
        doc_ids = torch.zeros_like(x, dtype=torch.int32) if self.return_document_ids else None
        return x, y, doc_ids
