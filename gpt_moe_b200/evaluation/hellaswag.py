"""HellaSwag evaluation.

One-shot prompted multiple choice: the context is preceded by one worked training example, each of
the four endings is appended in turn, and the ending with the highest length-normalised
log-probability of its own tokens wins (reference `evaluation/hellaswag.py:326-473`; the
`one_shot` variant scores the letters A-D instead, `:154-323`).  Examples are sharded over
data-parallel ranks; correct/processed counts are summed with an all-reduce.

Data comes from the `datasets` hub when reachable, or from JSONL files
(`hellaswag_train.jsonl`, `hellaswag_val.jsonl` with keys ctx / endings / label) under
`$HELLASWAG_DIR`.  Token log-probabilities are gathered on the device in one indexing op per batch
instead of one `.item()` per token.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Sequence

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..parallel import dist_utils as du
from ..runtime.precision import linear_precision_phase


def _load_split(split: str) -> List[Dict]:
    folder = os.environ.get("HELLASWAG_DIR")
    if folder:
        name = {"train": "hellaswag_train.jsonl", "validation": "hellaswag_val.jsonl"}[split]
        with open(os.path.join(folder, name)) as f:
            return [json.loads(line) for line in f if line.strip()]
    from datasets import load_dataset
    return list(load_dataset("hellaswag", split=split))


def load_hellaswag_data(run) -> None:
    run.hellaswag_train_dataset = _load_split("train")
    val = _load_split("validation")
    total = len(val)
    if run.parallel_mode == "pp":
        start, end = 0, total
    else:
        per_rank = (total + run.world_size - 1) // run.world_size
        start, end = run.rank * per_rank, min((run.rank + 1) * per_rank, total)
    run.local_hellaswag_val_dataset = val[start:end]
    message = f"[rank {run.rank}] gets HellaSwag sentences {start:,} to {end - 1:,}"
    print(message)
    messages = [message]
    if du.is_dist() and run.world_size > 1:
        messages = [None] * run.world_size
        dist.all_gather_object(messages, message)
    if run.master_process:
        run.log_buffer.extend(messages)
    du.barrier()


def one_shot_prefix(example: Dict) -> str:
    e = example["endings"]
    return (f"Sentence to pick the continuation of: {example['ctx']}\nContinuation options:\n"
            f"A) {e[0]}\nB) {e[1]}\nC) {e[2]}\nD) {e[3]}\n"
            f"Correct continuation: {chr(ord('A') + int(example['label']))})\n\n")


def continuation_scores(logits: torch.Tensor, input_ids: torch.Tensor, prefix_lengths: Sequence[int],
                        true_lengths: Sequence[int]) -> torch.Tensor:
    """Mean log-probability of tokens [prefix_len, true_len) of every row, predicted from the previous position."""
    log_probs = F.log_softmax(logits.float(), dim=-1)
    n, t = input_ids.shape
    token_lp = log_probs[:, :-1].gather(-1, input_ids[:, 1:, None]).squeeze(-1)          # [n, t-1]: log p(token j+1 | <= j)
    pos = torch.arange(1, t, device=input_ids.device)[None, :]
    pre = torch.as_tensor(prefix_lengths, device=input_ids.device)[:, None]
    end = torch.as_tensor(true_lengths, device=input_ids.device)[:, None]
    mask = (pos >= pre) & (pos < end)
    return (token_lp * mask).sum(dim=1) / mask.sum(dim=1).clamp(min=1)


def _finish(run, correct: int, processed: int, total_local: int, name: str) -> float:
    local = f"[rank {run.rank}] {name} local acc: {correct} / {total_local} = {correct / max(total_local, 1):.4f}"
    print(local)
    messages = [local]
    if du.is_dist() and run.world_size > 1:
        messages = [None] * run.world_size
        dist.all_gather_object(messages, local)
    if run.master_process:
        run.log_buffer.extend(messages)
    counts = torch.tensor([correct, processed], dtype=torch.long, device=run.device)
    du.all_reduce(counts)
    run.gpt_model.train()
    return counts[0].item() / max(counts[1].item(), 1)


def evaluate_hellaswag_standard(run, hellaswag_examples_per_batch: int = 16) -> float:
    raw, tok = run.raw_gpt_model, run.tokenizer
    examples = run.local_hellaswag_val_dataset
    prefix = one_shot_prefix(run.hellaswag_train_dataset[0])
    per_batch = max(1, hellaswag_examples_per_batch)
    multiple = raw.flex_block_size if getattr(raw, "use_flex_attention", False) and hasattr(raw, "flex_block_size") else 8
    correct = processed = 0
    run.gpt_model.eval()
    with linear_precision_phase(raw, "evaluation"), torch.no_grad():
        for start in range(0, len(examples), per_batch):
            batch = examples[start: start + per_batch]
            seqs, prefix_lens = [], []
            for ex in batch:
                ctx_ids = tok.encode(prefix + f"Sentence to pick the continuation of: {ex['ctx']}\n")
                for ending in ex["endings"][:4]:
                    ids = ctx_ids + tok.encode(f" {ending}")
                    if len(ids) > raw.max_seq_len:
                        raise ValueError(f"HellaSwag sequence too long ({len(ids)} > {raw.max_seq_len})")
                    seqs.append(ids)
                    prefix_lens.append(len(ctx_ids))
            alloc = min(raw.max_seq_len, math.ceil(max(len(s) for s in seqs) / multiple) * multiple)
            ids = torch.full((len(seqs), alloc), raw.pad_token_id, dtype=torch.long)
            for i, s in enumerate(seqs):
                ids[i, : len(s)] = torch.tensor(s, dtype=torch.long)
            ids = ids.to(run.device)
            with run.ctx:      # causal attention: real tokens never see the right padding, so no padding mask is needed
                logits = run.forward(raw, ids, attn_mask=None, ignore_doc_mask=True)
            if run.parallel_mode == "pp" and run.rank != run.world_size - 1:
                continue
            scores = continuation_scores(logits, ids, prefix_lens, [len(s) for s in seqs]).view(len(batch), 4)
            picks = scores.argmax(dim=1).tolist()
            correct += sum(int(p == int(ex["label"])) for p, ex in zip(picks, batch))
            processed += len(batch)
    return _finish(run, correct, processed, len(examples), "HellaSwag")


def evaluate_hellaswag_one_shot(run, hellaswag_examples_per_batch: int = 16) -> float:
    """Letter-scoring variant: the prompt lists options A-D and the model's next-token probabilities of
    " A".." D" after "Correct continuation:" are compared."""
    raw, tok = run.raw_gpt_model, run.tokenizer
    examples = run.local_hellaswag_val_dataset
    prefix = one_shot_prefix(run.hellaswag_train_dataset[0])
    letters = [tok.encode(f" {c}")[-1] for c in "ABCD"]
    per_batch = max(1, hellaswag_examples_per_batch)
    correct = processed = 0
    run.gpt_model.eval()
    with linear_precision_phase(raw, "evaluation"), torch.no_grad():
        for start in range(0, len(examples), per_batch):
            batch = examples[start: start + per_batch]
            seqs = []
            for ex in batch:
                e = ex["endings"]
                seqs.append(tok.encode(prefix + f"Sentence to pick the continuation of: {ex['ctx']}\nContinuation options:\n"
                                       f"A) {e[0]}\nB) {e[1]}\nC) {e[2]}\nD) {e[3]}\nCorrect continuation:")[-raw.max_seq_len:])
            alloc = min(raw.max_seq_len, math.ceil(max(len(s) for s in seqs) / 8) * 8)
            ids = torch.full((len(seqs), alloc), raw.pad_token_id, dtype=torch.long)
            for i, s in enumerate(seqs):
                ids[i, : len(s)] = torch.tensor(s, dtype=torch.long)
            ids = ids.to(run.device)
            with run.ctx:
                logits = run.forward(raw, ids, attn_mask=None, ignore_doc_mask=True)
            if run.parallel_mode == "pp" and run.rank != run.world_size - 1:
                continue
            last = torch.tensor([len(s) - 1 for s in seqs], device=run.device)
            final = logits[torch.arange(len(seqs), device=run.device), last].float()
            picks = final[:, letters].argmax(dim=1).tolist()
            correct += sum(int(p == int(ex["label"])) for p, ex in zip(picks, batch))
            processed += len(batch)
    return _finish(run, correct, processed, len(examples), "HellaSwag one-shot")
