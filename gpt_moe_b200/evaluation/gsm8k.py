"""GSM8K evaluation: few-shot greedy generation, `#### number` extraction, rank-strided examples.

Behaviour follows the reference (`evaluation/gsm8k.py:15-148`): the prompt starts with an instruction
line and the first N training problems with their worked solutions (calculator annotations
`<<...>>` removed); generation is greedy on a fixed-shape padded buffer without a KV cache (the
whole prefix is re-run for every new token) and a sequence stops at the first end-of-text token
or at a complete `#### number` line; the extracted decimal must equal the reference answer.
Data: the `datasets` hub, or `$GSM8K_DIR/{train,test}.jsonl` with keys question / answer.
"""
from __future__ import annotations

import json
import os
import re
from decimal import Decimal
from typing import Dict, List, Optional

import torch

from ..parallel import dist_utils as du
from ..runtime.precision import linear_precision_phase

_ANSWER = re.compile(r"(?:^|\n)####[ \t]*(-?[0-9]+(?:,[0-9]{3})*(?:\.[0-9]+)?)[ \t]*(?:\r?\n|$)")


def extract_gsm8k_answer(completion: str) -> Optional[Decimal]:
    match = _ANSWER.search(completion)
    return Decimal(match.group(1).replace(",", "")) if match else None


def _load_split(split: str) -> List[Dict]:
    folder = os.environ.get("GSM8K_DIR")
    if folder:
        with open(os.path.join(folder, f"{split}.jsonl")) as f:
            return [json.loads(line) for line in f if line.strip()]
    from datasets import load_dataset
    return list(load_dataset("openai/gsm8k", "main", split=split))


def load_gsm8k_data(run) -> None:
    cfg = run.training_config
    if cfg.gsm8k_interval != -1 and cfg.gsm8k_interval <= 0:
        raise ValueError("gsm8k_interval must be -1 or positive")
    if cfg.gsm8k_max_examples != -1 and cfg.gsm8k_max_examples <= 0:
        raise ValueError("gsm8k_max_examples must be -1 or positive")
    if cfg.gsm8k_num_shots < 0 or cfg.gsm8k_max_new_tokens <= 0 or cfg.gsm8k_examples_per_batch <= 0:
        raise ValueError("GSM8K requires nonnegative shots and positive token and batch limits")
    if not run.raw_gpt_model.is_causal:
        raise ValueError("GSM8K generation requires is_causal=True")
    prefix = "Solve each problem. End your answer with a line containing #### followed by the final number.\n\n"
    if cfg.gsm8k_num_shots:
        for ex in _load_split("train")[: cfg.gsm8k_num_shots]:
            prefix += f"Question: {ex['question']}\nAnswer: {re.sub(r'<<.*?>>', '', ex['answer'])}\n\n"
    test = _load_split("test")
    total = len(test) if cfg.gsm8k_max_examples <= 0 else min(len(test), cfg.gsm8k_max_examples)
    indices = range(total) if run.parallel_mode == "pp" else range(run.rank, total, run.world_size)
    run.local_gsm8k_examples = []
    for i in indices:
        answer = extract_gsm8k_answer(test[i]["answer"])
        if answer is None:
            raise ValueError(f"GSM8K test example {i} has no numeric reference answer")
        run.local_gsm8k_examples.append((run.tokenizer.encode(f"{prefix}Question: {test[i]['question']}\nAnswer:"), answer))
    longest = torch.tensor(max((len(ids) for ids, _ in run.local_gsm8k_examples), default=0), dtype=torch.long, device=run.device)
    if du.is_dist():
        torch.distributed.all_reduce(longest, op=torch.distributed.ReduceOp.MAX)
    if int(longest) + cfg.gsm8k_max_new_tokens > run.raw_gpt_model.max_seq_len:
        raise ValueError("GSM8K prompts and generation exceed max_seq_len; reduce gsm8k_num_shots or gsm8k_max_new_tokens")
    if run.master_process:
        message = (f"GSM8K: {total:,} test examples | first {cfg.gsm8k_num_shots} train examples as shots | "
                   f"greedy decoding | max new tokens: {cfg.gsm8k_max_new_tokens} | final answer: #### number")
        print(message)
        run.log_buffer.append(message)


@torch.no_grad()
def greedy_generate(run, prompts: List[List[int]], max_new_tokens: int, stop_on_answer: bool = True) -> List[str]:
    """Greedy continuation of every prompt on one padded [batch, max_len] buffer; returns the decoded completions."""
    raw, tok = run.raw_gpt_model, run.tokenizer
    eot = getattr(tok, "eot_token", raw.gpt_config.eos_token_id)
    lengths = [len(p) for p in prompts]
    width = max(lengths) + max_new_tokens
    ids = torch.full((len(prompts), width), raw.pad_token_id, dtype=torch.long, device=run.device)
    for i, p in enumerate(prompts):
        ids[i, : len(p)] = torch.tensor(p, dtype=torch.long, device=run.device)
    cursor = torch.tensor(lengths, device=run.device)
    done = torch.zeros(len(prompts), dtype=torch.bool, device=run.device)
    rows = torch.arange(len(prompts), device=run.device)
    for _ in range(max_new_tokens):
        upto = int(cursor.max())
        with run.ctx:
            logits = run.forward(raw, ids[:, :upto], attn_mask=None, ignore_doc_mask=True)
        if run.parallel_mode == "pp":
            nxt = torch.zeros(len(prompts), dtype=torch.long, device=run.device)
            if run.rank == run.world_size - 1:
                nxt = logits[rows, cursor - 1].argmax(dim=-1)
            torch.distributed.broadcast(nxt, src=run.world_size - 1)
        else:
            nxt = logits[rows, cursor - 1].argmax(dim=-1)
        nxt = torch.where(done, torch.full_like(nxt, raw.pad_token_id), nxt)
        ids[rows, cursor.clamp(max=width - 1)] = nxt
        cursor = torch.where(done, cursor, cursor + 1)
        done |= nxt == eot
        if stop_on_answer:
            for i in (~done).nonzero().flatten().tolist():
                text = tok.decode(ids[i, lengths[i]: int(cursor[i])].tolist())
                if _ANSWER.search(text) and text.endswith("\n"):
                    done[i] = True
        if bool(done.all()):
            break
    return [tok.decode([t for t in ids[i, lengths[i]: int(cursor[i])].tolist() if t != eot]) for i in range(len(prompts))]


def evaluate_gsm8k(run) -> float:
    cfg = run.training_config
    run.gpt_model.eval()
    correct = 0
    examples = run.local_gsm8k_examples
    with linear_precision_phase(run.raw_gpt_model, "evaluation"):
        for start in range(0, len(examples), cfg.gsm8k_examples_per_batch):
            batch = examples[start: start + cfg.gsm8k_examples_per_batch]
            completions = greedy_generate(run, [ids for ids, _ in batch], cfg.gsm8k_max_new_tokens)
            correct += sum(int(extract_gsm8k_answer(text) == answer) for text, (_, answer) in zip(completions, batch))
    counts = torch.tensor([correct, len(examples)], dtype=torch.long, device=run.device)
    if run.parallel_mode != "pp":
        du.all_reduce(counts)
    run.gpt_model.train()
    return counts[0].item() / max(counts[1].item(), 1)
