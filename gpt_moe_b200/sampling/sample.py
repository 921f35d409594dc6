"""Text sampling: batched temperature / top-k / top-p sampling on a pre-allocated padded buffer.

Same behaviour as the reference (`sampling/sample.py:13-191`): prompts are truncated to leave room
for `max_new_tokens`, the whole batch lives in one `[n, alloc_len]` tensor (rounded up to the
attention block size) that is re-run from the start for every new token (no KV cache), sampling
uses the "sampling" precision phase, and under pipeline parallelism the last stage draws the tokens
and broadcasts them.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..runtime.precision import linear_precision_phase


def get_sample_token_count(step: int, base: int = 5, step_interval: int = 1000, max_tokens: int = 50) -> int:
    return min(base + (step // step_interval) * base, max_tokens)


def filter_logits(logits: torch.Tensor, top_k: Optional[int], top_p: Optional[float]) -> torch.Tensor:
    """Mask logits outside the top-k set and outside the smallest set whose probability mass reaches top-p."""
    if top_k is not None and top_k > 0:
        kth = torch.topk(logits, min(top_k, logits.size(-1)), dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p is not None and 0.0 < top_p < 1.0:
        sorted_logits, order = torch.sort(logits, dim=-1, descending=True)
        mass = torch.softmax(sorted_logits, dim=-1).cumsum(dim=-1)
        drop = mass - torch.softmax(sorted_logits, dim=-1) >= top_p        # keep the token that crosses the threshold
        sorted_logits = sorted_logits.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, order, sorted_logits)
    return logits


@torch.no_grad()
def sample(run, sample_sequences: Sequence[str], max_new_tokens: int = 5, temperature: float = 0.7,
           top_k: Optional[int] = None, top_p: Optional[float] = None) -> List[str]:
    raw, tok = run.raw_gpt_model, run.tokenizer
    run.gpt_model.eval()
    outputs: List[str] = []
    with linear_precision_phase(raw, "sampling"):
        limit = raw.max_seq_len - max_new_tokens
        prompts = [tok.encode(text)[:limit] for text in sample_sequences]
        lengths = [len(p) for p in prompts]
        multiple = 8
        alloc = min(raw.max_seq_len, math.ceil((max(lengths) + max_new_tokens) / multiple) * multiple)
        ids = torch.full((len(prompts), alloc), raw.pad_token_id, dtype=torch.long, device=run.device)
        for i, p in enumerate(prompts):
            ids[i, : len(p)] = torch.tensor(p, dtype=torch.long, device=run.device)
        cursor = torch.tensor(lengths, device=run.device)
        rows = torch.arange(len(prompts), device=run.device)
        for _ in range(max_new_tokens):
            upto = int(cursor.max())
            with run.ctx:
                logits = run.forward(raw, ids[:, :upto], attn_mask=None, ignore_doc_mask=True)
            last_stage = run.parallel_mode != "pp" or run.rank == run.world_size - 1
            nxt = torch.zeros(len(prompts), dtype=torch.long, device=run.device)
            if last_stage:
                step_logits = logits[rows, cursor - 1].float()
                if temperature <= 0:
                    nxt = step_logits.argmax(dim=-1)
                else:
                    probs = F.softmax(filter_logits(step_logits / temperature, top_k, top_p), dim=-1)
                    nxt = torch.multinomial(probs, num_samples=1).squeeze(-1)
            if run.parallel_mode == "pp":
                dist.broadcast(nxt, src=run.world_size - 1)
            ids[rows, cursor] = nxt
            cursor = cursor + 1
        outputs = [tok.decode(ids[i, : int(cursor[i])].tolist()) for i in range(len(prompts))]
    if run.master_process:
        for text in outputs:
            message = f"sample: {text!r}"
            print(message)
            run.log_buffer.append(message)
    run.gpt_model.train()
    return outputs
