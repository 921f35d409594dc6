"""Token-indexed schedules (learning rate, sliding window, batch size).

Everything in training is scheduled by the number of training tokens processed so far rather
than by step, so a change of batch size does not distort the schedules.  Behavioural parity with
the reference `schedules/token.py:7-86`.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence


def get_token_based_adamw_lr(train_tokens_processed: int, lr_warmup_tokens: int,
                             lr_warmup_and_cosine_tokens: int, total_decay_tokens: int,
                             adamw_max_lr: float, adamw_hard_min_lr: float) -> float:
    """Linear warm-up, cosine decay to a hard floor, then flat (reference `schedules/token.py:7-22`)."""
    t = train_tokens_processed
    if t < lr_warmup_tokens:
        return (t + 1) * adamw_max_lr / lr_warmup_tokens
    if t >= lr_warmup_and_cosine_tokens:
        return adamw_hard_min_lr
    progress = (t - lr_warmup_tokens) / total_decay_tokens
    return adamw_hard_min_lr + 0.5 * (1.0 + math.cos(math.pi * progress)) * (adamw_max_lr - adamw_hard_min_lr)


def get_next_update_tokens(schedule_keys: Sequence[int], idx: int, max_tokens: int) -> int:
    """Token count at which entry `idx` of a schedule is replaced by the next one.

    When the first key is 0 the entry at `idx` is already active, so the next change is key
    `idx+1`; otherwise key `idx` itself is still pending (reference `schedules/token.py:25-27`).
    """
    nxt = idx + 1 if schedule_keys[0] == 0 else idx
    return schedule_keys[nxt] if nxt < len(schedule_keys) else max_tokens + 1


def enforce_flex_block_constraints(value: int, flex_block_size: int, enforce_even_blocks: bool) -> int:
    """Round a window down to whole attention blocks (at least one; optionally an even count)."""
    blocks = max(1, value // flex_block_size)
    if enforce_even_blocks:
        blocks = 2 * math.ceil(blocks / 2)
    return blocks * flex_block_size


def enforce_min_max_constraints(raw_values: Sequence[int], min_value: Optional[int],
                                max_value: Optional[int]) -> List[int]:
    """Clamp to [min, max] and force the sequence to be non-decreasing."""
    out: List[int] = []
    for v in raw_values:
        if min_value is not None:
            v = max(v, min_value)
        if max_value is not None:
            v = min(v, max_value)
        if out and v < out[-1]:
            v = out[-1]
        out.append(v)
    return out


def factor_schedule(start: int, factor: float, end: Optional[int] = None, count: Optional[int] = None) -> List[int]:
    """Geometric schedule: `start * factor**i` (count form) or repeated `int(x*factor)` up to `end`."""
    if count == 1:
        return [start]
    if count is not None:
        return [int(start * (factor ** i)) for i in range(count)]
    values, x = [], start
    while x <= end:
        values.append(x)
        x = int(x * factor)
    return values


def add_schedule(start: int, increment: int, end: Optional[int] = None, count: Optional[int] = None) -> List[int]:
    """Arithmetic schedule: `start + i*increment` for `count` entries, or up to and including `end`."""
    if count == 1:
        return [start]
    if count is not None:
        return [start + i * increment for i in range(count)]
    values, x = [], start
    while x <= end:
        values.append(x)
        x += increment
    return values


def custom_schedule(values: List[int]) -> List[int]:
    """Explicit list; a function so all three schedule kinds share one calling convention."""
    return values


SCHEDULE_FUNCTIONS = {f.__name__: f for f in (factor_schedule, add_schedule, custom_schedule)}
