"""Training entry point: `torchrun --standalone --nproc_per_node=N train.py [--preset NAME] [--set k=v ...]`.

Same launch contract as the reference script (`train.py:1-758`, `experiments/run.py:120-122`):
one process per GPU, RANK / LOCAL_RANK / WORLD_SIZE from the environment.  Without arguments the
two configuration dataclasses are used with their defaults, as in the reference; `--preset` and
`--set model.<field>=v` / `--set training.<field>=v` replace its edit-the-source workflow.
A single process without torchrun also works (world size 1).
"""
import os

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

import argparse

from gpt_moe_b200.config import apply_overrides, get_preset
from gpt_moe_b200.runtime.trainer import Trainer


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="default")
    ap.add_argument("--set", dest="overrides", action="append", default=[])
    ap.add_argument("--steps", type=int, default=None, help="stop after this many steps")
    ap.add_argument("--device", default=None, choices=[None, "cpu", "cuda"])
    args = ap.parse_args()
    gpt_config, training_config = get_preset(args.preset)
    apply_overrides(gpt_config, training_config, args.overrides)
    trainer = Trainer(gpt_config, training_config, device_type=args.device)
    try:
        trainer.fit(max_steps=args.steps)
    finally:
        trainer.close()


if __name__ == "__main__":
    main()
