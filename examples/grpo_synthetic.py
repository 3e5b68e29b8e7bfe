#!/usr/bin/env python
"""A complete GRPO loop on a synthetic task, small enough for a CPU: the policy is rewarded for
emitting token ids that are multiples of a chosen number, and the mean reward climbs.

    python examples/grpo_synthetic.py --steps 30                  # CPU or one GPU
    torchrun --nproc-per-node 8 examples/grpo_synthetic.py        # data parallel, one process per GPU

Every piece is the library's: generation with the fused sampler, group-normalised advantages,
the clipped-ratio loss, backward through the native operators, the deterministic gradient
all-reduce and the fused AdamW.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from kernel_align_b200.executors.trainer import GRPOTrainer  # noqa: E402
from kernel_align_b200.models.llama import LlamaConfig, LlamaModel  # noqa: E402
from kernel_align_b200.parallel.strategy import build_model, make_layout  # noqa: E402
from kernel_align_b200.utils.logger import logger  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--prompts", type=int, default=4, help="prompts per rank and step")
    ap.add_argument("--group", type=int, default=8)
    ap.add_argument("--new-tokens", type=int, default=8)
    ap.add_argument("--multiple-of", type=int, default=4)
    ap.add_argument("--lr", type=float, default=3e-3)
    ap.add_argument("--layers", type=int, default=2)
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    cuda = torch.cuda.is_available()
    if world > 1:
        if cuda:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl" if cuda else "gloo")
    layout = make_layout("data_parallel")
    device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    cfg = LlamaConfig(vocab_size=512, hidden=256, n_layers=args.layers, n_heads=4, n_kv_heads=2, head_dim=128, ffn=512,
                      max_pos=256)
    model: LlamaModel = build_model(cfg, layout, seed=0, device=device)

    def reward(prompts, new_tokens):
        return (new_tokens % args.multiple_of == 0).float().mean(1)

    trainer = GRPOTrainer(model, reward, group_size=args.group, max_new_tokens=args.new_tokens, temperature=1.0,
                          lr=args.lr, seed=1, data_parallel=world > 1, dp_group=layout.dp_group)
    gen = torch.Generator().manual_seed(100 + layout.dp_rank)
    first = last = None
    for step in range(args.steps):
        prompts = torch.randint(0, cfg.vocab_size, (args.prompts, 8), generator=gen).to(device)
        out = trainer.train_step(prompts)
        r = out["reward_mean"].item()
        first = r if first is None else first
        last = r
        logger.info_on_rank(f"step {out['step']:3d}  loss {out['loss'].item():+.4f}  mean reward {r:.3f}  "
                            f"clip fraction {float(out['clip_fraction']):.3f}")
    logger.info_on_rank(f"mean reward: {first:.3f} -> {last:.3f} (chance level {1 / args.multiple_of:.3f})")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return first, last


if __name__ == "__main__":
    main()
