#!/usr/bin/env python
"""Full GRPO step on a synthetic Llama: rollout (fused sampling) -> advantages -> policy
forward/backward on the native kernels -> deterministic gradient all-reduce (data parallel)
-> fused AdamW. Reports tokens/s of generated tokens and the loss of two identical runs.

    python benchmarks/bench_grpo_step.py --layers 4 --prompts 8 --group 8
    torchrun --nproc-per-node 8 benchmarks/bench_grpo_step.py --layers 32 --prompts 1 --group 64
    RL_ENGINE_PROFILE=basic python benchmarks/bench_grpo_step.py ...      # adds a per-operator table
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist

from _common import write_json
from kernel_align_b200.executors.trainer import GRPOTrainer
from kernel_align_b200.models.llama import LlamaConfig, LlamaModel


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--prompts", type=int, default=8, help="prompts per rank")
    ap.add_argument("--group", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--new-tokens", type=int, default=384)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--tiny", action="store_true", help="hidden 1024 instead of the 8B layer shapes")
    ap.add_argument("--micro-batch", type=int, default=None, help="sequences per backward pass of the policy update")
    ap.add_argument("--checkpoint-layers", action="store_true", help="recompute layer activations in backward")
    ap.add_argument("--zero", type=int, default=0, choices=[0, 1], help="1: shard the optimizer state over the ranks")
    ap.add_argument("--json-out", default=None)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank = dist.get_rank() if world > 1 else 0
    dev = torch.device("cuda", local)
    cfg = LlamaConfig.tiny(n_layers=args.layers) if args.tiny else LlamaConfig(n_layers=args.layers)

    def reward(prompts, new_tokens):
        return torch.randn(new_tokens.shape[0], device=new_tokens.device,
                           generator=torch.Generator(device=new_tokens.device).manual_seed(11 + rank))

    losses = []
    timings = []
    for run in range(2):
        from kernel_align_b200.parallel.tp_gemm import TPContext

        solo = TPContext.__new__(TPContext)
        solo.group, solo.rank, solo.world, solo.device, solo._arenas = None, 0, 1, dev, {}
        model = LlamaModel(cfg, tp=solo, seed=1, device=dev)
        model.checkpoint_layers = args.checkpoint_layers
        trainer = GRPOTrainer(model, reward, group_size=args.group, max_new_tokens=args.new_tokens, temperature=1.0,
                              top_k=50, top_p=0.95, lr=1e-6, seed=5, data_parallel=world > 1, micro_batch=args.micro_batch, zero_stage=args.zero)
        prompts = torch.randint(0, cfg.vocab_size, (args.prompts, args.prompt_len), device=dev,
                                generator=torch.Generator(device=dev).manual_seed(100 + rank))
        run_losses = []
        for step in range(args.steps):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = trainer.train_step(prompts)
            torch.cuda.synchronize()
            timings.append(time.perf_counter() - t0)
            run_losses.append(out["loss"].item())
        losses.append(run_losses)
        del trainer, model
        torch.cuda.empty_cache()
    tokens = args.prompts * args.group * args.new_tokens * world
    res = {"world": world, "layers": args.layers, "hidden": cfg.hidden, "vocab": cfg.vocab_size,
           "rollouts": args.prompts * args.group * world, "new_tokens": args.new_tokens,
           "step_s": min(timings), "tokens_per_s": tokens / min(timings),
           "loss_run0": losses[0], "loss_run1": losses[1], "bitwise_equal": losses[0] == losses[1]}
    from kernel_align_b200.utils.profiler import profiler

    if profiler.enabled:      # RL_ENGINE_PROFILE=basic|detailed: per-operator device time, slowest rank
        table = profiler.report(across_ranks=world > 1)
        if rank == 0:
            print(table)
    if rank == 0:
        print(json.dumps(res))
        write_json(args.json_out, res)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
