#!/usr/bin/env python
"""The parallel layouts on one small model: run under torchrun with 2, 4 or 8 processes
(GPUs when present, otherwise CPU processes over gloo).

    torchrun --nproc-per-node 4 examples/parallel_layouts.py --strategy hybrid --tp 2
    torchrun --nproc-per-node 2 examples/parallel_layouts.py --strategy model_parallel
    torchrun --nproc-per-node 2 examples/parallel_layouts.py --strategy pipeline_parallel

Every layout computes the per-token log-probabilities of the same batch; rank 0 prints their
checksum, which is the same number for every layout up to bf16 rounding of the column-parallel
products (and bitwise the same between `data_parallel` and `pipeline_parallel`).
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from kernel_align_b200.models.llama import LlamaConfig  # noqa: E402
from kernel_align_b200.parallel.pipeline import pipeline_logp_step  # noqa: E402
from kernel_align_b200.parallel.strategy import build_model, make_layout  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--strategy", default="hybrid",
                    choices=["data_parallel", "model_parallel", "pipeline_parallel", "hybrid"])
    ap.add_argument("--tp", type=int, default=None)
    ap.add_argument("--pp", type=int, default=None)
    args = ap.parse_args()
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl" if cuda else "gloo")
    device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    layout = make_layout(args.strategy, tp_size=args.tp, pp_size=args.pp)
    cfg = LlamaConfig(vocab_size=512, hidden=256, n_layers=4, n_heads=4, n_kv_heads=2, head_dim=128, ffn=512, max_pos=256)
    model = build_model(cfg, layout, seed=1, device=device)
    ids = torch.randint(0, cfg.vocab_size, (4, 24), generator=torch.Generator().manual_seed(2)).to(device)
    with torch.no_grad():
        if layout.pp_size > 1:
            logp, _ = pipeline_logp_step(model, ids, ids, n_micro=2)
        else:
            logp = model.token_logp(ids, ids)
    checksum = torch.zeros(1, dtype=torch.float64, device=device)
    if logp is not None:                       # pipeline: only the last stage holds the result
        checksum += logp.double().sum()
    if layout.pp_size > 1:
        dist.all_reduce(checksum)              # the other stages contribute zero
    if dist.get_rank() == 0:
        print(f"{args.strategy}: tp={layout.tp_size} pp={layout.pp_size} dp={layout.dp_size}  "
              f"sum of log-probs = {checksum.item():.4f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
