#!/usr/bin/env python
"""Sampling latency: fused sampler vs an unfused PyTorch implementation.

Same flags and defaults as the reference's benchmarks/benchmark_sampling.py:86-93
(``--g-sizes --vocab-size --top-k --top-p``), plus ``--dtype --temperature --seed --json-out``.
Timing is device time (CUDA events, warmed, median of 10, L2 flushed between calls), not a
single host-clock sample.
"""
from __future__ import annotations

import argparse

import torch
from tabulate import tabulate

from _common import time_cuda, write_json
from kernel_align_b200.kernels.sampling import SamplerBackend
from kernel_align_b200.platforms.device import device_ctx
from kernel_align_b200.utils.logger import logger


def native_sampling(logits, top_k=None, top_p=None, temperature=1.0):
    """Unfused PyTorch sampler (temperature -> top-k -> top-p -> softmax -> multinomial)."""
    x = logits.float() / temperature
    if top_k is not None:
        kth = torch.topk(x, min(top_k, x.size(-1)), dim=-1).values[:, -1:]
        x = x.masked_fill(x < kth, float("-inf"))
    if top_p is not None:
        srt, idx = torch.sort(x, descending=True, dim=-1)
        cum = torch.softmax(srt, -1).cumsum(-1)
        drop = cum > top_p
        drop[:, 1:] = drop[:, :-1].clone()
        drop[:, 0] = False
        x = x.masked_fill(torch.zeros_like(drop).scatter(1, idx, drop), float("-inf"))
    return torch.multinomial(torch.softmax(x, -1), 1).squeeze(-1)


def run_benchmark(args):
    if device_ctx.device.type != "cuda":
        raise SystemExit("this benchmark needs a CUDA device")
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}[args.dtype]
    sampler = SamplerBackend(seed=args.seed).to(device_ctx.device)
    rows, out = [], []
    logger.info_once(f"Sampling benchmark: V={args.vocab_size} top_k={args.top_k} top_p={args.top_p} "
                     f"T={args.temperature} dtype={args.dtype}")
    for g in [int(x) for x in args.g_sizes.split(",")]:
        gen = torch.Generator(device="cuda").manual_seed(args.seed)
        logits = (torch.randn(g, args.vocab_size, device="cuda", generator=gen) * args.sigma).to(dtype)
        t_native = time_cuda(lambda: native_sampling(logits, args.top_k, args.top_p, args.temperature))
        t_fused = time_cuda(lambda: sampler.sample(logits, top_k=args.top_k, top_p=args.top_p,
                                                   temperature=args.temperature, step=0))
        gbs = logits.numel() * logits.element_size() / t_fused / 1e6
        rows.append([g, f"{t_native:.3f} ms", f"{t_fused * 1e3:.1f} us", f"{t_native / t_fused:.1f}x", f"{gbs:.0f} GB/s"])
        out.append({"g": g, "native_ms": t_native, "fused_ms": t_fused, "logits_gb_per_s": gbs})
    print("\n" + "=" * 88)
    print(f"SAMPLING BENCHMARK (TopK={args.top_k}, TopP={args.top_p}, T={args.temperature}, {args.dtype})")
    print("=" * 88)
    print(tabulate(rows, headers=["Batch Size (G)", "PyTorch unfused", "Fused kernel", "Speedup", "Logits read"],
                   tablefmt="fancy_grid"))
    write_json(args.json_out, {"benchmark": "sampling", "args": vars(args), "results": out,
                               "device": torch.cuda.get_device_name()})


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--g-sizes", type=str, default="32,64,128,256")
    ap.add_argument("--vocab-size", type=int, default=128256)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--sigma", type=float, default=2.0, help="std of the synthetic logits")
    ap.add_argument("--dtype", type=str, default="bfloat16", choices=["float32", "bfloat16", "float16"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--json-out", type=str, default=None)
    run_benchmark(ap.parse_args())
