#!/usr/bin/env python
"""GRPO log-prob operator benchmark: peak extra VRAM and latency versus group size.

Same flags and defaults as the reference's benchmarks/benchmark_grpo_op.py:109-119
(``--g-sizes --seq-len --vocab-size``), plus ``--hidden --dtype --json-out``. Three columns:
  native      torch.log_softmax + gather on materialised logits (the reference's comparison)
  logits op   SamplerBackend.compute_logp on the same logits (one streaming pass, no temporary)
  fused       SamplerBackend.fused_logp from hidden states (logits never materialised)
"Extra VRAM" is the peak allocated above the op's inputs; timings are device time.
"""
from __future__ import annotations

import argparse

import torch
from tabulate import tabulate

from _common import time_cuda, write_json
from kernel_align_b200.kernels.sampling import SamplerBackend
from kernel_align_b200.ops import fused_logp
from kernel_align_b200.platforms.device import device_ctx
from kernel_align_b200.utils.logger import logger


def _peak_extra(fn):
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    fn()
    torch.cuda.synchronize()
    return (torch.cuda.max_memory_allocated() - base) / 2**30


def run_benchmark(args):
    if device_ctx.device.type != "cuda":
        raise SystemExit("this benchmark needs a CUDA device")
    dtype = {"bfloat16": torch.bfloat16, "float16": torch.float16}[args.dtype]
    sampler = SamplerBackend().to(device_ctx.device)
    gen = torch.Generator(device="cuda").manual_seed(0)
    weight = torch.empty(args.vocab_size, args.hidden, device="cuda", dtype=torch.bfloat16)
    for i in range(0, args.vocab_size, 16384):
        n = min(16384, args.vocab_size - i)
        weight[i:i + n] = (torch.randn(n, args.hidden, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
    fused_ws = fused_logp.workspace_bytes(args.vocab_size) / 2**30
    rows, out = [], []
    for g in [int(x) for x in args.g_sizes.split(",")]:
        n = g * args.seq_len
        hidden = torch.randn(n, args.hidden, device="cuda", generator=gen).to(torch.bfloat16)
        ids = torch.randint(0, args.vocab_size, (g, args.seq_len), device="cuda", generator=gen)
        rec = {"g": g, "rows": n}
        sampler.fused_logp(hidden, weight, ids.view(-1))  # allocate the persistent workspace
        rec["fused_extra_gib"] = _peak_extra(lambda: sampler.fused_logp(hidden, weight, ids.view(-1))) + fused_ws
        rec["fused_ms"] = time_cuda(lambda: sampler.fused_logp(hidden, weight, ids.view(-1)), iters=5,
                                    flush_l2=False)
        try:
            logits = torch.matmul(hidden, weight.t()).view(g, args.seq_len, args.vocab_size).to(dtype)
            rec["logits_gib"] = logits.numel() * 2 / 2**30
            rec["op_extra_gib"] = _peak_extra(lambda: sampler.compute_logp(logits, ids))
            rec["op_ms"] = time_cuda(lambda: sampler.compute_logp(logits, ids), iters=5, flush_l2=False)
            try:
                def native():
                    return torch.log_softmax(logits, -1).gather(-1, ids.unsqueeze(-1))
                rec["native_extra_gib"] = _peak_extra(native)
                rec["native_ms"] = time_cuda(native, iters=5, flush_l2=False)
            except torch.cuda.OutOfMemoryError:
                rec["native_extra_gib"] = rec["native_ms"] = None
            del logits
        except torch.cuda.OutOfMemoryError:
            logger.error(f"OOM materialising logits for G={g}")
        torch.cuda.empty_cache()
        f = lambda v, u: "OOM" if v is None else f"{v:.2f} {u}"  # noqa: E731
        rows.append([g, f(rec.get("native_extra_gib"), "GiB"), f(rec.get("op_extra_gib"), "GiB"),
                     f(rec["fused_extra_gib"], "GiB"), f(rec.get("native_ms"), "ms"), f(rec.get("op_ms"), "ms"),
                     f(rec["fused_ms"], "ms"), f"{n / rec['fused_ms'] * 1e3 / 1e6:.2f} M tok/s"])
        out.append(rec)
    print("\n" + "=" * 120)
    print(f"GRPO LOG-PROB OPERATOR BENCHMARK | {torch.cuda.get_device_name()} | SeqLen={args.seq_len} "
          f"Vocab={args.vocab_size} Hidden={args.hidden}")
    print("=" * 120)
    print(tabulate(rows, headers=["G", "native extra", "logits-op extra", "fused extra (incl. workspace)",
                                  "native", "logits op", "fused (from hidden)", "fused throughput"],
                   tablefmt="fancy_grid"))
    print("native / logits op start from materialised logits (a [G, L, V] tensor on top of the figures shown);\n"
          "fused starts from hidden states and includes the LM-head GEMM.")
    write_json(args.json_out, {"benchmark": "grpo_op", "args": vars(args), "results": out,
                               "device": torch.cuda.get_device_name()})


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description="GRPO log-prob operator benchmark")
    ap.add_argument("--g-sizes", type=str, default="8,16,32,64,128")
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--vocab-size", type=int, default=128256)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--dtype", type=str, default="bfloat16", choices=["bfloat16", "float16"])
    ap.add_argument("--json-out", type=str, default=None)
    run_benchmark(ap.parse_args())
