#!/usr/bin/env python
"""CPU tier benchmark: the C++ CPU library against plain PyTorch on the CPU, on the small
correctness configuration (hidden [4, 64, 256] fp32, LM head [1024, 256], 16-row chunks) and a
few larger ones. Prints a table and, with --json-out, a JSON record. No GPU involved.

    python benchmarks/bench_cpu.py [--json-out cpu.json]
"""
from __future__ import annotations

import argparse
import time

import torch
from tabulate import tabulate

from _common import write_json
from kernel_align_b200.ops import cpu_ops


def timed(fn, reps=5):
    fn()
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    return min(ts) * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json-out", default=None)
    args = ap.parse_args()
    g = torch.Generator().manual_seed(0)
    rows, out = [], []
    for (G, L, d, V) in ((4, 64, 256, 1024), (8, 128, 512, 8192), (4, 64, 1024, 32768)):
        hidden = torch.randn(G * L, d, generator=g)
        weight = torch.randn(V, d, generator=g) * 0.02
        ids = torch.randint(0, V, (G * L,), generator=g)
        ours = cpu_ops.lmhead_logp_cpu(hidden, weight, ids, chunk_rows=16)
        ref = torch.log_softmax(hidden @ weight.t(), -1).gather(1, ids[:, None])[:, 0]
        one = cpu_ops.lmhead_logp_cpu(hidden[:L], weight, ids[:L], chunk_rows=16)
        t_ours = timed(lambda: cpu_ops.lmhead_logp_cpu(hidden, weight, ids, chunk_rows=16))
        t_ref = timed(lambda: torch.log_softmax(hidden @ weight.t(), -1).gather(1, ids[:, None]))
        rec = {"op": "lmhead_logp", "G": G, "L": L, "hidden": d, "vocab": V, "ms": t_ours, "torch_ms": t_ref,
               "max_abs_err": (ours - ref).abs().max().item(), "batch1_equals_batchG": bool(torch.equal(one, ours[:L]))}
        out.append(rec)
        rows.append([f"fused log-prob G={G} L={L} d={d} V={V}", f"{t_ours:.2f} ms", f"{t_ref:.2f} ms",
                     f"{rec['max_abs_err']:.1e}", rec["batch1_equals_batchG"]])
    for (G, V) in ((64, 128256), (256, 128256)):
        logits = (torch.randn(G, V, generator=g) * 2).to(torch.bfloat16)
        t_ours = timed(lambda: cpu_ops.sample_cpu(logits, inv_temperature=1 / 0.7, top_k=50, top_p=0.9, seed=1, step=0))

        def native():
            x = logits.float() / 0.7
            v, i = torch.topk(x, 50, -1)
            p = torch.softmax(v, -1)
            c = torch.cumsum(p, -1)
            p = torch.where(c - p > 0.9, torch.zeros(()), p)
            return i.gather(1, torch.multinomial(p / p.sum(-1, keepdim=True), 1))

        t_ref = timed(native)
        a = cpu_ops.sample_cpu(logits, inv_temperature=1 / 0.7, top_k=50, top_p=0.9, seed=1, step=0)
        b = cpu_ops.sample_cpu(logits[:7], inv_temperature=1 / 0.7, top_k=50, top_p=0.9, seed=1, step=0)
        rec = {"op": "sample", "G": G, "vocab": V, "ms": t_ours, "torch_ms": t_ref,
               "batch7_equals_batchG": bool(torch.equal(a[:7], b))}
        out.append(rec)
        rows.append([f"sampling k=50 p=0.9 G={G} V={V}", f"{t_ours:.2f} ms", f"{t_ref:.2f} ms", "-",
                     rec["batch7_equals_batchG"]])
    print(tabulate(rows, headers=["case", "C++ library", "PyTorch CPU", "max abs err", "batch invariant (bitwise)"],
                   tablefmt="github"))
    write_json(args.json_out, {"benchmark": "cpu", "threads": torch.get_num_threads(), "results": out})


if __name__ == "__main__":
    main()
