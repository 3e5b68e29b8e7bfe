#!/usr/bin/env python
"""The four fused tensor-parallel GEMMs of a Llama-3-8B layer, one by one, on N GPUs (torchrun).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmarks/bench_tp_ops.py --tokens 32768 --json-out out.json

Per operator: the fused kernel (GEMM -> reduce-scatter, all-gather -> GEMM over peer memory),
cuBLAS + NCCL doing the same (``all_gather_into_tensor`` + matmul, matmul +
``reduce_scatter_tensor``), and the plain GEMM of the same shape without any exchange. CUDA
events, max over ranks, median. The roofline of a fused operator is the slower of its tensor
work at the measured cuBLAS peak and the bytes that have to cross NVLink (bf16 rows of the other
ranks in, or bf16 partial tiles out: (N - 1) / N of the tensor) at the measured 770 GB/s per
direction; the fraction reported is roofline time / achieved time.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

from _common import ROOT, write_json
from kernel_align_b200.ops import gemm
from kernel_align_b200.parallel.tp_gemm import TPContext, all_gather_gemm, gemm_reduce_scatter

NVLINK_GBS = 770.0


def peak_tflops() -> float:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"])
    return 1590.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--iters", type=int, default=8)
    ap.add_argument("--json-out", default=None)
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", local)
    g = torch.Generator(device=dev).manual_seed(0)
    tp = TPContext()
    t = args.tokens
    tf = peak_tflops()

    def r(*shape, sc=1.0):
        return (torch.randn(*shape, device=dev, generator=g) * sc).to(torch.bfloat16)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(args.iters):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            x = torch.tensor([e0.elapsed_time(e1)], device=dev)
            dist.all_reduce(x, op=dist.ReduceOp.MAX)
            ts.append(x.item())
        return statistics.median(ts)

    xl, xfull = r(t // world, 4096), r(t, 4096)
    wqkv, wgu = r(6144 // world, 4096, sc=0.02), r(28672 // world, 4096, sc=0.02)
    a, wo = r(t, 4096 // world), r(4096, 4096 // world, sc=0.02)
    f, wd = r(t, 14336 // world), r(4096, 14336 // world, sc=0.02)

    def nccl_ag_gemm(x, w):
        out = torch.empty(world * x.shape[0], x.shape[1], dtype=x.dtype, device=dev)
        dist.all_gather_into_tensor(out, x)
        return out @ w.t()

    def nccl_gemm_rs(x, w):
        y = x @ w.t()
        out = torch.empty(y.shape[0] // world, y.shape[1], dtype=y.dtype, device=dev)
        dist.reduce_scatter_tensor(out, y)
        return out

    cases = [
        ("qkv all-gather -> GEMM", lambda: all_gather_gemm(xl, wqkv, tp), lambda: nccl_ag_gemm(xl, wqkv),
         lambda: gemm.gemm_bi(xfull, wqkv), 2.0 * t * wqkv.shape[0] * 4096, t * 4096 * 2),
        ("gate_up all-gather -> GEMM", lambda: all_gather_gemm(xl, wgu, tp), lambda: nccl_ag_gemm(xl, wgu),
         lambda: gemm.gemm_bi(xfull, wgu), 2.0 * t * wgu.shape[0] * 4096, t * 4096 * 2),
        ("o_proj GEMM -> reduce-scatter", lambda: gemm_reduce_scatter(a, wo, tp, residual=xl), lambda: nccl_gemm_rs(a, wo),
         lambda: gemm.gemm_bi(a, wo), 2.0 * t * 4096 * a.shape[1], t * 4096 * 2),
        ("down GEMM -> reduce-scatter", lambda: gemm_reduce_scatter(f, wd, tp, residual=xl), lambda: nccl_gemm_rs(f, wd),
         lambda: gemm.gemm_bi(f, wd), 2.0 * t * 4096 * f.shape[1], t * 4096 * 2),
    ]
    out = []
    for name, ours, theirs, plain, flops, tensor_bytes in cases:
        t_fused, t_lib, t_plain = timed(ours), timed(theirs), timed(plain)
        link_ms = tensor_bytes * (world - 1) / world / NVLINK_GBS / 1e6
        mma_ms = flops / tf / 1e9
        roof = max(link_ms, mma_ms)
        row = {"op": name, "fused_ms": t_fused, "cublas_nccl_ms": t_lib, "plain_gemm_ms": t_plain,
               "roofline_ms": roof, "roofline_bound": "nvlink" if link_ms >= mma_ms else "tensor",
               "roofline_fraction": roof / t_fused, "vs_cublas_nccl": t_lib / t_fused}
        out.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    gemm.check_status(dev)
    if rank == 0:
        write_json(args.json_out, {"world": world, "tokens": t, "peak_tflops": tf, "nvlink_gbs": NVLINK_GBS, "results": out})
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
