#!/usr/bin/env python
"""Deterministic all-reduce against NCCL on N GPUs of one node (launch with torchrun).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_allreduce.py

For each size: the fixed-order peer-memory all-reduce (``csrc/sm100/allreduce_det.cu``, in place
on a symmetric vector) and ``torch.distributed.all_reduce`` (NCCL) on a tensor of the same
size, CUDA events, max over ranks, median of the timed calls. Bus bandwidth is
``2 (N - 1) / N * bytes / time``; the roofline of the peer-memory kernel is the NVLink rate per
direction (every rank pulls (N - 1) / N of the vector and pushes as much). Also times a
4096-element call right after the largest one (the small-tensor path must not inherit its size).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

from _common import ROOT, write_json  # noqa: F401
from kernel_align_b200.parallel.collectives import SymmetricVector, all_reduce_det


def timed(fn, iters, world):
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ts.append(t.item())
    return statistics.median(ts)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", default="1,16,64,256,1024")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json-out", default=None)
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    rows = []
    for mb in [int(x) for x in args.sizes_mb.split(",")]:
        n = mb * (1 << 20) // 4
        vec = SymmetricVector(n, torch.float32)
        vec.tensor.normal_()
        ref = torch.randn(n, device="cuda")
        t_own = timed(lambda: vec.all_reduce_(), args.iters, world)
        t_nccl = timed(lambda: dist.all_reduce(ref), args.iters, world)
        vec.check()
        bus = 2 * (world - 1) / world * n * 4
        rows.append({"mbytes": mb, "det_ms": t_own, "nccl_ms": t_nccl, "det_busbw_gbs": bus / t_own / 1e6,
                     "nccl_busbw_gbs": bus / t_nccl / 1e6, "det_vs_nccl": t_nccl / t_own})
        if rank == 0:
            print(json.dumps(rows[-1]), flush=True)
        del vec, ref
        torch.cuda.empty_cache()
    big = torch.randn(64 << 20, device="cuda")         # 256 MB through the copy-in / copy-out entry point
    all_reduce_det(big)
    small = torch.randn(4096, device="cuda")
    t_small = timed(lambda: all_reduce_det(small), args.iters, world)
    rows.append({"elements": 4096, "all_reduce_det_after_large_us": t_small * 1e3})
    if rank == 0:
        print(json.dumps(rows[-1]), flush=True)
        write_json(args.json_out, {"world": world, "results": rows})
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
