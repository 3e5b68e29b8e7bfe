#!/usr/bin/env python
"""Tensor-parallel Llama-3-8B decoder layer: device time per forward (and forward+backward)
versus a plain PyTorch + NCCL implementation of the same layer (cuBLAS, SDPA, all-gather /
reduce-scatter as separate collectives).

    python benchmarks/bench_tp_layer.py --batch 8                         # TP = 1
    torchrun --nproc-per-node 8 benchmarks/bench_tp_layer.py --batch 64   # TP = 8

Time is the max over ranks of CUDA-event timings (warmed, median of 10).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist
import torch.nn.functional as F

from _common import ROOT, write_json
from kernel_align_b200.models.llama import DecoderLayer, LlamaConfig
from kernel_align_b200.ops.layer_ops import rope_tables
from kernel_align_b200.parallel.tp_gemm import TPContext, rows_per_rank


def timed(fn, world, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ts.append(t.item())
    return statistics.median(ts)


def torch_layer(layer, tp, world):
    """The same layer with library kernels: cuBLAS GEMMs, SDPA, NCCL all-gather / reduce-scatter."""
    cfg = layer.cfg
    hd, hq, hkv = cfg.head_dim, layer.hq, layer.hkv

    def rms(v, w):
        return F.rms_norm(v, (v.shape[-1],), w, cfg.rms_eps)

    # differentiable collectives: the adjoint of an all-gather is a reduce-scatter and vice versa
    class _Gather(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x):
            out = torch.empty(world * x.shape[0], x.shape[1], dtype=x.dtype, device=x.device)
            dist.all_gather_into_tensor(out, x.contiguous())
            return out

        @staticmethod
        def backward(ctx, g):
            out = torch.empty(g.shape[0] // world, g.shape[1], dtype=g.dtype, device=g.device)
            dist.reduce_scatter_tensor(out, g.contiguous())
            return out

    class _ScatterSum(torch.autograd.Function):
        @staticmethod
        def forward(ctx, y):
            out = torch.empty(y.shape[0] // world, y.shape[1], dtype=y.dtype, device=y.device)
            dist.reduce_scatter_tensor(out, y.contiguous())
            return out

        @staticmethod
        def backward(ctx, g):
            out = torch.empty(world * g.shape[0], g.shape[1], dtype=g.dtype, device=g.device)
            dist.all_gather_into_tensor(out, g.contiguous())
            return out

    def gather(x):
        return x if world == 1 else _Gather.apply(x)

    def scatter_sum(y):
        return y if world == 1 else _ScatterSum.apply(y)

    def fwd(x_local, batch, seq_len, cos, sin):
        tokens = batch * seq_len
        h = gather(rms(x_local, layer.norm1))
        qkv = h @ layer.wqkv.t()
        q = qkv[:tokens, : hq * hd].view(batch, seq_len, hq, hd)
        k = qkv[:tokens, hq * hd:(hq + hkv) * hd].view(batch, seq_len, hkv, hd)
        v = qkv[:tokens, (hq + hkv) * hd:].view(batch, seq_len, hkv, hd)

        def rope(t):
            half = hd // 2
            c, s = cos[:seq_len, None, :].to(t.dtype), sin[:seq_len, None, :].to(t.dtype)
            return torch.cat([t[..., :half] * c - t[..., half:] * s, t[..., half:] * c + t[..., :half] * s], -1)

        q, k = rope(q), rope(k)
        a = F.scaled_dot_product_attention(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3),
                                           is_causal=True, enable_gqa=True)
        a = a.permute(0, 2, 1, 3).reshape(tokens, hq * hd)
        x_local = x_local + scatter_sum(a @ layer.wo.t())
        h = gather(rms(x_local, layer.norm2))
        gu = h @ layer.wgu.t()
        f = F.silu(gu[:, : gu.shape[1] // 2]) * gu[:, gu.shape[1] // 2:]
        return x_local + scatter_sum(f @ layer.wdown.t())

    return fwd


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--backward", action="store_true")
    ap.add_argument("--json-out", default=None)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank = dist.get_rank() if world > 1 else 0
    tp = TPContext()
    cfg = LlamaConfig.llama3_8b()
    layer = DecoderLayer(cfg, tp, seed=1, device=tp.device)
    cos, sin = rope_tables(cfg.max_pos, cfg.head_dim, cfg.rope_theta, device=tp.device)
    tokens = args.batch * args.seq_len
    rpr = rows_per_rank(tokens, world)
    x = torch.randn(rpr, cfg.hidden, device=tp.device).to(torch.bfloat16)
    pos = torch.arange(args.seq_len, device=tp.device).repeat(args.batch)
    ref = torch_layer(layer, tp, world)

    def ours():
        with torch.no_grad():
            return layer(x, args.batch, args.seq_len, pos, cos, sin)

    def theirs():
        with torch.no_grad():
            return ref(x, args.batch, args.seq_len, cos, sin)

    res = {"world": world, "batch": args.batch, "seq_len": args.seq_len, "tokens": tokens,
           "ours_fwd_ms": timed(ours, world), "torch_nccl_fwd_ms": timed(theirs, world)}
    if args.backward:
        xg = x.clone().requires_grad_()
        dy = torch.randn_like(x)

        def ours_fb():
            layer.zero_grad(set_to_none=True)
            layer(xg, args.batch, args.seq_len, pos, cos, sin).backward(dy)

        def theirs_fb():
            layer.zero_grad(set_to_none=True)
            ref(xg, args.batch, args.seq_len, cos, sin).backward(dy)

        res["ours_fwd_bwd_ms"] = timed(ours_fb, world, iters=5)
        res["torch_nccl_fwd_bwd_ms"] = timed(theirs_fb, world, iters=5)
    flops = 2.0 * tokens * cfg.hidden * ((cfg.n_heads + 2 * cfg.n_kv_heads) * cfg.head_dim + cfg.n_heads * cfg.head_dim
                                        + 3 * cfg.ffn) + 4.0 * args.batch * cfg.n_heads * args.seq_len ** 2 * cfg.head_dim / 2
    res["fwd_tflops_per_gpu"] = flops / world / res["ours_fwd_ms"] / 1e9
    if rank == 0:
        print(json.dumps(res))
        write_json(args.json_out, res)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
