#!/usr/bin/env python
"""Small, self-terminating workloads for profiler captures: one operator, a few launches.

    python benchmarks/profile_case.py --op fused_logp --rows 4736
    ncu --set full --clock-control none -k regex:fused_lmhead -s 2 -c 1 -o out \
        python benchmarks/profile_case.py --op fused_logp --rows 4736

Inputs are larger than the 126 MB L2 where the operator streams memory, but stay within a
few GB so that a multi-pass capture ends within a minute.
"""
from __future__ import annotations

import argparse

import torch

from _common import ROOT  # noqa: F401  (puts the repository root on sys.path)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True,
                    choices=["fused_logp", "logits_logp", "sampling", "rmsnorm", "swiglu", "gemm", "attention", "attention_bwd",
                             "grpo_loss", "rope", "adamw", "decode_attention", "gemm_skinny", "rmsnorm_bwd", "logp_bwd",
                             "decode_qkv", "sampling_top_p"])
    ap.add_argument("--rows", type=int, default=4736)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--launches", type=int, default=3)
    args = ap.parse_args()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    if args.op == "fused_logp":
        from kernel_align_b200.ops.fused_logp import lmhead_logp

        h = torch.randn(args.rows, args.hidden, device=dev, generator=g).to(torch.bfloat16)
        w = torch.empty(args.vocab, args.hidden, device=dev, dtype=torch.bfloat16)
        for i in range(0, args.vocab, 16384):
            n = min(16384, args.vocab - i)
            w[i:i + n] = (torch.randn(n, args.hidden, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        ids = torch.randint(0, args.vocab, (args.rows,), device=dev, generator=g)
        fn = lambda: lmhead_logp(h, w, ids)  # noqa: E731
    elif args.op == "logits_logp":
        from kernel_align_b200.ops.logits_logp import logits_logp

        x = (torch.randn(args.rows, args.vocab, device=dev, generator=g) * 2).to(torch.bfloat16)
        ids = torch.randint(0, args.vocab, (args.rows,), device=dev, generator=g)
        fn = lambda: logits_logp(x, ids)  # noqa: E731
    elif args.op == "sampling":
        from kernel_align_b200.ops.sampling import sample

        x = (torch.randn(args.rows, args.vocab, device=dev, generator=g) * 2).to(torch.bfloat16)
        fn = lambda: sample(x, top_k=50, top_p=0.9, temperature=0.7, seed=1, step=0)  # noqa: E731
    elif args.op == "sampling_top_p":       # no top-k: sample_general_kernel
        from kernel_align_b200.ops.sampling import sample

        x = (torch.randn(args.rows, args.vocab, device=dev, generator=g) * 2).to(torch.bfloat16)
        fn = lambda: sample(x, top_k=None, top_p=0.9, temperature=0.7, seed=1, step=0)  # noqa: E731
    elif args.op == "rmsnorm":
        from kernel_align_b200.ops.layer_ops import rmsnorm

        x = torch.randn(args.rows, args.hidden, device=dev, generator=g).to(torch.bfloat16)
        w = torch.ones(args.hidden, device=dev, dtype=torch.bfloat16)
        fn = lambda: rmsnorm(x, w, 1e-5, x)  # noqa: E731
    elif args.op == "swiglu":
        from kernel_align_b200.ops.layer_ops import swiglu

        x = torch.randn(args.rows, 2 * 14336, device=dev, generator=g).to(torch.bfloat16)
        fn = lambda: swiglu(x)  # noqa: E731
    elif args.op == "attention":
        from kernel_align_b200.ops.attention import attention

        b_, l = 4, args.rows if args.rows <= 8192 else 4096
        q = torch.randn(b_, l, 32, 128, device=dev, generator=g).to(torch.bfloat16)
        k = torch.randn(b_, l, 8, 128, device=dev, generator=g).to(torch.bfloat16)
        v = torch.randn(b_, l, 8, 128, device=dev, generator=g).to(torch.bfloat16)
        fn = lambda: attention(q, k, v)  # noqa: E731
    elif args.op == "attention_bwd":
        from kernel_align_b200.ops.attention import attention, attention_backward

        b_, l = 2, args.rows if args.rows <= 8192 else 4096
        q = torch.randn(b_, l, 32, 128, device=dev, generator=g).to(torch.bfloat16)
        k = torch.randn(b_, l, 8, 128, device=dev, generator=g).to(torch.bfloat16)
        v = torch.randn(b_, l, 8, 128, device=dev, generator=g).to(torch.bfloat16)
        o, lse = attention(q, k, v, return_lse=True)
        d_o = torch.randn_like(o)
        fn = lambda: attention_backward(q, k, v, o, d_o, lse, causal=True)  # noqa: E731
    elif args.op == "gemm":
        from kernel_align_b200.ops.gemm import gemm_bi

        a = torch.randn(8192, args.hidden, device=dev, generator=g).to(torch.bfloat16)
        b = (torch.randn(28672, args.hidden, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        fn = lambda: gemm_bi(a, b)  # noqa: E731
    elif args.op == "grpo_loss":
        from kernel_align_b200.ops.grpo_loss import grpo_loss

        groups, seq = max(256, args.rows // 512 * 4), 512      # [G, L] log-probs; bytes are tiny, the launch is the cost
        new = (torch.randn(groups, seq, device=dev, generator=g) * 0.1 - 2).requires_grad_()
        old = torch.randn(groups, seq, device=dev, generator=g) * 0.1 - 2
        adv = torch.randn(groups, device=dev, generator=g)

        def fn():
            new.grad = None
            loss = grpo_loss(new, old, adv)
            loss.backward()
            return loss
    elif args.op == "rope":
        from kernel_align_b200.ops.layer_ops import rope_, rope_tables

        rows = max(args.rows, 32768)
        x = torch.randn(rows, 32, 128, device=dev, generator=g).to(torch.bfloat16)     # 268 MB at 32768 rows
        pos = torch.arange(512, device=dev).repeat(rows // 512 + 1)[:rows]
        cos, sin = rope_tables(512, 128, 500000.0, device=dev)
        fn = lambda: rope_(x, pos, cos, sin)  # noqa: E731
    elif args.op == "adamw":
        from kernel_align_b200.ops.decode import FusedAdamW

        n = 1 << 27                                                                     # 2.7 GB of state and gradients
        w = torch.nn.Parameter((torch.randn(n, device=dev, generator=g) * 0.02).to(torch.bfloat16))
        w.grad = torch.randn(n, device=dev, generator=g).to(torch.bfloat16)
        opt = FusedAdamW([w], lr=1e-5)

        def fn():
            opt.step()
            return w
    elif args.op == "decode_attention":
        from kernel_align_b200.ops.decode import attention_decode

        b_, ctx = 256, 1024                                                             # 1.07 GB of K and V
        q = torch.randn(b_, 32, 128, device=dev, generator=g).to(torch.bfloat16)
        ck = torch.randn(b_, ctx, 8, 128, device=dev, generator=g).to(torch.bfloat16)
        cv = torch.randn(b_, ctx, 8, 128, device=dev, generator=g).to(torch.bfloat16)
        lens = torch.full((b_,), ctx, dtype=torch.int32, device=dev)
        fn = lambda: attention_decode(q, ck, cv, lens)  # noqa: E731
    elif args.op == "decode_qkv":
        from kernel_align_b200.ops.decode import decode_qkv_rope_cache
        from kernel_align_b200.ops.layer_ops import rope_tables

        b_, t = 64, 512
        qkv = torch.randn(b_, 48 * 128, device=dev, generator=g).to(torch.bfloat16)
        pos = torch.full((b_,), 100, device=dev)
        slot = torch.tensor([100], device=dev)
        cos, sin = rope_tables(t, 128, 500000.0, device=dev)
        ck = torch.zeros(b_, t, 8, 128, device=dev, dtype=torch.bfloat16)
        cv = torch.zeros_like(ck)
        fn = lambda: decode_qkv_rope_cache(qkv, pos, slot, cos, sin, ck, cv, 32, 8)  # noqa: E731
    elif args.op == "gemm_skinny":
        from kernel_align_b200.ops.gemm import gemm_bi

        a = torch.randn(8, args.hidden, device=dev, generator=g).to(torch.bfloat16)
        b = (torch.randn(28672, args.hidden, device=dev, generator=g) * 0.02).to(torch.bfloat16)   # 235 MB of weights
        fn = lambda: gemm_bi(a, b)  # noqa: E731
    elif args.op == "rmsnorm_bwd":
        from kernel_align_b200.ops.layer_ops import rmsnorm_fn

        rows = max(args.rows, 32768)
        x = torch.randn(rows, args.hidden, device=dev, generator=g).to(torch.bfloat16).requires_grad_()
        w = torch.ones(args.hidden, device=dev, dtype=torch.bfloat16).requires_grad_()
        dy = torch.randn(rows, args.hidden, device=dev, generator=g).to(torch.bfloat16)

        def fn():
            x.grad = None
            w.grad = None
            rmsnorm_fn(x, w, 1e-5).backward(dy)
            return x.grad
    elif args.op == "logp_bwd":
        from kernel_align_b200.ops.fused_logp import lmhead_logp

        rows = min(args.rows, 4096)
        h = torch.randn(rows, args.hidden, device=dev, generator=g).to(torch.bfloat16).requires_grad_()
        w = torch.nn.Parameter((torch.randn(args.vocab, args.hidden, device=dev, generator=g) * 0.02).to(torch.bfloat16))
        ids = torch.randint(0, args.vocab, (rows,), device=dev, generator=g)

        def fn():
            h.grad = None
            w.grad = None
            lmhead_logp(h, w, ids).sum().backward()
            return h.grad
    else:
        raise SystemExit(f"--op {args.op}: no profile case defined yet")
    for _ in range(args.launches):
        out = fn()
    torch.cuda.synchronize()
    print("done", tuple(out.shape) if hasattr(out, "shape") else "")


if __name__ == "__main__":
    main()
