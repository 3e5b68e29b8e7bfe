#!/usr/bin/env python
"""Per-operator device timings on one GPU, each against the library baseline and its roofline.

Rooflines use the measured peaks of this pod when MEASURED_PEAKS.json is present
(copy bandwidth and cuBLAS bf16 throughput), else the fallback figures 6.65 TB/s / 1.59 PFLOP/s.
CUDA events, >= 3 warm-ups, median of 10, L2 flushed between iterations for the memory-bound ops.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.nn.functional as F
from tabulate import tabulate

from _common import ROOT, time_cuda, write_json
from kernel_align_b200.ops import gemm
from kernel_align_b200.ops.attention import attention
from kernel_align_b200.ops.layer_ops import rmsnorm, swiglu
from kernel_align_b200.ops.logits_logp import logits_logp
from kernel_align_b200.ops.sampling import sample


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p["hbm_gbs"], p["bf16_tflops"], p.get("bf16_tflops_sustained", p["bf16_tflops"]), "of measured"
    return 6650.0, 1590.0, 1400.0, "of fallback"


def small_op_cases(dev, g, rows=32768, hidden=4096, groups=256, seq=512, batch=64, ctx=512, params=1 << 28):
    """The operators that are not GEMM-shaped and have no row of their own above: RoPE, the GRPO
    loss (forward + backward), decode attention, the fused AdamW step and the fused log-prob
    backward. Returns ``[(name, fn, baseline_fn or None, bytes moved)]``; sizes are arguments
    so that a CPU run can exercise the same calls on small shapes."""
    from kernel_align_b200.ops.decode import FusedAdamW, attention_decode
    from kernel_align_b200.ops.fused_logp import lmhead_logp
    from kernel_align_b200.ops.grpo_loss import grpo_loss
    from kernel_align_b200.ops.layer_ops import rope_, rope_tables

    cases = []
    heads = max(1, hidden // 128)
    q = torch.randn(rows, heads, 128, device=dev, generator=g).to(torch.bfloat16)
    pos = torch.arange(seq, device=dev).repeat(rows // seq + 1)[:rows]
    cos, sin = rope_tables(max(seq, 8), 128, 500000.0, device=dev)
    cases.append((f"rope {rows}x{heads}x128", lambda: rope_(q, pos, cos, sin), None, q.numel() * 2 * 2))

    new = (torch.randn(groups, seq, device=dev, generator=g) * 0.1 - 2).requires_grad_()
    old = torch.randn(groups, seq, device=dev, generator=g) * 0.1 - 2
    adv = torch.randn(groups, device=dev, generator=g)

    def loss_fb():
        new.grad = None
        grpo_loss(new, old, adv).backward()

    def loss_torch():
        n = new.detach().requires_grad_()
        r = torch.exp(n - old)
        a = adv[:, None]
        (-torch.minimum(r * a, r.clamp(0.8, 1.2) * a).mean()).backward()

    cases.append((f"grpo_loss fwd+bwd {groups}x{seq}", loss_fb, loss_torch, groups * seq * 4 * 4))

    hq, hkv = heads, max(1, heads // 4)
    qd = torch.randn(batch, hq, 128, device=dev, generator=g).to(torch.bfloat16)
    ck = torch.randn(batch, ctx, hkv, 128, device=dev, generator=g).to(torch.bfloat16)
    cv = torch.randn(batch, ctx, hkv, 128, device=dev, generator=g).to(torch.bfloat16)
    lens = torch.full((batch,), ctx, dtype=torch.int32, device=dev)
    cases.append((f"decode attention B={batch} ctx={ctx}", lambda: attention_decode(qd, ck, cv, lens), None,
                  (ck.numel() + cv.numel()) * 2))

    w = torch.nn.Parameter((torch.randn(params, device=dev, generator=g) * 0.02).to(torch.bfloat16))
    w.grad = torch.randn(params, device=dev, generator=g).to(torch.bfloat16)
    opt = FusedAdamW([w], lr=1e-5)
    cases.append((f"fused AdamW {params} params", opt.step, None, params * (2 + 2 + 12 + 12 + 2)))

    from kernel_align_b200.ops.layer_ops import rmsnorm_fn

    xn = torch.randn(rows, hidden, device=dev, generator=g).to(torch.bfloat16).requires_grad_()
    wn = torch.ones(hidden, device=dev, dtype=torch.bfloat16).requires_grad_()
    dyn = torch.randn(rows, hidden, device=dev, generator=g).to(torch.bfloat16)
    yn = rmsnorm_fn(xn, wn, 1e-5)

    def norm_bwd():
        xn.grad = None
        wn.grad = None
        yn.backward(dyn, retain_graph=True)

    xr = xn.detach().float().requires_grad_()
    wr = wn.detach().float().requires_grad_()
    yr = F.rms_norm(xr, (hidden,), wr, 1e-5)

    def norm_bwd_torch():
        xr.grad = None
        wr.grad = None
        yr.backward(dyn.float(), retain_graph=True)

    cases.append((f"rmsnorm backward {rows}x{hidden}", norm_bwd, norm_bwd_torch, rows * hidden * 2 * 3))

    vocab = 128256 if rows >= 4096 else 512
    m = min(rows, 8192)
    hs = torch.randn(m, hidden, device=dev, generator=g).to(torch.bfloat16).requires_grad_()
    wl = torch.nn.Parameter((torch.randn(vocab, hidden, device=dev, generator=g) * 0.02).to(torch.bfloat16))
    ids = torch.randint(0, vocab, (m,), device=dev, generator=g)

    def logp_fb():
        hs.grad = None
        wl.grad = None
        lmhead_logp(hs, wl, ids).sum().backward()

    cases.append((f"fused log-prob fwd+bwd {m}x{vocab}x{hidden}", logp_fb, None, 0))
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json-out", default=None)
    ap.add_argument("--reference-sampler", action="store_true",
                    help="also time the reference's SamplerBackend.sample from baseline/_ref (FlashInfer JIT)")
    args = ap.parse_args()
    dev = torch.device("cuda")
    hbm, tf_burst, tf_sus, tag = peaks()
    g = torch.Generator(device=dev).manual_seed(0)
    rows, out = [], []

    def rec(name, ms, base_ms, frac, note):
        rows.append([name, f"{ms * 1e3:.1f} us", f"{base_ms * 1e3:.1f} us" if base_ms else "-",
                     f"{base_ms / ms:.2f}x" if base_ms else "-", f"{frac:.2f} {tag}", note])
        out.append({"op": name, "ms": ms, "baseline_ms": base_ms, "roofline_fraction": frac, "note": note})

    # GEMM, Llama-3-8B layer shapes at 8192 tokens
    for name, (m, n, k) in {"gemm qkv 8192x6144x4096": (8192, 6144, 4096), "gemm gate_up 8192x28672x4096": (8192, 28672, 4096),
                            "gemm down 8192x4096x14336": (8192, 4096, 14336), "gemm 8192^3": (8192, 8192, 8192)}.items():
        a = torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16)
        b = (torch.randn(n, k, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        t = time_cuda(lambda: gemm.gemm_bi(a, b), flush_l2=False)
        tb = time_cuda(lambda: a @ b.t(), flush_l2=False)
        tfl = 2.0 * m * n * k / t / 1e9
        rec(name, t, tb, tfl / tf_burst, f"{tfl:.0f} TFLOP/s vs cuBLAS {2.0 * m * n * k / tb / 1e9:.0f}")
        del a, b
    # decode-sized GEMMs (8 rows): the weight-streaming kernel against cuBLAS, in bytes of weights per second
    from _common import time_cuda_graph
    for name, (n, k) in {"gemm decode wqkv 8x6144x4096": (6144, 4096), "gemm decode gate_up 8x28672x4096": (28672, 4096),
                         "gemm decode lm_head 8x128256x4096": (128256, 4096)}.items():
        a = torch.randn(8, k, device=dev, generator=g).to(torch.bfloat16)
        b = (torch.randn(n, k, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        t = time_cuda_graph(lambda: gemm.gemm_bi(a, b))
        tb = time_cuda_graph(lambda: a @ b.t())
        by = n * k * 2
        rec(name, t, tb, by / t / 1e6 / hbm, f"{by / t / 1e6:.0f} GB/s of weights vs cuBLAS {by / tb / 1e6:.0f}")
        del a, b
    # attention, B=16 L=512 and B=4 L=4096, 32q/8kv heads
    for b_, l in ((16, 512), (4, 4096)):
        q = torch.randn(b_, l, 32, 128, device=dev, generator=g).to(torch.bfloat16)
        k = torch.randn(b_, l, 8, 128, device=dev, generator=g).to(torch.bfloat16)
        v = torch.randn(b_, l, 8, 128, device=dev, generator=g).to(torch.bfloat16)
        t = time_cuda(lambda: attention(q, k, v), flush_l2=False)
        qs, ks, vs = (x.permute(0, 2, 1, 3) for x in (q, k, v))
        tb = time_cuda(lambda: F.scaled_dot_product_attention(qs, ks, vs, is_causal=True, enable_gqa=True), flush_l2=False)
        flops = 4.0 * b_ * 32 * l * l * 128 / 2
        rec(f"attention fwd B={b_} L={l}", t, tb, flops / t / 1e9 / tf_burst,
            f"{flops / t / 1e9:.0f} TFLOP/s (causal) vs torch SDPA {flops / tb / 1e9:.0f}")
        # backward: time (delta + dQ + dK/dV) alone against SDPA's backward alone
        from kernel_align_b200.ops.attention import attention_backward
        o, lse = attention(q, k, v, return_lse=True)
        d_o = torch.randn_like(o)
        t = time_cuda(lambda: attention_backward(q, k, v, o, d_o, lse, causal=True), flush_l2=False)
        qr, kr, vr = (x.detach().requires_grad_() for x in (qs, ks, vs))
        with torch.nn.attention.sdpa_kernel(torch.nn.attention.SDPBackend.FLASH_ATTENTION):
            orr = F.scaled_dot_product_attention(qr, kr, vr, is_causal=True, enable_gqa=True)
        dor = d_o.permute(0, 2, 1, 3)
        tb = time_cuda(lambda: torch.autograd.grad(orr, (qr, kr, vr), dor, retain_graph=True), flush_l2=False)
        bfl = 2.5 * flops
        rec(f"attention bwd B={b_} L={l}", t, tb, bfl / t / 1e9 / tf_burst,
            f"{bfl / t / 1e9:.0f} TFLOP/s (causal, 5 GEMMs) vs torch SDPA backward {bfl / tb / 1e9:.0f}")
        del o, lse, d_o, orr, qr, kr, vr
    # memory-bound ops
    x = torch.randn(32768, 4096, device=dev, generator=g).to(torch.bfloat16)
    w = torch.ones(4096, device=dev, dtype=torch.bfloat16)
    t = time_cuda(lambda: rmsnorm(x, w, 1e-5, x))
    tb = time_cuda(lambda: F.rms_norm((x + x).float(), (4096,), w.float(), 1e-5).to(torch.bfloat16))
    by = x.numel() * 2 * 4
    rec("rmsnorm+residual 32768x4096", t, tb, by / t / 1e6 / hbm, f"{by / t / 1e6:.0f} GB/s")
    gu = torch.randn(8192, 2 * 14336, device=dev, generator=g).to(torch.bfloat16)
    t = time_cuda(lambda: swiglu(gu))
    tb = time_cuda(lambda: F.silu(gu[:, :14336]) * gu[:, 14336:])
    by = gu.numel() * 2 * 1.5
    rec("swiglu 8192x14336", t, tb, by / t / 1e6 / hbm, f"{by / t / 1e6:.0f} GB/s")
    del x, gu
    lg = (torch.randn(16384, 128256, device=dev, generator=g) * 2).to(torch.bfloat16)
    ids = torch.randint(0, 128256, (16384,), device=dev, generator=g)
    t = time_cuda(lambda: logits_logp(lg, ids), iters=5)
    tb = time_cuda(lambda: torch.log_softmax(lg, -1).gather(-1, ids[:, None]), iters=5)
    by = lg.numel() * 2
    rec("logits_logp 16384x128256", t, tb, by / t / 1e6 / hbm, f"{by / t / 1e6:.0f} GB/s")
    del lg
    for gsz in (64, 256):
        lgs = (torch.randn(gsz, 128256, device=dev, generator=g) * 2).to(torch.bfloat16)
        t = time_cuda(lambda: sample(lgs, top_k=50, top_p=0.9, temperature=0.7, seed=1, step=0))
        tb = None
        if args.reference_sampler:
            import sys
            sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
            try:
                from rl_engine.kernels.sampling import SamplerBackend as RefSampler
                ref = RefSampler()
                tb = time_cuda(lambda: ref.sample(lgs, top_k=50, top_p=0.9, temperature=0.7), warmup=5)
            except Exception as e:  # noqa: BLE001
                print("reference sampler unavailable:", type(e).__name__, str(e)[:200])
        by = lgs.numel() * 2
        rec(f"sampling G={gsz} V=128256 k=50 p=0.9", t, tb, by / t / 1e6 / hbm, f"{by / t / 1e6:.0f} GB/s of logits")
        # no top-k (threshold search in a per-key count histogram for bf16 rows)
        t = time_cuda(lambda: sample(lgs, top_k=None, top_p=0.9, temperature=0.7, seed=1, step=0))
        tb = None
        if args.reference_sampler:
            try:
                tb = time_cuda(lambda: ref.sample(lgs, top_k=None, top_p=0.9, temperature=0.7), warmup=5)
            except Exception as e:  # noqa: BLE001
                print("reference sampler unavailable:", type(e).__name__, str(e)[:200])
        rec(f"sampling G={gsz} V=128256 p=0.9 only", t, tb, by / t / 1e6 / hbm, f"{by / t / 1e6:.0f} GB/s of logits")
    for name, fn, base, nbytes in small_op_cases(dev, g):
        t = time_cuda(fn, iters=5)
        tb = time_cuda(base, iters=5) if base is not None else None
        if nbytes:
            rec(name, t, tb, nbytes / t / 1e6 / hbm, f"{nbytes / t / 1e6:.0f} GB/s")
        else:
            m_, v_, k_ = 8192, 128256, 4096
            tfl = 6.0 * m_ * v_ * k_ / t / 1e9 + 2.0 * m_ * v_ * k_ / t / 1e9     # forward, recompute, dH, dW
            rec(name, t, tb, tfl / tf_burst, f"{tfl:.0f} TFLOP/s (4 GEMM-sized passes)")
    print(tabulate(rows, headers=["op", "ours", "baseline", "speedup", "roofline", "note"], tablefmt="github"))
    write_json(args.json_out, {"device": torch.cuda.get_device_name(), "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf_burst,
                                                                                 "bf16_tflops_sustained": tf_sus}, "results": out})


if __name__ == "__main__":
    main()
