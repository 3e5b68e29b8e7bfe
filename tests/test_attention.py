"""Attention: CPU library vs PyTorch SDPA; CUDA kernel vs fp32 SDPA and its invariance."""
import math

import pytest
import torch
import torch.nn.functional as F

from kernel_align_b200.ops.attention import attention


def _sdpa(q, k, v, causal):
    g = q.shape[2] // k.shape[2]
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    kf, vf = kf.repeat_interleave(g, 1), vf.repeat_interleave(g, 1)
    return F.scaled_dot_product_attention(qf, kf, vf, is_causal=causal).permute(0, 2, 1, 3)


def test_cpu_attention_matches_sdpa():
    g = torch.Generator().manual_seed(0)
    q = torch.randn(2, 37, 4, 16, generator=g)
    k = torch.randn(2, 37, 2, 16, generator=g)
    v = torch.randn(2, 37, 2, 16, generator=g)
    for causal in (True, False):
        out, lse = attention(q, k, v, causal=causal, return_lse=True)
        assert (out - _sdpa(q, k, v, causal)).abs().max().item() < 1e-5
        assert lse.shape == (2, 4, 37)
    assert torch.equal(attention(q[1:2], k[1:2], v[1:2]), attention(q, k, v)[1:2])


@pytest.mark.gpu
@pytest.mark.parametrize("b,l,hq,hkv,causal", [(2, 128, 4, 2, True), (3, 512, 8, 2, True), (2, 300, 4, 4, True),
                                                (2, 384, 4, 1, False), (1, 1024, 32, 8, True)])
def test_gpu_attention_matches_fp32_sdpa(cuda_device, b, l, hq, hkv, causal):
    from kernel_align_b200.ops.gemm import check_status

    g = torch.Generator(device=cuda_device).manual_seed(1)
    q = torch.randn(b, l, hq, 128, device=cuda_device, generator=g).to(torch.bfloat16)
    k = torch.randn(b, l, hkv, 128, device=cuda_device, generator=g).to(torch.bfloat16)
    v = torch.randn(b, l, hkv, 128, device=cuda_device, generator=g).to(torch.bfloat16)
    out, lse = attention(q, k, v, causal=causal, return_lse=True)
    check_status(cuda_device)
    ref = _sdpa(q, k, v, causal)
    assert (out.float() - ref).abs().max().item() < 0.03
    g_ = hq // hkv
    s = torch.einsum("blhd,bmhd->bhlm", q.float(), k.float().repeat_interleave(g_, 2)) / math.sqrt(128)
    if causal:
        s = s.masked_fill(torch.ones(l, l, device=cuda_device, dtype=torch.bool).triu(1), float("-inf"))
    assert (lse - torch.logsumexp(s, -1)).abs().max().item() < 2e-3


@pytest.mark.gpu
def test_gpu_attention_invariance_and_fused_qkv_views(cuda_device):
    g = torch.Generator(device=cuda_device).manual_seed(2)
    b, l, hq, hkv = 4, 512, 8, 2
    qkv = torch.randn(b, l, (hq + 2 * hkv) * 128, device=cuda_device, generator=g).to(torch.bfloat16)
    q = qkv[..., : hq * 128].view(b, l, hq, 128)
    k = qkv[..., hq * 128: (hq + hkv) * 128].view(b, l, hkv, 128)
    v = qkv[..., (hq + hkv) * 128:].view(b, l, hkv, 128)
    full = attention(q, k, v)
    assert torch.equal(full, attention(q, k, v))
    assert torch.equal(full, attention(q.contiguous(), k.contiguous(), v.contiguous()))
    assert torch.equal(attention(q[2:3], k[2:3], v[2:3]), full[2:3])          # batch 1 vs 4
    assert torch.equal(attention(q[:, :, 4:], k[:, :, 1:], v[:, :, 1:]), full[:, :, 4:])  # head shard (TP)


@pytest.mark.gpu
@pytest.mark.parametrize("b,l,hq,hkv,causal", [(2, 128, 4, 2, True), (2, 512, 8, 2, True), (1, 300, 4, 4, True),
                                                (2, 256, 4, 1, False)])
def test_gpu_attention_backward_matches_autograd(cuda_device, b, l, hq, hkv, causal):
    from kernel_align_b200.ops.attention import attention_fn
    from kernel_align_b200.ops.gemm import check_status

    g = torch.Generator(device=cuda_device).manual_seed(5)
    q = torch.randn(b, l, hq, 128, device=cuda_device, generator=g).to(torch.bfloat16)
    k = torch.randn(b, l, hkv, 128, device=cuda_device, generator=g).to(torch.bfloat16)
    v = torch.randn(b, l, hkv, 128, device=cuda_device, generator=g).to(torch.bfloat16)
    d_o = torch.randn(b, l, hq, 128, device=cuda_device, generator=g).to(torch.bfloat16)
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    attention_fn(qg, kg, vg, causal=causal).backward(d_o)
    check_status(cuda_device)
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    _sdpa(qr, kr, vr, causal).backward(d_o.float())
    for got, ref, name in ((qg.grad, qr.grad, "dq"), (kg.grad, kr.grad, "dk"), (vg.grad, vr.grad, "dv")):
        err = (got.float() - ref).abs().max().item()
        assert err <= 0.03 * ref.abs().max().item() + 1e-3, (name, err, ref.abs().max().item())
    # deterministic and batch invariant
    q2, k2, v2 = (t.clone().requires_grad_() for t in (q, k, v))
    attention_fn(q2, k2, v2, causal=causal).backward(d_o)
    assert torch.equal(q2.grad, qg.grad) and torch.equal(k2.grad, kg.grad) and torch.equal(v2.grad, vg.grad)
    q3, k3, v3 = (t[1:2].clone().requires_grad_() for t in (q, k, v)) if b > 1 else (None, None, None)
    if b > 1:
        attention_fn(q3, k3, v3, causal=causal).backward(d_o[1:2])
        assert torch.equal(q3.grad, qg.grad[1:2]) and torch.equal(k3.grad, kg.grad[1:2])
