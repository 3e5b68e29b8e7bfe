"""RMSNorm / RoPE / SwiGLU: CPU library vs PyTorch, CUDA kernels vs the CPU library."""
import pytest
import torch
import torch.nn.functional as F

from kernel_align_b200.ops.layer_ops import rmsnorm, rope_, rope_tables, swiglu


def _rms_ref(x, w, eps, res=None):
    xr = x.float() if res is None else (x.float() + res.float()).bfloat16().float()
    n = (xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + eps)).bfloat16().float()
    return (n * w.float()).bfloat16(), xr.bfloat16()


def _rope_ref(x, pos, cos, sin):
    h = x.shape[-1] // 2
    c, s = cos[pos][:, None, :], sin[pos][:, None, :]
    xf = x.float()
    return torch.cat([xf[..., :h] * c - xf[..., h:] * s, xf[..., h:] * c + xf[..., :h] * s], -1).bfloat16()


def test_cpu_layer_ops_match_pytorch():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(9, 256, generator=g).bfloat16()
    w = torch.randn(256, generator=g).bfloat16()
    r = torch.randn(9, 256, generator=g).bfloat16()
    y = rmsnorm(x, w, 1e-5)
    assert (y.float() - _rms_ref(x, w, 1e-5)[0].float()).abs().max() <= 0.04
    y2, ro = rmsnorm(x, w, 1e-5, r)
    ref, ref_ro = _rms_ref(x, w, 1e-5, r)
    assert torch.equal(ro, ref_ro) and (y2.float() - ref.float()).abs().max() <= 0.04
    assert torch.equal(rmsnorm(x[3:4], w, 1e-5), y[3:4])  # batch invariance
    q = torch.randn(11, 4, 128, generator=g).bfloat16()
    cos, sin = rope_tables(64, 128)
    pos = torch.randint(0, 64, (11,), generator=g)
    want = _rope_ref(q, pos, cos, sin)
    got = rope_(q.clone(), pos, cos, sin)
    assert (got.float() - want.float()).abs().max() <= 0.04
    gu = torch.randn(6, 512, generator=g).bfloat16()
    want = (F.silu(gu[:, :256].float()).bfloat16().float() * gu[:, 256:].float()).bfloat16()
    assert (swiglu(gu).float() - want.float()).abs().max() <= 0.04


@pytest.mark.gpu
def test_gpu_layer_ops_match_cpu_library(cuda_device):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(300, 4096, generator=g).bfloat16()
    w = (torch.randn(4096, generator=g) * 0.1 + 1).bfloat16()
    r = torch.randn(300, 4096, generator=g).bfloat16()
    y_cpu, ro_cpu = rmsnorm(x, w, 1e-5, r)
    y_gpu, ro_gpu = rmsnorm(x.to(cuda_device), w.to(cuda_device), 1e-5, r.to(cuda_device))
    assert torch.equal(ro_gpu.cpu(), ro_cpu)
    assert torch.equal(y_gpu.cpu(), y_cpu)  # same summation order, same rounding points
    y1 = rmsnorm(x.to(cuda_device), w.to(cuda_device), 1e-5)
    assert torch.equal(y1[17:18], rmsnorm(x[17:18].to(cuda_device), w.to(cuda_device), 1e-5))
    assert (y1.cpu().float() - _rms_ref(x, w, 1e-5)[0].float()).abs().max() <= 0.07

    q = torch.randn(512, 32, 128, generator=g).bfloat16()
    cos, sin = rope_tables(512, 128)
    pos = torch.arange(512)
    got = rope_(q.clone().to(cuda_device), pos.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device))
    assert torch.equal(got.cpu(), rope_(q.clone(), pos, cos, sin))
    # strided view: q part of a fused qkv projection
    qkv = torch.randn(64, 48, 128, generator=g).bfloat16().to(cuda_device)
    view = qkv[:, :32]
    want = rope_(view.clone().contiguous(), pos[:64].to(cuda_device), cos.to(cuda_device), sin.to(cuda_device))
    rope_(view, pos[:64].to(cuda_device), cos.to(cuda_device), sin.to(cuda_device))
    assert torch.equal(view, want)

    gu = torch.randn(200, 2 * 14336, generator=g).bfloat16()
    out = swiglu(gu.to(cuda_device)).cpu()
    want = (F.silu(gu[:, :14336].float()).bfloat16().float() * gu[:, 14336:].float()).bfloat16()
    assert (out.float() - want.float()).abs().max() <= 0.07
    sep = swiglu(gu[:, :14336].contiguous().to(cuda_device), gu[:, 14336:].contiguous().to(cuda_device)).cpu()
    assert torch.equal(sep, out)
