"""GPU tier, one GPU: the tensor-parallel kernels with world = 1 (local buffers)."""
import pytest
import torch

from kernel_align_b200.ops import gemm
from kernel_align_b200.parallel.tp_gemm import TPContext, all_gather_gemm, gemm_reduce_scatter

pytestmark = pytest.mark.gpu


def test_reduce_scatter_and_all_gather_world1(cuda_device):
    ctx = TPContext(device=cuda_device)
    g = torch.Generator(device=cuda_device).manual_seed(0)
    x = torch.randn(1000, 1024, device=cuda_device, generator=g).to(torch.bfloat16)
    w = (torch.randn(768, 1024, device=cuda_device, generator=g) * 0.03).to(torch.bfloat16)
    r = torch.randn(1000, 768, device=cuda_device, generator=g).to(torch.bfloat16)
    out = gemm_reduce_scatter(x, w, ctx, residual=r)
    out2 = gemm_reduce_scatter(x, w, ctx, residual=r)
    gemm.check_status(cuda_device)
    assert out.shape == (1000, 768) and torch.equal(out, out2)
    ref = (x.float() @ w.float().t()).bfloat16().float() + r.float()
    assert (out.float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item()
    # batch invariance of the sliced reduction
    part = gemm_reduce_scatter(x[100:356], w, ctx, residual=r[100:356])
    assert torch.equal(part, out[100:356])
    xa = x[:896]
    y = all_gather_gemm(xa, w, ctx)
    gemm.check_status(cuda_device)
    assert torch.equal(y, gemm.gemm_bi(xa, w))


def test_reduce_scatter_matches_cpu_rank_emulator(cuda_device):
    from kernel_align_b200.ops import cpu_ops

    ctx = TPContext(device=cuda_device)
    g = torch.Generator(device=cuda_device).manual_seed(4)
    x = torch.randn(200, 512, device=cuda_device, generator=g).to(torch.bfloat16)
    w = (torch.randn(128, 512, device=cuda_device, generator=g) * 0.05).to(torch.bfloat16)
    r = torch.randn(200, 128, device=cuda_device, generator=g).to(torch.bfloat16)
    out = gemm_reduce_scatter(x, w, ctx, residual=r)
    emu = cpu_ops.gemm_sliced_cpu(x.cpu(), w.cpu(), residual=r.cpu(), world=8)
    # same slices, same roundings, same tree; only the order inside a slice's dot product differs
    diff = (out.cpu().float() - emu).abs()
    assert diff.max().item() <= 0.02 * emu.abs().max().item()
    assert (diff > 0).float().mean().item() < 0.2
