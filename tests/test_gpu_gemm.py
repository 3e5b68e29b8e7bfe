"""GPU tier: tcgen05 GEMM in all operand layouts against fp32 PyTorch, and its invariance."""
import pytest
import torch

from kernel_align_b200.ops import gemm

pytestmark = pytest.mark.gpu


def _rand(dev, *shape, seed=0, scale=1.0):
    g = torch.Generator(device=dev).manual_seed(seed)
    return (torch.randn(*shape, device=dev, generator=g) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (300, 520, 136), (1000, 4096, 4096), (4096, 6144, 512)])
def test_gemm_nt(cuda_device, m, n, k):
    a, b = _rand(cuda_device, m, k, seed=1), _rand(cuda_device, n, k, seed=2, scale=0.05)
    c = gemm.gemm_bi(a, b)
    gemm.check_status(cuda_device)
    ref = a.float() @ b.float().t()
    assert (c.float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 1e-3
    c32 = gemm.gemm_bi(a, b, out_dtype=torch.float32)
    assert (c32 - ref).abs().max().item() <= 2e-3 * max(1.0, ref.abs().max().item())
    assert torch.equal(c, c32.to(torch.bfloat16))


@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (520, 264, 1000), (2048, 4096, 4096)])
def test_gemm_transposed_operands(cuda_device, m, n, k):
    a, b = _rand(cuda_device, m, k, seed=3), _rand(cuda_device, n, k, seed=4, scale=0.05)
    ref = gemm.gemm_bi(a, b, out_dtype=torch.float32)
    bt = b.t().contiguous()  # stored [K, N]
    at = a.t().contiguous()  # stored [K, M]
    for kw, (aa, bb) in {"nn": (a, bt), "tn": (at, bt), "tt": (at, b)}.items():
        out = gemm.gemm_bi(aa, bb, trans_a=kw[0] == "t", trans_b=(kw == "nn" or kw == "tn"), out_dtype=torch.float32)
        gemm.check_status(cuda_device)
        assert (out - ref).abs().max().item() <= 2e-3 * max(1.0, ref.abs().max().item()), kw


def test_gemm_bitwise_batch_invariant(cuda_device):
    a, b = _rand(cuda_device, 3000, 1024, seed=5), _rand(cuda_device, 2048, 1024, seed=6, scale=0.05)
    full = gemm.gemm_bi(a, b)
    assert torch.equal(full, gemm.gemm_bi(a, b))
    for lo, hi in ((0, 1), (17, 300), (2048, 3000)):
        assert torch.equal(gemm.gemm_bi(a[lo:hi], b), full[lo:hi])


def test_linear_autograd(cuda_device):
    x = _rand(cuda_device, 4, 96, 512, seed=7).requires_grad_()
    w = _rand(cuda_device, 768, 512, seed=8, scale=0.05).requires_grad_()
    y = gemm.linear(x, w)
    dy = _rand(cuda_device, 4, 96, 768, seed=9)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    (xr @ wr.t()).backward(dy.float())
    assert (x.grad.float() - xr.grad).abs().max().item() <= 0.02 * xr.grad.abs().max().item()
    assert (w.grad.float() - wr.grad).abs().max().item() <= 0.02 * wr.grad.abs().max().item()


@pytest.mark.parametrize("m", [1, 8, 16, 17, 33, 64])
@pytest.mark.parametrize("n,k", [(4096, 4096), (1000, 520), (28672, 4096), (4096, 14336)])
def test_skinny_gemm_equals_tiled_kernel_bitwise(cuda_device, m, n, k, monkeypatch):
    """The weight-streaming kernel for decode-sized batches must give the bits of the tiled
    kernel: otherwise a row's result would depend on the batch size it is computed in."""
    g = torch.Generator(device=cuda_device).manual_seed(m * 7 + n)
    a = torch.randn(80, k, device=cuda_device, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, device=cuda_device, generator=g) * 0.05).to(torch.bfloat16)
    tiled = gemm.gemm_bi(a, w)                      # 80 rows: the tiled kernel
    skinny = gemm.gemm_skinny(a[:m], w)
    gemm.check_status(cuda_device)
    assert torch.equal(skinny, tiled[:m])
    ref = a[:m].float() @ w.float().t()
    assert (skinny.float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 1e-3
    # and gemm_bi routes small batches to it
    assert torch.equal(gemm.gemm_bi(a[:m], w), tiled[:m])
    monkeypatch.setenv("KA_GEMM_SKINNY", "0")
    assert torch.equal(gemm.gemm_bi(a[:m], w), tiled[:m])
