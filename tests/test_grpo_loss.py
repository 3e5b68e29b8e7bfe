"""GRPO objective: CPU library and CUDA kernels against an autograd PyTorch reference."""
import pytest
import torch

from kernel_align_b200.ops.grpo_loss import group_advantages, grpo_loss


def _ref(ln, lo, adv, mask, lr, eps, beta, reduction):
    ratio = (ln - lo).exp()
    a = adv[:, None]
    obj = torch.minimum(ratio * a, ratio.clamp(1 - eps, 1 + eps) * a)
    loss = -obj
    if beta > 0:
        d = lr - ln
        loss = loss + beta * (d.exp() - d - 1)
    m = mask.float()
    if reduction == "token_mean":
        return (loss * m).sum() / m.sum()
    per = (loss * m).sum(1) / m.sum(1).clamp(min=1)
    valid = (m.sum(1) > 0).float()
    return (per * valid).sum() / valid.sum()


def _case(dev, seed=0, g=12, l=70):
    gen = torch.Generator().manual_seed(seed)
    lo = -torch.rand(g, l, generator=gen) * 3
    ln = lo + torch.randn(g, l, generator=gen) * 0.3
    lr = lo + torch.randn(g, l, generator=gen) * 0.2
    rewards = torch.randn(g, generator=gen)
    mask = torch.rand(g, l, generator=gen) > 0.2
    mask[3] = False
    return [t.to(dev) for t in (ln, lo, lr, rewards, mask)]


def _check(dev):
    ln, lo, lr, rewards, mask = _case(dev)
    adv = group_advantages(rewards, 4)
    r = rewards.view(-1, 4)
    want = ((r - r.mean(1, keepdim=True)) / (r.std(1, keepdim=True) + 1e-4)).view(-1)
    assert (adv - want).abs().max().item() < 1e-5
    for reduction in ("token_mean", "seq_mean"):
        for beta in (0.0, 0.04):
            x = ln.clone().requires_grad_()
            loss, stats = grpo_loss(x, lo, adv, mask=mask, logp_ref=lr, eps_low=0.2, beta=beta, reduction=reduction,
                                    return_stats=True)
            (loss * 2.0).backward()
            xr = ln.clone().requires_grad_()
            ref = _ref(xr, lo, adv, mask, lr, 0.2, beta, reduction)
            (ref * 2.0).backward()
            assert abs(loss.item() - ref.item()) < 1e-5, (reduction, beta)
            assert (x.grad - xr.grad).abs().max().item() < 1e-6
            assert stats[2].item() == mask.sum().item()
            again = grpo_loss(ln, lo, adv, mask=mask, logp_ref=lr, beta=beta, reduction=reduction)
            assert again.item() == loss.item()  # bitwise repeatable


def test_grpo_loss_cpu():
    _check(torch.device("cpu"))


@pytest.mark.gpu
def test_grpo_loss_gpu(cuda_device):
    _check(cuda_device)
    # Llama-sized: G=64 sequences of 512 tokens
    gen = torch.Generator(device=cuda_device).manual_seed(1)
    lo = -torch.rand(64, 512, device=cuda_device, generator=gen)
    ln = (lo + torch.randn(64, 512, device=cuda_device, generator=gen) * 0.1).requires_grad_()
    adv = group_advantages(torch.randn(64, device=cuda_device, generator=gen), 64)
    a = grpo_loss(ln, lo, adv)
    b = grpo_loss(ln, lo, adv)
    assert a.item() == b.item()
    a.backward()
    assert torch.isfinite(ln.grad).all()
