"""GPU tier: decoder layer and model on one GPU (TP = 1): against a plain PyTorch fp32
implementation, batch invariance, and gradients through every native operator."""
import math

import pytest
import torch
import torch.nn.functional as F

from kernel_align_b200.models.llama import DecoderLayer, LlamaConfig, LlamaModel
from kernel_align_b200.ops import gemm
from kernel_align_b200.ops.layer_ops import rope_tables
from kernel_align_b200.parallel.tp_gemm import TPContext

pytestmark = pytest.mark.gpu


def _ref_layer(layer, x, batch, seq_len, cos, sin):
    cfg = layer.cfg
    hd, hq, hkv = cfg.head_dim, layer.hq, layer.hkv
    xf = x.float()

    def rms(v, w):
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)) * w.float()

    def rope(t, pos):
        h = hd // 2
        c, s = cos[pos][:, None, :], sin[pos][:, None, :]
        return torch.cat([t[..., :h] * c - t[..., h:] * s, t[..., h:] * c + t[..., :h] * s], -1)

    pos = torch.arange(seq_len, device=x.device).repeat(batch)
    h = rms(xf, layer.norm1)
    qkv = h @ layer.wqkv.float().t()
    q = rope(qkv[:, : hq * hd].view(-1, hq, hd), pos).view(batch, seq_len, hq, hd)
    k = rope(qkv[:, hq * hd:(hq + hkv) * hd].view(-1, hkv, hd), pos).view(batch, seq_len, hkv, hd)
    v = qkv[:, (hq + hkv) * hd:].view(batch, seq_len, hkv, hd)
    g = hq // hkv
    a = F.scaled_dot_product_attention(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3).repeat_interleave(g, 1),
                                       v.permute(0, 2, 1, 3).repeat_interleave(g, 1), is_causal=True)
    a = a.permute(0, 2, 1, 3).reshape(-1, hq * hd)
    xf = xf + a @ layer.wo.float().t()
    h = rms(xf, layer.norm2)
    gu = h @ layer.wgu.float().t()
    f = F.silu(gu[:, : gu.shape[1] // 2]) * gu[:, gu.shape[1] // 2:]
    return xf + f @ layer.wdown.float().t()


def test_decoder_layer_matches_fp32_reference_and_is_batch_invariant(cuda_device):
    cfg = LlamaConfig.tiny()
    tp = TPContext(device=cuda_device)
    layer = DecoderLayer(cfg, tp, seed=3, device=cuda_device)
    cos, sin = rope_tables(cfg.max_pos, cfg.head_dim, cfg.rope_theta, device=cuda_device)
    batch, seq_len = 4, 256
    g = torch.Generator(device=cuda_device).manual_seed(0)
    x = torch.randn(batch * seq_len, cfg.hidden, device=cuda_device, generator=g).to(torch.bfloat16)
    pos = torch.arange(seq_len, device=cuda_device).repeat(batch)
    with torch.no_grad():
        y = layer(x, batch, seq_len, pos, cos, sin)
        ref = _ref_layer(layer, x, batch, seq_len, cos, sin)
        gemm.check_status(cuda_device)
        assert (y.float() - ref).abs().max().item() < 0.06 * ref.abs().max().item()
        assert torch.equal(y, layer(x, batch, seq_len, pos, cos, sin))
        one = layer(x[seq_len:2 * seq_len], 1, seq_len, pos[:seq_len], cos, sin)
        assert torch.equal(one, y[seq_len:2 * seq_len])


def test_model_forward_backward_produces_finite_repeatable_grads(cuda_device):
    from kernel_align_b200.ops.fused_logp import lmhead_logp

    cfg = LlamaConfig.tiny(n_layers=2)
    model = LlamaModel(cfg, seed=1, device=cuda_device)
    g = torch.Generator(device=cuda_device).manual_seed(2)
    ids = torch.randint(0, cfg.vocab_size, (2, 128), device=cuda_device, generator=g)

    def run():
        model.zero_grad(set_to_none=True)
        h = model.hidden_states(ids)
        logp = lmhead_logp(h[: ids.numel()], model.lm_head, ids.reshape(-1))
        loss = -logp.mean()
        loss.backward()
        return loss.detach().clone(), [p.grad.clone() for p in model.parameters() if p.grad is not None]

    l1, g1 = run()
    l2, g2 = run()
    gemm.check_status(cuda_device)
    assert torch.isfinite(l1) and abs(l1.item() - math.log(cfg.vocab_size)) < 1.0
    assert l1.item() == l2.item()
    assert len(g1) >= 4 * cfg.n_layers and all(torch.isfinite(t.float()).all() for t in g1)
    assert all(torch.equal(a, b) for a, b in zip(g1, g2))
