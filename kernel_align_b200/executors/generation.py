"""Rollout generation: prefill the prompts, then decode token by token with a KV cache, drawing
every token with the fused sampler and recording its log-probability.

Runs per data-parallel rank (``tp.world == 1``): each rank generates for its own prompts. All
heavy steps are the native kernels: GEMMs (``gemm_bi``), prefill attention, decode attention,
RMSNorm, RoPE, SwiGLU, the sampler and the logits log-prob kernel.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels.sampling import SamplerBackend
from ..ops.attention import attention
from ..ops.decode import attention_decode
from ..ops.gemm import gemm_bi
from ..ops.layer_ops import rmsnorm, rope_, swiglu
from ..ops.logits_logp import logits_logp


@torch.no_grad()
def _layer_step(layer, x, batch, seq_len, positions, cos, sin, cache_k, cache_v, start: int):
    """Run one decoder layer on ``seq_len`` new tokens per sequence starting at ``start``,
    appending their keys / values to the cache. Prefill when ``start == 0`` and ``seq_len > 1``."""
    cfg = layer.cfg
    hd, hq, hkv = cfg.head_dim, layer.hq, layer.hkv
    tokens = batch * seq_len
    h = rmsnorm(x, layer.norm1, cfg.rms_eps)
    qkv = gemm_bi(h, layer.wqkv)
    q = qkv[:, : hq * hd].reshape(tokens, hq, hd).contiguous()
    k = qkv[:, hq * hd:(hq + hkv) * hd].reshape(tokens, hkv, hd).contiguous()
    v = qkv[:, (hq + hkv) * hd:].reshape(batch, seq_len, hkv, hd)
    rope_(q, positions, cos, sin)
    rope_(k, positions, cos, sin)
    cache_k[:, start:start + seq_len] = k.view(batch, seq_len, hkv, hd)
    cache_v[:, start:start + seq_len] = v
    if seq_len > 1:
        a = attention(q.view(batch, seq_len, hq, hd), k.view(batch, seq_len, hkv, hd), v.contiguous(), causal=True)
        a = a.reshape(tokens, hq * hd)
    else:
        lens = torch.full((batch,), start + 1, dtype=torch.int32, device=x.device)
        a = attention_decode(q.view(batch, hq, hd), cache_k, cache_v, lens).reshape(batch, hq * hd)
    x = x + gemm_bi(a, layer.wo)
    h = rmsnorm(x, layer.norm2, cfg.rms_eps)
    x = x + gemm_bi(swiglu(gemm_bi(h, layer.wgu)), layer.wdown)
    return x


@torch.no_grad()
def generate(model, prompts: torch.Tensor, sampler: Optional[SamplerBackend] = None, max_new_tokens: int = 16,
             temperature: float = 1.0, top_k: Optional[int] = None, top_p: Optional[float] = None,
             group_size: int = 1, row_id_offset: int = 0) -> dict:
    """``prompts [P, Lp]`` -> ``group_size`` completions each.

    Returns ``sequences [P * G, Lp + T]`` (int64), ``logp [P * G, T]`` (log-probability of each
    sampled token under ``softmax(logits / temperature)``) and ``new_tokens [P * G, T]``.
    Random streams are keyed by ``row_id_offset + row``, so a row's completion does not depend
    on which other rows are generated with it.
    """
    if model.tp.world != 1:
        raise ValueError("generation runs per data-parallel rank (tensor-parallel world size 1)")
    sampler = sampler if sampler is not None else SamplerBackend()
    cfg = model.cfg
    dev = model.embed.device
    seqs = prompts.to(dev).repeat_interleave(group_size, 0)
    batch, lp = seqs.shape
    total = lp + max_new_tokens
    caches = [(torch.zeros(batch, total, l.hkv, cfg.head_dim, dtype=torch.bfloat16, device=dev),
               torch.zeros(batch, total, l.hkv, cfg.head_dim, dtype=torch.bfloat16, device=dev)) for l in model.layers]
    out_tokens = torch.empty(batch, max_new_tokens, dtype=torch.int64, device=dev)
    out_logp = torch.empty(batch, max_new_tokens, dtype=torch.float32, device=dev)
    row_ids = torch.arange(batch, device=dev) + row_id_offset
    # prefill
    x = torch.nn.functional.embedding(seqs.reshape(-1), model.embed)
    pos = torch.arange(lp, device=dev).repeat(batch)
    for layer, (ck, cv) in zip(model.layers, caches):
        x = _layer_step(layer, x, batch, lp, pos, model.rope_cos, model.rope_sin, ck, cv, 0)
    last = x.view(batch, lp, -1)[:, -1].contiguous()
    for t in range(max_new_tokens):
        h = rmsnorm(last, model.norm, cfg.rms_eps)
        logits = gemm_bi(h, model.lm_head)                                  # [batch, vocab] bf16
        tok = sampler.sample(logits, top_k=top_k, top_p=top_p, temperature=temperature, row_ids=row_ids).long()
        out_tokens[:, t] = tok
        out_logp[:, t] = logits_logp(logits, tok, scale=1.0 / temperature if temperature > 0 else 1.0)
        if t + 1 == max_new_tokens:
            break
        x = torch.nn.functional.embedding(tok, model.embed)
        pos = torch.full((batch,), lp + t, dtype=torch.int64, device=dev)
        for layer, (ck, cv) in zip(model.layers, caches):
            x = _layer_step(layer, x, batch, 1, pos, model.rope_cos, model.rope_sin, ck, cv, lp + t)
        last = x
    return {"sequences": torch.cat([seqs, out_tokens], 1), "new_tokens": out_tokens, "logp": out_logp}
