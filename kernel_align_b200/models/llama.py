"""Llama-3-style decoder built from the native operators, tensor-parallel and sequence-parallel.

Between blocks every rank holds ``rows_per_rank`` token rows of the residual stream (tokens are
flattened ``[B * L]`` and split contiguously; ``rows_per_rank`` is a multiple of 128, trailing
rows are zero padding). One layer:

    h = rmsnorm(x_local)                                            per-row kernel
    qkv = all_gather(h) @ Wqkv_shard^T                              fused AG -> GEMM
    q, k = rope(q), rope(k);  a = attention(q, k, v)                heads of this rank
    x_local = x_local + reduce_scatter(a @ Wo_shard^T)              fused GEMM -> RS (+ residual)
    h = rmsnorm(x_local)
    gu = all_gather(h) @ Wgu_shard^T;  f = swiglu(gu)               fused AG -> GEMM
    x_local = x_local + reduce_scatter(f @ Wdown_shard^T)           fused GEMM -> RS (+ residual)

Every step is either per row, per head, or reduces in the fixed 8-slice order, so the
residual stream is bitwise identical for any batch size and for TP = 1, 2, 4, 8.

The reference has no model; ``DistributedStrategy.MODEL_PARALLEL`` is only an enum value
(rl_engine/platforms/constants.py:63-67).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.utils.checkpoint

from ..ops.attention import attention_fn
from ..ops.layer_ops import rmsnorm_fn, rope_fn, rope_tables, swiglu_fn
from ..parallel.tp_gemm import TPContext, rows_per_rank
from ..parallel.tp_layers import column_parallel_linear, row_parallel_linear


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5
    max_pos: int = 8192
    init_std: float = 0.02

    @staticmethod
    def llama3_8b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def tiny(vocab_size: int = 2048, n_layers: int = 2) -> "LlamaConfig":
        """A small configuration with the same structure (GQA 4:1, head_dim 128) for tests."""
        return LlamaConfig(vocab_size=vocab_size, hidden=1024, n_layers=n_layers, n_heads=8, n_kv_heads=2,
                           head_dim=128, ffn=4096, max_pos=1024)


def _full_weight(rows: int, cols: int, std: float, seed: int, device) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed)
    out = torch.empty(rows, cols, dtype=torch.bfloat16, device=device)
    step = 4096
    for i in range(0, rows, step):
        n = min(step, rows - i)
        out[i:i + n] = (torch.randn(n, cols, generator=g) * std).to(torch.bfloat16).to(device)
    return out


class DecoderLayer(nn.Module):
    """One decoder block holding this rank's shards. Weights are generated for the *full*
    layer from ``seed`` and then sliced, so every TP degree sees the same model."""

    def __init__(self, cfg: LlamaConfig, tp: TPContext, seed: int, device):
        super().__init__()
        self.cfg, self.tp = cfg, tp
        w, r = tp.world, tp.rank
        d, hd = cfg.hidden, cfg.head_dim
        hq, hkv = cfg.n_heads // w, max(1, cfg.n_kv_heads // w)
        if cfg.n_heads % w or cfg.n_kv_heads % w:
            raise ValueError("heads must divide evenly over the tensor-parallel ranks")
        self.hq, self.hkv = hq, hkv
        wq = _full_weight(cfg.n_heads * hd, d, cfg.init_std, seed * 10 + 1, device)
        wk = _full_weight(cfg.n_kv_heads * hd, d, cfg.init_std, seed * 10 + 2, device)
        wv = _full_weight(cfg.n_kv_heads * hd, d, cfg.init_std, seed * 10 + 3, device)
        wo = _full_weight(d, cfg.n_heads * hd, cfg.init_std, seed * 10 + 4, device)
        wg = _full_weight(cfg.ffn, d, cfg.init_std, seed * 10 + 5, device)
        wu = _full_weight(cfg.ffn, d, cfg.init_std, seed * 10 + 6, device)
        wd = _full_weight(d, cfg.ffn, cfg.init_std, seed * 10 + 7, device)
        f = cfg.ffn // w
        self.wqkv = nn.Parameter(torch.cat([wq[r * hq * hd:(r + 1) * hq * hd], wk[r * hkv * hd:(r + 1) * hkv * hd],
                                            wv[r * hkv * hd:(r + 1) * hkv * hd]]).contiguous())
        self.wo = nn.Parameter(wo[:, r * hq * hd:(r + 1) * hq * hd].contiguous())
        self.wgu = nn.Parameter(torch.cat([wg[r * f:(r + 1) * f], wu[r * f:(r + 1) * f]]).contiguous())
        self.wdown = nn.Parameter(wd[:, r * f:(r + 1) * f].contiguous())
        self.norm1 = nn.Parameter(torch.ones(d, dtype=torch.bfloat16, device=device))
        self.norm2 = nn.Parameter(torch.ones(d, dtype=torch.bfloat16, device=device))

    def forward(self, x_local, batch: int, seq_len: int, positions, cos, sin):
        cfg, tp = self.cfg, self.tp
        hd = cfg.head_dim
        tokens = batch * seq_len
        h = rmsnorm_fn(x_local, self.norm1, cfg.rms_eps)
        qkv = column_parallel_linear(h, self.wqkv, tp)                       # [M_pad, (hq + 2 hkv) * hd]
        qkv = qkv[:tokens]
        q = qkv[:, : self.hq * hd].reshape(tokens, self.hq, hd)
        k = qkv[:, self.hq * hd:(self.hq + self.hkv) * hd].reshape(tokens, self.hkv, hd)
        v = qkv[:, (self.hq + self.hkv) * hd:].reshape(batch, seq_len, self.hkv, hd)
        q = rope_fn(q, positions, cos, sin).view(batch, seq_len, self.hq, hd)
        k = rope_fn(k, positions, cos, sin).view(batch, seq_len, self.hkv, hd)
        a = attention_fn(q, k, v, causal=True).reshape(tokens, self.hq * hd)
        m_pad = x_local.shape[0] * tp.world
        if m_pad != tokens:
            a = torch.cat([a, a.new_zeros(m_pad - tokens, a.shape[1])])
        x_local = row_parallel_linear(a, self.wo, tp, residual=x_local)
        h = rmsnorm_fn(x_local, self.norm2, cfg.rms_eps)
        gu = column_parallel_linear(h, self.wgu, tp)                         # [M_pad, 2 * ffn / world]
        f = swiglu_fn(gu)
        x_local = row_parallel_linear(f, self.wdown, tp, residual=x_local)
        return x_local


class LlamaModel(nn.Module):
    """Token embedding, ``n_layers`` decoder blocks, final norm and the (vocabulary-sharded,
    untied) LM-head weight used by the fused log-prob and sampling paths."""

    def __init__(self, cfg: LlamaConfig, tp: Optional[TPContext] = None, seed: int = 0, device=None):
        super().__init__()
        from ..ops.fused_logp import vocab_shard_range

        self.cfg = cfg
        self.tp = tp if tp is not None else TPContext(device=device)
        # activation checkpointing: set to True to store one tensor per layer instead of every
        # intermediate (about 17 tensors per layer) at the price of a second forward
        self.checkpoint_layers = False
        dev = self.tp.device
        self.embed = nn.Parameter(_full_weight(cfg.vocab_size, cfg.hidden, cfg.init_std, seed * 1000 + 1, dev))
        self.layers = nn.ModuleList([DecoderLayer(cfg, self.tp, seed * 1000 + 10 + i, dev) for i in range(cfg.n_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.hidden, dtype=torch.bfloat16, device=dev))
        head = _full_weight(cfg.vocab_size, cfg.hidden, cfg.init_std, seed * 1000 + 2, dev)
        lo, hi = vocab_shard_range(cfg.vocab_size, self.tp.rank, self.tp.world)
        self.vocab_range = (lo, hi)
        self.lm_head = nn.Parameter(head[lo:hi].contiguous())
        cos, sin = rope_tables(cfg.max_pos, cfg.head_dim, cfg.rope_theta, device=dev)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)

    def replicated_parameters(self) -> list:
        """Parameters that every tensor-parallel rank holds in full (embedding and norm weights);
        all others are shards."""
        out = [self.embed, self.norm]
        for layer in self.layers:
            out += [layer.norm1, layer.norm2]
        return out

    def reduce_replicated_grads(self) -> None:
        """Sum the gradients of the replicated parameters over the tensor-parallel group (call
        after backward, before the optimizer). Each rank normalises and embeds only its own token
        rows, so its gradient of a norm weight or of the embedding is a partial sum; without
        this step the copies of those parameters would drift apart. Fixed tree order."""
        if self.tp.world == 1:
            return
        from ..parallel.collectives import all_reduce_det

        for p in self.replicated_parameters():
            if not p.requires_grad:
                continue
            if p.grad is None:
                p.grad = torch.zeros_like(p)
            all_reduce_det(p.grad, self.tp.group)

    def rows_per_rank(self, tokens: int) -> int:
        return rows_per_rank(tokens, self.tp.world)

    def hidden_states(self, input_ids: torch.Tensor) -> torch.Tensor:
        """``input_ids [B, L]`` -> this rank's rows ``[rows_per_rank, hidden]`` of the final,
        normalised hidden states (token ``t`` lives on rank ``t // rows_per_rank``)."""
        batch, seq_len = input_ids.shape
        tokens = batch * seq_len
        rpr = self.rows_per_rank(tokens)
        r = self.tp.rank
        flat = input_ids.reshape(-1)
        lo, hi = min(tokens, r * rpr), min(tokens, (r + 1) * rpr)
        x = torch.nn.functional.embedding(flat[lo:hi], self.embed)
        if hi - lo < rpr:
            x = torch.cat([x, x.new_zeros(rpr - (hi - lo), x.shape[1])])
        positions = torch.arange(seq_len, device=flat.device).repeat(batch)
        recompute = self.checkpoint_layers and torch.is_grad_enabled()
        for layer in self.layers:
            if recompute:
                # keep only the layer's input; its activations are recomputed in backward (the
                # operators are deterministic, so the recomputed values are the same bits)
                x = torch.utils.checkpoint.checkpoint(layer, x, batch, seq_len, positions, self.rope_cos,
                                                      self.rope_sin, use_reentrant=False)
            else:
                x = layer(x, batch, seq_len, positions, self.rope_cos, self.rope_sin)
        return rmsnorm_fn(x, self.norm, self.cfg.rms_eps)

    def token_logp(self, input_ids: torch.Tensor, targets: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
        """Log-probability of ``targets [B, L]`` given ``input_ids [B, L]`` (fp32 ``[B, L]``, with
        autograd), on every rank of the tensor-parallel group. The layers leave every rank with
        its token rows of the hidden states; the LM head runs vocabulary parallel on them, the
        fused kernel gathering the other ranks' rows over NVLink while it works on its own and
        exchanging the (max, sum-exp, target) triples (over the CPU backend for CPU tensors)."""
        from ..ops.fused_logp import lmhead_logp, sharded_token_logp

        tokens = input_ids.numel()
        h = self.hidden_states(input_ids)
        if self.tp.world == 1:
            return lmhead_logp(h[:tokens], self.lm_head, targets.reshape(-1), scale=scale).view(targets.shape)
        return sharded_token_logp(h, self.lm_head, targets, self.cfg.vocab_size, self.tp, scale)
