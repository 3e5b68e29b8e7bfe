"""Pipeline parallelism over the decoder layers (GPipe schedule).

``PipelineStage`` holds a contiguous block of the decoder layers of a Llama model: stage 0 also
owns the token embedding, the last stage the final norm and the LM head. The weights come from
the same seeds as :class:`LlamaModel`, so an ``n``-stage pipeline is the same network as the
single-process model. ``pipeline_logp_step`` pushes ``n_micro`` micro-batches through the
stages (all forwards, then all backwards in reverse order), exchanging activations and their
gradients with point-to-point ``send`` / ``recv`` of ``torch.distributed`` (NCCL for CUDA
tensors, gloo for CPU tensors), and returns the per-token log-probabilities on the last
stage. Every operator is batch invariant, so the log-probabilities do not depend on the number
of micro-batches or stages: they are bitwise those of the unsplit model.

The reference only declares ``DistributedStrategy.PIPELINE_PARALLEL``
(rl_engine/platforms/constants.py:63-67); it has no pipeline code.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist
from torch import nn

from ..models.llama import DecoderLayer, LlamaConfig, _full_weight
from ..ops.fused_logp import lmhead_logp
from ..ops.layer_ops import rmsnorm_fn, rope_tables
from .tp_gemm import TPContext, rows_per_rank


def _solo_context(device) -> TPContext:
    ctx = TPContext.__new__(TPContext)
    ctx.group, ctx.rank, ctx.world, ctx.device, ctx._arenas = None, 0, 1, torch.device(device), {}
    return ctx


def stage_layers(n_layers: int, stage: int, n_stages: int) -> range:
    """Layer indices of ``stage``: as even a split as possible, earlier stages take the extra ones."""
    base, extra = divmod(n_layers, n_stages)
    lo = stage * base + min(stage, extra)
    return range(lo, lo + base + (1 if stage < extra else 0))


class PipelineStage(nn.Module):
    def __init__(self, cfg: LlamaConfig, stage: int, n_stages: int, seed: int = 0, device=None,
                 group: Optional[dist.ProcessGroup] = None, tp: Optional[TPContext] = None):
        super().__init__()
        if not 0 <= stage < n_stages or n_stages > cfg.n_layers:
            raise ValueError("need 0 <= stage < n_stages <= n_layers")
        dev = torch.device(device) if device is not None else \
            (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self.cfg, self.stage, self.n_stages, self.group = cfg, stage, n_stages, group
        # tp: shard this stage's layers over a tensor-parallel group as well (3-D layouts); the
        # pipeline group then links the ranks with the same tensor-parallel rank
        self.tp = tp if tp is not None else _solo_context(dev)
        self.first, self.last = stage == 0, stage == n_stages - 1
        self.layer_ids = stage_layers(cfg.n_layers, stage, n_stages)
        # the seeds of LlamaModel: embedding seed * 1000 + 1, head + 2, layer i + 10 + i
        self.layers = nn.ModuleList([DecoderLayer(cfg, self.tp, seed * 1000 + 10 + i, dev) for i in self.layer_ids])
        if self.first:
            self.embed = nn.Parameter(_full_weight(cfg.vocab_size, cfg.hidden, cfg.init_std, seed * 1000 + 1, dev))
        if self.last:
            from ..ops.fused_logp import vocab_shard_range

            self.norm = nn.Parameter(torch.ones(cfg.hidden, dtype=torch.bfloat16, device=dev))
            head = _full_weight(cfg.vocab_size, cfg.hidden, cfg.init_std, seed * 1000 + 2, dev)
            lo, hi = vocab_shard_range(cfg.vocab_size, self.tp.rank, self.tp.world)
            self.lm_head = nn.Parameter(head[lo:hi].contiguous())
        cos, sin = rope_tables(cfg.max_pos, cfg.head_dim, cfg.rope_theta, device=dev)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)

    @property
    def device(self) -> torch.device:
        return self.tp.device

    def run_layers(self, x: torch.Tensor, batch: int, seq_len: int) -> torch.Tensor:
        positions = torch.arange(seq_len, device=x.device).repeat(batch)
        for layer in self.layers:
            x = layer(x, batch, seq_len, positions, self.rope_cos, self.rope_sin)
        return x

    def embed_tokens(self, input_ids: torch.Tensor) -> torch.Tensor:
        """This tensor-parallel rank's token rows of the embedded micro-batch (zero padded)."""
        tokens = input_ids.numel()
        rpr = rows_per_rank(tokens, self.tp.world)
        flat = input_ids.reshape(-1)
        lo, hi = min(tokens, self.tp.rank * rpr), min(tokens, (self.tp.rank + 1) * rpr)
        x = torch.nn.functional.embedding(flat[lo:hi], self.embed)
        if hi - lo < rpr:
            x = torch.cat([x, x.new_zeros(rpr - (hi - lo), x.shape[1])])
        return x

    def token_logp(self, x_local: torch.Tensor, targets: torch.Tensor, scale: float) -> torch.Tensor:
        """Last stage: final norm and the LM head (vocabulary parallel over the tensor-parallel
        group) on this stage's output rows."""
        from ..ops.fused_logp import sharded_token_logp

        tokens = targets.numel()
        h = rmsnorm_fn(x_local, self.norm, self.cfg.rms_eps)
        if self.tp.world == 1:
            return lmhead_logp(h[:tokens], self.lm_head, targets.reshape(-1), scale=scale).view(targets.shape)
        return sharded_token_logp(h, self.lm_head, targets, self.cfg.vocab_size, self.tp, scale)

    def replicated_parameters(self) -> list:
        out = [self.embed] if self.first else []
        if self.last:
            out.append(self.norm)
        for layer in self.layers:
            out += [layer.norm1, layer.norm2]
        return out

    def reduce_replicated_grads(self) -> None:
        """As ``LlamaModel.reduce_replicated_grads``: sum the partial gradients of the weights
        that the tensor-parallel ranks of this stage hold in full."""
        if self.tp.world == 1:
            return
        from .collectives import all_reduce_det

        for p in self.replicated_parameters():
            if p.grad is None:
                p.grad = torch.zeros_like(p)
            all_reduce_det(p.grad, self.tp.group)


def _peer(stage_model: PipelineStage, stage: int) -> int:
    """Global rank of pipeline stage ``stage`` (ranks of the group in stage order)."""
    g = stage_model.group
    return dist.get_global_rank(g, stage) if g is not None else stage


def pipeline_logp_step(model: PipelineStage, input_ids: torch.Tensor, targets: torch.Tensor, n_micro: int,
                       loss_fn: Optional[Callable[[torch.Tensor, int], torch.Tensor]] = None, scale: float = 1.0):
    """One forward (+ backward when ``loss_fn`` is given) over ``input_ids [B, L]``.

    ``targets [B, L]`` are the ids whose log-probability is wanted (used on the last stage).
    ``loss_fn(logp_micro [b, L], micro_index)`` returns the scalar contribution of a micro-batch
    to the loss; gradients accumulate into the stage's parameters. Returns
    ``(logp [B, L] or None, loss or None)``: both live on the last stage only.
    """
    b, seq_len = input_ids.shape
    if b % n_micro:
        raise ValueError("the batch must split evenly into micro-batches")
    mb = b // n_micro
    dev = model.device
    cfg = model.cfg
    rpr = rows_per_rank(mb * seq_len, model.tp.world)
    train = loss_fn is not None
    saved = []          # per micro-batch: (input activation that needs a gradient, output or loss)
    logps = []
    total = None
    with torch.set_grad_enabled(train):
        for m in range(n_micro):
            ids_m = input_ids[m * mb:(m + 1) * mb].to(dev)
            if model.first:
                x_in = None
                x = model.embed_tokens(ids_m)
            else:
                x_in = torch.empty(rpr, cfg.hidden, dtype=torch.bfloat16, device=dev)
                dist.recv(x_in, src=_peer(model, model.stage - 1), group=model.group)
                if train:
                    x_in.requires_grad_()
                x = x_in
            x = model.run_layers(x, mb, seq_len)
            if model.last:
                tg = targets[m * mb:(m + 1) * mb].to(dev)
                logp = model.token_logp(x, tg, scale)
                logps.append(logp.detach())
                if train:
                    part = loss_fn(logp, m)
                    total = part.detach() if total is None else total + part.detach()
                    saved.append((x_in, part))
            else:
                dist.send(x.detach().contiguous(), dst=_peer(model, model.stage + 1), group=model.group)
                if train:
                    saved.append((x_in, x))
    if train:
        for m in reversed(range(n_micro)):
            x_in, out = saved[m]
            if model.last:
                out.backward()
            else:
                g_out = torch.empty(rpr, cfg.hidden, dtype=torch.bfloat16, device=dev)
                dist.recv(g_out, src=_peer(model, model.stage + 1), group=model.group)
                out.backward(g_out)
            if not model.first:
                dist.send(x_in.grad.contiguous(), dst=_peer(model, model.stage - 1), group=model.group)
            saved[m] = None
        model.reduce_replicated_grads()
    if model.last:
        return torch.cat(logps), total
    return None, None
