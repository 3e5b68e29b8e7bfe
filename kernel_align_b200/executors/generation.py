"""Rollout generation: prefill the prompts, then decode token by token with a KV cache, drawing
every token with the fused sampler and recording its log-probability.

Each data-parallel rank generates for its own prompts. All heavy steps are the native kernels:
GEMMs (``gemm_bi``), prefill attention, decode attention, RMSNorm, RoPE, SwiGLU, the sampler
and the logits log-prob kernel. With a tensor-parallel model the activations stay replicated
over the group (no sequence sharding for one token per sequence): every rank runs its heads
and its slice of the FFN, the two row-parallel products are written into peer-mapped memory
and summed there by the deterministic all-reduce, the LM-head shards become full logits the
same way (each rank fills its columns of a zeroed buffer), and every rank draws the same token
from the same seeded stream.

On CUDA the decode step (embedding -> every layer -> final norm -> LM-head logits: a few
hundred small launches) is captured once in a CUDA graph and replayed per token; position,
cache length and cache slot live in device tensors that the graph itself advances, so a
replay needs no host input but the token buffer. Sampling and the log-prob pick stay outside
the graph (their random stream is keyed by a host-side step counter).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels.sampling import SamplerBackend
from ..ops.attention import attention
from ..ops.decode import attention_decode, decode_qkv_rope_cache
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
    x = x + _tp_sum(gemm_bi(a, layer.wo), layer.tp)
    h = rmsnorm(x, layer.norm2, cfg.rms_eps)
    x = x + _tp_sum(gemm_bi(swiglu(gemm_bi(h, layer.wgu)), layer.wdown), layer.tp)
    return x


def _tp_sum(t: torch.Tensor, tp) -> torch.Tensor:
    """Sum of the ranks' partial products in the fixed tree order (in place)."""
    if tp.world > 1:
        from ..parallel.collectives import all_reduce_det

        all_reduce_det(t, tp.group)
    return t


def _full_logits(model, h: torch.Tensor) -> torch.Tensor:
    """``[batch, vocab]`` logits from the (vocabulary-sharded) LM head."""
    local = gemm_bi(h, model.lm_head)
    tp = model.tp
    if tp.world == 1:
        return local
    import torch.distributed as dist

    from ..ops.fused_logp import vocab_shard_range

    width = vocab_shard_range(model.cfg.vocab_size, 0, tp.world)[1]       # the widest shard (rank 0's)
    padded = local if local.shape[1] == width else torch.cat([local, local.new_zeros(local.shape[0], width - local.shape[1])], 1)
    pieces = [torch.empty_like(padded) for _ in range(tp.world)]
    dist.all_gather(pieces, padded.contiguous(), group=tp.group)
    cols = []
    for r, piece in enumerate(pieces):
        lo, hi = vocab_shard_range(model.cfg.vocab_size, r, tp.world)
        cols.append(piece[:, : hi - lo])
    return torch.cat(cols, 1).contiguous()


class _TPDecodeBuffers:
    """Peer-mapped buffers of a tensor-parallel decode step. The two row-parallel products of a
    layer are written straight into ``act`` and summed there in place by the deterministic
    all-reduce; the LM-head shards are written into their columns of ``logits`` (zero elsewhere)
    and the same all-reduce turns that into the full logits on every rank (adding zeros is exact).
    Both vectors keep their handshake epoch on the device, so the whole step, collectives
    included, can be captured in a CUDA graph."""

    def __init__(self, model, batch: int):
        from ..parallel.collectives import SymmetricVector

        cfg, tp = model.cfg, model.tp
        dev = model.embed.device
        self.batch = batch
        self.n_act, self.n_logits = batch * cfg.hidden, batch * cfg.vocab_size
        self.act = SymmetricVector(self.n_act, torch.bfloat16, tp.group, dev, device_epoch=True)
        self.logits = SymmetricVector(self.n_logits, torch.bfloat16, tp.group, dev, device_epoch=True)
        self.act_view = self.act.tensor[: self.n_act].view(batch, cfg.hidden)
        self.logits_view = self.logits.tensor[: self.n_logits].view(batch, cfg.vocab_size)
        lo, hi = model.vocab_range
        self.my_cols = self.logits_view[:, lo:hi]
        self.cols_aligned = self.my_cols.data_ptr() % 16 == 0 and cfg.vocab_size % 8 == 0

    def reduce_act(self) -> torch.Tensor:
        self.act.all_reduce_(numel=self.n_act)
        return self.act_view

    def full_logits(self, h: torch.Tensor, lm_head: torch.Tensor) -> torch.Tensor:
        self.logits.tensor.zero_()
        if self.cols_aligned:
            gemm_bi(h, lm_head, out=self.my_cols)
        else:
            self.my_cols.copy_(gemm_bi(h, lm_head))
        self.logits.all_reduce_(numel=self.n_logits)
        return self.logits_view


@torch.no_grad()
def _layer_decode(layer, x, delta, batch, pos_t, cos, sin, cache_k, cache_v, lens_t, slot_t, tpbuf=None):
    """One decoder layer on one new token per sequence, with every step-dependent quantity in
    a device tensor (``pos_t [B]`` int64 position, ``lens_t [B]`` int32 keys to attend to,
    ``slot_t [1]`` int64 cache slot), so the same launches can be replayed from a graph.

    ``x`` is the residual stream and ``delta`` the previous block's output that has not been
    added to it yet (``None`` for the first layer): each residual add runs inside the RMSNorm
    kernel that follows it. Nine launches: norm, qkv GEMM, split + RoPE + cache write, attention,
    output GEMM, add + norm, gate / up GEMM, SwiGLU, down GEMM; with a tensor-parallel model
    (``tpbuf``) the two row-parallel products are followed by an in-place all-reduce.
    Returns ``(x, delta)``."""
    cfg = layer.cfg
    if delta is None:
        h = rmsnorm(x, layer.norm1, cfg.rms_eps)
    else:
        h, x = rmsnorm(delta, layer.norm1, cfg.rms_eps, residual=x)
    qkv = gemm_bi(h, layer.wqkv)
    q = decode_qkv_rope_cache(qkv, pos_t, slot_t, cos, sin, cache_k, cache_v, layer.hq, layer.hkv)
    a = attention_decode(q, cache_k, cache_v, lens_t).reshape(batch, layer.hq * cfg.head_dim)
    if tpbuf is None:
        h, x = rmsnorm(gemm_bi(a, layer.wo), layer.norm2, cfg.rms_eps, residual=x)
        return x, gemm_bi(swiglu(gemm_bi(h, layer.wgu)), layer.wdown)
    gemm_bi(a, layer.wo, out=tpbuf.act_view)
    h, x = rmsnorm(tpbuf.reduce_act(), layer.norm2, cfg.rms_eps, residual=x)
    gemm_bi(swiglu(gemm_bi(h, layer.wgu)), layer.wdown, out=tpbuf.act_view)
    return x, tpbuf.reduce_act()     # consumed by the next RMSNorm before the buffer is written again


class _DecodeGraph:
    """The captured decode step. ``step(tok)`` consumes the tokens sampled at the previous
    position and returns the logits of the next one (a static buffer, overwritten per call)."""

    def __init__(self, model, caches, batch: int, first_pos: int):
        dev = model.embed.device
        self.model, self.caches, self.batch = model, caches, batch
        self.tok = torch.zeros(batch, dtype=torch.int64, device=dev)
        self.pos = torch.full((batch,), first_pos, dtype=torch.int64, device=dev)
        self.lens = torch.full((batch,), first_pos + 1, dtype=torch.int32, device=dev)
        self.slot = torch.full((1,), first_pos, dtype=torch.int64, device=dev)
        self.graph = None
        self.logits = None
        self.tpbuf = None
        if model.tp.world > 1:
            # peer-mapped memory is allocated collectively: keep it with the model, per batch size
            cache = model.__dict__.setdefault("_tp_decode_buffers", {})
            if batch not in cache:
                cache[batch] = _TPDecodeBuffers(model, batch)
            self.tpbuf = cache[batch]

    def _body(self):
        m = self.model
        x = torch.nn.functional.embedding(self.tok, m.embed)
        delta = None
        for layer, (ck, cv) in zip(m.layers, self.caches):
            x, delta = _layer_decode(layer, x, delta, self.batch, self.pos, m.rope_cos, m.rope_sin, ck, cv, self.lens,
                                     self.slot, self.tpbuf)
        h = rmsnorm(x, m.norm, m.cfg.rms_eps) if delta is None else rmsnorm(delta, m.norm, m.cfg.rms_eps, residual=x)[0]
        logits = gemm_bi(h, m.lm_head) if self.tpbuf is None else self.tpbuf.full_logits(h, m.lm_head)
        self.pos += 1
        self.lens += 1
        self.slot += 1
        return logits

    def step(self, tok: torch.Tensor, capture: bool) -> torch.Tensor:
        self.tok.copy_(tok)
        if self.graph is not None:
            self.graph.replay()
            return self.logits
        if not capture:
            return self._body()          # eager: also the warm-up that precedes a capture
        g = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(g):
                self.logits = self._body()
        except RuntimeError as e:
            # something on this path cannot be captured: stay eager (state tensors untouched,
            # a capture records launches without running them), and say so: an eager decode
            # step is two to three times slower
            from ..utils.logger import logger

            logger.warn_once(f"decode step could not be captured in a CUDA graph, running eagerly: {str(e)[:200]}")
            self.graph = None
            return self._body()
        self.graph = g
        g.replay()
        return self.logits


@torch.no_grad()
def generate(model, prompts: torch.Tensor, sampler: Optional[SamplerBackend] = None, max_new_tokens: int = 16,
             temperature: float = 1.0, top_k: Optional[int] = None, top_p: Optional[float] = None,
             group_size: int = 1, row_id_offset: int = 0, cuda_graph: bool = True,
             eos_token_id: Optional[int] = None, pad_token_id: int = 0) -> dict:
    """``prompts [P, Lp]`` -> ``group_size`` completions each.

    Returns ``sequences [P * G, Lp + T]`` (int64), ``logp [P * G, T]`` (log-probability of each
    sampled token under ``softmax(logits / temperature)``) and ``new_tokens [P * G, T]``. With
    ``eos_token_id`` a completion ends at its first EOS token: later positions hold
    ``pad_token_id`` with log-prob 0, and ``mask [P * G, T]`` (1.0 up to and including the EOS)
    says which positions count; the loop stops early once every row has ended.
    Random streams are keyed by ``row_id_offset + row``, so a row's completion does not depend
    on which other rows are generated with it.
    """
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
    logits = _full_logits(model, rmsnorm(last, model.norm, cfg.rms_eps))           # [batch, vocab] bf16
    # (a tensor-parallel step is captured as well: its all-reduces keep their epoch on the device)
    use_graph = cuda_graph and dev.type == "cuda" and max_new_tokens > 3
    dec = _DecodeGraph(model, caches, batch, lp) if dev.type == "cuda" else None
    finished = torch.zeros(batch, dtype=torch.bool, device=dev) if eos_token_id is not None else None
    mask = torch.zeros(batch, max_new_tokens, dtype=torch.float32, device=dev) if eos_token_id is not None else None
    if eos_token_id is not None:
        out_tokens.fill_(pad_token_id)
        out_logp.zero_()
    for t in range(max_new_tokens):
        tok = sampler.sample(logits, top_k=top_k, top_p=top_p, temperature=temperature, row_ids=row_ids).long()
        lp_t = logits_logp(logits, tok, scale=1.0 / temperature if temperature > 0 else 1.0)
        if finished is not None:
            alive = ~finished
            mask[:, t] = alive.float()
            tok = torch.where(alive, tok, torch.full_like(tok, pad_token_id))
            lp_t = torch.where(alive, lp_t, torch.zeros_like(lp_t))
            finished = finished | (tok == eos_token_id)
        out_tokens[:, t] = tok
        out_logp[:, t] = lp_t
        if t + 1 == max_new_tokens or (finished is not None and bool(finished.all())):
            break
        if dec is not None:
            # first decode step eager (loads every kernel at this shape), second one captured
            logits = dec.step(tok, capture=use_graph and t >= 1)
            continue
        x = torch.nn.functional.embedding(tok, model.embed)
        pos = torch.full((batch,), lp + t, dtype=torch.int64, device=dev)
        for layer, (ck, cv) in zip(model.layers, caches):
            x = _layer_step(layer, x, batch, 1, pos, model.rope_cos, model.rope_sin, ck, cv, lp + t)
        logits = _full_logits(model, rmsnorm(x, model.norm, cfg.rms_eps))
    out = {"sequences": torch.cat([seqs, out_tokens], 1), "new_tokens": out_tokens, "logp": out_logp}
    if mask is not None:
        out["mask"] = mask
    return out
