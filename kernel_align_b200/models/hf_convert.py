"""Loading Hugging Face Llama weights into :class:`LlamaModel`.

``config_from_hf(hf_config)`` maps a ``transformers.LlamaConfig`` to :class:`LlamaConfig`;
``load_hf_state_dict(model, state_dict)`` copies a ``LlamaForCausalLM`` state dict into a model
of any tensor-parallel degree: the q / k / v projections are fused per rank (this rank's heads),
gate and up are fused per rank (this rank's slice of the FFN), ``o_proj`` and ``down_proj`` are
split along their input dimension, and the LM head along the vocabulary in whole canonical
slices. The rotary convention (rotate-half, pairs ``(i, i + head_dim / 2)``) and the RMSNorm
are those of the Hugging Face implementation, so the two models compute the same function.

The reference has no model and no checkpoint loading; ``CheckpointFormat`` is an unused enum
(rl_engine/platforms/constants.py:69-73).
"""
from __future__ import annotations

from typing import Mapping

import torch

from .llama import LlamaConfig, LlamaModel


def config_from_hf(hf_config) -> LlamaConfig:
    scaling = getattr(hf_config, "rope_scaling", None)
    if scaling and scaling.get("rope_type", scaling.get("type", "default")) not in ("default", None):
        raise ValueError("only the plain rotary embedding is implemented (no rope scaling)")
    head_dim = getattr(hf_config, "head_dim", None) or hf_config.hidden_size // hf_config.num_attention_heads
    theta = getattr(hf_config, "rope_theta", None)
    if theta is None:
        theta = (getattr(hf_config, "rope_parameters", None) or {}).get("rope_theta", 10000.0)
    return LlamaConfig(vocab_size=hf_config.vocab_size, hidden=hf_config.hidden_size,
                       n_layers=hf_config.num_hidden_layers, n_heads=hf_config.num_attention_heads,
                       n_kv_heads=getattr(hf_config, "num_key_value_heads", hf_config.num_attention_heads),
                       head_dim=head_dim, ffn=hf_config.intermediate_size, rope_theta=float(theta),
                       rms_eps=float(hf_config.rms_norm_eps), max_pos=int(hf_config.max_position_embeddings))


@torch.no_grad()
def load_hf_state_dict(model: LlamaModel, state: Mapping[str, torch.Tensor]) -> None:
    """Copy ``LlamaForCausalLM`` weights (names ``model.layers.N.self_attn.q_proj.weight`` ...)
    into ``model``, taking this rank's shards. A tied head (no ``lm_head.weight``) uses the
    embedding matrix."""
    cfg, tp = model.cfg, model.tp
    r, hd = tp.rank, cfg.head_dim

    def get(name):
        key = name if name in state else name.removeprefix("model.")
        if key not in state:
            raise KeyError(f"missing weight {name}")
        return state[key]

    def put(param, value):
        if param.shape != value.shape:
            raise ValueError(f"shape mismatch: model {tuple(param.shape)} vs checkpoint {tuple(value.shape)}")
        param.copy_(value.to(device=param.device, dtype=param.dtype))

    put(model.embed, get("model.embed_tokens.weight"))
    put(model.norm, get("model.norm.weight"))
    head = state["lm_head.weight"] if "lm_head.weight" in state else get("model.embed_tokens.weight")
    lo, hi = model.vocab_range
    put(model.lm_head, head[lo:hi])
    for i, layer in enumerate(model.layers):
        p = f"model.layers.{i}."
        hq, hkv = layer.hq, layer.hkv
        f = cfg.ffn // tp.world
        q = get(p + "self_attn.q_proj.weight")[r * hq * hd:(r + 1) * hq * hd]
        k = get(p + "self_attn.k_proj.weight")[r * hkv * hd:(r + 1) * hkv * hd]
        v = get(p + "self_attn.v_proj.weight")[r * hkv * hd:(r + 1) * hkv * hd]
        put(layer.wqkv, torch.cat([q, k, v]))
        put(layer.wo, get(p + "self_attn.o_proj.weight")[:, r * hq * hd:(r + 1) * hq * hd])
        gate = get(p + "mlp.gate_proj.weight")[r * f:(r + 1) * f]
        up = get(p + "mlp.up_proj.weight")[r * f:(r + 1) * f]
        put(layer.wgu, torch.cat([gate, up]))
        put(layer.wdown, get(p + "mlp.down_proj.weight")[:, r * f:(r + 1) * f])
        put(layer.norm1, get(p + "input_layernorm.weight"))
        put(layer.norm2, get(p + "post_attention_layernorm.weight"))


def from_hf(hf_model, tp=None, device=None) -> LlamaModel:
    """A :class:`LlamaModel` with the architecture and weights of a ``LlamaForCausalLM``."""
    model = LlamaModel(config_from_hf(hf_model.config), tp=tp, seed=0, device=device)
    load_hf_state_dict(model, hf_model.state_dict())
    return model


@torch.no_grad()
def to_hf_state_dict(model: LlamaModel) -> dict:
    """The model's weights under ``LlamaForCausalLM`` names (the inverse of
    :func:`load_hf_state_dict`), e.g. to hand a trained policy to an inference engine. With a
    tensor-parallel model every rank gathers the other ranks' shards and returns the full
    state dict."""
    import torch.distributed as dist

    cfg, tp = model.cfg, model.tp
    hd = cfg.head_dim

    def gather(t: torch.Tensor) -> list:
        if tp.world == 1:
            return [t]
        parts = [torch.empty_like(t) for _ in range(tp.world)]
        dist.all_gather(parts, t.contiguous(), group=tp.group)
        return parts

    out = {"model.embed_tokens.weight": model.embed.detach().clone(), "model.norm.weight": model.norm.detach().clone()}
    if tp.world == 1:
        out["lm_head.weight"] = model.lm_head.detach().clone()
    else:
        from ..ops.fused_logp import vocab_shard_range

        width = vocab_shard_range(cfg.vocab_size, 0, tp.world)[1]
        mine = model.lm_head.detach()
        if mine.shape[0] < width:
            mine = torch.cat([mine, mine.new_zeros(width - mine.shape[0], mine.shape[1])])
        rows = []
        for r, part in enumerate(gather(mine)):
            lo, hi = vocab_shard_range(cfg.vocab_size, r, tp.world)
            rows.append(part[: hi - lo])
        out["lm_head.weight"] = torch.cat(rows)
    for i, layer in enumerate(model.layers):
        p = f"model.layers.{i}."
        hq, hkv = layer.hq, layer.hkv
        f = cfg.ffn // tp.world
        qkv = gather(layer.wqkv.detach())
        out[p + "self_attn.q_proj.weight"] = torch.cat([t[: hq * hd] for t in qkv])
        out[p + "self_attn.k_proj.weight"] = torch.cat([t[hq * hd:(hq + hkv) * hd] for t in qkv])
        out[p + "self_attn.v_proj.weight"] = torch.cat([t[(hq + hkv) * hd:] for t in qkv])
        out[p + "self_attn.o_proj.weight"] = torch.cat(gather(layer.wo.detach()), 1)
        gu = gather(layer.wgu.detach())
        out[p + "mlp.gate_proj.weight"] = torch.cat([t[:f] for t in gu])
        out[p + "mlp.up_proj.weight"] = torch.cat([t[f:] for t in gu])
        out[p + "mlp.down_proj.weight"] = torch.cat(gather(layer.wdown.detach()), 1)
        out[p + "input_layernorm.weight"] = layer.norm1.detach().clone()
        out[p + "post_attention_layernorm.weight"] = layer.norm2.detach().clone()
    return out


def load_pretrained(path: str, tp=None, device=None) -> LlamaModel:
    """Load a Llama checkpoint saved in Hugging Face format (``config.json`` + safetensors or
    ``.bin`` shards in a local directory) into a :class:`LlamaModel`: the checkpoint is read on
    the CPU with ``transformers`` and only this rank's shards are copied to ``device``."""
    import transformers

    hf = transformers.AutoModelForCausalLM.from_pretrained(path, torch_dtype=torch.bfloat16, low_cpu_mem_usage=True)
    model = from_hf(hf, tp=tp, device=device)
    del hf
    return model


def save_pretrained(model: LlamaModel, path: str) -> None:
    """Write the model as a Hugging Face Llama checkpoint (rank 0 of the tensor-parallel group
    writes; every rank takes part in gathering the shards)."""
    import transformers

    state = to_hf_state_dict(model)
    if model.tp.rank != 0:
        return
    cfg = model.cfg
    hf_cfg = transformers.LlamaConfig(hidden_size=cfg.hidden, intermediate_size=cfg.ffn, num_hidden_layers=cfg.n_layers,
                                      num_attention_heads=cfg.n_heads, num_key_value_heads=cfg.n_kv_heads,
                                      head_dim=cfg.head_dim, vocab_size=cfg.vocab_size, rms_norm_eps=cfg.rms_eps,
                                      rope_theta=cfg.rope_theta, max_position_embeddings=cfg.max_pos,
                                      tie_word_embeddings=False, attention_bias=False, mlp_bias=False,
                                      torch_dtype="bfloat16")
    hf = transformers.LlamaForCausalLM(hf_cfg).to(torch.bfloat16)
    missing, unexpected = hf.load_state_dict({k: v.cpu() for k, v in state.items()}, strict=False)
    missing = [k for k in missing if "rotary" not in k]
    if missing or unexpected:
        raise RuntimeError(f"state dict does not fit the Hugging Face model: missing {missing}, unexpected {unexpected}")
    hf.save_pretrained(path)
