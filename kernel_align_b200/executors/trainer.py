"""GRPO training step on the native operators.

One step = rollout (``generate``: G completions per prompt with the fused sampler, their
log-probabilities recorded) -> rewards -> group-normalised advantages -> policy forward with
autograd through the native kernels -> fused LM-head log-prob -> clipped-ratio loss ->
backward -> deterministic gradient all-reduce over the data-parallel ranks (overlapped with
backward, :class:`GradReducer`) -> fused AdamW. Every kernel on that path reduces in a fixed
order, so the loss of a step is bitwise reproducible run to run.

The reference has no trainer; its README lists GRPO as the target workload.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from ..kernels.sampling import SamplerBackend
from ..ops.decode import FusedAdamW
from ..ops.grpo_loss import group_advantages, grpo_loss
from ..utils.logger import logger
from ..utils.profiler import profile_range
from .generation import generate


class GRPOTrainer:
    def __init__(self, model, reward_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], *,
                 group_size: int = 8, max_new_tokens: int = 16, temperature: float = 1.0, top_k: Optional[int] = None,
                 top_p: Optional[float] = None, eps_clip: float = 0.2, beta: float = 0.0, lr: float = 1e-6,
                 weight_decay: float = 0.0, seed: int = 0, data_parallel: bool = False,
                 bucket_bytes: int = 64 << 20, dp_group: Optional["dist.ProcessGroup"] = None,
                 ref_model=None, updates_per_rollout: int = 1, eos_token_id: Optional[int] = None,
                 pad_token_id: int = 0, micro_batch: Optional[int] = None, zero_stage: int = 0,
                 max_grad_norm: Optional[float] = None):
        self.model = model
        self.reward_fn = reward_fn
        self.group_size, self.max_new_tokens = group_size, max_new_tokens
        self.temperature, self.top_k, self.top_p = temperature, top_k, top_p
        self.eps_clip, self.beta = eps_clip, beta
        # ref_model: a frozen policy for the KL term (beta > 0); without one the KL is taken to the
        # policy that produced the rollouts. updates_per_rollout: optimizer steps on one batch of
        # rollouts (after the first the ratio moves away from 1 and the clipping becomes active).
        self.ref_model, self.updates_per_rollout = ref_model, max(1, int(updates_per_rollout))
        self.eos_token_id, self.pad_token_id = eos_token_id, pad_token_id
        # micro_batch: sequences per backward pass of the policy update (gradient accumulation);
        # with model.checkpoint_layers it bounds the activation memory of a large rollout batch
        self.micro_batch = micro_batch
        # max_grad_norm: clip the global gradient norm (computed in a fixed order, over the
        # tensor-parallel shards too); applied as a scale inside the fused optimizer kernel
        self.max_grad_norm = max_grad_norm
        self.last_grad_norm: Optional[torch.Tensor] = None
        self.sampler = SamplerBackend(seed=seed)
        self.step_index = 0
        self.dp_group = dp_group
        self.dp = data_parallel and dist.is_available() and dist.is_initialized() and \
            dist.get_world_size(dp_group) > 1
        self.dp_rank = dist.get_rank(dp_group) if self.dp else 0
        self.dp_world = dist.get_world_size(dp_group) if self.dp else 1
        self.reducer = None
        self._bucket_bytes = bucket_bytes
        self.on_cuda = next(model.parameters()).device.type == "cuda"
        if self.dp and self.on_cuda:
            from ..parallel.collectives import GradReducer

            self.reducer = GradReducer(model.parameters(), group=dp_group, bucket_bytes=bucket_bytes, average=True)
        if zero_stage == 1 and self.dp:
            # optimizer state sharded over the data-parallel ranks (parallel/zero.py)
            from ..parallel.zero import ShardedAdamW

            self.optimizer = ShardedAdamW(model.parameters(), group=dp_group, lr=lr, weight_decay=weight_decay)
        elif zero_stage not in (0, 1):
            raise ValueError("zero_stage must be 0 or 1")
        else:
            self.optimizer = FusedAdamW(model.parameters(), lr=lr, weight_decay=weight_decay)
        self._opt_args = dict(lr=lr, weight_decay=weight_decay)
        # Ranks drift apart during a rollout (early stops, the user's reward function), and the
        # device-side waits of the fused collectives are bounded by a couple of seconds. A host
        # barrier over a CPU group at the start of every update absorbs the skew; what a device
        # wait still reports afterwards is a real failure (see _check_device_waits).
        tp = getattr(model, "tp", None)
        self._multi_rank = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1 and \
            (self.dp or (tp is not None and tp.world > 1))
        self._host_group = None
        if self._multi_rank and self.on_cuda and dist.get_backend() != "gloo":
            self._host_group = dist.new_group(backend="gloo")     # collective: every rank builds a trainer

    def rebind_data_parallel(self, group) -> None:
        """Continue on another data-parallel group (after ``parallel.health.shrink_group``: the
        ranks that are left). Call between steps."""
        self.dp_group = group
        self.dp_world = dist.get_world_size(group)
        self.dp_rank = dist.get_rank(group)
        self.dp = self.dp_world > 1
        # the groups of the old world still contain the ranks that left: meet on the new one
        self._host_group = None
        self._rendezvous_group = group
        from ..parallel.zero import ShardedAdamW

        if isinstance(self.optimizer, ShardedAdamW):
            # The departed ranks took their slices of the master weights and moments with them.
            # Re-shard over the new group: master weights restart from the bf16 parameters (which
            # every rank holds in full); the moments and the step count restart at zero (a fresh
            # optimizer, consistent bias correction). Load a checkpoint written by the new group
            # afterwards to continue with exact state.
            self.optimizer = ShardedAdamW(self.model.parameters(), group=group, **self._opt_args) if self.dp else \
                FusedAdamW(self.model.parameters(), **self._opt_args)
            logger.warn_once("ZeRO-1 optimizer state was re-sharded after the group changed: moments reset")
        if self.reducer is not None:
            self.reducer.close()
            self.reducer = None
        if self.dp and self.on_cuda:
            from ..parallel.collectives import GradReducer

            self.reducer = GradReducer(self.model.parameters(), group=group, bucket_bytes=self._bucket_bytes,
                                       average=True)

    # ------------------------------------------------------------------ phases
    def rollout(self, prompts: torch.Tensor) -> dict:
        """``prompts [P, Lp]`` of this rank -> sequences, sampled-token log-probs, rewards, advantages."""
        p = prompts.shape[0]
        out = generate(self.model, prompts, sampler=self.sampler, max_new_tokens=self.max_new_tokens,
                       temperature=self.temperature, top_k=self.top_k, top_p=self.top_p, group_size=self.group_size,
                       row_id_offset=self.dp_rank * p * self.group_size, eos_token_id=self.eos_token_id,
                       pad_token_id=self.pad_token_id)
        rewards = self.reward_fn(prompts.repeat_interleave(self.group_size, 0), out["new_tokens"]).float()
        out["rewards"] = rewards
        out["advantages"] = group_advantages(rewards, self.group_size)
        return out

    def policy_logp(self, sequences: torch.Tensor, prompt_len: int) -> torch.Tensor:
        """Log-probability of every generated token under the current policy, with autograd.
        Works for a tensor-parallel model as well (``LlamaModel.token_logp``)."""
        inputs, targets = sequences[:, :-1], sequences[:, 1:]
        logp = self.model.token_logp(inputs, targets, scale=1.0 / self.temperature if self.temperature > 0 else 1.0)
        return logp[:, prompt_len - 1:]

    def policy_update(self, sequences: torch.Tensor, logp_old: torch.Tensor, advantages: torch.Tensor,
                      prompt_len: int, mask: Optional[torch.Tensor] = None, logp_ref: Optional[torch.Tensor] = None):
        """The learner half of a step on given rollouts: policy forward, clipped-ratio loss,
        backward, gradient all-reduce over the data-parallel group, optimizer. The model may be
        tensor parallel (DP x TP: pass its data-parallel group as ``dp_group``); rollouts then come
        from elsewhere, since generation runs on an unsharded model. Returns ``(loss, stats)``."""
        dev = sequences.device
        self._host_rendezvous()
        if self.reducer is not None:
            self.reducer.zero_grad()
        else:
            self.optimizer.zero_grad(set_to_none=True)
        n_seq = sequences.shape[0]
        mb = n_seq if not self.micro_batch else max(1, min(int(self.micro_batch), n_seq))
        chunks = [(i, min(n_seq, i + mb)) for i in range(0, n_seq, mb)]
        # the loss is a mean over all valid tokens: a chunk enters with the share of tokens it holds
        if mask is not None:
            valid = mask.float().sum(1)
            total_valid = valid.sum().clamp_min(1.0)
        loss, stats = None, None
        for ci, (lo, hi) in enumerate(chunks):
            last = ci == len(chunks) - 1
            if self.reducer is not None:
                self.reducer.hold = not last
            with profile_range("grpo/policy_forward", dev):
                logp_new = self.policy_logp(sequences[lo:hi], prompt_len)
                ref = (logp_ref if logp_ref is not None else logp_old) if self.beta > 0 else None
                part, st = grpo_loss(logp_new, logp_old[lo:hi], advantages[lo:hi],
                                     mask=mask[lo:hi] if mask is not None else None, eps_low=self.eps_clip,
                                     beta=self.beta, logp_ref=ref[lo:hi] if ref is not None else None,
                                     return_stats=True)
                if len(chunks) > 1:
                    share = (valid[lo:hi].sum() / total_valid) if mask is not None else (hi - lo) / n_seq
                    part = part * share
                    st = torch.stack([st[0] * share, st[1] * share, st[2]])     # loss, clip fraction, tokens
            with profile_range("grpo/backward_and_grad_reduce", dev):
                part.backward()
            loss = part.detach() if loss is None else loss + part.detach()
            stats = st if stats is None else stats + st
        with profile_range("grpo/backward_and_grad_reduce", dev):
            if self.reducer is not None:
                self.reducer.finish()
            elif self.dp:
                # CPU ranks (gloo): the same fixed-order sum, one tensor at a time, no overlap
                from ..parallel.collectives import all_reduce_det

                for p in self.model.parameters():
                    if p.grad is not None:
                        all_reduce_det(p.grad, self.dp_group)
                        p.grad.div_(self.dp_world)
            if getattr(self.model, "tp", None) is not None and self.model.tp.world > 1:
                self.model.reduce_replicated_grads()     # norm and embedding weights of a sharded model
        scale = self._clip_scale()
        self._check_device_waits(dev)      # raises before the weights move if a reduction is incomplete
        with profile_range("grpo/optimizer", dev):
            self.optimizer.step(grad_scale=scale)
        return loss, stats

    def _host_rendezvous(self) -> None:
        """Every rank of the job arrives here before the update's first kernel is launched."""
        if not self._multi_rank:
            return
        if getattr(self, "_rendezvous_group", None) is not None:
            dist.barrier(self._rendezvous_group)
        elif self._host_group is not None:
            dist.barrier(self._host_group)
        elif not self.on_cuda:
            dist.barrier()

    def _check_device_waits(self, dev) -> None:
        """One read of all status blocks the step's kernels report into (gradient buckets,
        scratch all-reduces, the tensor-parallel GEMMs, the fused log-prob). On a timeout the
        optimizer does not step: the gradients may be partly reduced. The arenas must then be
        cleared on every rank (``PeerArena.zero``) before the step is repeated."""
        if not (self._multi_rank and self.on_cuda):
            return
        from ..parallel.collectives import check_device_status

        check_device_status(dev)

    def _clip_scale(self) -> float:
        if self.max_grad_norm is None:
            return 1.0
        tp = getattr(self.model, "tp", None)
        sharded_model = tp is not None and tp.world > 1
        replicated = {id(p) for p in self.model.replicated_parameters()} if sharded_model else set()
        zero = None
        sq_shard, sq_repl = zero, zero
        for p in self.model.parameters():              # parameter order: a fixed summation order
            if p.grad is None:
                continue
            term = p.grad.float().pow(2).sum()
            if id(p) in replicated:
                sq_repl = term if sq_repl is None else sq_repl + term
            else:
                sq_shard = term if sq_shard is None else sq_shard + term
        if sq_shard is None and sq_repl is None:
            return 1.0
        if sharded_model and sq_shard is not None:
            # shards of a tensor-parallel model: sum the ranks' parts in the fixed tree order;
            # replicated tensors (embedding, norms) are counted once
            from ..parallel.collectives import all_reduce_det

            sq_shard = sq_shard.reshape(1).clone()
            all_reduce_det(sq_shard, tp.group)
            sq_shard = sq_shard[0]
        sq = sq_shard if sq_repl is None else (sq_repl if sq_shard is None else sq_shard + sq_repl)
        norm = sq.sqrt()
        self.last_grad_norm = norm.detach()
        return float(min(1.0, self.max_grad_norm / (norm.item() + 1e-6)))

    def train_step(self, prompts: torch.Tensor) -> dict:
        prompt_len = prompts.shape[1]
        with profile_range("grpo/rollout", prompts.device):
            roll = self.rollout(prompts)
        logp_ref = None
        if self.ref_model is not None and self.beta > 0:
            with torch.no_grad():
                seq = roll["sequences"]
                scale = 1.0 / self.temperature if self.temperature > 0 else 1.0
                logp_ref = self.ref_model.token_logp(seq[:, :-1], seq[:, 1:], scale=scale)[:, prompt_len - 1:]
        for _ in range(self.updates_per_rollout):
            loss, stats = self.policy_update(roll["sequences"], roll["logp"], roll["advantages"], prompt_len,
                                             mask=roll.get("mask"), logp_ref=logp_ref)
        self.step_index += 1
        tokens = roll["new_tokens"].numel()
        return {"loss": loss.detach(), "clip_fraction": stats[1], "tokens": tokens,
                "reward_mean": roll["rewards"].mean(), "step": self.step_index}

    # ------------------------------------------------------------------ checkpoint / resume
    def _shard_id(self) -> tuple[int, int]:
        """(index, count) of this process's checkpoint file: one per (data-parallel rank,
        tensor-parallel rank), since every such process holds different state or shards."""
        tp = getattr(self.model, "tp", None)
        tp_rank, tp_world = (tp.rank, tp.world) if tp is not None else (0, 1)
        return self.dp_rank * tp_world + tp_rank, self.dp_world * tp_world

    def save(self, path: str) -> str:
        from ..utils.checkpoint import save_checkpoint

        rank, world = self._shard_id()
        return save_checkpoint(path, self.model, self.optimizer, self.sampler, self.step_index, rank=rank, world=world)

    def load(self, path: str) -> None:
        from ..utils.checkpoint import load_checkpoint

        rank, world = self._shard_id()
        info = load_checkpoint(path, self.model, self.optimizer, self.sampler, rank=rank, world=world)
        self.step_index = info["step"]
        logger.info_on_rank(f"resumed from {path} at step {self.step_index}")
