"""Optimizer-state sharding over the data-parallel ranks (ZeRO stage 1).

``ShardedAdamW`` keeps the fp32 master weights and the two moments of only ``1 / world`` of
every parameter on each rank: with AdamW those are 12 of the 16 bytes per parameter, so an
8B-parameter policy needs 12 GB instead of 96 GB of optimizer state per GPU at eight ranks.
A step updates this rank's slice with the same fused kernel (or the same formulas on CPU) as
:class:`~kernel_align_b200.ops.decode.FusedAdamW` and then gathers the updated bf16 slices of
all ranks into the parameter. The update is elementwise, so the parameters after a step are
bitwise those of the unsharded optimizer. Gradients must already be reduced over the group
(``GradReducer`` or ``all_reduce_det``), as for the unsharded optimizer.

The reference has no optimizer and no training loop.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native


class ShardedAdamW:
    def __init__(self, params, group: Optional[dist.ProcessGroup] = None, lr: float = 1e-6, betas=(0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.0):
        self.params = [p for p in params if p.requires_grad]
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.step_count = 0
        self.state = []
        for p in self.params:
            shard = -(-p.numel() // self.world)                     # elements per rank, the last ones padded
            lo = self.rank * shard
            mine = torch.zeros(shard, dtype=torch.float32, device=p.device)
            n = max(0, min(shard, p.numel() - lo))
            if n:
                mine[:n] = p.detach().reshape(-1)[lo:lo + n].float()
            self.state.append({"master": mine, "m": torch.zeros_like(mine), "v": torch.zeros_like(mine)})

    def zero_grad(self, set_to_none: bool = False) -> None:
        for p in self.params:
            if p.grad is not None:
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.zero_()

    def _grad_slice(self, p: torch.Tensor, shard: int) -> torch.Tensor:
        g = p.grad.contiguous().reshape(-1)
        lo = self.rank * shard
        n = max(0, min(shard, g.numel() - lo))
        out = g[lo:lo + n]
        if n < shard:
            out = torch.cat([out, out.new_zeros(shard - n)])
        return out.contiguous()

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0) -> None:
        self.step_count += 1
        b1, b2 = self.betas
        for p, st in zip(self.params, self.state):
            if p.grad is None:
                continue
            shard = st["master"].numel()
            g = self._grad_slice(p, shard)
            new = torch.empty(shard, dtype=p.dtype, device=p.device)
            if p.device.type != "cuda":
                gf = g.float() * grad_scale
                st["m"].mul_(b1).add_(gf, alpha=1 - b1)
                st["v"].mul_(b2).addcmul_(gf, gf, value=1 - b2)
                mh = st["m"] / (1 - b1 ** self.step_count)
                vh = st["v"] / (1 - b2 ** self.step_count)
                st["master"].mul_(1 - self.lr * self.weight_decay).addcdiv_(mh, vh.sqrt() + self.eps, value=-self.lr)
                new.copy_(st["master"].to(p.dtype))
            else:
                fn = _native.cuda().ka_adamw_step
                fn.restype = c_int
                fn.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_longlong, c_float, c_float,
                               c_float, c_float, c_float, c_int, c_float, c_int, c_void_p]
                sms = torch.cuda.get_device_properties(p.device).multi_processor_count
                rc = fn(new.data_ptr(), st["master"].data_ptr(), g.data_ptr(), int(g.dtype == torch.bfloat16),
                        st["m"].data_ptr(), st["v"].data_ptr(), shard, self.lr, b1, b2, self.eps, self.weight_decay,
                        self.step_count, grad_scale, sms, torch.cuda.current_stream(p.device).cuda_stream)
                if rc != 0:
                    raise RuntimeError(f"ka_adamw_step failed ({rc})")
            # every rank's updated slice -> the whole parameter
            if p.device.type == "cuda":
                full = torch.empty(self.world * shard, dtype=p.dtype, device=p.device)
                dist.all_gather_into_tensor(full, new, group=self.group)
            else:
                pieces = [torch.empty_like(new) for _ in range(self.world)]
                dist.all_gather(pieces, new, group=self.group)
                full = torch.cat(pieces)
            p.copy_(full[: p.numel()].view_as(p))

    def state_dict(self) -> dict:
        return {"step": self.step_count, "lr": self.lr, "betas": self.betas, "eps": self.eps,
                "weight_decay": self.weight_decay, "sharded": (self.rank, self.world),
                "state": [{k: v.clone() for k, v in st.items()} for st in self.state]}

    def load_state_dict(self, sd: dict) -> None:
        if tuple(sd.get("sharded", (self.rank, self.world))) != (self.rank, self.world):
            raise ValueError("this optimizer shard was saved by another rank or world size")
        self.step_count = sd["step"]
        self.lr, self.betas, self.eps, self.weight_decay = sd["lr"], tuple(sd["betas"]), sd["eps"], sd["weight_decay"]
        for st, src in zip(self.state, sd["state"]):
            for k in st:
                st[k].copy_(src[k])

    def state_bytes(self) -> int:
        """Bytes of optimizer state held by this rank."""
        return sum(t.numel() * t.element_size() for st in self.state for t in st.values())
