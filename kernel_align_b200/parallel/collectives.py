"""Deterministic collectives.

``all_reduce_det`` sums a tensor over the ranks of a group in the fixed order
``((0+1)+(2+3))+((4+5)+(6+7))`` in fp32, so the result is bitwise reproducible run to run and
identical on every rank. On CUDA the reduction is the peer-memory kernel of
``csrc/sm100/allreduce_det.cu`` working in place on symmetric buffers; on CPU (gloo) it is an
``all_gather`` followed by the same tree in PyTorch, which is also what the multi-process CPU
tests compare the GPU kernel's order against.

``GradReducer`` buckets a model's gradients into symmetric buffers and launches the all-reduce
of a bucket on a side stream as soon as the bucket's last gradient has been accumulated, so
communication overlaps the rest of the backward pass.

The reference declares ``DistributedStrategy.DATA_PARALLEL``
(rl_engine/platforms/constants.py:63-67) but implements no collective.
"""
from __future__ import annotations

import weakref
from ctypes import c_int, c_longlong, c_size_t, c_uint, c_ulonglong, c_void_p
from typing import Iterable, Optional, Sequence

import torch
import torch.distributed as dist

from .. import _native
from ..ops.fused_logp import default_timeout_ns
from ..utils.profiler import profiled


def tree_sum(parts: Sequence[torch.Tensor]) -> torch.Tensor:
    """Balanced pairwise sum in fp32, left to right at every level: the canonical order. With a
    count that is not a power of two the odd element of a level moves up unchanged (still one
    fixed order per count; used after a job has shrunk to the surviving ranks)."""
    level = [p.float() for p in parts]
    if not level:
        raise ValueError("tree_sum needs at least one part")
    while len(level) > 1:
        nxt = [level[i] + level[i + 1] for i in range(0, len(level) - 1, 2)]
        if len(level) & 1:
            nxt.append(level[-1])
        level = nxt
    return level[0]


class CollectiveTimeout(RuntimeError):
    """A bounded device-side wait of a fused collective ran out (a peer was late or gone)."""


_live_vectors: "weakref.WeakSet" = weakref.WeakSet()


class SymmetricVector:
    """A flat fp32 / bf16 vector in peer-mapped memory plus the flag block of the all-reduce."""

    def __init__(self, numel: int, dtype: torch.dtype, group: Optional[dist.ProcessGroup] = None, device=None,
                 device_epoch: bool = False):
        """``device_epoch``: keep the call counter that the handshake flags carry in device memory
        (the kernel advances it itself), so that ``all_reduce_`` can be captured in a CUDA graph
        and replayed. Every rank must choose the same mode for a vector."""
        from .peer import PeerArena

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.dtype = dtype
        esize = 4 if dtype == torch.float32 else 2
        gran = self.world * 4
        self.numel = (numel + gran - 1) // gran * gran
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        props = torch.cuda.get_device_properties(dev)
        lib = _native.cuda()
        lib.ka_allreduce_flag_bytes.restype = c_size_t
        lib.ka_allreduce_flag_bytes.argtypes = [c_int, c_int]
        self.data_bytes = (self.numel * esize + 255) // 256 * 256
        flag_bytes = lib.ka_allreduce_flag_bytes(self.world, props.multi_processor_count)
        self.arena = PeerArena(self.data_bytes + flag_bytes, self.group, dev)
        self.tensor = self.arena.buf[: self.numel * esize].view(dtype)
        self.epoch = 0
        self.sms = props.multi_processor_count
        self.status = torch.zeros(8, dtype=torch.int32, device=dev)
        self.epoch_dev = torch.zeros(2, dtype=torch.int32, device=dev) if device_epoch else None
        _live_vectors.add(self)

    def all_reduce_(self, stream: Optional[torch.cuda.Stream] = None, numel: Optional[int] = None) -> torch.Tensor:
        """Sum ``self.tensor`` (or its first ``numel`` elements, rounded up to ``world * 4``)
        over the group in place (enqueued on ``stream``). Every rank must pass the same count."""
        gran = self.world * 4
        n = self.numel if numel is None else min(self.numel, (int(numel) + gran - 1) // gran * gran)
        lib = _native.cuda()
        fn = lib.ka_allreduce_det_ex
        fn.restype = c_int
        fn.argtypes = [c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_uint, c_void_p, c_void_p, c_int,
                       c_ulonglong, c_void_p]
        self.epoch += 1
        bufs = (c_void_p * self.world)(*self.arena.ptrs)
        flags = (c_void_p * self.world)(*[p + self.data_bytes for p in self.arena.ptrs])
        st = stream if stream is not None else torch.cuda.current_stream(self.tensor.device)
        rc = fn(bufs, flags, n, int(self.dtype == torch.bfloat16), self.world, self.rank,
                self.epoch & 0xFFFFFFFF, self.epoch_dev.data_ptr() if self.epoch_dev is not None else None,
                self.status.data_ptr(), self.sms, default_timeout_ns(), st.cuda_stream)
        if rc != 0:
            raise RuntimeError(f"ka_allreduce_det rejected its arguments (code {rc})")
        return self.tensor

    def check(self) -> None:
        st = self.status.cpu().tolist()
        if st[0] != 0:
            self.status.zero_()
            raise CollectiveTimeout(f"deterministic all-reduce gave up: code {st[0]} at site {st[1]}, aux {st[3:6]}")


def check_device_status(device=None) -> None:
    """Read, with one device-to-host copy, the status blocks of every kernel with bounded waits
    that ran on ``device`` (all-reduce vectors and gradient buckets, the GEMM family with its
    fused reduce-scatter / all-gather, the fused log-prob) and raise :class:`CollectiveTimeout`
    if any wait gave up. A caller that sees the exception must not use the step's results:
    buffers may be half reduced. Clear the arenas on every rank (``PeerArena.zero``, collective)
    before the next attempt."""
    from ..ops import fused_logp, gemm

    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    blocks, names = [], []
    for v in list(_live_vectors):
        if v.status.device == dev:
            blocks.append(v.status)
            names.append(f"all-reduce vector ({v.numel} x {str(v.dtype).replace('torch.', '')})")
    blocks.append(gemm.status_buffer(dev)[:8])
    names.append("gemm / fused tensor-parallel gemm")
    for key, ws in fused_logp._workspaces.items():
        if key[0] == dev.index:
            blocks.append(ws.status[:8])
            names.append(f"fused lm-head log-prob (vocab {key[1]})")
    host = torch.stack([b.to(torch.int32) for b in blocks]).cpu()
    bad = [(names[i], host[i].tolist()) for i in range(len(blocks)) if int(host[i, 0]) != 0]
    if bad:
        for b in blocks:
            b.zero_()
        detail = "; ".join(f"{n}: code {st[0]} at site {st[1]}, block {st[2]}, aux {st[3:6]}" for n, st in bad)
        raise CollectiveTimeout("a device-side wait gave up: " + detail)


def reset_after_timeout() -> None:
    """After :class:`CollectiveTimeout`: clear all peer arenas and status blocks so that the
    step can be repeated. Collective over the default group (see ``peer.reset_all_arenas``)."""
    from .peer import reset_all_arenas

    reset_all_arenas()
    for v in list(_live_vectors):
        v.status.zero_()
        if v.epoch_dev is not None:
            v.epoch_dev.zero_()
        v.epoch = 0


_scratch: dict = {}
_SMALL_SCRATCH = 1 << 20      # elements of the scratch that serves small tensors


@profiled("all_reduce_det")
def all_reduce_det(tensor: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Fixed-order sum of ``tensor`` over ``group``, in place; every rank gets the same bits."""
    if not (dist.is_available() and dist.is_initialized()):
        return tensor
    g = group if group is not None else dist.group.WORLD
    world = dist.get_world_size(g)
    if world == 1:
        return tensor
    if tensor.device.type != "cuda":
        parts = [torch.empty_like(tensor) for _ in range(world)]
        dist.all_gather(parts, tensor.contiguous(), group=g)
        tensor.copy_(tree_sum(parts).to(tensor.dtype))
        return tensor
    dtype = torch.bfloat16 if tensor.dtype == torch.bfloat16 else torch.float32
    # Small tensors (norm weights, scalars, one decode step's activations) and large ones
    # (an embedding gradient) use separate scratch vectors, and a call only reduces the
    # elements it holds: a 4096-element sum after a 1 GB one stays a 4096-element sum.
    small = tensor.numel() <= _SMALL_SCRATCH
    key = (id(g), dtype, tensor.device.index, small)
    vec = _scratch.get(key)
    if vec is None or vec.numel < tensor.numel():
        vec = SymmetricVector(_SMALL_SCRATCH if small else tensor.numel(), dtype, g, tensor.device)
        _scratch[key] = vec       # the vector it replaces (a smaller large-tensor scratch) is dropped
    flat = tensor.reshape(-1)
    n = flat.numel()
    gran = world * 4
    n_pad = min(vec.numel, (n + gran - 1) // gran * gran)
    vec.tensor[:n].copy_(flat.to(dtype))
    if n_pad > n:
        vec.tensor[n:n_pad].zero_()
    vec.all_reduce_(numel=n_pad)
    tensor.copy_(vec.tensor[:n].view_as(tensor).to(tensor.dtype))
    return tensor


class GradReducer:
    """Bucketed, overlapped, deterministic gradient all-reduce for data parallelism.

    Parameters are packed (in reverse registration order, the order backward produces them)
    into buckets of about ``bucket_bytes`` (one dtype per bucket); each bucket is one
    :class:`SymmetricVector` and the parameters' ``.grad`` tensors are views into it, so no copy
    is needed. A bucket is reduced
    on ``self.stream`` as soon as all of its gradients have been accumulated. ``finish()`` makes
    the current stream wait for every bucket and divides by the world size if ``average``.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], group: Optional[dist.ProcessGroup] = None,
                 bucket_bytes: int = 64 << 20, average: bool = True):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.average = average
        self.params = [p for p in params if p.requires_grad]
        self.stream = torch.cuda.Stream()
        self.buckets: list[dict] = []
        cur, cur_bytes = [], 0
        for p in reversed(self.params):
            nbytes = p.numel() * p.element_size()
            if cur and (cur_bytes + nbytes > bucket_bytes or p.dtype != cur[0].dtype):
                self._make_bucket(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
        if cur:
            self._make_bucket(cur)
        self.hold = False      # set while gradients of all but the last micro-batch accumulate
        self._hooks = [p.register_post_accumulate_grad_hook(self._on_grad) for p in self.params]

    def _make_bucket(self, plist):
        total = sum(p.numel() for p in plist)
        # the bucket carries the parameters' dtype (what autograd produces); the all-reduce adds
        # in fp32 and rounds once at the end
        dtype = torch.bfloat16 if plist[0].dtype == torch.bfloat16 else torch.float32
        vec = SymmetricVector(total, dtype, self.group, plist[0].device)
        vec.tensor.zero_()
        off = 0
        for p in plist:
            p.grad = vec.tensor[off: off + p.numel()].view_as(p)
            off += p.numel()
        bucket = {"vec": vec, "params": plist, "pending": len(plist), "event": torch.cuda.Event()}
        for p in plist:
            p._ka_bucket = bucket
        self.buckets.append(bucket)

    def _on_grad(self, p):
        if self.hold:      # a micro-batch that is not the last: keep accumulating into the buckets
            return
        b = p._ka_bucket
        b["pending"] -= 1
        if b["pending"] == 0:
            ready = torch.cuda.Event()
            ready.record()
            self.stream.wait_event(ready)
            b["vec"].all_reduce_(self.stream)
            b["event"].record(self.stream)

    def finish(self) -> None:
        """Wait for all buckets; average; re-arm for the next backward pass."""
        cur = torch.cuda.current_stream()
        for b in self.buckets:
            if b["pending"] != 0:
                raise RuntimeError("a gradient bucket was not completed by this backward pass")
            cur.wait_event(b["event"])
            if self.average:
                b["vec"].tensor.mul_(1.0 / self.world)
            b["pending"] = len(b["params"])

    def zero_grad(self) -> None:
        for b in self.buckets:
            b["vec"].tensor.zero_()

    def check(self) -> None:
        for b in self.buckets:
            b["vec"].check()

    def close(self) -> None:
        """Detach from the parameters (before a reducer over another group replaces this one):
        the hooks are removed and the gradients stop being views of the buckets."""
        for h in self._hooks:
            h.remove()
        self._hooks = []
        for p in self.params:
            p.grad = None
