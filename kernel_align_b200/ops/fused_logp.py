"""Fused LM-head + per-token log-probability.

``lmhead_logp(hidden, weight, ids)`` returns ``log_softmax(scale * hidden @ weight.T)[ids]``
without ever materialising the ``[rows, vocab]`` logits. On CUDA it runs the hand-written
tcgen05/TMA kernel of ``csrc/sm100/fused_lmhead_logp.cu``; on CPU the C++ implementation of
``csrc/cpu/fused_logp_cpu.cpp``. Both follow the same canonical decomposition of the
vocabulary (8 slices, 1792-column sub-slices, balanced merge tree), so a row's result does
not depend on the batch it was computed in, nor on how many GPUs the vocabulary is sharded
over.

The reference computes the same quantity from materialised logits
(rl_engine/kernels/sampling.py:91-112, ``SamplerBackend.compute_logp``).
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import _native
from ..utils.profiler import profiled

N_SLICES = 8
DEFAULT_PANEL_ROWS = 32768


def default_timeout_ns() -> int:
    return int(float(os.environ.get("RL_ENGINE_TIMEOUT_MS", "2000")) * 1e6)


def vocab_shard_range(vocab: int, rank: int, world: int) -> tuple[int, int]:
    """Rows of the LM-head weight that rank ``rank`` of ``world`` holds: whole canonical slices."""
    if world not in (1, 2, 4, 8):
        raise ValueError("vocab parallel world size must be 1, 2, 4 or 8")
    vs = -(-vocab // N_SLICES)
    per = N_SLICES // world
    lo = min(vocab, rank * per * vs)
    hi = min(vocab, (rank + 1) * per * vs)
    return lo, hi


class KernelStatusError(RuntimeError):
    """A device-side bounded wait gave up; the message carries the status block."""


@dataclass
class _Workspace:
    buf: torch.Tensor
    status: torch.Tensor
    nbytes: int
    epoch: int = 1


_workspaces: dict[tuple, _Workspace] = {}


def _get_workspace(device: torch.device, vocab: int, panel_rows: int) -> _Workspace:
    key = (device.index, vocab, panel_rows)
    ws = _workspaces.get(key)
    if ws is None:
        lib = _native.cuda()
        nbytes = lib.ka_lmhead_logp_workspace_bytes(vocab, panel_rows)
        off = lib.ka_lmhead_logp_status_offset(vocab, panel_rows)
        buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        status = buf[off : off + 32].view(torch.int32)
        ws = _Workspace(buf=buf, status=status, nbytes=nbytes)
        _workspaces[key] = ws
    return ws


def workspace_bytes(vocab: int, panel_rows: int = DEFAULT_PANEL_ROWS) -> int:
    """Scratch the CUDA path holds for a given vocabulary: independent of the row count."""
    return int(_native.cuda().ka_lmhead_logp_workspace_bytes(vocab, panel_rows))


_WHERE = {1: "producer waiting for a free stage", 2: "MMA waiting for operands",
          3: "MMA waiting for a free accumulator", 4: "epilogue waiting for an accumulator",
          5: "waiting for a peer rank's flag", 6: "waiting for a peer rank's rows (gather flag)",
          7: "row pusher waiting for its staging copy"}


def check_status(ws_status: torch.Tensor) -> None:
    """Synchronise and raise if the last launches reported a timeout. Clears the status."""
    st = ws_status.cpu().tolist()
    if st[0] != 0:
        ws_status.zero_()
        raise KernelStatusError(
            f"fused_lmhead_logp gave up (code {st[0]}) at site {st[1]} "
            f"({_WHERE.get(st[1], '?')}), block {st[2]}, aux {st[3:6]}"
        )


# ---- schedule selection -------------------------------------------------------------------
# The kernel has two tile variants (a CTA pair per 256-row tile, or one CTA per 128-row tile) and
# a free parameter of its work order (how many vocabulary sub-slices run side by side). All of
# them give the same bits; they differ in cycles and in power. The pair variant needs about 15 %
# fewer cycles, the single-CTA variant draws less power per cycle. A B200 that runs this kernel
# back to back sits at its power cap and clocks down, so there the second one is often faster,
# by an amount that depends on the GPU; in a short burst at full clock the first one wins. So
# the first large call of a shape times the candidates on the actual inputs, a quarter of a
# second each, and keeps the fastest (as cuDNN's benchmark mode does for convolutions).
# KA_LOGP_SCHEDULE="<cta_group>,<cg>[,<m_fast>[,<l2_hint>]]" pins a schedule; KA_LOGP_AUTOTUNE=0 keeps the default.
# (cta_group, sub-slices side by side, work order, L2 eviction hint of the operand loads)
#   work order: bit 0 = consecutive CTAs take consecutive row tiles (else consecutive sub-slices),
#               bit 1 = groups of sub-slices are the outer loop (W stays in L2, H streams)
#   L2 hint: 0 none, 1 keep H / stream W, 2 keep H, 3 keep W
_SCHEDULES = [(2, 8, 0, 0), (2, 8, 0, 2), (2, 8, 2, 3), (2, 4, 2, 3), (2, 4, 1, 0), (1, 4, 0, 1), (1, 4, 0, 0),
              (1, 2, 0, 3), (1, 4, 2, 3)]
_TUNE_MIN_MS = 250.0      # a candidate runs at least this long: the clock settles under the power cap
# Calls too short to be worth timing take the CTA pair, four sub-slices side by side, row tiles
# fastest: 16384 / 32768 rows against the whole 128256-column head took 13.4 / 28.2 ms with it,
# 14.1 / 29.5 ms with the kernel's own choice of the group (cg 0), 13.9 / 28.9 ms with (2, 8, 2, 3).
_DEFAULT_SCHEDULE = (2, 4, 1, 0)
# A shard of the LM head that about fits the L2 twice over (a vocabulary sharded 4 or 8 ways) is
# walked W-stationary with the keep-W hint: 12.9 ms against 13.5 - 14.0 ms for the default order
# on a 16128-column shard, in a burst and at the power cap alike.
_SMALL_SHARD_SCHEDULE = (2, 8, 2, 3)
_SMALL_SHARD_BYTES = 300 << 20
# Timing the candidates takes a quarter of a second each, two seconds in all, at full power: it
# pays for calls of tens of milliseconds (one or two GPUs at G = 256), not for shorter ones,
# which take the default for their shard size.
_AUTOTUNE_MIN_MACS = 3.0e13
_tuned: dict = {}


def _pinned_schedule():
    env = os.environ.get("KA_LOGP_SCHEDULE")
    if not env:
        return None
    try:
        parts = [int(x) for x in env.split(",")]
        g, cg = parts[0], parts[1]
        m_fast = parts[2] if len(parts) > 2 else 0
        hint = parts[3] if len(parts) > 3 else 0
    except (ValueError, IndexError):
        raise ValueError('KA_LOGP_SCHEDULE must look like "2,8", "1,4", "1,2,1" or "1,2,0,3"') from None
    if g not in (1, 2) or not 0 <= cg <= 64 or m_fast not in (0, 1, 2, 3) or hint not in (0, 1, 2, 3):
        raise ValueError("KA_LOGP_SCHEDULE: cta_group is 1 or 2, cg between 0 and 64, work order 0..3, l2_hint 0..3")
    return g, cg, m_fast, hint


def _choose_schedule(key, macs: float, device, launch, shard_bytes: int = 1 << 62):
    """The schedule for this call: pinned, tuned earlier, tuned now, or the default."""
    pinned = _pinned_schedule()
    if pinned is not None:
        return pinned
    if key in _tuned:
        return _tuned[key]
    if macs < _AUTOTUNE_MIN_MACS or os.environ.get("KA_LOGP_AUTOTUNE", "1") == "0" or \
            torch.cuda.is_current_stream_capturing():
        return _SMALL_SHARD_SCHEDULE if shard_bytes <= _SMALL_SHARD_BYTES and macs >= 1.0e11 else _DEFAULT_SCHEDULE
    # What decides under the power cap is the rate a schedule sustains, and the clock needs a
    # few hundred milliseconds to settle after a change of load: a candidate first runs once
    # (timed, to size the rest), then as many calls as fill _TUNE_MIN_MS (at least two), and
    # those are what is compared.
    timings = {}
    for sched in _SCHEDULES:
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        launch(*sched)
        e1.record()
        e1.synchronize()
        n = max(2, min(64, int(_TUNE_MIN_MS / max(e0.elapsed_time(e1), 1e-3)) + 1))
        for _ in range(n):
            launch(*sched)
        e2.record()
        e2.synchronize()
        timings[sched] = e1.elapsed_time(e2) / n
    best = min(timings, key=timings.get)
    _tuned[key] = best
    from ..utils.logger import logger

    logger.info_once(f"fused_lmhead_logp schedule for {key[1:]}: cta_group {best[0]}, cg {best[1]}, m_fast {best[2]}, "
                     f"l2_hint {best[3]} ({', '.join(f'{g}/{c}/{o}/{h}: {t:.2f} ms' for (g, c, o, h), t in timings.items())})")
    return best


@dataclass
class VocabParallel:
    """Description of a vocabulary-parallel group for :func:`lmhead_logp`.

    ``exchange`` holds, per rank, the address of that rank's symmetric exchange buffer as
    mapped in this process (see :mod:`kernel_align_b200.parallel.peer`).
    """

    rank: int
    world: int
    exchange_ptrs: list[int] = field(default_factory=list)
    epoch: int = 1
    panel_rows: int = DEFAULT_PANEL_ROWS
    process_group: object = None   # torch.distributed group (None: the default group); CPU path and backward
    gather_ptrs: dict = field(default_factory=dict)   # hidden size -> addresses of every rank's gather arena

    def gather_arena_ptrs(self, k: int) -> list[int]:
        """Addresses of the ranks' gather arenas for hidden size ``k`` (row-sharded input),
        allocated collectively on first use: every rank must ask in the same order."""
        ptrs = self.gather_ptrs.get(k)
        if ptrs is None:
            from ..parallel.peer import attach_gather_arena

            ptrs = attach_gather_arena(self, k)
        return ptrs


def _lmhead_logp_forward(
    hidden: torch.Tensor,
    weight: torch.Tensor,
    ids: torch.Tensor,
    *,
    scale: float = 1.0,
    vocab: Optional[int] = None,
    group: Optional[VocabParallel] = None,
    return_lse: bool = False,
    panel_rows: int = DEFAULT_PANEL_ROWS,
    cta_group: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
    check: bool = False,
    row_sharded: bool = False,
    gather_output: bool = False,
):
    """Per-token log-probabilities of ``ids`` under ``softmax(scale * hidden @ weight.T)``.

    hidden: ``[..., K]`` bf16; weight: ``[V_local, K]`` bf16 (this rank's vocabulary shard,
    whole canonical slices, see :func:`vocab_shard_range`); ids: ``[...]`` integer, global
    ids. Ids outside ``[0, vocab)`` give 0. Returns fp32 ``[...]`` (and the log-sum-exp if
    ``return_lse``). With ``row_sharded`` the rank passes only its rows of the batch (the same
    number on every rank) and gets their results, or, with ``gather_output``, the flat
    ``[world * rows]`` results of the whole batch.
    """
    lead = hidden.shape[:-1]
    k = hidden.shape[-1]
    h2 = hidden.reshape(-1, k)
    m = h2.shape[0]
    if ids.numel() != m:
        raise ValueError("ids must have one entry per row of hidden")
    world = 1 if group is None else group.world
    rank = 0 if group is None else group.rank
    sharded = bool(row_sharded) and world > 1
    if sharded and gather_output:
        lead = (world * m,)
    v_global = int(vocab) if vocab is not None else int(weight.shape[0])
    lo, hi = vocab_shard_range(v_global, rank, world)
    if weight.shape[0] != hi - lo or weight.shape[1] != k:
        raise ValueError(f"weight shard must be [{hi - lo}, {k}], got {tuple(weight.shape)}")

    if hidden.device.type != "cuda":
        from . import cpu_ops

        if sharded:
            # the rows travel over the CPU backend first; the rest is the replicated-rows path
            import torch.distributed as dist

            pg = getattr(group, "process_group", None)
            hs = [torch.empty_like(h2) for _ in range(world)]
            iv = ids.reshape(-1).to(torch.int64).contiguous()
            ivs = [torch.empty_like(iv) for _ in range(world)]
            dist.all_gather(hs, h2.contiguous(), group=pg)
            dist.all_gather(ivs, iv, group=pg)
            res = _lmhead_logp_forward(torch.cat(hs), weight, torch.cat(ivs), scale=scale, vocab=vocab, group=group,
                                       return_lse=return_lse, panel_rows=panel_rows)
            if gather_output:
                return res
            sl = slice(rank * m, (rank + 1) * m)
            if return_lse:
                return res[0][sl].reshape(lead), res[1][sl].reshape(lead)
            return res[sl].reshape(lead)
        if world != 1:
            # vocabulary parallel over the CPU backend of torch.distributed (gloo): every rank
            # computes the states of its canonical slices, all ranks gather the eight of them in
            # slice order and merge them with the same tree as a single process would
            import torch.distributed as dist

            pg = getattr(group, "process_group", None)
            states, target = cpu_ops.lmhead_logp_shard_cpu(h2, weight, ids.reshape(-1), vocab=v_global, v_lo=lo,
                                                           scale=scale)
            per = N_SLICES // world
            if states.shape[1] < per:      # a trailing shard with fewer (or no) columns: empty slices
                pad = torch.zeros(m, per - states.shape[1], 2)
                pad[..., 0] = float("-inf")
                states = torch.cat([states, pad], 1)
            all_states = [torch.empty_like(states) for _ in range(world)]
            all_targets = [torch.empty_like(target) for _ in range(world)]
            dist.all_gather(all_states, states.contiguous(), group=pg)
            dist.all_gather(all_targets, target, group=pg)
            tsum = all_targets[0].clone()
            for t in all_targets[1:]:
                tsum += t
            res = cpu_ops.lmhead_logp_merge_cpu(torch.cat(all_states, 1), tsum, ids.reshape(-1), vocab=v_global,
                                                return_lse=return_lse)
            if return_lse:
                return res[0].reshape(lead), res[1].reshape(lead)
            return res.reshape(lead)
        res = cpu_ops.lmhead_logp_cpu(h2, weight, ids.reshape(-1), scale=scale, return_lse=return_lse)
        if return_lse:
            return res[0].reshape(lead), res[1].reshape(lead)
        return res.reshape(lead)

    if hidden.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise TypeError("the sm_100a path takes bf16 hidden states and weights")
    if k % 8 != 0:
        raise ValueError("hidden size must be a multiple of 8")
    lib = _native.cuda()
    h2 = h2.contiguous()
    w = weight.contiguous()
    ids64 = ids.reshape(-1).to(torch.int64).contiguous()
    m_out = world * m if (sharded and gather_output) else m
    logp = out.reshape(-1) if out is not None else torch.empty(m_out, dtype=torch.float32, device=hidden.device)
    if logp.numel() != m_out:
        raise ValueError(f"out must have {m_out} elements")
    lse = torch.empty(m_out, dtype=torch.float32, device=hidden.device) if return_lse else None
    if group is not None:
        panel_rows = group.panel_rows
    ws = _get_workspace(hidden.device, v_global, panel_rows)
    if sharded and panel_rows % (256 * world) != 0:
        raise ValueError("row-sharded input needs panel_rows to be a multiple of 256 * world")
    n_panels = -(-m // (panel_rows // world)) if sharded else -(-m // panel_rows)
    peer_arr = (ctypes.c_void_p * world)(*group.exchange_ptrs) if world > 1 else None
    gather_arr = (ctypes.c_void_p * world)(*group.gather_arena_ptrs(k)) if sharded else None
    props = torch.cuda.get_device_properties(hidden.device)
    stream = torch.cuda.current_stream(hidden.device).cuda_stream

    def launch(g: int, cg: int, m_fast: int = 0, hint: int = 0) -> None:
        """Enqueue one forward with the given schedule (consumes the epochs of its panels)."""
        if world > 1:
            epoch = group.epoch
            group.epoch += n_panels
        else:
            epoch = ws.epoch
            ws.epoch += n_panels
        if sharded:
            rc = lib.ka_lmhead_logp_forward_sharded(
                h2.data_ptr(), w.data_ptr(), ids64.data_ptr(), logp.data_ptr(),
                lse.data_ptr() if lse is not None else None,
                ws.buf.data_ptr(), ws.nbytes, peer_arr, gather_arr,
                m, k, v_global, hi - lo, lo, world, rank,
                epoch & 0xFFFFFFFF, float(scale), panel_rows, 1 if gather_output else 0, g, cg, m_fast, hint,
                props.multi_processor_count, default_timeout_ns(), stream,
            )
        else:
            rc = lib.ka_lmhead_logp_forward_sched(
                h2.data_ptr(), w.data_ptr(), ids64.data_ptr(), logp.data_ptr(),
                lse.data_ptr() if lse is not None else None,
                ws.buf.data_ptr(), ws.nbytes, peer_arr,
                m, k, v_global, hi - lo, lo, world, rank,
                epoch & 0xFFFFFFFF, float(scale), panel_rows, g, cg, m_fast, hint, props.multi_processor_count,
                default_timeout_ns(), stream,
            )
        if rc != 0:
            raise RuntimeError(f"ka_lmhead_logp_forward rejected its arguments (code {rc})")

    if cta_group is None:
        # keyed and sized by quantities that are the same on every rank of a group, so that all
        # ranks tune (a collective sequence of calls when the vocabulary is sharded) or none does
        rows_total = m * world if sharded else m
        key = (hidden.device.index, rows_total, k, v_global, world, sharded)
        sched = _choose_schedule(key, float(rows_total) * k * (v_global / world), hidden.device, launch,
                                 shard_bytes=int(v_global / world) * k * 2)
    else:
        sched = (int(cta_group), 0, 0, 0)
    launch(*sched)
    if check:
        check_status(ws.status)
    logp = logp.reshape(lead)
    if return_lse:
        return logp, lse.reshape(lead)
    return logp


def last_status(device: torch.device, vocab: int, panel_rows: int = DEFAULT_PANEL_ROWS) -> torch.Tensor:
    """The status block of the workspace for (device, vocab): int32[8], zero when healthy."""
    return _get_workspace(device, vocab, panel_rows).status


_GRAD_PANEL_BYTES = 8 << 30


def _logp_backward(hidden, weight, ids, lse, g, scale, vocab, group, need_dh, need_dw):
    """Gradients of the log-probabilities with respect to ``hidden`` (all rows, summed over the
    vocabulary shards of the group) and to this rank's ``weight`` shard. The logits are
    recomputed tile by tile inside the GEMM kernel (``kEpiLogitsGrad`` epilogue of
    ``csrc/sm100/gemm.cu``), which writes ``d_logits = g * scale * (onehot - softmax)`` as bf16
    for a panel of rows; two GEMMs follow: ``d_hidden = d_logits @ W``, ``d_W = d_logits^T @ hidden``."""
    from . import gemm as _gemm

    k = hidden.shape[-1]
    h2 = hidden.reshape(-1, k).contiguous()
    m = h2.shape[0]
    v_global = int(vocab) if vocab is not None else int(weight.shape[0])
    world = 1 if group is None else group.world
    rank = 0 if group is None else group.rank
    lo, hi = vocab_shard_range(v_global, rank, world)
    v_local = hi - lo
    ids64 = ids.reshape(-1).to(torch.int64).contiguous()
    valid = (ids64 >= 0) & (ids64 < v_global)
    g32 = (g.reshape(-1).float() * valid).contiguous()
    lse32 = lse.reshape(-1).float().contiguous()
    w = weight.contiguous()
    if hidden.device.type != "cuda":
        # the same formula in PyTorch (d_logits rounded to bf16 like the kernel's output)
        logits = float(scale) * (h2.float() @ w.float().t())
        d_logits = -(g32 * float(scale))[:, None] * torch.exp(logits - lse32[:, None])
        mine = valid & (ids64 >= lo) & (ids64 < hi)
        rows = torch.nonzero(mine).flatten()
        d_logits[rows, ids64[rows] - lo] += g32[rows] * float(scale)
        d_logits = d_logits.to(torch.bfloat16).float()
        d_hidden = (d_logits @ w.float()).to(hidden.dtype) if need_dh else None
        d_weight = (d_logits.t() @ h2.float()).to(weight.dtype) if need_dw else None
        if d_hidden is not None and world > 1:
            from ..parallel.collectives import all_reduce_det

            all_reduce_det(d_hidden, getattr(group, "process_group", None))
        return d_hidden, d_weight
    m_real = m
    if m % 8:
        # the weight-gradient GEMM contracts over the rows, whose count must be a multiple of 8:
        # pad with rows whose upstream gradient is zero (their d_logits are exactly zero)
        pad = 8 - m % 8
        h2 = torch.cat([h2, h2.new_zeros(pad, k)])
        ids64 = torch.cat([ids64, ids64.new_full((pad,), -1)])
        g32 = torch.cat([g32, g32.new_zeros(pad)])
        lse32 = torch.cat([lse32, lse32.new_zeros(pad)])
        m += pad
    lib = _native.cuda()
    fn = lib.ka_lmhead_logits_grad
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                           ctypes.c_float, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                           ctypes.c_ulonglong, ctypes.c_void_p]
    props = torch.cuda.get_device_properties(h2.device)
    stream = torch.cuda.current_stream(h2.device).cuda_stream
    rows_per_panel = max(256, min(m, (_GRAD_PANEL_BYTES // max(1, v_local * 2)) // 256 * 256))
    d_hidden = torch.empty_like(h2) if need_dh else None
    d_weight = None
    multi = rows_per_panel < m
    for r0 in range(0, m, rows_per_panel):
        r1 = min(m, r0 + rows_per_panel)
        d_logits = torch.empty(r1 - r0, v_local, dtype=torch.bfloat16, device=h2.device)
        rc = fn(h2[r0:r1].data_ptr(), w.data_ptr(), ids64[r0:r1].data_ptr(), lse32[r0:r1].data_ptr(),
                g32[r0:r1].data_ptr(), d_logits.data_ptr(), v_local, r1 - r0, v_local, k, float(scale), lo,
                _gemm.status_buffer(h2.device).data_ptr(), props.multi_processor_count, default_timeout_ns(),
                stream)
        if rc != 0:
            raise RuntimeError(f"ka_lmhead_logits_grad rejected its arguments (code {rc})")
        if need_dh:
            d_hidden[r0:r1] = _gemm.gemm_bi(d_logits, w, trans_b=True)
        if need_dw:
            part = _gemm.gemm_bi(d_logits, h2[r0:r1], trans_a=True, trans_b=True,
                                 out_dtype=torch.float32 if multi else torch.bfloat16)
            d_weight = part if d_weight is None else d_weight.add_(part)
        del d_logits
    if need_dh and m_real != m:
        d_hidden = d_hidden[:m_real].contiguous()
    if need_dh and world > 1:
        from ..parallel.collectives import all_reduce_det

        all_reduce_det(d_hidden, getattr(group, "process_group", None))
    if need_dw and d_weight.dtype != weight.dtype:
        d_weight = d_weight.to(weight.dtype)
    return d_hidden, d_weight


class _LmheadLogpFn(torch.autograd.Function):
    """Differentiable fused log-prob; backward in :func:`_logp_backward`."""

    @staticmethod
    def forward(ctx, hidden, weight, ids, scale, vocab, group, panel_rows, cta_group):
        logp, lse = _lmhead_logp_forward(hidden, weight, ids, scale=scale, vocab=vocab, group=group,
                                         return_lse=True, panel_rows=panel_rows, cta_group=cta_group)
        ctx.save_for_backward(hidden, weight, ids, lse)
        ctx.scale, ctx.vocab, ctx.group = scale, vocab, group
        ctx.mark_non_differentiable(lse)
        return logp, lse

    @staticmethod
    def backward(ctx, g, _g_lse):
        hidden, weight, ids, lse = ctx.saved_tensors
        d_hidden, d_weight = _logp_backward(hidden, weight, ids, lse, g, ctx.scale, ctx.vocab, ctx.group,
                                            ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        return (d_hidden.reshape(hidden.shape) if d_hidden is not None else None), d_weight, None, None, None, None, \
            None, None


def _all_gather_flat(x: torch.Tensor, group) -> torch.Tensor:
    """Concatenation of every rank's ``x`` (same shape on all ranks) along dimension 0."""
    import torch.distributed as dist

    pg = getattr(group, "process_group", None)
    x = x.contiguous()
    if x.device.type == "cuda":
        out = torch.empty(group.world * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=pg)
        return out
    pieces = [torch.empty_like(x) for _ in range(group.world)]
    dist.all_gather(pieces, x, group=pg)
    return torch.cat(pieces)


class _LmheadLogpShardedFn(torch.autograd.Function):
    """Differentiable fused log-prob on row-sharded hidden states. Forward gathers the rows
    inside the kernel; backward needs every row on every rank (each rank owns a vocabulary
    shard of the weight), so it gathers rows, ids and log-sum-exps with a collective, runs
    :func:`_logp_backward` and keeps this rank's rows of ``d_hidden``. With ``gather_output``
    the incoming gradient already covers all rows and must be the same on every rank."""

    @staticmethod
    def forward(ctx, hidden, weight, ids, scale, vocab, group, cta_group, gather_output):
        logp, lse = _lmhead_logp_forward(hidden, weight, ids, scale=scale, vocab=vocab, group=group, return_lse=True,
                                         cta_group=cta_group, row_sharded=True, gather_output=gather_output)
        ctx.save_for_backward(hidden, weight, ids, lse)
        ctx.scale, ctx.vocab, ctx.group, ctx.gather_output = scale, vocab, group, gather_output
        ctx.mark_non_differentiable(lse)
        return logp, lse

    @staticmethod
    def backward(ctx, g, _g_lse):
        hidden, weight, ids, lse = ctx.saved_tensors
        group = ctx.group
        k = hidden.shape[-1]
        h2 = hidden.reshape(-1, k)
        m = h2.shape[0]
        h_all = _all_gather_flat(h2, group)
        ids_all = _all_gather_flat(ids.reshape(-1).to(torch.int64), group)
        if ctx.gather_output:
            lse_all, g_all = lse.reshape(-1), g.reshape(-1)
        else:
            lse_all = _all_gather_flat(lse.reshape(-1), group)
            g_all = _all_gather_flat(g.reshape(-1).float(), group)
        d_hidden, d_weight = _logp_backward(h_all, weight, ids_all, lse_all, g_all, ctx.scale, ctx.vocab, group,
                                            ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        if d_hidden is not None:
            d_hidden = d_hidden[group.rank * m:(group.rank + 1) * m].reshape(hidden.shape)
        return d_hidden, d_weight, None, None, None, None, None, None


@profiled("lmhead_logp")
def lmhead_logp(hidden: torch.Tensor, weight: torch.Tensor, ids: torch.Tensor, *, scale: float = 1.0,
                vocab: Optional[int] = None, group: Optional[VocabParallel] = None, return_lse: bool = False,
                panel_rows: int = DEFAULT_PANEL_ROWS, cta_group: Optional[int] = None,
                out: Optional[torch.Tensor] = None, check: bool = False, row_sharded: bool = False,
                gather_output: bool = False):
    """Per-token log-probabilities of ``ids`` under ``softmax(scale * hidden @ weight.T)``.

    hidden: ``[..., K]`` bf16; weight: ``[V_local, K]`` bf16 (this rank's vocabulary shard,
    whole canonical slices, see :func:`vocab_shard_range`); ids: ``[...]`` integer, global
    ids. Ids outside ``[0, vocab)`` give 0. Returns fp32 ``[...]`` (and the log-sum-exp if
    ``return_lse``). Differentiable with respect to ``hidden`` and ``weight`` (the log-sum-exp
    is returned detached). ``cta_group`` (1 or 2) picks the tile variant; by default the first
    large call of a shape times the schedules and keeps the fastest (same bits either way).

    ``row_sharded`` (with a vocabulary-parallel ``group``): ``hidden`` and ``ids`` are this
    rank's rows of a batch of ``world * rows`` (global row = ``rank * rows + local row``); the
    kernel gathers the other ranks' rows over NVLink while it works on its own. The result
    covers this rank's rows, or with ``gather_output`` the whole batch, flat ``[world * rows]``,
    on every rank.
    """
    needs_grad = torch.is_grad_enabled() and (hidden.requires_grad or weight.requires_grad)
    sharded = row_sharded and group is not None and group.world > 1
    if needs_grad:
        if out is not None:
            raise ValueError("out= cannot be combined with inputs that require gradients: the result written "
                             "there would be detached from the graph")
        if sharded:
            logp, lse = _LmheadLogpShardedFn.apply(hidden, weight, ids, float(scale), vocab, group, cta_group,
                                                   bool(gather_output))
        else:
            logp, lse = _LmheadLogpFn.apply(hidden, weight, ids, float(scale), vocab, group, panel_rows, cta_group)
        return (logp, lse) if return_lse else logp
    return _lmhead_logp_forward(hidden, weight, ids, scale=scale, vocab=vocab, group=group, return_lse=return_lse,
                                panel_rows=panel_rows, cta_group=cta_group, out=out, check=check,
                                row_sharded=sharded, gather_output=gather_output)


def sharded_token_logp(h_local: torch.Tensor, lm_head: torch.Tensor, targets: torch.Tensor, vocab: int, tp,
                       scale: float = 1.0) -> torch.Tensor:
    """Log-probabilities of ``targets`` (any shape, ``tokens`` entries, the same on every rank)
    from the sequence-sharded final hidden states of a tensor-parallel model: rank ``r`` holds
    rows ``[r * rows, (r + 1) * rows)`` of the flattened tokens (trailing rows are padding) and a
    vocabulary shard of the LM head. The rows are gathered inside the fused kernel; every rank
    gets the full result, shaped like ``targets``. Differentiable."""
    tokens = targets.numel()
    rows = h_local.shape[0]
    flat = targets.reshape(-1)
    lo, hi = min(tokens, tp.rank * rows), min(tokens, (tp.rank + 1) * rows)
    ids_local = flat[lo:hi]
    if hi - lo < rows:
        ids_local = torch.cat([ids_local, ids_local.new_full((rows - (hi - lo),), -100)])
    if h_local.device.type == "cuda":
        from ..parallel.peer import vocab_parallel_group

        vp = vocab_parallel_group(vocab, group=tp.group)
    else:
        vp = VocabParallel(rank=tp.rank, world=tp.world, process_group=tp.group)
    full = lmhead_logp(h_local, lm_head, ids_local, vocab=vocab, group=vp, scale=scale, row_sharded=True,
                       gather_output=True)
    return full[:tokens].view(targets.shape)
