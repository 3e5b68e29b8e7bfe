#!/usr/bin/env python
"""Headline benchmark: GRPO per-token log-probability throughput at Llama-3-8B shapes.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)
    python bench.py --impl reference ...                     (the unmodified reference)

One step = log-probabilities of G*L target tokens given hidden states [G*L, 4096] (bf16)
and the LM-head weight [128256, 4096] (bf16), G=256, L=512, synthetic N(0,1) / N(0,0.02)
data. Own arm: the fused tcgen05 LM-head+logprob kernel. On N > 1 GPUs the headline is the
layout of the reference arm: every rank holds the whole LM head and receives G*L/N rows, no
communication inside the step. The vocabulary-parallel layout is timed as well and reported
under ``other_layout``: vocabulary and rows sharded over the ranks, the kernel pushes the rows to
the peers over NVLink while it computes, exchanges the partial (max, sum-exp, target) triples
the same way, and every rank ends with the results of its own rows (what a model with a
tensor-parallel LM head needs; ``--layout vocab`` makes it the headline). Reference arm:
`torch.matmul` (cuBLAS) feeding the reference's `SamplerBackend.compute_logp` from
baseline/_ref, rows split over the ranks (the reference has no distributed code, so data
parallelism over rows is the only way to use it unmodified on N GPUs).

Both arms stage their inputs the same way in the end-to-end loop and report, as a second
record, the latency of one sampling call (bf16 logits [G, 128256] ~ N(0, 2), temperature 0.7,
top-k 50, top-p 0.9, G = 64 / 128 / 256) through their own ``SamplerBackend.sample``.

Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
VOCAB = 128256
HIDDEN = 4096
BASELINE_TOKENS_PER_S = None  # the reference publishes no tokens/s figure


class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float = 0.0, t1: float = float("inf")) -> dict:
        """Summary of the samples taken between wall-clock times ``t0`` and ``t1`` (the timed
        region). The sampler is started before the warm-up, because nvidia-smi needs a few
        hundred milliseconds to produce its first line; if the timed region is shorter than the
        sampling period, the samples closest to it are used and ``window`` says so."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [l for t, l in self.lines if t0 <= t <= t1 + 0.05]
        window = "timed region"
        if not inside and self.lines:
            nearest = sorted(self.lines, key=lambda tl: min(abs(tl[0] - t0), abs(tl[0] - t1)))[:3]
            inside = [l for _, l in nearest]
            window = "nearest samples (timed region shorter than the sampling period)"
        for line in inside:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons), "window": window}


def init_dist(n_gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local),
                                timeout=datetime.timedelta(minutes=30))
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {n_gpus}")
    return rank, world, local


def barrier_sync(world: int):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class Deadline:
    """Ends the process with status 0 after ``seconds`` unless cancelled, rank 0 first printing
    ``make_line()``: the headline of a run must not be lost to a further, optional measurement
    that does not come back (ranks that fell out of step wait in a collective for minutes)."""

    def __init__(self, seconds: float, rank: int, make_line):
        self.rank, self.make_line = rank, make_line
        self.timer = threading.Timer(seconds, self._fire)
        self.timer.daemon = True

    def start(self):
        self.timer.start()
        return self

    def cancel(self):
        self.timer.cancel()

    def _fire(self):
        if self.rank == 0:
            print(json.dumps(self.make_line()), flush=True)
        os._exit(0)


def make_inputs(rows: int, v_rows: int, seed: int):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    hidden = torch.randn(rows, HIDDEN, device="cuda", generator=gen, dtype=torch.float32).to(torch.bfloat16)
    weight = torch.empty(v_rows, HIDDEN, device="cuda", dtype=torch.bfloat16)
    for i in range(0, v_rows, 16384):  # bounded fp32 temporary
        n = min(16384, v_rows - i)
        weight[i:i + n] = (torch.randn(n, HIDDEN, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
    ids = torch.randint(0, VOCAB, (rows,), device="cuda", generator=gen)
    return hidden, weight, ids


def settle(first_call, args):
    """Set-up work outside the measurements, the same for both arms: one call of the step
    (library initialisation, schedule timing, allocator growth), then an idle pause. Each of
    the two timed loops (device, end to end) then starts from the same state, W warm-up calls
    after a pause, instead of the second one inheriting the heat of the first: on these
    power-capped GPUs a loop that follows seconds of load ran up to 14 % slower."""
    if first_call is not None:
        first_call()
    torch.cuda.synchronize()
    time.sleep(args.cooldown)


def time_device(step, args, world, local):
    """W warm-up calls, then K calls between two CUDA events; max over ranks, with the clocks
    sampled while the timed calls run."""
    clocks = ClockSampler(local)
    clocks.start()
    for _ in range(args.warmup):
        step()
    barrier_sync(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier_sync(world)
    t0 = time.time()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier_sync(world)
    t1 = time.time()
    ms = max_over_ranks(e0.elapsed_time(e1), world) / args.steps
    return ms, clocks.stop(t0, t1)


def time_end_to_end(step, h_host, ids_host, out_host, args, world):
    """The same staging for both arms: every step copies its inputs from pinned host memory to
    one of two device buffers on a copy stream (so the copy of step i+1 overlaps the compute of
    step i), runs ``step(hidden, ids)`` and copies the result to pinned host memory."""
    copy_stream = torch.cuda.Stream()
    bufs = [(torch.empty(h_host.shape, dtype=h_host.dtype, device="cuda"),
             torch.empty(ids_host.shape, dtype=ids_host.dtype, device="cuda")) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    done = [torch.cuda.Event() for _ in range(2)]

    def stage(i):
        b = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(done[b])  # the compute that last used this buffer
            bufs[b][0].copy_(h_host, non_blocking=True)
            bufs[b][1].copy_(ids_host, non_blocking=True)
            ready[b].record(copy_stream)

    def run(n):
        stage(0)
        for i in range(n):
            b = i % 2
            if i + 1 < n:
                stage(i + 1)
            torch.cuda.current_stream().wait_event(ready[b])
            res = step(bufs[b][0], bufs[b][1])
            done[b].record()
            out_host.copy_(res.reshape(out_host.shape), non_blocking=True)
        torch.cuda.synchronize()

    for b in range(2):
        done[b].record()
    run(max(1, min(2, args.warmup)))
    barrier_sync(world)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    run(args.steps)
    t1.record()
    barrier_sync(world)
    return max_over_ranks(t0.elapsed_time(t1), world) / args.steps


SAMPLING_CONFIG = {"vocab": VOCAB, "dtype": "bf16", "logits": "N(0, 2)", "temperature": 0.7, "top_k": 50, "top_p": 0.9,
                   "timing": "CUDA events around each call, L2 flushed between calls, median of 30 after 5 warm-ups"}


def time_sampling(sample, calls: int = 30) -> dict:
    """Latency of one fused sampling call at G = 64 / 128 / 256 (microseconds, median)."""
    out = {}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(99)
    for g in (64, 128, 256):
        logits = (torch.randn(g, VOCAB, device="cuda", generator=gen) * 2.0).to(torch.bfloat16)
        for _ in range(5):
            sample(logits)
        times = []
        for _ in range(calls):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            sample(logits)
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3)
        out[f"g{g}_us"] = statistics.median(times)
        del logits
    return out


def all_ranks_ok(ok: bool, world: int) -> bool:
    """True when ``ok`` holds on every rank (so that all ranks take the same branch)."""
    if world == 1:
        return ok
    t = torch.tensor([0 if ok else 1], dtype=torch.int32, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return int(t.item()) == 0


def measure_own_layout(layout, args, rank, world, local, sampler, fused_logp):
    """Device-timed and end-to-end step of one layout of the own arm.

    ``rows``   every rank holds the whole LM head and takes G*L/N rows: no communication, the
               layout of the reference arm.
    ``vocab``  vocabulary and rows sharded; the kernel gathers the rows over NVLink and exchanges
               the partial (max, sum-exp, target) triples, every rank ends with its own rows.
    """
    rows = args.g * args.seq_len
    rows_local = rows // world
    extra = fused_logp.workspace_bytes(VOCAB)
    kw = dict(vocab=VOCAB)
    if layout == "vocab":
        from kernel_align_b200 import _native
        from kernel_align_b200.parallel.peer import gather_arena_bytes, vocab_parallel_group

        lo, hi = fused_logp.vocab_shard_range(VOCAB, rank, world)
        group = vocab_parallel_group(VOCAB)
        kw.update(group=group, row_sharded=True)
        extra += int(_native.cuda().ka_lmhead_logp_exchange_bytes(world, group.panel_rows))
        extra += gather_arena_bytes(group, HIDDEN)
        n_panels = -(-rows // fused_logp.DEFAULT_PANEL_ROWS)
        name = f"vp{world} (vocabulary sharded, rows sharded and gathered in-kernel)"
    else:
        lo, hi = 0, VOCAB
        n_panels = -(-rows_local // fused_logp.DEFAULT_PANEL_ROWS)
        name = f"dp{world} (rows split, full vocabulary per rank)" if world > 1 else "single"
    hidden, weight, ids = make_inputs(rows, hi - lo, seed=1234)
    hidden = hidden[rank * rows_local:(rank + 1) * rows_local].clone()
    ids = ids[rank * rows_local:(rank + 1) * rows_local].clone()

    settle(lambda: sampler.fused_logp(hidden, weight, ids, **kw), args)   # the first call times the schedules
    ms, clock_info = time_device(lambda: sampler.fused_logp(hidden, weight, ids, **kw), args, world, local)
    status = fused_logp.last_status(hidden.device, VOCAB)
    if not all_ranks_ok(int(status[0]) == 0, world):
        fused_logp.check_status(status)
        raise RuntimeError("a peer rank reported a device-side timeout")

    # ---- end to end through the public API: pinned host inputs in, log-probs out, per step
    h_host = hidden.cpu().pin_memory()
    ids_host = ids.cpu().pin_memory()
    out_host = torch.empty(rows_local, dtype=torch.float32).pin_memory()
    settle(None, args)
    e2e_ms = time_end_to_end(lambda h, i: sampler.fused_logp(h, weight, i, **kw), h_host, ids_host, out_host, args,
                             world)
    status = fused_logp.last_status(hidden.device, VOCAB)
    if not all_ranks_ok(int(status[0]) == 0, world):
        fused_logp.check_status(status)
        raise RuntimeError("a peer rank reported a device-side timeout")
    return {"parallelism": name, "ms_per_step": ms, "clocks": clock_info, "e2e_ms_per_step": e2e_ms,
            "h2d_bytes_per_step": (h_host.numel() * 2 + ids_host.numel() * 8) * world,
            "d2h_bytes_per_step": out_host.numel() * 4 * world, "extra_vram_bytes": extra,
            "gpu_launches": args.steps * n_panels}


def run_own(args, rank, world, local):
    sys.path.insert(0, ROOT)
    from kernel_align_b200.kernels.sampling import SamplerBackend
    from kernel_align_b200.ops import fused_logp

    rows = args.g * args.seq_len
    if rows % world:
        raise SystemExit("G * L must be divisible by the number of GPUs")
    sampler = SamplerBackend()
    sampling = None
    if rank == 0:
        sampling = time_sampling(lambda x: sampler.sample(x, top_k=50, top_p=0.9, temperature=0.7))
    if world == 1:
        layouts = ["rows"]
    elif args.layout == "auto":
        layouts = ["rows", "vocab"]   # the first one is the headline, the second a further record
    else:
        layouts = [args.layout]
    head = measure_own_layout(layouts[0], args, rank, world, local, sampler, fused_logp)
    ms, e2e_ms = head["ms_per_step"], head["e2e_ms_per_step"]
    value = rows / ms * 1e3
    line = {
        "metric": "grpo_logp_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": (value / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"model": "Llama-3-8B LM head (V=128256, d=4096)", "global_batch": args.g, "seq_len": args.seq_len,
                   "parallelism": head["parallelism"],
                   "l2": "inputs (hidden rows + LM head) larger than the 126 MB L2",
                   "idle_s_before_each_timed_loop": args.cooldown,
                   "extra_vram_bytes": head["extra_vram_bytes"]},
        "clocks": head["clocks"],
        "e2e": {"value": rows / e2e_ms * 1e3, "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": head["h2d_bytes_per_step"], "d2h_bytes_per_step": head["d2h_bytes_per_step"],
                "staging": "double-buffered H2D on a copy stream, total bytes over all ranks"},
        "sampling": sampling, "sampling_config": SAMPLING_CONFIG,
        "gpu_launches": head["gpu_launches"],
        "impl": "own",
    }
    for layout in layouts[1:]:
        # the headline is measured; the further record must not be able to lose it
        late = {"parallelism": layout, "unavailable": f"did not finish within {args.other_timeout:.0f} s"}
        deadline = Deadline(args.other_timeout, rank, lambda: {**line, "other_layout": late}).start()
        torch.cuda.empty_cache()
        try:
            r = measure_own_layout(layout, args, rank, world, local, sampler, fused_logp)
            other = {"parallelism": r["parallelism"], "ms_per_step": r["ms_per_step"],
                     "tokens_per_s": rows / r["ms_per_step"] * 1e3, "e2e_ms_per_step": r["e2e_ms_per_step"],
                     "e2e_tokens_per_s": rows / r["e2e_ms_per_step"] * 1e3, "extra_vram_bytes": r["extra_vram_bytes"],
                     "clocks": r["clocks"]}
        except Exception as e:  # noqa: BLE001  (all ranks leave together: see all_ranks_ok)
            other = {"parallelism": layout, "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
        deadline.cancel()
        line["other_layout"] = other
    return line


def run_reference(args, rank, world, local):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "rl_engine")):
        return {"impl": "reference", "unavailable": "baseline/_ref is missing: the reference is not installed"}
    sys.path.insert(0, ref_dir)
    try:
        from rl_engine.kernels.sampling import SamplerBackend as RefSampler
    except Exception as e:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"import of the reference failed: {type(e).__name__}: {e}"}

    rows = args.g * args.seq_len
    g_local = args.g // world
    rows_local = g_local * args.seq_len
    sampler = RefSampler().to("cuda")
    sampling = None
    if rank == 0:
        # the stock call as shipped (its fp32 copy and its second temperature division included);
        # FlashInfer compiles its kernels during the warm-up calls, outside the timed ones
        try:
            sampling = time_sampling(lambda x: sampler.sample(x, top_k=50, top_p=0.9, temperature=0.7))
        except Exception as e:  # noqa: BLE001
            sampling = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
    hidden, weight, ids = make_inputs(rows, VOCAB, seed=1234)
    hidden = hidden[rank * rows_local:(rank + 1) * rows_local].clone()
    ids = ids[rank * rows_local:(rank + 1) * rows_local].view(g_local, args.seq_len).clone()

    def step(h, i):
        logits = torch.matmul(h, weight.t()).view(g_local, args.seq_len, VOCAB)
        return sampler.compute_logp(logits, i)

    settle(lambda: step(hidden, ids), args)
    ms, clock_info = time_device(lambda: step(hidden, ids), args, world, local)
    peak = torch.cuda.max_memory_allocated()

    h_host = hidden.cpu().pin_memory()
    ids_host = ids.cpu().pin_memory()
    out_host = torch.empty(g_local, args.seq_len, dtype=hidden.dtype).pin_memory()
    settle(None, args)
    e2e_ms = time_end_to_end(step, h_host, ids_host, out_host, args, world)
    value = rows / ms * 1e3
    return {
        "metric": "grpo_logp_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": "Llama-3-8B LM head (V=128256, d=4096)", "global_batch": args.g, "seq_len": args.seq_len,
                   "parallelism": f"dp{world} (rows split, full vocabulary per rank)" if world > 1 else "single",
                   "l2": "inputs and logits larger than the 126 MB L2",
                   "idle_s_before_each_timed_loop": args.cooldown,
                   "path": "torch.matmul (cuBLAS) -> rl_engine SamplerBackend.compute_logp",
                   "peak_allocated_bytes": peak},
        "clocks": clock_info,
        "e2e": {"value": rows / e2e_ms * 1e3, "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": (h_host.numel() * 2 + ids_host.numel() * 8) * world,
                "d2h_bytes_per_step": out_host.numel() * out_host.element_size() * world,
                "staging": "double-buffered H2D on a copy stream, total bytes over all ranks"},
        "sampling": sampling, "sampling_config": SAMPLING_CONFIG,
        "gpu_launches": 0,
        "impl": "reference",
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["own", "reference"], default="own")
    ap.add_argument("--g", type=int, default=256, help="group size G (rows = G * seq_len)")
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--cooldown", type=float, default=4.0,
                    help="idle seconds before each timed loop (after set-up, and between the device and the "
                         "end-to-end loop), both arms")
    ap.add_argument("--other-timeout", type=float, default=150.0,
                    help="seconds the further layout record of the own arm may take before the run ends with "
                         "the headline alone")
    ap.add_argument("--layout", choices=["auto", "rows", "vocab"], default="auto",
                    help="own arm on N > 1 GPUs: rows split (full LM head per rank), vocabulary-parallel with "
                         "the in-kernel row gather, or (auto) the first as the headline and the second as a "
                         "further record")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if not torch.cuda.is_available():
        line = {"impl": args.impl, "unavailable": "no CUDA device visible"}
        print(json.dumps(line))
        return
    rank, world, local = init_dist(args.gpus)
    try:
        line = run_own(args, rank, world, local) if args.impl == "own" else run_reference(args, rank, world, local)
    finally:
        pass
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        # the line is out: a rank that cannot leave the group in a minute ends anyway, with status 0
        guard = Deadline(60.0, -1, dict).start()
        try:
            dist.barrier()
            dist.destroy_process_group()
        except Exception as e:  # noqa: BLE001
            print(f"bench.py: leaving the process group failed: {type(e).__name__}: {e}", file=sys.stderr)
        guard.cancel()


if __name__ == "__main__":
    main()
