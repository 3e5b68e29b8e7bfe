"""CPU multi-rank tier: gloo ranks on this host exercise the host-side logic of the
deterministic collectives and of failure detection (no GPU involved)."""
import os
import sys
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _init(rank, world, port, timeout_s=30):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))


def _allreduce_worker(rank, world, port, out_dir):
    _init(rank, world, port)
    from kernel_align_b200.parallel.collectives import all_reduce_det, tree_sum

    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(1000, generator=g) * (10.0 ** (rank - 1))
    mine = x.clone()
    all_reduce_det(mine)
    parts = [torch.randn(1000, generator=torch.Generator().manual_seed(100 + r)) * (10.0 ** (r - 1))
             for r in range(world)]
    want = tree_sum(parts)
    torch.save({"ok": bool(torch.equal(mine, want)), "val": mine}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_all_reduce_det_gloo_fixed_tree_order(tmp_path, world):
    port = 29700 + world
    mp.spawn(_allreduce_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    outs = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    assert all(o["ok"] for o in outs)
    for o in outs[1:]:
        assert torch.equal(o["val"], outs[0]["val"])  # every rank holds the same bits


def _failure_worker(rank, world, port, out_dir):
    _init(rank, world, port, timeout_s=20)
    from kernel_align_b200.parallel.collectives import all_reduce_det
    from kernel_align_b200.parallel.health import PeerLost, PeerMonitor

    mon = PeerMonitor(timeout_s=2.0)
    x = torch.ones(16)
    mon.check(0)
    all_reduce_det(x)  # step 0: everyone takes part
    leaver = world - 1
    if rank == leaver:
        # leave between steps, with nothing in flight; rank `leaver - 1` simply stops
        # answering instead (no announcement): both must be noticed
        mon.announce_leave()
        open(os.path.join(out_dir, f"r{rank}.left"), "w").close()
        time.sleep(6)  # keep the process (and its sockets) alive while the others look
        return
    t0 = time.time()
    try:
        mon.check(1)
        outcome = "completed"
    except PeerLost as e:
        outcome = f"PeerLost:{e.rank}"
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
        f.write(f"{outcome} {time.time() - t0:.1f}")
    time.sleep(1)


def test_missing_rank_is_detected_on_the_host(tmp_path):
    world = 4
    mp.spawn(_failure_worker, args=(world, 29720, str(tmp_path)), nprocs=world, join=True)
    assert (tmp_path / f"r{world - 1}.left").exists()
    for r in range(world - 1):
        outcome, secs = (tmp_path / f"r{r}.txt").read_text().split()
        assert outcome == f"PeerLost:{world - 1}", outcome
        assert float(secs) < 5


def _silent_worker(rank, world, port, out_dir):
    _init(rank, world, port, timeout_s=20)
    from kernel_align_b200.parallel.health import PeerLost, PeerMonitor

    mon = PeerMonitor(timeout_s=1.0)
    mon.check(0)
    if rank == 1:
        time.sleep(4)  # hangs on the host: never reaches step 1 in time, says nothing
        return
    t0 = time.time()
    try:
        mon.check(1)
        outcome = "completed"
    except PeerLost as e:
        outcome = f"PeerLost:{e.rank}"
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
        f.write(f"{outcome} {time.time() - t0:.1f}")
    time.sleep(4)


def test_silent_rank_times_out_on_the_host(tmp_path):
    mp.spawn(_silent_worker, args=(2, 29730, str(tmp_path)), nprocs=2, join=True)
    outcome, secs = (tmp_path / "r0.txt").read_text().split()
    assert outcome == "PeerLost:1" and 0.5 < float(secs) < 4


def test_tree_sum_order():
    from kernel_align_b200.parallel.collectives import tree_sum

    parts = [torch.tensor([1e8]), torch.tensor([1.0]), torch.tensor([-1e8]), torch.tensor([1.0])]
    # ((1e8 + 1) + (-1e8 + 1)) in fp32: 1e8 + 1 rounds to 1e8
    assert tree_sum(parts).item() == ((torch.tensor(1e8) + 1.0) + (torch.tensor(-1e8) + 1.0)).item()
    # a count that is not a power of two: the odd element moves up a level unchanged
    assert tree_sum(parts[:3]).item() == ((torch.tensor(1e8) + 1.0) + torch.tensor(-1e8)).item()
    with pytest.raises(ValueError):
        tree_sum([])


def _vp_worker(rank, world, port, out_dir):
    _init(rank, world, port)
    from kernel_align_b200.ops.fused_logp import VocabParallel, lmhead_logp, vocab_shard_range

    g = torch.Generator().manual_seed(11)
    m, k, v = 21, 72, 1003
    hidden = torch.randn(m, k, generator=g).to(torch.bfloat16)
    weight = (torch.randn(v, k, generator=g) * 0.1).to(torch.bfloat16)
    ids = torch.randint(-1, v + 1, (m,), generator=g)
    lo, hi = vocab_shard_range(v, rank, world)
    group = VocabParallel(rank=rank, world=world)
    logp, lse = lmhead_logp(hidden, weight[lo:hi], ids, vocab=v, group=group, scale=1.3, return_lse=True)
    # gradients: every rank gets the complete d_hidden (fixed-order sum over the shards)
    h = hidden.clone().requires_grad_()
    w = weight[lo:hi].clone().requires_grad_()
    lmhead_logp(h, w, ids, vocab=v, group=group, scale=1.3).sum().backward()
    torch.save({"logp": logp, "lse": lse, "dh": h.grad, "dw": w.grad, "lo": lo, "hi": hi},
               os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_vocab_parallel_logp_gloo_bitwise_equals_single_process(tmp_path, world):
    """The (max, sum-exp, target) merge across vocabulary shards, run by gloo ranks on the CPU
    library: every world size gives the bits of a single process."""
    from kernel_align_b200.ops.fused_logp import lmhead_logp

    mp.spawn(_vp_worker, args=(world, 29720 + world, str(tmp_path)), nprocs=world, join=True)
    g = torch.Generator().manual_seed(11)
    m, k, v = 21, 72, 1003
    hidden = torch.randn(m, k, generator=g).to(torch.bfloat16)
    weight = (torch.randn(v, k, generator=g) * 0.1).to(torch.bfloat16)
    ids = torch.randint(-1, v + 1, (m,), generator=g)
    logp, lse = lmhead_logp(hidden, weight, ids, scale=1.3, return_lse=True)
    h = hidden.clone().requires_grad_()
    w = weight.clone().requires_grad_()
    lmhead_logp(h, w, ids, scale=1.3).sum().backward()
    outs = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    for o in outs:
        assert torch.equal(o["logp"], logp) and torch.equal(o["lse"], lse)
        assert (o["dh"].float() - h.grad.float()).abs().max().item() <= 0.02 * h.grad.float().abs().max().item() + 1e-3
        assert torch.equal(o["dh"], outs[0]["dh"])            # identical on every rank
        assert (o["dw"].float() - w.grad[o["lo"]:o["hi"]].float()).abs().max().item() <= \
            0.02 * w.grad.float().abs().max().item() + 1e-3
    ref = torch.log_softmax(1.3 * hidden.float() @ weight.float().t(), -1)
    valid = (ids >= 0) & (ids < v)
    want = torch.where(valid, ref.gather(1, ids.clamp(0, v - 1)[:, None])[:, 0], torch.zeros(()))
    assert (logp - want).abs().max().item() < 1e-4


def _elastic_worker(rank, world, port, out_dir):
    _init(rank, world, port, timeout_s=30)
    from kernel_align_b200.parallel.collectives import all_reduce_det
    from kernel_align_b200.parallel.health import PeerLost, PeerMonitor, shrink_group

    mon = PeerMonitor(timeout_s=2.0)
    x = torch.full((8,), float(rank + 1))
    mon.check(0)
    all_reduce_det(x)                                  # step 0: all four ranks, sum = 10
    if rank == 3:
        mon.announce_leave()                           # leaves between steps, nothing in flight
        time.sleep(8)
        return
    try:
        mon.check(1)
        outcome = "no loss seen"
        group, ranks = None, list(range(world))
    except PeerLost as e:
        outcome = f"lost {e.rank}"
        group, ranks = shrink_group(mon, 1)
    y = torch.full((8,), float(rank + 1))
    all_reduce_det(y, group)                           # step 1 on the survivors: 1 + 2 + 3 = 6
    torch.save({"outcome": outcome, "ranks": ranks, "x": x, "y": y}, os.path.join(out_dir, f"r{rank}.pt"))
    time.sleep(1)


def test_job_shrinks_to_the_survivors_and_keeps_reducing(tmp_path):
    """Elastic recovery on the host: a rank leaves between steps, the others notice it, agree
    on the survivor list, form a group without it and keep running the fixed-order all-reduce
    (three ranks: the tree carries the odd element up)."""
    from kernel_align_b200.parallel.collectives import tree_sum

    mp.spawn(_elastic_worker, args=(4, 29731, str(tmp_path)), nprocs=4, join=True)
    outs = [torch.load(tmp_path / f"r{r}.pt") for r in range(3)]
    for o in outs:
        assert o["outcome"] == "lost 3" and o["ranks"] == [0, 1, 2]
        assert torch.equal(o["x"], torch.full((8,), 10.0)) and torch.equal(o["y"], torch.full((8,), 6.0))
    parts = [torch.tensor([0.1]), torch.tensor([0.2]), torch.tensor([0.3])]
    assert torch.equal(tree_sum(parts), (parts[0] + parts[1]) + parts[2])
    five = [torch.tensor([float(i)]) for i in range(5)]
    assert tree_sum(five).item() == 10.0
