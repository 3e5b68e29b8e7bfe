"""Child process of tests/test_gpu_multi.py: the peer-memory all-reduce equals the canonical
tree sum bit for bit, on every rank, for fp32 and bf16, and through GradReducer."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from kernel_align_b200.parallel.collectives import GradReducer, all_reduce_det, tree_sum  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", local)
    res = {}
    for dtype in (torch.float32, torch.bfloat16):
        for n in (1000, 3_000_001):
            g = torch.Generator(device=dev).manual_seed(7 + rank)
            x = (torch.randn(n, device=dev, generator=g) * (10.0 ** (rank % 3))).to(dtype)
            parts = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(parts, x)
            want = tree_sum(parts).to(dtype)
            for rep in range(2):
                y = x.clone()
                all_reduce_det(y)
                res[f"{dtype}_{n}_{rep}"] = bool(torch.equal(y, want))
    # gradient buckets with overlap
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.GELU(), torch.nn.Linear(512, 128)).to(dev)
    reducer = GradReducer(model.parameters(), bucket_bytes=256 << 10, average=True)
    data = torch.randn(64, 256, device=dev, generator=torch.Generator(device=dev).manual_seed(50 + rank))
    losses = []
    for it in range(2):
        reducer.zero_grad()
        loss = model(data).square().mean()
        loss.backward()
        reducer.finish()
        torch.cuda.synchronize()
        reducer.check()
        flat = torch.cat([p.grad.reshape(-1) for p in model.parameters()])
        losses.append(flat.clone())
    res["grad_repeatable"] = bool(torch.equal(losses[0], losses[1]))
    gathered = [torch.empty_like(losses[0]) for _ in range(world)]
    dist.all_gather(gathered, losses[0])
    res["grad_same_on_all_ranks"] = all(bool(torch.equal(gathered[0], t)) for t in gathered)
    # reference: local grads summed in tree order / world
    ref_model = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.GELU(), torch.nn.Linear(512, 128)).to(dev)
    ref_model.load_state_dict(model.state_dict())
    ref_model(data).square().mean().backward()
    local_flat = torch.cat([p.grad.reshape(-1) for p in ref_model.parameters()])
    parts = [torch.empty_like(local_flat) for _ in range(world)]
    dist.all_gather(parts, local_flat)
    res["grad_matches_tree"] = bool(torch.equal(tree_sum(parts) * (1.0 / world), losses[0]))
    flags = torch.tensor([int(all(res.values()))], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("RESULT " + json.dumps({"all_ranks_ok": bool(flags.item()), "world": world,
                                      **{str(k): v for k, v in res.items()}}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except Exception:  # make the failure visible in the parent's captured stdout
        import traceback

        print("WORKER_ERROR rank", os.environ.get("RANK"), traceback.format_exc()[-1500:], flush=True)
        raise
