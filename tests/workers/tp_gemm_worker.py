"""Child process of tests/test_gpu_multi.py: fused GEMM->reduce-scatter and all-gather->GEMM on
N GPUs equal the single-GPU run of the same kernels bit for bit, and fp32 PyTorch closely."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from kernel_align_b200.ops import gemm  # noqa: E402
from kernel_align_b200.parallel.tp_gemm import TPContext, all_gather_gemm, gemm_reduce_scatter  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", local)
    ctx = TPContext()
    solo = TPContext.__new__(TPContext)
    solo.group, solo.rank, solo.world, solo.device, solo._arenas = None, 0, 1, dev, {}
    res = {}
    g = torch.Generator(device=dev).manual_seed(3)
    for name, (m, n, k) in {"rs_small": (1024, 512, 1024), "rs_llama": (4096, 4096, 14336)}.items():
        x = torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16)
        w = (torch.randn(n, k, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        r = torch.randn(m, n, device=dev, generator=g).to(torch.bfloat16)
        full = gemm_reduce_scatter(x, w, solo, residual=r)          # TP=1 through the same kernel
        ks = k // world
        rpr = m // world
        for rep in range(3):
            part = gemm_reduce_scatter(x[:, rank * ks:(rank + 1) * ks], w[:, rank * ks:(rank + 1) * ks], ctx,
                                       residual=r[rank * rpr:(rank + 1) * rpr])
            res[f"{name}_{rep}"] = bool(torch.equal(part, full[rank * rpr:(rank + 1) * rpr]))
        ref = (x.float() @ w.float().t()).bfloat16().float() + r.float()
        res[f"{name}_err"] = (full.float() - ref).abs().max().item() / ref.abs().max().item()
    for name, (m, n, k) in {"ag_small": (1024, 1024, 512), "ag_llama": (4096, 6144, 4096)}.items():
        x = torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16)
        w = (torch.randn(n, k, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        full = gemm.gemm_bi(x, w)
        nl, rpr = n // world, m // world
        for rep in range(3):
            part = all_gather_gemm(x[rank * rpr:(rank + 1) * rpr], w[rank * nl:(rank + 1) * nl], ctx)
            res[f"{name}_{rep}"] = bool(torch.equal(part, full[:, rank * nl:(rank + 1) * nl]))
    torch.cuda.synchronize()
    gemm.check_status(dev)
    flags = torch.tensor([int(all(v for k_, v in res.items() if not k_.endswith("_err")))], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("RESULT " + json.dumps({"all_ranks_ok": bool(flags.item()), "world": world, **res}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except Exception:  # make the failure visible in the parent's captured stdout
        import traceback

        print("WORKER_ERROR rank", os.environ.get("RANK"), traceback.format_exc()[-1500:], flush=True)
        raise
