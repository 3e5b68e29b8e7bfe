"""Child process of tests/test_gpu_multi.py: vocabulary-parallel fused log-prob on N GPUs must
equal the single-GPU result bit for bit on every rank."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from kernel_align_b200.ops import fused_logp  # noqa: E402
from kernel_align_b200.parallel.peer import vocab_parallel_group  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", local)
    results = {}
    for name, (m, k, v, panel) in {"small": (700, 512, 20011, 512), "llama": (3000, 4096, 128256, 32768)}.items():
        g = torch.Generator(device=dev).manual_seed(5)
        h = torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16)
        w = (torch.randn(v, k, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        ids = torch.randint(0, v, (m,), device=dev, generator=g)
        ids[0] = -100
        single, single_lse = fused_logp.lmhead_logp(h, w, ids, return_lse=True, panel_rows=panel, check=True)
        lo, hi = fused_logp.vocab_shard_range(v, rank, world)
        vp = vocab_parallel_group(v, panel_rows=panel)
        shard = w[lo:hi].contiguous()
        for rep in range(3):  # repeated launches reuse the exchange buffers (alternating halves)
            out, lse = fused_logp.lmhead_logp(h, shard, ids, vocab=v, group=vp, return_lse=True, check=True)
            ok = bool(torch.equal(out, single)) and bool(torch.equal(lse, single_lse))
            results[f"{name}_{rep}"] = ok
        ref = torch.log_softmax(h.float() @ w.float().T, -1).gather(-1, ids.clamp(min=0)[:, None]).squeeze(-1)
        ref[0] = 0
        results[f"{name}_err"] = (out - ref).abs().max().item()
    # ---- rows sharded over the ranks: the kernel gathers them over NVLink while it computes.
    # Several panels with a ragged last one (small), one panel (llama); both output modes; the
    # results must equal the single-GPU ones bit for bit on every rank.
    for name, (m_local, k, v, panel) in {"small": (700, 512, 20011, 2048), "llama": (3000 // world, 4096, 128256, 32768),
                                         "tiny": (5, 256, 1000, 2048)}.items():
        g = torch.Generator(device=dev).manual_seed(11)
        m = m_local * world
        h = torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16)
        w = (torch.randn(v, k, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        ids = torch.randint(0, v, (m,), device=dev, generator=g)
        ids[1] = -100
        single, single_lse = fused_logp.lmhead_logp(h, w, ids, return_lse=True, panel_rows=panel, check=True)
        lo, hi = fused_logp.vocab_shard_range(v, rank, world)
        vp = vocab_parallel_group(v, panel_rows=panel)
        shard = w[lo:hi].contiguous()
        mine = slice(rank * m_local, (rank + 1) * m_local)
        h_loc, ids_loc = h[mine].contiguous(), ids[mine].contiguous()
        for rep in range(3):
            out, lse = fused_logp.lmhead_logp(h_loc, shard, ids_loc, vocab=v, group=vp, return_lse=True, check=True,
                                              row_sharded=True)
            results[f"sharded_{name}_{rep}"] = bool(torch.equal(out, single[mine])) and \
                bool(torch.equal(lse, single_lse[mine]))
            full, full_lse = fused_logp.lmhead_logp(h_loc, shard, ids_loc, vocab=v, group=vp, return_lse=True,
                                                    check=True, row_sharded=True, gather_output=True)
            results[f"sharded_all_{name}_{rep}"] = bool(torch.equal(full, single)) and \
                bool(torch.equal(full_lse, single_lse))
    flags = torch.tensor([int(all(v for k, v in results.items() if not k.endswith("_err")))], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("RESULT " + json.dumps({"all_ranks_ok": bool(flags.item()), "world": world, **results}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except Exception:  # make the failure visible in the parent's captured stdout
        import traceback

        print("WORKER_ERROR rank", os.environ.get("RANK"), traceback.format_exc()[-1500:], flush=True)
        raise
