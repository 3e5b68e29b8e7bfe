"""The per-operator profiler (ProfilingMode off / basic / detailed) on the CPU paths."""
import math
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kernel_align_b200.executors.trainer import GRPOTrainer
from kernel_align_b200.models.llama import LlamaConfig, LlamaModel
from kernel_align_b200.ops import gemm
from kernel_align_b200.platforms.constants import ProfilingMode
from kernel_align_b200.utils import profiler as prof

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_off_mode_records_nothing_and_hands_out_one_shared_context():
    prof.set_mode("off")
    prof.profiler.reset()
    assert prof.profile_range("x") is prof.profile_range("y")
    a = torch.randn(4, 64).to(torch.bfloat16)
    gemm.gemm_bi(a, a)
    assert prof.profiler.summary() == {}


def test_basic_mode_times_every_operator_of_a_grpo_step():
    prof.set_mode(ProfilingMode.BASIC)
    prof.profiler.reset()
    try:
        cfg = LlamaConfig(vocab_size=512, hidden=256, n_layers=1, n_heads=4, n_kv_heads=2, head_dim=128, ffn=512,
                          max_pos=256)
        trainer = GRPOTrainer(LlamaModel(cfg, seed=2, device=torch.device("cpu")),
                              lambda p, t: (t % 7 == 0).float().mean(1), group_size=2, max_new_tokens=3,
                              temperature=1.0, top_k=50, lr=1e-3, seed=3)
        prompts = torch.randint(0, cfg.vocab_size, (2, 8), generator=torch.Generator().manual_seed(9))
        trainer.train_step(prompts)
        s = prof.profiler.summary()
    finally:
        prof.set_mode("off")
    for name in ("grpo/rollout", "grpo/policy_forward", "grpo/backward_and_grad_reduce", "grpo/optimizer", "gemm_bi",
                 "attention", "attention_backward", "rmsnorm", "rope", "swiglu", "sample", "logits_logp", "lmhead_logp",
                 "grpo_loss", "attention_decode", "gemm_reduce_scatter"):
        assert name in s and s[name]["calls"] >= 1 and s[name]["total_ms"] >= 0.0, name
    assert s["grpo/rollout"]["total_ms"] >= s["sample"]["total_ms"]      # nested ranges
    assert all(math.isfinite(v["mean_ms"]) and v["max_ms"] <= v["total_ms"] + 1e-9 for v in s.values())
    table = prof.profiler.report()
    assert "operator" in table and "gemm_bi" in table
    prof.profiler.reset()


def _rank_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from kernel_align_b200.utils import profiler as p

    p.set_mode("detailed")      # NVTX is skipped on CPU tensors; the timing is the same as basic
    p.profiler._add("op", 10.0 * (rank + 1))
    p.profiler._add("other", 1.0)
    s = p.profiler.summary(across_ranks=True)
    torch.save(s, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_summary_across_ranks_takes_the_slowest_rank(tmp_path):
    mp.spawn(_rank_worker, args=(2, 29791, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        s = torch.load(tmp_path / f"r{r}.pt")
        assert s["op"]["total_ms"] == 20.0 and s["other"]["total_ms"] == 1.0
