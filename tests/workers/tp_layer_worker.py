"""Child process of tests/test_gpu_multi.py: a tensor-parallel decoder layer gives, on every
rank, exactly the rows (and the weight-gradient shards) of the single-GPU layer."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from kernel_align_b200.models.llama import DecoderLayer, LlamaConfig  # noqa: E402
from kernel_align_b200.ops import gemm  # noqa: E402
from kernel_align_b200.ops.layer_ops import rope_tables  # noqa: E402
from kernel_align_b200.parallel.tp_gemm import TPContext, rows_per_rank  # noqa: E402


def solo_context(dev):
    solo = TPContext.__new__(TPContext)
    solo.group, solo.rank, solo.world, solo.device, solo._arenas = None, 0, 1, dev, {}
    return solo


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", local)
    tp, solo = TPContext(), solo_context(dev)
    res = {}
    tiny = LlamaConfig(vocab_size=2048, hidden=1024, n_layers=2, n_heads=16, n_kv_heads=8, head_dim=128, ffn=4096,
                       max_pos=1024)
    cases = {"tiny": (tiny, [(1, 256), (8, 256)]), "llama8b": (LlamaConfig.llama3_8b(), [(1, 512), (8, 512), (64, 512)])}
    for name, (cfg, shapes) in cases.items():
        layer_tp = DecoderLayer(cfg, tp, seed=5, device=dev)
        layer_1 = DecoderLayer(cfg, solo, seed=5, device=dev)
        cos, sin = rope_tables(cfg.max_pos, cfg.head_dim, cfg.rope_theta, device=dev)
        first_seq = None      # the single-GPU output rows of sequence 0 at the first batch size
        g = torch.Generator(device=dev).manual_seed(11)
        max_tokens = max(b * l for b, l in shapes)
        x_all = torch.randn(max_tokens, cfg.hidden, device=dev, generator=g).to(torch.bfloat16)
        dy_all = torch.randn(max_tokens, cfg.hidden, device=dev, generator=g).to(torch.bfloat16)
        for batch, seq_len in shapes:
            tokens = batch * seq_len
            x, dy = x_all[:tokens].clone(), dy_all[:tokens].clone()     # every batch starts with the same rows
            pos = torch.arange(seq_len, device=dev).repeat(batch)
            # TP = 1
            x1 = x.clone().requires_grad_()
            rpr1 = rows_per_rank(tokens, 1)
            xin = torch.cat([x1, x1.new_zeros(rpr1 - tokens, cfg.hidden)]) if rpr1 != tokens else x1
            y1 = layer_1(xin, batch, seq_len, pos, cos, sin)[:tokens]
            layer_1.zero_grad(set_to_none=True)
            y1.backward(dy)
            # TP = world
            rpr = rows_per_rank(tokens, world)
            lo, hi = min(tokens, rank * rpr), min(tokens, (rank + 1) * rpr)
            xl = torch.zeros(rpr, cfg.hidden, device=dev, dtype=torch.bfloat16)
            xl[: hi - lo] = x[lo:hi]
            xl.requires_grad_()
            yl = layer_tp(xl, batch, seq_len, pos, cos, sin)
            dyl = torch.zeros(rpr, cfg.hidden, device=dev, dtype=torch.bfloat16)
            dyl[: hi - lo] = dy[lo:hi]
            layer_tp.zero_grad(set_to_none=True)
            yl.backward(dyl)
            key = f"{name}_b{batch}"
            res[key + "_fwd"] = bool(torch.equal(yl[: hi - lo], y1.detach()[lo:hi]))
            # per-row equality across batch sizes: sequence 0 is the same input in every batch and
            # must give the same output rows
            # (with the line above: for every tensor-parallel degree as well)
            if first_seq is None:
                first_seq = y1.detach()[:seq_len].clone()
            else:
                res[key + "_rows_equal_across_batch"] = bool(torch.equal(y1.detach()[:seq_len], first_seq))

            def close(a, b):
                if a.numel() == 0:
                    return True
                return bool((a.float() - b.float()).abs().max().item() <= 0.03 * b.float().abs().max().item() + 1e-6)

            # gradients: same mathematics; the contraction over the fused qkv / gate-up features is
            # grouped per rank, so the input gradient agrees to rounding, not bit for bit
            res[key + "_dx"] = close(xl.grad[: hi - lo], x1.grad[lo:hi])
            f = cfg.ffn // world
            res[key + "_dwdown"] = close(layer_tp.wdown.grad, layer_1.wdown.grad[:, rank * f:(rank + 1) * f])
            hq = cfg.n_heads // world * cfg.head_dim
            res[key + "_dwqkv_q"] = close(layer_tp.wqkv.grad[:hq], layer_1.wqkv.grad[rank * hq:(rank + 1) * hq])
        del layer_tp, layer_1
        torch.cuda.empty_cache()
    torch.cuda.synchronize()
    gemm.check_status(dev)
    flags = torch.tensor([int(all(res.values()))], device=dev)
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
