"""Child process of tests/test_gpu_multi.py: the model-level parallel layouts on GPUs.

World 2: tensor-parallel ``token_logp`` (sequence-sharded layers, fused row-gathering LM head)
equals the single-GPU model bit for bit; tensor-parallel generation gives both ranks the same
tokens and log-probs that agree with the single-GPU model's view of them; a two-stage pipeline
reproduces the unsplit model's log-probs bit for bit; ZeRO-1 keeps the weights of the unsharded
optimizer bit for bit; a trainer whose peer is late beyond the device wait limit raises and
does not step, and works again after the arenas have been cleared.
World 4: DP x TP (2 x 2) ``policy_update``: the loss is bitwise the single-GPU one, repeatable
run to run, and both replicas hold identical shards afterwards.
"""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from kernel_align_b200.executors.generation import generate  # noqa: E402
from kernel_align_b200.executors.trainer import GRPOTrainer  # noqa: E402
from kernel_align_b200.kernels.sampling import SamplerBackend  # noqa: E402
from kernel_align_b200.models.llama import LlamaConfig, LlamaModel  # noqa: E402
from kernel_align_b200.ops.grpo_loss import grpo_loss  # noqa: E402
from kernel_align_b200.parallel.tp_gemm import TPContext  # noqa: E402


def solo_context(dev):
    solo = TPContext.__new__(TPContext)
    solo.group, solo.rank, solo.world, solo.device, solo._arenas = None, 0, 1, dev, {}
    return solo


def reward(prompts, new_tokens):
    return (new_tokens % 5 == 0).float().mean(1)


def world2(rank, dev, res):
    cfg = LlamaConfig.tiny(n_layers=2)
    solo = solo_context(dev)
    tp = TPContext()
    single = LlamaModel(cfg, tp=solo, seed=1, device=dev)
    sharded = LlamaModel(cfg, tp=tp, seed=1, device=dev)
    g = torch.Generator(device=dev).manual_seed(3)
    seqs = torch.randint(0, cfg.vocab_size, (4, 96), device=dev, generator=g)

    # ---- token_logp: TP = 2 (rows gathered inside the fused LM-head kernel) vs TP = 1
    with torch.no_grad():
        want = single.token_logp(seqs[:, :-1], seqs[:, 1:], scale=1.25)
        got = sharded.token_logp(seqs[:, :-1], seqs[:, 1:], scale=1.25)
    res["tp_token_logp_bitwise"] = bool(torch.equal(want, got))
    # and its gradients reach every parameter (values: to rounding, as for the layer test)
    loss = -sharded.token_logp(seqs[:, :-1], seqs[:, 1:]).mean()
    loss.backward()
    loss1 = -single.token_logp(seqs[:, :-1], seqs[:, 1:]).mean()
    loss1.backward()
    lo, hi = sharded.vocab_range
    gh, gh1 = sharded.lm_head.grad.float(), single.lm_head.grad.float()[lo:hi]
    res["tp_head_grad_close"] = bool((gh - gh1).abs().max().item() <= 0.03 * gh1.abs().max().item() + 1e-6)
    res["tp_loss_bitwise"] = bool(torch.equal(loss.detach(), loss1.detach()))
    sharded.zero_grad(set_to_none=True)
    single.zero_grad(set_to_none=True)

    # ---- generation with the sharded model
    prompts = seqs[:3, :16]
    out_tp = generate(sharded, prompts, sampler=SamplerBackend(seed=5), max_new_tokens=6, temperature=0.8, top_k=50,
                      top_p=0.95, group_size=2)
    out_1 = generate(single, prompts, sampler=SamplerBackend(seed=5), max_new_tokens=6, temperature=0.8, top_k=50,
                     top_p=0.95, group_size=2)
    both = [torch.empty_like(out_tp["sequences"]) for _ in range(2)]
    dist.all_gather(both, out_tp["sequences"].contiguous())
    res["tp_generation_same_on_both_ranks"] = bool(torch.equal(both[0], both[1]))
    seq = out_tp["sequences"]
    with torch.no_grad():
        lp = single.token_logp(seq[:, :-1], seq[:, 1:], scale=1 / 0.8)[:, 15:]
    res["tp_generation_logp_err"] = (lp - out_tp["logp"]).abs().max().item()
    res["tp_generation_token_match_vs_tp1"] = (out_tp["new_tokens"] == out_1["new_tokens"]).float().mean().item()

    # ---- two-stage pipeline vs the unsplit model
    from kernel_align_b200.ops.fused_logp import lmhead_logp
    from kernel_align_b200.parallel.pipeline import PipelineStage, pipeline_logp_step

    cfg4 = LlamaConfig.tiny(n_layers=4)
    stage = PipelineStage(cfg4, rank, 2, seed=1, device=dev)
    ids = torch.randint(0, cfg4.vocab_size, (4, 64), device=dev, generator=g)
    n_tok = ids.numel()
    logp, _ = pipeline_logp_step(stage, ids, ids, n_micro=2, loss_fn=lambda lp_, m: -lp_.sum() / n_tok)
    whole = LlamaModel(cfg4, tp=solo, seed=1, device=dev)
    with torch.no_grad():
        h = whole.hidden_states(ids)
        ref = lmhead_logp(h[:n_tok], whole.lm_head, ids.reshape(-1)).view(4, 64)
    ok = torch.tensor([1 if (logp is None or torch.equal(logp, ref)) else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    res["pipeline_logp_bitwise"] = bool(ok.item())
    del stage, whole

    # ---- ZeRO-1 vs the unsharded optimizer, data parallel over the two ranks
    prompts_dp = torch.randint(0, cfg.vocab_size, (2, 16), device=dev,
                               generator=torch.Generator(device=dev).manual_seed(20 + rank))
    weights = {}
    for stage_id in (0, 1):
        model = LlamaModel(cfg, tp=solo, seed=4, device=dev)
        trainer = GRPOTrainer(model, reward, group_size=2, max_new_tokens=4, lr=1e-3, seed=3, top_k=50,
                              data_parallel=True, zero_stage=stage_id, weight_decay=0.01)
        losses = [trainer.train_step(prompts_dp)["loss"].item() for _ in range(2)]
        weights[stage_id] = (losses, model.lm_head.detach().clone(), model.layers[0].wqkv.detach().clone())
        trainer.reducer.close()
    res["zero1_weights_bitwise"] = weights[0][0] == weights[1][0] and bool(torch.equal(weights[0][1], weights[1][1])) \
        and bool(torch.equal(weights[0][2], weights[1][2]))

    # ---- a late peer: the device wait runs out, the trainer raises and does not step
    from kernel_align_b200.parallel import collectives

    model = LlamaModel(cfg, tp=solo, seed=6, device=dev)
    trainer = GRPOTrainer(model, reward, group_size=2, max_new_tokens=4, lr=1e-3, seed=3, top_k=50, data_parallel=True)
    roll = trainer.rollout(prompts_dp)
    before = model.lm_head.detach().clone()
    os.environ["RL_ENGINE_TIMEOUT_MS"] = "200"
    real_logp = trainer.policy_logp

    def late_logp(*a, **k):      # after the host rendezvous, before this rank's first gradient bucket
        if rank == 1:
            time.sleep(1.5)
        return real_logp(*a, **k)

    trainer.policy_logp = late_logp
    raised = False
    try:
        trainer.policy_update(roll["sequences"], roll["logp"], roll["advantages"], 16)
    except collectives.CollectiveTimeout:
        raised = True
    torch.cuda.synchronize()
    res["late_peer_raises"] = raised
    res["late_peer_no_step"] = bool(torch.equal(before, model.lm_head.detach()))
    os.environ["RL_ENGINE_TIMEOUT_MS"] = "2000"
    trainer.policy_logp = real_logp
    collectives.reset_after_timeout()
    loss, _ = trainer.policy_update(roll["sequences"], roll["logp"], roll["advantages"], 16)
    heads = [torch.empty_like(model.lm_head) for _ in range(2)]
    dist.all_gather(heads, model.lm_head.detach().contiguous())
    res["recovers_after_reset"] = bool(torch.isfinite(loss)) and bool(torch.equal(heads[0], heads[1])) and \
        not bool(torch.equal(before, heads[0]))


def world4(rank, dev, res):
    cfg = LlamaConfig.tiny(n_layers=2)
    tp_groups = [dist.new_group([0, 1]), dist.new_group([2, 3])]
    dp_groups = [dist.new_group([0, 2]), dist.new_group([1, 3])]
    replica, shard = rank // 2, rank % 2
    tp = TPContext(group=tp_groups[replica])
    g = torch.Generator(device=dev).manual_seed(40 + replica)      # each replica has its own rollouts
    seqs = torch.randint(0, cfg.vocab_size, (4, 48), device=dev, generator=g)
    logp_old = -torch.rand(4, 16, device=dev, generator=g) - 5.0
    adv = torch.randn(4, device=dev, generator=g)
    losses, shards = [], []
    for _ in range(2):
        model = LlamaModel(cfg, tp=tp, seed=1, device=dev)
        trainer = GRPOTrainer(model, reward, group_size=2, max_new_tokens=16, lr=1e-3, seed=3, data_parallel=True,
                              dp_group=dp_groups[shard])
        loss, _ = trainer.policy_update(seqs, logp_old, adv, prompt_len=32)
        losses.append(loss.detach().clone())
        shards.append((model.layers[0].wqkv.detach().clone(), model.lm_head.detach().clone()))
        trainer.reducer.close()
    res["hybrid_loss_repeatable"] = bool(torch.equal(losses[0], losses[1]))
    res["hybrid_weights_repeatable"] = all(bool(torch.equal(a, b)) for a, b in zip(shards[0], shards[1]))
    # the loss of a replica is the single-GPU loss on the same rollouts, bit for bit
    single = LlamaModel(cfg, tp=solo_context(dev), seed=1, device=dev)
    with torch.no_grad():
        lp = single.token_logp(seqs[:, :-1], seqs[:, 1:])[:, 31:]
        want = grpo_loss(lp, logp_old, adv)
    res["hybrid_loss_equals_single_gpu"] = bool(torch.equal(want, losses[0]))
    # after the update the two replicas hold the same shard
    mine = shards[1][0].contiguous()
    allw = [torch.empty_like(mine) for _ in range(4)]
    dist.all_gather(allw, mine)
    res["hybrid_replicas_equal"] = bool(torch.equal(allw[0], allw[2])) and bool(torch.equal(allw[1], allw[3])) and \
        not bool(torch.equal(allw[0], allw[1]))


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", local)
    res = {}
    if world == 2:
        world2(rank, dev, res)
    elif world == 4:
        world4(rank, dev, res)
    torch.cuda.synchronize()
    bools = [v for v in res.values() if isinstance(v, bool)]
    ok = all(bools) and res.get("tp_generation_logp_err", 0.0) < 0.1
    flags = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    gathered = [None] * world
    dist.all_gather_object(gathered, res)
    if rank == 0:
        print("RESULT " + json.dumps({"all_ranks_ok": bool(flags.item()), "world": world, "per_rank": gathered}),
              flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except Exception:  # make the failure visible in the parent's captured stdout
        import traceback

        print("WORKER_ERROR rank", os.environ.get("RANK"), traceback.format_exc()[-2500:], flush=True)
        raise
