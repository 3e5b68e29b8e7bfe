"""CPU tier: the C++ library against PyTorch, and its batch-invariance contract."""
import torch

from kernel_align_b200.kernels.sampling import SamplerBackend
from kernel_align_b200.ops import cpu_ops
from kernel_align_b200.ops.fused_logp import lmhead_logp, vocab_shard_range
from kernel_align_b200.ops.sampling import sample


def _config1():
    g = torch.Generator().manual_seed(0)
    hidden = torch.randn(4, 64, 256, generator=g)
    weight = torch.randn(1024, 256, generator=g) * 0.02
    ids = torch.randint(0, 1024, (4, 64), generator=g)
    return hidden, weight, ids


def test_fused_logp_matches_log_softmax_gather():
    hidden, weight, ids = _config1()
    out = cpu_ops.lmhead_logp_cpu(hidden.reshape(-1, 256), weight, ids.reshape(-1), chunk_rows=16).reshape(4, 64)
    ref = torch.log_softmax(hidden @ weight.T, -1).gather(-1, ids[..., None]).squeeze(-1)
    assert out.shape == (4, 64)
    assert (out - ref).abs().max().item() < 1e-5


def test_fused_logp_bitwise_batch_invariant():
    hidden, weight, ids = _config1()
    full = lmhead_logp(hidden, weight, ids)  # public entry point, CPU tensors
    for b in range(4):
        one = lmhead_logp(hidden[b:b + 1], weight, ids[b:b + 1])
        assert torch.equal(one[0], full[b])
    # chunk size and thread split never enter the arithmetic
    a = cpu_ops.lmhead_logp_cpu(hidden.reshape(-1, 256), weight, ids.reshape(-1), chunk_rows=16)
    b_ = cpu_ops.lmhead_logp_cpu(hidden.reshape(-1, 256), weight, ids.reshape(-1), chunk_rows=7)
    assert torch.equal(a, b_)


def test_fused_logp_scale_lse_and_ignored_ids():
    hidden, weight, ids = _config1()
    ids = ids.clone()
    ids[0, 0] = -100
    lp, lse = cpu_ops.lmhead_logp_cpu(hidden.reshape(-1, 256), weight, ids.reshape(-1), scale=1 / 0.7, return_lse=True)
    logits = (hidden @ weight.T).reshape(-1, 1024) / 0.7
    assert (lse - torch.logsumexp(logits, -1)).abs().max().item() < 1e-5
    assert lp[0].item() == 0.0


def test_logits_logp_2d_and_3d():
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(3, 5, 777, generator=g) * 3
    ids = torch.randint(0, 777, (3, 5), generator=g)
    s = SamplerBackend()
    out3 = s.compute_logp(logits, ids)
    ref = torch.log_softmax(logits, -1).gather(-1, ids[..., None]).squeeze(-1)
    assert out3.shape == (3, 5) and (out3 - ref).abs().max().item() < 1e-5
    out2 = s.compute_logp(logits.reshape(15, 777), ids.reshape(15))
    assert torch.equal(out2, out3.reshape(15))
    out_t = s.compute_logp(logits, ids, temperature=0.5)
    ref_t = torch.log_softmax(logits / 0.5, -1).gather(-1, ids[..., None]).squeeze(-1)
    assert (out_t - ref_t).abs().max().item() < 1e-5


def test_vocab_shard_range_covers_vocab():
    for v in (1024, 128256, 151936, 7):
        for world in (1, 2, 4, 8):
            spans = [vocab_shard_range(v, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == v
            for a, b in zip(spans, spans[1:]):
                assert a[1] == b[0]


def _kept_set(row, top_k, top_p, temperature):
    """Reference definition in plain PyTorch: the set of tokens the sampler may return."""
    y = row.float() / temperature
    order = sorted(range(len(y)), key=lambda i: (-y[i].item(), i))
    if top_k:
        order = order[:top_k]
    p = torch.softmax(y[order].double(), 0)
    keep, cum = [], 0.0
    for j, i in enumerate(order):
        if j > 0 and cum > top_p:
            break
        keep.append(i)
        cum += p[j].item()
    return set(keep)


def test_sampling_support_and_greedy():
    g = torch.Generator().manual_seed(2)
    logits = torch.randn(6, 3000, generator=g) * 2
    greedy = sample(logits, top_k=1)
    assert torch.equal(greedy.long(), logits.argmax(-1))
    assert torch.equal(sample(logits, temperature=0.0).long(), logits.argmax(-1))
    for top_k, top_p in ((50, 0.9), (None, 0.8), (2000, 0.95), (5, None)):
        allowed = [_kept_set(logits[r], top_k, 1.0 if top_p is None else top_p, 0.7) for r in range(6)]
        for step in range(20):
            tok = sample(logits, top_k=top_k, top_p=top_p, temperature=0.7, seed=3, step=step)
            for r in range(6):
                assert tok[r].item() in allowed[r], (top_k, top_p, step, r)


def test_sampling_batch_invariant_and_seeded():
    g = torch.Generator().manual_seed(3)
    logits = (torch.randn(16, 2048, generator=g) * 2).to(torch.bfloat16)
    full = sample(logits, top_k=50, top_p=0.9, temperature=0.7, seed=11, step=5)
    again = sample(logits, top_k=50, top_p=0.9, temperature=0.7, seed=11, step=5)
    assert torch.equal(full, again)
    part = sample(logits[4:9], top_k=50, top_p=0.9, temperature=0.7, seed=11, step=5,
                  row_ids=torch.arange(4, 9))
    assert torch.equal(part, full[4:9])
    other = sample(logits, top_k=50, top_p=0.9, temperature=0.7, seed=12, step=5)
    assert not torch.equal(full, other)


def test_sampling_distribution_matches_softmax():
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, -50.0]])
    counts = torch.zeros(5)
    n = 4000
    for step in range(n):
        counts[sample(logits, temperature=1.0, seed=5, step=step)[0]] += 1
    p = torch.softmax(logits[0], 0)
    assert (counts / n - p).abs().max().item() < 0.03
    # top-k 2 renormalises over the two best tokens
    counts = torch.zeros(5)
    for step in range(n):
        counts[sample(logits, top_k=2, temperature=1.0, seed=5, step=step)[0]] += 1
    p2 = torch.softmax(logits[0, :2], 0)
    assert counts[2:].sum() == 0 and (counts[:2] / n - p2).abs().max().item() < 0.03


def test_sampling_ties_prefer_low_ids():
    logits = torch.zeros(2, 500)
    tok = sample(logits, top_k=3, seed=1, step=0)
    assert all(t in (0, 1, 2) for t in tok.tolist())
    tok = sample(logits, top_k=None, top_p=0.01, seed=1, step=0)  # 1% of 500 equal tokens: ids 0..5
    assert all(t <= 5 for t in tok.tolist())


def test_cpu_gemm_and_rank_emulator():
    g = torch.Generator().manual_seed(7)
    a = torch.randn(37, 256, generator=g).bfloat16()
    b = (torch.randn(50, 256, generator=g) * 0.1).bfloat16()
    r = torch.randn(37, 50, generator=g).bfloat16()
    ref = a.float() @ b.float().t()
    assert (cpu_ops.gemm_cpu(a, b) - ref).abs().max().item() < 1e-4
    assert torch.equal(cpu_ops.gemm_cpu(a[5:6], b), cpu_ops.gemm_cpu(a, b)[5:6])
    outs = [cpu_ops.gemm_sliced_cpu(a, b, residual=r, world=w) for w in (1, 2, 4, 8)]
    for o in outs[1:]:
        assert torch.equal(o, outs[0])  # the emulated rank count never enters the arithmetic
    want = (ref.bfloat16().float() + r.float()).bfloat16().float()
    assert (outs[0] - want).abs().max().item() <= 0.05 * want.abs().max().item()


def test_results_do_not_depend_on_the_thread_count(monkeypatch):
    import torch

    from kernel_align_b200.ops import cpu_ops

    g = torch.Generator().manual_seed(4)
    h, w = torch.randn(37, 96, generator=g), torch.randn(700, 96, generator=g) * 0.1
    ids = torch.randint(0, 700, (37,), generator=g)
    logits = torch.randn(23, 900, generator=g) * 2
    outs = []
    for n in ("1", "3", "8"):
        monkeypatch.setenv("KA_CPU_THREADS", n)
        outs.append((cpu_ops.lmhead_logp_cpu(h, w, ids), cpu_ops.logits_logp_cpu(logits, ids[:23] % 900),
                     cpu_ops.sample_cpu(logits, inv_temperature=1.2, top_k=40, top_p=0.9, seed=5, step=2),
                     cpu_ops.gemm_cpu(h, w)))
    for o in outs[1:]:
        assert all(torch.equal(a, b) for a, b in zip(o, outs[0]))
