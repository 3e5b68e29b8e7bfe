"""GPU tier: the fused sampler returns exactly the tokens of the CPU definition."""
import pytest
import torch

from kernel_align_b200.kernels.sampling import SamplerBackend
from kernel_align_b200.ops import cpu_ops
from kernel_align_b200.ops.sampling import sample

pytestmark = pytest.mark.gpu


def _cpu(logits, top_k, top_p, temperature, seed, step, row_ids=None):
    return cpu_ops.sample_cpu(logits.cpu(), inv_temperature=1.0 / temperature, top_k=top_k or 0,
                              top_p=1.0 if top_p is None else top_p, seed=seed, step=step, row_ids=row_ids)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("top_k,top_p", [(50, 0.9), (1, None), (1024, 0.95), (7, None), (None, 0.9), (None, None),
                                         (3000, 0.8)])
def test_sampler_equals_cpu_definition(cuda_device, dtype, top_k, top_p):
    g = torch.Generator(device=cuda_device).manual_seed(0)
    logits = (torch.randn(24, 8000, device=cuda_device, generator=g) * 2).to(dtype)
    for step in (0, 1):
        tok = sample(logits, top_k=top_k, top_p=top_p, temperature=0.7, seed=9, step=step)
        ref = _cpu(logits, top_k, top_p, 0.7, 9, step)
        assert tok.dtype == torch.int32
        assert torch.equal(tok.cpu(), ref), (top_k, top_p, step)


def test_sampler_llama_vocab_headline_config(cuda_device):
    g = torch.Generator(device=cuda_device).manual_seed(1)
    logits = (torch.randn(256, 128256, device=cuda_device, generator=g) * 2).to(torch.bfloat16)
    tok = sample(logits, top_k=50, top_p=0.9, temperature=0.7, seed=1, step=3)
    assert torch.equal(tok[:32].cpu(), _cpu(logits[:32], 50, 0.9, 0.7, 1, 3))
    # batch invariance: rows 64..128 sampled alone, named by their row ids
    part = sample(logits[64:128], top_k=50, top_p=0.9, temperature=0.7, seed=1, step=3,
                  row_ids=torch.arange(64, 128))
    assert torch.equal(part, tok[64:128])
    assert torch.equal(tok, sample(logits, top_k=50, top_p=0.9, temperature=0.7, seed=1, step=3))


@pytest.mark.parametrize("cluster", ["1", "2", "4"])
def test_sampler_cluster_variants_equal_cpu_definition(cuda_device, cluster, monkeypatch):
    """Few rows of 16-bit logits are sampled by a cluster of CTAs per row; every variant must
    return the tokens of the CPU definition: a vocabulary with a scalar tail, heavy ties that
    overflow the candidate list, k from 1 to 1024."""
    monkeypatch.setenv("KA_SAMPLE_CLUSTER", cluster)
    g = torch.Generator(device=cuda_device).manual_seed(7)
    wide = (torch.randn(12, 50016, device=cuda_device, generator=g) * 2).to(torch.bfloat16)[:, :50011]
    for top_k, top_p in ((50, 0.9), (1, None), (1024, 0.95)):
        tok = sample(wide, top_k=top_k, top_p=top_p, temperature=0.7, seed=3, step=2)
        assert torch.equal(tok.cpu(), _cpu(wide, top_k, top_p, 0.7, 3, 2)), (cluster, top_k, top_p)
    ties = torch.zeros(4, 20000, device=cuda_device, dtype=torch.float16)
    ties[2, 19999] = 1.0
    tok = sample(ties, top_k=50, top_p=0.5, seed=2, step=0)
    assert torch.equal(tok.cpu(), _cpu(ties, 50, 0.5, 1.0, 2, 0))
    llama = (torch.randn(64, 128256, device=cuda_device, generator=g) * 2).to(torch.bfloat16)
    tok = sample(llama, top_k=50, top_p=0.9, temperature=0.7, seed=1, step=5)
    assert torch.equal(tok[:16].cpu(), _cpu(llama[:16], 50, 0.9, 0.7, 1, 5))
    monkeypatch.setenv("KA_SAMPLE_CLUSTER", "1")
    assert torch.equal(tok, sample(llama, top_k=50, top_p=0.9, temperature=0.7, seed=1, step=5))


def test_sampler_heavy_ties(cuda_device):
    # constant rows overflow the candidate list: the exact-select path cuts ties by token id
    logits = torch.zeros(4, 20000, device=cuda_device, dtype=torch.bfloat16)
    logits[1, 777] = 1.0
    for top_k, top_p in ((50, None), (50, 0.5), (None, 0.001), (5000, None)):
        tok = sample(logits, top_k=top_k, top_p=top_p, seed=2, step=0)
        assert torch.equal(tok.cpu(), _cpu(logits, top_k, top_p, 1.0, 2, 0)), (top_k, top_p)
    # quantised logits: many exact duplicates around the k-th value
    g = torch.Generator(device=cuda_device).manual_seed(3)
    q = (torch.randn(8, 50000, device=cuda_device, generator=g) * 4).round().to(torch.bfloat16)
    for top_k, top_p in ((50, 0.9), (1000, None), (None, 0.7)):
        tok = sample(q, top_k=top_k, top_p=top_p, seed=4, step=1)
        assert torch.equal(tok.cpu(), _cpu(q, top_k, top_p, 1.0, 4, 1)), (top_k, top_p)


def test_sampler_backend_module(cuda_device):
    s = SamplerBackend(seed=5)
    g = torch.Generator(device=cuda_device).manual_seed(6)
    logits = (torch.randn(8, 4096, device=cuda_device, generator=g)).to(torch.bfloat16)
    a = s.sample(logits, top_k=20, top_p=0.9, temperature=0.8)
    b = s.sample(logits, top_k=20, top_p=0.9, temperature=0.8)
    assert s.step == 2 and a.shape == (8,)
    s.set_rng_state({"seed": 5, "step": 0})
    assert torch.equal(s.sample(logits, top_k=20, top_p=0.9, temperature=0.8), a)
    assert torch.equal(s.sample(logits, top_k=20, top_p=0.9, temperature=0.8), b)
    assert torch.equal(s.sample(logits, top_k=1).long(), logits.float().argmax(-1))


def test_sampler_bf16_without_top_k_threshold_among_negative_values_and_nan(cuda_device):
    """bf16 rows without a (small) top-k search their threshold in a per-key count histogram,
    non-negative keys first; rows whose threshold lies among negative values, rows with NaN / inf
    entries and a Llama-sized vocabulary must give the CPU library's token."""
    g = torch.Generator(device=cuda_device).manual_seed(11)
    neg = (-torch.randn(6, 128256, device=cuda_device, generator=g).abs() * 2 - 1).to(torch.bfloat16)
    mixed = (torch.randn(6, 128256, device=cuda_device, generator=g) * 2).to(torch.bfloat16)
    odd = mixed.clone()
    odd[0, 5] = float("nan")
    odd[1, 77] = float("-inf")
    odd[2, :100] = float("nan")
    odd[3, 9] = 0.0
    odd[3, 10] = -0.0
    for name, logits in (("neg", neg), ("mixed", mixed), ("odd", odd)):
        for top_k, top_p, temp in ((None, 0.9, 0.7), (None, 0.999, 1.0), (None, 0.3, 1.5), (5000, 0.95, 0.7),
                                   (100000, None, 1.0), (None, None, 1.0)):
            tok = sample(logits, top_k=top_k, top_p=top_p, temperature=temp, seed=21, step=4)
            assert torch.equal(tok.cpu(), _cpu(logits, top_k, top_p, temp, 21, 4)), (name, top_k, top_p, temp)
