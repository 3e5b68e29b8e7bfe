"""torch.library registration of the operators: results equal the Python entry points, and the
fake implementations give the right shapes and dtypes (checked with torch.library.opcheck)."""
import torch

import kernel_align_b200.ops.library  # noqa: F401  (registers torch.ops.kernel_align_b200.*)
from kernel_align_b200.ops import gemm, layer_ops
from kernel_align_b200.ops.attention import attention
from kernel_align_b200.ops.fused_logp import lmhead_logp
from kernel_align_b200.ops.logits_logp import logits_logp
from kernel_align_b200.ops.sampling import sample

OPS = torch.ops.kernel_align_b200


def _inputs():
    g = torch.Generator().manual_seed(0)
    hidden = torch.randn(12, 64, generator=g).to(torch.bfloat16)
    weight = (torch.randn(200, 64, generator=g) * 0.1).to(torch.bfloat16)
    ids = torch.randint(0, 200, (12,), generator=g)
    logits = (torch.randn(12, 200, generator=g) * 2).to(torch.bfloat16)
    q = torch.randn(1, 20, 4, 128, generator=g).to(torch.bfloat16)
    kv = torch.randn(1, 20, 2, 128, generator=g).to(torch.bfloat16)
    return hidden, weight, ids, logits, q, kv


def test_registered_ops_equal_the_python_entry_points():
    hidden, weight, ids, logits, q, kv = _inputs()
    assert torch.equal(OPS.lmhead_logp(hidden, weight, ids, 1.25), lmhead_logp(hidden, weight, ids, scale=1.25))
    assert torch.equal(OPS.logits_logp(logits, ids, 1.0), logits_logp(logits, ids))
    assert torch.equal(OPS.sample(logits, 50, 0.9, 0.7, 3, 1),
                       sample(logits, top_k=50, top_p=0.9, temperature=0.7, seed=3, step=1))
    assert torch.equal(OPS.sample(logits, 0, 1.0, 1.0, 3, 1), sample(logits, seed=3, step=1))
    assert torch.equal(OPS.gemm_bi(hidden, weight, False, False), gemm.gemm_bi(hidden, weight))
    assert torch.equal(OPS.attention(q, kv, kv, True, -1.0), attention(q, kv, kv, causal=True))
    assert torch.equal(OPS.rmsnorm(hidden, torch.ones(64, dtype=torch.bfloat16), 1e-5),
                       layer_ops.rmsnorm(hidden, torch.ones(64, dtype=torch.bfloat16), 1e-5))
    assert torch.equal(OPS.swiglu(hidden), layer_ops.swiglu(hidden))


def test_fake_implementations_match_real_shapes_and_dtypes():
    hidden, weight, ids, logits, q, kv = _inputs()
    checks = ("test_schema", "test_faketensor")
    torch.library.opcheck(OPS.lmhead_logp.default, (hidden, weight, ids, 1.0), test_utils=checks)
    torch.library.opcheck(OPS.logits_logp.default, (logits, ids, 1.0), test_utils=checks)
    torch.library.opcheck(OPS.sample.default, (logits, 50, 0.9, 0.7, 3, 1), test_utils=checks)
    torch.library.opcheck(OPS.gemm_bi.default, (hidden, weight, False, False), test_utils=checks)
    torch.library.opcheck(OPS.attention.default, (q, kv, kv, True, -1.0), test_utils=checks)
    torch.library.opcheck(OPS.rmsnorm.default, (hidden, torch.ones(64, dtype=torch.bfloat16), 1e-5), test_utils=checks)
    torch.library.opcheck(OPS.swiglu.default, (hidden,), test_utils=checks)
