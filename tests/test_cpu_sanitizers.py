"""Sanitizer tier (CPU): every operator of the C++ CPU library runs once, on shapes with
ragged tails, in a child process that loads an AddressSanitizer + UndefinedBehaviorSanitizer
build of the library. A heap overflow, a misaligned or out-of-range access or signed overflow
in the library ends that process with a report and fails the test. (GPU memory checkers are
not available to this project; the CPU library is the oracle the GPU kernels are compared
with, so its own correctness is checked with the host tools.)"""
import os
import subprocess
import sys

import pytest

from kernel_align_b200 import _build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys, torch
sys.path.insert(0, %(root)r)
from kernel_align_b200.ops import cpu_ops
g = torch.Generator().manual_seed(0)
# fused LM-head log-prob: vocabulary not a multiple of the canonical slices, odd row count
h = torch.randn(37, 72, generator=g)
w = torch.randn(1003, 72, generator=g) * 0.05
ids = torch.randint(-2, 1005, (37,), generator=g)
lp, lse = cpu_ops.lmhead_logp_cpu(h, w, ids, return_lse=True)
assert torch.isfinite(lp).all()
# the vocabulary-parallel form: two shards of whole canonical slices, then the tree merge
vs = -(-1003 // 8)
states, targets = [], []
for lo, hi in ((0, 4 * vs), (4 * vs, 1003)):
    st, tg = cpu_ops.lmhead_logp_shard_cpu(h, w[lo:hi], ids, vocab=1003, v_lo=lo)
    states.append(st); targets.append(tg)
merged = cpu_ops.lmhead_logp_merge_cpu(torch.cat(states, 1), targets[0] + targets[1], ids, vocab=1003)
assert torch.equal(merged, lp)
# log-prob from logits, three dtypes
for dt in (torch.float32, torch.bfloat16, torch.float16):
    lg = (torch.randn(19, 1003, generator=g) * 2).to(dt)
    out = cpu_ops.logits_logp_cpu(lg, torch.randint(0, 1003, (19,), generator=g))
    assert torch.isfinite(out).all()
# sampling: greedy, top-k, top-p, both, on a ragged vocabulary
lg = (torch.randn(11, 1003, generator=g) * 2).to(torch.bfloat16)
for kw in (dict(top_k=1, top_p=1.0), dict(top_k=50, top_p=1.0), dict(top_k=0, top_p=0.9), dict(top_k=50, top_p=0.9),
           dict(top_k=5000, top_p=1.0), dict(top_k=0, top_p=1.0)):
    tok = cpu_ops.sample_cpu(lg, inv_temperature=1 / 0.7, seed=3, step=1, **kw)
    assert ((tok >= 0) & (tok < 1003)).all()
# GEMM oracle and the sliced reduce-scatter emulation
a = torch.randn(9, 64, generator=g)
b = torch.randn(13, 64, generator=g)
assert cpu_ops.gemm_cpu(a, b).shape == (9, 13)
for world in (1, 2, 4, 8):
    assert cpu_ops.gemm_sliced_cpu(a, b, residual=torch.randn(9, 13, generator=g), world=world).shape == (9, 13)
print("CHILD_OK")
"""

CHILD_LAYERS = r"""
import sys, torch
sys.path.insert(0, %(root)r)
from kernel_align_b200.ops.layer_ops import rmsnorm, rope_, rope_tables, swiglu
from kernel_align_b200.ops.attention import attention
from kernel_align_b200.ops.grpo_loss import group_advantages, grpo_loss
g = torch.Generator().manual_seed(1)
x = torch.randn(7, 200, generator=g).to(torch.bfloat16)
y = rmsnorm(x, torch.ones(200, dtype=torch.bfloat16), 1e-5, x)
assert all(torch.isfinite(t.float()).all() for t in (y if isinstance(y, tuple) else (y,)))
assert torch.isfinite(rmsnorm(x, torch.ones(200, dtype=torch.bfloat16), 1e-5).float()).all()
cos, sin = rope_tables(64, 128)
q = torch.randn(10, 3, 128, generator=g).to(torch.bfloat16)
rope_(q, torch.arange(10), cos, sin)
assert torch.isfinite(swiglu(torch.randn(5, 2 * 37, generator=g).to(torch.bfloat16)).float()).all()
qq = torch.randn(2, 45, 4, 128, generator=g).to(torch.bfloat16)
kk = torch.randn(2, 45, 2, 128, generator=g).to(torch.bfloat16)
vv = torch.randn(2, 45, 2, 128, generator=g).to(torch.bfloat16)
for causal in (True, False):
    assert torch.isfinite(attention(qq, kk, vv, causal=causal).float()).all()
adv = group_advantages(torch.randn(12, generator=g), 4)
new, old = torch.randn(12, 9, generator=g) * 0.1 - 2, torch.randn(12, 9, generator=g) * 0.1 - 2
loss = grpo_loss(new, old, adv)
assert torch.isfinite(loss)
print("CHILD_OK")
"""


@pytest.mark.parametrize("script", [CHILD, CHILD_LAYERS], ids=["logp_sampling_gemm", "layers_attention_loss"])
def test_cpu_library_is_clean_under_asan_and_ubsan(script):
    lib = _build.build_cpu_sanitized()
    runtime = _build.sanitizer_runtime()
    if lib is None or runtime is None:
        pytest.skip("no C++ compiler with sanitizer runtimes on this host")
    env = dict(os.environ)
    env.update({"LD_PRELOAD": runtime, "KA_CPU_LIB": str(lib), "OMP_NUM_THREADS": "2",
                "ASAN_OPTIONS": "detect_leaks=0:abort_on_error=0:halt_on_error=1",
                "UBSAN_OPTIONS": "print_stacktrace=1:halt_on_error=1"})
    res = subprocess.run([sys.executable, "-c", script % {"root": ROOT}], env=env, capture_output=True, text=True,
                         timeout=600)
    tail = (res.stdout + res.stderr)[-3000:]
    assert res.returncode == 0 and "CHILD_OK" in res.stdout, tail
    assert "ERROR: AddressSanitizer" not in res.stderr and "runtime error:" not in res.stderr, tail
