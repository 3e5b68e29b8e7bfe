"""Multi-GPU tier: child processes under torchrun, one rank per GPU (skipped with < 2 GPUs)."""
import json
import os
import signal
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run_worker(script, nproc, timeout=300, extra_env=None):
    env = dict(os.environ)
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(29500 + nproc), os.path.join(HERE, "workers", script)]
    # a session of its own, so that a launcher that runs out of time is ended together with its ranks
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env,
                            start_new_session=True)
    try:
        stdout, _ = proc.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)
        stdout, _ = proc.communicate()
        raise AssertionError(f"worker {script} ran out of time ({timeout} s): " + stdout[-1500:]) from None
    lines = [l for l in stdout.splitlines() if l.startswith("RESULT ")]
    if proc.returncode != 0 or not lines:
        i = stdout.find("WORKER_ERROR")
        raise AssertionError("worker failed: " + (stdout[i:i + 2500] if i >= 0 else stdout[-1500:]))
    return json.loads(lines[-1][len("RESULT "):])


def _world_sizes():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return [w for w in (2, 4, 8) if w <= n]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_vocab_parallel_logp_bitwise_equals_single_gpu(world):
    if world not in _world_sizes():
        pytest.skip(f"needs {world} GPUs")
    res = _run_worker("vp_logp_worker.py", world)
    assert res["all_ranks_ok"], res
    assert res["small_err"] < 2e-3 and res["llama_err"] < 2e-3


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_gemm_fused_collectives_bitwise_equal_single_gpu(world):
    if world not in _world_sizes():
        pytest.skip(f"needs {world} GPUs")
    res = _run_worker("tp_gemm_worker.py", world)
    assert res["all_ranks_ok"], res
    assert res["rs_small_err"] < 0.02 and res["rs_llama_err"] < 0.02


@pytest.mark.parametrize("world", [2, 4, 8])
def test_deterministic_all_reduce_and_grad_buckets(world):
    if world not in _world_sizes():
        pytest.skip(f"needs {world} GPUs")
    res = _run_worker("allreduce_worker.py", world)
    assert res["all_ranks_ok"], res


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_decoder_layer_bitwise_equals_single_gpu(world):
    if world not in _world_sizes():
        pytest.skip(f"needs {world} GPUs")
    res = _run_worker("tp_layer_worker.py", world)
    assert res["all_ranks_ok"], res


@pytest.mark.parametrize("world", [2, 4])
def test_model_parallel_layouts_on_gpus(world):
    """Tensor-parallel token_logp / generation, pipeline, ZeRO-1 and the late-peer path on two
    GPUs; DP x TP policy update on four (tests/workers/model_parallel_worker.py)."""
    if world not in _world_sizes():
        pytest.skip(f"needs {world} GPUs")
    # no in-switch reduction anywhere in these runs: one of them makes a rank late on purpose
    res = _run_worker("model_parallel_worker.py", world, timeout=420, extra_env={"NCCL_NVLS_ENABLE": "0"})
    assert res["all_ranks_ok"], res
