"""Infrastructure: logger, device context, registry, executor (the reference's
rl_engine/tests/test_dispatch.py, with assertions)."""
import logging

import pytest

from kernel_align_b200.executors.rollout import RolloutExecutor
from kernel_align_b200.kernels.registry import OpBackend, kernel_registry
from kernel_align_b200.platforms.constants import constants
from kernel_align_b200.platforms.device import device_ctx
from kernel_align_b200.utils.logger import LINE_FORMAT, init_logger, logger


class _Capture(logging.Handler):
    def __init__(self):
        super().__init__()
        self.records = []

    def emit(self, record):
        self.records.append(record.getMessage())


def test_logger_once_and_rank(monkeypatch):
    cap = _Capture()
    logger.addHandler(cap)
    try:
        logger.reset_once_cache()
        for _ in range(3):
            logger.info_once("unique message %s", "x")
        for _ in range(2):
            logger.warn_once("careful")
        assert cap.records.count("unique message x") == 1
        assert cap.records.count("careful") == 1
        monkeypatch.setenv("RANK", "1")
        logger.info_on_rank("only on zero", 0)
        logger.info_on_rank("only on one", 1)
        assert "only on zero" not in cap.records and "only on one" in cap.records
    finally:
        logger.removeHandler(cap)
    assert init_logger("RL-Engine") is logger
    assert LINE_FORMAT == "%(levelname)s %(asctime)s [%(name)s]: %(message)s"
    assert logger.propagate is False


def test_constants_surface():
    names = ["DeviceType", "BackendLib", "PrecisionType", "SamplingMethod", "MemoryFormat", "OperatorFusionLevel",
             "KernelOptimizationLevel", "LoggingLevel", "ProfilingMode", "DistributedStrategy", "CheckpointFormat",
             "ActivationFunction"]
    for n in names:
        assert hasattr(constants, n)
    assert constants.DeviceType.CUDA.value == "cuda"
    assert constants.BackendLib.NATIVE.value == "native"
    assert constants.DistributedStrategy.HYBRID.value == "hybrid"
    assert constants.ActivationFunction.SILU.value == "silu"


def test_device_and_registry():
    assert device_ctx.device_type in ("cuda", "cpu")
    assert device_ctx.is_rocm is False
    assert device_ctx.rank == 0 or device_ctx.world_size > 1
    import torch

    want = torch.bfloat16 if device_ctx.device.type == "cuda" else torch.float32
    assert device_ctx.get_preferred_dtype() == want
    assert kernel_registry.dispatch("fused_logp") == "SM100_FUSED_LOGP"
    assert kernel_registry.dispatch("attention") == "SM100_ATTENTION"
    assert kernel_registry.dispatch("sampling") == "SM100_SAMPLING"
    assert kernel_registry.dispatch_legacy("fused_logp") == "FLASHINFER"
    assert kernel_registry.dispatch_legacy("attention") == "FLASH_ATTN"
    with pytest.raises(ValueError, match="Supported backends"):
        OpBackend["NOPE"]
    fn = kernel_registry.resolve(kernel_registry.dispatch("fused_logp"))
    assert callable(fn)
    assert kernel_registry.get_op_path(OpBackend.FLASHINFER).endswith("lmhead_logp")


def test_executor_flow():
    result = RolloutExecutor().execute_rollout()
    assert result["status"] == "success"
    assert result["kernels"] == ["SM100_FUSED_LOGP", "SM100_ATTENTION"]


def test_every_registered_operator_resolves_to_code():
    for backend in OpBackend:
        fn = kernel_registry.resolve(backend)
        assert callable(fn), backend
    for op_type, want in {"fused_logp": "lmhead_logp", "logits_logp": "logits_logp", "sampling": "sample",
                          "attention": "attention", "rmsnorm": "rmsnorm", "rope": "rope_", "swiglu": "swiglu",
                          "gemm": "gemm_bi", "gemm_reduce_scatter": "gemm_reduce_scatter",
                          "all_gather_gemm": "all_gather_gemm", "all_reduce": "all_reduce_det",
                          "grpo_loss": "grpo_loss"}.items():
        assert kernel_registry.resolve(kernel_registry.dispatch(op_type)).__name__ == want, op_type


def test_packages_are_real_packages():
    import importlib

    for sub in ("utils", "platforms", "kernels", "executors", "ops", "parallel", "models"):
        mod = importlib.import_module(f"kernel_align_b200.{sub}")
        assert mod.__file__ and mod.__file__.endswith("__init__.py")


def test_sampling_method_and_precision_enums_are_wired():
    import torch

    from kernel_align_b200.kernels.sampling import SamplerBackend
    from kernel_align_b200.platforms.constants import constants
    from kernel_align_b200.platforms.device import device_ctx

    logits = torch.randn(5, 300, generator=torch.Generator().manual_seed(0))
    s = SamplerBackend(seed=2)
    greedy = s.sample_with(constants.SamplingMethod.GREEDY, logits)
    assert torch.equal(greedy.long(), logits.argmax(-1))
    a = s.sample_with("top_k_top_p", logits, top_k=20, top_p=0.8, temperature=0.7, step=3)
    b = s.sample(logits, top_k=20, top_p=0.8, temperature=0.7, step=3)
    assert torch.equal(a, b)
    assert torch.equal(s.sample_with("nucleus", logits, top_p=0.5, step=1), s.sample(logits, top_p=0.5, step=1))
    assert torch.equal(s.sample_with("top_k", logits, top_k=7, step=1), s.sample(logits, top_k=7, step=1))
    assert torch.equal(s.sample_with("temperature", logits, temperature=1.3, step=1),
                       s.sample(logits, temperature=1.3, step=1))
    assert device_ctx.dtype_of(constants.PrecisionType.BF16) is torch.bfloat16
    assert device_ctx.dtype_of("float16") is torch.float16
    import pytest

    with pytest.raises(ValueError):
        device_ctx.dtype_of(constants.PrecisionType.INT4)


def test_doctor_reports_and_self_tests():
    from kernel_align_b200 import doctor

    info = doctor.collect()
    assert info["libka_cpu"] and info["distributed"]["gloo"]
    st = doctor.self_test()
    assert st["logp_max_abs_err"] < 1e-4 and st["logp_batch_invariant"] and st["sampler_batch_invariant"]
    assert doctor.main(["--json"]) == 0


def test_every_registered_operator_resolves_to_a_callable():
    from kernel_align_b200.kernels.registry import OpBackend, kernel_registry

    for backend in OpBackend:
        assert callable(kernel_registry.resolve(backend)), backend
    assert kernel_registry.dispatch("attention_backward") == "SM100_ATTENTION_BWD"
    assert kernel_registry.dispatch("decode_attention") == "SM100_ATTENTION_DECODE"
    assert kernel_registry.dispatch("skinny_gemm") == "SM100_GEMM_SKINNY"
    assert kernel_registry.dispatch("group_advantages") == "SM100_ADVANTAGES"
    assert kernel_registry.dispatch("attention") == "SM100_ATTENTION"
