"""``python -m kernel_align_b200.doctor``: what this installation can do on this host.

Prints the package version, the state of the two native libraries (built / stale / missing,
with the compiler that would build them), the visible GPUs with their compute capability (the
kernels need sm_100), peer access between them, the distributed backends PyTorch offers, and
runs a two-second CPU self-test of the C++ library against PyTorch. Exit code 0 when at least
the CPU path works.
"""
from __future__ import annotations

import json
import os
import shutil
import sys


def collect() -> dict:
    import torch

    from . import __version__, _build

    info: dict = {"version": __version__, "torch": torch.__version__, "cuda_runtime": torch.version.cuda}
    info["nvcc"] = shutil.which("nvcc") or ("/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else None)
    info["cxx"] = shutil.which("g++")
    info["libka_sm100"] = str(_build.CUDA_LIB) if _build.CUDA_LIB.exists() else None
    info["libka_cpu"] = str(_build.CPU_LIB) if _build.CPU_LIB.exists() else None
    gpus = []
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            gpus.append({"index": i, "name": p.name, "capability": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                         "memory_gib": round(p.total_memory / 2**30, 1), "supported": p.major == 10})
        if len(gpus) > 1:
            info["peer_access_from_0"] = [bool(torch.cuda.can_device_access_peer(0, j)) for j in range(1, len(gpus))]
    info["gpus"] = gpus
    import torch.distributed as dist

    info["distributed"] = {"available": dist.is_available(),
                           "nccl": bool(dist.is_available() and dist.is_nccl_available()),
                           "gloo": bool(dist.is_available() and dist.is_gloo_available())}
    try:
        import torch.distributed._symmetric_memory  # noqa: F401

        info["symmetric_memory"] = True
    except Exception:  # noqa: BLE001
        info["symmetric_memory"] = False
    return info


def self_test() -> dict:
    """The CPU library against PyTorch on a small case, and bitwise batch invariance."""
    import torch

    from .ops import cpu_ops

    g = torch.Generator().manual_seed(0)
    h, w = torch.randn(32, 64, generator=g), torch.randn(200, 64, generator=g) * 0.1
    ids = torch.randint(0, 200, (32,), generator=g)
    got = cpu_ops.lmhead_logp_cpu(h, w, ids)
    want = torch.log_softmax(h @ w.t(), -1).gather(1, ids[:, None])[:, 0]
    logits = torch.randn(8, 500, generator=g)
    tok = cpu_ops.sample_cpu(logits, inv_temperature=1.0, top_k=20, top_p=0.9, seed=1, step=0)
    tok1 = cpu_ops.sample_cpu(logits[3:4], inv_temperature=1.0, top_k=20, top_p=0.9, seed=1, step=0,
                              row_ids=torch.tensor([3]))
    return {"logp_max_abs_err": float((got - want).abs().max()),
            "logp_batch_invariant": bool(torch.equal(cpu_ops.lmhead_logp_cpu(h[:1], w, ids[:1]), got[:1])),
            "sampler_batch_invariant": bool(tok[3] == tok1[0])}


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    info = collect()
    try:
        info["cpu_self_test"] = self_test()
        ok = info["cpu_self_test"]["logp_max_abs_err"] < 1e-4 and info["cpu_self_test"]["logp_batch_invariant"] \
            and info["cpu_self_test"]["sampler_batch_invariant"]
    except Exception as e:  # noqa: BLE001
        info["cpu_self_test"] = {"error": f"{type(e).__name__}: {e}"}
        ok = False
    if "--json" in argv:
        print(json.dumps(info, indent=1))
    else:
        print(f"kernel_align_b200 {info['version']}  (torch {info['torch']}, CUDA runtime {info['cuda_runtime']})")
        print(f"  sm_100a kernel library : {info['libka_sm100'] or 'not built'}   (nvcc: {info['nvcc'] or 'not found'})")
        print(f"  C++ CPU library        : {info['libka_cpu'] or 'not built'}   (g++: {info['cxx'] or 'not found'})")
        if info["gpus"]:
            for gpu in info["gpus"]:
                mark = "ok" if gpu["supported"] else "unsupported: the kernels are written for sm_100a"
                print(f"  GPU {gpu['index']}: {gpu['name']}, sm_{gpu['capability'].replace('.', '')}, {gpu['sms']} SMs, "
                      f"{gpu['memory_gib']} GiB  [{mark}]")
            if "peer_access_from_0" in info:
                print(f"  peer access from GPU 0 : {info['peer_access_from_0']}")
        else:
            print("  no GPU visible: CPU paths only")
        d = info["distributed"]
        print(f"  torch.distributed      : nccl={d['nccl']} gloo={d['gloo']} symmetric memory={info['symmetric_memory']}")
        print(f"  CPU self-test          : {info['cpu_self_test']}")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
