"""ctypes bindings to the two in-tree native libraries.

``cuda()`` returns the sm_100a kernel library and raises if it is missing: on a GPU host the
hand-written kernels are the only code path, there is no silent PyTorch fallback.
``cpu()`` returns the C++ CPU library (oracle for the tests and the CPU device path).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_longlong, c_size_t, c_uint, c_ulonglong, c_void_p
from functools import lru_cache

from . import _build


class NativeLibraryMissing(RuntimeError):
    pass


def _bind(lib, name, restype, argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = argtypes
    return fn


@lru_cache(maxsize=None)
def cuda() -> ctypes.CDLL:
    path = _build.build_cuda()
    if path is None or not path.exists():
        raise NativeLibraryMissing(
            "libka_sm100.so is not built; run `python -m kernel_align_b200._build` on a host with nvcc"
        )
    lib = ctypes.CDLL(str(path))
    _bind(lib, "ka_lmhead_logp_workspace_bytes", c_size_t, [c_int, c_int])
    _bind(lib, "ka_lmhead_logp_status_offset", c_int, [c_int, c_int])
    _bind(lib, "ka_lmhead_logp_exchange_bytes", c_size_t, [c_int, c_int])
    _bind(
        lib,
        "ka_lmhead_logp_forward",
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p,
         c_int, c_int, c_int, c_int, c_int, c_int, c_int,
         c_uint, c_float, c_int, c_int, c_int, c_ulonglong, c_void_p],
    )
    _bind(
        lib,
        "ka_lmhead_logp_forward_sched",
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p,
         c_int, c_int, c_int, c_int, c_int, c_int, c_int,
         c_uint, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_ulonglong, c_void_p],
    )
    _bind(lib, "ka_lmhead_logp_gather_bytes", c_size_t, [c_int, c_int, c_int])
    _bind(
        lib,
        "ka_lmhead_logp_forward_sharded",
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p,
         c_int, c_int, c_int, c_int, c_int, c_int, c_int,
         c_uint, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_ulonglong, c_void_p],
    )
    _bind(
        lib,
        "ka_sample",
        c_int,
        [c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_float, c_int, c_float,
         c_ulonglong, c_ulonglong, c_void_p, c_void_p],
    )
    _bind(
        lib,
        "ka_logits_logp",
        c_int,
        [c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p],
    )
    return lib


DTYPE_CODES = {"torch.float32": 0, "torch.bfloat16": 1, "torch.float16": 2}


def dtype_code(dtype) -> int:
    try:
        return DTYPE_CODES[str(dtype)]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}; expected float32, bfloat16 or float16") from None


@lru_cache(maxsize=None)
def cpu() -> ctypes.CDLL:
    # KA_CPU_LIB points the process at another build of the same library (the sanitizer tier
    # of the tests runs the CPU operators on an ASan / UBSan build in a child process)
    override = os.environ.get("KA_CPU_LIB")
    if override:
        return ctypes.CDLL(override)
    path = _build.build_cpu()
    if path is None or not path.exists():
        raise NativeLibraryMissing("libka_cpu.so is not built and no C++ compiler is available")
    return ctypes.CDLL(str(path))


def cuda_available() -> bool:
    import torch

    return torch.cuda.is_available()
