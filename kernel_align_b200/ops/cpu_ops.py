"""Python entry points of the C++ CPU library (``csrc/cpu``): the oracle the GPU tests
compare against and the implementation used when tensors live on the CPU."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from .. import _native


def _threads() -> int:
    return max(1, min(16, os.cpu_count() or 1))


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to(device="cpu", dtype=torch.float32).contiguous()


def _i64(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to(device="cpu", dtype=torch.int64).contiguous()


def lmhead_logp_cpu(hidden, weight, ids, *, scale: float = 1.0, chunk_rows: int = 16, return_lse: bool = False):
    """``log_softmax(scale * hidden @ weight.T)[ids]`` on the CPU, ``chunk_rows`` rows of
    logits live at a time per worker thread. Inputs are widened to fp32 (exact for bf16)."""
    lib = _native.cpu()
    h, w, i = _f32(hidden), _f32(weight), _i64(ids)
    m, k = h.shape
    v = w.shape[0]
    logp = torch.empty(m, dtype=torch.float32)
    lse = torch.empty(m, dtype=torch.float32) if return_lse else None
    fn = lib.ka_cpu_lmhead_logp
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int]
    rc = fn(h.data_ptr(), w.data_ptr(), i.data_ptr(), logp.data_ptr(), lse.data_ptr() if return_lse else None,
            m, k, v, float(scale), int(chunk_rows), _threads())
    if rc != 0:
        raise RuntimeError(f"ka_cpu_lmhead_logp failed ({rc})")
    return (logp, lse) if return_lse else logp


def logits_logp_cpu(logits, ids, *, scale: float = 1.0, return_lse: bool = False):
    lib = _native.cpu()
    x = _f32(logits)
    rows, v = x.shape
    i = _i64(ids)
    logp = torch.empty(rows, dtype=torch.float32)
    lse = torch.empty(rows, dtype=torch.float32) if return_lse else None
    fn = lib.ka_cpu_logits_logp
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_longlong, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int]
    rc = fn(x.data_ptr(), x.stride(0), rows, v, i.data_ptr(), float(scale), logp.data_ptr(),
            lse.data_ptr() if return_lse else None, _threads())
    if rc != 0:
        raise RuntimeError(f"ka_cpu_logits_logp failed ({rc})")
    return (logp, lse) if return_lse else logp


def sample_cpu(logits, *, inv_temperature: float, top_k: int, top_p: float, seed: int, step: int, row_ids=None):
    """Token ids (int32) under the sampler's definition; bit-exact mirror of the CUDA kernels."""
    lib = _native.cpu()
    x = _f32(logits)
    rows, v = x.shape
    out = torch.empty(rows, dtype=torch.int32)
    rid = _i64(row_ids) if row_ids is not None else None
    fn = lib.ka_cpu_sample
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_longlong, c_int, c_int, c_void_p, c_float, c_int, c_float, c_ulonglong, c_ulonglong,
                   c_void_p]
    rc = fn(x.data_ptr(), x.stride(0), rows, v, rid.data_ptr() if rid is not None else None,
            float(inv_temperature), int(top_k), float(top_p), int(seed) & (2**64 - 1), int(step) & (2**64 - 1),
            out.data_ptr())
    if rc != 0:
        raise RuntimeError(f"ka_cpu_sample failed ({rc})")
    return out


def gemm_cpu(a, b):
    """``a @ b.T`` in fp32 with a fixed per-element accumulation order (CPU oracle)."""
    lib = _native.cpu()
    af, bf = _f32(a), _f32(b)
    m, k = af.shape
    n = bf.shape[0]
    out = torch.empty(m, n, dtype=torch.float32)
    fn = lib.ka_cpu_gemm
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int]
    if fn(af.data_ptr(), bf.data_ptr(), out.data_ptr(), m, n, k) != 0:
        raise RuntimeError("ka_cpu_gemm failed")
    return out


def gemm_sliced_cpu(a, b, residual=None, world: int = 1):
    """CPU emulation of the fused GEMM -> reduce-scatter arithmetic (8 canonical K slices, bf16
    partials, fp32 tree). ``world`` only assigns slices to emulated ranks."""
    lib = _native.cpu()
    af, bf = _f32(a), _f32(b)
    rf = _f32(residual) if residual is not None else None
    m, k = af.shape
    n = bf.shape[0]
    out = torch.empty(m, n, dtype=torch.float32)
    fn = lib.ka_cpu_gemm_sliced
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int]
    if fn(af.data_ptr(), bf.data_ptr(), rf.data_ptr() if rf is not None else None, out.data_ptr(), m, n, k, world) != 0:
        raise RuntimeError("ka_cpu_gemm_sliced failed")
    return out
