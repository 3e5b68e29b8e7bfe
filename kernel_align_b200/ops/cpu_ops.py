"""Python entry points of the C++ CPU library (``csrc/cpu``): the oracle the GPU tests
compare against and the implementation used when tensors live on the CPU."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from .. import _native


def _threads() -> int:
    """Worker threads of the C++ library: ``KA_CPU_THREADS`` or up to 16 cores. Rows are split
    over the threads and a row's arithmetic is done by one thread, so the count never changes
    a result."""
    env = os.environ.get("KA_CPU_THREADS")
    if env:
        return max(1, int(env))
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


def lmhead_logp_shard_cpu(hidden, weight_shard, ids, *, vocab: int, v_lo: int, scale: float = 1.0):
    """One rank's part of the vocabulary-parallel log-prob: ``(states [m, n_slices, 2], target [m])``,
    the (max, sum) state of each canonical slice this shard holds and the scaled logit of the
    row's id when it lies in the shard (see ``ka_cpu_lmhead_logp_shard``)."""
    lib = _native.cpu()
    h, w, i64 = _f32(hidden), _f32(weight_shard), _i64(ids)
    m, k = h.shape
    v_local = w.shape[0]
    vs = -(-vocab // 8)
    n_slices = -(-v_local // vs) if v_local else 0
    states = torch.empty(m, n_slices, 2, dtype=torch.float32)
    target = torch.empty(m, dtype=torch.float32)
    fn = lib.ka_cpu_lmhead_logp_shard
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int]
    rc = fn(h.data_ptr(), w.data_ptr(), i64.data_ptr(), states.data_ptr(), target.data_ptr(), m, k, int(vocab),
            int(v_lo), v_local, float(scale), _threads())
    if rc != 0:
        raise RuntimeError(f"ka_cpu_lmhead_logp_shard failed ({rc}): the shard must be whole canonical slices")
    return states, target


def lmhead_logp_merge_cpu(states, target, ids, *, vocab: int, return_lse: bool = False):
    """Merge the eight slice states of every row (``states [m, 8, 2]`` in slice order) by the
    canonical tree and subtract from the target logit: the last step of the vocabulary-parallel
    log-prob, the same arithmetic as the single-process path."""
    lib = _native.cpu()
    st, tg, i64 = _f32(states), _f32(target), _i64(ids)
    m = st.shape[0]
    if st.shape[1:] != (8, 2):
        raise ValueError("states must be [m, 8, 2]")
    logp = torch.empty(m, dtype=torch.float32)
    lse = torch.empty(m, dtype=torch.float32)
    fn = lib.ka_cpu_lmhead_logp_merge
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int]
    if fn(st.data_ptr(), tg.data_ptr(), i64.data_ptr(), logp.data_ptr(), lse.data_ptr(), m, int(vocab)) != 0:
        raise RuntimeError("ka_cpu_lmhead_logp_merge failed")
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
