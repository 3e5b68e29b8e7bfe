"""Failure detection on the device, without faulting it: a wait whose flag nobody sets runs
into its (short) limit, the kernel returns, the status block says where it gave up, and the
context stays usable."""
import ctypes
from ctypes import c_int, c_longlong, c_uint, c_ulonglong, c_void_p

import pytest
import torch

from kernel_align_b200 import _native

pytestmark = pytest.mark.gpu


def test_all_reduce_wait_runs_out_and_reports(cuda_device):
    lib = _native.cuda()
    fn = lib.ka_allreduce_det
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_uint, c_void_p, c_int, c_ulonglong, c_void_p]
    lib.ka_allreduce_flag_bytes.restype = ctypes.c_size_t
    lib.ka_allreduce_flag_bytes.argtypes = [c_int, c_int]
    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    n = 4096
    # "rank 0" of a 2-rank group whose peer never launches: both buffers live on this GPU,
    # only one kernel runs, so nothing waits on a kernel that is not resident
    bufs = [torch.ones(n, device=cuda_device), torch.ones(n, device=cuda_device)]
    flags = [torch.zeros(lib.ka_allreduce_flag_bytes(2, sms) // 4, dtype=torch.int32, device=cuda_device)
             for _ in range(2)]
    status = torch.zeros(8, dtype=torch.int32, device=cuda_device)
    bp = (c_void_p * 2)(*[b.data_ptr() for b in bufs])
    fp = (c_void_p * 2)(*[f.data_ptr() for f in flags])
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = fn(bp, fp, n, 0, 2, 0, 1, status.data_ptr(), sms, 50_000_000, torch.cuda.current_stream().cuda_stream)
    t1.record()
    torch.cuda.synchronize()
    assert rc == 0
    st = status.cpu().tolist()
    assert st[0] == 2 and st[1] == 21, st      # kTimeoutFlag at the start handshake
    assert st[4] == 1 and st[5] == 0, st       # expected epoch 1, saw 0
    assert 40 < t0.elapsed_time(t1) < 1000     # gave up after ~50 ms, did not hang
    assert torch.equal(bufs[0], torch.ones(n, device=cuda_device))  # nothing was reduced
    # the context is intact: ordinary work still runs
    assert (torch.arange(10, device=cuda_device).sum().item()) == 45
