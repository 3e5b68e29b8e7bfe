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


def test_fused_logp_gather_wait_runs_out_and_reports(cuda_device):
    """Row-sharded fused log-prob as "rank 0" of two whose peer never launches: the kernel works
    through its own rows, pushes them to the peer's arena (memory of this GPU here), waits for
    the peer's rows at the gather flag, runs into the 100 ms limit, reports the site and
    returns; nothing hangs and the context stays usable."""
    lib = _native.cuda()
    m_local, k, vocab, panel = 512, 256, 4096, 1024
    g = torch.Generator(device=cuda_device).manual_seed(0)
    h = torch.randn(m_local, k, device=cuda_device, generator=g).to(torch.bfloat16)
    w = (torch.randn(vocab // 2, k, device=cuda_device, generator=g) * 0.02).to(torch.bfloat16)   # slices 0..3
    ids = torch.randint(0, vocab, (m_local,), device=cuda_device, generator=g)
    logp = torch.zeros(m_local, device=cuda_device)
    ws_bytes = lib.ka_lmhead_logp_workspace_bytes(vocab, panel)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=cuda_device)
    xb = lib.ka_lmhead_logp_exchange_bytes(2, panel)
    gb = lib.ka_lmhead_logp_gather_bytes(2, panel, k)
    exch = [torch.zeros(xb, dtype=torch.uint8, device=cuda_device) for _ in range(2)]
    gath = [torch.zeros(gb, dtype=torch.uint8, device=cuda_device) for _ in range(2)]
    xp = (c_void_p * 2)(*[t.data_ptr() for t in exch])
    gp = (c_void_p * 2)(*[t.data_ptr() for t in gath])
    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = lib.ka_lmhead_logp_forward_sharded(
        h.data_ptr(), w.data_ptr(), ids.data_ptr(), logp.data_ptr(), None, ws.data_ptr(), ws_bytes, xp, gp,
        m_local, k, vocab, vocab // 2, 0, 2, 0, 1, 1.0, panel, 0, 2, 0, 0, 0, sms, 100_000_000,
        torch.cuda.current_stream().cuda_stream)
    t1.record()
    torch.cuda.synchronize()
    assert rc == 0
    off = lib.ka_lmhead_logp_status_offset(vocab, panel)
    st = ws[off:off + 32].view(torch.int32).cpu().tolist()
    # a wait ran out: normally the producer's wait for the peer's rows (site 6), which starts first;
    # the waits downstream of it (operands 2, accumulator 4, the peer's partial results 5) are also legitimate
    assert st[0] in (1, 2) and st[1] in (2, 4, 5, 6), st
    assert 90 < t0.elapsed_time(t1) < 3000
    # this rank's rows did reach the "peer": the pusher does not depend on anybody
    pl = panel // 2
    pushed = gath[1][: 2 * 2 * pl * k * 2].view(torch.bfloat16).view(2, 2, pl, k)[1, 0, :m_local]   # generation 1 (epoch 1), source 0
    assert torch.equal(pushed, h)
    assert (torch.arange(10, device=cuda_device).sum().item()) == 45
