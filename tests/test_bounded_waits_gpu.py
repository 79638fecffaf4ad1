"""One GPU: every wait on a peer inside the communication kernels is bounded.  Each test launches a kernel
whose peer flag nobody will ever raise (the "peer" is a second flag block in local memory), with a wait bound
of a few milliseconds, and checks that the kernel returns, reports the documented status code, publishes
nothing, and leaves the context usable.  Nothing here faults, traps or hangs the GPU."""

from __future__ import annotations

import ctypes

import pytest
import torch

from areno_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _desc(flags0, flags1, part, h, y, status, wait_ms):
    from areno_b200.parallel.symm import TpDesc, _ptr_array

    arrays = [_ptr_array([flags0.data_ptr(), flags1.data_ptr()])] + [_ptr_array([t.data_ptr(), t.data_ptr()])
                                                                     for t in (part, h, y)]
    desc = TpDesc(2, 0, arrays[0], arrays[1], arrays[2], arrays[3], None, None, None, status.data_ptr(), wait_ms)
    return desc, arrays


def _status(dev):
    buf = _lib.status_buffer(dev)
    torch.cuda.synchronize()
    vals = buf.tolist()
    buf.zero_()
    return vals


@pytest.mark.parametrize("oneshot", [0, 1])
def test_fused_reduce_gives_up_on_a_silent_peer_and_publishes_nothing(oneshot):
    dev = torch.device("cuda", 0)
    rows, H = 8, 1024
    flags0 = torch.zeros(64, dtype=torch.int32, device=dev)
    flags1 = torch.zeros(64, dtype=torch.int32, device=dev)      # stands in for the peer; nobody raises our slot
    part = torch.randn(rows, H, device=dev).to(torch.bfloat16)
    h = torch.full((rows, H), 7.0, device=dev, dtype=torch.bfloat16)
    y = torch.full((rows, H), 7.0, device=dev, dtype=torch.bfloat16)
    status = _lib.status_buffer(dev)
    status.zero_()
    desc, keep = _desc(flags0, flags1, part, h, y, status, wait_ms=3)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    _lib.call("areno_tp_reduce_norm", ctypes.addressof(desc), 0, None, None, 0, 0.0, 1, rows, H, 1e-6, 0, oneshot, _lib.stream())
    end.record()
    vals = _status(dev)
    assert vals[0] == 7 and vals[2] == 1, vals          # code 7: the partial of peer 1 never became ready
    assert 2.0 < start.elapsed_time(end) < 500.0        # waited for the bound, not for ever
    assert torch.all(h == 7.0) and torch.all(y == 7.0)  # nothing was summed or published
    assert int(flags0[0]) == 1                          # the call counter still advanced: the next call is well-formed
    assert int(flags1[8]) == 1                          # the announcement reached the "peer"
    assert int(flags1[16]) == (0 if oneshot else 1)     # two-shot also announces (empty) publication, so nobody waits on it
    with pytest.raises(RuntimeError, match="status code=7"):
        status[0] = 7
        _lib.check_status(dev)
    # the context is intact: an ordinary kernel still runs and is correct
    a = torch.randn(64, 256, device=dev).to(torch.bfloat16)
    from areno_b200.ops import gemm

    out = gemm.gemm(a, a)
    torch.cuda.synchronize()
    assert torch.allclose(out.float(), a.float() @ a.float().t(), rtol=2e-2, atol=2e-1)


def test_group_barrier_gives_up_on_a_silent_peer():
    dev = torch.device("cuda", 0)
    flags0 = torch.zeros(64, dtype=torch.int32, device=dev)
    flags1 = torch.zeros(64, dtype=torch.int32, device=dev)
    dummy = torch.zeros(8, device=dev, dtype=torch.bfloat16)
    status = _lib.status_buffer(dev)
    status.zero_()
    desc, keep = _desc(flags0, flags1, dummy, dummy, dummy, status, wait_ms=2)
    _lib.call("areno_tp_barrier", ctypes.addressof(desc), _lib.stream())
    vals = _status(dev)
    assert vals[0] == 7 and vals[2] == 1, vals
    # a peer that does answer: raise its flags by hand, the same call now passes without a report
    flags0[8 + 1] = 2
    desc2, keep2 = _desc(flags0, flags1, dummy, dummy, dummy, status, wait_ms=2)
    _lib.call("areno_tp_barrier", ctypes.addressof(desc2), _lib.stream())
    assert _status(dev)[0] == 0


def test_gradient_reduce_scatter_gives_up_when_a_peer_never_announces():
    dev = torch.device("cuda", 0)
    from areno_b200.parallel import grad_comm  # noqa: F401  (registers the signatures)

    lib = _lib._load()
    lib.areno_dp_ready_bytes.restype = ctypes.c_longlong
    ready0 = torch.zeros(int(lib.areno_dp_ready_bytes()) // 4, dtype=torch.int32, device=dev)
    ready1 = torch.zeros_like(ready0)
    grads = torch.randn(4096, device=dev)
    before = grads.clone()
    status = _lib.status_buffer(dev)
    status.zero_()
    ready_ptrs = (ctypes.c_void_p * 2)(ready0.data_ptr(), ready1.data_ptr())
    grad_ptrs = (ctypes.c_void_p * 2)(grads.data_ptr(), grads.data_ptr())
    # this rank announces bucket 3, the "peer" never does
    _lib.call("areno_dp_grad_ready", 2, 0, ready_ptrs, grad_ptrs, status.data_ptr(), 3, 1, _lib.stream())
    _lib.call("areno_dp_grad_reduce_scatter", 2, 0, ready_ptrs, grad_ptrs, status.data_ptr(), 3, 1, 0, 2048,
              grads.data_ptr(), 4, 2, _lib.stream())
    vals = _status(dev)
    assert vals[0] == 8 and vals[1] == 3 and vals[2] == 1, vals     # code 8, bucket 3, peer 1
    assert torch.equal(grads, before)                                # nothing was reduced
