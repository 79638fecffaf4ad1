"""Data-parallel gradient reduce-scatter over peer memory, overlapped with backward.

``GradComm`` owns one symmetric region per rank (raw ``cudaMalloc`` exported with CUDA IPC and mapped by
every rank of the DP group): a block of flags followed by the fp32 gradient buckets of the optimizer, laid
out identically on every rank.  When a bucket's gradients are final on this rank, ``launch(bucket)`` raises
the bucket's ready flag on every rank from the compute stream and queues the reduce-scatter kernel on a
side stream: the owner of each shard pulls that shard from every rank's bucket with plain peer loads
(NVLink) and sums it in rank order into its own bucket, while backward continues.  ``finish()`` joins the
side stream, checks the status word (a peer that never raised its flag is reported, not waited for forever)
and runs a cross-rank barrier so nobody zeroes a bucket that a slower rank is still reading.

Replaces the per-parameter ``all_reduce`` after backward of the reference
(``areno/engine/training.py:157-169``) and the NCCL reduce-scatter this package uses otherwise.  No
multicast loads; every wait is bounded.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _lib
from .symm import TpDesc, _check, _ptr_array

_lib.register_signature("areno_dp_grad_ready", "iipppiip")
_lib.register_signature("areno_dp_grad_reduce_scatter", "iipppiillpiip")


class _Blob32:
    def __init__(self, addr: int, elems: int):
        self.__cuda_array_interface__ = {"shape": (elems,), "typestr": "<f4", "data": (addr, False), "version": 3,
                                         "strides": None}


class GradComm:
    def __init__(self, group, size: int, rank: int, total_elems: int, device: torch.device):
        self.group, self.n, self.rank, self.device = group, int(size), int(rank), device
        lib = _lib._load()
        lib.areno_tp_flags_bytes.restype = ctypes.c_longlong
        lib.areno_dp_ready_bytes.restype = ctypes.c_longlong
        self.barrier_bytes = int(lib.areno_tp_flags_bytes())
        self.ready_bytes = int(lib.areno_dp_ready_bytes())
        self.max_buckets = int(lib.areno_dp_max_buckets())
        self.header = (self.barrier_bytes + self.ready_bytes + 255) // 256 * 256
        self.total_elems = int(total_elems)
        total = self.header + 4 * self.total_elems
        base = ctypes.c_void_p()
        with torch.cuda.device(device):
            _check("areno_symm_alloc", _lib.fn("areno_symm_alloc")(ctypes.byref(base), total))
            handle = (ctypes.c_ubyte * 64)()
            _check("areno_ipc_export", _lib.fn("areno_ipc_export")(base, handle))
            handles: list = [None] * self.n
            dist.all_gather_object(handles, bytes(handle), group=group)
            self.bases: list[int] = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.bases.append(int(base.value))
                    continue
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                mapped = ctypes.c_void_p()
                _check("areno_ipc_import", _lib.fn("areno_ipc_import")(buf, ctypes.byref(mapped)))
                self.bases.append(int(mapped.value))
        self._local_base = int(base.value)
        self._barrier_ptrs = (ctypes.c_void_p * self.n)(*self.bases)
        self._ready_ptrs = (ctypes.c_void_p * self.n)(*[b + self.barrier_bytes for b in self.bases])
        self._grad_ptrs = (ctypes.c_void_p * self.n)(*[b + self.header for b in self.bases])
        self.grads = torch.as_tensor(_Blob32(self._local_base + self.header, self.total_elems), device=device)
        self.status = _lib.status_buffer(device)
        self.stream = torch.cuda.Stream(device=device)
        self.epoch = 0
        self.launched: set[int] = set()
        self.blocks = int(os.environ.get("ARENO_GRAD_RS_BLOCKS", "64"))
        # how long a reducer waits for a peer's gradients; ranks only meet here once per step, so the bound has to
        # cover the skew that a whole rollout + backward can build up between them (power capping alone gives
        # several per cent), while still ending a wait for a rank that is gone
        self.wait_ms = int(os.environ.get("ARENO_GRAD_RS_WAIT_MS", "20000"))
        # the rendezvous after the reduction uses the same bound: it is the only guard before the buckets are zeroed
        self._barrier_desc = TpDesc(self.n, self.rank, _ptr_array(self.bases), None, None, None, None, None, None,
                                    self.status.data_ptr(), self.wait_ms)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def view(self, offset: int, numel: int) -> torch.Tensor:
        """fp32 view of ``numel`` elements of the local gradient region starting at element ``offset``."""
        return self.grads[offset:offset + numel]

    def begin_step(self) -> None:
        """Called once per optimizer step, before the first ``launch``."""
        self.epoch += 1
        self.launched.clear()

    def launch(self, bucket: int, offset: int, shard: int) -> None:
        """The gradients of ``bucket`` (``n * shard`` elements at element ``offset`` of the region) are final
        on this rank: tell the peers and queue the reduction of this rank's shard."""
        if bucket in self.launched:
            return
        if bucket >= self.max_buckets:
            raise ValueError(f"bucket index {bucket} exceeds the flag table ({self.max_buckets})")
        self.launched.add(bucket)
        cur = torch.cuda.current_stream(self.device)
        _lib.call("areno_dp_grad_ready", self.n, self.rank, self._ready_ptrs, self._grad_ptrs, self.status.data_ptr(),
                  bucket, self.epoch, cur.cuda_stream)
        ev = torch.cuda.Event()
        ev.record(cur)
        self.stream.wait_event(ev)       # the reducer never waits for a kernel of its own GPU, only for peers
        lo = offset + self.rank * shard
        _lib.call("areno_dp_grad_reduce_scatter", self.n, self.rank, self._ready_ptrs, self._grad_ptrs,
                  self.status.data_ptr(), bucket, self.epoch, lo, shard, self.grads.data_ptr() + 4 * lo, self.blocks,
                  self.wait_ms, self.stream.cuda_stream)

    def finish(self) -> None:
        """Join the side stream, fail loudly if a peer never delivered, then rendezvous with the group."""
        cur = torch.cuda.current_stream(self.device)
        cur.wait_stream(self.stream)
        _lib.check_status()   # host read of the status word: a timed-out wait must not reach the optimizer
        _lib.call("areno_tp_barrier", ctypes.addressof(self._barrier_desc), cur.cuda_stream)

    def close(self) -> None:
        if not self.bases:
            return
        torch.cuda.synchronize(self.device)
        try:
            dist.barrier(group=self.group)
        except Exception:
            pass
        for r, b in enumerate(self.bases):
            if r != self.rank:
                _lib.fn("areno_ipc_close")(ctypes.c_void_p(b))
        _lib.fn("areno_symm_free")(ctypes.c_void_p(self._local_base))
        self.bases = []
