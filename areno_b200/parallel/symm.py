"""Peer-memory communicator of a tensor-parallel group and the fused ops built on it.

``TpComm`` allocates one symmetric region per rank (raw ``cudaMalloc`` so that it can be exported
with CUDA IPC; the caching allocator's expandable segments cannot), exchanges the IPC handles over
the TP process group and maps every peer's region.  On top of it:

* ``push_linear(x, weight)``: the row-parallel GEMM whose epilogue writes the partial product into
  lane ``my_rank`` of the current inbox slot on EVERY rank (``areno_gemm_bf16_push``);
* ``reduce_rmsnorm(partial, residual, weight, ...)``: rendezvous with the peers, sum the lanes of the
  local inbox, add the residual stream and apply the following RMSNorm in one kernel
  (``areno_tp_reduce_rmsnorm``).

Together they replace ``all_reduce(o_proj(x))`` + ``rmsnorm(h + residual)`` (collective C1 of the
reference, ``areno/engine/parallel/collectives.py:143-155`` + ``layers/norm.py``) without NCCL.  The
ops are inference-only (no autograd); training keeps the autograd collectives.

Safety: waits inside the kernels are bounded and report through a status word
(``check_status``); nothing here uses multicast loads.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import gemm as gemm_ops

_lib.register_signature("areno_symm_alloc", "pl")
_lib.register_signature("areno_symm_free", "p")
_lib.register_signature("areno_ipc_export", "pp")
_lib.register_signature("areno_ipc_import", "pp")
_lib.register_signature("areno_ipc_close", "p")
_lib.register_signature("areno_tp_reduce_rmsnorm", "iipppplppifpplifp")
_lib.register_signature("areno_tp_barrier", "iipppip")
_lib.register_signature("areno_gemm_bf16_push", "ppppiiilllpiplpp")


@dataclass
class TpPartial:
    """Result of ``push_linear``: the partial sums sit in slot ``slot`` of every rank's inbox."""

    comm: "TpComm"
    slot: int
    rows: int
    local: torch.Tensor  # this rank's own lane (a view into the local inbox)


class TpComm:
    def __init__(self, group, tp_size: int, tp_rank: int, hidden: int, max_rows: int, device: torch.device):
        if hidden % 8 != 0:
            raise ValueError("hidden size must be a multiple of 8")
        self.group, self.tp, self.rank = group, int(tp_size), int(tp_rank)
        self.hidden, self.max_rows, self.device = int(hidden), int(max_rows), device
        lib = _lib._load()
        lib.areno_tp_flags_bytes.restype = ctypes.c_longlong
        self.flags_bytes = int(lib.areno_tp_flags_bytes())
        self.lane_elems = self.max_rows * self.hidden
        self.slot_elems = self.tp * self.lane_elems
        self.inbox_bytes = 2 * self.slot_elems * 2
        total = self.flags_bytes + self.inbox_bytes
        base = ctypes.c_void_p()
        with torch.cuda.device(device):
            _check("areno_symm_alloc", _lib.fn("areno_symm_alloc")(ctypes.byref(base), total))
            handle = (ctypes.c_ubyte * 64)()
            _check("areno_ipc_export", _lib.fn("areno_ipc_export")(base, handle))
            handles: list = [None] * self.tp
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
        self._flag_ptrs = (ctypes.c_void_p * self.tp)(*self.bases)
        self.epoch = torch.zeros(int(lib.areno_tp_max_blocks()), dtype=torch.int32, device=device)
        self.status = _lib.status_buffer(device)
        self.calls = 0
        self._push_ptrs: dict[int, ctypes.Array] = {}
        # the local inbox as a tensor, for views of this rank's own lane
        self._inbox = _as_tensor(self._local_base + self.flags_bytes, 2 * self.slot_elems, device)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    # ---------------------------------------------------------------- addresses
    def _lane_addr(self, rank_base: int, slot: int, lane: int) -> int:
        return rank_base + self.flags_bytes + 2 * (slot * self.slot_elems + lane * self.lane_elems)

    def _peer_lane_ptrs(self, slot: int):
        arr = self._push_ptrs.get(slot)
        if arr is None:
            peers = [self._lane_addr(b, slot, self.rank) for r, b in enumerate(self.bases) if r != self.rank]
            arr = (ctypes.c_void_p * max(len(peers), 1))(*peers)
            self._push_ptrs[slot] = arr
        return arr

    def next_slot(self) -> int:
        slot = self.calls & 1
        self.calls += 1
        return slot

    # ---------------------------------------------------------------------- ops
    def push_linear(self, x: torch.Tensor, weight: torch.Tensor) -> TpPartial:
        """``x [rows, K_local] @ weight[N, K_local]^T`` delivered to every rank's inbox."""
        rows, k = x.shape
        n = weight.shape[0]
        if n != self.hidden or rows > self.max_rows:
            raise ValueError(f"push_linear: output [{rows}, {n}] does not fit the inbox [{self.max_rows}, {self.hidden}]")
        if not x.is_contiguous():
            x = x.contiguous()
        slot = self.next_slot()
        lo = slot * self.slot_elems + self.rank * self.lane_elems
        local = self._inbox[lo: lo + rows * n].view(rows, n)
        ws_ptr, ws_bytes = None, 0
        if rows <= 128 and k >= 512:  # decode-shaped: split-K, the fold kernel delivers to the peers
            ws = gemm_ops._workspace(x.device, 16 * rows * n * 4)
            ws_ptr, ws_bytes = ws.data_ptr(), ws.numel()
        _lib.call("areno_gemm_bf16_push", x.data_ptr(), weight.data_ptr(), local.data_ptr(), None, rows, n, k,
                  x.stride(0), weight.stride(0), n, self._peer_lane_ptrs(slot), self.tp - 1, ws_ptr, ws_bytes,
                  self.status.data_ptr(), _lib.stream())
        return TpPartial(self, slot, rows, local)

    def reduce_rmsnorm(self, part: TpPartial, residual, weight, eps: float, w_offset: float = 0.0,
                       want_y: bool = True):
        """Returns ``(y, h)``: ``h = residual + sum over ranks``, ``y = rmsnorm(h) * (weight + w_offset)``."""
        rows, n = part.rows, self.hidden
        h = torch.empty((rows, n), dtype=torch.bfloat16, device=self.device)
        y = torch.empty_like(h) if want_y else None
        slot_addr = self._lane_addr(self._local_base, part.slot, 0)
        wf32 = int(weight is not None and weight.dtype == torch.float32)
        if residual is not None and not residual.is_contiguous():
            residual = residual.contiguous()
        _lib.call("areno_tp_reduce_rmsnorm", self.tp, self.rank, self._flag_ptrs, self.epoch.data_ptr(),
                  self.status.data_ptr(), slot_addr, self.lane_elems, _lib.ptr(residual), _lib.ptr(weight), wf32,
                  float(w_offset), _lib.ptr(y), h.data_ptr(), rows, n, float(eps), _lib.stream())
        return y, h

    def barrier(self, blocks: int = 1) -> None:
        _lib.call("areno_tp_barrier", self.tp, self.rank, self._flag_ptrs, self.epoch.data_ptr(),
                  self.status.data_ptr(), int(blocks), _lib.stream())

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


def _check(name: str, rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")


class _Blob:
    """Exposes a raw device range through ``__cuda_array_interface__`` so torch can view it."""

    def __init__(self, addr: int, elems: int):
        self.__cuda_array_interface__ = {"shape": (elems,), "typestr": "<u2", "data": (addr, False), "version": 3,
                                         "strides": None}


def _as_tensor(addr: int, elems: int, device: torch.device) -> torch.Tensor:
    t = torch.as_tensor(_Blob(addr, elems), device=device)
    return t.view(torch.bfloat16)


# ------------------------------------------------------------------ registry
_COMMS: dict[int, TpComm] = {}


def get_tp_comm(ctx) -> TpComm | None:
    """The communicator registered for this layout (``None``: use the NCCL collectives)."""
    return _COMMS.get(id(ctx))


def setup_tp_comm(ctx, hidden: int, max_rows: int) -> TpComm | None:
    if ctx.tp_size <= 1 or ctx.device.type != "cuda":
        return None
    comm = _COMMS.get(id(ctx))
    if comm is None or comm.hidden != hidden or comm.max_rows < max_rows:
        if comm is not None:
            comm.close()
        comm = TpComm(ctx.tp_group, ctx.tp_size, ctx.tp_rank, hidden, max_rows, ctx.device)
        _COMMS[id(ctx)] = comm
    return comm
