"""Symmetric heap and the tensor-parallel communicator built on it.

``SymmHeap`` gives every rank of a process group one device allocation of the same size that all of
its peers map into their own address space, and, where the GPUs sit on one NVSwitch fabric that
supports it, a multicast mapping of the same pages for ``multimem`` instructions (in-switch
reduction and broadcast).  The allocation is made with the CUDA virtual-memory API
(``csrc/symm_heap.cu``); the shareable handles are POSIX file descriptors and travel between the
ranks over Unix-domain sockets.  Where that API is unavailable the heap falls back to ``cudaMalloc``
plus CUDA IPC (no multicast).

``TpComm`` lays the buffers of the fused row-parallel path out in such a heap (``csrc/comm.cu``):

* ``row_linear(x, weight)``: the row-parallel GEMM (o_proj / down_proj) writes this rank's partial
  product straight into the heap;
* ``new_partial(rows)``: a slot for a producer that writes its share itself; the vocabulary-parallel embedding
  lookup uses it (rows owned by other ranks are zero);
* ``reduce_rmsnorm(partial, residual, weight, ...)``: one kernel per rank reduces the partials over the
  group (each rank sums the rows it owns, through the switch or with plain peer loads), adds the
  residual stream, applies the following RMSNorm and publishes both results to every rank.

Together they replace ``all_reduce(o_proj(x))`` + ``rmsnorm(h + residual)`` (collective C1 of the
reference, ``areno/engine/parallel/collectives.py:143-155`` + ``layers/norm.py``) without NCCL.  The ops
are inference-only (no autograd); training keeps the autograd collectives.

Safety: every wait inside the kernels is bounded by wall time and reports through a status word
(``ops._lib.check_status``); nothing here uses a TMA load or cluster multicast.  ``ARENO_TP_MULTIMEM=0``
keeps the kernels on plain peer loads and stores.
"""

from __future__ import annotations

import ctypes
import os
import socket
import tempfile
import uuid
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import gemm as gemm_ops
from ..utils.log import get_logger

logger = get_logger()

_lib.register_signature("areno_symm_alloc", "pl")
_lib.register_signature("areno_symm_free", "p")
_lib.register_signature("areno_ipc_export", "pp")
_lib.register_signature("areno_ipc_import", "pp")
_lib.register_signature("areno_ipc_close", "p")
_lib.register_signature("areno_vmm_supported", "pp")
_lib.register_signature("areno_vmm_granularity", "ip")
_lib.register_signature("areno_vmm_alloc", "llppp")
_lib.register_signature("areno_vmm_import", "illpp")
_lib.register_signature("areno_vmm_release", "pll")
_lib.register_signature("areno_mc_create", "ilpp")
_lib.register_signature("areno_mc_import", "ip")
_lib.register_signature("areno_mc_add_device", "l")
_lib.register_signature("areno_mc_bind", "lllp" + "p")
_lib.register_signature("areno_mc_release", "lpli")
_lib.register_signature("areno_tp_reduce_norm", "plppifilifiip")
_lib.register_signature("areno_tp_barrier", "pp")


def _check(name: str, rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")


class TpDesc(ctypes.Structure):
    """Mirror of ``ArenoTpDesc`` (``csrc/comm.cu``)."""

    _fields_ = [("tp", ctypes.c_int), ("rank", ctypes.c_int),
                ("flags", ctypes.POINTER(ctypes.c_void_p)), ("part", ctypes.POINTER(ctypes.c_void_p)),
                ("h_out", ctypes.POINTER(ctypes.c_void_p)), ("y_out", ctypes.POINTER(ctypes.c_void_p)),
                ("part_mc", ctypes.c_void_p), ("h_mc", ctypes.c_void_p), ("y_mc", ctypes.c_void_p),
                ("status", ctypes.c_void_p), ("wait_ms", ctypes.c_int)]


def _ptr_array(values):
    return (ctypes.c_void_p * len(values))(*values)


# ------------------------------------------------------------------ descriptor exchange
def exchange_fds(group, rank: int, size: int, fds: list[int]) -> list[list[int]]:
    """Every rank sends the file descriptors ``fds`` to every other rank of ``group`` (Unix sockets,
    ``SCM_RIGHTS``).  Returns, per source rank, the descriptors as received here (own entry: ``fds``)."""
    path = os.path.join(tempfile.gettempdir(), f"areno_symm_{os.getpid()}_{uuid.uuid4().hex[:12]}.sock")
    server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    server.bind(path)
    server.listen(size)
    try:
        paths: list = [None] * size
        dist.all_gather_object(paths, path, group=group)   # every rank is listening once this returns
        for r, peer_path in enumerate(paths):
            if r == rank:
                continue
            with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
                c.connect(peer_path)
                socket.send_fds(c, [rank.to_bytes(4, "little")], list(fds))
        received: list[list[int]] = [list(fds) if r == rank else [] for r in range(size)]
        server.settimeout(120.0)
        for _ in range(size - 1):
            conn, _addr = server.accept()
            with conn:
                msg, got, _flags, _a = socket.recv_fds(conn, 16, max(len(fds), 1))
                received[int.from_bytes(msg[:4], "little")] = list(got)
        return received
    finally:
        server.close()
        try:
            os.unlink(path)
        except OSError:
            pass


class SymmHeap:
    """One same-sized device allocation per rank of ``group``, mapped by all of them.

    ``bases[r]`` is the address of rank r's allocation in THIS process (``bases[rank]`` is local memory);
    ``mc_base`` is the multicast address of the allocation (0 when unavailable)."""

    def __init__(self, group, size: int, rank: int, nbytes: int, device: torch.device, multicast: bool = True):
        self.group, self.size, self.rank, self.device = group, int(size), int(rank), device
        self.bases: list[int] = []
        self.mc_base = 0
        self.kind = "none"
        self._handles: list[int] = []
        self._mc_handle = 0
        self._mc_bound = False
        with torch.cuda.device(device):
            vmm, mc = ctypes.c_int(0), ctypes.c_int(0)
            rc = _lib.fn("areno_vmm_supported")(ctypes.byref(vmm), ctypes.byref(mc))
            ok = [None] * self.size
            want_vmm = rc == 0 and vmm.value == 1 and os.environ.get("ARENO_SYMM_HEAP", "vmm") != "ipc"
            dist.all_gather_object(ok, (want_vmm, bool(mc.value)), group=group)
            use_vmm = all(o[0] for o in ok)
            use_mc = multicast and use_vmm and self.size > 1 and all(o[1] for o in ok)
            if not (use_vmm and self._init_vmm(nbytes, use_mc)):
                self._release_vmm()
                self._init_ipc(nbytes)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    # ------------------------------------------------------------------ virtual-memory backend
    def _agree(self, ok: bool, what: str) -> bool:
        """Every rank reports whether its local step worked; the path is kept only if it worked everywhere."""
        states = [None] * self.size
        dist.all_gather_object(states, bool(ok), group=self.group)
        if not all(states):
            if self.rank == 0:
                logger.warning("symmetric heap: %s failed on ranks %s; using cudaMalloc + CUDA IPC", what,
                               [r for r, s in enumerate(states) if not s])
            return False
        return True

    def _init_vmm(self, nbytes: int, use_mc: bool) -> bool:
        """Allocate, exchange descriptors, map the peers.  Local failures are agreed on by the whole group after
        each phase, so either every rank ends up on this path or every rank takes the fallback."""
        gran = ctypes.c_longlong(0)
        rc = _lib.fn("areno_vmm_granularity")(self.size if use_mc else 1, ctypes.byref(gran))
        grans = [None] * self.size
        dist.all_gather_object(grans, int(gran.value) if rc == 0 else 0, group=self.group)
        if min(grans) <= 0:
            return False
        self.granule = max(grans)
        self.nbytes = (int(nbytes) + self.granule - 1) // self.granule * self.granule
        base, handle, fd = ctypes.c_void_p(), ctypes.c_ulonglong(0), ctypes.c_int(-1)
        rc = _lib.fn("areno_vmm_alloc")(self.nbytes, self.granule, ctypes.byref(base), ctypes.byref(handle), ctypes.byref(fd))
        self.bases = [0] * self.size
        self._handles = [0] * self.size
        if rc == 0:
            self.bases[self.rank], self._handles[self.rank] = int(base.value), int(handle.value)
            self.kind = "vmm"
        if not self._agree(rc == 0, "allocation"):
            if rc == 0:
                os.close(fd.value)
            return False
        ok = True
        try:
            received = exchange_fds(self.group, self.rank, self.size, [fd.value])
        except OSError as exc:
            logger.warning("symmetric heap: descriptor exchange failed: %s", exc)
            received, ok = [[] for _ in range(self.size)], False
        os.close(fd.value)
        for r, got in enumerate(received):
            if r == self.rank or not got:
                ok = ok and (r == self.rank)
                continue
            p, h = ctypes.c_void_p(), ctypes.c_ulonglong(0)
            rc = _lib.fn("areno_vmm_import")(got[0], self.nbytes, self.granule, ctypes.byref(p), ctypes.byref(h))
            os.close(got[0])
            if rc != 0:
                ok = False
                continue
            self.bases[r], self._handles[r] = int(p.value), int(h.value)
        if not self._agree(ok, "peer mapping"):
            return False
        if use_mc and os.environ.get("ARENO_TP_MULTIMEM", "1") != "0":
            self._init_multicast()
        return True

    def _init_multicast(self) -> None:
        """Multicast object over the same pages; any failure leaves the heap usable without it."""
        state = "ok"
        mc = ctypes.c_ulonglong(0)
        fd = ctypes.c_int(-1)
        if self.rank == 0:
            if _lib.fn("areno_mc_create")(self.size, self.nbytes, ctypes.byref(mc), ctypes.byref(fd)) != 0:
                state = "create failed"
        states = [None] * self.size
        dist.all_gather_object(states, state, group=self.group)
        if states[0] != "ok":
            logger.info("symmetric heap: no multicast object (%s); using plain peer loads / stores", states[0])
            return
        received = exchange_fds(self.group, self.rank, self.size, [fd.value] if self.rank == 0 else [])
        if self.rank == 0:
            os.close(fd.value)
        else:
            got = received[0]
            if not got or _lib.fn("areno_mc_import")(got[0], ctypes.byref(mc)) != 0:
                state = "import failed"
            if got:
                os.close(got[0])
        if state == "ok" and _lib.fn("areno_mc_add_device")(mc.value) != 0:
            state = "add_device failed"
        dist.all_gather_object(states, state, group=self.group)     # all devices are added before anyone binds
        self._mc_handle = int(mc.value)
        if any(s != "ok" for s in states):
            logger.info("symmetric heap: multicast set-up incomplete (%s); using plain peer loads / stores", states)
            self._drop_multicast()
            return
        p = ctypes.c_void_p()
        rc = _lib.fn("areno_mc_bind")(self._mc_handle, self._handles[self.rank], self.nbytes, self.granule, ctypes.byref(p))
        self._mc_bound = rc == 0
        dist.all_gather_object(states, "ok" if rc == 0 else f"bind failed ({rc})", group=self.group)
        if any(s != "ok" for s in states):
            logger.info("symmetric heap: multicast bind incomplete (%s); using plain peer loads / stores", states)
            if rc == 0:
                self.mc_base = int(p.value)
            self._drop_multicast()
            return
        self.mc_base = int(p.value)

    def _drop_multicast(self) -> None:
        if self._mc_handle:
            _lib.fn("areno_mc_release")(self._mc_handle, ctypes.c_void_p(self.mc_base or None), self.nbytes,
                                        1 if self._mc_bound else 0)
        self._mc_handle, self.mc_base, self._mc_bound = 0, 0, False

    def _release_vmm(self) -> None:
        if self.kind != "vmm":
            return
        self._drop_multicast()
        for r, (b, h) in enumerate(zip(self.bases, self._handles)):
            if b or h:
                _lib.fn("areno_vmm_release")(ctypes.c_void_p(b or None), self.nbytes, h)
        self.bases, self._handles, self.kind = [], [], "none"

    # ------------------------------------------------------------------ cudaMalloc + IPC backend
    def _init_ipc(self, nbytes: int) -> None:
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        base = ctypes.c_void_p()
        _check("areno_symm_alloc", _lib.fn("areno_symm_alloc")(ctypes.byref(base), self.nbytes))
        handle = (ctypes.c_ubyte * 64)()
        _check("areno_ipc_export", _lib.fn("areno_ipc_export")(base, handle))
        handles: list = [None] * self.size
        dist.all_gather_object(handles, bytes(handle), group=self.group)
        self.bases = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.bases.append(int(base.value))
                continue
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            mapped = ctypes.c_void_p()
            _check("areno_ipc_import", _lib.fn("areno_ipc_import")(buf, ctypes.byref(mapped)))
            self.bases.append(int(mapped.value))
        self.kind = "ipc"

    @property
    def local_base(self) -> int:
        return self.bases[self.rank]

    def close(self) -> None:
        if not self.bases:
            return
        torch.cuda.synchronize(self.device)
        try:
            dist.barrier(group=self.group)
        except Exception:
            pass
        with torch.cuda.device(self.device):
            if self.kind == "vmm":
                self._release_vmm()
            elif self.kind == "ipc":
                for r, b in enumerate(self.bases):
                    if r != self.rank:
                        _lib.fn("areno_ipc_close")(ctypes.c_void_p(b))
                _lib.fn("areno_symm_free")(ctypes.c_void_p(self.bases[self.rank]))
        self.bases = []


class _Blob:
    """Exposes a raw device range through ``__cuda_array_interface__`` so torch can view it."""

    def __init__(self, addr: int, elems: int, typestr: str = "<u2"):
        self.__cuda_array_interface__ = {"shape": (elems,), "typestr": typestr, "data": (addr, False), "version": 3,
                                         "strides": None}


def _as_tensor(addr: int, elems: int, device: torch.device) -> torch.Tensor:
    t = torch.as_tensor(_Blob(addr, elems), device=device)
    return t.view(torch.bfloat16)


@dataclass
class TpPartial:
    """A row-parallel result that is still spread over the group: every rank's share sits in slot
    ``slot`` of its own ``partial`` buffer."""

    comm: "TpComm"
    slot: int
    rows: int
    local: torch.Tensor  # this rank's share (a view into the local heap)


class TpComm:
    HEADER = 4096   # flag block (256 bytes) padded so the buffers start page-aligned

    def __init__(self, group, tp_size: int, tp_rank: int, hidden: int, max_rows: int, device: torch.device):
        if hidden % 8 != 0:
            raise ValueError("hidden size must be a multiple of 8")
        self.group, self.tp, self.rank = group, int(tp_size), int(tp_rank)
        self.hidden, self.max_rows, self.device = int(hidden), int(max_rows), device
        self.slot_elems = self.max_rows * self.hidden
        self.buf_bytes = (2 * self.slot_elems * 2 + 4095) // 4096 * 4096
        total = self.HEADER + 3 * self.buf_bytes
        self.heap = SymmHeap(group, self.tp, self.rank, total, device)
        bases = self.heap.bases
        self.off_part, self.off_h, self.off_y = self.HEADER, self.HEADER + self.buf_bytes, self.HEADER + 2 * self.buf_bytes
        self.status = _lib.status_buffer(device)
        mc = self.heap.mc_base
        # multimem (in-switch reduction / broadcast) pays from four ranks on; between two GPUs plain peer loads and
        # stores were measured faster (one remote operand instead of a round trip through the switch for both).
        # ARENO_TP_MULTIMEM=1 forces it wherever a multicast mapping exists, =0 never sets one up.
        self.use_mc = bool(mc) and (self.tp >= 4 or os.environ.get("ARENO_TP_MULTIMEM") == "1")
        self.wait_ms = int(os.environ.get("ARENO_TP_WAIT_MS", "2000"))
        self._arrays = [_ptr_array([b + off for b in bases]) for off in (0, self.off_part, self.off_h, self.off_y)]
        self.desc = TpDesc(self.tp, self.rank, self._arrays[0], self._arrays[1], self._arrays[2], self._arrays[3],
                           (mc + self.off_part) if mc else None, (mc + self.off_h) if mc else None,
                           (mc + self.off_y) if mc else None, self.status.data_ptr(), self.wait_ms)
        local = self.heap.local_base
        self._part = _as_tensor(local + self.off_part, 2 * self.slot_elems, device)
        self._h = _as_tensor(local + self.off_h, 2 * self.slot_elems, device)
        self._y = _as_tensor(local + self.off_y, 2 * self.slot_elems, device)
        self.calls = 0
        logger.info("tp communicator: tp=%d rank=%d heap=%s multicast=%s rows<=%d hidden=%d (%.1f MB per rank)",
                    self.tp, self.rank, self.heap.kind, self.use_mc, self.max_rows, self.hidden, total / 2**20)

    def next_slot(self) -> int:
        slot = self.calls & 1
        self.calls += 1
        return slot

    def one_shot(self, rows: int) -> bool:
        """One flag exchange and every rank reduces all rows itself, or the two-shot reduce-scatter + all-gather?
        One-shot moves ``rows x H`` into each rank with multimem and ``(tp - 1)`` times that with plain loads, against
        ``3 (tp - 1) / tp`` for two-shot.  Measured: one-shot wins between two ranks and for decode-sized calls, which
        are bound by the flag round trip (1.5x NCCL at 128 rows on 8 GPUs); from a few thousand rows on every rank
        pulling every row through the switch loses to the two-shot kernel on plain peer loads (4096 rows on 8 GPUs:
        502 us against 218 us, NCCL 248 us).  ``ARENO_TP_ONESHOT`` = 0 / 1 forces a choice."""
        forced = os.environ.get("ARENO_TP_ONESHOT")
        if forced in ("0", "1"):
            return forced == "1"
        return self.tp == 2 or rows <= 1024

    def multimem(self, rows: int) -> bool:
        """Switch-side reduction for this call?  Only with the one-shot kernel (see ``one_shot``), unless
        ``ARENO_TP_MULTIMEM=1`` asks for it everywhere."""
        if not self.use_mc:
            return False
        return self.one_shot(rows) or os.environ.get("ARENO_TP_MULTIMEM") == "1"

    def partial_view(self, slot: int, rows: int) -> torch.Tensor:
        lo = slot * self.slot_elems
        return self._part[lo: lo + rows * self.hidden].view(rows, self.hidden)

    # ---------------------------------------------------------------------- ops
    def row_linear(self, x: torch.Tensor, weight: torch.Tensor) -> TpPartial:
        """``x [rows, K_local] @ weight[N, K_local]^T`` left as this rank's partial in the heap."""
        rows = x.shape[0]
        if weight.shape[0] != self.hidden or rows > self.max_rows:
            raise ValueError(f"row_linear: output [{rows}, {weight.shape[0]}] does not fit the heap buffers "
                             f"[{self.max_rows}, {self.hidden}]")
        slot = self.next_slot()
        local = self.partial_view(slot, rows)
        gemm_ops.gemm(x, weight, out=local)
        return TpPartial(self, slot, rows, local)

    def new_partial(self, rows: int) -> TpPartial:
        """A fresh slot for a producer that writes its share itself (embedding lookup)."""
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows do not fit the heap buffers ({self.max_rows})")
        slot = self.next_slot()
        return TpPartial(self, slot, rows, self.partial_view(slot, rows))

    def reduce_rmsnorm(self, part: TpPartial, residual, weight, eps: float, w_offset: float = 0.0,
                       want_y: bool = True):
        """Returns ``(y, h)``: ``h = residual + sum over ranks``, ``y = rmsnorm(h) * (weight + w_offset)``.
        Both are views into the heap that stay valid until the call after next."""
        rows, n = part.rows, self.hidden
        lo = part.slot * self.slot_elems
        wf32 = int(weight is not None and weight.dtype == torch.float32)
        if residual is not None and not residual.is_contiguous():
            residual = residual.contiguous()
        _lib.call("areno_tp_reduce_norm", ctypes.addressof(self.desc), lo, _lib.ptr(residual), _lib.ptr(weight), wf32,
                  float(w_offset), int(want_y), rows, n, float(eps), int(self.multimem(rows)), int(self.one_shot(rows)),
                  _lib.stream())
        h = self._h[lo: lo + rows * n].view(rows, n)
        y = self._y[lo: lo + rows * n].view(rows, n) if want_y else None
        return y, h

    @torch.no_grad()
    def self_check(self, rows: int = 192, k_local: int = 512) -> float:
        """One fused row-parallel call on random data against GEMM + NCCL all-reduce + residual RMSNorm in
        PyTorch; returns the relative error of the normalised output (max over the group)."""
        from ..ops import norm as norm_ops

        rows = min(rows, self.max_rows)
        g = torch.Generator(device=self.device).manual_seed(99 + self.rank)
        shared = torch.Generator(device=self.device).manual_seed(5)
        x = torch.randn(rows, k_local, device=self.device, generator=g).to(torch.bfloat16)
        w = (torch.randn(self.hidden, k_local, device=self.device, generator=g) * 0.05).to(torch.bfloat16)
        res = torch.randn(rows, self.hidden, device=self.device, generator=shared).to(torch.bfloat16)
        nw = torch.ones(self.hidden, device=self.device, dtype=torch.bfloat16)
        y, _h = self.reduce_rmsnorm(self.row_linear(x, w), res, nw, 1e-6)
        ref = gemm_ops.gemm(x, w).float()
        dist.all_reduce(ref, group=self.group)
        y_ref = norm_ops.rmsnorm(ref.to(torch.bfloat16), nw, 1e-6, residual=res)
        y_ref = y_ref[0] if isinstance(y_ref, tuple) else y_ref
        err = ((y.float() - y_ref.float()).norm() / y_ref.float().norm().clamp_min(1e-12)).reshape(1)
        dist.all_reduce(err, op=dist.ReduceOp.MAX, group=self.group)
        return float(err)

    def barrier(self) -> None:
        _lib.call("areno_tp_barrier", ctypes.addressof(self.desc), _lib.stream())

    def close(self) -> None:
        self.heap.close()


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
