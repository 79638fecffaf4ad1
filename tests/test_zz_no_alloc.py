"""The allocation-free RMSNorm backward (`areno_rmsnorm_bwd_static`), driven through the exported C
symbol and compared with the ordinary entry point that takes caller scratch.  Kept in a file of its
own that sorts last: it must hold both on a fresh process and after every other GPU test has used
the library."""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_H = 8192
ERR_H_TOO_LARGE = -10


def _lib():
    from areno_b200.build import ensure_built, kernels_lib_path

    ensure_built()
    lib = ctypes.CDLL(str(kernels_lib_path()))
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    lib.areno_rmsnorm_bwd_static.restype = I
    lib.areno_rmsnorm_bwd_static.argtypes = [P, P, P, I, F, P, P, P, P, I, L, I, P]
    lib.areno_rmsnorm_bwd.restype = I
    lib.areno_rmsnorm_bwd.argtypes = [P, P, P, I, F, P, P, P, P, P, I, L, I, P]
    lib.areno_rmsnorm_bwd_blocks.restype = I
    lib.areno_rmsnorm_bwd_blocks.argtypes = [L]
    lib.areno_no_alloc_strerror.restype = ctypes.c_char_p
    lib.areno_no_alloc_strerror.argtypes = [I]
    return lib


def _case(rows, H, seed, with_res):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g)
    h = mk(rows, H).to(torch.bfloat16)
    dy = mk(rows, H).to(torch.bfloat16)
    w = (1 + 0.1 * mk(H)).to(torch.bfloat16)
    inv = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-6).contiguous()
    dres = mk(rows, H).to(torch.bfloat16) if with_res else None
    return dy, h, w, inv, dres


def _reference(dy, h, w, inv, dres):
    g = dy.float() * w.float()
    hf = h.float()
    c = (g * hf).mean(-1, keepdim=True) * inv[:, None] ** 2
    dx = inv[:, None] * (g - hf * c)
    if dres is not None:
        dx = dx + dres.float()
    dw = (dy.float() * hf * inv[:, None]).sum(0)
    return dx, dw


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _run_both(lib, rows, H, seed, with_res):
    dy, h, w, inv, dres = _case(rows, H, seed, with_res)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # outputs and the ordinary path's scratch are made before the call under test
    dx_s, dx_o = torch.empty_like(h), torch.empty_like(h)
    dw_s = torch.full((H,), float("nan"), device="cuda")
    dw_o = torch.empty(H, device="cuda")
    partial = torch.empty(lib.areno_rmsnorm_bwd_blocks(rows), H, device="cuda")
    torch.cuda.synchronize()
    before = torch.cuda.memory_stats()["allocation.all.allocated"]
    rc = lib.areno_rmsnorm_bwd_static(_ptr(dy), _ptr(h), _ptr(w), 0, 0.0, _ptr(inv), _ptr(dres), _ptr(dx_s), _ptr(dw_s),
                                      0, rows, H, stream)
    assert rc == 0, lib.areno_no_alloc_strerror(rc).decode()
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == before
    rc = lib.areno_rmsnorm_bwd(_ptr(dy), _ptr(h), _ptr(w), 0, 0.0, _ptr(inv), _ptr(dres), _ptr(dx_o), _ptr(partial),
                               _ptr(dw_o), 0, rows, H, stream)
    assert rc == 0
    torch.cuda.synchronize()
    dx_r, dw_r = _reference(dy, h, w, inv, dres)
    assert torch.equal(dx_s, dx_o)
    assert _rel(dw_s, dw_o) < 1e-5
    assert _rel(dx_s, dx_r) < 8e-3 and _rel(dw_s, dw_r) < 8e-3
    return dw_s


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    lib = _lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.areno_rmsnorm_bwd_static(None, None, None, 0, 0.0, None, None, None, None, 0, 0, 4096, stream) == 0
    # a wide, many-row call first, then a narrower one with fewer rows than scratch rows: the second
    # must not pick up anything the first left behind
    _run_both(lib, 1000, 4096, seed=1, with_res=True)
    _run_both(lib, 37, 1024, seed=2, with_res=False)
    _run_both(lib, 300, MAX_H, seed=3, with_res=False)


def test_accumulate_into_dw():
    lib = _lib()
    rows, H = 211, 2048
    dy, h, w, inv, _ = _case(rows, H, 4, False)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    dx = torch.empty_like(h)
    dw = torch.ones(H, device="cuda")
    rc = lib.areno_rmsnorm_bwd_static(_ptr(dy), _ptr(h), _ptr(w), 0, 0.0, _ptr(inv), None, _ptr(dx), _ptr(dw), 1, rows, H,
                                      stream)
    assert rc == 0
    torch.cuda.synchronize()
    _dx_r, dw_r = _reference(dy, h, w, inv, None)
    assert _rel(dw, dw_r + 1.0) < 8e-3


def test_sizes_beyond_the_maximum_are_refused():
    lib = _lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.areno_rmsnorm_bwd_static(None, None, None, 0, 0.0, None, None, None, None, 0, 16, MAX_H + 8, stream)
    assert rc == ERR_H_TOO_LARGE
    assert b"8192" in lib.areno_no_alloc_strerror(rc)
    assert lib.areno_rmsnorm_bwd_static(None, None, None, 0, 0.0, None, None, None, None, 0, 16, 100, stream) == -3
    torch.cuda.synchronize()
