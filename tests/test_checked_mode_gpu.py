"""One GPU, ``ARENO_BOUNDS_CHECK=1``: the checked mode validates every data-dependent index on the host before the
kernel that would use it is launched, so a bad index becomes a Python exception naming the operand and never reaches
the GPU.  The mode is read at import time, hence the child interpreter."""

from __future__ import annotations

import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import torch
    from areno_b200.ops import _lib, gemm, paged_attention as pa
    assert _lib.BOUNDS_CHECK
    dev = "cuda"
    hq, hkv, d, pages = 4, 2, 64, 8
    kc, vc, ks, vs = pa.alloc_kv_cache(pages, hkv, d, dev)
    qkv = torch.randn(3, (hq + 2 * hkv) * d, device=dev).to(torch.bfloat16)
    pos = torch.tensor([0, 1, 2], dtype=torch.int32, device=dev)
    good = torch.tensor([0, 65, -1], dtype=torch.int32, device=dev)
    pa.rope_append_kv(qkv.clone(), pos, good, kc, vc, ks, vs, hq, hkv, d)
    bad = torch.tensor([0, pages * pa.PAGE, 5], dtype=torch.int32, device=dev)      # one slot past the cache
    try:
        pa.rope_append_kv(qkv.clone(), pos, bad, kc, vc, ks, vs, hq, hkv, d)
        raise SystemExit("out-of-range slot was not caught")
    except IndexError as exc:
        assert "slot_mapping" in str(exc) and "max 512" in str(exc), exc
    q = torch.randn(2, hq, d, device=dev).to(torch.bfloat16)
    table = torch.tensor([[1, 2, 99], [3, 99, 99]], dtype=torch.int32, device=dev)    # 99 only in unused entries
    lens = torch.tensor([100, 10], dtype=torch.int32, device=dev)
    pa.paged_decode(q, kc, vc, ks, vs, table, lens, 0.125)
    try:
        pa.paged_decode(q, kc, vc, ks, vs, table, torch.tensor([190, 10], dtype=torch.int32, device=dev), 0.125)
        raise SystemExit("page id past the cache was not caught")
    except IndexError as exc:
        assert "block_table" in str(exc), exc
    # the split-K workspace carries a canary that a well-behaved GEMM leaves alone
    a = torch.randn(16, 4096, device=dev).to(torch.bfloat16)
    w = torch.randn(256, 4096, device=dev).to(torch.bfloat16)
    for _ in range(3):
        out = gemm.gemm(a, w)
    torch.cuda.synchronize()
    assert torch.allclose(out.float(), a.float() @ w.float().t(), rtol=3e-2, atol=1.0)
    _lib.check_canary("GEMM split-K workspace", gemm._WORKSPACES[0])
    _lib.check_status()
    print("checked mode ok")
""")


def test_checked_mode_catches_bad_indices_before_launch():
    env = dict(os.environ, ARENO_BOUNDS_CHECK="1", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0 and "checked mode ok" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-4000:]


def test_smoke_step_passes_under_checked_mode():
    """The flagship rollout + GRPO step with every index check switched on."""
    env = dict(os.environ, ARENO_BOUNDS_CHECK="1", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.run([sys.executable, "-c", "import __graft_entry__ as g; g.smoke()"], env=env, cwd=ROOT,
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0 and "smoke ok" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-4000:]
