"""GPU numerics of the sm_100a kernels against plain PyTorch fp32 references."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from areno_b200.ops import _lib
from areno_b200.ops import activation, attention, embedding, gemm, norm, rope


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.fixture(autouse=True)
def _status_ok():
    yield
    _lib.check_status()


GEMM_SHAPES = [
    (128, 256, 64), (128, 256, 128), (256, 512, 512), (100, 264, 328), (4096, 3584, 3584), (64, 4608, 3584),
    (1, 1024, 512), (333, 152064 // 8, 256), (512, 96, 1024),
]


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
@pytest.mark.parametrize("bn", [0, 256, 128, 64, 32])
def test_gemm_nt(m, n, k, bn):
    torch.manual_seed(0)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    out = gemm.gemm(a, b, bn=bn)
    assert _rel_err(out, ref) < 6e-3
    out32 = gemm.gemm(a, b, out_dtype=torch.float32, bn=bn)
    assert _rel_err(out32, ref) < 1e-4


@pytest.mark.parametrize("m,n,k", [(256, 512, 384), (4096, 3584, 1024), (200, 328, 264), (64, 3584, 4608)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, True), (True, False)])
@pytest.mark.parametrize("bn", [0, 256, 128, 64])
def test_gemm_majors(m, n, k, a_mn, b_mn, bn):
    torch.manual_seed(1)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    a_in = a.t().contiguous() if a_mn else a
    b_in = b.t().contiguous() if b_mn else b
    out = gemm.gemm(a_in, b_in, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32, bn=bn)
    assert _rel_err(out, ref) < 1e-4


def test_gemm_bias_and_accumulate():
    torch.manual_seed(2)
    a = torch.randn(300, 512, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(264, 512, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(264, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    out = gemm.gemm(a, b, bias=bias)
    assert _rel_err(out, ref + bias.float()) < 6e-3
    acc = torch.ones(300, 264, device="cuda", dtype=torch.float32)
    gemm.gemm(a, b, out=acc, accumulate=True)
    assert _rel_err(acc, ref + 1.0) < 1e-4


def test_gemm_tail_wave_split_epilogues():
    """448 output tiles on 148 SMs: the last 4 tiles are cut along K and folded by the tail kernel; every
    epilogue (bf16 + bias, fp32 store, fp32 accumulate) must survive that path, twice in a row (shared scratch)."""
    torch.manual_seed(21)
    a = torch.randn(4096, 512, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(3584, 512, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(3584, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    for _ in range(2):
        assert _rel_err(gemm.gemm(a, b, bias=bias), ref + bias.float()) < 6e-3
        acc = torch.ones(4096, 3584, device="cuda", dtype=torch.float32)
        gemm.gemm(a, b, out=acc, accumulate=True)
        assert _rel_err(acc, ref + 1.0) < 1e-4
        # weight-gradient layout: both operands MN-major
        acc2 = torch.zeros(4096, 3584, device="cuda", dtype=torch.float32)
        gemm.gemm(a.t().contiguous(), b.t().contiguous(), a_mn=True, b_mn=True, out=acc2, accumulate=True)
        assert _rel_err(acc2, ref) < 1e-4
    _lib.check_status()


def test_linear_autograd_matches_reference():
    torch.manual_seed(3)
    x = torch.randn(4, 96, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(328, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    bias = torch.randn(328, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = gemm.linear(x, w, bias)
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf, bf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_(), bias.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xf, wf, bf)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 6e-3
    assert _rel_err(x.grad, xf.grad) < 6e-3
    assert _rel_err(w.grad, wf.grad) < 6e-3
    assert _rel_err(bias.grad, bf.grad) < 6e-3


def test_linear_main_grad_fusion():
    torch.manual_seed(4)
    x = torch.randn(200, 256, device="cuda", dtype=torch.bfloat16)
    w = torch.nn.Parameter(torch.randn(128, 256, device="cuda", dtype=torch.bfloat16))
    w.main_grad = torch.zeros(128, 256, device="cuda", dtype=torch.float32)
    for _ in range(2):
        y = gemm.linear(x, w)
        y.backward(torch.ones_like(y))
    ref = 2 * torch.ones(200, 128, device="cuda").t() @ x.float()
    assert w.grad is None
    assert _rel_err(w.main_grad, ref) < 1e-4


@pytest.mark.parametrize("rows,h", [(7, 128), (513, 3584), (64, 4096), (33, 2048), (1000, 64)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(rows, h, with_res):
    torch.manual_seed(5)
    x = torch.randn(rows, h, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(h, device="cuda")).to(torch.bfloat16).requires_grad_()
    res = torch.randn(rows, h, device="cuda", dtype=torch.bfloat16, requires_grad=True) if with_res else None
    out = norm.rmsnorm(x, w, 1e-6, residual=res)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    rr = res.detach().float().requires_grad_() if with_res else None
    hr = xr + rr if with_res else xr
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    if with_res:
        y, hnew = out
        g, gh = torch.randn_like(y), torch.randn_like(hnew)
        torch.autograd.backward([y, hnew], [g, gh])
        torch.autograd.backward([yr, hr], [g.float(), gh.float()])
        assert _rel_err(hnew, hr) < 5e-3
        assert _rel_err(res.grad, rr.grad) < 8e-3
    else:
        y = out
        g = torch.randn_like(y)
        y.backward(g)
        yr.backward(g.float())
    assert _rel_err(y, yr) < 5e-3
    assert _rel_err(x.grad, xr.grad) < 8e-3
    assert _rel_err(w.grad, wr.grad) < 8e-3


@pytest.mark.parametrize("kind", ["silu", "gelu_tanh"])
def test_gated_act(kind):
    torch.manual_seed(6)
    x = torch.randn(77, 2 * 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    f = activation.silu_and_mul if kind == "silu" else activation.gelu_tanh_and_mul
    y = f(x)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    a, b = xr.chunk(2, -1)
    act = torch.nn.functional.silu(a) if kind == "silu" else torch.nn.functional.gelu(a, approximate="tanh")
    yr = act * b
    yr.backward(g.float())
    assert _rel_err(y, yr) < 5e-3
    assert _rel_err(x.grad, xr.grad) < 8e-3


@pytest.mark.parametrize("name", ["silu", "sigmoid", "softplus"])
def test_unary(name):
    x = (4 * torch.randn(1000, device="cuda")).to(torch.bfloat16).requires_grad_()
    y = getattr(activation, name)(x)
    y.backward(torch.ones_like(y))
    xr = x.detach().float().requires_grad_()
    fr = {"silu": torch.nn.functional.silu, "sigmoid": torch.sigmoid,
          "softplus": lambda t: torch.nn.functional.softplus(t, threshold=20.0)}[name]
    yr = fr(xr)
    yr.backward(torch.ones_like(yr))
    assert _rel_err(y, yr) < 5e-3
    assert _rel_err(x.grad, xr.grad) < 8e-3


@pytest.mark.parametrize("rot,interleaved", [(128, False), (64, False), (128, True)])
def test_rope(rot, interleaved):
    torch.manual_seed(7)
    x = torch.randn(50, 6, 128, device="cuda", dtype=torch.bfloat16)
    pos = torch.randint(0, 4000, (50,), device="cuda", dtype=torch.int32)
    ref = rope.rope_reference(x, pos, 1e6, rot, None, interleaved)
    out = rope.apply_rope(x.clone(), pos, 1e6, rot, None, interleaved)
    assert _rel_err(out, ref) < 6e-3


def test_embedding():
    torch.manual_seed(8)
    table = torch.nn.Parameter(torch.randn(100, 64, device="cuda", dtype=torch.bfloat16))
    ids = torch.randint(0, 200, (4, 33), device="cuda")
    out = embedding.embedding(ids, table, vocab_start=50)
    ref = embedding.embedding_reference(ids, table.detach(), 50)
    assert torch.equal(out, ref)
    g = torch.randn_like(out)
    out.backward(g)
    tr = table.detach().float().requires_grad_()
    mask = ((ids >= 50) & (ids < 150)).unsqueeze(-1)
    outr = torch.nn.functional.embedding((ids - 50).clamp(0, 99), tr) * mask
    outr.backward(g.float())
    assert _rel_err(table.grad, tr.grad) < 6e-3


ATTN_CASES = [
    # (q_lens, k_lens, hq, hkv, d, causal, window)
    ([64], None, 2, 2, 128, True, 0),
    ([37, 129, 5], None, 4, 2, 128, True, 0),
    ([300, 77], None, 7, 1, 128, True, 0),
    ([100, 200], None, 4, 4, 64, True, 0),
    ([16, 40], [80, 40], 4, 2, 128, True, 0),
    ([150], None, 2, 1, 128, False, 0),
    ([260, 90], None, 2, 1, 128, True, 96),
    ([1000, 513, 128, 1], None, 8, 2, 128, True, 0),   # many key tiles: every ring / phase of the tcgen05 forward
    ([700], [1500], 4, 1, 128, True, 0),               # chunked prefill shape: queries see a cached prefix
    ([700, 130, 64], None, 8, 2, 64, True, 0),         # head size 64 on the tcgen05 forward
    ([300], [900], 4, 4, 64, False, 0),
    ([100, 200], None, 4, 2, 256, True, 0),      # head_dim 256: backward runs as two 128-column CTAs
    ([260, 90], [300, 90], 2, 1, 256, True, 96),
]


@pytest.mark.parametrize("q_lens,k_lens,hq,hkv,d,causal,window", ATTN_CASES)
def test_attention_fwd_bwd(q_lens, k_lens, hq, hkv, d, causal, window):
    torch.manual_seed(9)
    meta = attention.build_varlen_meta(q_lens, k_lens, device="cuda")
    q = torch.randn(meta.total_q, hq, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(meta.total_k, hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(meta.total_k, hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    scale = d ** -0.5
    o = attention.varlen_attention(q, k, v, meta, scale, causal, window)
    g = torch.randn_like(o)
    o.backward(g)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    orf = attention._reference_autograd(qr, kr, vr, meta, scale, causal, window)
    orf.backward(g.float())
    assert _rel_err(o, orf) < 8e-3
    assert _rel_err(q.grad, qr.grad) < 1.5e-2
    assert _rel_err(k.grad, kr.grad) < 1.5e-2
    assert _rel_err(v.grad, vr.grad) < 1.5e-2


def test_qkv_attention_packed():
    torch.manual_seed(10)
    hq, hkv, d = 4, 2, 128
    meta = attention.build_varlen_meta([70, 130], device="cuda")
    t = meta.total_q
    qkv = torch.randn(t, (hq + 2 * hkv) * d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    pos = torch.cat([torch.arange(70), torch.arange(130)]).to("cuda", torch.int32)
    out = attention.qkv_attention(qkv.clone(), pos, meta, hq, hkv, d, theta=1e6)
    g = torch.randn_like(out)
    (gin,) = torch.autograd.grad(out, qkv, g)
    qkv_r = qkv.detach().float().cpu().requires_grad_()
    meta_c = attention.build_varlen_meta([70, 130])
    out_r = attention.qkv_attention(qkv_r, pos.cpu(), meta_c, hq, hkv, d, theta=1e6)
    (gr,) = torch.autograd.grad(out_r, qkv_r, g.float().cpu())
    assert _rel_err(out.cpu(), out_r) < 1e-2
    assert _rel_err(gin.cpu(), gr) < 2e-2
