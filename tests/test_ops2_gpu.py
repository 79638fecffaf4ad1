"""GPU numerics: paged KV ops, log-prob, sampler, optimizer and policy-loss kernels."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from areno_b200.ops import _lib, logprob, optim, paged_attention as pa, policy_loss, sampling


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.fixture(autouse=True)
def _status_ok():
    yield
    _lib.check_status()


def _fill_cache(fp8, hq, hkv, d, lens, theta=1e6):
    torch.manual_seed(0)
    dev = "cuda"
    b = len(lens)
    max_pages = (max(lens) + pa.PAGE - 1) // pa.PAGE + 1
    num_pages = b * max_pages + 3
    kc, vc, ks, vs = pa.alloc_kv_cache(num_pages, hkv, d, dev, fp8)
    perm = torch.randperm(num_pages)[: b * max_pages].view(b, max_pages).to(torch.int32)
    block_table = perm.to(dev)
    total = sum(lens)
    qkv = torch.randn(total, (hq + 2 * hkv) * d, device=dev, dtype=torch.bfloat16)
    pos = torch.cat([torch.arange(n) for n in lens]).to(dev, torch.int32)
    slots = torch.cat([perm[i, torch.arange(n) // pa.PAGE].long() * pa.PAGE + torch.arange(n) % pa.PAGE
                       for i, n in enumerate(lens)]).to(dev, torch.int32)
    qkv_ref = qkv.clone().cpu()
    kc_r, vc_r, ks_r, vs_r = pa.alloc_kv_cache(num_pages, hkv, d, "cpu", fp8)
    pa.rope_append_kv(qkv, pos, slots, kc, vc, ks, vs, hq, hkv, d, theta=theta)
    pa.rope_append_kv(qkv_ref, pos.cpu(), slots.cpu(), kc_r, vc_r, ks_r, vs_r, hq, hkv, d, theta=theta)
    return qkv, qkv_ref, (kc, vc, ks, vs), (kc_r, vc_r, ks_r, vs_r), block_table


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("hq,hkv,d", [(28, 4, 128), (8, 8, 64), (32, 2, 128), (8, 2, 256)])
def test_rope_append_and_paged_decode(fp8, hq, hkv, d):
    lens = [1, 63, 64, 65, 300, 1000]
    qkv, qkv_ref, cache, cache_ref, block_table = _fill_cache(fp8, hq, hkv, d, lens)
    assert _rel_err(qkv.cpu(), qkv_ref) < 6e-3
    kc, vc, ks, vs = cache
    deq = pa._dequant(kc, ks).cpu()
    deq_ref = pa._dequant(cache_ref[0], cache_ref[2])
    assert _rel_err(deq, deq_ref) < (7e-2 if fp8 else 6e-3)
    b = len(lens)
    q = torch.randn(b, hq, d, device="cuda", dtype=torch.bfloat16)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    scale = d ** -0.5
    out = pa.paged_decode(q, kc, vc, ks, vs, block_table, seq_lens, scale)
    ref = pa.paged_decode_reference(q, kc, vc, ks, vs, block_table, seq_lens, scale)
    assert _rel_err(out, ref) < 1e-2
    out1 = pa.paged_decode(q, kc, vc, ks, vs, block_table, seq_lens, scale, max_context=200)  # fewer splits
    ref1 = pa.paged_decode_reference(q, kc, vc, ks, vs, block_table, seq_lens.clamp(max=192), scale)
    short = seq_lens <= 192
    assert _rel_err(out1[short], ref1[short]) < 1e-2
    outw = pa.paged_decode(q, kc, vc, ks, vs, block_table, seq_lens, scale, window=100)
    refw = pa.paged_decode_reference(q, kc, vc, ks, vs, block_table, seq_lens, scale, window=100)
    assert _rel_err(outw, refw) < 1e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_selected_logprobs_fwd_bwd(dtype):
    torch.manual_seed(1)
    rows, v = 37, 5000
    base = (3 * torch.randn(rows, v, device="cuda")).to(dtype)
    targets = torch.randint(0, v, (rows,), device="cuda")
    x = base.clone().requires_grad_()
    lp, ent = logprob.selected_logprobs(x, targets, need_entropy=True)
    xr = base.float().clone().requires_grad_()
    lpr = torch.log_softmax(xr, -1).gather(-1, targets[:, None]).squeeze(-1)
    pr = torch.softmax(xr, -1)
    entr = -(pr * torch.log_softmax(xr, -1)).sum(-1)
    assert _rel_err(lp, lpr) < 1e-4
    assert _rel_err(ent, entr) < 1e-3
    g1, g2 = torch.randn(rows, device="cuda"), 0.1 * torch.randn(rows, device="cuda")
    (gx,) = torch.autograd.grad([lp, ent], x, [g1, g2])
    (gr,) = torch.autograd.grad([lpr, entr], xr, [g1, g2])
    assert _rel_err(gx, gr) < (2e-2 if dtype == torch.bfloat16 else 1e-3)


def test_selected_logprobs_vocab_shards_combine():
    torch.manual_seed(2)
    rows, v = 16, 4096
    x = torch.randn(rows, v, device="cuda")
    t = torch.randint(0, v, (rows,), device="cuda")
    full = logprob.selected_logprobs(x, t)
    st = [logprob._stats(x[:, i * 1024:(i + 1) * 1024].contiguous(), t, i * 1024) for i in range(4)]
    m = torch.stack([s[0] for s in st]).max(0).values
    ssum = sum(s[1] * torch.exp(s[0] - m) for s in st)
    tgt = sum(s[3] for s in st)
    assert _rel_err(tgt - (m + torch.log(ssum)), full) < 1e-5


def test_sampler_greedy_and_logprob():
    torch.manual_seed(3)
    x = torch.randn(9, 1000, device="cuda")
    tok, lp = sampling.sample(x, temperature=0.0)
    assert torch.equal(tok, x.argmax(-1))
    ref = torch.log_softmax(x, -1).gather(-1, tok[:, None]).squeeze(-1)
    assert _rel_err(lp, ref) < 1e-5
    xb = x.to(torch.bfloat16)
    tokb, _ = sampling.sample(xb, temperature=0.0)
    assert torch.equal(tokb, xb.float().argmax(-1))


def test_sampler_distribution_matches_softmax():
    torch.manual_seed(4)
    v = 64
    logits = torch.randn(1, v, device="cuda") * 2
    n = 40000
    x = logits.expand(n, v).contiguous()
    uid = torch.arange(n, device="cuda", dtype=torch.int64)
    tok, lp = sampling.sample(x, temperature=0.7, seed=123, row_uid=uid)
    freq = torch.bincount(tok, minlength=v).float() / n
    p = torch.softmax(logits[0] / 0.7, -1)
    assert (freq - p).abs().max().item() < 0.012
    # same key -> same draw; different seed -> different draws
    tok2, _ = sampling.sample(x, temperature=0.7, seed=123, row_uid=uid)
    assert torch.equal(tok, tok2)
    tok3, _ = sampling.sample(x, temperature=0.7, seed=124, row_uid=uid)
    assert not torch.equal(tok, tok3)


def test_sampler_topk_topp_support_and_masks():
    torch.manual_seed(5)
    v = 500
    logits = torch.randn(1, v, device="cuda") * 3
    n = 5000
    x = logits.expand(n, v).contiguous()
    uid = torch.arange(n, device="cuda", dtype=torch.int64)
    tok, _ = sampling.sample(x, temperature=1.0, top_k=5, seed=1, row_uid=uid)
    top5 = set(logits[0].topk(5).indices.tolist())
    assert set(tok.unique().tolist()) <= top5 and len(set(tok.unique().tolist())) >= 3
    tok, _ = sampling.sample(x, temperature=1.0, top_p=0.5, seed=2, row_uid=uid)
    p = torch.softmax(logits[0], -1)
    ps, pi = p.sort(descending=True)
    keep = set(pi[((ps.cumsum(0) - ps) <= 0.5)].tolist())
    assert set(tok.unique().tolist()) <= keep
    # suppression and min-new-tokens EOS masking
    best = int(logits[0].argmax())
    second = int(logits[0].topk(2).indices[1])
    cls = sampling.build_token_classes(v, suppress_ids=[best], eos_ids=[second], device="cuda")
    gen = torch.zeros(n, dtype=torch.int32, device="cuda")
    tok, _ = sampling.sample(x, temperature=0.0, cls=cls, gen_count=gen, min_new=2)
    assert int(tok[0]) not in (best, second)
    gen += 5
    tok, _ = sampling.sample(x, temperature=0.0, cls=cls, gen_count=gen, min_new=2)
    assert int(tok[0]) == second


def test_sampler_shards_combine():
    torch.manual_seed(6)
    b, v, tp = 32, 4096, 4
    x = torch.randn(b, v, device="cuda")
    uid = torch.arange(b, device="cuda", dtype=torch.int64)
    tok, lp = sampling.sample(x, temperature=1.0, seed=77, row_uid=uid)
    parts = torch.empty(tp, b, 6, device="cuda")
    for r in range(tp):
        sampling.sample(x[:, r * 1024:(r + 1) * 1024].contiguous(), temperature=1.0, seed=77, row_uid=uid,
                        vocab_start=r * 1024, part=parts[r])
    tok2, lp2 = sampling.combine_shards(parts)
    assert torch.equal(tok, tok2)
    assert _rel_err(lp2, lp) < 1e-5


def test_adamw_fp32_matches_reference():
    torch.manual_seed(7)
    n = 100003
    p0 = torch.randn(n)
    state = [p0.clone(), torch.zeros(n), torch.zeros(n)]
    dstate = [t.cuda() for t in state]
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    for step in range(1, 4):
        g = torch.randn(n)
        optim.adamw_fp32(*state, g, None, 1e-3, 0.9, 0.999, 1e-8, 0.01, step, 0.5)
        optim.adamw_fp32(*dstate, g.cuda(), out, 1e-3, 0.9, 0.999, 1e-8, 0.01, step, 0.5)
    assert _rel_err(dstate[0].cpu(), state[0]) < 1e-6
    assert _rel_err(dstate[2].cpu(), state[2]) < 1e-4
    assert torch.equal(out.cpu(), dstate[0].cpu().to(torch.bfloat16))


def test_adamw_8bit_tracks_fp32():
    torch.manual_seed(8)
    n = 4096 + 17
    nb = (n + 31) // 32
    p = torch.randn(n, device="cuda")
    ref = [p.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")]
    master = p.clone()
    mq = torch.zeros(n, dtype=torch.int8, device="cuda")
    vq = torch.zeros(n, dtype=torch.uint8, device="cuda")
    ms = torch.full((nb,), 1e-30, device="cuda")
    vs = torch.full((nb,), 1e-30, device="cuda")
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    for step in range(1, 6):
        g = torch.randn(n, device="cuda")
        optim.adamw_fp32(*ref, g, None, 1e-2, 0.9, 0.999, 1e-8, 0.0, step)
        optim.adamw_8bit(master, mq, vq, ms, vs, g, out, 1e-2, 0.9, 0.999, 1e-8, 0.0, step)
    assert _rel_err(master - p, ref[0] - p) < 0.1


def test_sumsq_and_scale():
    x = torch.randn(1_000_003, device="cuda")
    s = optim.sumsq(x)
    assert abs(s.item() - x.double().pow(2).sum().item()) / s.item() < 1e-5
    factor = torch.tensor([0.5], device="cuda")
    y = x.clone()
    optim.scale_(y, 2.0, factor)
    assert torch.allclose(y, x)


@pytest.mark.parametrize("kl_type", [None, "low_var_kl", "kl", "abs", "mse"])
@pytest.mark.parametrize("use_old", [True, False])
def test_policy_loss_tokens(kl_type, use_old):
    torch.manual_seed(9)
    n = 1000
    lp = (-torch.rand(n, device="cuda") * 3).requires_grad_()
    old = (lp.detach() + 0.3 * torch.randn(n, device="cuda")) if use_old else None
    ref = lp.detach() + 0.2 * torch.randn(n, device="cuda")
    adv = torch.randn(n, device="cuda")
    loss, kl, flags = policy_loss.policy_loss_tokens(lp, old, adv, ref, 0.2, 0.2, 3.0, kl_type)
    lpr = lp.detach().clone().requires_grad_()
    lr_, klr, fr = policy_loss.policy_loss_tokens_reference(lpr, old, adv, ref, 0.2, 0.2, 3.0, kl_type)
    assert _rel_err(loss, lr_) < 1e-5
    assert torch.equal(flags, fr.int())
    tot = loss.sum() + (0.1 * kl.sum() if kl is not None else 0.0)
    totr = lr_.sum() + (0.1 * klr.sum() if klr is not None else 0.0)
    (g,) = torch.autograd.grad(tot, lp)
    (gr,) = torch.autograd.grad(totr, lpr)
    assert _rel_err(g, gr) < 1e-4


@pytest.mark.parametrize("rows,n,k", [(64, 3584, 3584), (128, 3584, 18944), (1, 3584, 3584), (64, 1024, 256)])
def test_splitk_partials_residual_rmsnorm(rows, n, k):
    """Skinny GEMM leaving split-K partials + fused fold/residual/RMSNorm == GEMM, add, norm."""
    from areno_b200.ops import gemm, norm

    torch.manual_seed(11)
    x = torch.randn(rows, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.03).to(torch.bfloat16)
    res = torch.randn(rows, n, device="cuda").to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(n, device="cuda")).to(torch.bfloat16)
    part = gemm.gemm_partials(x, w)
    h_ref = ((x.float() @ w.float().t()) + res.float()).to(torch.bfloat16).float()
    y_ref = h_ref * torch.rsqrt(h_ref.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()
    if isinstance(part, gemm.SplitKPartial):
        assert part.splits > 1
        y, h = norm.splitk_residual_rmsnorm(part, res, nw, 1e-6)
    else:
        y, h = norm.rmsnorm(part, nw, 1e-6, residual=res)
    rel = lambda a, b: float((a.float() - b).norm() / b.norm())
    assert rel(h, h_ref) < 8e-3 and rel(y, y_ref) < 8e-3


@pytest.mark.parametrize("m,inter,k,act", [(64, 18944, 3584, "silu"), (300, 1000, 512, "gelu_tanh"), (4096, 4096, 1024, "silu")])
def test_gated_linear_matches_linear_then_activation(m, inter, k, act):
    """The gate / up GEMM with the activation in its epilogue against the two-kernel path (same bf16 rounding
    of the pre-activation, so the results agree to the last bit up to instruction contraction)."""
    from areno_b200.ops import activation, gemm

    torch.manual_seed(11)
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, device="cuda") * k ** -0.5).to(torch.bfloat16)
    with torch.no_grad():
        fused = gemm.gated_linear(x, w, act)
        gu = gemm.linear(x, w)
        ref = activation.silu_and_mul(gu) if act == "silu" else activation.gelu_tanh_and_mul(gu)
    _lib.check_status()
    assert fused.shape == ref.shape == (m, inter)
    assert _rel_err(fused, ref) < 2e-3
    assert float((fused == ref).float().mean()) > 0.99


@pytest.mark.parametrize("hq,hkv,d,bias,norm,rot,fp8", [(28, 4, 128, True, False, 128, False), (8, 2, 128, False, True, 128, True),
                                                     (4, 4, 64, True, True, 32, False)])
def test_fold_rope_append_matches_separate_kernels(hq, hkv, d, bias, norm, rot, fp8):
    """Split-K fold + bias + head norm + rope + KV append in one launch against the kernels it replaces."""
    from areno_b200.ops import attention as attn_ops, gemm

    torch.manual_seed(12)
    t, k = 48, 3584
    n = (hq + 2 * hkv) * d
    x = torch.randn(t, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * k ** -0.5).to(torch.bfloat16)
    b = torch.randn(n, device="cuda").to(torch.bfloat16) if bias else None
    qw = (1 + 0.1 * torch.randn(d, device="cuda")) if norm else None
    kw = (1 + 0.1 * torch.randn(d, device="cuda")) if norm else None
    positions = torch.randint(0, 500, (t,), dtype=torch.int32, device="cuda")
    slots = torch.randperm(4 * pa.PAGE, device="cuda")[:t].to(torch.int32)
    slots[5] = -1
    cache_a = pa.alloc_kv_cache(4, hkv, d, "cuda", fp8)
    cache_b = pa.alloc_kv_cache(4, hkv, d, "cuda", fp8)
    with torch.no_grad():
        ref = gemm.linear(x, w, b)
        if norm:
            q3 = ref[:, : hq * d].unflatten(1, (hq, d))
            k3 = ref[:, hq * d:(hq + hkv) * d].unflatten(1, (hkv, d))
            attn_ops._headnorm_fwd(q3, qw, 0.0, q3, 1e-6)
            attn_ops._headnorm_fwd(k3, kw, 0.0, k3, 1e-6)
        pa.rope_append_kv(ref, positions, slots, *cache_a, hq, hkv, d, theta=1e6, rot_dim=rot)
        part = gemm.gemm_partials(x, w)
        assert isinstance(part, gemm.SplitKPartial) and part.splits > 1
        out = pa.fold_rope_append_kv(part, b, positions, slots, *cache_b, hq, hkv, d, theta=1e6, rot_dim=rot,
                                     q_norm_w=qw, k_norm_w=kw, norm_eps=1e-6)
    _lib.check_status()
    assert _rel_err(out, ref) < 2e-3 and float((out == ref).float().mean()) > 0.98
    for ca, cb in zip(cache_a, cache_b):
        if ca is not None:
            assert _rel_err(cb.float(), ca.float()) < 5e-3


@pytest.mark.parametrize("rows,k,n,valid,softcap", [(300, 512, 1000, 1000, 0.0), (129, 256, 520, 515, 0.0),
                                                    (64, 384, 4104, 4100, 30.0), (5, 128, 256, 256, 0.0)])
def test_lm_head_statistics_from_the_gemm_epilogue(rows, k, n, valid, softcap):
    """Selected-token log-prob and entropy straight from the LM-head GEMM epilogue (no logits tensor) against
    fp32 log_softmax().gather() of the bf16-rounded logits; also as two vocabulary shards that combine."""
    torch.manual_seed(3)
    h = torch.randn(rows, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.2).to(torch.bfloat16)
    t = torch.randint(0, valid, (rows,), device="cuda")
    z = (h.float() @ w.float().t()).to(torch.bfloat16).float()[:, :valid]
    if softcap:
        z = (softcap * torch.tanh(z / softcap)).to(torch.bfloat16).float()
    logp = torch.log_softmax(z, -1)
    lp_ref = logp.gather(-1, t[:, None]).squeeze(-1)
    ent_ref = -(logp.exp() * logp).sum(-1)
    st = logprob.fused_head_stats(h, w, t, 0, valid, softcap)
    lp, lse, ex = logprob._combine(st, None)
    assert _rel_err(lp, lp_ref) < 2e-3
    assert _rel_err(lse - ex, ent_ref) < 2e-3
    if valid == n and n % 16 == 0:
        half = n // 2
        parts = [logprob.fused_head_stats(h, w[i * half:(i + 1) * half].contiguous(), t, i * half, half, softcap)
                 for i in range(2)]
        m = torch.stack([p[0] for p in parts]).max(0).values
        ssum = sum(p[1] * torch.exp(p[0] - m) for p in parts)
        tgt = sum(p[3] for p in parts)
        assert _rel_err(tgt - (m + torch.log(ssum)), lp_ref) < 2e-3
    _lib.check_status()


@pytest.mark.parametrize("softcap", [0.0, 20.0])
def test_lm_head_logprobs_fused_forward_and_gradients(softcap, monkeypatch):
    """``lm_head_logprobs`` (forward from the GEMM epilogue when no logits are kept, backward through recomputed
    logits, soft-cap included) against PyTorch autograd on fp32."""
    from areno_b200.engine.logprobs import lm_head_logprobs
    from areno_b200.models.layers import VocabParallelLMHead
    from areno_b200.parallel.context import single_process_context

    single_process_context("cuda")
    torch.manual_seed(4)
    rows, k, vocab = 200, 256, 1003
    head = VocabParallelLMHead(vocab, k, torch.bfloat16, "cuda")
    with torch.no_grad():
        head.weight.copy_((torch.randn_like(head.weight.float()) * 0.3).to(torch.bfloat16))
    base = torch.randn(rows, k, device="cuda").to(torch.bfloat16)
    t = torch.randint(0, vocab, (rows,), device="cuda")
    g1, g2 = torch.randn(rows, device="cuda"), 0.1 * torch.randn(rows, device="cuda")

    def reference():
        x = base.float().clone().requires_grad_()
        w = head.weight.detach().float().clone().requires_grad_()
        z = (x @ w.t())[:, :vocab]
        if softcap:
            z = softcap * torch.tanh(z / softcap)
        logp = torch.log_softmax(z, -1)
        lp = logp.gather(-1, t[:, None]).squeeze(-1)
        ent = -(logp.exp() * logp).sum(-1)
        gx, gw = torch.autograd.grad([lp, ent], [x, w], [g1, g2])
        return lp.detach(), ent.detach(), gx, gw

    lp_r, ent_r, gx_r, gw_r = reference()
    with torch.no_grad():          # scoring path: statistics from the epilogue
        lp0, ent0 = lm_head_logprobs(head, base, t, chunk=128, need_entropy=True, softcap=softcap or None)
    assert _rel_err(lp0, lp_r) < 5e-3 and _rel_err(ent0, ent_r) < 1e-2
    for keep in ("0", "1"):        # training path with and without the logits kept from forward
        monkeypatch.setenv("ARENO_LOGPROB_KEEP_LOGITS", keep)
        x = base.clone().requires_grad_()
        head.weight.grad = None
        lp, ent = lm_head_logprobs(head, x, t, chunk=128, need_entropy=True, softcap=softcap or None)
        assert _rel_err(lp, lp_r) < 5e-3 and _rel_err(ent, ent_r) < 1e-2
        gx, gw = torch.autograd.grad([lp, ent], [x, head.weight], [g1, g2])
        assert _rel_err(gx, gx_r) < 3e-2 and _rel_err(gw, gw_r) < 3e-2
    _lib.check_status()
