"""Selected-token log-probs and entropy of the LM head on the CPU: against a full softmax, under row chunking, with a
padded vocabulary shard and logit soft-capping, gradients against cross entropy, and the vocabulary-parallel form on
two gloo ranks against the single-process values.  Behaviours follow the reference's ``tests/test_logprobs_cpu.py``."""

from __future__ import annotations

import os
import socket
import traceback

import pytest
import torch
import torch.multiprocessing as mp

from areno_b200.engine.logprobs import lm_head_logprobs
from areno_b200.ops.logprob import selected_logprobs_reference
from areno_b200.parallel.context import single_process_context


def _head(vocab, hidden, seed=0):
    from areno_b200.models.layers import VocabParallelLMHead

    head = VocabParallelLMHead(vocab, hidden, torch.float32, "cpu")
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        head.weight.copy_(torch.randn(head.weight.shape, generator=g) * 0.5)
    return head


def _case(rows=10, vocab=13, hidden=8, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(rows, hidden, generator=g), torch.randint(0, vocab, (rows,), generator=g)


@pytest.fixture(autouse=True)
def _ctx():
    single_process_context()


def test_logprobs_and_entropy_match_a_full_softmax_over_the_real_vocabulary():
    head = _head(13, 8)                               # the shard is padded to 16 rows: 3 columns are not vocabulary
    assert head.per_rank == 16 and head.valid_local == 13
    hidden, targets = _case()
    lp, ent = lm_head_logprobs(head, hidden, targets, need_entropy=True)
    logp = torch.log_softmax(hidden @ head.weight[:13].T, -1)
    assert torch.allclose(lp, logp.gather(-1, targets[:, None]).squeeze(-1), atol=1e-6)
    assert torch.allclose(ent, -(logp.exp() * logp).sum(-1), atol=1e-6)
    assert lp.dtype == torch.float32 and lp.shape == (10,)
    only_lp = lm_head_logprobs(head, hidden, targets)
    assert torch.equal(only_lp, lp)


def test_row_chunking_does_not_change_values_or_gradients():
    head = _head(13, 8)
    hidden, targets = _case()
    outs = []
    for chunk in (3, 4096):
        h = hidden.clone().requires_grad_(True)
        head.weight.grad = None
        lp, ent = lm_head_logprobs(head, h, targets, chunk=chunk, need_entropy=True)
        (lp.sum() + 0.1 * ent.sum()).backward()
        outs.append((lp.detach(), ent.detach(), h.grad.clone(), head.weight.grad.clone()))
    for a, b in zip(*outs):
        assert torch.allclose(a, b, atol=1e-6)


def test_gradient_is_the_cross_entropy_gradient():
    head = _head(13, 8)
    hidden, targets = _case()
    h1 = hidden.clone().requires_grad_(True)
    (-lm_head_logprobs(head, h1, targets).mean()).backward()
    g_w = head.weight.grad.clone()
    head.weight.grad = None
    h2 = hidden.clone().requires_grad_(True)
    torch.nn.functional.cross_entropy(h2 @ head.weight[:13].T, targets).backward()
    assert torch.allclose(h1.grad, h2.grad, atol=1e-6) and torch.allclose(g_w, head.weight.grad, atol=1e-6)
    assert torch.count_nonzero(g_w[13:]) == 0                        # padding rows of the shard get no gradient


def test_soft_capping_is_applied_before_the_softmax():
    head = _head(13, 8)
    hidden, targets = _case()
    lp = lm_head_logprobs(head, hidden * 4, targets, softcap=5.0)
    logits = torch.tanh((hidden * 4) @ head.weight[:13].T / 5.0) * 5.0
    want = torch.log_softmax(logits, -1).gather(-1, targets[:, None]).squeeze(-1)
    assert torch.allclose(lp, want, atol=1e-6)
    assert not torch.allclose(lp, lm_head_logprobs(head, hidden * 4, targets), atol=1e-3)


def test_int32_targets_and_no_rows():
    head = _head(13, 8)
    hidden, targets = _case()
    assert torch.equal(lm_head_logprobs(head, hidden, targets.int()), lm_head_logprobs(head, hidden, targets))
    x = torch.randn(4, 6)
    assert selected_logprobs_reference(x[:0], torch.zeros(0, dtype=torch.long)).shape == (0,)


def test_reference_statistics_of_a_shard_window():
    """A rank's shard contributes the target's logit only when the target lies inside its window."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(5, 12, generator=g)
    t = torch.tensor([0, 5, 6, 11, 3])
    full_lp, full_ent = selected_logprobs_reference(x, t, 0, None, True)
    logp = torch.log_softmax(x, -1)
    assert torch.allclose(full_lp, logp.gather(-1, t[:, None]).squeeze(-1), atol=1e-6)
    assert torch.allclose(full_ent, -(logp.exp() * logp).sum(-1), atol=1e-6)
    # outside the window the "target logit" term is zero, so the value is minus the shard's log-sum-exp
    right = selected_logprobs_reference(x[:, 6:], t, 6)
    assert torch.allclose(right[:2], -torch.logsumexp(x[:2, 6:], -1), atol=1e-6)
    assert torch.allclose(right[2], x[2, 6] - torch.logsumexp(x[2, 6:], -1), atol=1e-6)


# ---------------------------------------------------------------------------------------- two gloo ranks

def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, ret):
    try:
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        from areno_b200.models.layers import VocabParallelLMHead
        from areno_b200.parallel.context import destroy_parallel, init_parallel

        init_parallel(rank, world, tp_size=2, master_port=port, backend="gloo", device=torch.device("cpu"), timeout_s=120)
        vocab, hidden_size = 21, 8                    # 11 -> 16 rows per rank; rank 1 holds 5 real rows
        full = _head(vocab, hidden_size)              # built under the TP context: local shapes
        g = torch.Generator().manual_seed(0)
        whole = torch.randn(32, hidden_size, generator=g) * 0.5          # the same "full" weight on both ranks
        head = VocabParallelLMHead(vocab, hidden_size, torch.float32, "cpu")
        assert head.per_rank == 16 and head.valid_local == (16 if rank == 0 else 5) and full.per_rank == 16
        with torch.no_grad():
            head.weight.zero_()
            head.weight[: head.valid_local].copy_(whole[head.vocab_start: head.vocab_start + head.valid_local])
        hidden, targets = _case(rows=9, vocab=vocab, hidden=hidden_size, seed=4)
        h = hidden.clone().requires_grad_(True)
        lp, ent = lm_head_logprobs(head, h, targets, chunk=4, need_entropy=True)
        (lp.sum() + 0.3 * ent.sum()).backward()
        ret[rank] = dict(lp=lp.detach(), ent=ent.detach(), dh=h.grad.clone(), dw=head.weight.grad.clone(),
                         start=head.vocab_start, valid=head.valid_local, whole=whole)
        destroy_parallel()
    except BaseException:  # noqa: BLE001
        ret[rank] = traceback.format_exc()


def test_vocabulary_parallel_values_and_gradients_match_one_process():
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    procs = [mp.get_context("spawn").Process(target=_rank_main, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    out = [ret.get(r) for r in range(2)]
    for o in out:
        assert isinstance(o, dict), o
    whole = out[0]["whole"][:21]
    hidden, targets = _case(rows=9, vocab=21, hidden=8, seed=4)
    h = hidden.clone().requires_grad_(True)
    w = whole.clone().requires_grad_(True)
    logp = torch.log_softmax(h @ w.T, -1)
    lp = logp.gather(-1, targets[:, None]).squeeze(-1)
    ent = -(logp.exp() * logp).sum(-1)
    (lp.sum() + 0.3 * ent.sum()).backward()
    for o in out:
        assert torch.allclose(o["lp"], lp.detach(), atol=1e-5) and torch.allclose(o["ent"], ent.detach(), atol=1e-5)
        lo, n = o["start"], o["valid"]
        assert torch.allclose(o["dw"][:n], w.grad[lo:lo + n], atol=1e-5) and torch.count_nonzero(o["dw"][n:]) == 0
    # each rank holds the hidden gradient through its own shard; the row-parallel seam sums them
    assert torch.allclose(out[0]["dh"] + out[1]["dh"], h.grad, atol=1e-5)
