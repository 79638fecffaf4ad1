"""Randomised schedules through the inference engine on the CPU: requests of random lengths and budgets arrive at random
steps, slots, prefill budget and page pool are small enough to force queueing, chunked prefill and evictions.  Greedy
tokens must equal what the model generates for each prompt on its own with a full forward pass every step, whatever
the schedule was; stop tokens end a sequence exactly where the stand-alone generation meets one.  Every model family
takes the same walks (their per-slot state has to survive slot reuse and evictions), and two equivalences that the
families' own state handling could break are checked for all of them: a packed training batch against its sequences
one by one, and gradients with and without recomputed layers."""

from __future__ import annotations

import random

import pytest
import torch

from areno_b200.engine.inference import InferenceEngine, SamplingParams
from areno_b200.models.dense import DenseCausalLM, TrainMeta, init_weights
from areno_b200.ops.attention import build_varlen_meta
from areno_b200.parallel.context import single_process_context
from tests.helpers import tiny_config


@pytest.fixture(autouse=True)
def _fp32_pages(monkeypatch):
    """KV pages in fp32 instead of bf16: the comparison is about scheduling and state, not about page precision."""
    from areno_b200.ops import paged_attention as pa

    def fp32_pages(num_pages, kv_heads, head_dim, device, fp8=False):
        shape = (num_pages, kv_heads, pa.PAGE, head_dim)
        return torch.zeros(shape, device=device), torch.zeros(shape, device=device), None, None

    monkeypatch.setattr(pa, "alloc_kv_cache", fp32_pages)


def _dense():
    m = DenseCausalLM(tiny_config())
    init_weights(m, 7)
    return m


def _hybrid():
    """Softmax attention interleaved with gated delta rule layers: convolution and recurrent state per engine slot,
    which must be reset when a slot is reused and rebuilt when an evicted sequence is prefilled again."""
    from areno_b200.models.hybrid import HybridCausalLM
    from tests.test_hybrid_cpu import hybrid_config

    m = HybridCausalLM(hybrid_config())
    init_weights(m, 7)
    with torch.no_grad():
        for layer in m._linear_layers():
            layer.attn.A_log.fill_(-1.0)
            layer.attn.dt_bias.fill_(0.5)
    return m


def _bailing():
    """Decayed linear attention (a running state per slot) next to softmax attention and a grouped sigmoid router."""
    from tests.test_bailing_cpu import _model, bailing_config

    return _model(bailing_config(), seed=7)


def _gemma4():
    """Sliding-window and global layers with their own head geometry, tail layers that share the KV of earlier ones,
    per-layer input embeddings, dense + MoE feed-forward, soft-capped logits."""
    from tests.test_gemma4_cpu import _model, gemma_config

    return _model(gemma_config(), seed=7)


def _moe():
    from areno_b200.models import registry
    from tests.test_moe_cpu import moe_config

    adapter = registry.get_adapter("qwen3_moe")
    m = adapter.build(moe_config())
    adapter.init_random(m, 7)
    return m


@pytest.fixture(scope="module", params=["dense", "hybrid", "bailing", "gemma4", "moe"])
def model(request):
    single_process_context()
    return {"dense": _dense, "hybrid": _hybrid, "bailing": _bailing, "gemma4": _gemma4, "moe": _moe}[request.param]()


def _alone(model, prompt, max_new, stop):
    """Greedy continuation by full forward passes; the stop token is kept, as the engine keeps it."""
    toks = []
    with torch.no_grad():
        for _ in range(max_new):
            toks.append(int(_logits(model, prompt + toks)[-1].argmax(-1)))
            if toks[-1] in stop:
                return toks, "stop"
    return toks, "length"


def _logits(model, tokens):
    ids = torch.tensor(tokens)
    with torch.no_grad():
        h = model(ids, torch.arange(len(ids)), TrainMeta(build_varlen_meta([len(ids)]), False)).hidden_states
        return model.compute_logits(h).float()


# Cached and stand-alone passes add numbers in different orders: a token whose logit is within this margin of the best
# one counts as the greedy choice (random-init logits have many near-ties).
NEAR_TIE = 2e-3


def _run_and_check(model, reqs, *, slots, budget, num_pages, stop, arrivals, tag):
    """Drive the engine step by step with the given arrivals and check every finished request against the model run on
    its own.  Returns how many sequences were evicted for lack of pages and resumed."""
    n_req = len(reqs)
    longest = max(len(p) + n for p, n in reqs)
    eng = InferenceEngine(model, 512, "cpu", max_slots=slots, max_model_len=(longest + 63) // 64 * 64,
                          max_prefill_tokens=budget, num_pages=num_pages)
    eng.begin(SamplingParams(temperature=0.0), stop, 16)
    arrivals = sorted(arrivals)
    rid_of, finished, step = {}, {}, 0
    while len(finished) < n_req:
        while arrivals and arrivals[0][0] <= step:
            _, i = arrivals.pop(0)
            rid_of[eng.add_request(reqs[i][0], reqs[i][1])] = i
        for req in eng.step():
            finished[rid_of[req.rid]] = req
        step += 1
        assert step < 3000, "the engine stopped making progress"
    exact = 0
    for i, (prompt, max_new) in enumerate(reqs):
        got = finished[i]
        want, _reason = _alone(model, prompt, max_new, stop)
        exact += got.tokens == want
        # every token is the greedy choice given the tokens before it, up to near-ties
        logits = _logits(model, prompt + got.tokens)[len(prompt) - 1:-1]
        chosen = logits.gather(-1, torch.tensor(got.tokens)[:, None]).squeeze(-1)
        assert bool((chosen >= logits.max(-1).values - NEAR_TIE).all()), (tag, i, len(prompt), max_new)
        # and it ended where it had to: at its first stop token, or at its budget without having met one
        if got.reason == "stop":
            assert got.tokens[-1] in stop and not set(got.tokens[:-1]) & set(stop) and len(got.tokens) <= max_new
        else:
            assert got.reason == "length" and len(got.tokens) == max_new and not set(got.tokens) & set(stop)
        ref_lp = torch.log_softmax(logits, -1).gather(-1, torch.tensor(got.tokens)[:, None]).squeeze(-1)
        assert torch.allclose(ref_lp, torch.tensor(got.logprobs), atol=3e-3)
    assert exact >= n_req // 2                 # near-ties are rare: most requests match token for token
    assert eng.idle and eng.sched.num_free_pages == num_pages
    return sum(1 for r in eng._requests.values() if r.kept_tokens)


@pytest.mark.parametrize("seed", range(8))
def test_any_schedule_gives_the_stand_alone_greedy_tokens(model, seed):
    single_process_context()
    rng = random.Random(seed)
    slots = rng.choice([2, 3, 4])
    budget = rng.choice([16, 32, 64])
    n_req = rng.randint(4, 8)
    reqs = [([rng.randrange(3, 512) for _ in range(rng.randint(2, 90))], rng.randint(1, 14)) for _ in range(n_req)]
    per_seq = (max(len(p) + n for p, n in reqs) + 63) // 64
    num_pages = rng.choice([per_seq + 1, per_seq * 2, per_seq * slots])
    # a stop token that some stand-alone generation actually produces, so that both finish reasons occur
    probe, _ = _alone(model, reqs[0][0], reqs[0][1], ())
    stop = (probe[len(probe) // 2],) if rng.random() < 0.7 else ()
    arrivals = [(rng.randint(0, 25), i) for i in range(n_req)]
    _run_and_check(model, reqs, slots=slots, budget=budget, num_pages=num_pages, stop=stop, arrivals=arrivals, tag=seed)


@pytest.mark.parametrize("seed", range(3))
def test_sequences_that_outgrow_a_tight_page_pool_are_evicted_and_resume(model, seed):
    """Prompts that end just below a page boundary, three of them decoding at once over four pages: when they cross
    the boundary together there is no page for everybody, some go back to the queue with what they have generated and
    are prefilled again later (for the stateful families: with their recurrent state rebuilt from those tokens)."""
    single_process_context()
    rng = random.Random(100 + seed)
    reqs = [([rng.randrange(3, 512) for _ in range(rng.randint(58, 62))], rng.randint(10, 14)) for _ in range(5)]
    evicted = _run_and_check(model, reqs, slots=3, budget=64, num_pages=4, stop=(), arrivals=[(0, i) for i in range(5)],
                             tag=("tight", seed))
    assert evicted >= 1


def test_a_packed_training_batch_equals_every_sequence_on_its_own(model):
    """Variable-length packing must not leak anything across sequence boundaries: not attention, not a sliding window,
    and not the convolution or recurrent state of the linear-attention families."""
    single_process_context()
    g = torch.Generator().manual_seed(11)
    lens = [9, 1, 23, 14]
    rows = [torch.randint(3, 512, (n,), generator=g) for n in lens]
    ids = torch.cat(rows)
    pos = torch.cat([torch.arange(n) for n in lens])
    with torch.no_grad():
        packed = model(ids, pos, TrainMeta(build_varlen_meta(lens), False)).hidden_states
        k = 0
        for row in rows:
            n = len(row)
            alone = model(row, torch.arange(n), TrainMeta(build_varlen_meta([n]), False)).hidden_states
            assert torch.allclose(packed[k:k + n], alone, atol=2e-5), (n, float((packed[k:k + n] - alone).abs().max()))
            k += n


def test_recompute_reproduces_the_gradients_of_every_family(model):
    """Layers that are recomputed in backward must rebuild exactly what they produced in forward, including routing
    decisions and the scans of the linear-attention layers."""
    single_process_context()
    g = torch.Generator().manual_seed(12)
    lens = [10, 17]
    ids = torch.randint(3, 512, (sum(lens),), generator=g)
    pos = torch.cat([torch.arange(n) for n in lens])

    def grads(ckpt):
        for p in model.parameters():
            p.grad = None
        model.train()
        out = model(ids, pos, TrainMeta(build_varlen_meta(lens), activation_checkpointing=ckpt))
        loss = out.hidden_states.float().pow(2).mean()
        loss.backward()
        model.eval()
        return float(loss.detach()), {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}

    base_loss, base = grads(False)
    loss, got = grads(True)
    assert loss == pytest.approx(base_loss, rel=1e-6) and got.keys() == base.keys() and len(base) > 4
    for name in base:
        assert torch.allclose(got[name], base[name], atol=1e-6, rtol=1e-4), name
    for p in model.parameters():
        p.grad = None
