"""Activation recompute in the decoder stack on the CPU: the same loss and gradients with every layer recomputed, with
the first N layers only and with none; no recompute without gradients or in inference; the per-layer gradient hook
fires from the last layer to the first.  Behaviours follow the reference's ``tests/test_recompute_cpu.py``."""

from __future__ import annotations

import pytest
import torch

from areno_b200.models import dense
from areno_b200.models.dense import DenseCausalLM, TrainMeta, init_weights
from areno_b200.ops.attention import build_varlen_meta
from areno_b200.parallel.context import single_process_context
from tests.helpers import tiny_config


def _model(layers=3):
    single_process_context()
    model = DenseCausalLM(tiny_config(num_hidden_layers=layers))
    init_weights(model, 1)
    return model


def _loss_and_grads(model, meta):
    ids = torch.arange(3, 3 + 11)
    pos = torch.cat([torch.arange(6), torch.arange(5)])
    for p in model.parameters():
        p.grad = None
    out = model(ids, pos, meta)
    loss = out.hidden_states.float().pow(2).mean()
    loss.backward()
    return float(loss.detach()), {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}


def _meta(**kw):
    return TrainMeta(build_varlen_meta([6, 5]), **kw)


def test_recompute_changes_neither_the_loss_nor_any_gradient(monkeypatch):
    model = _model()
    calls = {"n": 0}
    real = dense.checkpoint

    def counting(fn, *a, **k):
        calls["n"] += 1
        return real(fn, *a, **k)

    monkeypatch.setattr(dense, "checkpoint", counting)
    base_loss, base = _loss_and_grads(model, _meta(activation_checkpointing=False))
    assert calls["n"] == 0
    for layers, want_calls in ((None, 3), (2, 2), (0, 0), (9, 3)):
        calls["n"] = 0
        loss, grads = _loss_and_grads(model, _meta(activation_checkpointing=True, checkpoint_layers=layers))
        assert calls["n"] == want_calls, layers
        assert loss == pytest.approx(base_loss, rel=1e-6) and grads.keys() == base.keys()
        for name in base:
            assert torch.allclose(grads[name], base[name], atol=1e-6), (layers, name)


def test_no_recompute_without_gradients_or_in_inference(monkeypatch):
    model = _model(layers=2)
    monkeypatch.setattr(dense, "checkpoint", lambda *a, **k: (_ for _ in ()).throw(AssertionError("recompute used")))
    ids, pos = torch.arange(3, 9), torch.arange(6)
    with torch.no_grad():
        model(ids, pos, TrainMeta(build_varlen_meta([6]), activation_checkpointing=True))


def test_layer_gradient_hook_fires_from_the_last_layer_to_the_first():
    model = _model()
    order = []
    _loss_and_grads(model, _meta(activation_checkpointing=True, checkpoint_layers=1, layer_grad_hook=order.append))
    # the hook of layer i runs when the gradient of its input arrives: every later layer has finished by then.  The
    # first layer's input is the embedding output, whose hook closes the sequence.
    assert order == sorted(order, reverse=True) and set(order) <= {0, 1, 2} and order[0] == 2
    order.clear()
    with torch.no_grad():
        model(torch.arange(3, 9), torch.arange(6), TrainMeta(build_varlen_meta([6]), layer_grad_hook=order.append))
    assert order == []
