"""Two gloo ranks on CPU: the hybrid (softmax + Gated DeltaNet) families at tensor-parallel size 2 must
reproduce the single-process model: same hidden states from a checkpoint cut into shards at load, same
gradients (shard by shard, replicated ones after the TP sum), same greedy tokens from cached inference, and a
checkpoint saved from the shards that equals the one they were loaded from.  The gradient norm the sharded
optimizer computes after its TP reductions is compared as well (for the plain dense and MoE families too): it is
one number that is wrong as soon as any replicated parameter is summed when it should not be, or the reverse."""

from __future__ import annotations

import os
import socket
import traceback

import pytest
import torch
import torch.multiprocessing as mp

from areno_b200.parallel.context import single_process_context

from .test_hybrid_cpu import hybrid_config


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _variant(name: str):
    if name == "dense":
        return hybrid_config()
    if name == "kv_replicated":       # one KV head shared by both ranks, untied head (vocab-parallel lm_head)
        return hybrid_config(num_key_value_heads=1, tie_word_embeddings=False)
    return hybrid_config(model_type="qwen3_5_moe", num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
                         shared_expert_intermediate_size=48, norm_topk_prob=True, extra={"shared_expert_gate": True})


def _run(model, ids, lens):
    from areno_b200.models.dense import TrainMeta
    from areno_b200.ops.attention import build_varlen_meta

    pos = torch.cat([torch.arange(n) for n in lens])
    h = model(ids, pos, TrainMeta(build_varlen_meta(lens), False)).hidden_states
    loss = h.float().pow(2).mean()      # logits are vocab-sharded under TP; the greedy tokens cover the head
    loss.backward()
    return h.detach(), float(loss.detach())


def _optimizer_grad_norm(model) -> float:
    from areno_b200.engine.config import OptimizerConfig
    from areno_b200.engine.optim import ShardedAdamW

    opt = ShardedAdamW(model, OptimizerConfig(lr=1e-3))
    opt.fold_param_grads()
    opt.reduce_gradients()
    return float(torch.sqrt(opt.grad_norm_sq()))


def _reshard_equal(tp_model, cfg, adapter, src, ctx) -> bool:
    """Load the checkpoint once more at tp=1 and cut this rank's layout out of that replica in memory."""
    from areno_b200.parallel.context import ParallelContext, use_context
    from areno_b200.parallel.reshard import reshard_into

    with use_context(ParallelContext(device=torch.device("cpu"))):
        full = adapter.build(cfg)
        adapter.load_weights(full, src, cfg)
    cut = adapter.build(cfg)          # built under the TP context: local shapes
    reshard_into(cut, full, ctx.tp_rank, ctx.tp_size)
    return all(torch.equal(a, b) for (_n, a), (_m, b) in zip(tp_model.named_parameters(), cut.named_parameters()))


def _greedy(model, prompts, n_new):
    from areno_b200.engine.inference import InferenceEngine, SamplingParams

    eng = InferenceEngine(model, 512, "cpu", max_slots=2, max_model_len=128, max_prefill_tokens=32)
    return eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=n_new).tokens


def _rank_main(rank, world, port, ret, src, dst, variant):
    try:
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        import torch.distributed as dist

        from areno_b200.models import registry
        from areno_b200.parallel.context import destroy_parallel, init_parallel

        ctx = init_parallel(rank, world, tp_size=world, master_port=port, backend="gloo", device=torch.device("cpu"),
                            timeout_s=120)
        cfg = _variant(variant)
        adapter = registry.get_adapter(cfg.model_type)
        model = adapter.build(cfg)
        adapter.load_weights(model, src, cfg)
        g = torch.Generator().manual_seed(3)
        ids = torch.randint(3, 512, (40,), generator=g)
        h, loss = _run(model, ids, [25, 15])
        gdn = model.layers[0].attn
        norm_grad = gdn.norm_weight.grad.clone()
        dist.all_reduce(norm_grad, group=ctx.tp_group)
        qn = model.layers[1].attn.q_norm.weight.grad.clone()
        dist.all_reduce(qn, group=ctx.tp_group)
        tokens = _greedy(model, [[5, 9, 77, 130], [200, 3, 8]], 5)
        adapter.save_weights(model, dst, cfg)
        raw = dict(h=h, loss=loss, norm_grad=norm_grad, q_norm_grad=qn, in_qkvz=gdn.in_qkvz.grad.clone(),
                   A_log=gdn.A_log.grad.clone(), out_proj=gdn.out_proj.weight.grad.clone(),
                   input_norm=model.layers[0].input_norm.weight.grad.clone(), tokens=tokens)
        raw["reshard_equal"] = _reshard_equal(model, cfg, adapter, src, ctx)
        raw["grad_norm"] = _optimizer_grad_norm(model)   # every parameter at once: reduced the way the trainer does it
        ret[rank] = raw
        destroy_parallel()
    except BaseException:  # noqa: BLE001
        ret[rank] = traceback.format_exc()


@pytest.mark.parametrize("variant", ["dense", "kv_replicated", "moe"])
def test_hybrid_tp2_matches_single_process(tmp_path, variant):
    from areno_b200.engine.checkpoint import SafetensorsIndex
    from areno_b200.models import registry

    single_process_context()
    cfg = _variant(variant)
    adapter = registry.get_adapter(cfg.model_type)
    ref = adapter.build(cfg)
    adapter.init_random(ref, 11)
    src, dst = str(tmp_path / "src"), str(tmp_path / "dst")
    adapter.save_weights(ref, src, cfg)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(3, 512, (40,), generator=g)
    h_ref, loss_ref = _run(ref, ids, [25, 15])
    tokens_ref = _greedy(ref, [[5, 9, 77, 130], [200, 3, 8]], 5)
    ref_grads = {n: p.grad.clone() for n, p in ref.named_parameters() if p.grad is not None}
    norm_ref = _optimizer_grad_norm(ref)

    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_rank_main, args=(world, _free_port(), ret, src, dst, variant), nprocs=world, join=True)
    gdn = ref.layers[0].attn
    kd, vd = gdn.key_dim, gdn.value_dim
    G = ref_grads
    q, k, v, z = G['layers.0.attn.in_qkvz'].split([kd, kd, vd, vd], 0)
    for r in range(world):
        out = ret[r]
        assert isinstance(out, dict), out
        assert torch.allclose(out["h"], h_ref, atol=2e-5, rtol=1e-4)
        assert abs(out["loss"] - loss_ref) < 1e-5 * max(1.0, abs(loss_ref))
        assert out["tokens"] == tokens_ref
        assert abs(out["grad_norm"] - norm_ref) < 1e-4 * norm_ref, (out["grad_norm"], norm_ref)
        # replicated parameters: the TP sum of the per-rank gradients is the full gradient
        assert torch.allclose(out["norm_grad"], G["layers.0.attn.norm_weight"], atol=1e-6, rtol=1e-4)
        assert torch.allclose(out["q_norm_grad"], G["layers.1.attn.q_norm.weight"], atol=1e-6, rtol=1e-4)
        assert torch.allclose(out["input_norm"], G["layers.0.input_norm.weight"], atol=1e-6, rtol=1e-4)
        # sharded parameters: the rank's gradient is its slice of the full one
        want = torch.cat([t.chunk(world, 0)[r] for t in (q, k, v, z)], 0)
        assert torch.allclose(out["in_qkvz"], want, atol=1e-6, rtol=1e-4)
        assert torch.allclose(out["A_log"], G["layers.0.attn.A_log"].chunk(world, 0)[r], atol=1e-6, rtol=1e-4)
        assert torch.allclose(out["out_proj"], G["layers.0.attn.out_proj.weight"].chunk(world, 1)[r], atol=1e-6, rtol=1e-4)
    # a TP layout cut out of the single-process replica in memory equals the one cut out of the checkpoint
    assert all(o["reshard_equal"] for o in (ret[0], ret[1]))
    # the checkpoint written from the shards is the checkpoint they came from
    a, b = SafetensorsIndex(src), SafetensorsIndex(dst)
    assert sorted(a.keys()) == sorted(b.keys())
    for key in a.keys():
        assert torch.equal(a.get(key), b.get(key)), key


# ------------------------------------------------------------------ plain dense / MoE families, same question
def _plain_cfg(kind: str):
    from .helpers import tiny_config

    if kind == "gemma4":           # sliding + global layers (global KV head replicated), KV-shared tail, PLE, MoE branch
        from .test_gemma4_cpu import gemma_config

        return gemma_config()
    if kind in ("bailing_gqa", "bailing_mla"):   # lightning-attention layers + GQA or latent attention, grouped sigmoid router
        from .test_bailing_cpu import bailing_config

        return bailing_config(mla=kind == "bailing_mla", qkv_bias=True)
    if kind == "dense_kv_rep":     # qkv bias, one KV head on two ranks, per-head norms
        return tiny_config(model_type="qwen3", num_key_value_heads=1, qkv_bias=True, qk_norm=True, num_hidden_layers=2)
    return tiny_config(model_type="qwen3_moe", qk_norm=True, qkv_bias=False, num_experts=4, num_experts_per_tok=2,
                       moe_intermediate_size=32, norm_topk_prob=True, num_hidden_layers=2)


def _plain_rank(rank, world, port, ret, src, kind, dst=None):
    try:
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        from areno_b200.models import registry
        from areno_b200.parallel.context import destroy_parallel, init_parallel

        init_parallel(rank, world, tp_size=world, master_port=port, backend="gloo", device=torch.device("cpu"),
                      timeout_s=120)
        cfg = _plain_cfg(kind)
        adapter = registry.get_adapter(cfg.model_type)
        model = adapter.build(cfg)
        adapter.load_weights(model, src, cfg)
        ids = torch.randint(3, 512, (40,), generator=torch.Generator().manual_seed(3))
        h, loss = _run(model, ids, [25, 15])
        if dst is not None:
            adapter.save_weights(model, dst, cfg)
        tokens = _greedy(model, [[5, 9, 77, 130], [200, 3, 8]], 5)      # cached inference with sharded heads / state
        ret[rank] = dict(h=h, loss=loss, grad_norm=_optimizer_grad_norm(model), tokens=tokens)
        destroy_parallel()
    except BaseException:  # noqa: BLE001
        ret[rank] = traceback.format_exc()


@pytest.mark.parametrize("kind", ["dense_kv_rep", "moe", "gemma4", "bailing_gqa", "bailing_mla"])
def test_tp2_gradient_norm_matches_single_process(tmp_path, kind):
    from areno_b200.engine.checkpoint import SafetensorsIndex
    from areno_b200.models import registry

    single_process_context()
    cfg = _plain_cfg(kind)
    adapter = registry.get_adapter(cfg.model_type)
    ref = adapter.build(cfg)
    adapter.init_random(ref, 5)
    if kind == "gemma4":
        with torch.no_grad():          # spread the routing over all experts (a zero router scale sends every token the same way)
            for layer in ref.layers:
                layer.router.scale.fill_(1.0)
                layer.moe.per_expert_scale.copy_(torch.linspace(0.8, 1.2, layer.moe.per_expert_scale.numel()))
    src, dst = str(tmp_path / "src"), str(tmp_path / "dst")
    adapter.save_weights(ref, src, cfg)
    ids = torch.randint(3, 512, (40,), generator=torch.Generator().manual_seed(3))
    h_ref, loss_ref = _run(ref, ids, [25, 15])
    tokens_ref = _greedy(ref, [[5, 9, 77, 130], [200, 3, 8]], 5)
    norm_ref = _optimizer_grad_norm(ref)
    ret = mp.Manager().dict()
    mp.spawn(_plain_rank, args=(2, _free_port(), ret, src, kind, dst), nprocs=2, join=True)
    for r in range(2):
        out = ret[r]
        assert isinstance(out, dict), out
        assert torch.allclose(out["h"], h_ref, atol=2e-5, rtol=1e-4)
        assert abs(out["grad_norm"] - norm_ref) < 1e-4 * norm_ref, (out["grad_norm"], norm_ref)
        assert out["tokens"] == tokens_ref
    a, b = SafetensorsIndex(src), SafetensorsIndex(dst)       # written from the shards == loaded from
    assert sorted(a.keys()) == sorted(b.keys())
    for key in a.keys():
        assert torch.equal(a.get(key), b.get(key)), key


# ------------------------------------------------------------------ sequence parallelism over the TP group
def _sp_rank(rank, world, port, ret, src, kind, ckpt):
    try:
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        from areno_b200.engine.config import OptimizerConfig
        from areno_b200.engine.optim import ShardedAdamW
        from areno_b200.models import registry
        from areno_b200.models.dense import TrainMeta
        from areno_b200.ops.attention import build_varlen_meta
        from areno_b200.parallel.context import destroy_parallel, init_parallel

        init_parallel(rank, world, tp_size=world, master_port=port, backend="gloo", device=torch.device("cpu"),
                      timeout_s=120)
        cfg = _sp_cfg(kind)
        adapter = registry.get_adapter(cfg.model_type)
        model = adapter.build(cfg)
        adapter.load_weights(model, src, cfg)
        ids = torch.randint(3, 512, (39,), generator=torch.Generator().manual_seed(3))     # odd: exercises the padding
        pos = torch.cat([torch.arange(n) for n in (25, 14)])
        meta = TrainMeta(build_varlen_meta([25, 14]), ckpt, sequence_parallel=True)
        import torch.distributed as dist

        calls = {"rs": 0, "ar": 0}
        real_rs, real_ar = dist.reduce_scatter_tensor, dist.all_reduce

        def count_rs(*a, **k):
            calls["rs"] += 1
            return real_rs(*a, **k)

        def count_ar(*a, **k):
            calls["ar"] += 1
            return real_ar(*a, **k)

        dist.reduce_scatter_tensor, dist.all_reduce = count_rs, count_ar
        h = model(ids, pos, meta).hidden_states
        forward_calls = dict(calls)
        dist.reduce_scatter_tensor, dist.all_reduce = real_rs, real_ar
        h.float().pow(2).mean().backward()
        opt = ShardedAdamW(model, OptimizerConfig(lr=1e-3), sequence_parallel=True)
        opt.fold_param_grads()
        opt.reduce_gradients()
        ret[rank] = dict(h=h.detach(), grad_norm=float(torch.sqrt(opt.grad_norm_sq())), forward_calls=forward_calls)
        destroy_parallel()
    except BaseException:  # noqa: BLE001
        ret[rank] = traceback.format_exc()


def _sp_cfg(kind):
    if kind == "hybrid_moe":
        return _variant("moe")
    return _plain_cfg(kind)


@pytest.mark.parametrize("kind,ckpt", [("dense_kv_rep", False), ("moe", True), ("hybrid_moe", False), ("bailing_mla", True)])
def test_sequence_parallel_tp2_matches_single_process(tmp_path, kind, ckpt):
    from areno_b200.models import registry
    from areno_b200.models.dense import TrainMeta
    from areno_b200.ops.attention import build_varlen_meta

    single_process_context()
    cfg = _sp_cfg(kind)
    adapter = registry.get_adapter(cfg.model_type)
    ref = adapter.build(cfg)
    adapter.init_random(ref, 7)
    src = str(tmp_path / "src")
    adapter.save_weights(ref, src, cfg)
    ids = torch.randint(3, 512, (39,), generator=torch.Generator().manual_seed(3))
    pos = torch.cat([torch.arange(n) for n in (25, 14)])
    h_ref = ref(ids, pos, TrainMeta(build_varlen_meta([25, 14]), False)).hidden_states
    h_ref.float().pow(2).mean().backward()
    norm_ref = _optimizer_grad_norm(ref)
    ret = mp.Manager().dict()
    mp.spawn(_sp_rank, args=(2, _free_port(), ret, src, kind, ckpt), nprocs=2, join=True)
    for r in range(2):
        out = ret[r]
        assert isinstance(out, dict), out
        assert out["h"].shape == h_ref.shape
        # the forward really ran sharded: reduce-scatters at the TP seams (embedding + two per layer), no all-reduce
        assert out["forward_calls"]["rs"] >= 1 + 2 * cfg.num_hidden_layers and out["forward_calls"]["ar"] == 0
        assert torch.allclose(out["h"], h_ref.detach(), atol=2e-5, rtol=1e-4)
        assert abs(out["grad_norm"] - norm_ref) < 1e-4 * norm_ref, (out["grad_norm"], norm_ref)
