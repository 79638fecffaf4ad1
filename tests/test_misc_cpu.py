"""Smaller SDK pieces: algorithm registry, tool-call parsers, metrics writer, model references,
sampling reference (distribution and determinism), layering of imports, bundled examples."""

from __future__ import annotations

import ast
import importlib.util
import os
import pathlib
from types import SimpleNamespace

import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]


# ---------------------------------------------------------------- algorithm registry
def test_algorithm_registry_and_loss_binding():
    from areno_b200.api.algorithms import AlgorithmSpec, get_algorithm, list_algorithms, register_algorithm
    from areno_b200.api.loss_fns import grpo_loss_fn
    from areno_b200.api.trainer_config import PolicyTrainerConfig

    names = set(list_algorithms())
    assert {"sft", "dpo", "gspo", "grpo", "ppo"} <= names
    assert get_algorithm(" GRPO ").name == "grpo" and get_algorithm("sft").requires_rollout is False
    cfg = PolicyTrainerConfig(algo="gspo", ckpt="m", dataset_path="d", gspo_clip_eps=0.123)
    bound = get_algorithm("gspo").make_loss_fn(cfg)
    assert bound.keywords == {"clip_eps": 0.123}
    assert get_algorithm("ppo").resolve_trainer_cls().__name__ == "PPOTrainer"
    with pytest.raises(ValueError, match="unknown algorithm"):
        get_algorithm("nope")
    spec = AlgorithmSpec("my_algo", lambda: object, grpo_loss_fn, requires_rollout=True, experimental=True)
    register_algorithm(spec)
    with pytest.raises(ValueError, match="already registered"):
        register_algorithm(spec)
    register_algorithm(spec, replace=True)
    assert get_algorithm("my_algo").experimental


# ------------------------------------------------------------------ tool-call parsers
TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {
    "type": "object", "properties": {"city": {"type": "string"}, "unit": {"type": "string", "enum": ["c", "f"]}}}}},
    {"type": "function", "function": {"name": "add", "parameters": {"type": "object", "properties": {
        "a": {"type": "integer"}, "b": {"type": "integer"}}}}}]


def test_tool_call_parsers():
    import json

    from areno_b200.api.tool_call_parser import get_tool_call_parser, list_tool_call_parsers

    assert {"json", "qwen", "gemma4", "minicpm"} <= set(list_tool_call_parsers())
    q = get_tool_call_parser("qwen")
    res = q.parse('thinking...\n<tool_call>\n{"name": "add", "arguments": {"a": 1, "b": 2}}\n</tool_call>', TOOLS, None)
    assert [c["function"]["name"] for c in res.tool_calls] == ["add"]
    assert json.loads(res.tool_calls[0]["function"]["arguments"]) == {"a": 1, "b": 2}
    two = q.parse('<tool_call>{"name":"add","arguments":{"a":1,"b":2}}</tool_call>'
                  '<tool_call>{"name":"get_weather","arguments":{"city":"Oslo"}}</tool_call>', TOOLS, None)
    assert [c["function"]["name"] for c in two.tool_calls] == ["add", "get_weather"]
    # unknown tools and a forced tool_choice are respected
    assert q.parse('<tool_call>{"name":"rm_rf","arguments":{}}</tool_call>', TOOLS, None).tool_calls == []
    forced = {"type": "function", "function": {"name": "add"}}
    only = q.parse('<tool_call>{"name":"get_weather","arguments":{"city":"x"}}</tool_call>', TOOLS, forced)
    assert all(c["function"]["name"] == "add" for c in only.tool_calls)
    j = get_tool_call_parser("json")
    assert j.parse('{"name": "get_weather", "arguments": {"city": "Rome"}}', TOOLS, None).tool_calls[0]["function"]["name"] == "get_weather"
    assert j.parse("no tools here", TOOLS, None).tool_calls == []
    assert get_tool_call_parser(None).__class__ is j.__class__


# ---------------------------------------------------------------------------- metrics
def test_metrics_recorder_writes_event_files(tmp_path):
    from areno_b200.api import TrainSequence
    from areno_b200.api.metrics import MetricsRecorder

    batch = [TrainSequence(tokens=[1, 2, 3, 4], prompt_mask=[True, True, False, False], logprobs=[0, 0, -1.0, -2.0],
                           advantages=[0, 0, 1.0, 1.0], reward=1.0),
             TrainSequence(tokens=[1, 2, 3], prompt_mask=[True, False, False], logprobs=[0, -1.0, -0.5],
                           advantages=[0, -1.0, -1.0], reward=0.0)]
    with MetricsRecorder(str(tmp_path)) as rec:
        rec.record_train_step(step=1, train_result={"loss": 0.5, "grad_norm": 1.0, "lr": 1e-6}, train_batch=batch,
                              timings={"rollout": 1.0, "train": 2.0})
    assert any(name.startswith("events.out.tfevents") for name in os.listdir(tmp_path))


# ---------------------------------------------------------------------- model references
def test_model_refs(tmp_path):
    from areno_b200.api.trainer_config import PPOTrainerConfig
    from areno_b200.cli.model_refs import resolve_model_path, resolve_model_refs_for_config

    d = tmp_path / "m"
    d.mkdir()
    assert resolve_model_path(str(d)) == str(d) and resolve_model_path(None) is None
    with pytest.raises(FileNotFoundError):
        resolve_model_path("./definitely/not/here")
    cfg = PPOTrainerConfig(algo="ppo", ckpt=str(d), dataset_path="x", ref_ckpt=str(d), reward_ckpt=None)
    out = resolve_model_refs_for_config(cfg)
    assert out.ckpt == str(d) and out.ref_ckpt == str(d) and out.reward_ckpt is None and out is not cfg
    # a repo id shared by several roles is fetched once
    import sys
    import types

    from areno_b200.cli.model_refs import resolve_model_ref

    calls = []
    fake = types.ModuleType("huggingface_hub")
    fake.snapshot_download = lambda repo_id: calls.append(repo_id) or f"/cache/{repo_id}"
    old = sys.modules.get("huggingface_hub")
    sys.modules["huggingface_hub"] = fake
    try:
        cfg = PPOTrainerConfig(algo="ppo", ckpt="org/model", dataset_path="x", ref_ckpt="org/model", critic_ckpt="org/model",
                               reward_ckpt="org/reward")
        out = resolve_model_refs_for_config(cfg)
        assert (out.ckpt, out.ref_ckpt, out.critic_ckpt, out.reward_ckpt) == ("/cache/org/model",) * 3 + ("/cache/org/reward",)
        assert calls == ["org/model", "org/reward"]
        cache = {}
        assert resolve_model_ref("org/other", cache) == resolve_model_ref("org/other", cache) and calls.count("org/other") == 1
        assert resolve_model_ref("org/other") == "/cache/org/other" and calls.count("org/other") == 2      # no cache, no reuse
    finally:
        if old is None:
            sys.modules.pop("huggingface_hub", None)
        else:
            sys.modules["huggingface_hub"] = old


# ------------------------------------------------------------------- sampling reference
def test_keyed_sampling_is_reproducible_shard_consistent_and_distributed_correctly():
    from areno_b200.ops import sampling

    torch.manual_seed(0)
    logits = torch.randn(6, 64)
    uid = torch.arange(6)
    step = torch.zeros(6, dtype=torch.int32)
    a, lp_a = sampling.sample(logits, 1.0, seed=7, row_uid=uid, gen_count=step)
    b, _ = sampling.sample(logits, 1.0, seed=7, row_uid=uid, gen_count=step)
    c, _ = sampling.sample(logits, 1.0, seed=8, row_uid=uid, gen_count=step)
    assert torch.equal(a, b) and not torch.equal(a, c)
    assert torch.allclose(lp_a, torch.log_softmax(logits, -1).gather(1, a[:, None]).squeeze(1), atol=1e-5)
    # two vocabulary shards combine to the same draw as the full row
    parts = []
    for r in range(2):
        rec = torch.empty(6, 6)
        sampling.sample(logits[:, r * 32:(r + 1) * 32].contiguous(), 1.0, seed=7, row_uid=uid, gen_count=step,
                        vocab_start=r * 32, part=rec)
        parts.append(rec)
    tok, lp = sampling.combine_shards(torch.stack(parts))
    assert torch.equal(tok, a) and torch.allclose(lp, lp_a, atol=1e-5)
    # empirical distribution of one row follows softmax; top-k never leaves the k best
    row = torch.tensor([[2.0, 1.0, 0.0, -1.0]]).repeat(4000, 1)
    draws, _ = sampling.sample(row, 1.0, seed=1, row_uid=torch.arange(4000), gen_count=torch.zeros(4000, dtype=torch.int32))
    freq = torch.bincount(draws, minlength=4).float() / 4000
    assert torch.allclose(freq, torch.softmax(row[0], -1), atol=0.03)
    topk, _ = sampling.sample(row, 1.0, top_k=2, seed=1, row_uid=torch.arange(4000), gen_count=torch.zeros(4000, dtype=torch.int32))
    assert set(topk.tolist()) == {0, 1}
    greedy, _ = sampling.sample(logits, 0.0)
    assert torch.equal(greedy, logits.argmax(-1))


# --------------------------------------------------------------------- import layering
def _imports(path: pathlib.Path) -> set[str]:
    out = set()
    tree = ast.parse(path.read_text())
    pkg = ".".join(path.relative_to(ROOT).with_suffix("").parts[:-1])
    for node in ast.walk(tree):
        if isinstance(node, ast.Import):
            out.update(a.name for a in node.names)
        elif isinstance(node, ast.ImportFrom):
            if node.level:
                base = pkg.split(".")[: len(pkg.split(".")) - node.level + 1]
                out.add(".".join(base + ([node.module] if node.module else [])))
            elif node.module:
                out.add(node.module)
    return out


def test_layering_ops_and_engine_do_not_import_the_sdk_or_cli():
    """Lower layers never import upper ones: ops < models/parallel < engine < api < cli."""
    for layer, banned in (("ops", ("areno_b200.engine", "areno_b200.api", "areno_b200.cli", "areno_b200.models")),
                          ("parallel", ("areno_b200.engine", "areno_b200.api", "areno_b200.cli", "areno_b200.models")),
                          ("models", ("areno_b200.api", "areno_b200.cli")),
                          ("engine", ("areno_b200.api",))):
        for path in (ROOT / "areno_b200" / layer).rglob("*.py"):
            for mod in _imports(path):
                bad = [b for b in banned if mod == b or mod.startswith(b + ".")]
                if layer == "engine" and mod.startswith("areno_b200.cli.model_refs"):
                    continue  # path resolution helper shared with the CLI
                assert not bad, f"{path.relative_to(ROOT)} imports {mod}"


def test_nothing_committed_imports_working_files():
    import re

    for path in list((ROOT / "areno_b200").rglob("*.py")) + [ROOT / "bench.py", ROOT / "__graft_entry__.py"]:
        assert not re.search(r"(^|[\"'/\s.])_work(/|\b\.|[\"'])", path.read_text()), path


# ---------------------------------------------------------------------------- examples
def _load(path: str):
    spec = importlib.util.spec_from_file_location(pathlib.Path(path).stem, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_examples_pass_the_cli_preflight_and_behave(tmp_path):
    from areno_b200.cli.train import trainer_config_from_options

    ex = ROOT / "examples"
    cfg = trainer_config_from_options(
        algo="grpo", ckpt="m", dataset_path="tictactoe:8",
        dataset_loader_fn=str(ex / "agentic/tictactoe/dataset_loader.py"),
        agent_fn=str(ex / "agentic/tictactoe/run_agent.py"), reward_fn_path=str(ex / "agentic/tictactoe/reward.py"))
    assert cfg.agent_fn.endswith("run_agent.py")
    for name in ("shopping", "duelgrid", "coding"):
        trainer_config_from_options(
            algo="gspo", ckpt="m", dataset_path=f"{name}:8", dataset_loader_fn=str(ex / f"agentic/{name}/dataset_loader.py"),
            agent_fn=str(ex / f"agentic/{name}/run_agent.py"), reward_fn_path=str(ex / f"agentic/{name}/reward.py"))
    trainer_config_from_options(algo="sft", ckpt="m", dataset_path="alpaca",
                                dataset_loader_fn=str(ex / "sft/alpaca/dataset_loader.py"))
    trainer_config_from_options(algo="gspo", ckpt="m", dataset_path="gsm8k",
                                dataset_loader_fn=str(ex / "math/dataset_loader.py"),
                                reward_fn_path=str(ex / "math/reward.py"))
    rows = _load(str(ex / "math/dataset_loader.py")).load_training_dataset(
        "x", default_loader=lambda p: [{"question": "1+1?", "answer": "so #### 2"}], load_dataset=None, load_from_disk=None)
    assert rows == [{"prompt": rows[0]["prompt"], "answer": "2"}] and "1+1?" in rows[0]["prompt"]
    reward = _load(str(ex / "math/reward.py")).reward_fn
    assert reward(SimpleNamespace(completion="it is #### 2", answer="2")) == 1.0
    assert reward(SimpleNamespace(completion="it is 3", answer="2")) == 0.0
    sft = _load(str(ex / "sft/alpaca/dataset_loader.py")).load_training_dataset(
        "x", default_loader=lambda p: [{"instruction": "Say hi", "input": "", "output": "hi"}, {"instruction": "", "output": "x"}],
        load_dataset=None, load_from_disk=None)
    assert sft == [{"prompt": "Say hi", "response": "hi"}]
    games = _load(str(ex / "agentic/tictactoe/dataset_loader.py")).load_training_dataset(
        "tictactoe:8", default_loader=None, load_dataset=None, load_from_disk=None)
    assert len(games) == 8
    ttt_reward = _load(str(ex / "agentic/tictactoe/reward.py")).reward_fn
    assert ttt_reward(SimpleNamespace(tool_results=[{"content": '{"result": "win"}'}])) == 1.0
    assert ttt_reward(SimpleNamespace(tool_results=[])) == 0.0


def test_native_libraries_are_current():
    """The in-tree libraries travel with the source; a stale build would be recompiled by every rank."""
    from areno_b200 import build

    for path in (build.kernels_lib_path(), build.runtime_lib_path()):
        assert path.exists(), f"{path} missing: run python -m areno_b200.build"
    before = build.kernels_lib_path().stat().st_mtime_ns
    build.ensure_built()
    assert build.kernels_lib_path().stat().st_mtime_ns == before, "kernel library was stale and had to be rebuilt"


def test_gradient_buckets_know_when_they_are_final():
    """Buckets are handed to the peer-memory reduce-scatter as backward passes the layers they depend on:
    the layer map, the per-bucket lowest layer and the launch order are checked with a recording stand-in for
    the communicator (the hook itself fires from autograd on the CPU as well)."""
    import torch

    from areno_b200.engine.config import OptimizerConfig
    from areno_b200.engine.optim import ShardedAdamW, _layer_index_of
    from areno_b200.models.dense import DenseCausalLM, TrainMeta, init_weights
    from areno_b200.ops.attention import build_varlen_meta
    from areno_b200.parallel.context import single_process_context

    from .helpers import tiny_config

    single_process_context()
    model = DenseCausalLM(tiny_config(num_hidden_layers=3, tie_word_embeddings=False))
    init_weights(model, 0)
    layer_of = _layer_index_of(model)
    assert layer_of[id(model.embed.weight)] == -1 and layer_of[id(model.lm_head.weight)] == 3
    assert layer_of[id(model.layers[1].mlp.down.weight)] == 1 and layer_of[id(model.norm.weight)] == 3
    opt = ShardedAdamW(model, OptimizerConfig(lr=1e-3, fp32_master_bucket_numel=40_000))
    assert opt.grad_comm is None and opt.begin_overlap() is None            # one rank: nothing to reduce
    lows = [b.min_layer for b in opt.buckets]
    assert -1 in lows and 3 in lows and all(-1 <= v <= 3 for v in lows)

    class Recorder:
        def __init__(self):
            self.launched, self.order = set(), []

        def begin_step(self):
            self.launched.clear()

        def launch(self, i, off, shard):
            if i not in self.launched:
                self.launched.add(i)
                self.order.append(i)

        def finish(self):
            pass

    opt.grad_comm, opt.dp = Recorder(), 2
    events = []
    hook = opt.begin_overlap()
    assert hook is not None

    def traced(layer):
        before = len(opt.grad_comm.order)
        hook(layer)
        events.append((layer, opt.grad_comm.order[before:]))

    ids = torch.randint(3, 512, (40,))
    meta = TrainMeta(build_varlen_meta([40]), True, layer_grad_hook=traced)
    h = model(ids, torch.arange(40), meta).hidden_states
    model.compute_logits(h).float().logsumexp(-1).mean().backward()
    assert [layer for layer, _ in events] == [2, 1, 0]                      # backward walks the layers downwards
    for layer, launched in events:
        assert launched and all(opt.buckets[i].min_layer >= layer for i in launched)
    not_yet = [i for i, b in enumerate(opt.buckets) if i not in opt.grad_comm.launched]
    assert not_yet and all(opt.buckets[i].min_layer == -1 for i in not_yet)   # the embedding leaves at the very end


def test_checkpoint_compare_tool(tmp_path):
    import torch
    from safetensors.torch import save_file

    from areno_b200.utils.compare_ckpt import compare, main

    a = {"model.w": torch.arange(12, dtype=torch.float32).view(3, 4), "model.b": torch.ones(4), "only.a": torch.zeros(2)}
    b = {"model.w": a["model.w"].clone(), "model.b": torch.ones(4) * 1.5, "only.b": torch.zeros(2)}
    b["model.w"][0, 0] = 2.0
    for name, tensors in (("a", a), ("b", b)):
        (tmp_path / name).mkdir()
        save_file(tensors, str(tmp_path / name / "model.safetensors"))
    rep = compare(str(tmp_path / "a"), str(tmp_path / "b"))
    assert rep["missing_in_other"] == ["only.a"] and rep["extra_in_other"] == ["only.b"] and not rep["identical"]
    by_key = {r["key"]: r for r in rep["tensors"]}
    assert by_key["model.b"]["max_abs"] == 0.5 and by_key["model.w"]["max_abs"] == 2.0
    assert rep["tensors"][0]["key"] == "model.b"                     # sorted by relative difference
    assert compare(str(tmp_path / "a"), str(tmp_path / "a"))["identical"]
    assert main([str(tmp_path / "a"), str(tmp_path / "a"), "--pattern", "model.*"]) == 0
    assert main([str(tmp_path / "a"), str(tmp_path / "b"), "--json"]) == 1


def test_trace_ranges_off_by_default_and_timed_when_enabled():
    import contextlib
    import time

    from areno_b200.utils import tracing

    tracing.configure(nvtx=False, timers=False)
    assert isinstance(tracing.trace_range("x"), contextlib.nullcontext)   # shared no-op: nothing allocated
    assert tracing.trace_range("x") is tracing.trace_range("y")
    tracing.configure(timers=True)
    try:
        for _ in range(3):
            with tracing.trace_range("phase/a"):
                time.sleep(0.002)

        @tracing.traced("phase/b")
        def work(v):
            return v + 1

        assert work(1) == 2
        rep = tracing.phase_report()
        assert rep["phase/a"]["count"] == 3 and rep["phase/a"]["ms"] >= 5.0
        assert rep["phase/b"]["count"] == 1
        assert tracing.phase_report() == {}                  # the report resets the counters
        with tracing.trace_range("phase/c"):
            pass
        merged = tracing.phase_report_max()                  # no process group: the local report
        assert set(merged) == {"phase/c"}
        assert "phase/c" in tracing.format_report(merged)
    finally:
        tracing.configure(nvtx=False, timers=False)


def test_rollout_loop_reports_named_phases():
    """A CPU generate call leaves prefill and decode ranges in the phase report."""
    import torch

    from areno_b200.engine.config import ModelConfig
    from areno_b200.engine.inference import InferenceEngine, SamplingParams
    from areno_b200.models.dense import DenseCausalLM, init_weights
    from areno_b200.parallel.context import single_process_context
    from areno_b200.utils import tracing

    single_process_context()
    cfg = ModelConfig(model_type="qwen2", vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=32, rope_theta=1e4, qk_norm=False,
                      qkv_bias=True, dtype=torch.float32)
    model = DenseCausalLM(cfg)
    init_weights(model, 0)
    eng = InferenceEngine(model, 512, "cpu", max_slots=2, max_model_len=64, max_prefill_tokens=64)
    tracing.configure(timers=True)
    try:
        tracing.phase_report()
        eng.generate([[5, 6, 7], [9, 10]], SamplingParams(temperature=0.0), max_new_tokens=4)
        rep = tracing.phase_report()
    finally:
        tracing.configure(nvtx=False, timers=False)
    assert rep["rollout/prefill"]["count"] >= 1
    assert rep["rollout/decode_step"]["count"] >= 3


def test_metrics_fall_back_to_jsonl_without_tensorboard(tmp_path, monkeypatch):
    import builtins
    import json

    from areno_b200.api import metrics

    real_import = builtins.__import__

    def no_tensorboard(name, *args, **kwargs):
        if name.startswith("torch.utils.tensorboard") or name.startswith("tensorboardX"):
            raise ImportError(name)
        return real_import(name, *args, **kwargs)

    monkeypatch.setattr(builtins, "__import__", no_tensorboard)
    writer = metrics.create_tensorboard_writer(str(tmp_path))
    assert isinstance(writer, metrics.JsonlScalarWriter)
    writer.add_scalar("train/loss", 0.5, 3)
    writer.flush()
    writer.close()
    rows = [json.loads(line) for line in open(tmp_path / "metrics.jsonl")]
    assert rows[0]["tag"] == "train/loss" and rows[0]["value"] == 0.5 and rows[0]["step"] == 3


def test_importing_the_sdk_and_cli_entry_points_stays_light():
    """``import areno_b200.api`` / the CLI group must not pull in torch, transformers, the engine or the kernels:
    ``areno --help``, ``areno env`` and option validation have to work (and be fast) on a machine without a GPU stack."""
    import subprocess
    import sys

    code = ("import sys; import areno_b200.api; import areno_b200.cli.main; "
            "print([m for m in ('torch', 'transformers', 'fastapi', 'datasets', 'areno_b200.engine', 'areno_b200.ops', "
            "'areno_b200.models') if m in sys.modules])")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=str(ROOT), timeout=120)
    assert out.returncode == 0 and out.stdout.strip() == "[]", out.stdout + out.stderr


def test_a_missing_compiler_is_reported_with_the_next_step(monkeypatch):
    from areno_b200 import build

    monkeypatch.setattr(build, "NVCC", "/nonexistent/cuda/bin/nvcc")
    with pytest.raises(RuntimeError, match="CUDA_HOME") as err:
        build.build_kernels(force=True)
    assert "12.8" in str(err.value) and "areno check" in str(err.value) and "no GPU is needed" in str(err.value)
    build.ensure_built()                       # an up-to-date library needs no compiler at all
