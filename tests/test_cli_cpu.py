"""CLI layer: option surface, validation rules, hook pre-flight, config classes, summary, dataset
loading, the auto-tuner's search and the diagnostics commands.  Pure CPU."""

from __future__ import annotations

import json

import click
import pytest
from click.testing import CliRunner

from areno_b200.api.trainer_config import DPOTrainerConfig, PolicyTrainerConfig, PPOTrainerConfig, TrainerConfig
from areno_b200.cli import auto_tune as at
from areno_b200.cli import datasets as ds
from areno_b200.cli import train as cli_train
from areno_b200.cli.main import main as cli_main


def _reward_file(tmp_path, body="def reward_fn(record):\n    return 1.0\n"):
    p = tmp_path / "reward.py"
    p.write_text(body)
    return str(p)


def _base(tmp_path, **kw):
    opts = dict(ckpt="some/model", dataset_path="data.jsonl", reward_fn_path=_reward_file(tmp_path))
    opts.update(kw)
    return opts


def test_option_surface_and_defaults():
    names = [cli_train.option_name(f) for f, _kw, _g in cli_train.OPTIONS]
    assert len(names) == len(set(names)) == 64  # 62 reference options + kv-dtype + expert-parallel
    d = cli_train._defaults()
    assert (d["algo"], d["tp_size"], d["world_size"], d["batch_size"], d["n_samples"]) == ("gspo", 4, 8, 32, 8)
    assert (d["max_prompt_tokens"], d["max_new_tokens"], d["mini_bs"], d["score_micro_bs"]) == (1024, 3071, 16, 8)
    assert (d["lr"], d["min_lr"], d["lr_decay_steps"], d["lr_decay_style"]) == (1e-6, 1e-7, 1000, "cosine")
    assert (d["gspo_clip_eps"], d["grpo_clip_eps"], d["dpo_beta"], d["critic_warmup_steps"]) == (3e-4, 0.2, 0.1, 20)
    assert (d["save_interval"], d["epochs"], d["mem_frac"], d["tune_max_samples"]) == (100, 10, 0.9, 256)
    assert {g for _f, _k, g in cli_train.OPTIONS} == set(cli_train.GROUP_ORDER)


def test_help_is_grouped():
    out = CliRunner().invoke(cli_train.train_command, ["--help"]).output
    pos = [out.index(f"{g} options") for g in cli_train.GROUP_ORDER]
    assert pos == sorted(pos)
    assert "--no-activation-checkpointing" in out and "--kv-dtype" in out


def test_config_class_per_algorithm(tmp_path):
    loader = tmp_path / "loader.py"
    loader.write_text("def load_training_dataset(path, **kw):\n    return []\n")
    cfg = cli_train.trainer_config_from_options(**_base(tmp_path, algo="gspo"))
    assert type(cfg) is PolicyTrainerConfig and cfg.algo == "gspo" and cfg.keep_rollout_state
    cfg = cli_train.trainer_config_from_options(**_base(tmp_path, algo="ppo", reward_ckpt="rm", drop_rollout_state=True,
                                                        lr=2e-6, disable_thinking=True))
    assert type(cfg) is PPOTrainerConfig and cfg.reward_ckpt == "rm" and not cfg.keep_rollout_state
    assert cfg.optimizer_lr == 2e-6 and cfg.chat_template_enable_thinking is False
    cfg = cli_train.trainer_config_from_options(**_base(tmp_path, algo="dpo", reward_fn_path=None, dpo_beta=0.3))
    assert type(cfg) is DPOTrainerConfig and cfg.dpo_beta == 0.3 and not hasattr(cfg, "n_samples")
    cfg = cli_train.trainer_config_from_options(**_base(tmp_path, algo="sft", reward_fn_path=None,
                                                        dataset_loader_fn=str(loader)))
    assert type(cfg) is TrainerConfig and not hasattr(cfg, "reward_fn_path")
    ac = cfg.areno_config()
    assert ac.tp_size == 4 and ac.optimizer["lr"] == 1e-6 and ac.runtime["kv_dtype"] == "bf16" and not ac.expert_parallel
    cfg = cli_train.trainer_config_from_options(**_base(tmp_path, algo="grpo", tp_size=1, expert_parallel=True))
    assert cfg.expert_parallel and cfg.areno_config().expert_parallel
    with pytest.raises(ValueError, match="tp_size must be 1"):
        cli_train.trainer_config_from_options(**_base(tmp_path, algo="grpo", tp_size=2, expert_parallel=True))


@pytest.mark.parametrize("override,needle", [
    (dict(ckpt=None), "--ckpt is required"),
    (dict(dataset_path=None), "--dataset-path is required"),
    (dict(algo="sft", reward_fn_path=None), "--dataset-loader-fn is required"),
    (dict(algo="nope"), "unknown algorithm"),
    (dict(algo="dpo", reward_fn_path=None, tune_params=True), "--tune-params currently supports rollout"),
    (dict(mem_frac=0.0), "--mem-frac must be in (0, 1]"),
    (dict(mem_frac=1.5), "--mem-frac must be in (0, 1]"),
    (dict(tune_max_samples=0), "--tune-max-samples must be positive"),
    (dict(reward_fn_path=None), "--reward-fn-path or --reward-ckpt is required"),
    (dict(save_interval=0), "--save-interval must be positive"),
    (dict(epochs=0), "--epochs must be positive"),
    (dict(max_steps=0), "--max-steps must be positive"),
    (dict(tp_size=0), "--tp-size must be positive"),
    (dict(world_size=6, tp_size=4), "--world-size must be divisible by --tp-size"),
    (dict(n_samples=0), "--n-samples must be positive"),
    (dict(gradient_accumulation_steps=0), "--gradient-accumulation-steps must be positive"),
    (dict(max_context_len=0), "--max-context-len must be positive"),
    (dict(max_running_prompts=0), "--max-running-prompts must be positive"),
    (dict(agent_timeout_s=0), "--agent-timeout-s must be positive"),
    (dict(lr=0.0), "--lr must be positive"),
    (dict(min_lr=-1.0), "--min-lr must be non-negative"),
    (dict(weight_decay=-0.1), "--weight-decay must be non-negative"),
    (dict(temperature=0.0), "--temperature must be positive"),
    (dict(algo="gspo", gspo_clip_eps=0.0), "--gspo-clip-eps must be positive"),
    (dict(algo="grpo", grpo_clip_eps=0.0), "--grpo-clip-eps must be positive"),
    (dict(algo="ppo", gamma=0.0), "--gamma must be positive"),
    (dict(critic_warmup_steps=-1), "--critic-warmup-steps must be non-negative"),
])
def test_validation_rules(tmp_path, override, needle):
    with pytest.raises(click.UsageError) as err:
        cli_train.trainer_config_from_options(**_base(tmp_path, **override))
    assert needle in err.value.format_message()


def test_rules_scoped_to_algorithm(tmp_path):
    # a bad GRPO epsilon is irrelevant to GSPO; rollout-only knobs are irrelevant to DPO
    cli_train.trainer_config_from_options(**_base(tmp_path, algo="gspo", grpo_clip_eps=0.0))
    cli_train.trainer_config_from_options(**_base(tmp_path, algo="dpo", reward_fn_path=None, n_samples=0, temperature=0.0))


def test_hook_preflight(tmp_path):
    missing = str(tmp_path / "nope.py")
    with pytest.raises(click.UsageError, match="file does not exist"):
        cli_train.trainer_config_from_options(**_base(tmp_path, reward_fn_path=missing))
    bad = tmp_path / "bad.py"
    bad.write_text("def reward_fn(:\n")
    with pytest.raises(click.UsageError, match="cannot parse Python file"):
        cli_train.trainer_config_from_options(**_base(tmp_path, reward_fn_path=str(bad)))
    wrong = tmp_path / "wrong.py"
    wrong.write_text("def reward(record):\n    return 0\n")
    with pytest.raises(click.UsageError, match="must define callable reward_fn"):
        cli_train.trainer_config_from_options(**_base(tmp_path, reward_fn_path=str(wrong)))
    arity = tmp_path / "arity.py"
    arity.write_text("def reward_fn(a, b):\n    return 0\n")
    with pytest.raises(click.UsageError, match="must define callable reward_fn"):
        cli_train.trainer_config_from_options(**_base(tmp_path, reward_fn_path=str(arity)))
    agent = tmp_path / "agent.py"
    agent.write_text("async def run_agent(ctx, batch, extra=None):\n    return []\n")
    cfg = cli_train.trainer_config_from_options(**_base(tmp_path, agent_fn=str(agent)))
    assert cfg.agent_fn == str(agent)
    one_arg = tmp_path / "agent1.py"
    one_arg.write_text("def run_agent(ctx):\n    return []\n")
    with pytest.raises(click.UsageError, match="run_agent"):
        cli_train.trainer_config_from_options(**_base(tmp_path, agent_fn=str(one_arg)))
    # hooks are parsed, never executed
    boom = tmp_path / "boom.py"
    boom.write_text("raise SystemExit('executed')\ndef reward_fn(*records):\n    return 0\n")
    cli_train.trainer_config_from_options(**_base(tmp_path, reward_fn_path=str(boom)))
    loader = tmp_path / "ld.py"
    loader.write_text("def custom(path, **kw):\n    return []\n")
    cli_train.trainer_config_from_options(**_base(tmp_path, dataset_loader_fn=f"{loader}:custom"))
    with pytest.raises(click.UsageError, match="load_training_dataset"):
        cli_train.trainer_config_from_options(**_base(tmp_path, dataset_loader_fn=str(loader)))


def test_summary(tmp_path):
    cfg = cli_train.trainer_config_from_options(**_base(tmp_path, algo="grpo", world_size=8, tp_size=2))
    text = cli_train.format_training_config_summary(cfg)
    for needle in ("PolicyOnlyTrainer", "grpo_loss_fn", "dp_size", "max_running_prompts", "256",
                   "no checkpoint output path configured"):
        assert needle in text
    cfg = cli_train.trainer_config_from_options(**_base(tmp_path, algo="dpo", reward_fn_path=None, save_path="/tmp/x"))
    text = cli_train.format_training_config_summary(cfg)
    assert "n/a" in text and "WARNING" not in text


def test_dataset_loading(tmp_path):
    rows = [{"prompt": f"q{i}", "answer": str(i)} for i in range(5)]
    f = tmp_path / "train.jsonl"
    f.write_text("\n".join(json.dumps(r) for r in rows))
    data = ds.load_dataset_for_training(str(f), dataset_loader_fn=None)
    assert len(data) == 5 and data[0]["prompt"] == "q0"
    folder = tmp_path / "dir"
    folder.mkdir()
    (folder / "a.jsonl").write_text("\n".join(json.dumps(r) for r in rows[:2]))
    (folder / "b.jsonl").write_text("\n".join(json.dumps(r) for r in rows[2:]))
    assert len(ds.load_dataset_for_training(str(folder), dataset_loader_fn=None)) == 5
    loader = tmp_path / "loader.py"
    loader.write_text("def load_training_dataset(path, *, default_loader, load_dataset, load_from_disk):\n"
                      "    return [dict(r, extra=1) for r in default_loader(path)]\n")
    out = ds.load_dataset_for_training(str(f), dataset_loader_fn=str(loader))
    assert out[0]["extra"] == 1
    with pytest.raises(ValueError):
        ds.builder_for_suffix(".xlsx")
    calls = []

    def fake_load(name, *a, **kw):
        calls.append((name, a, kw))
        if not a:
            raise ValueError("Config name is missing. Please pick one among the available configs: ['main', 'socratic']")
        return "ok"

    assert ds.load_hf_dataset_ref("openai/gsm8k", fake_load) == "ok" and calls[-1][1] == ("main",)
    assert ds.load_hf_dataset_ref("repo:cfg:test", fake_load) == "ok" and calls[-1][2] == {"split": "test"}
    with pytest.raises(ValueError):
        ds.load_hf_dataset_ref("a:b:c:d", fake_load)


# ------------------------------------------------------------------------- auto tune
def _policy_cfg(**kw):
    base = dict(algo="gspo", ckpt="m", dataset_path="d", batch_size=32, n_samples=8, mini_bs=16)
    base.update(kw)
    return PolicyTrainerConfig(**base)


def test_auto_tune_helpers():
    assert at.powers_of_two_up_to(9) == [1, 2, 4, 8] and at.floor_power_of_two(100) == 64
    assert at.sparse_select(list(range(100)), 5) == [0, 25, 50, 74, 99]
    assert at.mini_bs_values(16, 6) == [1, 2, 4] and at.mini_bs_values(3, 100) == [1, 2]
    assert at.is_oom_error("CUDA out of memory. Tried to allocate")
    assert at.is_oom_error("worker exited without reporting result (exitcode -9)")
    assert not at.is_oom_error("shape mismatch")
    assert at.is_tp_compat_error("num_key_value_heads must be divisible by tp") and not at.is_tp_compat_error("boom")
    cands = at.rollout_candidates(_policy_cfg(), auto_max_samples=256)
    assert [c.max_running_prompts for c in cands] == [256, 128, 64, 32, 16, 8, 4, 2, 1]
    assert at.dummy_token_budgets(max_prompt_tokens=1024, max_new_tokens=3071, max_context_len=2048) == (1024, 1024)
    assert len(at.enumerate_candidates(_policy_cfg(), auto_max_samples=64)) > 5


def test_auto_tune_search():
    seen = []

    def probe(config, cand, stage):
        seen.append((stage, cand.max_running_prompts, cand.mini_bs))
        if stage == "rollout":
            frac = cand.max_running_prompts / 128  # 64 -> 0.5 fits, 128 -> 1.0 does not
            if cand.max_running_prompts == 256:
                return at.AutoTuneMeasurement(cand, 1.0, ok=False, error="CUDA out of memory")
            return at.AutoTuneMeasurement(cand, frac, ok=True)
        return at.AutoTuneMeasurement(cand, 0.3 + cand.mini_bs * 0.1, ok=True)

    res = at.auto_tune_config(_policy_cfg(), mem_frac=0.8, auto_max_samples=256, probe_fn=probe)
    assert [s for s in seen if s[0] == "rollout"] == [("rollout", 256, 1), ("rollout", 128, 1), ("rollout", 64, 1)]
    assert [s[2] for s in seen if s[0] == "train"] == [16, 8, 4]
    c = res.config
    assert (c.max_running_prompts, c.batch_size, c.n_samples, c.mini_bs, c.keep_rollout_state) == (64, 8, 8, 4, False)
    assert "mini_bs=4" in at.format_auto_tune_summary(res)
    # user-fixed concurrency skips the rollout stage
    seen.clear()
    res = at.auto_tune_config(_policy_cfg(max_running_prompts=32), mem_frac=0.95, probe_fn=probe)
    assert all(s[0] == "train" for s in seen) and res.config.batch_size == 4
    with pytest.raises(RuntimeError, match="could not find a candidate"):
        at.auto_tune_config(_policy_cfg(), mem_frac=0.001, probe_fn=probe)
    with pytest.raises(ValueError):
        at.auto_tune_config(TrainerConfig(algo="sft", ckpt="m", dataset_path="d"), probe_fn=probe)


def test_probe_classifies_errors(monkeypatch):
    cand = at.rollout_candidates(_policy_cfg())[0]
    monkeypatch.setattr(at, "_run_dummy_probe", lambda *a, **k: (_ for _ in ()).throw(RuntimeError("CUDA out of memory")))
    m = at.probe_candidate_with_dummy_run(_policy_cfg(), cand, "rollout")
    assert not m.ok and m.peak_mem_frac == 1.0
    monkeypatch.setattr(at, "_run_dummy_probe", lambda *a, **k: (_ for _ in ()).throw(RuntimeError("unrelated")))
    with pytest.raises(RuntimeError, match="unrelated"):
        at.probe_candidate_with_dummy_run(_policy_cfg(), cand, "rollout")


# ------------------------------------------------------------------------ diagnostics
def test_main_group_and_diagnostics():
    runner = CliRunner()
    out = runner.invoke(cli_main, ["--help"]).output
    for name in ("check", "env", "serve", "train"):
        assert name in out
    res = runner.invoke(cli_main, ["env", "--json"])
    assert res.exit_code == 0
    report = json.loads(res.output)
    assert {"torch", "cuda", "gpus", "native", "dependencies", "env", "paths"} <= set(report)
    res = runner.invoke(cli_main, ["check"])
    assert "AReno-B200 check:" in res.output and res.exit_code in (0, 1)
    from areno_b200.cli.diagnostics import run_checks

    rows = {r.name: r for r in run_checks(report)}
    assert rows["Python >= 3.10"].status == "PASS"
    report["gpus"] = [{"index": 0, "name": "H100", "capability": "9.0", "memory_gb": 80, "sm_count": 132}]
    rows = {r.name: r for r in run_checks(report)}
    assert rows["GPUs are sm_100 (B200 class)"].status == "FAIL"


@pytest.mark.parametrize("algo", ["grpo", "ppo", "dpo", "sft", "grpo --agentic", "ppo --world-size 2 --tp-size 2"])
def test_train_smoke_script_runs_the_cli_path_end_to_end(algo):
    """``ci/train_smoke.py`` drives option validation -> dataset -> trainer factory -> fit -> save on CPU, for the
    rollout algorithms, PPO with its reference and critic roles, the two offline algorithms, and an agent function
    behind the local proxy; the last case runs PPO tensor parallel over two spawned gloo ranks."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    proc = subprocess.run([sys.executable, str(root / "ci" / "train_smoke.py"), "--algo", *algo.split(), "--steps", "2", "--device", "cpu"],
                          capture_output=True, text=True, timeout=600, cwd=str(root))
    assert proc.returncode == 0, proc.stderr[-2000:]
    out = json.loads(proc.stdout.strip().splitlines()[-1])
    assert out["steps_done"] == 2 and out["checkpoints"] and out["metric_files"]


def test_every_option_has_help_and_a_row_in_the_reference_page():
    from pathlib import Path

    page = (Path(__file__).resolve().parents[1] / "docs" / "cli_train.md").read_text()
    for flag, kw, _group in cli_train.OPTIONS:
        assert kw.get("help"), flag
        assert f"| `{flag}` |" in page and kw["help"] in page, flag
