"""``areno train``: option surface, validation, hook pre-flight, config build and the run loop.

The 62 options, their defaults and their five help groups (Basic / Rollout / Train / Checkpoint /
Observability) are those of the reference CLI (``areno/cli/train.py:46-128,942-1093``); ``--kv-dtype`` and ``--expert-parallel``
is an addition (fp8 KV pages).  User hook files (``--dataset-loader-fn``, ``--reward-fn-path``,
``--agent-fn``) are checked by parsing their AST before any model is loaded; they are never executed
during validation.
"""

from __future__ import annotations

import ast
from pathlib import Path
from types import SimpleNamespace

import click

from ..api.defaults import DEFAULT_METRICS_LOG_DIR
from .datasets import split_loader_fn_spec

# (flag, kwargs, group).  Flag strings follow click conventions.
OPTIONS = [
    # ------------------------------------------------------------------ Basic
    ("--algo", dict(default="gspo", show_default=True, help="Algorithm: sft, dpo, gspo, grpo, ppo or a registered name."), "Basic"),
    ("--ckpt", dict(default=None, help="Actor checkpoint: local HF directory or Hugging Face repo id."), "Basic"),
    ("--dataset-path", dict(default=None, help="Dataset file, directory or HF reference repo[:config[:split]]."), "Basic"),
    ("--dataset-loader-fn", dict(default=None, help="file.py[:fn] returning normalised rows."), "Basic"),
    ("--reward-fn-path", dict(default=None, help="Python file defining reward_fn(record)."), "Basic"),
    ("--ref-ckpt", dict(default=None, help="Reference policy checkpoint (PPO / DPO); defaults to --ckpt."), "Basic"),
    ("--reward-ckpt", dict(default=None, help="Reward model checkpoint (PPO)."), "Basic"),
    ("--critic-ckpt", dict(default=None, help="Critic initial checkpoint (PPO); defaults to --ckpt."), "Basic"),
    ("--epochs", dict(default=10, show_default=True, type=int), "Basic"),
    ("--max-steps", dict(default=None, type=int, help="Stop after this many optimizer steps."), "Basic"),
    ("--tune-params", dict(is_flag=True, default=False, help="Probe memory and pick rollout / train batch sizes."), "Basic"),
    # ---------------------------------------------------------------- Rollout
    ("--mem-frac", dict(default=0.9, show_default=True, type=float), "Rollout"),
    ("--tune-max-samples", dict(default=256, show_default=True, type=int), "Rollout"),
    ("--tp-size", dict(default=4, show_default=True, type=int), "Rollout"),
    ("--world-size", dict(default=8, show_default=True, type=int), "Rollout"),
    ("--batch-size", dict(default=32, show_default=True, type=int, help="Prompts per step."), "Rollout"),
    ("--n-samples", dict(default=8, show_default=True, type=int, help="Completions per prompt."), "Rollout"),
    ("--max-prompt-tokens", dict(default=1024, show_default=True, type=int), "Rollout"),
    ("--max-new-tokens", dict(default=3071, show_default=True, type=int), "Rollout"),
    ("--max-context-len", dict(default=None, type=int), "Rollout"),
    ("--temperature", dict(default=1.0, show_default=True, type=float), "Rollout"),
    ("--top-k", dict(default=-1, show_default=True, type=int), "Rollout"),
    ("--top-p", dict(default=1.0, show_default=True, type=float), "Rollout"),
    ("--greedy", dict(is_flag=True, default=False), "Rollout"),
    ("--max-running-prompts", dict(default=None, type=int, help="Default: batch_size * n_samples."), "Rollout"),
    ("--drop-rollout-state", dict(is_flag=True, default=False, help="Free KV cache and decode graphs before training."), "Rollout"),
    ("--eager-decode", dict(is_flag=True, default=False, help="Disable CUDA-graph decode."), "Rollout"),
    ("--attn-backend", dict(default="flash", show_default=True, type=click.Choice(["flash", "native"])), "Rollout"),
    ("--kv-dtype", dict(default="bf16", show_default=True, type=click.Choice(["bf16", "fp8"])), "Rollout"),
    ("--expert-parallel", dict(is_flag=True, default=False,
                               help="Mixture-of-experts models: deal the experts out over the GPUs (needs --tp-size 1)."), "Rollout"),
    ("--disable-thinking", dict(is_flag=True, default=False), "Rollout"),
    ("--agent-fn", dict(default=None, help="Python file defining run_agent(ctx, batch)."), "Rollout"),
    ("--agent-timeout-s", dict(default=300.0, show_default=True, type=float), "Rollout"),
    # ------------------------------------------------------------------ Train
    ("--mini-bs", dict(default=16, show_default=True, type=int, help="Sequences per micro-batch (before the DP split)."), "Train"),
    ("--score-micro-bs", dict(default=8, show_default=True, type=int), "Train"),
    ("--gradient-accumulation-steps", dict(default=None, type=int, help="Default: one optimizer step per batch."), "Train"),
    ("--lr", dict(default=1e-6, show_default=True, type=float), "Train"),
    ("--min-lr", dict(default=1e-7, show_default=True, type=float), "Train"),
    ("--lr-decay-steps", dict(default=1000, show_default=True, type=int), "Train"),
    ("--lr-decay-style", dict(default="cosine", show_default=True, type=click.Choice(["constant", "linear", "cosine"])), "Train"),
    ("--adam-beta1", dict(default=0.9, show_default=True, type=float), "Train"),
    ("--adam-beta2", dict(default=0.999, show_default=True, type=float), "Train"),
    ("--adam-8bit", dict(is_flag=True, default=False), "Train"),
    ("--weight-decay", dict(default=0.01, show_default=True, type=float), "Train"),
    ("--grad-clip-norm", dict(default=1.0, show_default=True, type=float), "Train"),
    ("--activation-checkpointing/--no-activation-checkpointing", dict(default=True, show_default=True), "Train"),
    ("--train-tool-results", dict(is_flag=True, default=False), "Train"),
    ("--gspo-clip-eps", dict(default=3e-4, show_default=True, type=float), "Train"),
    ("--grpo-clip-eps", dict(default=0.2, show_default=True, type=float), "Train"),
    ("--dpo-beta", dict(default=0.1, show_default=True, type=float), "Train"),
    ("--critic-warmup-steps", dict(default=20, show_default=True, type=int), "Train"),
    ("--critic-lr", dict(default=1e-5, show_default=True, type=float), "Train"),
    ("--use-kl-loss/--no-use-kl-loss", dict(default=True, show_default=True), "Train"),
    ("--kl-loss-coef", dict(default=0.001, show_default=True, type=float), "Train"),
    ("--kl-loss-type", dict(default="low_var_kl", show_default=True, type=click.Choice(["kl", "abs", "mse", "low_var_kl"])), "Train"),
    ("--clip-eps", dict(default=0.2, show_default=True, type=float), "Train"),
    ("--clip-ratio-c", dict(default=3.0, show_default=True, type=float), "Train"),
    ("--value-clip-eps", dict(default=0.5, show_default=True, type=float), "Train"),
    ("--value-loss-coef", dict(default=0.5, show_default=True, type=float), "Train"),
    ("--gamma", dict(default=1.0, show_default=True, type=float), "Train"),
    ("--lam", dict(default=0.95, show_default=True, type=float), "Train"),
    # ------------------------------------------------------------- Checkpoint
    ("--save-path", dict(default=None, help="Directory for step_{n:06d} checkpoints."), "Checkpoint"),
    ("--save-interval", dict(default=100, show_default=True, type=int), "Checkpoint"),
    # ---------------------------------------------------------- Observability
    ("--metrics-log-dir", dict(default=DEFAULT_METRICS_LOG_DIR, show_default=True), "Observability"),
]
GROUP_ORDER = ["Basic", "Rollout", "Train", "Checkpoint", "Observability"]

# Help text of the options that do not carry one above (kept apart so that the table stays one line per flag).
_HELP = {
    "--epochs": "Passes over the dataset.",
    "--mem-frac": "Fraction of GPU memory --tune-params may plan for.",
    "--tune-max-samples": "Largest n_samples * batch the tuner tries.",
    "--tp-size": "Tensor-parallel width (training and rollout).",
    "--world-size": "Number of GPUs; data-parallel width is world / tp.",
    "--max-prompt-tokens": "Prompts longer than this are skipped (and counted in the log).",
    "--max-new-tokens": "Completion budget per sample.",
    "--max-context-len": "Cap on a whole trajectory (agentic: prompt plus every turn); default: the model's limit.",
    "--temperature": "Sampling temperature.",
    "--top-k": "Keep the k most likely tokens (-1: off).",
    "--top-p": "Nucleus sampling mass (1.0: off).",
    "--greedy": "Arg-max decoding (temperature 0).",
    "--attn-backend": "Accepted for compatibility; both values select this package's kernels.",
    "--kv-dtype": "KV page storage: bf16, or fp8 (e4m3 with one scale per token and KV head).",
    "--disable-thinking": "Render chat templates with enable_thinking=False where the template takes it.",
    "--agent-timeout-s": "Time limit of one proxied chat completion.",
    "--score-micro-bs": "Sequences per scoring micro-batch of the reference / critic / reward roles.",
    "--lr": "Peak learning rate.",
    "--min-lr": "Floor of the decay schedule.",
    "--lr-decay-steps": "Optimizer steps over which the rate decays to --min-lr.",
    "--lr-decay-style": "Shape of the decay.",
    "--adam-beta1": "AdamW beta1.",
    "--adam-beta2": "AdamW beta2.",
    "--adam-8bit": "Block-scaled 8-bit AdamW moments (fp32 master weights stay).",
    "--weight-decay": "Decoupled weight decay.",
    "--grad-clip-norm": "Global gradient-norm clip.",
    "--activation-checkpointing/--no-activation-checkpointing":
        "Recompute layer activations in backward when memory is short (decided from free memory per micro-batch).",
    "--train-tool-results": "Agentic: also train on tool-result tokens (default: context only).",
    "--gspo-clip-eps": "GSPO sequence-ratio clip.",
    "--grpo-clip-eps": "GRPO token-ratio clip.",
    "--dpo-beta": "DPO temperature.",
    "--critic-warmup-steps": "PPO: steps that train only the critic.",
    "--critic-lr": "PPO critic learning rate.",
    "--use-kl-loss/--no-use-kl-loss": "PPO: add a KL-to-reference penalty to the actor loss.",
    "--kl-loss-coef": "PPO: weight of that penalty.",
    "--kl-loss-type": "PPO: KL estimator.",
    "--clip-eps": "PPO ratio clip.",
    "--clip-ratio-c": "PPO dual-clip bound for negative advantages.",
    "--value-clip-eps": "PPO value clip.",
    "--value-loss-coef": "PPO value-loss weight.",
    "--gamma": "PPO discount.",
    "--lam": "PPO GAE lambda.",
    "--save-interval": "Save every this many steps.",
    "--metrics-log-dir": "TensorBoard event files (metrics.jsonl without a TensorBoard package).",
}
for _flag, _kw, _group in OPTIONS:
    _kw.setdefault("help", _HELP.get(_flag))



def option_name(flag: str) -> str:
    return flag.split("/")[0].lstrip("-").replace("-", "_")


class GroupedCommand(click.Command):
    """``--help`` lists options under the five group headings."""

    def format_options(self, ctx, formatter):
        by_name = {option_name(flag): group for flag, _kw, group in OPTIONS}
        grouped: dict[str, list] = {g: [] for g in GROUP_ORDER}
        other = []
        for param in self.get_params(ctx):
            rec = param.get_help_record(ctx)
            if rec is None:
                continue
            (grouped[by_name[param.name]] if param.name in by_name else other).append(rec)
        for g in GROUP_ORDER:
            if grouped[g]:
                with formatter.section(f"{g} options"):
                    formatter.write_dl(grouped[g])
        if other:
            with formatter.section("Other options"):
                formatter.write_dl(other)


# ------------------------------------------------------------------- hook pre-flight
def _find_function(tree: ast.Module, name: str):
    for node in tree.body:
        if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef)) and node.name == name:
            return node
    return None


def _accepts_positional(fn, count: int) -> bool:
    a = fn.args
    n_pos = len(a.posonlyargs) + len(a.args)
    required = n_pos - len(a.defaults)
    return required <= count if a.vararg is not None else required <= count <= n_pos


def validate_python_callable(path: Path, symbol: str, *, option: str, expected: str, positional_args: int | None = None):
    if not path.exists():
        raise click.UsageError(f"{option} file does not exist: {path}; expected callable {expected}")
    if not path.is_file():
        raise click.UsageError(f"{option} path is not a file: {path}; expected callable {expected}")
    try:
        tree = ast.parse(path.read_text(encoding="utf-8"), filename=str(path))
    except (OSError, SyntaxError, UnicodeDecodeError) as exc:
        raise click.UsageError(f"{option} cannot parse Python file: {path}; expected callable {expected}; "
                               f"{type(exc).__name__}: {exc}") from exc
    fn = _find_function(tree, symbol)
    if fn is None or (positional_args is not None and not _accepts_positional(fn, positional_args)):
        raise click.UsageError(f"{option} {path} must define callable {expected}")


def preflight_task_hooks(args, algorithm) -> None:
    if args.dataset_loader_fn is not None:
        try:
            path, fn_name = split_loader_fn_spec(args.dataset_loader_fn)
        except ValueError as exc:
            raise click.UsageError(str(exc)) from exc
        validate_python_callable(path, fn_name, option="--dataset-loader-fn", expected=f"{fn_name}(...)", positional_args=1)
    if algorithm.requires_rollout and args.reward_fn_path is not None:
        validate_python_callable(Path(args.reward_fn_path).expanduser().resolve(), "reward_fn",
                                 option="--reward-fn-path", expected="reward_fn(record)", positional_args=1)
    if args.agent_fn is not None:
        validate_python_callable(Path(args.agent_fn).expanduser().resolve(), "run_agent", option="--agent-fn",
                                 expected="run_agent(ctx, batch)", positional_args=2)


# ------------------------------------------------------------------------ validation
# (option attribute, flag, rule, scope).  rule: ">0" strictly positive, ">=0" non-negative;
# scope: None = always, "rollout" = rollout algorithms only, else the one algorithm it applies to.
_RANGE_RULES = [
    ("save_interval", "--save-interval", ">0", None), ("epochs", "--epochs", ">0", None),
    ("max_steps", "--max-steps", ">0", None), ("tp_size", "--tp-size", ">0", None),
    ("world_size", "--world-size", ">0", None), ("batch_size", "--batch-size", ">0", None),
    ("n_samples", "--n-samples", ">0", "rollout"), ("mini_bs", "--mini-bs", ">0", None),
    ("score_micro_bs", "--score-micro-bs", ">0", None),
    ("gradient_accumulation_steps", "--gradient-accumulation-steps", ">0", None),
    ("max_prompt_tokens", "--max-prompt-tokens", ">0", None), ("max_new_tokens", "--max-new-tokens", ">0", None),
    ("max_context_len", "--max-context-len", ">0", None),
    ("max_running_prompts", "--max-running-prompts", ">0", "rollout"),
    ("agent_timeout_s", "--agent-timeout-s", ">0", None), ("lr", "--lr", ">0", None),
    ("min_lr", "--min-lr", ">=0", None), ("lr_decay_steps", "--lr-decay-steps", ">0", None),
    ("adam_beta1", "--adam-beta1", ">0", None), ("adam_beta2", "--adam-beta2", ">0", None),
    ("weight_decay", "--weight-decay", ">=0", None), ("grad_clip_norm", "--grad-clip-norm", ">0", None),
    ("temperature", "--temperature", ">0", "rollout"), ("top_p", "--top-p", ">0", "rollout"),
    ("gspo_clip_eps", "--gspo-clip-eps", ">0", "gspo"), ("grpo_clip_eps", "--grpo-clip-eps", ">0", "grpo"),
    ("dpo_beta", "--dpo-beta", ">0", "dpo"), ("critic_lr", "--critic-lr", ">0", "ppo"),
    ("kl_loss_coef", "--kl-loss-coef", ">0", "ppo"), ("clip_eps", "--clip-eps", ">0", "ppo"),
    ("clip_ratio_c", "--clip-ratio-c", ">0", "ppo"), ("value_clip_eps", "--value-clip-eps", ">0", "ppo"),
    ("value_loss_coef", "--value-loss-coef", ">0", "ppo"), ("gamma", "--gamma", ">0", "ppo"),
    ("lam", "--lam", ">0", "ppo"), ("critic_warmup_steps", "--critic-warmup-steps", ">=0", None),
]


def algorithm_for_cli(name: str):
    from ..api.algorithms import get_algorithm

    try:
        return get_algorithm(name)
    except ValueError as exc:
        raise click.UsageError(str(exc)) from exc


def _defaults() -> dict:
    out = {}
    for flag, kw, _group in OPTIONS:
        out[option_name(flag)] = kw.get("default")
    return out


def validate_options(args, algorithm) -> None:
    if args.ckpt is None:
        raise click.UsageError("--ckpt is required")
    if args.dataset_path is None:
        raise click.UsageError("--dataset-path is required")
    if algorithm.name == "sft" and args.dataset_loader_fn is None:
        raise click.UsageError("--dataset-loader-fn is required for --algo sft")
    if args.tune_params and not algorithm.requires_rollout:
        raise click.UsageError("--tune-params currently supports rollout-based algorithms")
    if not 0 < float(args.mem_frac) <= 1:
        raise click.UsageError("--mem-frac must be in (0, 1]")
    if int(args.tune_max_samples) <= 0:
        raise click.UsageError("--tune-max-samples must be positive")
    if algorithm.requires_rollout and args.reward_fn_path is None and args.reward_ckpt is None:
        raise click.UsageError("--reward-fn-path or --reward-ckpt is required")
    for attr, flag, rule, scope in _RANGE_RULES:
        if scope == "rollout" and not algorithm.requires_rollout:
            continue
        if scope not in (None, "rollout") and scope != algorithm.name:
            continue
        value = getattr(args, attr)
        if value is None:
            continue
        if rule == ">0" and value <= 0:
            raise click.UsageError(f"{flag} must be positive")
        if rule == ">=0" and value < 0:
            raise click.UsageError(f"{flag} must be non-negative")
        if attr == "world_size" and args.world_size % args.tp_size != 0:
            raise click.UsageError("--world-size must be divisible by --tp-size")


# CLI attribute -> config field, where the names differ.
_RENAMES = {"lr": "optimizer_lr", "min_lr": "optimizer_min_lr", "adam_beta1": "optimizer_beta1",
            "adam_beta2": "optimizer_beta2"}


def config_class_for(algorithm):
    """The narrowest config dataclass an algorithm needs: offline trainers never see rollout,
    reward or clip fields."""
    from ..api import trainer_config as tc

    if algorithm.name == "dpo":
        return tc.DPOTrainerConfig
    if algorithm.name == "sft":
        return tc.TrainerConfig
    if algorithm.name == "ppo":
        return tc.PPOTrainerConfig
    return tc.PolicyTrainerConfig


def trainer_config_from_args(args):
    from dataclasses import fields

    algorithm = algorithm_for_cli(args.algo)
    cls = config_class_for(algorithm)
    values = {_RENAMES.get(k, k): v for k, v in vars(args).items()}
    values["algo"] = algorithm.name
    values["keep_rollout_state"] = not args.drop_rollout_state
    values["chat_template_enable_thinking"] = False if args.disable_thinking else None
    wanted = {f.name for f in fields(cls)}
    return cls(**{k: v for k, v in values.items() if k in wanted})


def trainer_config_from_options(**options):
    """Validate click option values and build the typed trainer config.  Missing keys take the CLI
    defaults, so tests and programmatic callers may pass only what they set."""
    merged = _defaults()
    merged.update(options)
    args = SimpleNamespace(**merged)
    algorithm = algorithm_for_cli(args.algo)
    validate_options(args, algorithm)
    preflight_task_hooks(args, algorithm)
    return trainer_config_from_args(args)


# --------------------------------------------------------------------------- summary
def _opt(value, default="none") -> str:
    return default if value is None else str(value)


def _yn(value: bool) -> str:
    return "yes" if value else "no"


def summary_sections(config, *, reward_ckpt: str | None = None) -> list[tuple[str, list[tuple[str, str]]]]:
    from ..api.algorithms import get_algorithm
    from ..api.trainer_config import PolicyTrainerConfig, PPOTrainerConfig, RolloutTrainerConfig

    algorithm = get_algorithm(config.algo)
    loss_fn = algorithm.make_loss_fn(config)
    loss_name = getattr(getattr(loss_fn, "func", loss_fn), "__name__", type(loss_fn).__name__)
    if isinstance(config, PPOTrainerConfig):
        reward_ckpt = config.reward_ckpt
    rollout = [("batch_size", str(config.batch_size)), ("max_prompt_tokens", str(config.max_prompt_tokens)),
               ("max_new_tokens", str(config.max_new_tokens)),
               ("max_context_len", _opt(config.max_context_len, "model limit"))]
    if isinstance(config, RolloutTrainerConfig):
        rollout += [("n_samples", str(config.n_samples)),
                    ("max_running_prompts", str(config.resolved_max_running_prompts())),
                    ("sampling", f"greedy={_yn(config.greedy)}, temperature={config.temperature}, "
                                 f"top_k={config.top_k}, top_p={config.top_p}")]
    else:
        rollout += [("n_samples", "n/a"), ("max_running_prompts", "n/a"), ("sampling", "n/a")]
    return [
        ("Task", [("algo", config.algo), ("trainer", algorithm.resolve_trainer_cls().__name__), ("loss_fn", loss_name),
                  ("ckpt", config.ckpt), ("dataset_path", config.dataset_path),
                  ("dataset_loader_fn", _opt(config.dataset_loader_fn)),
                  ("reward_fn_path", _opt(getattr(config, "reward_fn_path", None)) if isinstance(config, PolicyTrainerConfig) else "n/a"),
                  ("reward_ckpt", _opt(reward_ckpt)), ("agent_fn", _opt(config.agent_fn)), ("epochs", str(config.epochs))]),
        ("Runtime", [("world_size", str(config.world_size)), ("tp_size", str(config.tp_size)),
                     ("dp_size", str(config.world_size // config.tp_size) if config.tp_size else "n/a"),
                     ("attn_backend", config.attn_backend), ("kv_dtype", config.kv_dtype),
                     ("expert_parallel", _yn(config.expert_parallel)),
                     ("decode", "eager" if config.eager_decode else "cuda-graph"),
                     ("keep_rollout_state", _yn(config.keep_rollout_state)),
                     ("activation_checkpointing", _yn(config.activation_checkpointing)),
                     ("thinking", _opt(config.chat_template_enable_thinking, "tokenizer default"))]),
        ("Rollout", rollout),
        ("Training", [("max_steps", _opt(config.max_steps)), ("mini_bs", str(config.mini_bs)),
                      ("score_micro_bs", str(config.score_micro_bs)),
                      ("gradient_accumulation_steps", _opt(config.gradient_accumulation_steps, "auto")),
                      ("optimizer", f"lr={config.optimizer_lr}, min_lr={config.optimizer_min_lr}, "
                                    f"decay={config.lr_decay_style}/{config.lr_decay_steps}, "
                                    f"betas=({config.optimizer_beta1}, {config.optimizer_beta2}), "
                                    f"weight_decay={config.weight_decay}, adam_8bit={_yn(config.adam_8bit)}"),
                      ("grad_clip_norm", str(config.grad_clip_norm))]),
        ("Outputs", [("save_path", _opt(config.save_path)), ("save_interval", str(config.save_interval)),
                     ("metrics_log_dir", _opt(config.metrics_log_dir))]),
    ]


def format_training_config_summary(config, *, reward_ckpt: str | None = None, color: bool = False) -> str:
    import shutil
    import textwrap

    def style(text, **kw):
        return click.style(text, **kw) if color else text

    width = shutil.get_terminal_size(fallback=(100, 24)).columns
    lines = [style("AReno-B200 training config", fg="bright_white", bold=True)]
    for title, rows in summary_sections(config, reward_ckpt=reward_ckpt):
        key_w = max(len(k) for k, _ in rows)
        val_w = max(20, width - key_w - 4)
        lines += ["", style(title, fg="bright_blue", bold=True), style("-" * len(title), fg="bright_black")]
        for key, value in rows:
            chunks = textwrap.wrap(value, width=val_w, break_long_words=True, break_on_hyphens=False) or [""]
            lines.append("  " + style(key.ljust(key_w), fg="bright_black") + "  " + chunks[0])
            lines += ["  " + " " * key_w + "  " + c for c in chunks[1:]]
    if config.save_path is None:
        lines.append(style("WARNING", fg="yellow", bold=True)
                     + ": no checkpoint output path configured (--save-path); checkpoints will not be saved.")
    return "\n".join(lines)


# ------------------------------------------------------------------------------- run
def run(trainer_config, *, backend_type=None, load_dataset=None, load_from_disk=None):
    """Build the trainer registered for ``config.algo`` and run ``fit()`` to completion."""
    from .. import api
    from ..api.algorithms import get_algorithm
    from ..api.rewards import load_reward_fn
    from ..api.trainer_config import PolicyTrainerConfig
    from ..api.trainer_factory import build_trainer
    from .datasets import load_dataset_for_training
    from .model_refs import resolve_model_refs_for_config

    trainer_config = resolve_model_refs_for_config(trainer_config)
    loss_fn = get_algorithm(trainer_config.algo).make_loss_fn(trainer_config)
    reward_path = trainer_config.reward_fn_path if isinstance(trainer_config, PolicyTrainerConfig) else None
    reward_fn = load_reward_fn(reward_path) if reward_path else None
    instance = api.Trainer(trainer_config.world_size, trainer_config.ckpt, backend_type=backend_type or api.Areno,
                           metrics_log_dir=trainer_config.metrics_log_dir, custom_config=trainer_config.areno_config())
    dataset = load_dataset_for_training(trainer_config.dataset_path, dataset_loader_fn=trainer_config.dataset_loader_fn,
                                        load_dataset=load_dataset, load_from_disk=load_from_disk)
    trainer = build_trainer(trainer_config, instance=instance, dataset=dataset, reward_fn=reward_fn, loss_fn=loss_fn)
    trainer.fit()
    return trainer


def _train_callback(**options) -> None:
    import logging

    trainer_config = trainer_config_from_options(**options)
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(name)s: %(message)s")
    if options.get("tune_params"):
        from .auto_tune import auto_tune_config, format_auto_tune_summary

        result = auto_tune_config(trainer_config, mem_frac=options["mem_frac"],
                                  auto_max_samples=options["tune_max_samples"])
        trainer_config = result.config
        line = format_auto_tune_summary(result)
        if line:
            click.echo(line, color=True)
    click.echo(format_training_config_summary(trainer_config, reward_ckpt=options.get("reward_ckpt"), color=True),
               color=True)
    run(trainer_config)


def _build_command() -> click.Command:
    fn = _train_callback
    for flag, kw, _group in reversed(OPTIONS):
        fn = click.option(flag, **kw)(fn)
    return click.command(name="train", cls=GroupedCommand, context_settings={"max_content_width": 120, "help_option_names": ["-h", "--help"]},
                         help="Train a model with SFT, DPO, GSPO, GRPO, PPO or a registered algorithm.")(fn)


train_command = _build_command()


def main() -> None:
    train_command.main(prog_name="areno train")


if __name__ == "__main__":
    main()
