"""End-to-end training smoke test for CI: a few optimizer steps of an RL algorithm on arithmetic word problems.

    python ci/train_smoke.py --algo gspo --steps 2 --device cpu
    python ci/train_smoke.py --algo grpo --steps 3 --device cuda --world-size 2
    python ci/train_smoke.py --algo ppo --steps 2        # reference and critic roles from the same tiny checkpoint
    python ci/train_smoke.py --algo dpo --steps 2        # preference pairs, reference role
    python ci/train_smoke.py --algo sft --steps 2        # prompt / response rows through this file's loader
    python ci/train_smoke.py --algo grpo --steps 2 --agentic   # agent function + local OpenAI-compatible proxy

Everything is made on the spot in a temporary directory, so the job needs no network: a tiny random-weight
``qwen2`` checkpoint, a word-level tokenizer saved in the Hugging Face format, a JSONL dataset of additions and this
file as the reward function (``--reward-fn-path ci/train_smoke.py``).  The run goes through the same code as
``areno train`` (option validation, dataset loading, trainer factory, ``fit``) and must finish the requested number
of steps, write TensorBoard / JSONL scalars and save a loadable checkpoint.  Role of ``ci/modal_gsm8k_gspo.py`` in
the reference, without the hosted GPU service and the downloaded model.
"""

from __future__ import annotations

import argparse
import json
import os
import random
import re
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


# ------------------------------------------------------------------ reward (loaded by --reward-fn-path)
def reward_fn(record) -> float:
    """1.0 when the last integer of the completion equals the answer, else 0."""
    found = re.findall(r"-?\d+", getattr(record, "completion", "") or "")
    try:
        return 1.0 if found and int(found[-1]) == int(str(getattr(record, "answer", "")).strip()) else 0.0
    except ValueError:
        return 0.0


# ------------------------------------------------------------------ fixtures
WORDS = ["what", "is", "plus", "the", "sum", "of", "and", "answer", "?", ":", "+", "="] + [str(i) for i in range(200)]


def write_tokenizer(path: str) -> int:
    """A whitespace word-level tokenizer with pad / bos / eos / unk, saved so that ``AutoTokenizer`` loads it."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    vocab = {"<pad>": 0, "<s>": 1, "</s>": 2, "<unk>": 3}
    for w in WORDS:
        vocab.setdefault(w, len(vocab))
    tok = Tokenizer(models.WordLevel(vocab=vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, pad_token="<pad>", bos_token="<s>", eos_token="</s>",
                                   unk_token="<unk>")
    fast.save_pretrained(path)
    return len(vocab)


def write_checkpoint(path: str, vocab: int, seed: int = 0) -> None:
    import torch

    from areno_b200.engine.config import ModelConfig
    from areno_b200.models import registry
    from areno_b200.parallel.context import single_process_context

    single_process_context()
    cfg = ModelConfig(model_type="qwen2", vocab_size=max(256, (vocab + 63) // 64 * 64), hidden_size=128,
                      intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                      head_dim=32, rope_theta=1e4, qk_norm=False, qkv_bias=True, dtype=torch.bfloat16,
                      max_position_embeddings=512)
    adapter = registry.get_adapter("qwen2")
    model = adapter.build(cfg)
    adapter.init_random(model, seed)
    adapter.save_weights(model, path, cfg)


def write_dataset(path: str, n: int, seed: int = 0) -> None:
    """Rows carry every column any algorithm reads: ``answer`` (RL), ``response`` (SFT), ``chosen`` / ``rejected`` (DPO)."""
    rng = random.Random(seed)
    with open(path, "w") as f:
        for _ in range(n):
            a, b = rng.randrange(100), rng.randrange(100)
            good, bad = f"the answer : {a + b}", f"the answer : {(a + b + 1 + rng.randrange(50)) % 200}"
            f.write(json.dumps({"prompt": f"what is {a} plus {b} ?", "answer": str(a + b), "response": good,
                                "chosen": good, "rejected": bad}) + "\n")


def load_training_dataset(dataset_path, *, default_loader, load_dataset, load_from_disk):
    """Loader for ``--dataset-loader-fn ci/train_smoke.py`` (SFT requires one): the JSONL rows as they are."""
    with open(dataset_path) as f:
        return [json.loads(line) for line in f if line.strip()]


# ------------------------------------------------------------------ run
def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--algo", default="gspo", choices=["gspo", "grpo", "ppo", "dpo", "sft"])
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--world-size", type=int, default=1)
    ap.add_argument("--tp-size", type=int, default=1)
    ap.add_argument("--agentic", action="store_true",
                    help="rollouts through an agent function and the local OpenAI-compatible proxy (the one-step "
                         "tic-tac-toe example) instead of plain prompt -> completion")
    ap.add_argument("--keep", default=None, help="directory to keep the artefacts in (default: a temporary one)")
    args = ap.parse_args(argv)
    if args.device == "cpu":
        os.environ["CUDA_VISIBLE_DEVICES"] = ""     # the engine picks CPU + gloo when no GPU is visible

    from areno_b200.cli import train as cli_train

    with tempfile.TemporaryDirectory() as tmp:
        work = args.keep or tmp
        os.makedirs(work, exist_ok=True)
        ckpt, data, save, logs = (os.path.join(work, n) for n in ("model", "train.jsonl", "saved", "tfevent"))
        os.makedirs(ckpt, exist_ok=True)
        write_checkpoint(ckpt, write_tokenizer(ckpt))
        write_dataset(data, 64)
        options = dict(
            algo=args.algo, ckpt=ckpt, dataset_path=data, save_path=save,
            save_interval=args.steps, metrics_log_dir=logs, epochs=1, max_steps=args.steps, tp_size=args.tp_size,
            world_size=args.world_size, batch_size=4, n_samples=4, mini_bs=8, max_prompt_tokens=32, max_new_tokens=8,
            lr=1e-4, activation_checkpointing=False)
        me = os.path.abspath(__file__)
        if args.algo in ("gspo", "grpo", "ppo"):
            options["reward_fn_path"] = me
        if args.algo == "ppo":
            options.update(ref_ckpt=ckpt, critic_ckpt=ckpt, critic_warmup_steps=0)
        if args.algo == "dpo":
            options.update(ref_ckpt=ckpt, dataset_loader_fn=me)
        if args.algo == "sft":
            options.update(dataset_loader_fn=me)
        if args.agentic:
            if args.algo not in ("gspo", "grpo"):
                ap.error("--agentic goes with --algo gspo or grpo")
            ex = os.path.join(ROOT, "examples", "agentic", "tictactoe")
            options.update(dataset_path="tictactoe:16", dataset_loader_fn=os.path.join(ex, "dataset_loader_no_tool.py"),
                           agent_fn=os.path.join(ex, "run_agent_no_tool.py"),
                           reward_fn_path=os.path.join(ex, "reward_no_tool.py"), max_prompt_tokens=128,
                           agent_timeout_s=120)
        config = cli_train.trainer_config_from_options(**options)
        trainer = cli_train.run(config)
        steps_done = int(getattr(trainer, "global_step", getattr(trainer, "step", args.steps)))
        saved = [d for d in (os.listdir(save) if os.path.isdir(save) else [])]
        scalars = os.listdir(logs) if os.path.isdir(logs) else []
        print(json.dumps({"algo": args.algo, "steps_requested": args.steps, "steps_done": steps_done,
                          "checkpoints": saved, "metric_files": scalars}))
        if not saved:
            print("no checkpoint was written", file=sys.stderr)
            return 1
        if not scalars:
            print("no metrics were written", file=sys.stderr)
            return 1
        from areno_b200.models import registry

        registry.config_from_pretrained(os.path.join(save, sorted(saved)[-1]))     # the saved directory is loadable
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
