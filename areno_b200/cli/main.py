"""``areno`` command group.  Sub-commands are imported only when selected, so ``areno --help`` and
``areno check`` do not pay for torch or the engine (``areno/cli/main.py:14-48`` in the reference)."""

from __future__ import annotations

import importlib

import click

COMMANDS = {
    "check": ("areno_b200.cli.diagnostics", "check_command", "Check whether this machine is ready to run the framework."),
    "env": ("areno_b200.cli.diagnostics", "env_command", "Print an environment / support report."),
    "train": ("areno_b200.cli.train", "train_command", "Run SFT, DPO, GSPO, GRPO or PPO training."),
    "serve": ("areno_b200.cli.serve", "serve_command", "Serve an OpenAI-compatible chat API."),
}


class LazyGroup(click.Group):
    def list_commands(self, ctx):
        return sorted(COMMANDS)

    def get_command(self, ctx, name):
        entry = COMMANDS.get(name)
        if entry is None:
            return None
        return getattr(importlib.import_module(entry[0]), entry[1])

    def format_commands(self, ctx, formatter):
        with formatter.section("Commands"):
            formatter.write_dl([(name, COMMANDS[name][2]) for name in self.list_commands(ctx)])


@click.group(cls=LazyGroup, context_settings={"help_option_names": ["-h", "--help"]},
             help="Run LLM post-training jobs on B200 nodes or start the OpenAI-compatible server.")
def main() -> None:
    pass


if __name__ == "__main__":
    main()
