"""``flexengine <command> [options]``.

One program with sub-commands, as the reference has (its ``flexengine serve|benchmark|...``,
src/flexengine/serving/cli/__init__.py); the commands here are this engine's: the reference's server and
experiment runners are not part of it.  ``generate`` takes the engine options of the reference's ``serve``
under the same names (src/flexengine/serving/cli/server.py:7-54).  A command's module is imported only when it
is chosen, so ``flexengine --help`` does not load PyTorch.
"""
from __future__ import annotations

import argparse
import sys
from importlib import import_module
from typing import NamedTuple


class Command(NamedTuple):
    module: str          # has ``main(argv) -> int``
    summary: str


COMMANDS = {
    "generate": Command("flexengine_b200.cli.generate", "generate tokens for prompts given as text or token ids"),
    "replay": Command("flexengine_b200.engine.replay", "feed given token ids step by step and write the logits"),
    "bench": Command("flexengine_b200.bench", "measure decode, prefill and serving workloads (one JSON line)"),
    "random-model": Command("flexengine_b200.cli.random_model", "write a model folder with seeded random weights"),
    "build": Command("flexengine_b200.cli.build", "compile the CUDA kernel libraries for sm_100a"),
}


def _parser() -> argparse.ArgumentParser:
    listing = "\n".join(f"  {name:<14}{c.summary}" for name, c in COMMANDS.items())
    p = argparse.ArgumentParser(prog="flexengine", formatter_class=argparse.RawDescriptionHelpFormatter,
                                description="A single-GPU inference engine for NVIDIA B200.",
                                epilog="commands:\n" + listing + "\n\n'flexengine <command> --help' shows a command's options.")
    p.add_argument("command", choices=list(COMMANDS), metavar="<command>")
    p.add_argument("options", nargs=argparse.REMAINDER, help="passed to the command")
    return p


def main(argv=None) -> int:
    chosen = _parser().parse_args(sys.argv[1:] if argv is None else list(argv))
    return int(import_module(COMMANDS[chosen.command].module).main(chosen.options) or 0)
