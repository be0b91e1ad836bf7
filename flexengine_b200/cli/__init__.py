"""``flexengine <command> [options]``: one dispatcher over sub-commands, in the manner of the
reference's command line (src/flexengine/serving/cli/__init__.py:8-38).  The server
commands of the reference are not part of this engine; ``generate`` takes the engine
options of its ``serve`` command under the same names (src/flexengine/serving/cli/server.py:7-54)."""
from __future__ import annotations

import importlib
import sys
from collections.abc import Sequence

COMMANDS = {
    "generate": ("flexengine_b200.cli.generate", "main", "Generate tokens for prompts given as text or token ids"),
    "replay": ("flexengine_b200.engine.replay", "main", "Replay token ids step by step and write logits"),
    "random-model": ("flexengine_b200.cli.random_model", "main", "Write a model folder with seeded random weights"),
    "build": ("flexengine_b200.cli.build", "main", "Compile the CUDA kernel libraries"),
    "bench": ("flexengine_b200.cli.bench", "main", "Decode and prefill throughput on the Qwen2.5-7B shape (one JSON line)"),
}


def usage() -> str:
    lines = ["usage: flexengine <command> [options]", "", "commands:"]
    width = max(map(len, COMMANDS))
    lines.extend(f"  {name:<{width}}  {text}" for name, (_, _, text) in COMMANDS.items())
    return "\n".join(lines)


def main(argv: Sequence[str] | None = None) -> None:
    arguments = list(sys.argv[1:] if argv is None else argv)
    if not arguments or arguments[0] in {"-h", "--help"}:
        print(usage())
        return
    command = arguments.pop(0)
    if command not in COMMANDS:
        raise SystemExit(f"unknown command: {command}\n\n{usage()}")
    module_name, function_name, _ = COMMANDS[command]
    module = importlib.import_module(module_name)
    code = getattr(module, function_name)(arguments)
    if code:
        raise SystemExit(code)


if __name__ == "__main__":
    main()
