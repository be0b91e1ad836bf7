"""``flexengine bench [options]``: the checkout's ``bench.py`` (decode and prefill throughput on the
Qwen2.5-7B shape with random weights, one JSON line) under the dispatcher, so that every entry
point is reachable from one command.  The reference's benchmarks drive its HTTP server
(src/flexengine/research/benchmark/runner.py:26-105); this one runs in process."""
from __future__ import annotations

import importlib.util
import os
import sys


def main(argv=None) -> int:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "bench.py")
    if not os.path.isfile(path):
        print(f"flexengine bench: {path} not found (the benchmark lives at the root of the checkout)", file=sys.stderr)
        return 2
    spec = importlib.util.spec_from_file_location("flexengine_bench", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    saved = sys.argv
    sys.argv = [path] + list(sys.argv[2:] if argv is None else argv)
    try:
        return int(module.main() or 0)
    finally:
        sys.argv = saved
