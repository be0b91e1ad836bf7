"""Trace replay: the replay loop on the CPU (reference kernels), and ``bin/trace_run`` as a
program on the GPU in float32 and bfloat16, for the four ways of cutting the work."""
import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import kernel_refs
from flexengine_b200.engine import replay as replay_module

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def to_lines(steps) -> list:
    return [json.dumps({"step": i, "entries": [{"id": rid, "tokens": toks, "want": want} for rid, toks, want in entries],
                        "end": ended}) for i, (entries, ended) in enumerate(steps)]


def read_results(out_dir, steps, vocab) -> dict:
    results, fed = {}, {}
    for i, (entries, ended) in enumerate(steps):
        wanted = sum(len(w) for _, _, w in entries)
        path = os.path.join(out_dir, f"{i}.f32")
        if wanted == 0:
            assert not os.path.exists(path)
        else:
            data = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
            row = 0
            for rid, toks, want in entries:
                for w in want:
                    results[(rid, fed.get(rid, 0) + w)] = torch.from_numpy(data[row].copy())
                    row += 1
        for rid, toks, _ in entries:
            fed[rid] = fed.get(rid, 0) + len(toks)
        for rid in ended:
            fed.pop(rid, None)
    return results


def max_tokens_needed(steps) -> int:
    """Most tokens live requests hold at any time, each rounded up to a multiple of 64."""
    fed, peak = {}, 0
    for entries, ended in steps:
        for rid, toks, _ in entries:
            fed[rid] = fed.get(rid, 0) + len(toks)
        peak = max(peak, sum(-(-n // 64) * 64 for n in fed.values()))
        for rid in ended:
            fed.pop(rid, None)
    return peak


def scenarios(name):
    rng = random.Random(17)
    vocab = helpers.CONFIGS[name]["vocab_size"]
    requests = {f"q{i}": helpers.random_prompt(rng, n, vocab) for i, n in enumerate([70, 33, 101, 48])}
    more = dict(requests)
    more.update({f"z{i}": helpers.random_prompt(rng, n, vocab) for i, n in enumerate([90, 40, 65])})
    sparse = helpers.steps_mixed(more, random.Random(2), live=4)
    # some steps want nothing, some only the last place
    sparse = [([(rid, toks, ([] if i % 3 == 0 else want[-1:])) for rid, toks, want in entries], ended)
              for i, (entries, ended) in enumerate(sparse)]
    return {"whole": (requests, helpers.steps_whole(requests)),
            "last_decoded": (requests, helpers.steps_last_decoded(requests, 32)),
            "portions": (requests, helpers.steps_portions(requests, rng)),
            "mixed": (more, helpers.steps_mixed(more, rng, live=4)),
            "sparse": (more, sparse)}


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    return {name: helpers.make_model_dir(tmp_path_factory, name, seed=31) for name in ("A", "B")}


@pytest.mark.parametrize("kind", ["whole", "mixed", "sparse"])
def test_replay_loop_on_cpu(model_dirs, kind, tmp_path):
    requests, steps = scenarios("A")[kind]
    runner = replay_module.build_runner(model_dirs["A"], "float32", max_tokens_needed(steps), device="cpu", ops=kernel_refs)
    done = []
    replay_module.replay(runner, to_lines(steps), str(tmp_path), done.append)
    assert done == list(range(len(steps)))
    assert runner.cache.used_pages == 0
    results = read_results(str(tmp_path), steps, 256)
    for (rid, pos), row in results.items():
        want = helpers.plain_logits(model_dirs["A"], requests[rid][:pos + 1])[-1]
        helpers.assert_logits_close(row, want, "float32", f"{kind} {rid}@{pos}")


def run_trace_program(model_dir, dtype, steps, out_dir, env=None):
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens_needed(steps))]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    for i, line in enumerate(to_lines(steps)):
        proc.stdin.write(line + "\n")
        proc.stdin.flush()
        answer = proc.stdout.readline().strip()      # the next step may come only after this
        assert answer == f"done {i}", answer
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_trace_run_program(model_dirs, name, dtype, tmp_path):
    vocab = helpers.CONFIGS[name]["vocab_size"]
    plain = {}
    for kind, (requests, steps) in scenarios(name).items():
        out_dir = str(tmp_path / kind)
        run_trace_program(model_dirs[name], dtype, steps, out_dir)
        results = read_results(out_dir, steps, vocab)
        if kind != "sparse":
            helpers.compare_with_plain(model_dirs[name], results, requests, dtype, f"trace_run {name}/{kind}/{dtype}", config=name)
        else:
            for (rid, pos), row in results.items():
                if rid not in plain:
                    plain[rid] = helpers.plain_logits(model_dirs[name], requests[rid])
                helpers.assert_logits_close(row, plain[rid][pos], dtype, f"sparse {rid}@{pos}", name)
