"""A fourth toy architecture, registered, built and run from this file alone, for what the other toys leave out:

* the head and the tail of the model are parts too: an embedding that scales its rows and a head that soft-caps
  its logits;
* two paged cache groups with page sizes of their own (8 tokens beside 32), one of them a window;
* a mixer whose prompt path takes portions in whole blocks of four tokens only, which it tells the scheduler
  through its cache group (``chunk_granularity``), and whose decode path keeps its per-request state with device
  indices, so that it can run inside a CUDA graph whose batch is padded: a padding request has state slot -1
  and must leave every slot as it was.

Runs on the CPU with the reference kernels and, marked ``gpu``, with the CUDA kernels (with decode graphs there).
"""
import math
import random
from dataclasses import dataclass

import pytest
import torch

import helpers
import kernel_refs
import plain_model
from flexengine_b200.cache import CacheManager
from flexengine_b200.config import EngineConfig, register_architecture
from flexengine_b200.engine import ModelRunner, StepEntry
from flexengine_b200.engine.runtime import Engine
from flexengine_b200.parts import (CacheGroupSpec, Embedding, Head, LayerSpec, Mixer, ModelPlan, PartSpec, RunEntry,
                                   WeightBinding, WeightSource, register_embedding, register_head, register_mixer)
from flexengine_b200.weights import load_model, write_random_model

DEVICES = [pytest.param("cpu", id="cpu"), pytest.param("cuda:0", id="gpu", marks=pytest.mark.gpu)]
BLOCK = 4


def provider(device):
    if device == "cpu":
        return kernel_refs
    from flexengine_b200 import ops
    return ops


class ScaledEmbedding(Embedding):
    def __init__(self, vocab_size: int, hidden_size: int, scale: float):
        self.vocab_size, self.hidden_size, self.scale = int(vocab_size), int(hidden_size), float(scale)

    def parameter_shapes(self):
        return {"weight": ((self.vocab_size, self.hidden_size), "matrix")}

    def forward(self, ctx):
        return ctx.ops.embedding(ctx.token_ids, self.weight) * self.scale


class SoftcapHead(Head):
    def __init__(self, vocab_size: int, hidden_size: int, cap: float):
        self.vocab_size, self.hidden_size, self.cap = int(vocab_size), int(hidden_size), float(cap)

    def parameter_shapes(self):
        return {"weight": ((self.vocab_size, self.hidden_size), "matrix")}

    def forward(self, ctx, h):
        logits = ctx.ops.linear(h, self.weight, None, out_float32=True)
        return self.cap * torch.tanh(logits / self.cap)


class BlockwiseMeanMixer(Mixer):
    """out_i = W . mean(h_0 .. h_i), the state being the running sum and the count.

    Its prompt path works in whole blocks of ``BLOCK`` tokens: a portion of more than one token has to start on
    a block boundary (it raises otherwise; only the last portion of a context may end inside a block).  A step of
    single tokens takes the decode path, which is written for CUDA graphs: slots come from the device tensor,
    and a request whose slot is negative (padding) adds nothing anywhere."""
    seen_portions: list = []          # (start, length) of every multi-token portion, for the tests to look at

    def __init__(self, hidden_size: int):
        self.hidden_size = int(hidden_size)
        self.proj_weight = None

    def parameter_shapes(self):
        return {"proj.weight": ((self.hidden_size, self.hidden_size), "matrix")}

    def cache_need(self):
        return {"kind": "state", "state_shape": (self.hidden_size + 1,), "chunk_granularity": BLOCK}

    def forward(self, ctx, h, entry):
        state = ctx.groups[entry.cache_group].state(entry.cache_slot)          # [max_requests, H + 1]
        H = self.hidden_size
        if ctx.max_q_len == 1:
            slots = ctx.state_slots
            real = (slots >= 0).to(torch.float32)[:, None]
            where = slots.clamp(min=0).long()
            step = torch.cat([h.float(), torch.ones((h.shape[0], 1), dtype=torch.float32, device=h.device)], dim=1) * real
            if entry.write_cache:
                state.index_add_(0, where, step)               # a padding row adds zeros: every slot stays as it was
                now = state[where]
            else:
                now = state[where] + step
            mean = now[:, :H] / now[:, H:].clamp(min=1.0)
            return ctx.ops.linear(mean.to(h.dtype), self.proj_weight)
        out = torch.empty(h.shape, dtype=torch.float32, device=h.device)
        row = 0
        for slot, start, n in zip(ctx.host_state_slots, ctx.host_starts, ctx.host_lengths):
            if n > 1:
                if start % BLOCK:
                    raise ValueError(f"a portion of {n} tokens starts at {start}, inside a block of {BLOCK}")
                BlockwiseMeanMixer.seen_portions.append((start, n))
            x = h[row:row + n].float()
            sums = state[slot, :H] + torch.cumsum(x, 0)
            counts = state[slot, H] + torch.arange(1, n + 1, device=h.device, dtype=torch.float32)
            out[row:row + n] = sums / counts[:, None]
            if entry.write_cache:
                state[slot, :H] = sums[-1]
                state[slot, H] = counts[-1]
            row += n
        return ctx.ops.linear(out.to(h.dtype), self.proj_weight)


@dataclass(frozen=True)
class BlockwiseConfig:
    vocab_size: int
    hidden_size: int
    window: int
    cap: float

    @classmethod
    def from_dict(cls, data):
        return cls(int(data["vocab_size"]), int(data["hidden_size"]), int(data["window"]), float(data["cap"]))


CONFIG = {"architectures": ["ToyBlockwiseForCausalLM"], "vocab_size": 83, "hidden_size": 48, "window": 21, "cap": 3.0}
NQ, NKV, D, I, EPS, THETA = 3, 1, 16, 40, 1e-5, 700.0
PAGE_FULL, PAGE_WINDOW = 8, 32


def build_plan(cfg: BlockwiseConfig) -> ModelPlan:
    h, v = cfg.hidden_size, cfg.vocab_size
    norm = PartSpec("rmsnorm", {"hidden_size": h, "eps": EPS})
    position = PartSpec("rope_half_split", {"head_dim": D, "theta": THETA})

    def attention(window):
        return PartSpec("attention", {"hidden_size": h, "num_heads": NQ, "num_kv_heads": NKV, "head_dim": D,
                                      "window": window, "position": position})
    ffn = PartSpec("swiglu", {"hidden_size": h, "intermediate_size": I})
    layers = [LayerSpec(attention(0), ffn, norm), LayerSpec(PartSpec("toy_blockwise_mean", {"hidden_size": h}), ffn, norm),
              LayerSpec(attention(cfg.window), ffn, norm)]
    run = [RunEntry(0, 0, 0, True), RunEntry(1, 1, 0, True), RunEntry(2, 2, 0, True)]
    groups = [CacheGroupSpec("all_keys", "full", slots=1, kv_heads=NKV, head_dim=D, page_size=PAGE_FULL),
              CacheGroupSpec("running_mean", "state", slots=1, state_shape=(h + 1,), chunk_granularity=BLOCK),
              CacheGroupSpec("recent_keys", "window", slots=1, kv_heads=NKV, head_dim=D, window=cfg.window,
                             page_size=PAGE_WINDOW)]

    def src(name, *shape):
        return WeightSource(name, tuple(shape))
    bindings = [WeightBinding(("embedding", "weight"), (src("embed.weight", v, h),)),
                WeightBinding(("lm_head", "weight"), alias_of=("embedding", "weight"), absent=("head.weight",),
                              why="this toy ties its head to its embedding"),
                WeightBinding(("final_norm", "weight"), (src("norm.weight", h),), kind="vector")]
    for l, layer in enumerate(layers):
        p = f"layers.{l}."
        bindings += [WeightBinding(("layer", l, "input_norm", "weight"), (src(p + "norm1.weight", h),), kind="vector"),
                     WeightBinding(("layer", l, "post_mixer_norm", "weight"), (src(p + "norm2.weight", h),), kind="vector"),
                     WeightBinding(("layer", l, "feed_forward", "gate_up.weight"), (src(p + "gate.weight", I, h), src(p + "up.weight", I, h))),
                     WeightBinding(("layer", l, "feed_forward", "down.weight"), (src(p + "down.weight", h, I),))]
        if layer.mixer.kind == "attention":
            bindings += [WeightBinding(("layer", l, "mixer", "qkv.weight"), (src(p + "q.weight", NQ * D, h), src(p + "k.weight", NKV * D, h), src(p + "v.weight", NKV * D, h))),
                         WeightBinding(("layer", l, "mixer", "qkv.bias"), (src(p + "q.bias", NQ * D), src(p + "k.bias", NKV * D), src(p + "v.bias", NKV * D)), kind="vector"),
                         WeightBinding(("layer", l, "mixer", "out.weight"), (src(p + "o.weight", h, NQ * D),))]
        else:
            bindings.append(WeightBinding(("layer", l, "mixer", "proj.weight"), (src(p + "proj.weight", h, h),)))
    init = {"default": ("normal", 0.0, 0.15), "suffix": {"norm1.weight": ("normal", 1.0, 0.05), "norm2.weight": ("normal", 1.0, 0.05),
                                                           "norm.weight": ("normal", 1.0, 0.05)}}
    sizes = {"vocab_size": v, "hidden_size": h}
    return ModelPlan("ToyBlockwiseForCausalLM", v, h, layers, run, groups, norm, bindings, init=init,
                     embedding=PartSpec("toy_scaled_embedding", dict(sizes, scale=math.sqrt(h))),
                     head=PartSpec("toy_softcap_head", dict(sizes, cap=cfg.cap)))


register_embedding("toy_scaled_embedding", ScaledEmbedding)
register_head("toy_softcap_head", SoftcapHead)
register_mixer("toy_blockwise_mean", BlockwiseMeanMixer)
register_architecture("ToyBlockwiseForCausalLM", BlockwiseConfig, build_plan)


def reference_logits(w: dict, ids) -> torch.Tensor:
    """The toy over one whole sequence, from the plain implementation's parts."""
    T = len(ids)
    pos = torch.arange(T)
    inv = plain_model.rope_inverse_frequencies(D, THETA, "cpu")
    x = w["embed.weight"][torch.tensor(ids)] * math.sqrt(CONFIG["hidden_size"])

    def ffn(l, x):
        p = f"layers.{l}."
        h = plain_model.rms_norm(x, w[p + "norm2.weight"], EPS)
        return x + plain_model.swiglu_mlp(h, w[p + "gate.weight"], w[p + "up.weight"], w[p + "down.weight"])

    def attend(l, x, window):
        p = f"layers.{l}."
        names = {"q_proj.weight": w[p + "q.weight"], "k_proj.weight": w[p + "k.weight"], "v_proj.weight": w[p + "v.weight"],
                 "q_proj.bias": w[p + "q.bias"], "k_proj.bias": w[p + "k.bias"], "v_proj.bias": w[p + "v.bias"],
                 "o_proj.weight": w[p + "o.weight"]}
        h = plain_model.rms_norm(x, w[p + "norm1.weight"], EPS)
        return x + plain_model.attention_block(h, names, "", pos, NQ, NKV, D, inv, window)

    x = ffn(0, attend(0, x, 0))
    h = plain_model.rms_norm(x, w["layers.1.norm1.weight"], EPS)
    x = ffn(1, x + (torch.cumsum(h, 0) / torch.arange(1, T + 1)[:, None]) @ w["layers.1.proj.weight"].T)
    x = ffn(2, attend(2, x, CONFIG["window"]))
    logits = plain_model.rms_norm(x, w["norm.weight"], EPS) @ w["embed.weight"].T
    return CONFIG["cap"] * torch.tanh(logits / CONFIG["cap"])


def reference_greedy(w: dict, prompt, count: int) -> list:
    ids, out = list(prompt), []
    for _ in range(count):
        out.append(int(reference_logits(w, ids)[-1].argmax()))
        ids.append(out[-1])
    return out


@pytest.fixture(scope="module")
def toy_dir(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("blockwise"))
    write_random_model(CONFIG, d, seed=12, dtype="float32")
    return d


def aligned_mixed_steps(requests: dict, rng: random.Random, live: int, decode_tail: int) -> list:
    """Like ``helpers.steps_mixed``, with every portion but a context's last a whole number of blocks."""
    waiting, active, steps = list(requests.items()), {}, []
    while waiting or active:
        while waiting and len(active) < live:
            rid, ids = waiting.pop(0)
            active[rid] = [ids, 0]
        entries, ended = [], []
        for rid in list(active):
            ids, fed = active[rid]
            if len(active) > 1 and rng.random() < 0.2:
                continue
            prompt_left = len(ids) - decode_tail - fed
            if prompt_left <= 0:
                n = 1
            else:
                n = min(rng.choice((BLOCK, 2 * BLOCK, 3 * BLOCK, 5 * BLOCK)), prompt_left)      # the last one may be ragged
            entries.append((rid, ids[fed:fed + n], list(range(n))))
            active[rid][1] = fed + n
            if fed + n == len(ids):
                ended.append(rid)
                del active[rid]
        if entries:
            steps.append((entries, ended))
    return steps


@pytest.mark.parametrize("device", DEVICES)
def test_blockwise_toy_steps_match_its_reference(toy_dir, device):
    _cfg, plan, model = load_model(toy_dir, "float32", device)
    assert type(model.embedding).__name__ == "ScaledEmbedding" and type(model.head).__name__ == "SoftcapHead"
    _, w = plain_model.read_model_folder(toy_dir)
    rng = random.Random(2)
    requests = {f"b{i}": helpers.random_prompt(rng, n, CONFIG["vocab_size"]) for i, n in enumerate([61, 14, 37, 90, 26])}
    steps = aligned_mixed_steps(requests, rng, live=3, decode_tail=5)
    # an int page count is in pages of the default size (16 here); each group gets what holds the same tokens
    pages_of_16 = helpers.peak_pages(steps, 32) * 2
    cache = CacheManager(plan.cache_groups, pages_of_16, 16, 3, torch.float32, device)
    assert (cache.groups[0].page_size, cache.groups[2].page_size) == (PAGE_FULL, PAGE_WINDOW)
    assert cache.groups[0].pool.num_pages == 2 * pages_of_16 and cache.groups[2].pool.num_pages == pages_of_16 // 2
    assert cache.chunk_granularity == BLOCK and cache.sharing_unit == 32
    runner = ModelRunner(model, cache, ops=provider(device))
    most_window_pages = 0
    results, fed = {}, {}
    for entries, ended in steps:
        out = runner.step([StepEntry(rid, toks, want) for rid, toks, want in entries])
        row = 0
        for rid, toks, want in entries:
            base = fed.get(rid, 0)
            for place in want:
                results[(rid, base + place)] = out[row].float().cpu()
                row += 1
            fed[rid] = base + len(toks)
        most_window_pages = max(most_window_pages, cache.groups[2].pool.used_pages)
        for rid in ended:
            runner.finish(rid)
        cache.assert_invariants()
    assert cache.groups[0].pool.used_pages == 0 and cache.groups[2].pool.used_pages == 0
    assert most_window_pages <= 3 * 2                # window 21 in pages of 32: two pages a request at most
    for rid, ids in requests.items():
        got = torch.stack([results[(rid, p)] for p in range(len(ids))])
        helpers.assert_logits_close(got, reference_logits(w, ids), "float32", f"blockwise {rid}")
    if device != "cpu":
        provider(device).check_status(device)


def test_an_unaligned_portion_is_refused_by_the_mixer_itself(toy_dir):
    _cfg, plan, model = load_model(toy_dir, "float32", "cpu")
    cache = CacheManager(plan.cache_groups, 8, 16, 2, torch.float32, "cpu")
    runner = ModelRunner(model, cache, ops=kernel_refs)
    runner.step([StepEntry("a", [1, 2, 3, 4, 5, 6], [])])
    with pytest.raises(ValueError, match="inside a block"):
        runner.step([StepEntry("a", [7, 8, 9], [])])


@pytest.mark.parametrize("device", DEVICES)
def test_the_scheduler_cuts_portions_in_whole_blocks(toy_dir, device):
    """Through the engine: adaptive policy with a chunk size and budgets that are no multiples of the block, so few
    pages that requests are preempted and recompute; on the GPU decode steps replay CUDA graphs whose buckets
    (1, 2, 4, 5) pad three live requests with one whose state slot is -1.  Tokens equal the reference's."""
    _cfg, plan, model = load_model(toy_dir, "float32", device)
    _, w = plain_model.read_model_folder(toy_dir)
    gpu = device != "cpu"
    config = EngineConfig(model=toy_dir, device=device, dtype="float32", max_model_len=96, max_num_seqs=5,
                          max_num_batched_tokens=23, prefill_chunk_size=10, kv_block_size=16, kv_num_blocks=9,
                          max_output_tokens=16, scheduler_policy="adaptive", cuda_graph=gpu, trace_steps=False)
    engine = Engine.from_model(model, config, ops=provider(device))
    assert engine.scheduler.granularity == BLOCK
    BlockwiseMeanMixer.seen_portions = []
    rng = random.Random(8)
    prompts = [helpers.random_prompt(rng, n, CONFIG["vocab_size"]) for n in (33, 7, 18)]
    outputs = engine.generate(prompts, max_tokens=9)
    for prompt, out in zip(prompts, outputs):
        assert out.token_ids == reference_greedy(w, prompt, 9)
    seen = BlockwiseMeanMixer.seen_portions
    assert seen and all(start % BLOCK == 0 for start, _ in seen)
    assert any(n % BLOCK == 0 and n < 33 for _, n in seen), "a long prompt was cut, in whole blocks"
    assert any(n == 8 for _, n in seen), "a chunk size of 10 rounds down to 8"
    assert engine.cache.used_pages == 0 and len(engine.cache.free_state_slots) == 5
    if gpu:
        assert engine.runner.graph_replays > 0 and 4 in engine.runner._graphs
        provider(device).check_status(device)
    # so few pages that the longest request is preempted and recomputes its context, again in whole blocks
    tight = Engine.from_model(model, EngineConfig(model=toy_dir, device=device, dtype="float32", max_model_len=48,
                                                  max_num_seqs=2, max_num_batched_tokens=64, kv_block_size=16,
                                                  kv_num_blocks=4, max_output_tokens=16, cuda_graph=gpu,
                                                  trace_steps=False), ops=provider(device))
    # the older request crosses into its second page of 32 while the younger holds the only other one
    tight_prompts = [helpers.random_prompt(rng, n, CONFIG["vocab_size"]) for n in (30, 18, 7)]
    outputs = tight.generate(tight_prompts, max_tokens=9)
    assert [o.token_ids for o in outputs] == [reference_greedy(w, p, 9) for p in tight_prompts]
    assert tight.preemption_count >= 1 and tight.cache.used_pages == 0
