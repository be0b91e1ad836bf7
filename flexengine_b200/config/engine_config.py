"""Engine settings: one frozen dataclass, validated, readable from ``FLEX_<FIELD>`` variables.

Names, defaults and checks follow the reference's EngineConfig
(src/flexengine/engine/config.py:17-62) and its environment convention
(config.py:64-86).  ``attention_backend`` and ``rmsnorm_backend`` are gone (there is
one kernel path); ``dtype`` is "bfloat16" or "float32"; ``kv_num_blocks=0`` sizes the
pool from free device memory; ``overlap_steps`` (no counterpart in the reference) lets the
host plan and launch a step while the device still runs the one before.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, fields, replace

POLICIES = ("fcfs", "decode_first", "slo_aware", "adaptive")
DTYPES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}


@dataclass(frozen=True)
class EngineConfig:
    model: str = ""
    device: str = "cuda:0"
    dtype: str = "bfloat16"
    max_model_len: int = 2048
    max_num_seqs: int = 8
    max_num_batched_tokens: int = 128
    prefill_chunk_size: int = 128
    max_waiting: int = 64
    kv_block_size: int = 16
    kv_num_blocks: int = 1024          # 0: fill what device memory is left
    kv_memory_fraction: float = 0.9    # used only when kv_num_blocks == 0
    cuda_graph: bool = False
    overlap_steps: bool = True         # launch a step before the host has read the tokens of the one before
    scheduler_policy: str = "fcfs"
    ttft_slo_ms: float = 2000.0
    itl_slo_ms: float = 200.0
    idle_sleep_seconds: float = 0.003
    trace_dir: str = ""
    trace_steps: bool = True
    max_output_tokens: int = 512
    random_seed: int = 42

    def __post_init__(self) -> None:
        for name in ("max_model_len", "max_num_seqs", "max_num_batched_tokens", "prefill_chunk_size",
                     "kv_block_size", "max_output_tokens"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive")
        if self.kv_num_blocks < 0:
            raise ValueError("kv_num_blocks must be positive (or 0 to size it from free memory)")
        if self.max_waiting < 0:
            raise ValueError("max_waiting must be nonnegative")
        if self.scheduler_policy not in POLICIES:
            raise ValueError("Unknown scheduler_policy")
        if self.dtype not in DTYPES:
            raise ValueError(f"Unknown dtype {self.dtype!r}; expected one of {sorted(DTYPES)}")
        object.__setattr__(self, "dtype", DTYPES[self.dtype])
        if self.kv_num_blocks and self.kv_num_blocks * self.kv_block_size < self.max_model_len:
            raise ValueError("KV pool cannot contain one max-length request")

    def with_block_size(self, kv_block_size: int) -> "EngineConfig":
        """The same settings with pages of another size and as many of them as hold at least the same number of
        tokens (the reference compares page sizes at equal capacity, src/flexengine/engine/config.py:8-14)."""
        if kv_block_size <= 0:
            raise ValueError("kv_block_size must be positive")
        tokens = self.kv_num_blocks * self.kv_block_size
        return replace(self, kv_block_size=int(kv_block_size), kv_num_blocks=-(-tokens // int(kv_block_size)))

    @classmethod
    def from_env(cls, **overrides) -> "EngineConfig":
        def truth(v: str) -> bool:
            return v.lower() in ("true", "yes", "1")

        kwargs = {}
        for f in fields(cls):
            raw = os.getenv(f"FLEX_{f.name.upper()}")
            if raw is None:
                continue
            kind = type(f.default)
            kwargs[f.name] = truth(raw) if kind is bool else kind(raw)
        kwargs.update({k: v for k, v in overrides.items() if v is not None})
        return cls(**kwargs)
