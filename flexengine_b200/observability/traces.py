"""Step and request records as JSON lines, run metadata, and NVTX ranges.

Append-only ``steps.jsonl`` / ``requests.jsonl`` and ``run_metadata.json`` as in the
reference (src/flexengine/operations/observability/traces.py:15-53); NVTX ranges are
no-ops without CUDA.
"""
from __future__ import annotations

import json
import os
import platform
import threading
from contextlib import contextmanager
from dataclasses import asdict, is_dataclass
from datetime import datetime, timezone

import torch


@contextmanager
def nvtx(name: str):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class TraceWriter:
    def __init__(self, directory: str):
        self.directory = directory
        self.lock = threading.Lock()
        if directory:
            os.makedirs(directory, exist_ok=True)

    def write(self, name: str, item: dict) -> None:
        if not self.directory:
            return
        with self.lock, open(os.path.join(self.directory, f"{name}.jsonl"), "a", encoding="utf8") as f:
            f.write(json.dumps(item, ensure_ascii=False, default=str) + "\n")

    def metadata(self, config, model: str | None = None) -> None:
        if not self.directory:
            return
        data = {
            "timestamp_utc": datetime.now(timezone.utc).isoformat(),
            "python": platform.python_version(), "torch": torch.__version__,
            "cuda_available": torch.cuda.is_available(),
            "device_name": torch.cuda.get_device_name(0) if torch.cuda.is_available() else None,
            "config": asdict(config) if is_dataclass(config) else dict(vars(config)),
            "model": model if model is not None else getattr(config, "model", ""),
        }
        with open(os.path.join(self.directory, "run_metadata.json"), "w", encoding="utf8") as f:
            json.dump(data, f, ensure_ascii=False, indent=2, default=str)
