"""What a run leaves behind: JSON-lines streams, a description of the run, and profiler ranges.

The folder layout is the one the reference's tools read (src/flexengine/operations/observability/traces.py):
``steps.jsonl`` and ``requests.jsonl`` grow by one line per step or finished request, ``run_metadata.json`` says
what ran.  A ``RunTrace`` without a folder records nothing and costs nothing; with one, each stream's file is
opened once and kept open, and a line is written and flushed under a lock (the engine's worker thread and a
caller's thread may both finish requests).
"""
from __future__ import annotations

import dataclasses
import datetime
import json
import os
import platform
import threading

import torch


class marked:
    """``with marked("kv/reserve"):`` shows as a named range in a profiler's timeline when CUDA is in use."""
    __slots__ = ("name", "pushed")

    def __init__(self, name: str):
        self.name, self.pushed = name, False

    def __enter__(self):
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            torch.cuda.nvtx.range_push(self.name)
            self.pushed = True
        return self

    def __exit__(self, *exc):
        if self.pushed:
            torch.cuda.nvtx.range_pop()
        return False


class RunTrace:
    def __init__(self, folder: str = ""):
        self.folder = folder or ""
        self._files: dict = {}
        self._guard = threading.Lock()
        if self.folder:
            os.makedirs(self.folder, exist_ok=True)

    @property
    def enabled(self) -> bool:
        return bool(self.folder)

    def record(self, stream: str, item: dict) -> None:
        """Append ``item`` as one line of ``<stream>.jsonl``."""
        if not self.folder:
            return
        line = json.dumps(item, ensure_ascii=False, default=str)
        with self._guard:
            f = self._files.get(stream)
            if f is None:
                f = self._files[stream] = open(os.path.join(self.folder, stream + ".jsonl"), "a", encoding="utf8")
            f.write(line + "\n")
            f.flush()

    def describe(self, config, **extra) -> None:
        """Write ``run_metadata.json``: the settings, the software and the device of this run."""
        if not self.folder:
            return
        settings = dataclasses.asdict(config) if dataclasses.is_dataclass(config) else dict(vars(config))
        cuda = torch.cuda.is_available()
        about = {"timestamp_utc": datetime.datetime.now(datetime.timezone.utc).isoformat(),
                 "model": extra.pop("model", settings.get("model", "")), "config": settings,
                 "software": {"python": platform.python_version(), "torch": torch.__version__,
                              "cuda": torch.version.cuda},
                 "device": {"cuda_available": cuda, "name": torch.cuda.get_device_name(0) if cuda else None}}
        about.update(extra)
        with open(os.path.join(self.folder, "run_metadata.json"), "w", encoding="utf8") as f:
            json.dump(about, f, ensure_ascii=False, indent=2, default=str)

    def close(self) -> None:
        with self._guard:
            for f in self._files.values():
                f.close()
            self._files.clear()
