"""``flexengine build``: compile every CUDA kernel library for sm_100a."""
from __future__ import annotations


def main(argv=None) -> int:
    from ..ops import library
    for path in library.build_all(force="--force" in (argv or [])):
        print(path)
    return 0
