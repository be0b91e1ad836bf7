from .traces import RunTrace, marked

__all__ = ["RunTrace", "marked"]
