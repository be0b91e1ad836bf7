from .traces import TraceWriter, nvtx

__all__ = ["TraceWriter", "nvtx"]
