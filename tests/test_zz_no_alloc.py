"""The allocation-free decode attention entry point, called through its exported C symbol.

Some hosts of the kernel library may not allocate device memory where they call it (a fixed
memory plan, someone else's process, a point where an allocation would stall the device), so
``fe_paged_decode_mma_static`` takes the split-KV scratch from an array built into the library.
The test drives it the way such a host would, with ctypes on raw pointers, twice in a row on
different inputs, and compares each result with the ordinary entry point, which gets its
scratch from the caller.  This file is collected last on purpose: if it fails, a run that
stops at the first failure has already run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, requests, nq, nkv, d, ps, positions):
    gen = torch.Generator(device=DEV)
    gen.manual_seed(seed)
    pages_per = [-(-(p + 1) // ps) for p in positions]
    total = sum(pages_per) + 2
    perm = torch.randperm(total, generator=gen, device=DEV).to(torch.int32)
    kc = torch.randn(total, nkv, ps, d, generator=gen, device=DEV).to(torch.bfloat16)
    vc = torch.randn(total, nkv, ps, d, generator=gen, device=DEV).to(torch.bfloat16)
    table = torch.full((requests, max(pages_per)), -1, dtype=torch.int32, device=DEV)
    k = 0
    for r, n in enumerate(pages_per):
        table[r, :n] = perm[k:k + n]
        k += n
    q = torch.randn(requests, (nq + 2 * nkv) * d, generator=gen, device=DEV).to(torch.bfloat16)
    cu_q = torch.arange(requests + 1, dtype=torch.int32, device=DEV)
    q_start = torch.tensor(positions, dtype=torch.int32, device=DEV)
    return q, kc, vc, table, cu_q, q_start


def test_static_scratch_entry_point_matches_the_ordinary_one():
    from flexengine_b200 import ops
    from flexengine_b200.ops import library
    lib = library.load("bf16")
    fn = lib.fe_paged_decode_mma_static
    fn.restype = ctypes.c_int
    lib.fe_static_scratch_bytes.restype = ctypes.c_longlong
    assert lib.fe_static_scratch_bytes() == 8 << 20
    vp, ll, ci, cf = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
    nq, nkv, d, ps, splits = 14, 2, 128, 16, 5
    positions = [0, 31, 32, 100, 511, 700, 1023, 64]
    status = ops.status_word(DEV)
    for call, seed in enumerate((11, 12)):                # two calls in a row share the built-in array
        q, kc, vc, table, cu_q, q_start = _case(seed, len(positions), nq, nkv, d, ps, positions)
        scale = 1.0 / math.sqrt(d)
        want = ops.paged_decode_mma(q, q.stride(0), kc, vc, table, cu_q, q_start, len(positions), nq, nkv, d, ps, scale,
                                    0, splits)
        got = torch.full((len(positions), nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        allocated = torch.cuda.memory_allocated(DEV)
        rc = fn(vp(q.data_ptr()), ll(q.stride(0)), vp(got.data_ptr()), ll(got.stride(0)), vp(kc.data_ptr()),
                vp(vc.data_ptr()), vp(table.data_ptr()), ci(table.shape[1]), vp(cu_q.data_ptr()), vp(q_start.data_ptr()),
                ci(len(positions)), ci(nq), ci(nkv), ci(d), ci(ps), ci(kc.shape[0]), cf(scale), ci(0), ci(splits),
                vp(status.data_ptr()), vp(torch.cuda.current_stream().cuda_stream))
        assert rc == 0, lib.fe_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(DEV) == allocated          # the call took nothing from the allocator
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        assert torch.isfinite(got.float()).all(), f"call {call}"
    ops.check_status(DEV)
    # more scratch than the built-in array holds: refused with the reason, nothing launched
    rc = fn(vp(q.data_ptr()), ll(q.stride(0)), vp(got.data_ptr()), ll(got.stride(0)), vp(kc.data_ptr()), vp(vc.data_ptr()),
            vp(table.data_ptr()), ci(table.shape[1]), vp(cu_q.data_ptr()), vp(q_start.data_ptr()), ci(len(positions)),
            ci(nq), ci(nkv), ci(d), ci(ps), ci(kc.shape[0]), cf(scale), ci(0), ci(200), vp(status.data_ptr()),
            vp(torch.cuda.current_stream().cuda_stream))
    assert rc != 0 and b"built-in array holds" in lib.fe_last_error()


def _call_static(lib, q, got, kc, vc, table, cu_q, q_start, requests, nq, nkv, d, ps, scale, window, splits, status):
    vp, ll, ci, cf = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
    return lib.fe_paged_decode_mma_static(
        vp(q.data_ptr()), ll(q.stride(0)), vp(got.data_ptr()), ll(got.stride(0)), vp(kc.data_ptr()), vp(vc.data_ptr()),
        vp(table.data_ptr()), ci(table.shape[1]), vp(cu_q.data_ptr()), vp(q_start.data_ptr()), ci(requests), ci(nq), ci(nkv),
        ci(d), ci(ps), ci(kc.shape[0]), cf(scale), ci(window), ci(splits), vp(status.data_ptr()),
        vp(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_entry_point_at_its_edges():
    """One split (no scratch at all), a window, the largest batch the built-in array holds and the first one it
    does not: the refused call launches nothing, so its output buffer keeps its fill and no status bit is set."""
    from flexengine_b200 import ops
    from flexengine_b200.ops import library
    lib = library.load("bf16")
    lib.fe_paged_decode_scratch_bytes.restype = ctypes.c_longlong
    status = ops.status_word(DEV)
    scale = 1.0 / math.sqrt(128)
    # (requests, nq, nkv, splits, window): 127 x 16 x 8 x 129 floats are 512 bytes under the 8 MiB of the array
    for requests, nq, nkv, splits, window in ((6, 14, 2, 1, 0), (6, 14, 2, 4, 50), (127, 16, 2, 8, 0)):
        positions = [(37 * r + 5) % 300 + 260 for r in range(requests)]
        q, kc, vc, table, cu_q, q_start = _case(20 + requests, requests, nq, nkv, 128, 16, positions)
        need = lib.fe_paged_decode_scratch_bytes(requests, nq, 128, splits)
        assert need <= lib.fe_static_scratch_bytes() and (splits > 1) == (need > 0)
        want = ops.paged_decode_mma(q, q.stride(0), kc, vc, table, cu_q, q_start, requests, nq, nkv, 128, 16, scale, window, splits)
        got = torch.full((requests, nq * 128), float("nan"), dtype=torch.bfloat16, device=DEV)
        rc = _call_static(lib, q, got, kc, vc, table, cu_q, q_start, requests, nq, nkv, 128, 16, scale, window, splits, status)
        assert rc == 0, lib.fe_last_error().decode()
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    assert lib.fe_static_scratch_bytes() - need == 512
    # one request more does not fit: refused before anything is launched
    requests = 128
    positions = [300] * requests
    q, kc, vc, table, cu_q, q_start = _case(5, requests, 16, 2, 128, 16, positions)
    assert lib.fe_paged_decode_scratch_bytes(requests, 16, 128, 8) > lib.fe_static_scratch_bytes()
    got = torch.full((requests, 16 * 128), float("nan"), dtype=torch.bfloat16, device=DEV)
    rc = _call_static(lib, q, got, kc, vc, table, cu_q, q_start, requests, 16, 2, 128, 16, scale, 0, 8, status)
    torch.cuda.synchronize()
    assert rc != 0 and b"built-in array holds" in lib.fe_last_error()
    assert bool(torch.isnan(got.float()).all()), "a refused call must not write its output"
    ops.check_status(DEV)
