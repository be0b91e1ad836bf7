"""The kernels as Python functions over CUDA tensors.

Every function here launches hand-written CUDA from ``csrc/`` on the current stream;
the only library calls are bfloat16 matrix products (cuBLAS through ``torch.mm``), where
the reference uses a library too (src/flexengine/inference/models/qwen2.py:99-101,129-135).
There is no CPU path: tensors must be on a CUDA device, and a missing or unbuildable
kernel library raises.

Conventions: activations are float32 (true 32-bit path) or bfloat16; the residual stream,
norm weights, biases and logits are float32; index tensors are int32.
"""
from __future__ import annotations

import torch

from . import library

# Arguments go to the entry points as plain Python values: the loader has given every entry point the parameter
# types of its C declaration (ops/library.py), so ctypes converts them itself, and refuses a call whose number of
# arguments or kinds of values do not fit.  These names say which C type a value is meant for.
_c_int, _c_ll, _c_float = int, int, float

# The library's bfloat16 products add the partial sums of a split K up in float: its default allows bfloat16 there, which
# costs two to four times the error of one bfloat16 rounding at K of a few thousand (measured against the
# weight-streaming kernel of this package, whose results are the float sums rounded once).
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

_status: dict = {}
launches = 0          # kernels of this package launched so far (library matrix products not counted)


def _core():
    return library.load("core")


def _ptr(t):
    return t.data_ptr() if t is not None else None


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream's handle; asked for at every launch, so by the shortest way there is."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _code(dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise TypeError(f"kernels take float32 or bfloat16, not {dtype}")


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("flexengine_b200.ops runs on CUDA tensors only; there is no CPU path")


def _run(lib, name: str, *args) -> None:
    global launches
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise RuntimeError(f"{name} failed: {lib.fe_last_error().decode()}")
    launches += 1


def status_word(device) -> torch.Tensor:
    """The device word in which kernels record a guarded fault (bad token, page or slot)."""
    word = _status.get(device)                     # asked for at every launch: the device object itself is the key
    if word is None:
        key = str(torch.device(device))
        if key not in _status:
            with torch.inference_mode(False):      # a plain tensor, writable from any mode
                _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
        word = _status[device] = _status[key]
    return word


STATUS_BITS = ((1, "token id out of range"), (2, "page id out of range"), (4, "cache slot out of range"),
               (8, "a bounded wait ran out"))


def describe_status(value: int) -> str:
    """What the bits of a status word say, in words."""
    return ", ".join(n for bit, n in STATUS_BITS if value & bit) or f"unknown bits {value}"


def check_status(device) -> None:
    """Synchronises; raises if a kernel met an index it had to skip since the last check."""
    word = status_word(device)
    value = int(word.item())
    if value:
        word.zero_()
        raise RuntimeError("kernel status: " + describe_status(value))


# ------------------------------------------------------------------------------------------------
def embedding(token_ids, table):
    """float32 residual rows [T, H] = table[token_ids]."""
    _need_cuda(token_ids, table)
    T, (V, H) = token_ids.numel(), table.shape
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _run(_core(), "fe_embedding", _ptr(token_ids), _ptr(table), _ptr(out), _c_int(T), _c_int(H), _c_int(V),
         _c_int(_code(table.dtype)), _ptr(status_word(table.device)), _stream())
    return out


def carry_tokens(token_ids, rows, sources, previous):
    """token_ids[rows[i]] = previous[sources[i]] where rows[i] >= 0 (all int32, in place): what the
    step before sampled becomes this step's input without a round trip through the host."""
    _need_cuda(token_ids, rows, sources, previous)
    if previous.dtype != torch.int32 or token_ids.dtype != torch.int32:
        raise TypeError("carry_tokens: int32 tensors")
    _run(_core(), "fe_carry_tokens", _ptr(token_ids), _ptr(rows), _ptr(sources), _ptr(previous), _c_int(rows.numel()),
         _c_int(token_ids.numel()), _c_int(previous.numel()), _ptr(status_word(token_ids.device)), _stream())


UPCOMING_MAX_ROWS = 16            # a step of this many tokens or fewer leaves the memory system idle between products
UPCOMING_BYTES_MERGE = 16 << 20   # the same for the merge kernel of decode attention, ahead of the output projection
UPCOMING_TAIL_BYTES = 16 << 20    # what the blocks of a weight-streaming product ask into L2 of the next matrix as they end
UPCOMING_BYTES = 10 << 20         # how much of the next weight matrix a norm asks into L2 ahead of its product: what the
                                  # memory system delivers while the norm runs (8-12 MB measured best on the 7B shape)


def _upcoming(tensor, rows: int, limit: int = UPCOMING_BYTES):
    """(pointer, bytes) of the start of ``tensor`` for a kernel's prefetching blocks; nothing for large steps."""
    if tensor is None or rows > UPCOMING_MAX_ROWS or not tensor.is_cuda:
        return None, 0
    return _ptr(tensor), _c_ll(min(tensor.numel() * tensor.element_size(), limit))


def add_rmsnorm(residual, delta, weight, eps, out_dtype, rows=None, upcoming=None):
    """Fused residual add + RMSNorm.  rows=None: residual += delta in place (all rows) and every row
    is normalised; rows given: only those rows are read (residual[rows] + delta[rows]), nothing is
    written back.  ``upcoming``: the weight matrix that the next kernel streams; in a decode step extra
    blocks of this kernel, which barely touches memory, ask for its start to be brought into L2."""
    _need_cuda(residual, delta, weight, rows)
    T, H = residual.shape
    if residual.dtype != torch.float32 or weight.dtype != torch.float32:
        raise TypeError("the residual stream and norm weights are float32")
    if delta is not None and (delta.dtype != out_dtype or delta.shape != residual.shape or not delta.is_contiguous()):
        raise ValueError("add_rmsnorm: delta must be contiguous, shaped like the residual, in the compute dtype")
    n_out = T if rows is None else rows.numel()
    out = torch.empty((n_out, H), dtype=out_dtype, device=residual.device)
    _run(_core(), "fe_add_rmsnorm", _ptr(residual), _ptr(delta), _ptr(weight), _c_float(eps), _ptr(out), _ptr(rows),
         _c_int(n_out), _c_int(H), _c_int(T), _c_int(_code(out_dtype)), *_upcoming(upcoming, T), _stream())
    return out


FUSES_RESIDUAL_NORM = True      # linear(..., follow=) may end a branch: see Prenormed


class Prenormed:
    """Rows that are halfway through an RMSNorm, as the residual epilogue of the weight-streaming GEMM leaves them
    (csrc/gemm_skinny.cu): ``scaled`` = bfloat16(residual * norm weight), not yet divided by the rows' root mean
    square, and ``sumsq`` [tiles of 16 columns, 8], every tile's share of the rows' sums of squares.  The products
    that consume a norm (``linear``, ``linear_swiglu``, ``qkv_projection``) take it in place of a tensor and
    finish the norm in their own epilogue; where that kernel does not apply, ``materialize`` runs the norm
    kernel over the residual, which holds the sum already."""
    __slots__ = ("scaled", "sumsq", "eps", "residual", "weight")

    def __init__(self, scaled, sumsq, eps, residual, weight):
        self.scaled, self.sumsq, self.eps, self.residual, self.weight = scaled, sumsq, float(eps), residual, weight

    shape = property(lambda self: self.scaled.shape)
    dtype = property(lambda self: self.scaled.dtype)
    device = property(lambda self: self.scaled.device)

    def materialize(self):
        return add_rmsnorm(self.residual, None, self.weight, self.eps, self.scaled.dtype)


def _rows_and_scale(x):
    """(tensor, sumsq pointer, tiles, eps) of an input of the weight-streaming kernel for up to 8 rows."""
    if isinstance(x, Prenormed):
        return x.scaled, _ptr(x.sumsq), _c_int(x.sumsq.shape[0]), _c_float(x.eps)
    return x, None, _c_int(0), _c_float(0.0)


def _fits(x, w) -> str:
    """Which weight-streaming kernel takes this product, if any: "skinny" (up to 8 rows) or ""."""
    return "skinny" if skinny_ok(x.scaled if isinstance(x, Prenormed) else x, w) else ""


def gemm_fp32(x, w, bias=None):
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    _run(_core(), "fe_gemm_fp32", _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(M), _c_int(N), _c_int(K), _stream())
    return out


def linear(x, w, bias=None, out_float32=False, follow=None, upcoming=None):
    """y = x w^T (+ bias); x [M, K], w [N, K].  A float32 weight runs the true 32-bit product
    (CUDA cores, no reduced-precision mode) whatever the activation dtype; a bfloat16 weight
    runs on tensor cores with float32 accumulation.

    ``follow`` = (residual, norm weight, eps): the product ends a branch of a layer; its result is to be added to
    the float32 residual stream [M, N] and an RMSNorm reads the sum next.  Where the weight-streaming kernel runs (a
    decode step), it does both in its epilogue and a ``Prenormed`` comes back; otherwise the plain product does,
    and the caller adds and normalises as usual.  ``upcoming``: the matrix that the kernel after this one streams;
    the weight-streaming kernel asks for its start to be brought into L2 as its blocks end."""
    kernel = _fits(x, w)
    if isinstance(x, Prenormed) and not kernel:
        x = x.materialize()
        kernel = _fits(x, w)
    rows = x.scaled if isinstance(x, Prenormed) else x
    _need_cuda(rows, w, bias)
    if follow is not None and bias is None and not out_float32 and kernel:
        residual, norm_weight, norm_eps = follow
        M, N = rows.shape[0], w.shape[0]
        if (residual.dtype == torch.float32 and tuple(residual.shape) == (M, N) and residual.is_contiguous()
                and norm_weight.dtype == torch.float32 and norm_weight.numel() == N):
            scaled = torch.empty((M, N), dtype=torch.bfloat16, device=rows.device)
            _rows, sumsq, tiles, eps = _rows_and_scale(x)
            table = torch.empty((-(-N // 16), 8), dtype=torch.float32, device=rows.device)
            _run(_bf16(), "fe_skinny_gemm_residual", _ptr(rows), _ptr(w), _ptr(residual), _ptr(norm_weight), _ptr(scaled),
                 _ptr(table), _c_int(M), _c_int(N), _c_int(rows.shape[1]), sumsq, tiles, eps,
                 *_upcoming(upcoming, M, UPCOMING_TAIL_BYTES), _stream())
            return Prenormed(scaled, table, norm_eps, residual, norm_weight)
    if kernel and w.dtype == torch.bfloat16:
        wide = out_float32 or bias is not None           # a bias is added in float32, before the one rounding
        y = skinny_gemm(x, w, EPI_F32 if wide else EPI_BF16, upcoming=upcoming)
        if bias is not None:
            y += bias
        return y if out_float32 or not wide else y.to(torch.bfloat16)
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise ValueError(f"linear: shapes {tuple(x.shape)} x {tuple(w.shape)}")
    if not x.is_contiguous():
        x = x.contiguous()
    if w.dtype == torch.float32:
        y = gemm_fp32(x if x.dtype == torch.float32 else x.float(), w, bias)
        return y if (out_float32 or x.dtype == torch.float32) else y.to(x.dtype)
    if w.dtype != torch.bfloat16 or x.dtype != torch.bfloat16:
        raise TypeError(f"linear: weight {w.dtype} with activations {x.dtype}")
    wide = out_float32 or bias is not None           # a bias is added in float32, before the one rounding
    y = torch.mm(x, w.t(), out_dtype=torch.float32) if wide else torch.mm(x, w.t())
    if bias is not None:
        y += bias
    return y if out_float32 or not wide else y.to(torch.bfloat16)


SKINNY_MAX_ROWS = 8          # beyond this the library product is as fast or faster
SKINNY_QKV_MAX_ROWS = 8      # the fused projection + bias + rotation + cache write takes one 8-row tile of tokens
EPI_BF16, EPI_F32, EPI_SWIGLU = 0, 1, 2


def skinny_ok(x, w) -> bool:
    """Whether the weight-streaming kernel is used for this product: bfloat16, up to 8 rows (the
    kernel itself takes up to 16), K a multiple of 64."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 1 <= x.shape[0] <= SKINNY_MAX_ROWS
            and x.shape[1] % 64 == 0 and x.is_contiguous() and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def skinny_gemm(x, w, epilogue: int = EPI_BF16, upcoming=None):
    """x [M <= 16, K] (a tensor or a Prenormed) times w [N, K]^T by streaming w once; see csrc/gemm_skinny.cu."""
    x, sumsq, tiles, eps = _rows_and_scale(x)
    M, K = x.shape
    N = w.shape[0]
    if epilogue == EPI_SWIGLU:
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    else:
        out = torch.empty((M, N), dtype=torch.float32 if epilogue == EPI_F32 else torch.bfloat16, device=x.device)
    _run(_bf16(), "fe_skinny_gemm_scaled", _ptr(x), _ptr(w), _ptr(out), _c_int(M), _c_int(N), _c_int(K), _c_int(epilogue),
         sumsq, tiles, eps, *_upcoming(upcoming, M, UPCOMING_TAIL_BYTES), _stream())
    return out


FUSED_NORM_MAX_ROWS = SKINNY_MAX_ROWS     # steps of up to this many tokens do their norms in the products' epilogues


TCGEN05_MIN_K = 1024
TCGEN05_MIN_ROWS = 1024      # measured: from about this many rows the fused kernel matches the library + activation


def tcgen05_ok(x, w) -> bool:
    """Whether the tcgen05 kernel is used for this product: bfloat16, many rows (prefill), K a multiple of 8 and
    long enough for the products of a tile to cover its epilogue (at K = 896 the library + activation is 10 % ahead,
    from K = 1,536 on the fused kernel is)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] >= TCGEN05_MIN_ROWS
            and x.shape[1] >= TCGEN05_MIN_K and x.shape[1] % 8 == 0 and x.is_contiguous() and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tcgen05(x, w, epilogue: int = EPI_BF16):
    """x [M, K] times w [N, K]^T on tcgen05 tensor cores (TMA operands, TMEM accumulator);
    epilogue EPI_BF16 or EPI_SWIGLU.  See csrc/gemm_tcgen05.cu."""
    _need_cuda(x, w)
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not x.is_contiguous() or not w.is_contiguous():
        raise TypeError("gemm_tcgen05 takes contiguous bfloat16 operands")
    out = torch.empty((M, N // 2 if epilogue == EPI_SWIGLU else N), dtype=torch.bfloat16, device=x.device)
    _run(_bf16(), "fe_gemm_tcgen05", _ptr(x), _ptr(w), _ptr(out), _c_int(M), _c_int(N), _c_int(K), _c_int(epilogue),
         _ptr(status_word(x.device)), _stream())
    return out


def swiglu(gate_up, intermediate):
    _need_cuda(gate_up)
    T = gate_up.shape[0]
    if gate_up.shape[1] != 2 * intermediate or not gate_up.is_contiguous():
        raise ValueError("swiglu: input must be contiguous [T, 2 * intermediate]")
    out = torch.empty((T, intermediate), dtype=gate_up.dtype, device=gate_up.device)
    _run(_core(), "fe_swiglu", _ptr(gate_up), _ptr(out), _c_int(T), _c_int(intermediate),
         _c_int(_code(gate_up.dtype)), _stream())
    return out


def linear_swiglu(x, w, intermediate, upcoming=None):
    """silu(x Wg^T) * (x Wu^T) with w = [Wg; Wu] ([2I, K]); one kernel for a handful of rows."""
    kernel = _fits(x, w) if w.shape[0] == 2 * intermediate else ""
    if isinstance(x, Prenormed) and not kernel:
        x = x.materialize()
        kernel = _fits(x, w) if w.shape[0] == 2 * intermediate else ""
    if kernel == "skinny":
        return skinny_gemm(x, w, EPI_SWIGLU, upcoming=upcoming)
    if tcgen05_ok(x, w) and w.shape[0] == 2 * intermediate:
        return gemm_tcgen05(x, w, EPI_SWIGLU)
    return swiglu(linear(x, w), intermediate)


def qkv_bias_rope_cache(qkv, bias, positions, inv_freq, rot, slot_mapping, k_cache, v_cache,
                        nq, nkv, d, page_size, src=None):
    """qkv [T, (nq + 2 nkv) d] = projection + bias, with the rotary encoding of the query and key heads;
    key and value heads are also written to their cache slots (slot_mapping None: no write).  The
    projection is ``qkv`` itself (rewritten in place) or ``src``, a float32 tensor of the same shape: a
    bfloat16 result is then rounded once, after bias and rotation."""
    _need_cuda(qkv, bias, positions, inv_freq, slot_mapping, k_cache, v_cache, src)
    T, width = qkv.shape
    if width != (nq + 2 * nkv) * d or not qkv.is_contiguous():
        raise ValueError("qkv_bias_rope_cache: qkv must be contiguous [T, (nq + 2 nkv) d]")
    if src is not None and (src.shape != qkv.shape or not src.is_contiguous() or src.dtype not in (torch.float32, qkv.dtype)):
        raise ValueError("qkv_bias_rope_cache: src must be contiguous, shaped like qkv, float32 or of its dtype")
    src_float = src is not None and src.dtype == torch.float32 and qkv.dtype != torch.float32
    if k_cache.dtype != qkv.dtype or tuple(k_cache.shape[1:]) != (nkv, page_size, d) or not k_cache.is_contiguous() \
            or not v_cache.is_contiguous():
        raise ValueError("qkv_bias_rope_cache: cache must be contiguous [pages, nkv, page_size, d] in the compute dtype")
    if bias is not None and bias.dtype != torch.float32:
        raise TypeError("biases are float32")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rot // 2):
        raise ValueError("inv_freq must be float32 [rot / 2]")
    num_slots = k_cache.shape[0] * page_size
    _run(_core(), "fe_qkv_bias_rope_cache", _ptr(qkv if src is None else src), _c_int(1 if src_float else 0), _ptr(qkv),
         _ptr(bias), _ptr(positions), _ptr(inv_freq), _c_int(rot),
         _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), _c_int(T), _c_int(nq), _c_int(nkv), _c_int(d),
         _c_int(page_size), _c_ll(num_slots), _c_int(_code(qkv.dtype)), _ptr(status_word(qkv.device)), _stream())


def qkv_projection(h, w, bias, positions, inv_freq, rot, slot_mapping, k_cache, v_cache, nq, nkv, d, page_size):
    """The query/key/value projection of an attention layer: h w^T + bias, rotary encoding of the
    query and key heads, new keys and values written to their cache slots (slot_mapping None: no
    write).  Returns qkv [T, (nq + 2 nkv) d].  For a handful of rows (decode) with the whole head
    rotated this is ONE kernel (csrc/gemm_skinny.cu); otherwise the product and the fused
    bias/rotation/cache-write kernel."""
    kernel = _fits(h, w)
    if isinstance(h, Prenormed) and not kernel:
        h = h.materialize()
        kernel = _fits(h, w)
    rows = h.scaled if isinstance(h, Prenormed) else h
    _need_cuda(rows, w, bias, positions, inv_freq, slot_mapping, k_cache, v_cache)
    whole_head = (inv_freq is not None and rot == d and k_cache.dtype == torch.bfloat16 and w.shape[0] == (nq + 2 * nkv) * d
                  and (bias is None or bias.dtype == torch.float32))
    if kernel == "skinny" and whole_head and d % 16 == 0 and rows.shape[0] <= SKINNY_QKV_MAX_ROWS:
        T = rows.shape[0]
        _rows, sumsq, tiles, eps = _rows_and_scale(h)
        out = torch.empty((T, w.shape[0]), dtype=torch.bfloat16, device=rows.device)
        _run(_bf16(), "fe_skinny_qkv", _ptr(rows), _ptr(w), _ptr(out), _ptr(bias), _ptr(positions), _ptr(inv_freq),
             _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), _c_int(T), _c_int(rows.shape[1]), _c_int(nq), _c_int(nkv),
             _c_int(d), _c_int(page_size), _c_ll(k_cache.shape[0] * page_size), sumsq, tiles, eps,
             _ptr(status_word(rows.device)), _stream())
        return out
    if isinstance(h, Prenormed):
        h = h.materialize()
    if h.dtype == torch.float32:
        qkv = linear(h, w)
        qkv_bias_rope_cache(qkv, bias, positions, inv_freq, rot, slot_mapping, k_cache, v_cache, nq, nkv, d, page_size)
        return qkv
    # the product stays float32 until bias and rotation are in, as in the fused kernel: a token's keys and values
    # are rounded once whichever path its step took
    product = linear(h, w, out_float32=True)
    qkv = torch.empty(product.shape, dtype=h.dtype, device=h.device)
    qkv_bias_rope_cache(qkv, bias, positions, inv_freq, rot, slot_mapping, k_cache, v_cache, nq, nkv, d, page_size,
                        src=product)
    return qkv


def paged_attention_simt(q, q_stride, k_cache, v_cache, block_table, cu_q, q_start, token_request, T, nq, nkv, d,
                         page_size, scale, window):
    out = torch.empty((T, nq * d), dtype=k_cache.dtype, device=k_cache.device)
    _run(_core(), "fe_paged_attention_simt", _ptr(q), _c_ll(q_stride), _ptr(out), _c_ll(nq * d), _ptr(k_cache),
         _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _ptr(cu_q), _ptr(q_start),
         _ptr(token_request), _c_int(T), _c_int(nq), _c_int(nkv), _c_int(d), _c_int(page_size),
         _c_int(k_cache.shape[0]), _c_float(scale), _c_int(window), _c_int(_code(k_cache.dtype)),
         _ptr(status_word(k_cache.device)), _stream())
    return out


_scratch: dict = {}
_scratch_kept: list = []     # every scratch buffer ever handed out (see scratch())
_sm_count: dict = {}


def sm_count(device=None) -> int:
    """Multiprocessors of ``device`` (the current CUDA device when None), as the driver reports them:
    the one number every launch heuristic here scales with (the kernels' own host code asks the same
    attribute through the helper in ``csrc/errors.cu``)."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if index not in _sm_count:
        _sm_count[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return _sm_count[index]


def _bf16():
    return library.load("bf16")


def scratch(device, nbytes: int) -> torch.Tensor:
    """Scratch memory of at least ``nbytes`` bytes on ``device``, grown on demand.  A buffer that has been
    handed out is never freed: a CUDA graph captured with it keeps its address, and replays it long after a
    larger buffer has taken its place for new calls."""
    have = _scratch.get(device)
    if have is None or have.numel() < nbytes:
        key = str(torch.device(device))            # "cuda:0" and torch.device("cuda:0") share one buffer
        have = _scratch.get(key)
        if have is None or have.numel() < nbytes:
            with torch.inference_mode(False):
                have = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
            _scratch_kept.append(have)
        for k in [k for k in _scratch if str(torch.device(k)) == key]:
            _scratch[k] = have
        _scratch[key] = _scratch[device] = have
    return have


DECODE_MAX_SPLITS = 256      # what the merge kernel of decode attention takes (fe_paged_decode_max_splits)


def decode_splits(requests: int, nkv: int, max_ctx_len: int, sms: int | None = None) -> int:
    """How many ways the keys of a request are split in decode.  Between half a round and one round of resident
    blocks (six blocks fit an SM; never more than a round: a few blocks over it would run alone after it): towards
    the full round when a split still has six tiles of 32 keys or more to walk, towards the half when splits
    would get short and the merge dominate; never a split shorter than two tiles, never more splits than the
    merge kernel takes (one request with one or two key/value heads at a very long context would ask for more)."""
    sms = sms or sm_count()
    tiles = max(1, -(-max_ctx_len // 32))
    pairs = max(1, requests * nkv)
    most = max(1, 6 * sms // pairs)               # rounded down: a few blocks over the round would run alone after it
    least = max(1, (3 * sms + pairs // 2) // pairs)
    want = min(most, max(least, tiles // 6), DECODE_MAX_SPLITS)
    return int(max(1, min(want, tiles // 2)))


def paged_decode_mma(q, q_stride, k_cache, v_cache, block_table, cu_q, q_start, requests, nq, nkv, d, page_size,
                     scale, window, splits, out=None, upcoming=None):
    """Tensor-core decode attention (one token per request), keys split ``splits`` ways.  ``upcoming``: the
    matrix that the next kernel streams (the output projection); extra blocks of the merge kernel ask for its
    start to be brought into L2."""
    if out is None:
        out = torch.empty((requests, nq * d), dtype=torch.bfloat16, device=k_cache.device)
    lib = _bf16()
    need = lib.fe_paged_decode_scratch_bytes(_c_int(requests), _c_int(nq), _c_int(d), _c_int(splits))
    work = scratch(k_cache.device, need) if need else None
    _run(lib, "fe_paged_decode_mma_upcoming", _ptr(q), _c_ll(q_stride), _ptr(out), _c_ll(out.stride(0)), _ptr(work),
         _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _ptr(cu_q), _ptr(q_start),
         _c_int(requests), _c_int(nq), _c_int(nkv), _c_int(d), _c_int(page_size), _c_int(k_cache.shape[0]),
         _c_float(scale), _c_int(window), _c_int(splits), *_upcoming(upcoming, requests, UPCOMING_BYTES_MERGE),
         _ptr(status_word(k_cache.device)), _stream())
    return out


DECODE_CLUSTER_MAX_SPLITS = 16       # blocks of one thread-block cluster (fe_paged_decode_cluster_max_splits)
DECODE_CLUSTER_MAX_TILES = 8         # a split of a cluster walks at most this many tiles of 32 keys ...
DECODE_CLUSTER_ONE_ROUND_MIN = 8     # ... and a cluster is cut down to fit one round only if this many splits remain
_CLUSTERS_RESIDENT: dict = {}


def clusters_resident(requests: int, nq: int, nkv: int, d: int, splits: int) -> int:
    """How many clusters of ``splits`` blocks of the decode kernel the device holds at once (asked of the driver once
    per shape): a cluster lives inside one of the GPU's processing clusters, so it is fewer than blocks / splits."""
    key = (requests, nq, nkv, d, splits)
    if key not in _CLUSTERS_RESIDENT:
        _CLUSTERS_RESIDENT[key] = int(_bf16().fe_paged_decode_cluster_resident(requests, nq, nkv, d, splits))
    return _CLUSTERS_RESIDENT[key]


def decode_cluster_splits(splits: int, max_ctx_len: int, clusters: int = 0, resident=None) -> int:
    """How many splits the cluster kernel takes for a step that ``decode_splits`` would split ``splits`` ways, or 0
    when the two-kernel form is the better one: a long context of a small batch, which wants more splits than a
    cluster holds, keeps them and the separate merge (batch 8 at 8,192 tokens: 3.53 against 3.59 ms a step of the 7B
    shape, at 16,384: 4.12 against 4.24; batch 1 at 16,384: 3.0 against 3.8).

    ``clusters``: how many clusters the step needs (requests x key/value heads); ``resident(s)``: how many clusters of
    s blocks the device holds at once.  A few clusters over one round run alone after it: 32 clusters of 15 or 16
    blocks, of which fewer than 32 fit, make a step 3.25 ms long where clusters of 8 to 14 make it 3.11 to 3.13, and
    64 clusters of 9 cost 4.07 ms where 64 of 8 cost 3.80.  So the count is cut down to the largest that fits one
    round, if that leaves eight splits or more; large batches, whose clusters of two to six blocks take several
    rounds anyway, keep their count (batch 64: three splits 4.88 ms, two 4.97)."""
    if splits <= 1:
        return 0
    most = min(splits, DECODE_CLUSTER_MAX_SPLITS)
    if splits > most and -(-max_ctx_len // 32) > most * DECODE_CLUSTER_MAX_TILES:
        return 0
    if resident is None or clusters <= 0:
        return most
    fit = next((s for s in range(most, 1, -1) if resident(s) >= clusters), 0)
    if fit >= min(most, DECODE_CLUSTER_ONE_ROUND_MIN):
        return fit
    return most if resident(most) > 0 else 0


def paged_decode_cluster(q, q_stride, k_cache, v_cache, block_table, cu_q, q_start, requests, nq, nkv, d, page_size,
                         scale, window, splits, out=None):
    """Decode attention with the splits of each (request, key/value head) as one thread-block cluster that merges
    its partial results through distributed shared memory: one launch, no scratch memory; splits <= 16."""
    if out is None:
        out = torch.empty((requests, nq * d), dtype=torch.bfloat16, device=k_cache.device)
    _run(_bf16(), "fe_paged_decode_cluster", _ptr(q), _c_ll(q_stride), _ptr(out), _c_ll(out.stride(0)), _ptr(k_cache),
         _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _ptr(cu_q), _ptr(q_start), _c_int(requests),
         _c_int(nq), _c_int(nkv), _c_int(d), _c_int(page_size), _c_int(k_cache.shape[0]), _c_float(scale), _c_int(window),
         _c_int(splits), _ptr(status_word(k_cache.device)), _stream())
    return out


def paged_prefill_mma(q, q_stride, k_cache, v_cache, block_table, cu_q, q_start, T, requests, max_q_len, nq, nkv, d,
                      page_size, scale, window):
    """Tensor-core attention for portions of any length (decoded tokens are portions of one)."""
    out = torch.empty((T, nq * d), dtype=torch.bfloat16, device=k_cache.device)
    _run(_bf16(), "fe_paged_prefill_mma", _ptr(q), _c_ll(q_stride), _ptr(out), _c_ll(nq * d), _ptr(k_cache),
         _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _ptr(cu_q), _ptr(q_start), _c_int(requests),
         _c_int(max_q_len), _c_int(nq), _c_int(nkv), _c_int(d), _c_int(page_size), _c_int(k_cache.shape[0]),
         _c_float(scale), _c_int(window), _ptr(status_word(k_cache.device)), _stream())
    return out


def tcgen05_attention_ok(max_q_len, nq, nkv, d, lengths=None, starts=None, sms: int | None = None):
    """The tcgen05 prefill kernel takes head sizes 64 and 128, portions of any length: measured against the
    mma.sync kernel it is level on portions of a few tokens and ahead everywhere else, the more the longer the
    context.  Other head sizes go to the mma.sync kernel, and so does a step of many requests that bring a few
    tokens each to short contexts (``lengths`` and ``starts`` given): one tcgen05 block is resident on an SM and
    costs a few microseconds before its first tile, where several of the lighter blocks share an SM."""
    if d not in (64, 128):
        return False
    if lengths:
        group = nq // nkv
        blocks = nkv * sum(-(-n * group // 256) for n in lengths)
        rows = nkv * group * sum(lengths)
        longest = max(s + n for s, n in zip(starts, lengths))
        if blocks > (sms or sm_count()) and rows < 96 * blocks and longest <= 1024:
            return False
    return True


PREFILL_MAX_SPLITS = 32
PREFILL_TILES_PER_SPLIT = 4      # a split walks at least this many tiles of 64 keys
PREFILL_SPLIT_FROM_TILES = 16    # shorter walks are over before a second kernel could merge them


def prefill_splits(lengths, starts, nq, nkv, window=0, sms: int | None = None) -> int:
    """Into how many blocks the tcgen05 prefill kernel shares out the keys of each pair of row tiles.  One block
    a multiprocessor is resident; a short portion late in a long context fills few of them, and each walks the whole
    context, so its keys are split until the blocks about cover the device."""
    group = nq // nkv
    blocks = nkv * sum(-(-n * group // 256) for n in lengths)
    longest = max(min(s + n, window + n) if window > 0 else s + n for s, n in zip(starts, lengths))
    tiles = -(-longest // 64)
    if tiles < PREFILL_SPLIT_FROM_TILES:
        return 1
    return int(max(1, min((sms or sm_count()) // max(1, blocks), tiles // PREFILL_TILES_PER_SPLIT, PREFILL_MAX_SPLITS)))


def paged_prefill_tcgen05(q, q_stride, k_cache, v_cache, block_table, cu_q, q_start, T, requests, max_q_len, nq, nkv, d,
                          page_size, scale, window, splits=1):
    """Prefill attention on tcgen05 tensor cores: 128 (query, head) rows a block, head sizes 64 and 128.
    ``splits`` > 1 shares the keys of each pair of row tiles out over that many blocks and merges their results."""
    out = torch.empty((T, nq * d), dtype=torch.bfloat16, device=k_cache.device)
    part = scratch(k_cache.device, 4 * T * nq * splits * (d + 1)) if splits > 1 else None
    _run(_bf16(), "fe_paged_prefill_tcgen05", _ptr(q), _c_ll(q_stride), _ptr(out), _c_ll(nq * d), _ptr(k_cache),
         _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _ptr(cu_q), _ptr(q_start), _c_int(requests),
         _c_int(max_q_len), _c_int(nq), _c_int(nkv), _c_int(d), _c_int(page_size), _c_int(k_cache.shape[0]),
         _c_float(scale), _c_int(window), _c_int(splits), _ptr(part),
         _c_ll(T), _ptr(status_word(k_cache.device)), _stream())
    return out


def paged_attention(qkv, k_cache, v_cache, block_table, ctx, nq, nkv, d, page_size, scale, window, upcoming=None):
    """Causal grouped-query attention of the step's tokens over their requests' pages.
    qkv [T, >= nq d] holds the (rotated) queries in its first nq d columns; returns [T, nq d].
    float32 runs on CUDA cores (true 32-bit); bfloat16 on tensor cores: the split-KV decode
    kernel when every request brings one token, else a prefill kernel (tcgen05 for portions of
    head size 64 or 128, mma.sync otherwise)."""
    _need_cuda(qkv, k_cache, v_cache, block_table)
    T = qkv.shape[0]
    if qkv.dtype != k_cache.dtype:
        raise TypeError("queries and cache differ in dtype")
    if qkv.dtype == torch.float32:
        return paged_attention_simt(qkv, qkv.stride(0), k_cache, v_cache, block_table, ctx.cu_q, ctx.q_start,
                                    ctx.token_request, T, nq, nkv, d, page_size, scale, window)
    requests = ctx.cu_q.numel() - 1
    if ctx.max_q_len == 1 and nq // nkv <= 16:
        splits = decode_splits(requests, nkv, ctx.max_ctx_len)
        clustered = decode_cluster_splits(splits, ctx.max_ctx_len, requests * nkv,
                                          lambda s: clusters_resident(requests, nq, nkv, d, s))
        if clustered:
            return paged_decode_cluster(qkv, qkv.stride(0), k_cache, v_cache, block_table, ctx.cu_q, ctx.q_start, requests,
                                        nq, nkv, d, page_size, scale, window, clustered)
        return paged_decode_mma(qkv, qkv.stride(0), k_cache, v_cache, block_table, ctx.cu_q, ctx.q_start, requests,
                                nq, nkv, d, page_size, scale, window, splits, upcoming=upcoming)
    lengths = getattr(ctx, "host_lengths", None)
    if tcgen05_attention_ok(ctx.max_q_len, nq, nkv, d, lengths, getattr(ctx, "host_starts", None)):
        splits = prefill_splits(lengths, ctx.host_starts, nq, nkv, window) if lengths else 1
        return paged_prefill_tcgen05(qkv, qkv.stride(0), k_cache, v_cache, block_table, ctx.cu_q, ctx.q_start, T, requests,
                                     ctx.max_q_len, nq, nkv, d, page_size, scale, window, splits)
    return paged_prefill_mma(qkv, qkv.stride(0), k_cache, v_cache, block_table, ctx.cu_q, ctx.q_start, T, requests,
                             ctx.max_q_len, nq, nkv, d, page_size, scale, window)


def sample(logits, temperature, top_k, seed, draw, blocks: int = 0):
    """int32 [R]: one token per row of float32 logits [R, V]; see csrc/sampling.cu.  ``blocks``: how many thread
    blocks (a cluster of 1, 2, 4 or 8) share a row; 0 lets the kernel library choose by the number of rows.  The
    tokens do not depend on it."""
    _need_cuda(logits, temperature, top_k, seed, draw)
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise TypeError("sample: logits must be float32 with unit column stride")
    if temperature.dtype != torch.float32 or top_k.dtype != torch.int32 or seed.dtype != torch.int64 \
            or draw.dtype != torch.int64:
        raise TypeError("sample: temperature float32, top_k int32, seed and draw int64")
    out = torch.empty(R, dtype=torch.int32, device=logits.device)
    if blocks:
        _run(_core(), "fe_sample_blocks", _ptr(logits), _c_ll(logits.stride(0)), _c_int(R), _c_int(V), _ptr(temperature),
             _ptr(top_k), _ptr(seed), _ptr(draw), _ptr(out), _c_int(blocks), _stream())
    else:
        _run(_core(), "fe_sample", _ptr(logits), _c_ll(logits.stride(0)), _c_int(R), _c_int(V), _ptr(temperature),
             _ptr(top_k), _ptr(seed), _ptr(draw), _ptr(out), _stream())
    return out


# ---- a whole decoder layer as one call --------------------------------------------------------------------------
import ctypes as _ct


class _FeLayer(_ct.Structure):
    """Mirror of ``struct FeLayer`` (csrc/layer_executor.cu): field for field, in its order."""
    _fields_ = [(n, _ct.c_void_p) for n in ("input_norm", "post_norm", "qkv_weight", "qkv_bias", "out_weight", "gate_up_weight",
                                             "down_weight", "inv_freq")] + \
               [("eps", _ct.c_float), ("scale", _ct.c_float)] + \
               [(n, _ct.c_int) for n in ("hidden", "nq", "nkv", "d", "intermediate", "rot", "window")]


class _FeStep(_ct.Structure):
    """Mirror of ``struct FeStep``."""
    _fields_ = [(n, _ct.c_void_p) for n in ("positions", "slot_mapping", "block_table", "cu_q", "q_start", "residual", "workspace",
                                             "attention_scratch", "status")] + \
               [("workspace_bytes", _ct.c_longlong)] + \
               [(n, _ct.c_int) for n in ("T", "R", "bt_stride", "max_q_len", "page_size", "num_pages", "attention", "splits",
                                         "gate_up_tcgen05")]


NATIVE_LAYER_MIN_ROWS = SKINNY_MAX_ROWS + 1      # fewer rows take the fused weight-streaming kernels, one by one
_workspace: dict = {}
_native_off = False           # set when cuBLAS could not be found from the library: kernel by kernel from then on


class NativeLayer:
    """The weights and sizes of one pre-norm attention + SwiGLU layer in the form ``fe_layer_forward`` takes them (the
    cache is the step's: a model may be run over one cache manager after another).  Holds references to the tensors
    it points at."""

    def __init__(self, input_norm, post_norm, eps, qkv_weight, qkv_bias, out_weight, gate_up_weight, down_weight, inv_freq,
                 rot, nq, nkv, d, scale, window):
        self.keep = (input_norm, post_norm, qkv_weight, qkv_bias, out_weight, gate_up_weight, down_weight, inv_freq)
        _need_cuda(*[t for t in self.keep if t is not None])
        self.hidden, self.intermediate = int(out_weight.shape[0]), int(down_weight.shape[1])
        self.nq, self.nkv, self.d, self.window = nq, nkv, d, window
        self.c = _FeLayer(_ptr(input_norm), _ptr(post_norm), _ptr(qkv_weight), _ptr(qkv_bias), _ptr(out_weight),
                          _ptr(gate_up_weight), _ptr(down_weight), _ptr(inv_freq),
                          float(eps), float(scale), self.hidden, nq, nkv, d, self.intermediate, int(rot), int(window))

    @staticmethod
    def fits(*matrices) -> bool:
        return all(m is not None and m.is_cuda and m.dtype == torch.bfloat16 and m.is_contiguous() and m.data_ptr() % 16 == 0
                   and m.shape[1] % 8 == 0 for m in matrices)


def _layer_workspace(device, nbytes: int) -> torch.Tensor:
    have = _workspace.get(device)
    if have is None or have.numel() < nbytes:
        with torch.inference_mode(False):
            have = _workspace[device] = torch.empty(nbytes, dtype=torch.uint8, device=device)
    return have


def native_step(ctx, group, layer: NativeLayer, residual, write_cache: bool):
    """The step's side of ``fe_layer_forward`` for layers of this shape: built once per step and cache group."""
    T, requests = residual.shape[0], ctx.cu_q.numel() - 1
    nq, nkv, d = layer.nq, layer.nkv, layer.d
    scratch_bytes = 0
    if ctx.max_q_len == 1 and nq // nkv <= 16:
        splits = decode_splits(requests, nkv, ctx.max_ctx_len)
        clustered = decode_cluster_splits(splits, ctx.max_ctx_len, requests * nkv,
                                          lambda s: clusters_resident(requests, nq, nkv, d, s))
        kind, splits = (0, clustered) if clustered else (1, splits)
        if kind == 1:
            scratch_bytes = _bf16().fe_paged_decode_scratch_bytes(_c_int(requests), _c_int(nq), _c_int(d), _c_int(splits))
    elif tcgen05_attention_ok(ctx.max_q_len, nq, nkv, d, ctx.host_lengths, ctx.host_starts):
        kind, splits = 2, prefill_splits(ctx.host_lengths, ctx.host_starts, nq, nkv, layer.window)
        scratch_bytes = 4 * T * nq * splits * (d + 1) if splits > 1 else 0
    else:
        kind, splits = 3, 1
    need = _bf16().fe_layer_workspace_bytes(_c_int(T), _c_int(layer.hidden), _c_int(nq), _c_int(nkv), _c_int(d), _c_int(layer.intermediate))
    work = _layer_workspace(residual.device, need)
    attention_scratch = scratch(residual.device, scratch_bytes) if scratch_bytes else None
    gate_up_tcgen05 = T >= TCGEN05_MIN_ROWS and layer.hidden >= TCGEN05_MIN_K
    step = _FeStep(_ptr(ctx.positions), _ptr(group.slot_mapping) if write_cache else None, _ptr(group.block_table), _ptr(ctx.cu_q),
                   _ptr(ctx.q_start), _ptr(residual), _ptr(work), _ptr(attention_scratch), _ptr(status_word(residual.device)),
                   work.numel(), T, requests, int(group.block_table.shape[1]), int(ctx.max_q_len), int(group.page_size),
                   int(group.storage.shape[2]), kind, int(splits), 1 if gate_up_tcgen05 else 0)
    step.keep = (work, attention_scratch, residual)
    # entry points of this package behind one layer, counted as ``_run`` counts them: two norms, rotation and cache
    # write, attention (with its merge, if any), the activation or the fused gate/up product
    step.launches = 5
    return step


def layer_forward(layer: NativeLayer, step, k_cache, v_cache, pending, out):
    """One layer through ``fe_layer_forward``; False when the library cannot (no cuBLAS in the process): the caller
    then runs the layer kernel by kernel, now and from then on."""
    global _native_off, launches
    lib = _bf16()
    rc = lib.fe_layer_forward(_ct.byref(layer.c), _ct.byref(step), _ptr(k_cache), _ptr(v_cache), _ptr(pending), _ptr(out), _stream())
    if rc == 3:
        _native_off = True
        return False
    if rc != 0:
        raise RuntimeError(f"fe_layer_forward failed: {lib.fe_last_error().decode()}")
    launches += step.launches
    return True


def native_layers_usable(ctx) -> bool:
    return (not _native_off and ctx.dtype == torch.bfloat16 and ctx.num_tokens >= NATIVE_LAYER_MIN_ROWS
            and not torch.cuda.is_current_stream_capturing())
