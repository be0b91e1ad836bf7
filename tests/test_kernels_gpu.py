"""Each CUDA kernel alone against its plain PyTorch reference, at sizes other than the engine's:
widths and vocabularies that are no powers of two, head sizes in steps of 16, ragged tails,
reversed and scattered block tables, windows, and inputs made so that a far key matters."""
import math
import random
import types

import pytest
import torch

import kernel_refs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from flexengine_b200 import ops as cuda_ops
    return cuda_ops


def bar(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def rand(shape, dtype, gen, scale=1.0):
    return (torch.randn(shape, generator=gen, device=DEV, dtype=torch.float32) * scale).to(dtype)


@pytest.fixture()
def gen():
    g = torch.Generator(device=DEV)
    g.manual_seed(1234)
    return g


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("V,H", [(301, 80), (1000, 3584), (17, 24)])
def test_embedding(dtype, V, H, gen):
    table = rand((V, H), dtype, gen)
    ids = torch.randint(0, V, (37,), device=DEV, dtype=torch.int32, generator=gen)
    got = ops().embedding(ids, table)
    assert got.dtype == torch.float32
    torch.testing.assert_close(got, kernel_refs.embedding(ids, table), atol=0, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H", [(1, 64), (5, 80), (7, 3584), (3, 5000), (2, 24)])
def test_add_rmsnorm(dtype, T, H, gen):
    weight = 1 + 0.1 * torch.randn(H, device=DEV, generator=gen)
    for eps in (1e-6, 1e-2):
        residual = torch.randn(T, H, device=DEV, generator=gen)
        delta = rand((T, H), dtype, gen)
        r1, r2 = residual.clone(), residual.clone()
        got = ops().add_rmsnorm(r1, delta, weight, eps, dtype)
        want = kernel_refs.add_rmsnorm(r2, delta, weight, eps, dtype)
        torch.testing.assert_close(got.float(), want.float(), **bar(dtype))
        torch.testing.assert_close(r1, r2, atol=1e-6, rtol=1e-6)          # residual updated in place
        got0 = ops().add_rmsnorm(r1, None, weight, eps, dtype)
        torch.testing.assert_close(got0.float(), kernel_refs.add_rmsnorm(r2, None, weight, eps, dtype).float(), **bar(dtype))
        rows = torch.tensor([T - 1, 0, T // 2], device=DEV, dtype=torch.int32)
        keep = r1.clone()
        got_rows = ops().add_rmsnorm(r1, delta, weight, eps, dtype, rows)
        want_rows = kernel_refs.add_rmsnorm(r2, delta, weight, eps, dtype, rows)
        torch.testing.assert_close(got_rows.float(), want_rows.float(), **bar(dtype))
        torch.testing.assert_close(r1, keep, atol=0, rtol=0)             # rows mode leaves the residual alone
        # the hint at the matrix that comes next changes nothing but what lies in L2 (odd sizes: the last line is partial)
        nxt = rand((333, 77), torch.bfloat16, gen)
        r3, r4 = residual.clone(), residual.clone()
        hinted = ops().add_rmsnorm(r3, delta, weight, eps, dtype, upcoming=nxt)
        torch.testing.assert_close(hinted, ops().add_rmsnorm(r4, delta, weight, eps, dtype), atol=0, rtol=0)
        torch.testing.assert_close(r3, r4, atol=0, rtol=0)


@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (33, 130, 70), (64, 64, 16), (100, 301, 257), (3, 1000, 3584)])
def test_gemm_fp32_is_true_fp32(M, N, K, gen):
    x = torch.randn(M, K, device=DEV, generator=gen)
    w = torch.randn(N, K, device=DEV, generator=gen)
    b = torch.randn(N, device=DEV, generator=gen)
    want = (x.double() @ w.double().T + b.double())
    got = ops().linear(x, w, b)
    assert got.dtype == torch.float32
    # float32 accumulation over K terms of unit variance: error ~ sqrt(K) * 2^-24 * |terms|
    torch.testing.assert_close(got.double(), want, atol=2e-6 * math.sqrt(K) * 4, rtol=1e-5)
    # a row's result does not depend on how many rows are in the batch
    alone = ops().linear(x[:1].contiguous(), w, b)
    assert torch.equal(alone[0], got[0])


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (8, 301 * 8, 80), (130, 384, 192)])
def test_linear_bf16(M, N, K, gen):
    x, w = rand((M, K), torch.bfloat16, gen), rand((N, K), torch.bfloat16, gen, 0.05)
    want = x.float() @ w.float().T
    torch.testing.assert_close(ops().linear(x, w).float(), want, atol=2e-2, rtol=2e-2)
    got32 = ops().linear(x, w, None, out_float32=True)
    assert got32.dtype == torch.float32
    torch.testing.assert_close(got32, want, atol=1e-3, rtol=1e-3)
    # a weight stored in 32-bit stays so: the product is the true float32 one
    got = ops().linear(x, w.float())
    torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M", [1, 2, 7, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(301, 64), (24, 192), (768, 384), (4608, 3584), (16, 18944), (7184, 128), (9624, 64)])
def test_skinny_gemm(M, N, K, gen):
    # (7184, 128), (9624, 64): more 16-row tiles than one round of resident blocks (two tiles a block), one with a
    # ragged end; (16, 18944): one tile and a long K (sixteen warps split K)
    x, w = rand((M, K), torch.bfloat16, gen), rand((N, K), torch.bfloat16, gen, 0.05)
    want = x.float() @ w.float().T
    torch.testing.assert_close(ops().skinny_gemm(x, w, ops().EPI_F32), want, atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(ops().skinny_gemm(x, w, ops().EPI_BF16).float(), want, atol=2e-2, rtol=2e-2)
    if N % 2 == 0:
        got = ops().skinny_gemm(x, w, ops().EPI_SWIGLU)
        assert tuple(got.shape) == (M, N // 2)
        torch.testing.assert_close(got.float(), kernel_refs.swiglu(want.to(torch.bfloat16), N // 2).float(), atol=2e-2, rtol=3e-2)
    # the dispatch uses it for up to 8 rows and gives the same numbers either way
    torch.testing.assert_close(ops().linear(x, w).float(), want, atol=2e-2, rtol=2e-2)
    # twice the same: the reduction order is fixed
    assert torch.equal(ops().skinny_gemm(x, w, ops().EPI_F32), ops().skinny_gemm(x, w, ops().EPI_F32))


@pytest.mark.parametrize("M,N,K", [(13, 3581, 10240), (64, 2085, 3776), (135, 1000, 18944), (8, 3581, 10240)])
def test_products_are_float_sums_rounded_once_whichever_kernel_takes_them(M, N, K, gen):
    """A long K is split by the library's kernels; their partial sums must be added in float (the library's default
    would allow bfloat16 there: errors of up to four roundings).  Whether a product goes to the weight-streaming
    kernel (up to 8 rows) or to the library, its error is that of one bfloat16 rounding of the float result."""
    x, w = rand((M, K), torch.bfloat16, gen), rand((N, K), torch.bfloat16, gen, 0.05)
    want = x.float() @ w.float().T
    rounding = (want.to(torch.bfloat16).float() - want).abs().max()
    got = ops().linear(x, w)
    assert float((got.float() - want).abs().max()) <= 1.02 * float(rounding) + 1e-3
    wide = ops().linear(x, w, out_float32=True)
    torch.testing.assert_close(wide, want, atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (128, 128, 256), (100, 200, 192), (300, 384, 3584), (2048, 512, 320),
                                   (129, 24, 72), (2300, 520, 128), (4097, 256, 64), (4300, 264, 64)])
def test_gemm_tcgen05(M, N, K, gen):
    """The tcgen05 / TMEM / TMA product against float32 PyTorch: tails in M, N and K, several
    passes round the ring of stages, both epilogues."""
    x, w = rand((M, K), torch.bfloat16, gen), rand((N, K), torch.bfloat16, gen, 0.05)
    want = x.float() @ w.float().T
    bar16 = dict(atol=2e-2 * max(1.0, float(want.abs().max()) / 4), rtol=2e-2)
    torch.testing.assert_close(ops().gemm_tcgen05(x, w, ops().EPI_BF16).float(), want, **bar16)
    if N % 2 == 0:
        got = ops().gemm_tcgen05(x, w, ops().EPI_SWIGLU)
        assert tuple(got.shape) == (M, N // 2)
        g, u = want[:, :N // 2], want[:, N // 2:]
        torch.testing.assert_close(got.float(), g / (1 + torch.exp(-g)) * u, **bar16)
    ops().check_status(DEV)


def test_gemm_tcgen05_refuses_what_it_cannot_take(gen):
    with pytest.raises(RuntimeError, match="multiple of 8"):
        ops().gemm_tcgen05(rand((4, 60), torch.bfloat16, gen), rand((32, 60), torch.bfloat16, gen))


@pytest.mark.parametrize("M", [1, 5, 8])
@pytest.mark.parametrize("N,K", [(301, 4224), (1536, 8960), (40, 4096)])
def test_skinny_gemm_narrow_matrix_long_k(M, N, K, gen):
    """Fewer 16-row tiles than SMs and a long K: sixteen warps a block split K (66 steps leave the last warps less)."""
    x, w = rand((M, K), torch.bfloat16, gen), rand((N, K), torch.bfloat16, gen, 0.05)
    want = x.float() @ w.float().T
    torch.testing.assert_close(ops().skinny_gemm(x, w, ops().EPI_F32), want, atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(ops().linear(x, w).float(), want, atol=2e-2, rtol=2e-2)
    assert torch.equal(ops().skinny_gemm(x, w, ops().EPI_F32), ops().skinny_gemm(x, w, ops().EPI_F32))


def test_skinny_gemm_refuses_what_it_cannot_take(gen):
    x, w = rand((4, 80), torch.bfloat16, gen), rand((32, 80), torch.bfloat16, gen)
    with pytest.raises(RuntimeError, match="multiple of 64"):
        ops().skinny_gemm(x, w)
    with pytest.raises(RuntimeError, match="1 to 16"):
        ops().skinny_gemm(rand((17, 64), torch.bfloat16, gen), rand((32, 64), torch.bfloat16, gen))
    torch.testing.assert_close(ops().linear(x, w).float(), x.float() @ w.float().T, atol=2e-2, rtol=2e-2)   # library product


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(1, 160), (9, 112), (33, 18944)])
def test_swiglu(dtype, T, I, gen):
    x = rand((T, 2 * I), dtype, gen, 2.0)
    torch.testing.assert_close(ops().swiglu(x, I).float(), kernel_refs.swiglu(x, I).float(), **bar(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rot,ps", [(4, 2, 16, 16, 16), (6, 1, 32, 32, 32), (5, 5, 48, 32, 16),
                                             (28, 4, 128, 128, 16), (3, 3, 64, 0, 8)])
def test_qkv_bias_rope_cache(dtype, nq, nkv, d, rot, ps, gen):
    T, pages = 19, 12
    qkv = rand((T, (nq + 2 * nkv) * d), dtype, gen)
    bias = torch.randn((nq + 2 * nkv) * d, device=DEV, generator=gen) * 0.1
    # large positions too: the angle is position * inv_freq in float32
    positions = torch.tensor([0, 1, 2, 15, 16, 17, 255, 4095, 32767, 100000, 131071] + list(range(40, 48)),
                             device=DEV, dtype=torch.int32)
    inv_freq = None
    if rot:
        inv_freq = (1.0 / 1e6 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot)).to(DEV)
    slots = torch.randperm(pages * ps, device=DEV, generator=gen)[:T].to(torch.int32)
    slots[3] = -1                                       # a padded token writes nothing
    caches = [torch.zeros(2, pages, nkv, ps, d, device=DEV, dtype=dtype) for _ in range(2)]
    a, b = qkv.clone(), qkv.clone()
    ops().qkv_bias_rope_cache(a, bias, positions, inv_freq, rot, slots, caches[0][0], caches[0][1], nq, nkv, d, ps)
    kernel_refs.qkv_bias_rope_cache(b, bias, positions, inv_freq, rot, slots, caches[1][0], caches[1][1], nq, nkv, d, ps)
    # sin/cos of a large float32 angle: both sides take the same float32 angle, so they agree to rounding
    torch.testing.assert_close(a.float(), b.float(), **bar(dtype))
    torch.testing.assert_close(caches[0].float(), caches[1].float(), **bar(dtype))
    # without a slot mapping nothing is written
    c = qkv.clone()
    untouched = torch.zeros_like(caches[0])
    ops().qkv_bias_rope_cache(c, bias, positions, inv_freq, rot, None, untouched[0], untouched[1], nq, nkv, d, ps)
    assert float(untouched.abs().max()) == 0.0
    torch.testing.assert_close(c.float(), b.float(), **bar(dtype))
    ops().check_status(DEV)


@pytest.mark.parametrize("M", [1, 5, 8])
@pytest.mark.parametrize("nq,nkv,d,ps,K", [(4, 2, 16, 16, 64), (6, 1, 32, 32, 192), (6, 3, 48, 16, 128), (28, 4, 128, 16, 3584)])
def test_fused_qkv_projection(M, nq, nkv, d, ps, K, gen):
    """Decode-sized projection with bias, rotation and cache write in the GEMM's epilogue, against
    the unfused reference."""
    pages = 12
    h = rand((M, K), torch.bfloat16, gen)
    w = rand(((nq + 2 * nkv) * d, K), torch.bfloat16, gen, 0.05)
    bias = torch.randn((nq + 2 * nkv) * d, device=DEV, generator=gen) * 0.1
    positions = torch.tensor([0, 1, 17, 255, 4095, 32767, 100000, 131071][:M], device=DEV, dtype=torch.int32)
    inv_freq = (1.0 / 1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d)).to(DEV)
    slots = torch.randperm(pages * ps, device=DEV, generator=gen)[:M].to(torch.int32)
    if M > 2:
        slots[2] = -1
    caches = [torch.zeros(2, pages, nkv, ps, d, device=DEV, dtype=torch.bfloat16) for _ in range(2)]
    got = ops().qkv_projection(h, w, bias, positions, inv_freq, d, slots, caches[0][0], caches[0][1], nq, nkv, d, ps)
    want = kernel_refs.qkv_projection(h, w, bias, positions, inv_freq, d, slots, caches[1][0], caches[1][1], nq, nkv, d, ps)
    # one rounding on both sides: at most one step of bfloat16 where the float32 sums fall either side of a tie
    torch.testing.assert_close(got.float(), want.float(), atol=2e-3, rtol=8e-3)
    torch.testing.assert_close(caches[0].float(), caches[1].float(), atol=2e-3, rtol=8e-3)
    untouched = torch.zeros_like(caches[0])
    ops().qkv_projection(h, w, None, positions, inv_freq, d, None, untouched[0], untouched[1], nq, nkv, d, ps)
    assert float(untouched.abs().max()) == 0.0
    ops().check_status(DEV)


@pytest.mark.parametrize("nq,nkv,d,ps,K", [(6, 3, 48, 16, 128), (28, 4, 128, 16, 3584)])
def test_a_token_gets_the_same_keys_whichever_projection_path_its_step_takes(nq, nkv, d, ps, K, gen):
    """Five tokens through the fused decode kernel (one launch: product, bias, rotation, cache write) and the same
    five among twelve through the library product kept in float32 and the bias/rotation kernel: both round once,
    after bias and rotation, so nearly every element is the same bfloat16 number and none is further than one step."""
    pages, M, more = 12, 5, 12
    h = rand((more, K), torch.bfloat16, gen)
    w = rand(((nq + 2 * nkv) * d, K), torch.bfloat16, gen, 0.05)
    bias = torch.randn((nq + 2 * nkv) * d, device=DEV, generator=gen) * 0.1
    positions = torch.tensor([0, 1, 17, 255, 4095, 32767, 100000, 131071, 5, 6, 7, 8], device=DEV, dtype=torch.int32)
    inv_freq = (1.0 / 1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d)).to(DEV)
    slots = torch.randperm(pages * ps, device=DEV, generator=gen)[:more].to(torch.int32)
    caches = [torch.zeros(2, pages, nkv, ps, d, device=DEV, dtype=torch.bfloat16) for _ in range(2)]
    few = ops().qkv_projection(h[:M].contiguous(), w, bias, positions[:M].contiguous(), inv_freq, d, slots[:M].contiguous(),
                               caches[0][0], caches[0][1], nq, nkv, d, ps)
    many = ops().qkv_projection(h, w, bias, positions, inv_freq, d, slots, caches[1][0], caches[1][1], nq, nkv, d, ps)
    torch.testing.assert_close(few.float(), many[:M].float(), atol=2e-3, rtol=8e-3)
    same = (few == many[:M]).float().mean().item()
    assert same > 0.98, f"only {same:.3f} of the elements agree exactly: one path rounds twice"
    for slot in slots[:M].tolist():
        page, off = slot // ps, slot % ps
        torch.testing.assert_close(caches[0][:, page, :, off].float(), caches[1][:, page, :, off].float(), atol=2e-3, rtol=8e-3)
    ops().check_status(DEV)


def _attention_case(dtype, nq, nkv, d, ps, chunks, window, gen, order="scattered", boost=None, splits=None,
                    simt=False, tcgen05=False, ramp=None, cluster=False):
    """chunks: [(start, n)] per request.  Fills the cache for positions < start + n."""
    R = len(chunks)
    lens = [s + n for s, n in chunks]
    pages_per = [-(-l // ps) for l in lens]
    total_pages = sum(pages_per) + 3
    perm = list(range(total_pages))
    if order == "scattered":
        random.Random(0).shuffle(perm)
    elif order == "reversed":
        perm = perm[::-1]
    kc = rand((total_pages, nkv, ps, d), dtype, gen)
    vc = rand((total_pages, nkv, ps, d), dtype, gen)
    bt = torch.full((R, max(pages_per)), -1, dtype=torch.int32)
    k = 0
    for r, n in enumerate(pages_per):
        bt[r, :n] = torch.tensor(perm[k:k + n], dtype=torch.int32)
        k += n
    T = sum(n for _, n in chunks)
    qkv = rand((T, (nq + 2 * nkv) * d), dtype, gen)
    if boost is not None:
        # make one far key decisive for the last query of request 0: align the key with the query
        r0_len = lens[0]
        t_far = boost
        page, off = int(bt[0, t_far // ps]), t_far % ps
        last_row = chunks[0][1] - 1
        ratio = nq // nkv
        for g in range(nkv):
            qvec = qkv[last_row, g * ratio * d:(g * ratio + 1) * d].clone()
            for h in range(g * ratio, (g + 1) * ratio):          # the heads of a group share the query
                qkv[last_row, h * d:(h + 1) * d] = qvec
            kc[page, g, off] = (qvec.float() * 4.0).to(dtype)
        vc[page, :, off] = 10.0
        assert t_far < r0_len
    if ramp is not None:
        # every key along dimension 0 grows with its position and every query has a positive component there:
        # each later key beats the earlier ones by a wide margin
        qkv[:, :nq * d].view(T, nq, d)[:, :, 0] = 4.0
        for r, n in enumerate(pages_per):
            for t in range(lens[r]):
                kc[int(bt[r, t // ps]), :, t % ps, 0] = ramp * t
    cu = [0]
    for _, n in chunks:
        cu.append(cu[-1] + n)
    ctx = types.SimpleNamespace(
        max_q_len=max(n for _, n in chunks), max_ctx_len=max(lens),
        host_starts=[s for s, _ in chunks], host_lengths=[n for _, n in chunks],
        cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
        q_start=torch.tensor([s for s, _ in chunks], dtype=torch.int32, device=DEV),
        token_request=torch.tensor([r for r, (_, n) in enumerate(chunks) for _ in range(n)], dtype=torch.int32, device=DEV))
    bt = bt.to(DEV)
    scale = 1.0 / math.sqrt(d)
    want = kernel_refs.paged_attention(qkv, kc, vc, bt, ctx, nq, nkv, d, ps, scale, window)
    if splits is not None and cluster:   # the same splits as one thread-block cluster per (request, key/value head)
        got = ops().paged_decode_cluster(qkv, qkv.stride(0), kc, vc, bt, ctx.cu_q, ctx.q_start, R, nq, nkv, d, ps, scale,
                                         window, splits)
    elif splits is not None:          # the split-KV decode kernel, asked for by name
        got = ops().paged_decode_mma(qkv, qkv.stride(0), kc, vc, bt, ctx.cu_q, ctx.q_start, R, nq, nkv, d, ps, scale,
                                     window, splits)
    elif tcgen05:                     # the tcgen05 prefill kernel, asked for by name; an integer > 1 splits the keys
        got = ops().paged_prefill_tcgen05(qkv, qkv.stride(0), kc, vc, bt, ctx.cu_q, ctx.q_start, T, R, ctx.max_q_len, nq,
                                          nkv, d, ps, scale, window, splits=int(tcgen05))
    elif simt:
        got = ops().paged_attention_simt(qkv, qkv.stride(0), kc, vc, bt, ctx.cu_q, ctx.q_start, ctx.token_request, T,
                                         nq, nkv, d, ps, scale, window)
    else:
        got = ops().paged_attention(qkv, kc, vc, bt, ctx, nq, nkv, d, ps, scale, window)
    return got, want, chunks


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,ps", [(4, 2, 16, 16), (6, 1, 32, 32), (6, 3, 48, 16), (28, 4, 128, 16),
                                         (2, 2, 256, 8), (5, 1, 80, 16)])
def test_paged_attention_shapes(dtype, nq, nkv, d, ps, gen):
    # lengths around page and 32-key block edges; decode tokens beside portions
    chunks = [(0, 1), (0, 17), (15, 2), (31, 1), (32, 1), (33, 5), (0, 64), (129, 1), (100, 30)]
    got, want, _ = _attention_case(dtype, nq, nkv, d, ps, chunks, 0, gen)
    torch.testing.assert_close(got.float(), want.float(), **bar(dtype))
    ops().check_status(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("order", ["reversed", "scattered", "ordered"])
def test_paged_attention_block_tables(dtype, order, gen):
    got, want, _ = _attention_case(dtype, 6, 2, 32, 16, [(512, 1), (0, 129), (250, 7)], 0, gen, order=order)
    torch.testing.assert_close(got.float(), want.float(), **bar(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 5, 16, 33, 100])
def test_paged_attention_window(dtype, window, gen):
    got, want, _ = _attention_case(dtype, 4, 2, 32, 16, [(200, 1), (0, 70), (90, 12)], window, gen)
    torch.testing.assert_close(got.float(), want.float(), **bar(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 15, 16, 17, 333, 700])
def test_paged_attention_finds_a_far_key(dtype, far, gen):
    # one key among 800 is made decisive; the output of the last query must be its value (10)
    got, want, chunks = _attention_case(dtype, 4, 2, 64, 16, [(799, 1), (3, 2)], 0, gen, boost=far)
    torch.testing.assert_close(got.float(), want.float(), **bar(dtype))
    assert float((got[0].float() - 10.0).abs().max()) < 0.5


@pytest.mark.parametrize("splits", [1, 2, 3, 7, 40])
@pytest.mark.parametrize("nq,nkv,d,ps", [(4, 2, 16, 16), (6, 1, 32, 32), (6, 3, 48, 16), (28, 4, 128, 16), (16, 1, 64, 8),
                                         (2, 2, 256, 16), (5, 5, 80, 64)])
def test_split_kv_decode_kernel(nq, nkv, d, ps, splits, gen):
    # one token per request at contexts around tile (32), page and split edges
    chunks = [(p, 1) for p in (0, 1, 15, 16, 31, 32, 33, 63, 64, 100, 255, 256, 700, 1023)]
    got, want, _ = _attention_case(torch.bfloat16, nq, nkv, d, ps, chunks, 0, gen, splits=splits)
    torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    ops().check_status(DEV)


@pytest.mark.parametrize("splits", [1, 2, 3, 7, 8, 9, 14, 16])
@pytest.mark.parametrize("nq,nkv,d,ps", [(4, 2, 16, 16), (6, 1, 32, 32), (6, 3, 48, 16), (28, 4, 128, 16), (16, 1, 64, 8),
                                         (2, 2, 256, 16), (5, 5, 80, 64)])
def test_cluster_decode_kernel(nq, nkv, d, ps, splits, gen):
    """The splits of a (request, key/value head) as one thread-block cluster, merged through distributed shared
    memory: clusters of up to 8 blocks (portable) and up to 16; contexts so short that some splits have no key."""
    chunks = [(p, 1) for p in (0, 1, 15, 16, 31, 32, 33, 63, 64, 100, 255, 256, 700, 1023)]
    got, want, _ = _attention_case(torch.bfloat16, nq, nkv, d, ps, chunks, 0, gen, splits=splits, cluster=True)
    torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    ops().check_status(DEV)


def test_cluster_decode_kernel_window_far_key_and_limits(gen):
    chunks = [(p, 1) for p in (0, 5, 40, 64, 300, 999)]
    for window in (1, 32, 33, 200):
        got, want, _ = _attention_case(torch.bfloat16, 8, 2, 64, 16, chunks, window, gen, splits=4, cluster=True)
        torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    for far in (0, 17, 333, 798):
        got, want, _ = _attention_case(torch.bfloat16, 4, 2, 64, 16, [(799, 1), (3, 1)], 0, gen, boost=far, splits=5, cluster=True)
        torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
        assert float((got[0].float() - 10.0).abs().max()) < 0.5
    # splits whose sums differ by hundreds of powers of two are weighed against each other
    got, want, _ = _attention_case(torch.bfloat16, 4, 2, 64, 16, [(900, 1), (37, 1)], 0, gen, splits=7, cluster=True, ramp=0.6)
    torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    with pytest.raises(RuntimeError, match="cluster"):
        _attention_case(torch.bfloat16, 4, 2, 64, 16, [(300, 1)], 0, gen, splits=17, cluster=True)
    assert ops().decode_cluster_splits(14, 2048) == 14 and ops().decode_cluster_splits(32, 2048) == 16
    # cut down to what fits the device in one round, as long as eight splits remain
    fits = {16: 20, 15: 24, 14: 35, 13: 36, 9: 60, 8: 74, 3: 190, 2: 296}
    resident = lambda s: fits.get(s, fits[min(k for k in fits if k >= s)])
    assert ops().decode_cluster_splits(21, 4096, 32, resident) == 14
    assert ops().decode_cluster_splits(13, 4096, 64, resident) == 8
    assert ops().decode_cluster_splits(3, 4096, 256, resident) == 3 and ops().decode_cluster_splits(16, 4096, 4, resident) == 16
    assert ops().decode_cluster_splits(12, 4096, 32, lambda s: 0) == 0
    real = lambda s: ops().clusters_resident(8, 28, 4, 128, s)
    assert real(2) >= real(8) >= real(16) >= 1
    chosen = ops().decode_cluster_splits(21, 4096, 32, real)
    assert 8 <= chosen <= 16 and real(chosen) >= 32
    assert ops().decode_cluster_splits(27, 32768) == 0 and ops().decode_cluster_splits(1, 10) == 0
    ops().check_status(DEV)


@pytest.mark.parametrize("M", [1, 5, 8])
@pytest.mark.parametrize("N,K,N2", [(3584, 3584, 4608), (1536, 8960, 2 * 8960), (192, 384, 256), (80, 128, 64), (3584, 18944, 512)])
def test_residual_epilogue_begins_the_norm_and_the_next_product_finishes_it(M, N, K, N2, gen):
    """A product that ends a branch adds to the residual stream in its epilogue and leaves the rows times the next
    norm's weight with each tile's share of their sums of squares; the product after it scales its accumulators by
    rsqrt(mean square + eps).  Against: residual += x W^T; h = rmsnorm(residual) * w; h W2^T."""
    eps = 1e-6
    x = rand((M, K), torch.bfloat16, gen)
    w = rand((N, K), torch.bfloat16, gen, 0.02)
    w2 = rand((N2, N), torch.bfloat16, gen, 0.05)
    residual = torch.randn(M, N, device=DEV, generator=gen)
    norm_weight = 1 + 0.1 * torch.randn(N, device=DEV, generator=gen)
    want_residual = residual + x.float() @ w.float().T
    want_h = kernel_refs.add_rmsnorm(want_residual.clone(), None, norm_weight, eps, torch.bfloat16)
    began = ops().linear(x, w, follow=(residual, norm_weight, eps))
    assert isinstance(began, ops().Prenormed) and began.residual is residual
    torch.testing.assert_close(residual, want_residual, atol=1e-3, rtol=1e-4)
    torch.testing.assert_close(began.scaled.float(), (want_residual * norm_weight).to(torch.bfloat16).float(), atol=1e-2, rtol=1e-2)
    torch.testing.assert_close(began.sumsq.sum(0)[:M], want_residual.pow(2).sum(-1), atol=1e-2, rtol=1e-4)
    assert float(began.sumsq.sum(0)[M:].abs().max() if M < 8 else 0.0) == 0.0
    torch.testing.assert_close(began.materialize().float(), want_h.float(), **bar(torch.bfloat16))
    # the consumers: a plain product (float32 and bfloat16 results), gate/up with the activation, and a second branch end
    want = want_h.float() @ w2.float().T
    scale = float(want.abs().max())
    torch.testing.assert_close(ops().linear(began, w2, out_float32=True), want, atol=1e-2 * scale, rtol=2e-2)
    torch.testing.assert_close(ops().linear(began, w2).float(), want, atol=1e-2 * scale, rtol=2e-2)
    got = ops().linear_swiglu(began, w2, N2 // 2)
    torch.testing.assert_close(got.float(), kernel_refs.linear_swiglu(want_h, w2, N2 // 2).float(), atol=1e-2 * scale * scale, rtol=3e-2)
    if N % 64 == 0:
        second = torch.randn(M, N2, device=DEV, generator=gen)
        expect = second + want
        again = ops().linear(began, w2, follow=(second, torch.ones(N2, device=DEV), eps))
        assert isinstance(again, ops().Prenormed)
        torch.testing.assert_close(second, expect, atol=1e-2 * scale, rtol=2e-2)
    ops().check_status(DEV)


def test_fused_qkv_projection_takes_rows_on_their_way_through_a_norm(gen):
    nq, nkv, d, ps, K, M, pages = 28, 4, 128, 16, 3584, 6, 12
    eps = 1e-6
    residual = torch.randn(M, K, device=DEV, generator=gen)
    norm_weight = 1 + 0.1 * torch.randn(K, device=DEV, generator=gen)
    x = rand((M, 256), torch.bfloat16, gen)
    began = ops().linear(x, rand((K, 256), torch.bfloat16, gen, 0.05), follow=(residual, norm_weight, eps))
    h = kernel_refs.add_rmsnorm(residual.clone(), None, norm_weight, eps, torch.bfloat16)
    w = rand(((nq + 2 * nkv) * d, K), torch.bfloat16, gen, 0.05)
    bias = torch.randn((nq + 2 * nkv) * d, device=DEV, generator=gen) * 0.1
    positions = torch.tensor([0, 1, 17, 255, 4095, 32767], device=DEV, dtype=torch.int32)
    inv_freq = (1.0 / 1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d)).to(DEV)
    slots = torch.randperm(pages * ps, device=DEV, generator=gen)[:M].to(torch.int32)
    caches = [torch.zeros(2, pages, nkv, ps, d, device=DEV, dtype=torch.bfloat16) for _ in range(2)]
    got = ops().qkv_projection(began, w, bias, positions, inv_freq, d, slots, caches[0][0], caches[0][1], nq, nkv, d, ps)
    want = kernel_refs.qkv_projection(h, w, bias, positions, inv_freq, d, slots, caches[1][0], caches[1][1], nq, nkv, d, ps)
    torch.testing.assert_close(got.float(), want.float(), atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(caches[0].float(), caches[1].float(), atol=3e-2, rtol=3e-2)
    ops().check_status(DEV)


@pytest.mark.parametrize("window", [1, 31, 32, 33, 200])
def test_split_kv_decode_kernel_window_and_far_key(window, gen):
    chunks = [(p, 1) for p in (0, 5, 40, 64, 300, 999)]
    for splits in (1, 4):
        got, want, _ = _attention_case(torch.bfloat16, 8, 2, 64, 16, chunks, window, gen, splits=splits)
        torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    for far in (0, 17, 333, 798):
        got, want, _ = _attention_case(torch.bfloat16, 4, 2, 64, 16, [(799, 1), (3, 1)], 0, gen, boost=far, splits=5)
        torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
        assert float((got[0].float() - 10.0).abs().max()) < 0.5


@pytest.mark.parametrize("nq,nkv,d,ps", [(2, 2, 64, 16), (28, 4, 128, 16), (6, 3, 128, 24), (5, 1, 64, 8), (16, 1, 128, 32)])
def test_tcgen05_prefill_kernel(nq, nkv, d, ps, gen):
    # portions around the 64-key tile, the 128- and 256-row block edges; short ones beside long ones
    chunks = [(0, 1), (0, 64), (63, 2), (0, 300), (100, 129), (1000, 3), (5, 37), (64, 64)]
    got, want, _ = _attention_case(torch.bfloat16, nq, nkv, d, ps, chunks, 0, gen, tcgen05=True)
    torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    ops().check_status(DEV)


@pytest.mark.parametrize("window", [1, 63, 64, 65, 200])
def test_tcgen05_prefill_kernel_window_and_far_key(window, gen):
    chunks = [(0, 300), (200, 77), (999, 1), (60, 10)]
    got, want, _ = _attention_case(torch.bfloat16, 8, 2, 128, 16, chunks, window, gen, tcgen05=True)
    torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    for far in (0, 63, 64, 333, 700):
        got, want, _ = _attention_case(torch.bfloat16, 4, 2, 64, 16, [(600, 200), (3, 2)], 0, gen, boost=far, tcgen05=True)
        torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
        assert float((got[199].float() - 10.0).abs().max()) < 0.5
    ops().check_status(DEV)


def test_tcgen05_prefill_kernel_long_contexts_go_round_its_rings(gen):
    # dozens of key tiles per block: the four-stage key/value ring and both score buffers are used many times over;
    # a portion far into its context, a long portion from position 0, and one under a window
    got, want, _ = _attention_case(torch.bfloat16, 14, 2, 128, 16, [(2000, 700), (0, 1500)], 0, gen, tcgen05=True)
    torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    got, want, _ = _attention_case(torch.bfloat16, 4, 1, 64, 32, [(3000, 333)], 1000, gen, tcgen05=True)
    torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    ops().check_status(DEV)


def test_tcgen05_prefill_kernel_moves_its_reference_point(gen):
    # scores that grow along the keys by far more than 2^8 make every row rescale its output in tensor memory
    nq, nkv, d, ps, n = 4, 2, 64, 16, 400
    got, want, _ = _attention_case(torch.bfloat16, nq, nkv, d, ps, [(0, n), (37, 200)], 0, gen, tcgen05=True, ramp=0.6)
    torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    with pytest.raises(RuntimeError, match="head size"):
        _attention_case(torch.bfloat16, 4, 2, 32, 16, [(0, 300)], 0, gen, tcgen05=True)


@pytest.mark.parametrize("splits", [2, 3, 8, 32])
def test_tcgen05_prefill_kernel_with_split_keys(splits, gen):
    # the keys of every pair of row tiles shared out over several blocks and merged: splits that get nothing (short
    # contexts), that lie wholly behind a row's position, and a decisive key in the first, a middle and the last split
    chunks = [(0, 1), (1000, 3), (0, 300), (2000, 70), (63, 2), (500, 129)]
    for nq, nkv, d, ps in [(28, 4, 128, 16), (5, 1, 64, 8)]:
        got, want, _ = _attention_case(torch.bfloat16, nq, nkv, d, ps, chunks, 0, gen, tcgen05=splits)
        torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    for far in (0, 63, 64, 1027, 2040, 2100):
        got, want, _ = _attention_case(torch.bfloat16, 4, 2, 64, 16, [(2048, 60), (3, 2)], 0, gen, boost=far, tcgen05=splits)
        torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
        assert float((got[59].float() - 10.0).abs().max()) < 0.5
    for window in (1, 65, 700):
        got, want, _ = _attention_case(torch.bfloat16, 8, 2, 128, 16, [(1500, 40), (10, 5)], window, gen, tcgen05=splits)
        torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    # each split moves its own reference point, and the merge weighs splits whose sums differ by hundreds of powers of two
    got, want, _ = _attention_case(torch.bfloat16, 4, 2, 64, 16, [(900, 100), (37, 200)], 0, gen, tcgen05=splits, ramp=0.6)
    torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    ops().check_status(DEV)
    with pytest.raises(RuntimeError, match="splits"):
        _attention_case(torch.bfloat16, 4, 2, 64, 16, [(0, 300)], 0, gen, tcgen05=33)


@pytest.mark.parametrize("nkv", [1, 2])
def test_one_request_with_few_heads_at_a_very_long_context(nkv, gen):
    """One decoding request, one or two key/value heads, 66,000 keys: a round of the device would be more splits
    than the merge kernel takes; the dispatch asks for the kernel's most, and the far key is still found."""
    assert ops().decode_splits(1, nkv, 66000) == ops().DECODE_MAX_SPLITS == library_max_splits()
    got, want, _ = _attention_case(torch.bfloat16, 2 * nkv, nkv, 64, 16, [(65999, 1)], 0, gen, boost=31)
    torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    assert float(got.float().abs().max()) > 5.0           # the boosted key at position 31 carries the value 10
    ops().check_status(DEV)


def library_max_splits() -> int:
    from flexengine_b200.ops import library
    return int(library.load("bf16").fe_paged_decode_max_splits())


def test_dispatch_takes_the_tcgen05_kernel_for_its_head_sizes(gen):
    assert ops().tcgen05_attention_ok(300, 4, 2, 128) and ops().tcgen05_attention_ok(2, 4, 2, 64)
    assert not ops().tcgen05_attention_ok(4096, 4, 2, 96)
    # very many requests with a few tokens each at short contexts: the lighter blocks of the mma.sync kernel
    ok = ops().tcgen05_attention_ok
    assert not ok(8, 28, 4, 128, [8] * 256, [0] * 256) and not ok(64, 28, 4, 128, [1] * 60 + [64], [200] * 60 + [0])
    assert ok(32, 28, 4, 128, [32] * 64, [0] * 64) and ok(500, 28, 4, 128, [1] * 30 + [500], [2000] * 30 + [0])
    got, want, _ = _attention_case(torch.bfloat16, 8, 2, 128, 16, [(50, 1)] * 100 + [(0, 40)], 0, gen)
    torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    got, want, _ = _attention_case(torch.bfloat16, 4, 2, 128, 16, [(0, 300), (100, 1), (7, 2)], 0, gen)
    torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    # a short portion late in a long context beside decoded tokens: the dispatch splits its keys
    chunks = [(3000, 48), (700, 1), (0, 2)]
    assert ops().prefill_splits([n for _, n in chunks], [s for s, _ in chunks], 14, 2) > 1
    got, want, _ = _attention_case(torch.bfloat16, 14, 2, 128, 16, chunks, 0, gen)
    torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    ops().check_status(DEV)


def test_bfloat16_on_cuda_cores_for_shapes_the_tensor_core_kernels_refuse(gen):
    # 24 query heads on one key/value head is beyond the decode kernel's 16: the dispatch takes another path
    got, want, _ = _attention_case(torch.bfloat16, 24, 1, 32, 16, [(40, 1), (7, 1)], 0, gen)
    torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    got, want, _ = _attention_case(torch.bfloat16, 6, 2, 48, 16, [(40, 1), (0, 37)], 0, gen, simt=True)
    torch.testing.assert_close(got.float(), want.float(), **bar(torch.bfloat16))
    with pytest.raises(RuntimeError, match="up to 16"):
        _attention_case(torch.bfloat16, 24, 1, 32, 16, [(40, 1)], 0, gen, splits=2)


def test_sample_greedy_and_ties():
    logits = torch.randn(5, 301, device=DEV)
    logits[1, 7] = logits[1, 200] = 50.0            # a tie goes to the lowest index
    logits[2, 300] = 60.0
    zeros_f, zeros_i = torch.zeros(5, device=DEV), torch.zeros(5, dtype=torch.int32, device=DEV)
    z64 = torch.zeros(5, dtype=torch.int64, device=DEV)
    got = ops().sample(logits, zeros_f, zeros_i, z64, z64)
    assert got.tolist() == kernel_refs.sample(logits, zeros_f, zeros_i, z64, z64).tolist()
    assert got[1] == 7 and got[2] == 300


@pytest.mark.parametrize("V", [301, 152064])
def test_sample_temperature_top_k(V):
    torch.manual_seed(0)
    R = 24
    logits = torch.randn(R, V, device=DEV) * 3
    logits[5, 10] = logits[5, 20] = logits[5, 30] = 9.0     # ties at the top-k edge
    temperature = torch.tensor([0.8, 1.0, 5.0, 0.3] * 6, device=DEV)
    top_k = torch.tensor([0, 1, 2, 40, 0, 2, 300, V, V + 5, 7, 0, 3] * 2, dtype=torch.int32, device=DEV)
    seed = torch.arange(100, 100 + R, dtype=torch.int64, device=DEV)
    for draw_no in range(6):
        draw = torch.full((R,), draw_no, dtype=torch.int64, device=DEV)
        got = ops().sample(logits, temperature, top_k, seed, draw).cpu()
        again = ops().sample(logits, temperature, top_k, seed, draw).cpu()
        assert torch.equal(got, again)
        for r in range(R):
            x = (logits[r].cpu().double() / float(temperature[r]))
            k = int(top_k[r])
            keep = torch.ones(V, dtype=torch.bool)
            if 0 < k < V:
                keep[:] = False
                keep[torch.sort(x, descending=True, stable=True).indices[:k]] = True
            assert keep[got[r]], f"row {r}: sampled a token outside the top {k}"
            e = torch.where(keep, torch.exp(x - x.max()), torch.zeros_like(x))
            cum = torch.cumsum(e, 0)
            target = kernel_refs.uniform_from(int(seed[r]), draw_no) * float(cum[-1])
            lo = float(cum[got[r] - 1]) if got[r] > 0 else 0.0
            hi = float(cum[got[r]])
            slack = 1e-5 * float(cum[-1])
            assert lo - slack <= target <= hi + slack, f"row {r}: draw outside the token's interval"
    # a row's draw does not depend on its place in the batch
    perm = torch.randperm(R)
    draw = torch.full((R,), 3, dtype=torch.int64, device=DEV)
    base = ops().sample(logits, temperature, top_k, seed, draw).cpu()
    shuffled = ops().sample(logits[perm.to(DEV)].contiguous(), temperature[perm.to(DEV)], top_k[perm.to(DEV)],
                            seed[perm.to(DEV)], draw).cpu()
    assert torch.equal(shuffled, base[perm])


@pytest.mark.parametrize("V", [11, 301, 5000, 152064, 152063])
def test_sample_does_not_depend_on_how_many_blocks_share_a_row(V):
    """A row is sampled by a cluster of one to eight blocks, by how many rows the step has: the token must be the
    same for every size (the vocabulary is cut into the same 256 segments, and their masses are added up in the same
    order), so a request's tokens do not depend on the size of its batch."""
    torch.manual_seed(1)
    R = 12
    logits = torch.randn(R, V, device=DEV) * 2
    logits[3, : min(V, 8)] = 7.0                              # ties at the top-k edge, in the first segment
    logits[4, V - 1] = logits[4, V // 2] = logits[4, 0] = 9.0        # and in segments of different blocks
    logits[6, 5] = float("nan")
    temperature = torch.tensor([0.0, 0.7, 1.0, 0.9, 0.5, 2.0] * 2, device=DEV)
    top_k = torch.tensor([0, 0, 50, 5, 2, V, 1, 3, 0, 40, 7, V - 1], dtype=torch.int32, device=DEV)
    seed = torch.arange(7, 7 + R, dtype=torch.int64, device=DEV)
    for draw_no in range(8):
        draw = torch.full((R,), draw_no, dtype=torch.int64, device=DEV)
        chosen = ops().sample(logits, temperature, top_k, seed, draw).cpu()
        for blocks in (1, 2, 4, 8):
            assert torch.equal(ops().sample(logits, temperature, top_k, seed, draw, blocks=blocks).cpu(), chosen), (blocks, draw_no)
    # and not on the number of rows of the step: a row alone, and among a hundred
    many = logits.repeat(9, 1)
    draw = torch.full((9 * R,), 3, dtype=torch.int64, device=DEV)
    among = ops().sample(many, temperature.repeat(9), top_k.repeat(9), seed.repeat(9), draw).cpu()
    for r in range(R):
        alone = ops().sample(logits[r:r + 1], temperature[r:r + 1], top_k[r:r + 1], seed[r:r + 1], draw[:1]).cpu()
        assert int(alone[0]) == int(among[r]) == int(among[5 * R + r])
    ops().check_status(DEV)


def test_sample_follows_the_distribution():
    V = 11
    logits = torch.tensor([[0.0, 1.0, 2.0, -1.0, 0.5, 3.0, -2.0, 1.5, 0.2, 2.5, -0.5]], device=DEV)
    n = 20000
    rows = logits.expand(n, V).contiguous()
    t = torch.full((n,), 0.7, device=DEV)
    k = torch.full((n,), 5, dtype=torch.int32, device=DEV)
    seed = torch.full((n,), 77, dtype=torch.int64, device=DEV)
    draw = torch.arange(n, dtype=torch.int64, device=DEV)
    got = ops().sample(rows, t, k, seed, draw).cpu()
    import plain_model
    want = plain_model.sampling_distribution(logits[0], 0.7, 5)
    freq = torch.bincount(got.long(), minlength=V).double() / n
    assert float((freq - want.double()).abs().max()) < 0.015
