// Paged causal grouped-query attention for prefill portions on the fifth-generation tensor cores.
//
// Math as the reference's block-wise path (inference/attention/paged.py:50-70): scores
// q.k / sqrt(d), key t visible to the query at position p iff t <= p (and t > p - window when
// window > 0), running maximum / sum / output in float (online softmax), query head h reads
// key/value head h / (nq / nkv).
//
// A block takes 128 rows of one (request, key/value head): row m is the pair (query m / G, head
// m % G of the group), so the group shares every key it loads.  Keys are walked in tiles of 128
// aligned to position 0.  Per tile:
//   S = Q K^T    tcgen05.mma 128 x 128 x d, Q and K in shared memory (K-major, 128-byte swizzle),
//                S in tensor memory
//   softmax      warps 0..3, one thread per row: read S with tcgen05.ld, mask, running maximum and
//                sum in float, P = exp2(...) as bfloat16 into shared memory (the A operand of the
//                next product), rescale the row's output registers
//   PV           tcgen05.mma 128 x d x 128, P (K-major) times V (rows of V as they lie in the
//                cache: MN-major operand), into a second tensor-memory buffer, added to the
//                output registers by the softmax threads
// Warps 4..7 gather the next tile's keys and values from the pages with 16-byte asynchronous
// copies into a two-stage ring while the others compute.  Products are issued by thread 0.
//
// Every wait on an mbarrier is bounded; when one runs out the block records it in the status
// word and all its threads leave their loops together at the next group barrier; tensor memory is
// freed before the block returns.
#include <math_constants.h>

#include "common.cuh"

using namespace fe;

namespace {

constexpr int ROWS = 128;        // rows of a block = UMMA M
constexpr int KEYS = 128;        // keys per tile
constexpr int BLOCK_BYTES = 128 * 128;   // one [128 rows x 64 elements] swizzled block
constexpr int KV_STAGES = 2;
constexpr int THREADS = 256;
constexpr int TMEM_COLS = 256;   // S at column 0, PV at column 128
constexpr long long WAIT_LIMIT = 4000000000LL;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_test(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    if (mbar_test(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_test(bar, parity)) {
        if (clock64() - t0 > WAIT_LIMIT) return false;
    }
    return true;
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void group_barrier(int id) { asm volatile("bar.sync %0, 128;\n" ::"r"(id) : "memory"); }

// Shared-memory descriptors, 128-byte swizzle.  K-major: rows 128 bytes apart, 8-row groups 1024
// bytes apart.  MN-major (V as it lies in the cache: one row per key, 64 head elements = 128 bytes
// of a row per block): 64-element blocks along the head dimension ``lbo`` bytes apart, 8-key groups
// 1024 bytes apart.
__device__ __forceinline__ unsigned long long desc_k_major(const void* p) {
    const unsigned long long addr = smem_u32(p);
    return ((addr & 0x3FFFFull) >> 4) | ((1024ull >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ unsigned long long desc_mn_major(const void* p, unsigned lbo_bytes) {
    const unsigned long long addr = smem_u32(p);
    return ((addr & 0x3FFFFull) >> 4) | ((unsigned long long)(lbo_bytes >> 4) << 16) | ((1024ull >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}
// float accumulator, bfloat16 operands; b_mn: B is MN-major
__host__ __device__ constexpr unsigned instr_desc(int m, int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                     unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_load32(unsigned taddr, float* v) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// Byte offset of 16-byte chunk ``c`` (0 .. D/8 - 1) of row ``r`` in a tile made of [128 x 64] swizzled blocks.
__device__ __forceinline__ int swizzled(int r, int c) {
    return (c >> 3) * BLOCK_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4);
}

template <int D>
__global__ void __launch_bounds__(THREADS)
paged_prefill_tcgen05_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out, long long out_stride,
                             const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                             const int* __restrict__ block_table, int bt_stride, const int* __restrict__ cu_q,
                             const int* __restrict__ q_start, int nq, int nkv, int ps, int num_pages, float scale_log2,
                             int window, int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long kv_full[KV_STAGES], kv_empty[KV_STAGES], mma_bar;
    __shared__ long long offs[KEYS];
    __shared__ unsigned tmem_holder;
    __shared__ volatile int give_up;
    constexpr int DB = D / 64;                       // 64-element blocks per row
    constexpr int TILE_BYTES = DB * BLOCK_BYTES;     // one Q, K or V tile
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* q_s = smem;
    unsigned char* p_s = q_s + TILE_BYTES;           // [128 rows x 128 keys] = two blocks
    unsigned char* kv_s = p_s + 2 * BLOCK_BYTES;     // stage s: K at kv_s + s * 2 * TILE_BYTES, V after it

    griddep_wait();
    griddep_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5;
    const int kvh = blockIdx.y, r = blockIdx.z;
    const int G = nq / nkv;
    const int tok0 = cu_q[r], n_q = cu_q[r + 1] - tok0;
    const int rows = n_q * G;
    const int m_block = (gridDim.x - 1 - blockIdx.x) * ROWS;        // the rows with the most keys first
    if (m_block >= rows) return;
    const int start = q_start[r];
    // keys this block needs: from the window edge of its first query to its last query
    const int qi_first = m_block / G, qi_last = min(n_q - 1, (m_block + ROWS - 1) / G);
    const int hi = start + qi_last;
    const int lo = window > 0 ? max(0, start + qi_first - window + 1) : 0;
    const int t_begin = lo / KEYS, n_tiles = hi / KEYS - t_begin + 1;

    if (tid == 0) {
        for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&kv_full[s], 128); mbar_init(&kv_empty[s], 1); }
        mbar_init(&mma_bar, 1);
        give_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_holder)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }

    // this thread's row (compute threads only)
    const int m = m_block + (tid & 127);
    const bool valid = tid < 128 && m < rows;
    const int qi = valid ? m / G : 0, head = kvh * G + (valid ? m % G : 0);
    const int pos = valid ? start + qi : -1;
    const int row_lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (tid < 128) {
        // the query row into shared memory, swizzled like a TMA tile (zeros for padding rows)
        const bf16* src = q + (size_t)(tok0 + qi) * q_stride + (size_t)head * D;
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (valid) v = *reinterpret_cast<const uint4*>(src + c * 8);
            *reinterpret_cast<uint4*>(q_s + swizzled(tid, c)) = v;
        }
        fence_proxy_async();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = tmem_holder;

    if (tid >= 128) {
        // ---- loaders: thread lt looks up key lt of the tile, then all copy ----
        const int lt = tid - 128;
        const int ps_shift = (ps & (ps - 1)) == 0 ? __ffs(ps) - 1 : -1;
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1;
            if (!mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1)) give_up = 1;      // free from the start
            const int key = (t_begin + j) * KEYS + lt;
            long long off = -1;
            if (key >= lo && key <= hi) {
                const int page = block_table[(size_t)r * bt_stride + (ps_shift >= 0 ? key >> ps_shift : key / ps)];
                if (page < 0 || page >= num_pages) {
                    if (status) atomicOr(status, FE_STATUS_BAD_PAGE);
                } else {
                    const int within = ps_shift >= 0 ? key & (ps - 1) : key % ps;
                    off = (((long long)page * nkv + kvh) * ps + within) * D;
                }
            }
            offs[lt] = off;
            group_barrier(2);
            if (give_up) break;                                    // the same for all loaders after the barrier
            unsigned char* k_s = kv_s + s * 2 * TILE_BYTES;
            unsigned char* v_s = k_s + TILE_BYTES;
            constexpr int CPR = D / 8;
            for (int idx = lt; idx < KEYS * CPR; idx += 128) {
                const int row = idx / CPR, c = idx % CPR;
                const long long ro = offs[row];
                const bool ok = ro >= 0;
                const long long from = ok ? ro + c * 8 : 0;
                const int o = swizzled(row, c);
                cp_async16(k_s + o, kc + from, ok ? 16 : 0);
                cp_async16(v_s + o, vc + from, ok ? 16 : 0);
            }
            cp_async_wait_all();
            fence_proxy_async();
            mbar_arrive(&kv_full[s]);
            group_barrier(2);                                      // offs may be rewritten
        }
    } else {
        // ---- compute: one thread per row; thread 0 also issues the products ----
        float o_acc[D];
#pragma unroll
        for (int i = 0; i < D; ++i) o_acc[i] = 0.f;
        float row_max = -CUDART_INF_F, row_sum = 0.f;
        unsigned mma_phase = 0;
        const unsigned lane_addr = tmem_base + ((unsigned)(warp * 32) << 16);
        constexpr unsigned idesc_s = instr_desc(ROWS, KEYS, false), idesc_pv = instr_desc(ROWS, D, true);
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1;
            const unsigned char* k_s = kv_s + s * 2 * TILE_BYTES;
            const unsigned char* v_s = k_s + TILE_BYTES;
            if (tid == 0) {
                if (!mbar_wait(&kv_full[s], (j >> 1) & 1)) give_up = 1;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma(tmem_base, desc_k_major(q_s + (ks >> 2) * BLOCK_BYTES) + 2 * (ks & 3),
                         desc_k_major(k_s + (ks >> 2) * BLOCK_BYTES) + 2 * (ks & 3), idesc_s, ks > 0 ? 1u : 0u);
                umma_commit(&mma_bar);
            }
            if (!mbar_wait(&mma_bar, mma_phase)) give_up = 1;
            mma_phase ^= 1;
            tc_fence_after();
            // scores of this row: maximum first, then the exponentials (two passes over tensor memory)
            const int key0 = (t_begin + j) * KEYS;
            float mx = -CUDART_INF_F;
#pragma unroll 1
            for (int c = 0; c < KEYS; c += 32) {
                float v[32];
                tmem_load32(lane_addr + c, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int key = key0 + c + i;
                    if (key <= pos && key >= row_lo) mx = fmaxf(mx, v[i]);
                }
            }
            const float m_new = fmaxf(row_max, mx * scale_log2);
            const float m_safe = m_new == -CUDART_INF_F ? 0.f : m_new;
            const float alpha = ex2(row_max - m_safe);             // 2^-inf = 0 at the start
            row_max = m_new;
            float sum = 0.f;
#pragma unroll 1
            for (int c = 0; c < KEYS; c += 32) {
                float v[32];
                tmem_load32(lane_addr + c, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int key = key0 + c + i;
                    const bool vis = key <= pos && key >= row_lo;
                    v[i] = vis ? ex2(fmaf(v[i], scale_log2, -m_safe)) : 0.f;
                    sum += v[i];
                }
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 pk;
                    unsigned* w = reinterpret_cast<unsigned*>(&pk);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __nv_bfloat162 pair = __floats2bfloat162_rn(v[i + 2 * e], v[i + 2 * e + 1]);
                        w[e] = *reinterpret_cast<const unsigned*>(&pair);
                    }
                    *reinterpret_cast<uint4*>(p_s + swizzled(tid, (c + i) >> 3)) = pk;
                }
            }
            row_sum = row_sum * alpha + sum;
            if (alpha != 1.f) {
#pragma unroll
                for (int i = 0; i < D; ++i) o_acc[i] *= alpha;
            }
            fence_proxy_async();
            tc_fence_before();
            group_barrier(1);                                      // P is complete; S has been read by all
            if (give_up) break;                                    // the same for all compute threads after the barrier
            if (tid == 0) {
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < KEYS / 16; ++ks)
                    umma(tmem_base + 128, desc_k_major(p_s + (ks >> 2) * BLOCK_BYTES) + 2 * (ks & 3),
                         desc_mn_major(v_s, BLOCK_BYTES) + ks * (2048 >> 4), idesc_pv, ks > 0 ? 1u : 0u);
                umma_commit(&kv_empty[s]);                         // the stage may be refilled once these have read it
                umma_commit(&mma_bar);
            }
            if (!mbar_wait(&mma_bar, mma_phase)) give_up = 1;
            mma_phase ^= 1;
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < D; c += 32) {
                float v[32];
                tmem_load32(lane_addr + 128 + c, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) o_acc[c + i] += v[i];
            }
            tc_fence_before();
        }
        if (valid && !give_up) {
            const float inv = row_sum > 0.f ? 1.f / row_sum : 0.f;
            bf16* dst = out + (size_t)(tok0 + qi) * out_stride + (size_t)head * D;
#pragma unroll
            for (int c = 0; c < D; c += 8) {
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = o_acc[c + i] * inv;
                store8<bf16>(dst + c, v);
            }
        }
    }
    __syncthreads();
    if (give_up && tid == 0 && status) atomicOr(status, FE_STATUS_WAIT_EXPIRED);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
}

constexpr float LOG2E = 1.4426950408889634f;

template <int D>
int launch(const void* q, long long q_stride, void* out, long long out_stride, const void* kc, const void* vc,
           const int* block_table, int bt_stride, const int* cu_q, const int* q_start, int requests, int max_q_len, int nq,
           int nkv, int ps, int num_pages, float scale, int window, int* status, cudaStream_t stream) {
    const size_t smem = (size_t)(D / 64) * BLOCK_BYTES * (1 + 2 * KV_STAGES) + 2 * BLOCK_BYTES + 1024;
    const cudaError_t err = cudaFuncSetAttribute(paged_prefill_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FE_REQUIRE(err == cudaSuccess, "paged_prefill_tcgen05: %s", cudaGetErrorString(err));
    const long long rows = (long long)max_q_len * (nq / nkv);
    const long long tiles = (rows + ROWS - 1) / ROWS;
    FE_REQUIRE(tiles <= 2147483647LL && nkv <= 65535 && requests <= 65535, "paged_prefill_tcgen05: grid too large");
    fe::launch(paged_prefill_tcgen05_kernel<D>, dim3((unsigned)tiles, nkv, requests), THREADS, smem, stream, (const bf16*)q, q_stride,
               (bf16*)out, out_stride, (const bf16*)kc, (const bf16*)vc, block_table, bt_stride, cu_q, q_start, nq, nkv, ps,
               num_pages, scale * LOG2E, window, status);
    return fe_check_launch("paged_prefill_tcgen05");
}

}  // namespace

// Head sizes 64 and 128, bfloat16.  Other arguments as fe_paged_prefill_mma.
extern "C" int fe_paged_prefill_tcgen05(const void* q, long long q_stride, void* out, long long out_stride, const void* kc,
                                        const void* vc, const int* block_table, int bt_stride, const int* cu_q,
                                        const int* q_start, int requests, int max_q_len, int nq, int nkv, int d, int ps,
                                        int num_pages, float scale, int window, int* status, cudaStream_t stream) {
    FE_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "paged_prefill_tcgen05: bad head counts %d/%d", nq, nkv);
    FE_REQUIRE(d == 64 || d == 128, "paged_prefill_tcgen05: head size %d; this kernel takes 64 and 128", d);
    FE_REQUIRE(ps > 0 && num_pages > 0 && window >= 0, "paged_prefill_tcgen05: bad page size, page count or window");
    FE_REQUIRE(q_stride % 8 == 0 && out_stride % 8 == 0 && (((size_t)q | (size_t)out | (size_t)kc | (size_t)vc) & 15) == 0,
               "paged_prefill_tcgen05: rows must start on 16-byte boundaries");
    FE_REQUIRE(requests >= 0 && max_q_len >= 0, "paged_prefill_tcgen05: bad request count or length");
    if (requests == 0 || max_q_len == 0) return 0;
    if (d == 64)
        return launch<64>(q, q_stride, out, out_stride, kc, vc, block_table, bt_stride, cu_q, q_start, requests, max_q_len, nq, nkv,
                          ps, num_pages, scale, window, status, stream);
    return launch<128>(q, q_stride, out, out_stride, kc, vc, block_table, bt_stride, cu_q, q_start, requests, max_q_len, nq, nkv, ps,
                       num_pages, scale, window, status, stream);
}
