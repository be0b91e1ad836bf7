// Paged causal grouped-query attention for prefill portions on the fifth-generation tensor cores.
//
// Math as the reference's block-wise path (inference/attention/paged.py:50-70): scores
// q.k / sqrt(d), key t visible to the query at position p iff t <= p (and t > p - window when
// window > 0), running maximum / sum / output in float (online softmax), query head h reads
// key/value head h / (nq / nkv).
//
// A block takes 256 rows of one (request, key/value head) as two tiles of 128: row m is the pair
// (query m / G, head m % G of the group), so the group shares every key it loads.  Keys are walked
// in tiles of 64 aligned to position 0.  Per key tile j and row tile i:
//   S_i(j) = Q_i K^T  tcgen05.mma 128 x 64 x d, Q and K in shared memory (K-major, 128-byte
//                     swizzle), into one of two score buffers of the row tile in tensor memory
//   softmax           warps 4i..4i+3, one thread per row: the 64 scores into registers with
//                     tcgen05.ld, mask, running maximum and sum in float, P = exp2(...) as
//                     bfloat16 written over the scores in tensor memory with tcgen05.st
//   O_i += P V        tcgen05.mma 128 x d x 64, P from tensor memory, V from shared memory as it
//                     lies in the cache (one row per key: MN-major operand), accumulated in tensor
//                     memory over all key tiles
// The scores run two key tiles ahead of the softmax (S_i(j+2) is issued right after P_i(j) V,
// into the buffer that P_i(j) leaves), so the softmax threads rarely wait and the tensor cores
// fill in between.  The reference point of the exponentials moves only when a row's maximum has
// grown by more than 2^8; the sum and O_i are then rescaled in place (after the last P V of the
// row tile has completed), which is rare after the first tiles, so O_i stays in tensor memory
// until the end.
// Warps 8..11 gather keys and values from the pages with 16-byte asynchronous copies into a
// four-stage ring; lane 0 of warp 12 + i issues the products of row tile i.
//
// Every wait on an mbarrier is bounded, and ends early once any thread of the block has given up;
// the block then records it in the status word, leaves its loops and frees its tensor memory.
#include <math_constants.h>

#include "common.cuh"

using namespace fe;

namespace {

constexpr int ROWS = 128;        // rows of a row tile = UMMA M; a block takes two
constexpr int KEYS = 64;         // keys per tile
constexpr int Q_BLOCK = ROWS * 128;      // bytes of one [128 rows x 64 elements] swizzled block of Q
constexpr int KV_BLOCK = KEYS * 128;     // bytes of one [64 keys x 64 elements] swizzled block of K or V
constexpr int KV_STAGES = 4;
constexpr int THREADS = 448;     // warps 0..7 softmax (two row tiles), 8..11 loaders, 12 + i issues the products of row tile i
constexpr int TMEM_COLS = 512;   // score buffer b of row tile i at column 64 (2 i + b), O_i at column 256 + 128 i
constexpr long long WAIT_LIMIT = 2000000000LL;
constexpr float RESCALE_STEP = 8.f;      // log2 of the growth of a row's maximum that moves its reference point

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
// false when the wait ran out or another thread of the block has given up; sets the flag itself then
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* give_up) {
    if (mbar_test(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_test(bar, parity)) {
        if (*give_up) return false;
        if (clock64() - t0 > WAIT_LIMIT) {
            *give_up = 1;
            return false;
        }
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
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_but() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
__device__ __forceinline__ void loader_barrier() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }

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
// D[tmem] (+)= A[smem] B[smem]
__device__ __forceinline__ void umma_ss(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                        unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] B[smem]: A lies row per lane, two bfloat16 per 32-bit column
__device__ __forceinline__ void umma_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long bdesc, unsigned idesc,
                                        unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
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
// Four loads of 32 columns in flight at once: issue all, then one wait; the empty statements tie the
// registers to the wait so that nothing reads them before it.
__device__ __forceinline__ void tmem_issue_load32(unsigned taddr, unsigned* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tie32(unsigned* r) {
    asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                      "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
                      "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                      "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]) :: "memory");
}
__device__ __forceinline__ void tmem_store32(unsigned taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
        ::"r"(taddr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]), "f"(v[8]),
          "f"(v[9]), "f"(v[10]), "f"(v[11]), "f"(v[12]), "f"(v[13]), "f"(v[14]), "f"(v[15]), "f"(v[16]), "f"(v[17]),
          "f"(v[18]), "f"(v[19]), "f"(v[20]), "f"(v[21]), "f"(v[22]), "f"(v[23]), "f"(v[24]), "f"(v[25]), "f"(v[26]),
          "f"(v[27]), "f"(v[28]), "f"(v[29]), "f"(v[30]), "f"(v[31])
        : "memory");
}
__device__ __forceinline__ void tmem_store16(unsigned taddr, const unsigned* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// Byte offset of 16-byte chunk ``c`` (0 .. D/8 - 1) of row ``r`` in a tile made of [rows x 64] swizzled blocks.
__device__ __forceinline__ int swizzled(int r, int c, int block_bytes) {
    return (c >> 3) * block_bytes + r * 128 + (((c & 7) ^ (r & 7)) << 4);
}

// The softmax of one row over a key tile, the 64 scores in registers.  MASKED: the tile crosses
// the causal edge or the window's edge for some row of the warp; ``hi`` and ``lo`` are then this
// row's last and first visible key relative to the tile.
__device__ __forceinline__ float max3(float a, float b, float c) {
    float m;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(m) : "f"(a), "f"(b), "f"(c));
    return m;
}
template <bool MASKED>
__device__ __forceinline__ float row_max(const unsigned* r, int hi, int lo) {
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, m2 = -CUDART_INF_F, m3 = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < KEYS; i += 8) {
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            v[e] = __uint_as_float(r[i + e]);
            if (MASKED && (i + e > hi || i + e < lo)) v[e] = -CUDART_INF_F;
        }
        m0 = max3(m0, v[0], v[1]), m1 = max3(m1, v[2], v[3]), m2 = max3(m2, v[4], v[5]), m3 = max3(m3, v[6], v[7]);
    }
    return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}
// P = 2^(s scale - ref) as bfloat16 pairs over the scores' own columns (32 of the 64); returns the row's sum.
// The multiply-adds and the sums run two floats per instruction.
template <bool MASKED>
__device__ __forceinline__ float row_exp(const unsigned* r, unsigned p_addr, int hi, int lo, float scale_log2, float ref) {
    float2 sum = make_float2(0.f, 0.f);
    const float2 scale2 = make_float2(scale_log2, scale_log2), ref2 = make_float2(-ref, -ref);
#pragma unroll
    for (int c = 0; c < KEYS; c += 32) {
        unsigned packed[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int k = c + 2 * i;
            const float2 t = __ffma2_rn(make_float2(__uint_as_float(r[k]), __uint_as_float(r[k + 1])), scale2, ref2);
            float2 e = make_float2(ex2(t.x), ex2(t.y));
            if (MASKED) {
                if (k > hi || k < lo) e.x = 0.f;
                if (k + 1 > hi || k + 1 < lo) e.y = 0.f;
            }
            sum = __fadd2_rn(sum, e);
            const __nv_bfloat162 pair = __floats2bfloat162_rn(e.x, e.y);
            packed[i] = *reinterpret_cast<const unsigned*>(&pair);
        }
        tmem_store16(p_addr + (c >> 1), packed);
    }
    return sum.x + sum.y;
}

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
paged_prefill_tcgen05_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out, long long out_stride,
                             const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                             const int* __restrict__ block_table, int bt_stride, const int* __restrict__ cu_q,
                             const int* __restrict__ q_start, int nq, int nkv, int ps, int num_pages, float scale_log2,
                             int window, int splits, float* __restrict__ part_o, float* __restrict__ part_lse,
                             int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long kv_full[KV_STAGES], kv_empty[KV_STAGES], s_ready[2][2], p_ready[2][2], pv_done[2], o_final[2];
    __shared__ long long offs[2][KEYS];
    __shared__ unsigned tmem_holder;
    __shared__ volatile int give_up;
    constexpr int DB = D / 64;                       // 64-element blocks per row
    constexpr int Q_BYTES = DB * Q_BLOCK;            // one row tile of Q
    constexpr int KV_BYTES = DB * KV_BLOCK;          // one key tile of K or of V
    constexpr unsigned FULL = 0xffffffffu;
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* q_s = smem;                       // row tile i at q_s + i * Q_BYTES
    unsigned char* kv_s = q_s + 2 * Q_BYTES;         // stage s: K at kv_s + s * 2 * KV_BYTES, V after it

    griddep_wait();
    griddep_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.y, r = blockIdx.z;
    const int G = nq / nkv;
    const int tok0 = cu_q[r], n_q = cu_q[r + 1] - tok0;
    const int rows = n_q * G;
    // blockIdx.x = (pair of row tiles, split of its keys); the rows with the most keys first
    const int split = blockIdx.x % splits;
    const int m_pair = (gridDim.x / splits - 1 - blockIdx.x / splits) * 2 * ROWS;
    if (m_pair >= rows) return;
    const bool two = m_pair + ROWS < rows;                          // else the second row tile is empty and left out
    const int start = q_start[r];
    // keys this block needs: from the window edge of its first query to its last query
    const int qi_first = m_pair / G, qi_last = min(n_q - 1, (m_pair + (two ? 2 : 1) * ROWS - 1) / G);
    const int hi = start + qi_last;
    const int lo = window > 0 ? max(0, start + qi_first - window + 1) : 0;
    // this block's share of the key tiles; with one split, all of them
    const int all_tiles = hi / KEYS - lo / KEYS + 1, per_split = (all_tiles + splits - 1) / splits;
    const int t_begin = lo / KEYS + split * per_split, n_tiles = min(per_split, all_tiles - split * per_split);
    if (n_tiles <= 0) {
        // nothing left for this split: its rows say so, and the merge reads nothing more of them
        const int m = m_pair + tid;
        if (tid < 2 * ROWS && m < rows)
            part_lse[((size_t)(tok0 + m / G) * nq + kvh * G + m % G) * splits + split] = -CUDART_INF_F;
        return;
    }

    if (tid == 0) {
        for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&kv_full[s], 128); mbar_init(&kv_empty[s], two ? 2 : 1); }
        for (int i = 0; i < 2; ++i) {
            for (int b = 0; b < 2; ++b) { mbar_init(&s_ready[i][b], 1); mbar_init(&p_ready[i][b], 128); }
            mbar_init(&pv_done[i], 1);
            mbar_init(&o_final[i], 1);
        }
        give_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 12) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_holder)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }

    // softmax threads: row tile ``ti``, row ``tid & 127`` of it
    const int ti = warp >> 2;
    const bool softmax_thread = warp < 8 && (ti == 0 || two);
    const int m = m_pair + ti * ROWS + (tid & 127);
    const bool valid = softmax_thread && m < rows;
    const int qi = valid ? m / G : 0, head = kvh * G + (valid ? m % G : 0);
    const int pos = valid ? start + qi : -1;
    const int row_lo = window > 0 ? max(0, pos - window + 1) : 0;
    // where this thread's row starts in q and in out (in elements); other lanes fetch it by shuffle
    const long long q_off = valid ? (long long)(tok0 + qi) * q_stride + (long long)head * D : -1;
    const long long out_off = valid ? (long long)(tok0 + qi) * out_stride + (long long)head * D : -1;
    constexpr int CPR = D / 8;                       // 16-byte chunks per row
    constexpr int RPI = 32 / CPR;                    // rows a warp moves per instruction: a row's chunks side by side
    if (softmax_thread) {
        // the warp's 32 query rows into shared memory, swizzled like a TMA tile (zeros for padding rows)
        unsigned char* dst = q_s + ti * Q_BYTES;
        const int c = lane % CPR;
#pragma unroll
        for (int k = 0; k < CPR; ++k) {
            const int row_in_warp = k * RPI + lane / CPR;
            const long long from = __shfl_sync(FULL, q_off, row_in_warp);
            cp_async16(dst + swizzled((warp & 3) * 32 + row_in_warp, c, Q_BLOCK), q + (from >= 0 ? from + c * 8 : 0), from >= 0 ? 16 : 0);
        }
        cp_async_wait_all();
        fence_proxy_async();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = tmem_holder;

    if (warp >= 8 && warp < 12) {
        // ---- loaders: the first 64 look up one key of the tile each, then all copy ----
        const int lt = tid - 256;
        const int ps_shift = (ps & (ps - 1)) == 0 ? __ffs(ps) - 1 : -1;
        constexpr int ROW_STEP = 128 / CPR;                        // 8 (head size 128) or 16 (head size 64) rows per pass
        const int chunk = lt % CPR, row0 = lt / CPR, smem_off0 = swizzled(row0, chunk, KV_BLOCK);
        // A tile is handed over LOADS_AHEAD iterations after its copies were started, before the wait for the next free
        // stage: two tiles are on their way from memory at a time (a cold miss takes about as long as a tile's softmax),
        // and tile t is handed over once the products of tile t - 3 are done, a full tile before its scores are wanted.
        constexpr int LOADS_AHEAD = 2;
        for (int j = 0; j < n_tiles + LOADS_AHEAD; ++j) {
            if (j >= LOADS_AHEAD) {
                cp_async_wait_but<LOADS_AHEAD - 1>();              // tile j - LOADS_AHEAD has arrived
                fence_proxy_async();
                mbar_arrive(&kv_full[(j - LOADS_AHEAD) % KV_STAGES]);
            }
            if (j < n_tiles) {
                const int s = j % KV_STAGES;
                mbar_wait(&kv_empty[s], ((j / KV_STAGES) & 1) ^ 1, &give_up);     // free from the start
                long long* tile_offs = offs[j & 1];
                if (lt < KEYS) {
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
                    tile_offs[lt] = off;
                }
                loader_barrier();                                  // the other buffer of offs is read by no one by now
                if (give_up) break;                                // the same for all loaders after the barrier
                unsigned char* k_s = kv_s + s * 2 * KV_BYTES;
                unsigned char* v_s = k_s + KV_BYTES;
                // this thread's chunk of a row is always the same; its rows are ROW_STEP apart, which keeps row & 7
#pragma unroll
                for (int k = 0; k < KEYS / ROW_STEP; ++k) {
                    const long long ro = tile_offs[row0 + k * ROW_STEP];
                    const bool ok = ro >= 0;
                    const long long from = ok ? ro + chunk * 8 : 0;
                    cp_async16(k_s + smem_off0 + k * ROW_STEP * 128, kc + from, ok ? 16 : 0);     // keys out of range read as zeros
                    cp_async16(v_s + smem_off0 + k * ROW_STEP * 128, vc + from, ok ? 16 : 0);
                }
            }
            cp_async_commit();                                     // one group an iteration, empty ones at the end
        }
        cp_async_wait_all();
    } else if (warp >= 12) {
        // ---- lane 0 of warp 12 + i issues the products of row tile i; the tensor cores keep each thread's order ----
        const int i = warp - 12;
        if (lane == 0 && (i == 0 || two)) {
            constexpr unsigned idesc_s = instr_desc(ROWS, KEYS, false), idesc_pv = instr_desc(ROWS, D, true);
            constexpr unsigned STAGE16 = (2 * KV_BYTES) >> 4;      // a stage's size in descriptor units
            const unsigned long long q_desc = desc_k_major(q_s + i * Q_BYTES), k_desc0 = desc_k_major(kv_s),
                                     v_desc0 = desc_mn_major(kv_s + KV_BYTES, KV_BLOCK);
            const unsigned s_col = tmem_base + 2 * i * 64, o_col = tmem_base + 256 + i * 128;
            auto issue_s = [&](int j) {                            // S_i of key tile j into score buffer j & 1
                const unsigned long long k_desc = k_desc0 + (unsigned)(j % KV_STAGES) * STAGE16;
                const unsigned dst = s_col + (j & 1) * 64;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(dst, q_desc + (((ks >> 2) * Q_BLOCK + (ks & 3) * 32) >> 4),
                            k_desc + (((ks >> 2) * KV_BLOCK + (ks & 3) * 32) >> 4), idesc_s, ks > 0 ? 1u : 0u);
                umma_commit(&s_ready[i][j & 1]);
            };
            bool ok = true;
            for (int j = 0; j < 2 && j < n_tiles && ok; ++j) {
                ok = mbar_wait(&kv_full[j], 0, &give_up);
                tc_fence_after();
                if (ok) issue_s(j);
            }
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j % KV_STAGES;
                ok = mbar_wait(&p_ready[i][j & 1], (j >> 1) & 1, &give_up);
                if (!ok) break;
                tc_fence_after();
                const unsigned long long v_desc = v_desc0 + (unsigned)s * STAGE16;
                const unsigned p_col = s_col + (j & 1) * 64;
#pragma unroll
                for (int ks = 0; ks < KEYS / 16; ++ks)
                    umma_ts(o_col, p_col + ks * 8, v_desc + ks * (2048 >> 4), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                umma_commit(&pv_done[i]);
                umma_commit(&kv_empty[s]);                         // the stage may be refilled once both row tiles have read it
                if (j + 2 < n_tiles) {
                    ok = mbar_wait(&kv_full[(j + 2) % KV_STAGES], ((j + 2) / KV_STAGES) & 1, &give_up);
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(j + 2);                                // runs after P_i V above: it overwrites P_i
                }
            }
            if (ok) umma_commit(&o_final[i]);
        }
        __syncwarp();
    } else if (softmax_thread) {
        // ---- softmax: one thread per row ----
        const unsigned lane_bits = (unsigned)((warp & 3) * 32) << 16;
        const unsigned o_addr = tmem_base + lane_bits + 256 + ti * 128;
        const int pos_min = __reduce_min_sync(FULL, pos), lo_max = __reduce_max_sync(FULL, row_lo);
        float m_ref = -CUDART_INF_F, row_sum = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            ok = __all_sync(FULL, mbar_wait(&s_ready[ti][j & 1], (j >> 1) & 1, &give_up));
            if (!ok) break;
            tc_fence_after();
            const unsigned s_addr = tmem_base + lane_bits + (2 * ti + (j & 1)) * 64;
            unsigned raw[KEYS];
            tmem_issue_load32(s_addr, raw);
            tmem_issue_load32(s_addr + 32, raw + 32);
            tmem_load_wait();
            tie32(raw);
            tie32(raw + 32);
            const int key0 = (t_begin + j) * KEYS;
            const bool unmasked = key0 + KEYS - 1 <= pos_min && key0 >= lo_max;      // for the whole warp
            const int rel_hi = pos - key0, rel_lo = row_lo - key0;
            const float mx = unmasked ? row_max<false>(raw, rel_hi, rel_lo) : row_max<true>(raw, rel_hi, rel_lo);
            const float m_new = fmaxf(m_ref, mx * scale_log2);
            if (__any_sync(FULL, m_new > m_ref + RESCALE_STEP)) {
                // move the reference point to the new maximum: O and the sum were taken against the old one
                const float alpha = m_new == -CUDART_INF_F ? 1.f : ex2(m_ref - m_new);
                if (j > 0) {
                    ok = __all_sync(FULL, mbar_wait(&pv_done[ti], (j - 1) & 1, &give_up));      // O_i is at rest
                    if (!ok) break;
                    tc_fence_after();
                    row_sum *= alpha;
#pragma unroll 1
                    for (int c = 0; c < D; c += 32) {
                        float v[32];
                        tmem_load32(o_addr + c, v);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] *= alpha;
                        tmem_store32(o_addr + c, v);
                    }
                }
                m_ref = m_new;
            }
            const float m_safe = m_ref == -CUDART_INF_F ? 0.f : m_ref;
            row_sum += unmasked ? row_exp<false>(raw, s_addr, rel_hi, rel_lo, scale_log2, m_safe)
                                : row_exp<true>(raw, s_addr, rel_hi, rel_lo, scale_log2, m_safe);
            tmem_store_wait();
            tc_fence_before();
            mbar_arrive(&p_ready[ti][j & 1]);
        }
        if (ok) ok = __all_sync(FULL, mbar_wait(&o_final[ti], 0, &give_up));
        // partial results are staged where keys and values lay: the other row tile must have read its last ones
        if (ok && splits > 1 && two) ok = __all_sync(FULL, mbar_wait(&o_final[ti ^ 1], 0, &give_up));
        if (ok && splits == 1) {
            tc_fence_after();
            const float inv = row_sum > 0.f ? 1.f / row_sum : 0.f;
            // O through shared memory (this row tile's Q is no longer read), so that the warp writes whole rows:
            // thread = row on the way in, a row's 16-byte chunks side by side on the way out
            unsigned char* stage = q_s + ti * Q_BYTES + (warp & 3) * 32 * (2 * D);
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
                float v[32];
                tmem_load32(o_addr + c, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] *= inv;
#pragma unroll
                for (int i = 0; i < 32; i += 8)
                    store8<bf16>(reinterpret_cast<bf16*>(stage + lane * (2 * D) + ((((c + i) >> 3) ^ (lane & 7)) << 4)), v + i);
            }
            __syncwarp();
            const int c = lane % CPR;
#pragma unroll
            for (int k = 0; k < CPR; ++k) {
                const int row_in_warp = k * RPI + lane / CPR;
                const long long to = __shfl_sync(FULL, out_off, row_in_warp);
                const uint4 v = *reinterpret_cast<const uint4*>(stage + row_in_warp * (2 * D) + ((c ^ (row_in_warp & 7)) << 4));
                if (to >= 0) *reinterpret_cast<uint4*>(out + to + c * 8) = v;
            }
        } else if (ok) {
            // this split's share of the row: O / sum in float32 and the logarithm of the sum, for the merge
            tc_fence_after();
            const float inv = row_sum > 0.f ? 1.f / row_sum : 0.f;
            const long long slot = valid ? ((long long)(tok0 + qi) * nq + head) * splits + split : -1;
            if (valid) part_lse[slot] = row_sum > 0.f ? m_ref + log2f(row_sum) : -CUDART_INF_F;
            float* stage = reinterpret_cast<float*>(kv_s + (size_t)ti * (ROWS * 4 * D) + (warp & 3) * (32 * 4 * D));
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
                float v[32];
                tmem_load32(o_addr + c, v);
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4*>(stage + lane * D + ((((c + i) >> 2) ^ (lane & 7)) << 2)) =
                        make_float4(v[i] * inv, v[i + 1] * inv, v[i + 2] * inv, v[i + 3] * inv);
            }
            __syncwarp();
            constexpr int CPR4 = D / 4, RPI4 = 32 / CPR4;       // 16-byte chunks of a float32 row; rows per instruction
            const int c = lane % CPR4;
#pragma unroll 4
            for (int k = 0; k < CPR4; ++k) {
                const int row_in_warp = k * RPI4 + lane / CPR4;
                const long long to = __shfl_sync(FULL, slot, row_in_warp);
                const float4 v = *reinterpret_cast<const float4*>(stage + row_in_warp * D + ((c ^ (row_in_warp & 7)) << 2));
                if (to >= 0) *reinterpret_cast<float4*>(part_o + to * D + c * 4) = v;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (give_up && tid == 0 && status) atomicOr(status, FE_STATUS_WAIT_EXPIRED);
    if (warp == 12) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
}

constexpr float LOG2E = 1.4426950408889634f;
constexpr int MAX_SPLITS = 32;                       // the merge keeps one split's weight per lane

// One warp per (token, head): the splits' shares of the row, weighted by what each split saw of the softmax sum.
template <int D>
__global__ void __launch_bounds__(128)
prefill_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, bf16* __restrict__ out,
                     long long out_stride, int nq, int splits, long long items) {
    griddep_wait();
    griddep_launch_dependents();
    const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= items) return;
    const int lane = threadIdx.x & 31;
    const long long token = item / nq;
    const int head = (int)(item % nq);
    const float lse = lane < splits ? part_lse[item * splits + lane] : -CUDART_INF_F;
    const float mx = warp_max(lse);
    const float w = mx == -CUDART_INF_F ? 0.f : exp2f(lse - mx);       // 0 for a split that saw no key of this row
    const float total = warp_sum(w);
    const float inv = total > 0.f ? 1.f / total : 0.f;
    constexpr int CHUNKS = D / 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
        const float ws = __shfl_sync(0xffffffffu, w, s);
        if (ws == 0.f || lane >= CHUNKS) continue;                     // such a split's share was never written
        const float4 v = *reinterpret_cast<const float4*>(part_o + (item * splits + s) * D + lane * 4);
        acc.x += ws * v.x; acc.y += ws * v.y; acc.z += ws * v.z; acc.w += ws * v.w;
    }
    if (lane < CHUNKS) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
        uint2 packed;
        packed.x = *reinterpret_cast<const unsigned*>(&lo);
        packed.y = *reinterpret_cast<const unsigned*>(&hi);
        *reinterpret_cast<uint2*>(out + token * out_stride + (long long)head * D + lane * 4) = packed;
    }
}

template <int D>
int launch(const void* q, long long q_stride, void* out, long long out_stride, const void* kc, const void* vc,
           const int* block_table, int bt_stride, const int* cu_q, const int* q_start, int requests, int max_q_len, int nq,
           int nkv, int ps, int num_pages, float scale, int window, int splits, float* scratch, long long total_tokens,
           int* status, cudaStream_t stream) {
    const size_t smem = (size_t)(D / 64) * (2 * Q_BLOCK + 2 * KV_STAGES * KV_BLOCK) + 1024;
    const cudaError_t err = cudaFuncSetAttribute(paged_prefill_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FE_REQUIRE(err == cudaSuccess, "paged_prefill_tcgen05: %s", cudaGetErrorString(err));
    const long long rows = (long long)max_q_len * (nq / nkv);
    const long long tiles = (rows + 2 * ROWS - 1) / (2 * ROWS) * splits;
    FE_REQUIRE(tiles <= 2147483647LL && nkv <= 65535 && requests <= 65535, "paged_prefill_tcgen05: grid too large");
    // partial results: [token, head, split, D] float32, then [token, head, split] logarithms of the sums
    float* part_o = splits > 1 ? scratch : nullptr;
    float* part_lse = splits > 1 ? scratch + (size_t)total_tokens * nq * splits * D : nullptr;
    fe::launch(paged_prefill_tcgen05_kernel<D>, dim3((unsigned)tiles, nkv, requests), THREADS, smem, stream, (const bf16*)q, q_stride,
               (bf16*)out, out_stride, (const bf16*)kc, (const bf16*)vc, block_table, bt_stride, cu_q, q_start, nq, nkv, ps,
               num_pages, scale * LOG2E, window, splits, part_o, part_lse, status);
    if (fe_check_launch("paged_prefill_tcgen05")) return 1;
    if (splits > 1) {
        const long long items = total_tokens * nq;
        FE_REQUIRE((items + 3) / 4 <= 2147483647LL, "paged_prefill_tcgen05: merge grid too large");
        fe::launch(prefill_merge_kernel<D>, dim3((unsigned)((items + 3) / 4)), 128, 0, stream, (const float*)part_o,
                   (const float*)part_lse, (bf16*)out, out_stride, nq, splits, items);
        return fe_check_launch("paged_prefill_tcgen05 merge");
    }
    return 0;
}

}  // namespace

// Head sizes 64 and 128, bfloat16.  Other arguments as fe_paged_prefill_mma.  With ``splits`` > 1 (at most 32) the key
// tiles of every pair of row tiles are shared out over that many blocks, whose results a second kernel merges:
// for short portions late in a long context, which alone would keep few blocks busy.  ``scratch`` then holds
// ``fe_paged_prefill_tcgen05_scratch_floats`` floats; ``total_tokens`` is the number of rows of q.
extern "C" long long fe_paged_prefill_tcgen05_scratch_floats(long long total_tokens, int nq, int d, int splits) {
    return splits > 1 ? total_tokens * nq * splits * (d + 1) : 0;
}

extern "C" int fe_paged_prefill_tcgen05(const void* q, long long q_stride, void* out, long long out_stride, const void* kc,
                                        const void* vc, const int* block_table, int bt_stride, const int* cu_q,
                                        const int* q_start, int requests, int max_q_len, int nq, int nkv, int d, int ps,
                                        int num_pages, float scale, int window, int splits, void* scratch,
                                        long long total_tokens, int* status, cudaStream_t stream) {
    FE_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "paged_prefill_tcgen05: bad head counts %d/%d", nq, nkv);
    FE_REQUIRE(d == 64 || d == 128, "paged_prefill_tcgen05: head size %d; this kernel takes 64 and 128", d);
    FE_REQUIRE(ps > 0 && num_pages > 0 && window >= 0, "paged_prefill_tcgen05: bad page size, page count or window");
    FE_REQUIRE(q_stride % 8 == 0 && out_stride % 8 == 0 && (((size_t)q | (size_t)out | (size_t)kc | (size_t)vc) & 15) == 0,
               "paged_prefill_tcgen05: rows must start on 16-byte boundaries");
    FE_REQUIRE(requests >= 0 && max_q_len >= 0, "paged_prefill_tcgen05: bad request count or length");
    FE_REQUIRE(splits >= 1 && splits <= MAX_SPLITS, "paged_prefill_tcgen05: %d splits; 1 to %d", splits, MAX_SPLITS);
    FE_REQUIRE(splits == 1 || (scratch != nullptr && ((size_t)scratch & 15) == 0 && total_tokens > 0),
               "paged_prefill_tcgen05: splits need scratch memory on a 16-byte boundary and the number of tokens");
    if (requests == 0 || max_q_len == 0) return 0;
    if (d == 64)
        return launch<64>(q, q_stride, out, out_stride, kc, vc, block_table, bt_stride, cu_q, q_start, requests, max_q_len, nq, nkv,
                          ps, num_pages, scale, window, splits, (float*)scratch, total_tokens, status, stream);
    return launch<128>(q, q_stride, out, out_stride, kc, vc, block_table, bt_stride, cu_q, q_start, requests, max_q_len, nq, nkv, ps,
                       num_pages, scale, window, splits, (float*)scratch, total_tokens, status, stream);
}
