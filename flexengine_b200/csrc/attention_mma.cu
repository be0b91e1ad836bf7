// Paged causal grouped-query attention on tensor cores (bfloat16 inputs, float accumulation,
// float online softmax), for decode and for prefill portions.
//
// Math as the reference's block-wise path (inference/attention/paged.py:50-70): running maximum,
// running sum and value accumulator in float; key t is visible to the query at position p iff
// t <= p (and t > p - window when window > 0); query head h reads key/value head h / (nq / nkv).
//
// Both kernels walk the keys in tiles of 32 aligned to position 0.  A tile's keys and values are
// gathered page by page with 16-byte asynchronous copies (cp.async) into a ring of shared-memory
// stages whose rows are padded by 16 bytes against bank conflicts, read back with ldmatrix and
// multiplied with mma.sync.m16n8k16.  One thread per key looks its page up and leaves the row's
// offset in shared memory; the copies then cost a handful of instructions each.  (Row-sized bulk
// copies of the TMA engine were measured slower here: at 256 bytes a copy the engine, not HBM,
// set the pace.)  The 16 rows of an MMA tile are the query heads of one key/value group
// (decode) or (query, head-of-group) pairs (prefill), so the group shares every key it loads.
//
// decode:  two warps per (split of the keys, key/value head, request).  The splits of one (request, key/value
//          head) are a thread-block cluster that merges its partial results through distributed shared memory
//          (up to 16 splits); with more splits they go to scratch memory and are merged by a second kernel.
// prefill: four warps per (tile of 64 rows, key/value head, request); the warps share the
//          key/value stages.
#include <math_constants.h>

#define FE_PDL_CLASS 2      // FE_PDL_DECODE_ATTENTION
#include "common.cuh"

using namespace fe;

namespace {

constexpr int TK = 32;          // keys per compute tile (one key per lane when gathering)

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, int src_bytes) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
// D[16x8] += A[16x16] (row) * B[16x8] (col), bf16 inputs, float accumulators
__device__ __forceinline__ void mma16816(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}
// 2^x in float (the hardware's approximation, 2 ulp); 2^-inf = 0
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Rows of a stage are PITCH = DMAX + 8 elements apart: the 16 bytes of padding shift consecutive
// rows by one bank group, so the eight rows an ldmatrix touches never collide.
template <int DMAX> __host__ __device__ constexpr int pitch() { return DMAX + 8; }

struct KvSource {
    const bf16* kc;
    const bf16* vc;
    const int* table;      // this request's row of the block table
    int nkv, kvh, d, ps, ps_shift, num_pages;     // ps_shift: log2(ps) when ps is a power of two, else -1
};

// Element offset of key ``key``'s row in the cache, or -1 for a key outside [lo, hi] (or whose
// page id is out of range, which also sets the status word).
__device__ __forceinline__ long long row_offset(const KvSource& src, int key, int lo, int hi, int* status) {
    if (key < lo || key > hi) return -1;
    const int page = src.table[src.ps_shift >= 0 ? key >> src.ps_shift : key / src.ps];
    if (page < 0 || page >= src.num_pages) {
        if (status) atomicOr(status, FE_STATUS_BAD_PAGE);
        return -1;
    }
    const int within = src.ps_shift >= 0 ? key & (src.ps - 1) : key % src.ps;
    return (((long long)page * src.nkv + src.kvh) * src.ps + within) * src.d;
}

// Copy ROWS key rows and ROWS value rows into a stage with 16-byte asynchronous copies, THREADS
// threads sharing the work.  ``offs`` (shared memory) holds each row's offset in the cache, -1
// for rows that are filled with zeros instead (their scores are masked; zero values keep
// 0 * v finite).
template <int DMAX, int THREADS, int ROWS>
__device__ __forceinline__ void copy_rows(bf16* ks, bf16* vs, const KvSource& src, const long long* offs) {
    const int cpr = src.d >> 3;                       // 16-byte chunks per row
    const int step_r = THREADS / cpr, step_c = THREADS - step_r * cpr;
    int r = threadIdx.x / cpr, c = threadIdx.x - r * cpr;
    for (int idx = threadIdx.x; idx < ROWS * cpr; idx += THREADS) {
        const long long off = offs[r];
        const bool valid = off >= 0;
        const long long from = valid ? off + (c << 3) : 0;
        const int o = r * pitch<DMAX>() + (c << 3);
        cp_async16(ks + o, src.kc + from, valid ? 16 : 0);
        cp_async16(vs + o, src.vc + from, valid ? 16 : 0);
        r += step_r; c += step_c;
        if (c >= cpr) { c -= cpr; ++r; }
    }
}

// One warp, KEYS keys (32, or 16 when two warps share a tile): s = Q K^T, mask (only where ``masked``), online
// softmax in float with the running maximum kept in log2 units, o += P V.  ``ks``/``vs`` point at the first row.
// pos0/pos1 and lo0/lo1: last and first visible key of the queries in rows g and g + 8.
// UPPER = false: rows 8..15 of the tile are padding and their softmax is skipped.
template <int DMAX, bool UPPER, int KEYS = TK>
__device__ __forceinline__ void compute_tile(const bf16* ks, const bf16* vs, const unsigned (*qfrag)[4],
                                             float (*o)[4], float* m, float* l, int first_key, int d,
                                             float scale_log2, int pos0, int pos1, int lo0, int lo1, bool masked) {
    const int lane = threadIdx.x & 31, t = lane & 3;
    const int mat = lane >> 3, mrow = lane & 7;
    float s[KEYS / 8][4];
#pragma unroll
    for (int j = 0; j < KEYS / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    {
        // row = jp*16 + (mat>>1)*8 + mrow, 16-byte chunk = ksx*2 + (mat&1)
        const bf16* kbase = ks + ((mat >> 1) * 8 + mrow) * pitch<DMAX>() + (mat & 1) * 8;
#pragma unroll
        for (int ksx = 0; ksx < DMAX / 16; ++ksx) {
            if (ksx * 16 < d) {
#pragma unroll
                for (int jp = 0; jp < KEYS / 16; ++jp) {
                    unsigned r0, r1, r2, r3;
                    ldmatrix_x4(r0, r1, r2, r3, kbase + jp * 16 * pitch<DMAX>() + ksx * 16);
                    mma16816(s[jp * 2], qfrag[ksx], r0, r1);
                    mma16816(s[jp * 2 + 1], qfrag[ksx], r2, r3);
                }
            }
        }
    }
    if (masked) {
#pragma unroll
        for (int j = 0; j < KEYS / 8; ++j) {
#pragma unroll
            for (int e = 0; e < (UPPER ? 4 : 2); ++e) {
                const int key = first_key + j * 8 + 2 * t + (e & 1);
                const bool vis = e < 2 ? (key <= pos0 && key >= lo0) : (key <= pos1 && key >= lo1);
                if (!vis) s[j][e] = -CUDART_INF_F;
            }
        }
    }
    float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < KEYS / 8; ++j) {
        mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
        if (UPPER) mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    if (UPPER) { mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2)); }
    const float mn0 = fmaxf(m[0], mx0 * scale_log2), mn1 = UPPER ? fmaxf(m[1], mx1 * scale_log2) : m[1];
    const float ms0 = mn0 == -CUDART_INF_F ? 0.f : mn0, ms1 = mn1 == -CUDART_INF_F ? 0.f : mn1;
    const bool changed = mn0 != m[0] || (UPPER && mn1 != m[1]);
    if (__any_sync(0xffffffffu, changed)) {
        const float al0 = ex2(m[0] - ms0), al1 = UPPER ? ex2(m[1] - ms1) : 1.f;   // 2^-inf = 0 at the start
        l[0] *= al0;
        if (UPPER) l[1] *= al1;
#pragma unroll
        for (int n = 0; n < DMAX / 8; ++n) {
            o[n][0] *= al0; o[n][1] *= al0;
            if (UPPER) { o[n][2] *= al1; o[n][3] *= al1; }
        }
        m[0] = mn0; m[1] = mn1;
    }
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int j = 0; j < KEYS / 8; ++j) {
        s[j][0] = ex2(fmaf(s[j][0], scale_log2, -ms0)); s[j][1] = ex2(fmaf(s[j][1], scale_log2, -ms0));
        sum0 += s[j][0] + s[j][1];
        if (UPPER) {
            s[j][2] = ex2(fmaf(s[j][2], scale_log2, -ms1)); s[j][3] = ex2(fmaf(s[j][3], scale_log2, -ms1));
            sum1 += s[j][2] + s[j][3];
        }
    }
    l[0] += sum0; l[1] += sum1;                       // per-thread partial sums of the rows
    {
        // row = kk*16 + (mat&1)*8 + mrow, 16-byte chunk = np*2 + (mat>>1)
        const bf16* vbase = vs + ((mat & 1) * 8 + mrow) * pitch<DMAX>() + (mat >> 1) * 8;
#pragma unroll
        for (int kk = 0; kk < KEYS / 16; ++kk) {
            unsigned a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = UPPER ? pack_bf16(s[2 * kk][2], s[2 * kk][3]) : 0u;
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = UPPER ? pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]) : 0u;
#pragma unroll
            for (int np = 0; np < DMAX / 16; ++np) {
                if (np * 16 < d) {
                    unsigned r0, r1, r2, r3;
                    ldmatrix_x4_trans(r0, r1, r2, r3, vbase + kk * 16 * pitch<DMAX>() + np * 16);
                    mma16816(o[np * 2], a, r0, r1);
                    mma16816(o[np * 2 + 1], a, r2, r3);
                }
            }
        }
    }
}

// Query fragments of one 16-row tile: row g -> src0, row g + 8 -> src1 (nullptr: a padding row).
template <int DMAX>
__device__ __forceinline__ void load_q(unsigned (*qfrag)[4], const bf16* src0, const bf16* src1, int d) {
    const int t = threadIdx.x & 3;
#pragma unroll
    for (int ksx = 0; ksx < DMAX / 16; ++ksx) {
        qfrag[ksx][0] = qfrag[ksx][1] = qfrag[ksx][2] = qfrag[ksx][3] = 0u;
        if (ksx * 16 < d) {
            const int c = ksx * 16 + 2 * t;
            if (src0) { qfrag[ksx][0] = *reinterpret_cast<const unsigned*>(src0 + c);
                        qfrag[ksx][2] = *reinterpret_cast<const unsigned*>(src0 + c + 8); }
            if (src1) { qfrag[ksx][1] = *reinterpret_cast<const unsigned*>(src1 + c);
                        qfrag[ksx][3] = *reinterpret_cast<const unsigned*>(src1 + c + 8); }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// decode: grid (splits, nkv, requests), two warps, a ring of 32-key stages.  Every request brings
// exactly one token.  A warp's stream of dependent instructions, not memory, bounds what one warp
// gets through, and shared memory bounds how many blocks fit an SM: so the two warps of a block
// share every stage they load, each takes 16 of its 32 keys with running statistics of its own,
// and the two results are merged once at the end.
constexpr int DECODE_WARPS = 2;
constexpr int DECODE_KEYS = TK / DECODE_WARPS;   // keys of a stage per warp

// CLUSTER: the blocks of one (request, key/value head), one per split of the keys, are a thread-block cluster.  Each
// leaves its partial result in its own shared memory; after a cluster barrier every block merges its share of the
// output elements, reading the other blocks' partial results through distributed shared memory.  No scratch memory,
// no second kernel, and the merge takes the splits in index order whichever block runs where.
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float ld_cluster(const float* own, unsigned rank) {
    // the same variable in the shared memory of block ``rank`` of this cluster
    unsigned remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"((unsigned)__cvta_generic_to_shared(own)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote));
    return v;
}
constexpr int CLUSTER_MAX_SPLITS = 16;

// STAGES: the ring of 32-key stages; STAGES - 1 tiles are on their way while one is multiplied.  A block that walks
// only a few tiles (short contexts split many ways) spends its life waiting for memory: a deeper ring asks for its
// tiles earlier.
template <int DMAX, bool UPPER, bool CLUSTER = false, int STAGES = 2>
__global__ void __launch_bounds__(DECODE_WARPS * 32)
paged_decode_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out, long long out_stride,
                    float* __restrict__ part_o, float* __restrict__ part_lse, const bf16* __restrict__ kc,
                    const bf16* __restrict__ vc, const int* __restrict__ block_table, int bt_stride,
                    const int* __restrict__ cu_q, const int* __restrict__ q_start, int nq, int nkv, int d, int ps,
                    int num_pages, float scale_log2, int window, int* __restrict__ status) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ long long offs[TK];
    __shared__ long long first_offs[STAGES - 1][TK];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    constexpr int TILE = TK * pitch<DMAX>();         // elements per K (or V) stage
    constexpr int THREADS = DECODE_WARPS * 32;
    const int split = blockIdx.x, splits = gridDim.x, kvh = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int G = nq / nkv;
    const int tok = cu_q[b];
    const int pos = q_start[b];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int tile_lo = lo / TK, tile_hi = pos / TK;
    const int per = (tile_hi - tile_lo + 1 + splits - 1) / splits;
    const int t_begin = tile_lo + split * per, t_end = min(tile_hi + 1, t_begin + per);
    const int n_tiles = max(0, t_end - t_begin);

    KvSource src{kc, vc, block_table + (size_t)b * bt_stride, nkv, kvh, d, ps, (ps & (ps - 1)) == 0 ? __ffs(ps) - 1 : -1,
                 num_pages};
    // thread r < 32 looks up key r of a tile; then the block copies the 32 rows.  The first STAGES - 1 tiles are asked
    // for at once; every step of the loop then asks for one more.  A group of copies is committed at every turn, empty
    // or not, so that "all but the youngest STAGES - 2 groups have landed" always means "tile ``it`` has landed".
    constexpr int AHEAD = STAGES - 1;
    static_assert(AHEAD * TK <= DECODE_WARPS * 32, "one thread per key of the tiles asked for at the start");
    // all the first tiles' keys are looked up at once (one trip to the block table, not one per tile)
    if (threadIdx.x < AHEAD * TK) {
        const int a = threadIdx.x / TK, k = threadIdx.x - a * TK;
        first_offs[a][k] = a < n_tiles ? row_offset(src, (t_begin + a) * TK + k, lo, pos, status) : -1;
    }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < AHEAD; ++a) {
        if (a < n_tiles) copy_rows<DMAX, THREADS, TK>(smem + a * 2 * TILE, smem + a * 2 * TILE + TILE, src, first_offs[a]);
        cp_async_commit();
    }

    unsigned qfrag[DMAX / 16][4];
    const bf16* qrow = q + (size_t)tok * q_stride + (size_t)kvh * G * d;
    load_q<DMAX>(qfrag, g < G ? qrow + (size_t)g * d : nullptr, (UPPER && g + 8 < G) ? qrow + (size_t)(g + 8) * d : nullptr, d);

    float o[DMAX / 8][4];
#pragma unroll
    for (int n = 0; n < DMAX / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};

    for (int it = 0; it < n_tiles; ++it) {
        // the stage of tile it - 1 is free (both warps finished it): tile it + AHEAD goes there
        long long next = -1;
        const bool more = it + AHEAD < n_tiles;
        if (more && threadIdx.x < TK) next = row_offset(src, (t_begin + it + AHEAD) * TK + threadIdx.x, lo, pos, status);
        cp_async_wait<AHEAD - 1>();                  // this thread's part of tile ``it`` has landed
        __syncthreads();                             // ... and everyone else's; the offsets of the last copy have been read
        if (more) {
            if (threadIdx.x < TK) offs[threadIdx.x] = next;
            __syncthreads();
            bf16* st = smem + ((it + AHEAD) % STAGES) * 2 * TILE;
            copy_rows<DMAX, THREADS, TK>(st, st + TILE, src, offs);
        }
        cp_async_commit();
        const bf16* sp = smem + (it % STAGES) * 2 * TILE + warp * DECODE_KEYS * pitch<DMAX>();
        const int first = (t_begin + it) * TK + warp * DECODE_KEYS;
        compute_tile<DMAX, UPPER, DECODE_KEYS>(sp, sp + TILE, qfrag, o, m, l, first, d, scale_log2, pos, pos, lo, lo,
                                               first + DECODE_KEYS - 1 > pos || first < lo);
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
    // the second warp hands its running statistics and output to the first through the stages' memory (free now),
    // thread to thread: both hold the same rows and columns
    __syncthreads();
    float* hand = reinterpret_cast<float*>(smem_raw);                 // [DMAX / 2 + 4][32] floats
    if (warp == 1) {
#pragma unroll
        for (int n = 0; n < DMAX / 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) hand[(n * 4 + e) * 32 + lane] = o[n][e];
        hand[(DMAX / 2) * 32 + lane] = m[0]; hand[(DMAX / 2 + 1) * 32 + lane] = m[1];
        hand[(DMAX / 2 + 2) * 32 + lane] = l[0]; hand[(DMAX / 2 + 3) * 32 + lane] = l[1];
    }
    __syncthreads();
    if (warp == 1 && !CLUSTER) return;
    // where a block of a cluster leaves its partial result: rows of d + 1 floats (the head's output, then the
    // logarithm of its sum), behind the memory the two warps exchange their results through
    float* mine = reinterpret_cast<float*>(smem_raw) + (DMAX / 2 + 4) * 32;
    if (warp == 0) {
#pragma unroll
    for (int i = 0; i < (UPPER ? 2 : 1); ++i) {
        const float m1 = hand[(DMAX / 2 + i) * 32 + lane], l1 = hand[(DMAX / 2 + 2 + i) * 32 + lane];
        const float mn = fmaxf(m[i], m1);
        const float a0 = mn == -CUDART_INF_F ? 0.f : ex2(m[i] - mn), a1 = mn == -CUDART_INF_F ? 0.f : ex2(m1 - mn);
        l[i] = l[i] * a0 + l1 * a1;
        m[i] = mn;
#pragma unroll
        for (int n = 0; n < DMAX / 8; ++n) {
            o[n][2 * i] = o[n][2 * i] * a0 + hand[(n * 4 + 2 * i) * 32 + lane] * a1;
            o[n][2 * i + 1] = o[n][2 * i + 1] * a0 + hand[(n * 4 + 2 * i + 1) * 32 + lane] * a1;
        }
    }
#pragma unroll
    for (int i = 0; i < (UPPER ? 2 : 1); ++i) {
        const int row = g + 8 * i;
        if (row >= G) continue;
        const int head = kvh * G + row;
        const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
        if (CLUSTER) {
            float* po = mine + (size_t)row * (d + 1);
#pragma unroll
            for (int n = 0; n < DMAX / 8; ++n) {
                const int col = n * 8 + 2 * t;
                if (col < d) { po[col] = o[n][2 * i] * inv; po[col + 1] = o[n][2 * i + 1] * inv; }
            }
            if (t == 0) po[d] = l[i] > 0.f ? m[i] + log2f(l[i]) : -CUDART_INF_F;
        } else if (splits == 1) {
            bf16* op = out + (size_t)tok * out_stride + (size_t)head * d;
#pragma unroll
            for (int n = 0; n < DMAX / 8; ++n) {
                const int col = n * 8 + 2 * t;
                if (col < d)
                    *reinterpret_cast<__nv_bfloat162*>(op + col) = __floats2bfloat162_rn(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
            }
        } else {
            const size_t slot = ((size_t)b * nq + head) * splits + split;
            float* po = part_o + slot * d;
#pragma unroll
            for (int n = 0; n < DMAX / 8; ++n) {
                const int col = n * 8 + 2 * t;
                if (col < d) *reinterpret_cast<float2*>(po + col) = make_float2(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
            }
            if (t == 0) part_lse[slot] = l[i] > 0.f ? m[i] + log2f(l[i]) : -CUDART_INF_F;
        }
    }
    }   // warp 0
    if (CLUSTER) {
        cluster_barrier();                        // every block's partial result is in its shared memory
        // element e = (head of the group, column): the cluster's threads share them out; each adds the splits in
        // index order, weighted by 2^(logarithm of the split's sum - the largest of them)
        const int total = G * d;
        for (int e = split * THREADS + threadIdx.x; e < total; e += splits * THREADS) {
            const int row = e / d, col = e - row * d;
            const float* lse_at = mine + (size_t)row * (d + 1) + d;
            const float* val_at = mine + (size_t)row * (d + 1) + col;
            float lse[CLUSTER_MAX_SPLITS], val[CLUSTER_MAX_SPLITS];
            float mx = -CUDART_INF_F;
#pragma unroll
            for (int s2 = 0; s2 < CLUSTER_MAX_SPLITS; ++s2) {
                lse[s2] = s2 < splits ? ld_cluster(lse_at, s2) : -CUDART_INF_F;
                val[s2] = s2 < splits ? ld_cluster(val_at, s2) : 0.f;
                mx = fmaxf(mx, lse[s2]);
            }
            float sum = 0.f, acc = 0.f;
#pragma unroll
            for (int s2 = 0; s2 < CLUSTER_MAX_SPLITS; ++s2) {
                const float w = (s2 < splits && mx != -CUDART_INF_F) ? ex2(lse[s2] - mx) : 0.f;
                sum += w;
                acc += w * val[s2];
            }
            out[(size_t)tok * out_stride + (size_t)(kvh * G + row) * d + col] = __float2bfloat16_rn(sum > 0.f ? acc / sum : 0.f);
        }
        cluster_barrier();                        // nobody leaves while its shared memory may still be read
    }
}

// Merge the splits: grid (nq, requests), one thread per element of the head.  The weights of the
// splits are computed once per block; the sums run four splits at a time so that their loads
// overlap (the order of the additions is fixed all the same).
constexpr int MAX_SPLITS_SHARED = 256;
constexpr int COMBINE_MAX_GROUPS = 8;        // sets of threads that share the splits of one (request, head) in the merge

__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                      bf16* __restrict__ out, long long out_stride, const int* __restrict__ cu_q,
                                      int nq, int d, int splits, int groups, int requests,
                                      const void* __restrict__ upcoming, long long upcoming_bytes) {
    if ((int)blockIdx.y >= requests) {
        // rows of blocks beyond the requests: the merge barely touches memory, so they start the matrix that the
        // next kernel streams (the output projection) into L2
        const long long workers = (long long)(gridDim.y - requests) * gridDim.x * blockDim.x;
        prefetch_l2_share(upcoming, upcoming_bytes,
                          ((long long)(blockIdx.y - requests) * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x, workers);
        return;
    }
    griddep_wait();
    griddep_launch_dependents();
    __shared__ float weight[MAX_SPLITS_SHARED];
    __shared__ float sums[COMBINE_MAX_GROUPS][128];
    __shared__ float inv_total;
    const int head = blockIdx.x, b = blockIdx.y;
    const size_t base = ((size_t)b * nq + head) * splits;
    if (threadIdx.x < 32) {
        // all of a lane's logarithms are asked for at once: one trip to memory, not one per 32 splits
        float lse[MAX_SPLITS_SHARED / 32];
        float mx = -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < MAX_SPLITS_SHARED / 32; ++i) {
            const int s = threadIdx.x + 32 * i;
            lse[i] = s < splits ? part_lse[base + s] : -CUDART_INF_F;
            mx = fmaxf(mx, lse[i]);
        }
        mx = warp_max(mx);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_SPLITS_SHARED / 32; ++i) {
            const int s = threadIdx.x + 32 * i;
            const float w = mx == -CUDART_INF_F ? 0.f : exp2f(lse[i] - mx);
            if (s < splits) weight[s] = w;
            sum += s < splits ? w : 0.f;
        }
        sum = warp_sum(sum);
        if (threadIdx.x == 0) inv_total = sum > 0.f ? 1.f / sum : 0.f;
    }
    __syncthreads();
    // ``groups`` sets of threads share the splits out among them (split s goes to set s % groups), so that a
    // long list of splits is a few trips to memory deep; their sums are added in a fixed order
    const int cols = blockDim.x / groups, grp = threadIdx.x / cols, col = threadIdx.x - grp * cols;
    bf16* op = out + (size_t)cu_q[b] * out_stride + (size_t)head * d;
    const float* po = part_o + base * d;
    for (int j0 = 0; j0 < d; j0 += cols) {
        const int j = j0 + col;
        float acc = 0.f;
        if (j < d) {
            int s = grp;
            for (; s + 3 * groups < splits; s += 4 * groups) {
                const float v0 = po[(size_t)s * d + j], v1 = po[(size_t)(s + groups) * d + j];
                const float v2 = po[(size_t)(s + 2 * groups) * d + j], v3 = po[(size_t)(s + 3 * groups) * d + j];
                acc += weight[s] * v0; acc += weight[s + groups] * v1;
                acc += weight[s + 2 * groups] * v2; acc += weight[s + 3 * groups] * v3;
            }
            for (; s < splits; s += groups) acc += weight[s] * po[(size_t)s * d + j];
        }
        if (groups > 1) {
            sums[grp][col] = acc;
            __syncthreads();
            if (grp == 0) {
                for (int g = 1; g < groups; ++g) acc += sums[g][col];
            }
            __syncthreads();                         // before the next round of columns overwrites the sums
        }
        if (grp == 0 && j < d) op[j] = __float2bfloat16_rn(acc * inv_total);
    }
}

// ---------------------------------------------------------------------------------------------
// prefill: grid (row tiles, nkv, requests), four warps, two stages of 64 keys.  Row m of a
// (request, kv head) is the pair (query m / G, head m % G of the group); a block takes 64
// consecutive rows; blocks with the most keys to walk (the last rows) are scheduled first.
constexpr int PREFILL_WARPS = 4;
constexpr int PREFILL_ROWS = PREFILL_WARPS * 16;
constexpr int PREFILL_KEYS = 64;                 // keys per stage
constexpr int PREFILL_STAGES = 2;

template <int DMAX>
__global__ void __launch_bounds__(PREFILL_WARPS * 32)
paged_prefill_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out, long long out_stride,
                     const bf16* __restrict__ kc, const bf16* __restrict__ vc, const int* __restrict__ block_table,
                     int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ q_start, int nq, int nkv,
                     int d, int ps, int num_pages, float scale_log2, int window, int* __restrict__ status) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ long long offs[2][PREFILL_KEYS];
    constexpr int THREADS = PREFILL_WARPS * 32;
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    constexpr int STAGE = PREFILL_KEYS * pitch<DMAX>();   // elements per K (or V) stage
    const int kvh = blockIdx.y, r = blockIdx.z;
    const int G = nq / nkv;
    const int tok0 = cu_q[r], n_q = cu_q[r + 1] - tok0;
    const int rows = n_q * G;
    const int m_block = (gridDim.x - 1 - blockIdx.x) * PREFILL_ROWS;
    if (m_block >= rows) return;
    const int start = q_start[r];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int m0 = m_block + warp * 16 + g, m1 = m0 + 8;
    const bool v0 = m0 < rows, v1 = m1 < rows;
    const int qi0 = v0 ? m0 / G : 0, qi1 = v1 ? m1 / G : 0;
    const int pos0 = v0 ? start + qi0 : -1, pos1 = v1 ? start + qi1 : -1;
    const int lo0 = window > 0 ? max(0, pos0 - window + 1) : 0, lo1 = window > 0 ? max(0, pos1 - window + 1) : 0;
    const int head0 = kvh * G + (v0 ? m0 % G : 0), head1 = kvh * G + (v1 ? m1 % G : 0);

    // keys this block needs: from the window edge of its first query to its last query
    const int qi_first = m_block / G, qi_last = min(n_q - 1, (m_block + PREFILL_ROWS - 1) / G);
    const int hi = start + qi_last;
    const int lo = window > 0 ? max(0, start + qi_first - window + 1) : 0;
    const int s_begin = lo / PREFILL_KEYS, n_stages = hi / PREFILL_KEYS - s_begin + 1;
    KvSource src{kc, vc, block_table + (size_t)r * bt_stride, nkv, kvh, d, ps, (ps & (ps - 1)) == 0 ? __ffs(ps) - 1 : -1,
                 num_pages};
    // threads 0 .. 63 look up one key each of the stage after next; all threads copy
    if (threadIdx.x < PREFILL_KEYS) {
        offs[0][threadIdx.x] = row_offset(src, s_begin * PREFILL_KEYS + threadIdx.x, lo, hi, status);
        offs[1][threadIdx.x] = n_stages > 1 ? row_offset(src, (s_begin + 1) * PREFILL_KEYS + threadIdx.x, lo, hi, status) : -1;
    }
    __syncthreads();
    copy_rows<DMAX, THREADS, PREFILL_KEYS>(smem, smem + STAGE, src, offs[0]);
    cp_async_commit();

    unsigned qfrag[DMAX / 16][4];
    load_q<DMAX>(qfrag, v0 ? q + (size_t)(tok0 + qi0) * q_stride + (size_t)head0 * d : nullptr,
                 v1 ? q + (size_t)(tok0 + qi1) * q_stride + (size_t)head1 * d : nullptr, d);
    float o[DMAX / 8][4];
#pragma unroll
    for (int n = 0; n < DMAX / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};

    // this warp's rows: the first and last position any of them has, and the widest window edge
    const int w_first = m_block + warp * 16, w_last = min(rows - 1, w_first + 15);
    const bool w_any = w_first < rows;
    const int w_pos_min = w_any ? start + w_first / G : -1, w_pos_max = w_any ? start + w_last / G : -1;
    const int w_lo_min = window > 0 ? max(0, w_pos_min - window + 1) : 0;
    const int w_lo_max = window > 0 ? max(0, w_pos_max - window + 1) : 0;

    for (int it = 0; it < n_stages; ++it) {
        cp_async_wait<0>();
        __syncthreads();                 // stage ``it`` has landed; everyone is done with stage it - 1
        if (it + 1 < n_stages) {
            bf16* st = smem + ((it + 1) & 1) * 2 * STAGE;
            copy_rows<DMAX, THREADS, PREFILL_KEYS>(st, st + STAGE, src, offs[(it + 1) & 1]);
        }
        cp_async_commit();
        const bf16* st = smem + (it & 1) * 2 * STAGE;
#pragma unroll
        for (int sub = 0; sub < PREFILL_KEYS / TK; ++sub) {
            const int first = (s_begin + it) * PREFILL_KEYS + sub * TK;
            if (w_any && first <= w_pos_max && first + TK - 1 >= w_lo_min) {
                // rows differ in what they see only near the diagonal and the window edge
                const bool masked = first + TK - 1 > w_pos_min || first < w_lo_max || !(v0 && v1);
                compute_tile<DMAX, true>(st + sub * TK * pitch<DMAX>(), st + STAGE + sub * TK * pitch<DMAX>(), qfrag, o, m,
                                         l, first, d, scale_log2, pos0, pos1, lo0, lo1, masked);
            }
        }
        // offsets of stage it + 2 go where those of stage ``it`` were: all copies of stage ``it``'s
        // offsets were issued before the barrier above, and the next barrier publishes the new ones
        if (it + 2 < n_stages && threadIdx.x < PREFILL_KEYS)
            offs[it & 1][threadIdx.x] = row_offset(src, (s_begin + it + 2) * PREFILL_KEYS + threadIdx.x, lo, hi, status);
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (!(i == 0 ? v0 : v1)) continue;
        const int qi = i == 0 ? qi0 : qi1, head = i == 0 ? head0 : head1;
        const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
        bf16* op = out + (size_t)(tok0 + qi) * out_stride + (size_t)head * d;
#pragma unroll
        for (int n = 0; n < DMAX / 8; ++n) {
            const int col = n * 8 + 2 * t;
            if (col < d)
                *reinterpret_cast<__nv_bfloat162*>(op + col) = __floats2bfloat162_rn(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
        }
    }
}

constexpr float LOG2E = 1.4426950408889634f;

template <int DMAX> size_t decode_smem(int stages = 2) { return (size_t)stages * 2 * TK * pitch<DMAX>() * sizeof(bf16); }
template <int DMAX> size_t prefill_smem() { return (size_t)PREFILL_STAGES * 2 * PREFILL_KEYS * pitch<DMAX>() * sizeof(bf16); }

template <typename K> int allow_smem(K kernel, size_t bytes, const char* what) {
    if (bytes > 48 * 1024) {
        const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (err != cudaSuccess) {
            fe_set_error("%s: %s", what, cudaGetErrorString(err));
            return 1;
        }
    }
    return 0;
}

int check_common(const char* what, int nq, int nkv, int d, int ps, int num_pages, int window, long long q_stride,
                 long long out_stride) {
    FE_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "%s: bad head counts %d/%d", what, nq, nkv);
    FE_REQUIRE(d >= 16 && d <= 256 && d % 16 == 0, "%s: head size %d is not a multiple of 16 in [16, 256]", what, d);
    FE_REQUIRE(ps > 0 && num_pages > 0 && window >= 0, "%s: bad page size, page count or window", what);
    FE_REQUIRE(q_stride % 8 == 0 && out_stride % 2 == 0, "%s: row strides must keep 16-byte alignment", what);
    return 0;
}

}  // namespace

// The most key splits the merge kernel takes (its per-split weights live in shared memory).
extern "C" int fe_paged_decode_max_splits(void) { return MAX_SPLITS_SHARED; }

// Number of bytes of scratch the decode kernel needs for ``splits`` > 1 (0 for one split):
// float partial outputs [requests, nq, splits, d] followed by float log-sum-exps [requests, nq, splits].
extern "C" long long fe_paged_decode_scratch_bytes(int requests, int nq, int d, int splits) {
    if (splits <= 1) return 0;
    return (long long)requests * nq * splits * (d + 1) * (long long)sizeof(float);
}

// ``upcoming`` (may be null): memory that the kernel after this one will stream, ``upcoming_bytes`` of it; with more
// than one split, extra blocks of the merge kernel ask for it to be brought into L2.
extern "C" int fe_paged_decode_mma_upcoming(const void* q, long long q_stride, void* out, long long out_stride, void* scratch,
                                            const void* kc, const void* vc, const int* block_table, int bt_stride,
                                            const int* cu_q, const int* q_start, int requests, int nq, int nkv, int d, int ps,
                                            int num_pages, float scale, int window, int splits, const void* upcoming,
                                            long long upcoming_bytes, int* status, cudaStream_t stream) {
    if (check_common("paged_decode", nq, nkv, d, ps, num_pages, window, q_stride, out_stride)) return 1;
    FE_REQUIRE(nq / nkv <= 16, "paged_decode: %d query heads per key/value head; this kernel takes up to 16", nq / nkv);
    FE_REQUIRE(splits >= 1 && splits <= MAX_SPLITS_SHARED && requests >= 0,
               "paged_decode: %d splits; this kernel takes 1 to %d", splits, MAX_SPLITS_SHARED);
    FE_REQUIRE(splits == 1 || scratch != nullptr, "paged_decode: %d splits need scratch memory", splits);
    if (requests == 0) return 0;
    float* part_o = (float*)scratch;
    float* part_lse = part_o ? part_o + (size_t)requests * nq * splits * d : nullptr;
    const dim3 grid(splits, nkv, requests);
    const float scale_log2 = scale * LOG2E;
#define FE_DECODE(DMAX, UPPER)                                                                                    \
    do {                                                                                                          \
        if (allow_smem(paged_decode_kernel<DMAX, UPPER>, decode_smem<DMAX>(), "paged_decode")) return 1;          \
        fe::launch(paged_decode_kernel<DMAX, UPPER>, grid, DECODE_WARPS * 32, decode_smem<DMAX>(), stream,                               \
            (const bf16*)q, q_stride, (bf16*)out, out_stride, part_o, part_lse, (const bf16*)kc, (const bf16*)vc, \
            block_table, bt_stride, cu_q, q_start, nq, nkv, d, ps, num_pages, scale_log2, window, status);        \
    } while (0)
    const bool upper = nq / nkv > 8;
    if (d <= 64) { if (upper) FE_DECODE(64, true); else FE_DECODE(64, false); }
    else if (d <= 128) { if (upper) FE_DECODE(128, true); else FE_DECODE(128, false); }
    else { if (upper) FE_DECODE(256, true); else FE_DECODE(256, false); }
#undef FE_DECODE
    if (fe_check_launch("paged_decode")) return 2;
    if (splits > 1) {
        FE_REQUIRE(upcoming_bytes >= 0, "paged_decode: negative byte count");
        const int extra = upcoming && upcoming_bytes > 0 ? 2 : 0;
        const int cols = d >= 128 ? 128 : 64;
        const int groups = splits >= 64 ? 8 : splits >= 32 ? 4 : splits >= 16 ? 2 : 1;
        fe::launch(decode_combine_kernel, dim3(nq, requests + extra), cols * groups, 0, stream,
            part_o, part_lse, (bf16*)out, out_stride, cu_q, nq, d, splits, groups, requests, upcoming, upcoming_bytes);
        return fe_check_launch("paged_decode combine");
    }
    return 0;
}

// The same attention with the splits of a (request, key/value head) as one thread-block cluster that merges its
// partial results through distributed shared memory: one kernel, no scratch memory.  1 <= splits <= 16 (clusters
// of more than 8 blocks are asked for as a non-portable size); the cluster must fit the device, else an error.
extern "C" int fe_paged_decode_cluster_max_splits(void) { return CLUSTER_MAX_SPLITS; }

// How many clusters of ``splits`` blocks of the kernel that fe_paged_decode_cluster would launch for these sizes are
// resident on the device at once (a cluster lives inside one processing cluster of the GPU, so this is less than
// the blocks that fit divided by ``splits``); 0 when the device cannot place such a cluster at all, -1 on an error.
// A step that needs a few clusters more than this runs them alone after the round.
extern "C" int fe_paged_decode_cluster_resident(int requests, int nq, int nkv, int d, int splits) {
    FE_REQUIRE(splits >= 1 && splits <= CLUSTER_MAX_SPLITS && requests >= 1 && nq >= 1 && nkv >= 1 && d >= 1 && d <= 256,
               "paged_decode (cluster): bad sizes");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, nkv, requests);
    cfg.blockDim = dim3(DECODE_WARPS * 32);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const bool deep = (long long)splits * nkv * requests <= 4LL * fe_sm_count();
    int clusters = 0;
#define FE_RESIDENT_STAGES(DMAX, UPPER, STAGES)                                                                        \
    do {                                                                                                               \
        auto kernel = paged_decode_kernel<DMAX, UPPER, true, STAGES>;                                                  \
        if (allow_smem(kernel, decode_smem<DMAX>(STAGES), "paged_decode (cluster)")) return -1;                        \
        if (splits > 8 && cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) { \
            cudaGetLastError();                                                                                        \
            return 0;                                                                                                  \
        }                                                                                                              \
        cfg.dynamicSmemBytes = decode_smem<DMAX>(STAGES);                                                              \
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) {                                  \
            cudaGetLastError();                                                                                        \
            return 0;                                                                                                  \
        }                                                                                                              \
    } while (0)
#define FE_RESIDENT(DMAX, UPPER)                                                                                       \
    do {                                                                                                               \
        if (deep) FE_RESIDENT_STAGES(DMAX, UPPER, 3); else FE_RESIDENT_STAGES(DMAX, UPPER, 2);                         \
    } while (0)
    const bool upper = nq / nkv > 8;
    if (d <= 64) { if (upper) FE_RESIDENT(64, true); else FE_RESIDENT(64, false); }
    else if (d <= 128) { if (upper) FE_RESIDENT(128, true); else FE_RESIDENT(128, false); }
    else { if (upper) FE_RESIDENT(256, true); else FE_RESIDENT(256, false); }
#undef FE_RESIDENT
#undef FE_RESIDENT_STAGES
    return clusters;
}

extern "C" int fe_paged_decode_cluster(const void* q, long long q_stride, void* out, long long out_stride,
                                       const void* kc, const void* vc, const int* block_table, int bt_stride,
                                       const int* cu_q, const int* q_start, int requests, int nq, int nkv, int d, int ps,
                                       int num_pages, float scale, int window, int splits, int* status,
                                       cudaStream_t stream) {
    if (check_common("paged_decode", nq, nkv, d, ps, num_pages, window, q_stride, out_stride)) return 1;
    FE_REQUIRE(nq / nkv <= 16, "paged_decode: %d query heads per key/value head; this kernel takes up to 16", nq / nkv);
    FE_REQUIRE(splits >= 1 && splits <= CLUSTER_MAX_SPLITS && requests >= 0,
               "paged_decode (cluster): %d splits; a cluster takes 1 to %d", splits, CLUSTER_MAX_SPLITS);
    FE_REQUIRE(nkv <= 65535 && requests <= 65535, "paged_decode (cluster): grid too large");
    if (requests == 0) return 0;
    const float scale_log2 = scale * LOG2E;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, nkv, requests);
    cfg.blockDim = dim3(DECODE_WARPS * 32);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = (fe_pdl_enabled() & 16) != 0;     // a class of its own
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    // a ring of three stages while all blocks still fit the device at once with it (four of them an SM at head size 128)
    const long long blocks = (long long)splits * nkv * requests;
    const bool deep = blocks <= 4LL * fe_sm_count();
#define FE_DECODE_CLUSTER(DMAX, UPPER)                                                                                 \
    do {                                                                                                               \
        if (deep) FE_DECODE_CLUSTER_STAGES(DMAX, UPPER, 3); else FE_DECODE_CLUSTER_STAGES(DMAX, UPPER, 2);             \
    } while (0)
#define FE_DECODE_CLUSTER_STAGES(DMAX, UPPER, STAGES)                                                                  \
    do {                                                                                                               \
        auto kernel = paged_decode_kernel<DMAX, UPPER, true, STAGES>;                                                  \
        if (allow_smem(kernel, decode_smem<DMAX>(STAGES), "paged_decode (cluster)")) return 1;                         \
        if (splits > 8) {                                                                                              \
            const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);    \
            FE_REQUIRE(err == cudaSuccess, "paged_decode (cluster): %s", cudaGetErrorString(err));                      \
        }                                                                                                              \
        cfg.dynamicSmemBytes = decode_smem<DMAX>(STAGES);                                                              \
        const cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, (const bf16*)q, q_stride, (bf16*)out, out_stride,     \
            (float*)nullptr, (float*)nullptr, (const bf16*)kc, (const bf16*)vc, block_table, bt_stride, cu_q, q_start, \
            nq, nkv, d, ps, num_pages, scale_log2, window, status);                                                    \
        FE_REQUIRE(err == cudaSuccess, "paged_decode (cluster of %d): %s", splits, cudaGetErrorString(err));           \
    } while (0)
    const bool upper = nq / nkv > 8;
    if (d <= 64) { if (upper) FE_DECODE_CLUSTER(64, true); else FE_DECODE_CLUSTER(64, false); }
    else if (d <= 128) { if (upper) FE_DECODE_CLUSTER(128, true); else FE_DECODE_CLUSTER(128, false); }
    else { if (upper) FE_DECODE_CLUSTER(256, true); else FE_DECODE_CLUSTER(256, false); }
#undef FE_DECODE_CLUSTER
#undef FE_DECODE_CLUSTER_STAGES
    return fe_check_launch("paged_decode (cluster)");
}

extern "C" int fe_paged_decode_mma(const void* q, long long q_stride, void* out, long long out_stride, void* scratch,
                                   const void* kc, const void* vc, const int* block_table, int bt_stride,
                                   const int* cu_q, const int* q_start, int requests, int nq, int nkv, int d, int ps,
                                   int num_pages, float scale, int window, int splits, int* status,
                                   cudaStream_t stream) {
    return fe_paged_decode_mma_upcoming(q, q_stride, out, out_stride, scratch, kc, vc, block_table, bt_stride, cu_q, q_start,
                                        requests, nq, nkv, d, ps, num_pages, scale, window, splits, nullptr, 0, status, stream);
}

extern "C" int fe_paged_prefill_mma(const void* q, long long q_stride, void* out, long long out_stride,
                                    const void* kc, const void* vc, const int* block_table, int bt_stride,
                                    const int* cu_q, const int* q_start, int requests, int max_q_len, int nq, int nkv,
                                    int d, int ps, int num_pages, float scale, int window, int* status,
                                    cudaStream_t stream) {
    if (check_common("paged_prefill", nq, nkv, d, ps, num_pages, window, q_stride, out_stride)) return 1;
    FE_REQUIRE(requests >= 0 && max_q_len >= 0, "paged_prefill: bad request count or length");
    if (requests == 0 || max_q_len == 0) return 0;
    const long long rows = (long long)max_q_len * (nq / nkv);
    const long long tiles = (rows + PREFILL_ROWS - 1) / PREFILL_ROWS;
    FE_REQUIRE(tiles <= 2147483647LL && nkv <= 65535 && requests <= 65535, "paged_prefill: grid too large");
    const dim3 grid((unsigned)tiles, nkv, requests);
    const float scale_log2 = scale * LOG2E;
#define FE_PREFILL(DMAX)                                                                                       \
    do {                                                                                                       \
        if (allow_smem(paged_prefill_kernel<DMAX>, prefill_smem<DMAX>(), "paged_prefill")) return 1;           \
        fe::launch(paged_prefill_kernel<DMAX>, grid, PREFILL_WARPS * 32, prefill_smem<DMAX>(), stream,                 \
            (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kc, (const bf16*)vc, block_table,  \
            bt_stride, cu_q, q_start, nq, nkv, d, ps, num_pages, scale_log2, window, status);                  \
    } while (0)
    if (d <= 64) FE_PREFILL(64);
    else if (d <= 128) FE_PREFILL(128);
    else FE_PREFILL(256);
#undef FE_PREFILL
    return fe_check_launch("paged_prefill");
}

// ---------------------------------------------------------------------------------------------
// The same decode attention for callers that cannot allocate: the scratch memory is a fixed
// array of this library (see no_alloc_api.h for who needs this and what the limits are).
#include "no_alloc_api.h"

// In host code this name is only a handle for the symbol, not a device address: the address a
// kernel can use comes from cudaGetSymbolAddress, looked up once per device below.
static __device__ __align__(256) unsigned char g_static_decode_scratch[FE_STATIC_SCRATCH_BYTES];

extern "C" long long fe_static_scratch_bytes(void) { return (long long)FE_STATIC_SCRATCH_BYTES; }

extern "C" int fe_paged_decode_mma_static(const void* q, long long q_stride, void* out, long long out_stride,
                                          const void* kc, const void* vc, const int* block_table, int bt_stride,
                                          const int* cu_q, const int* q_start, int requests, int nq, int nkv, int d,
                                          int ps, int num_pages, float scale, int window, int splits, int* status,
                                          cudaStream_t stream) {
    constexpr int MAX_DEVICES = 64;
    static void* address_on[MAX_DEVICES] = {nullptr};
    int device = -1;
    cudaError_t err = cudaGetDevice(&device);
    FE_REQUIRE(err == cudaSuccess, "paged_decode (static scratch): cudaGetDevice: %s", cudaGetErrorString(err));
    FE_REQUIRE(device >= 0 && device < MAX_DEVICES, "paged_decode (static scratch): device %d is out of range", device);
    if (address_on[device] == nullptr) {
        // set-up, once per device, with that device current: ask the runtime where the array lives there
        void* where = nullptr;
        err = cudaGetSymbolAddress(&where, g_static_decode_scratch);
        FE_REQUIRE(err == cudaSuccess && where != nullptr, "paged_decode (static scratch): cudaGetSymbolAddress: %s",
                   cudaGetErrorString(err));
        address_on[device] = where;
    }
    FE_REQUIRE(requests >= 0 && nq > 0 && d > 0 && splits >= 1, "paged_decode (static scratch): bad sizes");
    const long long need = fe_paged_decode_scratch_bytes(requests, nq, d, splits);
    FE_REQUIRE(need <= (long long)FE_STATIC_SCRATCH_BYTES,
               "paged_decode (static scratch): %d requests x %d heads x %d splits x head size %d need %lld bytes of "
               "scratch; the built-in array holds %lld (use fewer splits or requests, or the entry point that takes "
               "the caller's scratch)", requests, nq, splits, d, need, (long long)FE_STATIC_SCRATCH_BYTES);
    return fe_paged_decode_mma(q, q_stride, out, out_stride, address_on[device], kc, vc, block_table, bt_stride, cu_q,
                               q_start, requests, nq, nkv, d, ps, num_pages, scale, window, splits, status, stream);
}
