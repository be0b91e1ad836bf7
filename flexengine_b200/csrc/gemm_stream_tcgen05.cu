// y[M, N] = x[M, K] . W[N, K]^T for 9 to 128 rows (decode at medium batch, short portions):
// a stream of the weight matrix through the fifth-generation tensor cores, operands swapped.
//
// The 128 rows of a W tile are the M of tcgen05.mma (128 x MB x 16, MB = the batch rounded up to a
// multiple of 16), the activations are its N, the accumulator [128 W rows, MB] lives in TMEM.  A
// block owns one W tile and one slice of K; warp 0 (one lane) streams 16 KB of W and the matching
// slice of x per stage with TMA into a ring of stages (about 100 KB of W in flight per SM, which is
// what HBM latency times bandwidth asks for), warp 1 (one lane) issues the MMAs, warps 2..5 read
// the accumulator and write it transposed.  Narrow matrices are split along K over several blocks;
// their float partial sums are added in a fixed order by a small second kernel (deterministic).
// Epilogues: bfloat16, float (vocabulary projection), SwiGLU (a tile is 64 gate rows and their 64
// up rows; the halves meet in shared memory).
// The reference runs these products through cuBLAS (inference/models/qwen2.py:99-101,129-135).
//
// Measured on B200 against cuBLAS (same products, inside CUDA graphs): on a par for the wide gate/up
// product with the activation fused (48.3 against 49.0 us at 16 rows), on a par for the down
// projection, 5 to 30 % behind on the narrow and the very wide ones.  It is therefore not what
// ``linear`` picks by itself; it is kept, tested, as the starting point of a persistent variant.
//
// Every wait on an mbarrier is bounded; when one runs out the block records it in the status
// word, every role leaves its loop, tensor memory is freed and the block returns.
#include <cuda.h>

#include "common.cuh"

using namespace fe;

namespace {

constexpr int TILE_ROWS = 128;      // W rows per block = UMMA M
constexpr int BK = 64;              // k elements per stage (one 128-byte swizzle atom)
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int W_BYTES = TILE_ROWS * BK * 2;          // 16 KB
constexpr int X_BYTES_MAX = 128 * BK * 2;            // room for up to 128 rows of x
constexpr int STAGE_BYTES = W_BYTES + X_BYTES_MAX;
constexpr int TMEM_COLS = 128;
constexpr long long WAIT_LIMIT = 4000000000LL;

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2, EPI_PARTIAL = 3 };

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
// c0 (elements along K) is a multiple of 64, so c0 * 2 bytes is a multiple of 16.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
// K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart (see gemm_tcgen05.cu)
__device__ __forceinline__ unsigned long long smem_desc(const void* p) {
    const unsigned long long addr = smem_u32(p);
    return ((addr & 0x3FFFFull) >> 4) | ((1024ull >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__host__ __device__ constexpr unsigned instr_desc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                     unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }

// 16 consecutive accumulator columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_load16(unsigned taddr, float* v) {
    unsigned r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// grid (W tiles, K splits).  MB: rows of x rounded up to a multiple of 16 (the UMMA N).
// STAGES: 3 (97 KB of shared memory: two blocks per SM, one fills its ring while the other drains its
// accumulator; for wide matrices with many tiles) or 6 (one block per SM with a deep ring; for narrow
// matrices split along K, where a block streams for a long time).
template <int EPI, int STAGES>
__global__ void __launch_bounds__(THREADS)
stream_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   void* __restrict__ out, int M, int MB, int N, int K, int kb_per_split, int up_row_offset,
                   int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], accum_bar;
    __shared__ unsigned tmem_holder;
    __shared__ volatile int give_up;
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    griddep_wait();
    griddep_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    // rows of W behind this tile: 128 consecutive rows, or 64 gate rows and their 64 up rows
    const int rows_per_tile = EPI == EPI_SWIGLU ? 64 : TILE_ROWS;
    const int n0 = tile * rows_per_tile;
    const int num_kb_total = (K + BK - 1) / BK;
    const int kb_begin = split * kb_per_split, kb_end = min(num_kb_total, kb_begin + kb_per_split);
    const int num_kb = max(0, kb_end - kb_begin);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&accum_bar, 1);
        give_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_holder)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = tmem_holder;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer: W does not depend on the previous kernel, x does (already waited above) ----
        const unsigned stage_tx = (unsigned)(W_BYTES + MB * BK * 2);
        for (int i = 0; i < num_kb && !give_up; ++i) {
            const int s = i % STAGES, use = i / STAGES;
            if (!mbar_wait(&empty_bar[s], (use & 1) ^ 1)) { give_up = 1; break; }
            unsigned char* w = smem + s * STAGE_BYTES;
            const int k0 = (kb_begin + i) * BK;
            mbar_arrive_expect_tx(&full_bar[s], stage_tx);
            if (EPI == EPI_SWIGLU) {
                tma_load_2d(w, &map_w, k0, n0, &full_bar[s]);                                   // 64 gate rows
                tma_load_2d(w + 64 * BK * 2, &map_w, k0, up_row_offset + n0, &full_bar[s]);     // their up rows
            } else {
                tma_load_2d(w, &map_w, k0, n0, &full_bar[s]);
            }
            tma_load_2d(w + W_BYTES, &map_x, k0, 0, &full_bar[s]);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        const unsigned idesc = instr_desc(TILE_ROWS, MB);
        for (int i = 0; i < num_kb && !give_up; ++i) {
            const int s = i % STAGES, use = i / STAGES;
            if (!mbar_wait(&full_bar[s], use & 1)) { give_up = 1; break; }
            tc_fence_after();
            const unsigned char* w = smem + s * STAGE_BYTES;
            const unsigned long long adesc = smem_desc(w), bdesc = smem_desc(w + W_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) umma(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
            umma_commit(&empty_bar[s]);
        }
        umma_commit(&accum_bar);
    } else if (warp >= 2) {
        // ---- epilogue: warp w reads TMEM lanes 32 (w % 4) .. + 31; lane = W row of the tile ----
        const bool ok = mbar_wait(&accum_bar, 0);
        if (!ok) give_up = 1;
        tc_fence_after();
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const unsigned lane_addr = tmem_base + ((unsigned)(quarter * 32) << 16);
        float* xch = reinterpret_cast<float*>(smem);              // the ring is idle once the accumulator is complete
        const int pitch = MB + 1;
        if (ok && num_kb > 0) {
            for (int c = 0; c < MB; c += 16) {
                float v[16];
                tmem_load16(lane_addr + c, v);
                if (EPI == EPI_SWIGLU) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) xch[row * pitch + c + j] = v[j];
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = c + j;
                        if (m < M && n0 + row < N) {
                            if (EPI == EPI_BF16) reinterpret_cast<bf16*>(out)[(size_t)m * N + n0 + row] = __float2bfloat16_rn(v[j]);
                            else if (EPI == EPI_F32) reinterpret_cast<float*>(out)[(size_t)m * N + n0 + row] = v[j];
                            else reinterpret_cast<float*>(out)[((size_t)split * M + m) * N + n0 + row] = v[j];
                        }
                    }
                }
            }
        } else if (ok && EPI == EPI_PARTIAL) {
            for (int m = 0; m < M; ++m)
                if (n0 + row < N) reinterpret_cast<float*>(out)[((size_t)split * M + m) * N + n0 + row] = 0.f;
        }
        if (EPI == EPI_SWIGLU) {
            asm volatile("bar.sync 1, 128;\n" ::: "memory");      // the four epilogue warps only
            if (ok) {
                const int I = up_row_offset;                      // output width
                const int t = threadIdx.x - 64, r = t & 63, half = t >> 6;
                const int m_lo = half * (MB / 2), m_hi = m_lo + MB / 2;
                for (int m = m_lo; m < m_hi; ++m) {
                    if (m < M && n0 + r < I) {
                        const float g = xch[r * pitch + m], u = xch[(r + 64) * pitch + m];
                        reinterpret_cast<bf16*>(out)[(size_t)m * I + n0 + r] = __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
                    }
                }
            }
        }
    }
    __syncthreads();
    if (give_up && threadIdx.x == 0 && status) atomicOr(status, FE_STATUS_WAIT_EXPIRED);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
}

// out[m, n] = sum over splits of part[s, m, n], in ascending s.
__global__ void reduce_partials_kernel(const float* __restrict__ part, bf16* __restrict__ out, long long total, int splits) {
    griddep_wait();
    griddep_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < splits; ++s) v += part[(size_t)s * total + i];
        out[i] = __float2bfloat16_rn(v);
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    }
    return fn;
}

int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
    EncodeTiled encode = encode_fn();
    FE_REQUIRE(encode != nullptr, "stream_gemm: cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FE_REQUIRE(rc == CUDA_SUCCESS, "stream_gemm: cuTensorMapEncodeTiled failed with code %d", (int)rc);
    return 0;
}

template <int EPI, int STAGES>
int launch_with(const CUtensorMap& map_w, const CUtensorMap& map_x, void* out, int M, int MB, int N, int K, int tiles,
                int splits, int kb_per_split, int up_row_offset, int* status, cudaStream_t stream) {
    const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
    const cudaError_t err = cudaFuncSetAttribute(stream_gemm_kernel<EPI, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FE_REQUIRE(err == cudaSuccess, "stream_gemm: %s", cudaGetErrorString(err));
    fe::launch(stream_gemm_kernel<EPI, STAGES>, dim3(tiles, splits), THREADS, smem, stream, map_w, map_x, out, M, MB, N, K,
               kb_per_split, up_row_offset, status);
    return fe_check_launch("stream_gemm");
}

template <int EPI>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, void* out, int M, int MB, int N, int K, int tiles, int splits,
           int kb_per_split, int up_row_offset, int* status, cudaStream_t stream) {
    if (tiles * splits > 2 * fe_sm_count())
        return launch_with<EPI, 3>(map_w, map_x, out, M, MB, N, K, tiles, splits, kb_per_split, up_row_offset, status, stream);
    return launch_with<EPI, 6>(map_w, map_x, out, M, MB, N, K, tiles, splits, kb_per_split, up_row_offset, status, stream);
}

}  // namespace

// How many K splits fe_stream_gemm_tcgen05 uses for a plain bfloat16 product, and the bytes of
// float scratch it then needs (0 for one split).
extern "C" int fe_stream_gemm_splits(int N, int K) {
    const int tiles = (N + TILE_ROWS - 1) / TILE_ROWS, num_kb = (K + BK - 1) / BK;
    int splits = (fe_sm_count() + tiles / 2) / tiles;
    if (splits > num_kb / 4) splits = num_kb / 4;
    return splits < 1 ? 1 : splits;
}

// epilogue 0: bfloat16 [M, N]; 1: float [M, N]; 2: SwiGLU, W is [N = 2 I, K], out bfloat16 [M, I].
// ``scratch``: float [splits, M, N] when fe_stream_gemm_splits(N, K) > 1 and the epilogue is 0.
extern "C" int fe_stream_gemm_tcgen05(const void* x, const void* W, void* out, void* scratch, int M, int N, int K,
                                      int epilogue, int* status, cudaStream_t stream) {
    FE_REQUIRE(M >= 1 && M <= 128, "stream_gemm: %d rows; this kernel takes 1 to 128", M);
    FE_REQUIRE(N >= 1 && K >= 8 && K % 8 == 0, "stream_gemm: K = %d must be a positive multiple of 8", K);
    FE_REQUIRE((((size_t)x | (size_t)W) & 15) == 0, "stream_gemm: operands must be 16-byte aligned");
    const int MB = (M + 15) / 16 * 16;
    const int num_kb = (K + BK - 1) / BK;
    CUtensorMap map_w, map_x;
    if (make_map(&map_x, x, M, K, MB)) return 1;
    if (epilogue == EPI_SWIGLU) {
        FE_REQUIRE(N % 2 == 0, "stream_gemm: SwiGLU needs an even number of weight rows, got %d", N);
        const int I = N / 2;
        if (make_map(&map_w, W, N, K, 64)) return 1;
        return launch<EPI_SWIGLU>(map_w, map_x, out, M, MB, N, K, (I + 63) / 64, 1, num_kb, I, status, stream);
    }
    if (make_map(&map_w, W, N, K, TILE_ROWS)) return 1;
    const int tiles = (N + TILE_ROWS - 1) / TILE_ROWS;
    if (epilogue == EPI_F32) return launch<EPI_F32>(map_w, map_x, out, M, MB, N, K, tiles, 1, num_kb, 0, status, stream);
    FE_REQUIRE(epilogue == EPI_BF16, "stream_gemm: unknown epilogue %d", epilogue);
    const int splits = fe_stream_gemm_splits(N, K);
    if (splits == 1) return launch<EPI_BF16>(map_w, map_x, out, M, MB, N, K, tiles, 1, num_kb, 0, status, stream);
    FE_REQUIRE(scratch != nullptr, "stream_gemm: %d K splits need scratch memory", splits);
    const int per = (num_kb + splits - 1) / splits;
    if (launch<EPI_PARTIAL>(map_w, map_x, scratch, M, MB, N, K, tiles, splits, per, 0, status, stream)) return 1;
    const long long total = (long long)M * N;
    const long long most = 8LL * fe_sm_count();
    const int blocks = (int)((total + 255) / 256 < most ? (total + 255) / 256 : most);
    fe::launch(reduce_partials_kernel, blocks, 256, 0, stream, (const float*)scratch, (bf16*)out, total, splits);
    return fe_check_launch("stream_gemm reduce");
}
