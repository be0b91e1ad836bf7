// y[M, N] = x[M, K] . W[N, K]^T on the fifth-generation tensor cores: tcgen05.mma with the
// accumulator in tensor memory (TMEM), operands brought to shared memory by TMA tensor copies
// (128-byte swizzle), completion tracked by mbarriers.  bfloat16 inputs, float accumulation.
//
// Blocks are persistent: one per SM, each walks over output tiles (row tiles fastest, so blocks
// that run together share their rows of W: W is larger than L2 and then comes from HBM once).
// Warp 0 (one lane) is the TMA producer, warp 1 (one lane) issues the MMAs and owns the TMEM
// allocation, warps 2..5 are the epilogue: each reads its quarter of the accumulator's lanes with
// tcgen05.ld and writes the rows out.  The accumulator is double-buffered in TMEM (2 x 256
// columns), so the epilogue of one tile runs under the MMAs of the next.  UMMA shape 128 x 256 x 16.
//   plain epilogue:  a 128 x 256 output tile, bfloat16
//   SwiGLU epilogue: W is [2I, K] (gate rows, then up rows); the block loads 128 gate rows and
//                    their 128 up rows as one 256-row B tile, so accumulator columns j and 128 + j
//                    belong to output column j: out = silu(gate) * up, a 128 x 128 tile of bfloat16 [M, I].
// The reference runs these products through cuBLAS (inference/models/qwen2.py:99-101,129-130).
//
// Every wait on an mbarrier is bounded (about two seconds): when it runs out the thread records it
// in the status word and raises a flag that makes every role leave its loop; all threads still
// meet at the final barrier, tensor memory is freed, the block returns.  No cluster launch, no
// multicast.
#include <cuda.h>

#include "common.cuh"

using namespace fe;

namespace {

constexpr int BM = 128;             // rows of the output tile = UMMA M
constexpr int BK = 64;              // k elements per stage: 128 bytes, one swizzle atom wide
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int THREADS = 192;
constexpr long long WAIT_LIMIT = 4000000000LL;      // clock cycles

enum { EPI_BF16 = 0, EPI_SWIGLU = 2 };

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
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

// 2-D tiled TMA load: coordinates (c0 = element along K, c1 = row).  c0 * 2 bytes is always a
// multiple of 128 here, so the 16-byte rule on the innermost coordinate holds.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1,
                                            unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows 128 bytes apart, groups
// of 8 rows 1024 bytes apart.
__device__ __forceinline__ unsigned long long smem_desc(const void* p) {
    const unsigned long long addr = smem_u32(p);
    return ((addr & 0x3FFFFull) >> 4)          // start address
           | (0ull << 16)                      // leading-dimension byte offset: unused for swizzled K-major
           | ((1024ull >> 4) << 32)            // stride-dimension byte offset between 8-row groups
           | (1ull << 46)                      // descriptor version of this architecture
           | (2ull << 61);                     // 128-byte swizzle
}

// Instruction descriptor: float accumulator, bfloat16 A and B, both K-major, M x N tile.
__host__ __device__ constexpr unsigned instr_desc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

__device__ __forceinline__ void umma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                     unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on ``bar`` once every MMA issued so far by this thread has finished (and read its operands).
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }

// 32 consecutive accumulator columns of this thread's TMEM lane.
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

template <int NCOLS> __device__ __forceinline__ void tmem_alloc(unsigned* holder) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(holder)), "n"(NCOLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
template <int NCOLS> __device__ __forceinline__ void tmem_dealloc(unsigned taddr) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "n"(NCOLS) : "memory");
}

// The order of the tiles: row tiles fastest inside a panel of PANEL row tiles, the panels one after the other.  Blocks
// that run together then share their rows of W (W comes from HBM once per panel), and the rows of x that a panel
// needs (4,096 x K) stay in L2 while all of W passes by; with every row tile of a long prompt in flight at once
// (8,192 rows) the output being written pushes x out of L2 between two column tiles.  Gate/up with SwiGLU under a
// long-running load, 8,192 rows: 7B widths 1.80 -> 1.74 ms, 14B widths 2.07 -> 1.79 ms (panels of 8 / 16 / 24 row
// tiles: 1.93 / 1.78 / 1.75 and 1.95 / 1.82 / 1.81); up to 4,096 rows nothing changes.
constexpr int PANEL = 32;
__device__ __forceinline__ void tile_origin(int t, int m_tiles, int n_tiles, int out_cols, int& m0, int& n0) {
    const int per_panel = PANEL * n_tiles;
    const int panel = t / per_panel, within = t - panel * per_panel;
    const int rows_here = min(PANEL, m_tiles - panel * PANEL);      // the last panel may hold fewer row tiles
    m0 = (panel * PANEL + within % rows_here) * BM;
    n0 = (within / rows_here) * out_cols;
}

constexpr int BN = 256;             // accumulator columns of one tile = UMMA N
constexpr int ACC_BUFFERS = 2;

template <int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    bf16* __restrict__ out, int M, int N_out, int K, int up_row_offset, int m_tiles, int n_tiles,
                    int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES];
    __shared__ __align__(8) unsigned long long acc_full[ACC_BUFFERS], acc_empty[ACC_BUFFERS];
    __shared__ unsigned tmem_holder;
    __shared__ volatile int give_up;
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int OUT_COLS = EPI == EPI_SWIGLU ? 128 : 256;      // output columns per tile
    // the dynamic segment is aligned by hand: the swizzle atoms want 1024 bytes
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    griddep_wait();
    griddep_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (K + BK - 1) / BK;
    const int total_tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < ACC_BUFFERS; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        give_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) tmem_alloc<ACC_BUFFERS * BN>(&tmem_holder);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = tmem_holder;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        int kbg = 0;                                   // k blocks issued so far, over all tiles
        for (int t = blockIdx.x; t < total_tiles && !give_up; t += gridDim.x) {
            int m0, n0;
            tile_origin(t, m_tiles, n_tiles, OUT_COLS, m0, n0);
            for (int kb = 0; kb < num_kb; ++kb, ++kbg) {
                const int s = kbg % STAGES, use = kbg / STAGES;
                if (!mbar_wait(&empty_bar[s], (use & 1) ^ 1)) { give_up = 1; break; }   // parity 1 passes at once at the start
                unsigned char* a = smem + s * STAGE_BYTES;
                unsigned char* b = a + A_BYTES;
                mbar_arrive_expect_tx(&full_bar[s], STAGE_BYTES);
                tma_load_2d(a, &map_a, kb * BK, m0, &full_bar[s]);
                tma_load_2d(b, &map_b, kb * BK, n0, &full_bar[s]);                      // 128 rows of W (gate rows for SwiGLU)
                tma_load_2d(b + 128 * BK * 2, &map_b, kb * BK, (EPI == EPI_SWIGLU ? up_row_offset + n0 : n0 + 128),
                            &full_bar[s]);                                              // the next 128 rows, or their up rows
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        constexpr unsigned idesc = instr_desc(BM, BN);
        int kbg = 0, i = 0;
        for (int t = blockIdx.x; t < total_tiles && !give_up; t += gridDim.x, ++i) {
            const int buf = i & 1;
            if (!mbar_wait(&acc_empty[buf], ((i >> 1) & 1) ^ 1)) { give_up = 1; break; }     // the epilogue has drained it
            tc_fence_after();
            const unsigned acc = tmem_base + buf * BN;
            for (int kb = 0; kb < num_kb; ++kb, ++kbg) {
                const int s = kbg % STAGES, use = kbg / STAGES;
                if (!mbar_wait(&full_bar[s], use & 1)) { give_up = 1; break; }
                tc_fence_after();
                const unsigned char* a = smem + s * STAGE_BYTES;
                const unsigned long long adesc = smem_desc(a), bdesc = smem_desc(a + A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    // 16 elements along K = 32 bytes inside the swizzle atom: +2 in the address field
                    umma(acc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&empty_bar[s]);            // the stage is free once these MMAs have read it
            }
            umma_commit(&acc_full[buf]);               // arrives even after a failed wait, so the epilogue is released
        }
    } else if (warp >= 2) {
        // ---- epilogue: warp w may read TMEM lanes 32 (w % 4) .. + 31 ----
        const int quarter = warp & 3;
        int i = 0;
        for (int t = blockIdx.x; t < total_tiles && !give_up; t += gridDim.x, ++i) {
            const int buf = i & 1;
            int m0, n0;
            tile_origin(t, m_tiles, n_tiles, OUT_COLS, m0, n0);
            if (!mbar_wait(&acc_full[buf], (i >> 1) & 1)) { give_up = 1; break; }
            tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
            const unsigned lane_addr = tmem_base + buf * BN + ((unsigned)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < OUT_COLS; c += 32) {
                float v[32];
                tmem_load32(lane_addr + c, v);
                if (EPI == EPI_SWIGLU) {
                    float u[32];
                    tmem_load32(lane_addr + 128 + c, u);
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = v[j] / (1.f + expf(-v[j])) * u[j];
                }
                if (row < M) {
                    bf16* dst = out + (size_t)row * N_out + n0 + c;
                    if (n0 + c + 32 <= N_out && (N_out & 7) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) store8<bf16>(dst + j, v + j);
                    } else {
                        for (int j = 0; j < 32; ++j)
                            if (n0 + c + j < N_out) dst[j] = __float2bfloat16_rn(v[j]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);       // this warp has read its quarter of the buffer
        }
    }
    __syncthreads();
    if (give_up && threadIdx.x == 0 && status) atomicOr(status, FE_STATUS_WAIT_EXPIRED);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc<ACC_BUFFERS * BN>(tmem_base);
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

// A [rows, cols] bfloat16 row-major matrix as a 2-D tensor map with boxes of box_rows x 64 elements.
int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
    EncodeTiled encode = encode_fn();
    FE_REQUIRE(encode != nullptr, "gemm_tcgen05: cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FE_REQUIRE(rc == CUDA_SUCCESS, "gemm_tcgen05: cuTensorMapEncodeTiled failed with code %d", (int)rc);
    return 0;
}

template <int EPI>
int launch(const void* x, const void* W, void* out, int M, int N, int K, int* status, cudaStream_t stream) {
    const int n_out = EPI == EPI_SWIGLU ? N / 2 : N;
    constexpr int OUT_COLS = EPI == EPI_SWIGLU ? 128 : 256;
    CUtensorMap map_a, map_b;
    if (make_map(&map_a, x, M, K, BM)) return 1;
    if (make_map(&map_b, W, N, K, 128)) return 1;
    const size_t smem = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 1024;
    cudaError_t err = cudaFuncSetAttribute(gemm_tcgen05_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FE_REQUIRE(err == cudaSuccess, "gemm_tcgen05: %s", cudaGetErrorString(err));
    const int sms = fe_sm_count();
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (n_out + OUT_COLS - 1) / OUT_COLS;
    const long long total = (long long)m_tiles * n_tiles;
    const int blocks = (int)(total < sms ? total : sms);        // one persistent block per SM
    fe::launch(gemm_tcgen05_kernel<EPI>, blocks, THREADS, smem, stream, map_a, map_b, (bf16*)out, M, n_out, K, n_out,
               m_tiles, n_tiles, status);
    return fe_check_launch("gemm_tcgen05");
}

}  // namespace

// epilogue 0: out bfloat16 [M, N]; 2: SwiGLU, W is [N = 2 I, K] (gate rows, then up rows), out bfloat16 [M, I].
extern "C" int fe_gemm_tcgen05(const void* x, const void* W, void* out, int M, int N, int K, int epilogue, int* status,
                               cudaStream_t stream) {
    FE_REQUIRE(M >= 1 && N >= 1 && K >= 8, "gemm_tcgen05: bad sizes M=%d N=%d K=%d", M, N, K);
    FE_REQUIRE(K % 8 == 0, "gemm_tcgen05: K = %d must be a multiple of 8 (rows must start on 16-byte boundaries)", K);
    FE_REQUIRE((((size_t)x | (size_t)W) & 15) == 0, "gemm_tcgen05: operands must be 16-byte aligned");
    if (epilogue == EPI_BF16) return launch<EPI_BF16>(x, W, out, M, N, K, status, stream);
    if (epilogue == EPI_SWIGLU) {
        FE_REQUIRE(N % 2 == 0, "gemm_tcgen05: SwiGLU needs an even number of weight rows, got %d", N);
        return launch<EPI_SWIGLU>(x, W, out, M, N, K, status, stream);
    }
    FE_REQUIRE(false, "gemm_tcgen05: unknown epilogue %d", epilogue);
}
