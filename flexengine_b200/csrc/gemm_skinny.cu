// y[M, N] = x[M, K] . W[N, K]^T for a handful of rows (decode): the product is a stream of the
// weight matrix, so the kernel is built around reading W once at full HBM speed.
//
// One block takes 16 rows of W (swap-AB: the rows of W are the 16 rows of mma.sync.m16n8k16,
// the batch is its 8 columns).  Its eight warps split K; every lane reads 32 contiguous bytes
// of "its" two W rows per step straight into MMA fragments.  The fragment layout wants
// k = {2t, 2t+1, 2t+8, 2t+9} per lane; since a dot product does not care in which order k is
// summed, lane t instead takes the 16 contiguous elements k0 + 16t .. +15 of a 64-wide step and
// the activations are read with the same pattern, so both operands are 16-byte loads.  The eight
// partial sums of a block are added in shared memory in a fixed order (deterministic).
//
// Epilogues: bfloat16 output; float output (vocabulary projection); SwiGLU, where a block pairs
// 8 gate rows with their 8 up rows of a [2I, K] matrix and writes silu(gate) * up; the fused
// query/key/value epilogue; and the residual epilogue, which ends a branch of a layer and begins
// the norm that follows it (below).
// The reference runs these products through cuBLAS (inference/models/qwen2.py:99-101,129-135).
//
// Residual add and RMSNorm without a kernel of their own.  In a decode step a norm moves a few kilobytes
// between two products that stream hundreds of megabytes; as a kernel it costs a launch and a few trips to
// memory.  Instead the product that ends a branch (output projection, down projection) adds its result to the
// float residual stream in its epilogue, writes the new residual times the next norm's weight as bfloat16,
// and leaves each block's share of the rows' sums of squares in a small table; the product that consumes the
// norm (query/key/value, gate/up) adds the table up in a fixed order while its first weights are on their way
// and multiplies its accumulators by rsqrt(mean square + eps): a row's scale is a factor of every term of its
// dot products, so it may be applied after them.
#define FE_PDL_CLASS 1      // FE_PDL_STREAMING_GEMM
#include "common.cuh"

using namespace fe;

namespace {

constexpr int WARPS_USUAL = 8, WARPS_NARROW = 16;
constexpr int KSTEP = 64;       // k elements per warp step (4 MMAs)

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2, EPI_QKV = 3, EPI_RESID = 4 };

// The residual epilogue: out[m][n] is not written; residual[m][n] += product, scaled[m][n] = bfloat16(residual *
// norm_weight[n]), sumsq[tile][m] = this tile's share of the sum of squares of row m of the new residual.
struct ResidEpilogue {
    float* residual;            // [M, N] float, updated in place (every element by the one block that owns it)
    const float* norm_weight;   // [N]
    bf16* scaled;               // [M, N]
    float* sumsq;               // [tiles of 16 columns][8]
};

// What a consumer of such a norm gets instead of normalised rows: the table of partial sums of squares.
// ``next``: memory that the kernel after this one streams first (may be null): as a block leaves its loop it asks for its
// share of the first ``next_bytes`` to be brought into L2, so that the next kernel's first loads, which would
// otherwise go out to an idle memory system after the launch gap, are met there.
struct RowScale {
    const float* sumsq;         // [tiles][8] or nullptr: the input is normalised already
    int tiles;
    float eps;
    int width;                  // elements of a row (the mean is over them)
    const void* next;
    long long next_bytes;
};

// What the fused query/key/value epilogue needs beside the product: bias, rotary table, where the
// new keys and values go in the paged cache (see elementwise.cu for the unfused form of the same).
struct QkvEpilogue {
    const float* bias;          // [(nq + 2 nkv) d] or nullptr
    const int* positions;       // [M]
    const float* inv_freq;      // [d / 2]
    const int* slot_mapping;    // [M] or nullptr (no cache write)
    bf16* kc;
    bf16* vc;
    int nq, nkv, d, ps;
    long long num_slots;
    int* status;
};

// Tile ``tile`` of the fused epilogue: rotated heads (queries and keys) pair feature j with its
// rotation partner j + d/2 in accumulator rows g and g + 8, so one thread holds both; value heads
// take 16 consecutive features.
__device__ __forceinline__ void qkv_tile_rows(const QkvEpilogue& e, int tile, int g, int& row0, int& row1, int& head,
                                              int& j0) {
    const int half = e.d >> 1;
    const int rot_tiles = (e.nq + e.nkv) * (half >> 3);
    if (tile < rot_tiles) {
        head = tile / (half >> 3);
        j0 = (tile - head * (half >> 3)) << 3;
        row0 = head * e.d + j0 + g;
        row1 = row0 + half;
    } else {
        const int t = tile - rot_tiles;
        head = e.nq + e.nkv + t / (e.d >> 4);
        j0 = (t % (e.d >> 4)) << 4;
        row0 = head * e.d + j0 + g;
        row1 = row0 + 8;
    }
}

__device__ __forceinline__ uint4 ld_stream(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_keep(const bf16* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

__device__ __forceinline__ void mma16816(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// RT: 16-row tiles of W per block (2 for wide matrices: fewer, longer-lived blocks that fill the
//     GPU in whole rounds, and the activations are read once for both tiles)
// PF: k steps whose loads go out together before their math (bytes in flight per lane = RT * PF * 64)
// WARPS: warps that split K (8; 16 for a narrow matrix with a long K, whose few blocks leave SMs empty: the blocks
//     it has then keep twice as many loads in flight)
template <int NT, int EPI, int RT, int PF, int WARPS>
// blocks an SM: three of the light variant (80 registers a thread), two of the others with eight warps (128)
__global__ void __launch_bounds__(WARPS * 32, WARPS == 16 ? 1 : (NT == 1 && RT == 1 && PF == 2) ? 3 : NT == 1 ? 2 : 1)
skinny_gemm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, void* __restrict__ out, int M, int N, int K,
                   int I, const QkvEpilogue qkv, const ResidEpilogue resid, const RowScale scale, const int units) {
    __shared__ float red[WARPS][RT * NT * 8 * 16];
    __shared__ float scale_part[WARPS * 4][8];     // partial sums of squares: [share of the tiles][row]
    extern __shared__ __align__(16) float scale_table[];      // [scale.tiles][8], when the input rows are to be scaled
    __shared__ float row_scale[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // A block takes the units (RT tiles each) blockIdx.x, blockIdx.x + gridDim.x, ...: one, unless the matrix has more
    // units than blocks fit the device at once; then the grid is one resident round of blocks that stay, so that the
    // table of the rows' scales is fetched and added up once a block and not once a unit.
    // rows of W behind accumulator rows g and g + 8 of tile r of unit u, as pointers to this lane's part of a k step
    auto weight_rows = [&](int u, const bf16* (&w0)[RT], const bf16* (&w1)[RT]) {
        const int first = u * (EPI == EPI_SWIGLU ? 8 : 16) * RT;
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            int row0, row1;
            if (EPI == EPI_SWIGLU) {
                row0 = min(first + r * 8 + g, I - 1);       // gate row
                row1 = I + row0;                            // its up row
            } else if (EPI == EPI_QKV) {
                int head, j0;
                qkv_tile_rows(qkv, u, g, row0, row1, head, j0);
            } else {
                row0 = min(first + r * 16 + g, N - 1);
                row1 = min(first + r * 16 + g + 8, N - 1);
            }
            w0[r] = W + (size_t)row0 * K + 16 * t;
            w1[r] = W + (size_t)row1 * K + 16 * t;
        }
    };
    const bf16* xr[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) xr[nt] = nt * 8 + g < M ? x + (size_t)(nt * 8 + g) * K + 16 * t : nullptr;
    // every warp owns one contiguous eighth of K (whole steps), so that the PF steps it loads together
    // are one contiguous run of each row in memory; the loads of PF steps go out together, then their math
    const int steps = K / KSTEP;
    const int per_warp = (steps + WARPS - 1) / WARPS;
    const int s_begin = warp * per_warp, s_end = min(steps, s_begin + per_warp);
    // the weights of PF steps: loaded together, then used; the first PF steps of a block's NEXT unit are asked for
    // before the epilogue of the one that ends, so that the block's loads do not pause while it adds up and writes
    uint4 a0[PF][RT][2], a1[PF][RT][2];
    auto load_weights = [&](const bf16* const (&w0)[RT], const bf16* const (&w1)[RT], int s) {
#pragma unroll
        for (int p = 0; p < PF; ++p) {
            const int sp = s + p;
            if (sp < s_end) {
                const size_t k = (size_t)sp * KSTEP;
#pragma unroll
                for (int r = 0; r < RT; ++r) {
                    a0[p][r][0] = ld_stream(w0[r] + k); a0[p][r][1] = ld_stream(w0[r] + k + 8);
                    a1[p][r][0] = ld_stream(w1[r] + k); a1[p][r][1] = ld_stream(w1[r] + k + 8);
                }
            }
        }
    };
    constexpr bool STAYS = RT > 1;              // only the two-tile blocks of a wide matrix are launched to stay
    bool ahead = false;                         // the first steps of this unit are in the registers already
    // A block takes the units (RT tiles each) blockIdx.x, blockIdx.x + gridDim.x, ...: one, unless the matrix has more
    // units than blocks fit the device at once; then the grid is one resident round of blocks that stay, so that the
    // table of the rows' scales is fetched and added up once a block and not once a unit.
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
    const bool first_unit = unit == (int)blockIdx.x, last_unit = unit + (int)gridDim.x >= units;
    const int n0 = unit * (EPI == EPI_SWIGLU ? 8 : 16) * RT;
    const bf16* w0[RT];
    const bf16* w1[RT];
    weight_rows(unit, w0, w1);

    float acc[RT][NT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[r][nt][0] = acc[r][nt][1] = acc[r][nt][2] = acc[r][nt][3] = 0.f;

    for (int s = s_begin; s < s_end; s += PF) {
        uint4 b[PF][NT][2];
        if (!(STAYS && ahead && s == s_begin)) load_weights(w0, w1, s);
        // the weights above depend on no kernel; the activations below are the previous kernel's
        // output, so the first batch of weight loads is already in flight while that kernel ends
        if (s == s_begin && first_unit) {
            griddep_wait();
            // the table of the rows' sums of squares is needed in the epilogue: asynchronous copies bring it into
            // shared memory meanwhile, so that no thread waits for it now and no block waits for memory at its end
            if (scale.sumsq != nullptr) {
                for (int chunk = threadIdx.x; chunk < scale.tiles * 2; chunk += WARPS * 32) {
                    const unsigned dst = (unsigned)__cvta_generic_to_shared(scale_table + chunk * 4);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(scale.sumsq + (size_t)chunk * 4));
                }
                asm volatile("cp.async.commit_group;\n" ::);
            }
        }
#pragma unroll
        for (int p = 0; p < PF; ++p) {
            const int sp = s + p;
            if (sp < s_end) {
                const size_t k = (size_t)sp * KSTEP;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    if (xr[nt]) { b[p][nt][0] = ld_keep(xr[nt] + k); b[p][nt][1] = ld_keep(xr[nt] + k + 8); }
                    else { b[p][nt][0] = make_uint4(0, 0, 0, 0); b[p][nt][1] = make_uint4(0, 0, 0, 0); }
                }
            }
        }
#pragma unroll
        for (int p = 0; p < PF; ++p) {
            if (s + p < s_end) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int r = 0; r < RT; ++r) {
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            mma16816(acc[r][nt], a0[p][r][h].x, a1[p][r][h].x, a0[p][r][h].y, a1[p][r][h].y,
                                     b[p][nt][h].x, b[p][nt][h].y);
                            mma16816(acc[r][nt], a0[p][r][h].z, a1[p][r][h].z, a0[p][r][h].w, a1[p][r][h].w,
                                     b[p][nt][h].z, b[p][nt][h].w);
                        }
                    }
                }
            }
        }
    }
    ahead = false;
    if (STAYS && !last_unit) {
        const bf16* nw0[RT];
        const bf16* nw1[RT];
        weight_rows(unit + gridDim.x, nw0, nw1);
        load_weights(nw0, nw1, s_begin);
        ahead = true;
    }
    if (last_unit) {
        griddep_launch_dependents();           // the next kernel may start its own first loads as this one's blocks end
        if (scale.next != nullptr)
            prefetch_l2_share(scale.next, scale.next_bytes, (long long)blockIdx.x * (WARPS * 32) + threadIdx.x,
                              (long long)gridDim.x * (WARPS * 32));
    }
    if (s_begin >= s_end && first_unit) {      // a warp without work has not waited yet, nor started its copies
        griddep_wait();
        if (scale.sumsq != nullptr) {
            for (int chunk = threadIdx.x; chunk < scale.tiles * 2; chunk += WARPS * 32) {
                const unsigned dst = (unsigned)__cvta_generic_to_shared(scale_table + chunk * 4);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(scale.sumsq + (size_t)chunk * 4));
            }
            asm volatile("cp.async.commit_group;\n" ::);
        }
    }
    // accumulator (tile r, row g + 8 (e >> 1), batch column nt * 8 + 2t + (e & 1)) -> red[warp][(r, column, row)]
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                red[warp][(r * NT * 8 + nt * 8 + 2 * t + (e & 1)) * 16 + g + 8 * (e >> 1)] = acc[r][nt][e];
    if (scale.sumsq != nullptr && first_unit) asm volatile("cp.async.wait_all;\n" ::: "memory");
    __syncthreads();
    if (scale.sumsq != nullptr && first_unit) {
        // thread = (row m, one of WARPS * 4 shares of the tiles): a thread adds its tiles in ascending order; the
        // shares are then added in a fixed order
        const int m = threadIdx.x & 7, share = threadIdx.x >> 3;
        float sum = 0.f;
        for (int tile = share; tile < scale.tiles; tile += WARPS * 4) sum += scale_table[tile * 8 + m];
        scale_part[share][m] = sum;
        __syncthreads();
        if (threadIdx.x < 8) {
            float sum = 0.f;
#pragma unroll
            for (int share = 0; share < WARPS * 4; ++share) sum += scale_part[share][threadIdx.x];
            row_scale[threadIdx.x] = rsqrtf(sum / (float)scale.width + scale.eps);
        }
        __syncthreads();
    }
    if (EPI == EPI_QKV) {
        // bias, rotation by the token's position, and the write of new keys and values to their pages
        int row0, row1, head, j0;
        qkv_tile_rows(qkv, unit, 0, row0, row1, head, j0);
        const bool rotated = head < qkv.nq + qkv.nkv;
        const int partner = rotated ? qkv.d >> 1 : 8;
        for (int idx = threadIdx.x; idx < NT * 8 * 8; idx += WARPS * 32) {
            const int m = idx >> 3, r = idx & 7;
            if (m >= M) continue;
            float a = 0.f, c = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) { a += red[w][m * 16 + r]; c += red[w][m * 16 + r + 8]; }
            if (scale.sumsq != nullptr) { a *= row_scale[m]; c *= row_scale[m]; }
            const int f0 = row0 + r, f1 = f0 + partner;              // features of the two values
            if (qkv.bias) { a += qkv.bias[f0]; c += qkv.bias[f1]; }
            if (rotated) {
                float sn, cs;
                sincosf((float)qkv.positions[m] * qkv.inv_freq[j0 + r], &sn, &cs);
                const float ra = a * cs - c * sn, rc = c * cs + a * sn;
                a = ra; c = rc;
            }
            const bf16 ba = __float2bfloat16_rn(a), bc = __float2bfloat16_rn(c);
            bf16* o = reinterpret_cast<bf16*>(out) + (size_t)m * N;
            o[f0] = ba; o[f1] = bc;
            if (head >= qkv.nq && qkv.slot_mapping) {
                const long long slot = qkv.slot_mapping[m];
                if (slot >= qkv.num_slots) {
                    if (qkv.status) atomicOr(qkv.status, FE_STATUS_BAD_SLOT);
                } else if (slot >= 0) {
                    const bool is_k = head < qkv.nq + qkv.nkv;
                    const int kvh = is_k ? head - qkv.nq : head - qkv.nq - qkv.nkv;
                    bf16* dst = (is_k ? qkv.kc : qkv.vc) +
                                (((slot / qkv.ps) * qkv.nkv + kvh) * qkv.ps + (slot % qkv.ps)) * qkv.d;
                    dst[f0 - head * qkv.d] = ba;
                    dst[f1 - head * qkv.d] = bc;
                }
            }
        }
    } else if (EPI == EPI_SWIGLU) {
        for (int idx = threadIdx.x; idx < RT * NT * 8 * 8; idx += WARPS * 32) {
            const int r = idx / (NT * 64), rest = idx - r * (NT * 64);
            const int m = rest >> 3, row = rest & 7;
            const int n = n0 + r * 8 + row;
            if (m >= M || n >= I) continue;
            float gate = 0.f, up = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                gate += red[w][(r * NT * 8 + m) * 16 + row];
                up += red[w][(r * NT * 8 + m) * 16 + row + 8];
            }
            if (scale.sumsq != nullptr) { gate *= row_scale[m]; up *= row_scale[m]; }
            reinterpret_cast<bf16*>(out)[(size_t)m * I + n] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
        }
    } else if (EPI == EPI_RESID) {
        // NT == 1: idx = (tile r, row m of the batch, column of the tile); the 16 columns of a (tile, row) sit in
        // 16 consecutive lanes, which add their squares up with shuffles
        for (int idx = threadIdx.x; idx < RT * 128; idx += WARPS * 32) {
            const int r = idx >> 7, m = (idx >> 4) & 7, row = idx & 15;
            const int n = n0 + r * 16 + row;
            float square = 0.f;
            if (m < M && n < N) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) v += red[w][(r * 8 + m) * 16 + row];
                if (scale.sumsq != nullptr) v *= row_scale[m];
                const size_t at = (size_t)m * N + n;
                const float sum = resid.residual[at] + v;
                resid.residual[at] = sum;
                resid.scaled[at] = __float2bfloat16_rn(sum * resid.norm_weight[n]);
                square = sum * sum;
            }
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) square += __shfl_xor_sync(0xffffffffu, square, o);
            const int tile = unit * RT + r;
            if (row == 0 && tile * 16 < N) resid.sumsq[(size_t)tile * 8 + m] = square;
        }
    } else {
        for (int idx = threadIdx.x; idx < RT * NT * 8 * 16; idx += WARPS * 32) {
            const int r = idx / (NT * 128), rest = idx - r * (NT * 128);
            const int m = rest >> 4, row = rest & 15;
            const int n = n0 + r * 16 + row;
            if (m >= M || n >= N) continue;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) v += red[w][(r * NT * 8 + m) * 16 + row];
            if (scale.sumsq != nullptr) v *= row_scale[m];
            if (EPI == EPI_F32) reinterpret_cast<float*>(out)[(size_t)m * N + n] = v;
            else reinterpret_cast<bf16*>(out)[(size_t)m * N + n] = __float2bfloat16_rn(v);
        }
    }
    if (!last_unit) __syncthreads();           // the next unit's partial sums go where these were read
    }
}

template <int EPI>
int launch(const void* x, const void* W_, void* out, int M, int N, int K, int I, cudaStream_t stream,
           const QkvEpilogue& qkv = QkvEpilogue{}, const ResidEpilogue& resid = ResidEpilogue{}, const RowScale& scale = RowScale{}) {
    const int tiles = EPI == EPI_SWIGLU ? (I + 7) / 8 : (N + 15) / 16;
    // Three one-tile blocks are resident on an SM (80 registers a thread), two of the others (120 to 128).  A matrix
    // with more tiles than one round of one-tile blocks takes two tiles a block: a few blocks over the round would
    // run alone after it (448 tiles: 15.9 -> 13.6 us).  A narrow one, whose blocks are all resident at once even two
    // to an SM: every warp sends twice as many loads ahead, which halves the number of round trips to memory.
    const int sms = fe_sm_count();
    const size_t table_bytes = scale.sumsq != nullptr ? (size_t)scale.tiles * 8 * sizeof(float) : 0;
    const bool wide = EPI != EPI_QKV && tiles > 3 * sms;
    const bool deep = !wide && tiles <= 2 * sms;
    const int units = wide ? (tiles + 1) / 2 : tiles;
    // The two-tile blocks of a wide matrix stay for one unit after the other: one resident round of them (two an SM).
    // The gate/up product of a 3,584-wide model with rows on their way through a norm: 47.6 -> 44.0 us (2,368 tiles:
    // four units a block; the rows' scales once a block, the next unit's first loads under the epilogue); the
    // vocabulary product (9,504 tiles): 164 -> 160 us.  Results are the same bit for bit.
    const int blocks = wide && units > 2 * sms ? 2 * sms : units;
    // fewer blocks than SMs, and at least one round of loads (four steps) for each of sixteen warps
    const bool narrow = (EPI == EPI_BF16 || EPI == EPI_F32 || EPI == EPI_RESID) && M <= 8 && tiles <= sms && K / KSTEP >= 4 * WARPS_NARROW;
#define FE_SKINNY(NT, RT, PF, W) \
    fe::launch(skinny_gemm_kernel<NT, EPI, RT, PF, W>, blocks, W * 32, table_bytes, stream, (const bf16*)x, (const bf16*)W_, out, M, N, K, I, qkv, resid, scale, units)
    if (narrow) FE_SKINNY(1, 1, 4, WARPS_NARROW);
    else if (EPI == EPI_RESID && M > 8) return 1;          // refused by the entry point already
    else if (M <= 8) { if (wide) FE_SKINNY(1, 2, 2, WARPS_USUAL); else if (deep) FE_SKINNY(1, 1, 4, WARPS_USUAL); else FE_SKINNY(1, 1, 2, WARPS_USUAL); }
    else { if (wide) FE_SKINNY(2, 2, 2, WARPS_USUAL); else if (deep) FE_SKINNY(2, 1, 4, WARPS_USUAL); else FE_SKINNY(2, 1, 2, WARPS_USUAL); }
#undef FE_SKINNY
    return fe_check_launch("skinny_gemm");
}

}  // namespace

// The input rows' scales, when the input is a residual times a norm's weight and not yet divided by its root mean
// square (see the top of this file): ``sumsq`` [sumsq_tiles][8] is the table the residual epilogue left.
static int check_scale(const char* what, const float* sumsq, int sumsq_tiles, int M, int K) {
    if (sumsq == nullptr) return 0;
    FE_REQUIRE(M <= 8, "%s: rows are scaled from a table of sums of squares for up to 8 rows, got %d", what, M);
    FE_REQUIRE(sumsq_tiles == (K + 15) / 16, "%s: the table of sums of squares has %d tiles; a row of %d elements has %d",
               what, sumsq_tiles, K, (K + 15) / 16);
    FE_REQUIRE(sumsq_tiles <= 1024 && ((size_t)sumsq & 15) == 0, "%s: the table of sums of squares must be 16-byte aligned "
               "and hold at most 1024 tiles (rows of up to 16384 elements)", what);
    return 0;
}

// epilogue: 0 bfloat16 [M, N]; 1 float [M, N]; 2 SwiGLU: W is [2 I, K] (gate rows, then up rows), out bfloat16 [M, I].
// ``sumsq`` (may be null): see check_scale.
extern "C" int fe_skinny_gemm_scaled(const void* x, const void* W, void* out, int M, int N, int K, int epilogue,
                                     const float* sumsq, int sumsq_tiles, float eps, const void* next, long long next_bytes,
                                     cudaStream_t stream) {
    FE_REQUIRE(M >= 1 && M <= 16, "skinny_gemm: %d rows; this kernel takes 1 to 16", M);
    FE_REQUIRE(N > 0 && K > 0 && K % KSTEP == 0, "skinny_gemm: K = %d must be a positive multiple of %d", K, KSTEP);
    FE_REQUIRE((((size_t)x | (size_t)W) & 15) == 0, "skinny_gemm: operands must be 16-byte aligned");
    if (check_scale("skinny_gemm", sumsq, sumsq_tiles, M, K)) return 1;
    FE_REQUIRE(next_bytes >= 0, "skinny_gemm: negative byte count");
    const RowScale scale{sumsq, sumsq_tiles, eps, K, next, next_bytes};
    if (epilogue == EPI_BF16) return launch<EPI_BF16>(x, W, out, M, N, K, 0, stream, QkvEpilogue{}, ResidEpilogue{}, scale);
    if (epilogue == EPI_F32) return launch<EPI_F32>(x, W, out, M, N, K, 0, stream, QkvEpilogue{}, ResidEpilogue{}, scale);
    if (epilogue == EPI_SWIGLU) {
        FE_REQUIRE(N % 2 == 0, "skinny_gemm: SwiGLU needs an even number of weight rows, got %d", N);
        return launch<EPI_SWIGLU>(x, W, out, M, N, K, N / 2, stream, QkvEpilogue{}, ResidEpilogue{}, scale);
    }
    FE_REQUIRE(false, "skinny_gemm: unknown epilogue %d", epilogue);
}

extern "C" int fe_skinny_gemm(const void* x, const void* W, void* out, int M, int N, int K, int epilogue,
                              cudaStream_t stream) {
    return fe_skinny_gemm_scaled(x, W, out, M, N, K, epilogue, nullptr, 0, 0.f, nullptr, 0, stream);
}

// The product that ends a branch of a layer: residual[M, N] += x W^T (float, in place); scaled[M, N] = bfloat16(new
// residual * norm_weight); sumsq_out[ceil(N / 16)][8] = each 16-column tile's share of the rows' sums of squares.
// ``sumsq_in`` (may be null): the scales of the input rows, as for fe_skinny_gemm_scaled.  M <= 8.
extern "C" int fe_skinny_gemm_residual(const void* x, const void* W, float* residual, const float* norm_weight, void* scaled,
                                       float* sumsq_out, int M, int N, int K, const float* sumsq_in, int sumsq_tiles,
                                       float eps, const void* next, long long next_bytes, cudaStream_t stream) {
    FE_REQUIRE(M >= 1 && M <= 8, "skinny_gemm_residual: %d rows; this kernel takes 1 to 8", M);
    FE_REQUIRE(N > 0 && K > 0 && K % KSTEP == 0, "skinny_gemm_residual: K = %d must be a positive multiple of %d", K, KSTEP);
    FE_REQUIRE((((size_t)x | (size_t)W) & 15) == 0, "skinny_gemm_residual: operands must be 16-byte aligned");
    FE_REQUIRE(residual && norm_weight && scaled && sumsq_out, "skinny_gemm_residual: a null pointer");
    if (check_scale("skinny_gemm_residual", sumsq_in, sumsq_tiles, M, K)) return 1;
    const ResidEpilogue resid{residual, norm_weight, (bf16*)scaled, sumsq_out};
    FE_REQUIRE(next_bytes >= 0, "skinny_gemm_residual: negative byte count");
    return launch<EPI_RESID>(x, W, nullptr, M, N, K, 0, stream, QkvEpilogue{}, resid,
                             RowScale{sumsq_in, sumsq_tiles, eps, K, next, next_bytes});
}

// The query/key/value projection of an attention layer with its epilogue fused: y = x W^T + bias,
// half-split rotation of the query and key heads by the tokens' positions, in place into
// out [M, (nq + 2 nkv) d] (bfloat16), and the write of the new keys and values into their cache
// slots.  The whole head is rotated (rotary width = head size, a multiple of 16); M <= 8.
// ``sumsq`` (may be null): the scales of the input rows, as for fe_skinny_gemm_scaled.
extern "C" int fe_skinny_qkv(const void* x, const void* W, void* out, const float* bias, const int* positions,
                             const float* inv_freq, const int* slot_mapping, void* kc, void* vc, int M, int K, int nq,
                             int nkv, int d, int ps, long long num_slots, const float* sumsq, int sumsq_tiles, float eps,
                             int* status, cudaStream_t stream) {
    FE_REQUIRE(M >= 1 && M <= 8, "skinny_qkv: %d rows; this kernel takes 1 to 8", M);
    FE_REQUIRE(K > 0 && K % KSTEP == 0, "skinny_qkv: K = %d must be a positive multiple of %d", K, KSTEP);
    FE_REQUIRE(d >= 16 && d % 16 == 0 && nq > 0 && nkv > 0 && ps > 0, "skinny_qkv: bad head size or counts");
    FE_REQUIRE(positions != nullptr && inv_freq != nullptr, "skinny_qkv: positions and the rotary table are required");
    FE_REQUIRE((((size_t)x | (size_t)W) & 15) == 0, "skinny_qkv: operands must be 16-byte aligned");
    if (check_scale("skinny_qkv", sumsq, sumsq_tiles, M, K)) return 1;
    QkvEpilogue e{bias, positions, inv_freq, slot_mapping, (bf16*)kc, (bf16*)vc, nq, nkv, d, ps, num_slots, status};
    return launch<EPI_QKV>(x, W, out, M, (nq + 2 * nkv) * d, K, 0, stream, e, ResidEpilogue{},
                           RowScale{sumsq, sumsq_tiles, eps, K, nullptr, 0});
}
