// Paged causal grouped-query attention on CUDA cores, float arithmetic throughout.
//
// One warp per (token, query head).  Keys are taken in blocks of 32 that are aligned to absolute
// position 0, one key per lane; scores, running maximum, running sum and the value accumulator
// are float (online softmax, as the reference's block-wise path:
// inference/attention/paged.py:50-70).  Key t is visible to the query at position p iff t <= p
// (and t > p - window when window > 0) (paged.py:31-32).  Query head h reads key/value head
// h / (nq / nkv) (paged.py:29-30).  Because the blocks are aligned to position 0 and taken in
// order, the result for a query does not depend on how its request was cut into steps.
//
// This kernel serves the true 32-bit path for every shape, and bfloat16 for shapes the tensor
// core kernels do not take.
#include <math_constants.h>

#include "common.cuh"

using namespace fe;

template <typename T, int DPL>
__global__ void paged_attention_simt_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out,
                                            long long out_stride, const T* __restrict__ kc,
                                            const T* __restrict__ vc, const int* __restrict__ block_table,
                                            int bt_stride, const int* __restrict__ cu_q,
                                            const int* __restrict__ q_start, const int* __restrict__ token_req,
                                            int T_tokens, int nq, int nkv, int d, int ps, int num_pages, float scale,
                                            int window, int* __restrict__ status) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ float q_smem[];
    const int lane = threadIdx.x & 31;
    const int warp_in_block = threadIdx.x >> 5;
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + warp_in_block;
    if (warp >= (long long)T_tokens * nq) return;
    const int tok = (int)(warp / nq), h = (int)(warp % nq);
    const int r = token_req[tok];
    const int pos = q_start[r] + (tok - cu_q[r]);
    const int kvh = h / (nq / nkv);
    float* qs = q_smem + (size_t)warp_in_block * d;
    const T* qp = q + (size_t)tok * q_stride + (size_t)h * d;
    for (int j = lane; j < d; j += 32) qs[j] = to_float(qp[j]);
    __syncwarp();

    float m = -CUDART_INF_F, l = 0.f;
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.f;

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* table = block_table + (size_t)r * bt_stride;
    for (int kb = (lo / 32) * 32; kb <= pos; kb += 32) {
        const int t = kb + lane;
        bool valid = t >= lo && t <= pos;
        float s = -CUDART_INF_F;
        long long base = 0;
        if (valid) {
            const int page = table[t / ps];
            if (page < 0 || page >= num_pages) {
                if (status) atomicOr(status, FE_STATUS_BAD_PAGE);
                valid = false;
            } else {
                base = (((long long)page * nkv + kvh) * ps + (t % ps)) * d;
                const T* kp = kc + base;
                float dot = 0.f;
                for (int j = 0; j < d; j += 8) {
                    float kv[8];
                    load8<T>(kp + j, kv);
#pragma unroll
                    for (int e = 0; e < 8; ++e) dot = fmaf(qs[j + e], kv[e], dot);
                }
                s = dot * scale;
            }
        }
        const float bm = warp_max(s);
        if (bm == -CUDART_INF_F) continue;            // nothing visible in this block (bad pages only)
        const float m_new = fmaxf(m, bm);
        const float alpha = expf(m - m_new);           // exp(-inf) = 0 on the first block
        const float p = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] *= alpha;
        const int count = min(32, pos - kb + 1);
        for (int tt = 0; tt < count; ++tt) {
            const float pt = __shfl_sync(0xffffffffu, p, tt);
            const long long vb = __shfl_sync(0xffffffffu, base, tt);
            if (pt != 0.f) {
                const T* vp = vc + vb;
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    const int j = lane + 32 * i;
                    if (j < d) acc[i] = fmaf(pt, to_float(vp[j]), acc[i]);
                }
            }
        }
        m = m_new;
    }
    T* op = out + (size_t)tok * out_stride + (size_t)h * d;
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int j = lane + 32 * i;
        if (j < d) op[j] = from_float<T>(acc[i] * inv);
    }
}

template <typename T>
static int launch_simt(const void* q, long long q_stride, void* out, long long out_stride, const void* kc,
                       const void* vc, const int* block_table, int bt_stride, const int* cu_q, const int* q_start,
                       const int* token_req, int T_tokens, int nq, int nkv, int d, int ps, int num_pages,
                       float scale, int window, int* status, cudaStream_t stream) {
    const int warps = 4;
    const long long total = (long long)T_tokens * nq;
    const int blocks = (int)((total + warps - 1) / warps);
    const size_t smem = (size_t)warps * d * sizeof(float);
#define FE_LAUNCH_SIMT(DPL)                                                                                      \
    fe::launch(paged_attention_simt_kernel<T, DPL>, blocks, warps * 32, smem, stream,                                    \
        (const T*)q, q_stride, (T*)out, out_stride, (const T*)kc, (const T*)vc, block_table, bt_stride, cu_q,   \
        q_start, token_req, T_tokens, nq, nkv, d, ps, num_pages, scale, window, status)
    if (d <= 32) FE_LAUNCH_SIMT(1);
    else if (d <= 64) FE_LAUNCH_SIMT(2);
    else if (d <= 128) FE_LAUNCH_SIMT(4);
    else FE_LAUNCH_SIMT(8);
#undef FE_LAUNCH_SIMT
    return fe_check_launch("paged_attention_simt");
}

extern "C" int fe_paged_attention_simt(const void* q, long long q_stride, void* out, long long out_stride,
                                       const void* kc, const void* vc, const int* block_table, int bt_stride,
                                       const int* cu_q, const int* q_start, const int* token_req, int T_tokens,
                                       int nq, int nkv, int d, int ps, int num_pages, float scale, int window,
                                       int dtype, int* status, cudaStream_t stream) {
    FE_REQUIRE(T_tokens >= 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "paged_attention: bad head counts %d/%d", nq, nkv);
    FE_REQUIRE(d >= 16 && d <= 256 && d % 16 == 0, "paged_attention: head size %d is not a multiple of 16 in [16, 256]", d);
    FE_REQUIRE(ps > 0 && num_pages > 0 && window >= 0, "paged_attention: bad page size, page count or window");
    FE_REQUIRE(q_stride % 8 == 0, "paged_attention: query row stride %lld must be a multiple of 8 elements", q_stride);
    if (T_tokens == 0) return 0;
    if (dtype == FE_F32)
        return launch_simt<float>(q, q_stride, out, out_stride, kc, vc, block_table, bt_stride, cu_q, q_start,
                                  token_req, T_tokens, nq, nkv, d, ps, num_pages, scale, window, status, stream);
    if (dtype == FE_BF16)
        return launch_simt<bf16>(q, q_stride, out, out_stride, kc, vc, block_table, bt_stride, cu_q, q_start,
                                 token_req, T_tokens, nq, nkv, d, ps, num_pages, scale, window, status, stream);
    FE_REQUIRE(false, "paged_attention: unknown dtype %d", dtype);
}
