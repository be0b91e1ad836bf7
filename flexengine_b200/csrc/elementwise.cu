// Embedding gather, fused residual add + RMSNorm, fused QKV bias + rotary encoding + paged
// cache write, and the SwiGLU activation.  Formulas:
//   RMSNorm  y = x * rsqrt(mean(x^2) + eps) * w                 (reference: inference/kernels/rmsnorm.py:24-32)
//   rotary   pairs (j, j + rot/2), angle = position * inv_freq   (reference: inference/models/qwen2.py:73-77)
//   SwiGLU   silu(g) * u, silu(g) = g / (1 + exp(-g))            (reference: tests/unit/test_synthetic_qwen.py:35-36)
// All arithmetic is float; sine, cosine, exp and rsqrt are the accurate library forms.
#include "common.cuh"

using namespace fe;

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                                 int H, int V, int* __restrict__ status) {
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0 && status) atomicOr(status, FE_STATUS_BAD_TOKEN);
        for (int j = threadIdx.x; j < H; j += blockDim.x) o[j] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) o[j] = to_float(row[j]);
}

extern "C" int fe_embedding(const int* ids, const void* table, float* out, int T, int H, int V, int dtype,
                            int* status, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && H > 0 && V > 0, "embedding: bad sizes T=%d H=%d V=%d", T, H, V);
    if (T == 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == FE_F32)
        embedding_kernel<float><<<T, threads, 0, stream>>>(ids, (const float*)table, out, H, V, status);
    else if (dtype == FE_BF16)
        embedding_kernel<bf16><<<T, threads, 0, stream>>>(ids, (const bf16*)table, out, H, V, status);
    else
        FE_REQUIRE(false, "embedding: unknown dtype %d", dtype);
    return fe_check_launch("embedding");
}

// ---------------------------------------------------------------------------------------------
// One block per output row.  rows == nullptr: row i; the residual is updated in place (residual
// += delta).  rows != nullptr: output row i reads residual row rows[i] (+ delta row rows[i]) and
// the residual is left as it is.  The row is staged in shared memory (H floats).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const float* __restrict__ weight, float eps, T* __restrict__ out,
                                   const int* __restrict__ rows, int H, int n_rows_total) {
    extern __shared__ float row[];
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    int r = rows ? rows[i] : i;
    if (r < 0 || r >= n_rows_total) r = 0;          // guarded: rows are checked on the host
    float* res = residual + (size_t)r * H;
    const T* del = delta ? delta + (size_t)r * H : nullptr;
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float v = res[j];
        if (del) v += to_float(del[j]);
        row[j] = v;
        if (!rows && del) res[j] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / (float)H + eps);
    T* o = out + (size_t)i * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) o[j] = from_float<T>(row[j] * inv * weight[j]);
}

extern "C" int fe_add_rmsnorm(float* residual, const void* delta, const float* weight, float eps, void* out,
                              const int* rows, int n_out, int H, int n_rows_total, int dtype, cudaStream_t stream) {
    FE_REQUIRE(n_out >= 0 && H > 0, "add_rmsnorm: bad sizes n=%d H=%d", n_out, H);
    if (n_out == 0) return 0;
    const size_t smem = (size_t)H * sizeof(float);
    FE_REQUIRE(smem <= 200 * 1024, "add_rmsnorm: hidden size %d needs %zu bytes of shared memory (limit 204800)", H, smem);
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    cudaError_t err = cudaSuccess;
    if (dtype == FE_F32) {
        if (smem > 48 * 1024)
            err = cudaFuncSetAttribute(add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        FE_REQUIRE(err == cudaSuccess, "add_rmsnorm: %s", cudaGetErrorString(err));
        add_rmsnorm_kernel<float><<<n_out, threads, smem, stream>>>(residual, (const float*)delta, weight, eps,
                                                                     (float*)out, rows, H, n_rows_total);
    } else if (dtype == FE_BF16) {
        if (smem > 48 * 1024)
            err = cudaFuncSetAttribute(add_rmsnorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        FE_REQUIRE(err == cudaSuccess, "add_rmsnorm: %s", cudaGetErrorString(err));
        add_rmsnorm_kernel<bf16><<<n_out, threads, smem, stream>>>(residual, (const bf16*)delta, weight, eps,
                                                                    (bf16*)out, rows, H, n_rows_total);
    } else {
        FE_REQUIRE(false, "add_rmsnorm: unknown dtype %d", dtype);
    }
    return fe_check_launch("add_rmsnorm");
}

// ---------------------------------------------------------------------------------------------
// grid (T, nq + 2 nkv): one block per (token, head).  Query heads: bias + rotation, written back
// in place.  Key heads: bias + rotation, written back and to the key pages.  Value heads: bias,
// written back and to the value pages.  Cache layout [pages, nkv, page_size, d]; slot = page *
// page_size + offset; a negative slot writes nothing.
template <typename T>
__global__ void qkv_bias_rope_cache_kernel(T* __restrict__ qkv, const float* __restrict__ bias,
                                           const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                           int rot, const int* __restrict__ slot_mapping, T* __restrict__ kc,
                                           T* __restrict__ vc, int nq, int nkv, int d, int ps, long long num_slots,
                                           int* __restrict__ status) {
    const int t = blockIdx.x, head = blockIdx.y;
    const int width = (nq + 2 * nkv) * d;
    T* x = qkv + (size_t)t * width + (size_t)head * d;
    const float* b = bias ? bias + (size_t)head * d : nullptr;
    const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
    T* dst = nullptr;
    if (!is_q && slot_mapping) {
        const long long slot = slot_mapping[t];
        if (slot >= num_slots) {
            if (threadIdx.x == 0 && status) atomicOr(status, FE_STATUS_BAD_SLOT);
        } else if (slot >= 0) {
            const long long page = slot / ps, off = slot % ps;
            const int kvh = is_k ? head - nq : head - nq - nkv;
            dst = (is_k ? kc : vc) + ((page * nkv + kvh) * ps + off) * d;
        }
    }
    const int half = rot / 2;
    const bool rotate = (is_q || is_k) && inv_freq != nullptr && rot > 0;
    if (rotate) {
        const float pos = (float)positions[t];
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            float a = to_float(x[j]), c = to_float(x[j + half]);
            if (b) { a += b[j]; c += b[j + half]; }
            float sn, cs;
            sincosf(pos * inv_freq[j], &sn, &cs);
            const T ra = from_float<T>(a * cs - c * sn), rc = from_float<T>(c * cs + a * sn);
            x[j] = ra; x[j + half] = rc;
            if (dst) { dst[j] = ra; dst[j + half] = rc; }
        }
        for (int j = rot + threadIdx.x; j < d; j += blockDim.x) {
            float a = to_float(x[j]);
            if (b) a += b[j];
            const T ra = from_float<T>(a);
            x[j] = ra;
            if (dst) dst[j] = ra;
        }
    } else {
        for (int j = threadIdx.x; j < d; j += blockDim.x) {
            float a = to_float(x[j]);
            if (b) a += b[j];
            const T ra = from_float<T>(a);
            x[j] = ra;
            if (dst) dst[j] = ra;
        }
    }
}

extern "C" int fe_qkv_bias_rope_cache(void* qkv, const float* bias, const int* positions, const float* inv_freq,
                                      int rot, const int* slot_mapping, void* kc, void* vc, int T, int nq, int nkv,
                                      int d, int ps, long long num_slots, int dtype, int* status, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && nq > 0 && nkv > 0 && d > 0 && ps > 0, "qkv_bias_rope_cache: bad sizes");
    FE_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "qkv_bias_rope_cache: rotary width %d does not fit head size %d", rot, d);
    if (T == 0) return 0;
    const dim3 grid(T, nq + 2 * nkv);
    const int threads = d / 2 >= 64 ? 64 : 32;
    if (dtype == FE_F32)
        qkv_bias_rope_cache_kernel<float><<<grid, threads, 0, stream>>>((float*)qkv, bias, positions, inv_freq, rot,
                                                                        slot_mapping, (float*)kc, (float*)vc, nq, nkv,
                                                                        d, ps, num_slots, status);
    else if (dtype == FE_BF16)
        qkv_bias_rope_cache_kernel<bf16><<<grid, threads, 0, stream>>>((bf16*)qkv, bias, positions, inv_freq, rot,
                                                                       slot_mapping, (bf16*)kc, (bf16*)vc, nq, nkv, d,
                                                                       ps, num_slots, status);
    else
        FE_REQUIRE(false, "qkv_bias_rope_cache: unknown dtype %d", dtype);
    return fe_check_launch("qkv_bias_rope_cache");
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long total, int I) {
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / I;
        const int i = (int)(idx % I);
        const float g = to_float(gate_up[t * 2 * I + i]);
        const float u = to_float(gate_up[t * 2 * I + I + i]);
        out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
    }
}

extern "C" int fe_swiglu(const void* gate_up, void* out, int T, int I, int dtype, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && I > 0, "swiglu: bad sizes");
    if (T == 0) return 0;
    const long long total = (long long)T * I;
    const int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (dtype == FE_F32)
        swiglu_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, total, I);
    else if (dtype == FE_BF16)
        swiglu_kernel<bf16><<<(int)blocks, threads, 0, stream>>>((const bf16*)gate_up, (bf16*)out, total, I);
    else
        FE_REQUIRE(false, "swiglu: unknown dtype %d", dtype);
    return fe_check_launch("swiglu");
}
