// Embedding gather, fused residual add + RMSNorm, fused QKV bias + rotary encoding + paged
// cache write, and the SwiGLU activation.  Formulas:
//   RMSNorm  y = x * rsqrt(mean(x^2) + eps) * w                 (reference: inference/kernels/rmsnorm.py:24-32)
//   rotary   pairs (j, j + rot/2), angle = position * inv_freq   (reference: inference/models/qwen2.py:73-77)
//   SwiGLU   silu(g) * u, silu(g) = g / (1 + exp(-g))            (reference: tests/unit/test_synthetic_qwen.py:35-36)
// All arithmetic is float; sine, cosine, exp and rsqrt are the accurate library forms.
#define FE_PDL_CLASS 4      // FE_PDL_ELEMENTWISE
#include "common.cuh"

using namespace fe;

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                                 int H, int V, int* __restrict__ status) {
    griddep_wait();
    griddep_launch_dependents();
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
        fe::launch(embedding_kernel<float>, T, threads, 0, stream, ids, (const float*)table, out, H, V, status);
    else if (dtype == FE_BF16)
        fe::launch(embedding_kernel<bf16>, T, threads, 0, stream, ids, (const bf16*)table, out, H, V, status);
    else
        FE_REQUIRE(false, "embedding: unknown dtype %d", dtype);
    return fe_check_launch("embedding");
}

// ---------------------------------------------------------------------------------------------
// token_ids[rows[i]] = previous[sources[i]] for every i with rows[i] >= 0: the tokens that the step
// before sampled go into this step's input on the device, before the host has seen them.
__global__ void carry_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ rows,
                                    const int* __restrict__ sources, const int* __restrict__ previous, int n, int T,
                                    int n_previous, int* __restrict__ status) {
    griddep_wait();
    griddep_launch_dependents();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int r = rows[i], s = sources[i];
    if (r < 0) return;
    if (r >= T || s < 0 || s >= n_previous) {
        if (status) atomicOr(status, FE_STATUS_BAD_TOKEN);
        return;
    }
    token_ids[r] = previous[s];
}

extern "C" int fe_carry_tokens(int* token_ids, const int* rows, const int* sources, const int* previous, int n, int T,
                               int n_previous, int* status, cudaStream_t stream) {
    FE_REQUIRE(n >= 0 && T >= 0 && n_previous >= 0, "carry_tokens: bad sizes");
    if (n == 0) return 0;
    fe::launch(carry_tokens_kernel, (n + 127) / 128, 128, 0, stream, token_ids, rows, sources, previous, n, T, n_previous,
               status);
    return fe_check_launch("carry_tokens");
}

// ---------------------------------------------------------------------------------------------
// One block per output row.  rows == nullptr: row i; the residual is updated in place (residual
// += delta).  rows != nullptr: output row i reads residual row rows[i] (+ delta row rows[i]) and
// the residual is left as it is.  The row is staged in shared memory (H floats).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const float* __restrict__ weight, float eps, T* __restrict__ out,
                                   const int* __restrict__ rows, int H, int n_rows_total, int n_out,
                                   const void* __restrict__ upcoming, long long upcoming_bytes) {
    if ((int)blockIdx.x >= n_out) {         // blocks beyond the rows: start the next kernel's weights into L2
        prefetch_l2_share(upcoming, upcoming_bytes, (long long)(blockIdx.x - n_out) * blockDim.x + threadIdx.x,
                          (long long)(gridDim.x - n_out) * blockDim.x);
        return;
    }
    griddep_wait();
    griddep_launch_dependents();
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

// The same, four elements at a time (H % 4 == 0): 16-byte loads and stores of the float residual.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                           __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<const unsigned*>(&a);
        raw.y = *reinterpret_cast<const unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename T>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                       const float* __restrict__ weight, float eps, T* __restrict__ out,
                                       const int* __restrict__ rows, int H, int n_rows_total, int n_out,
                                       const void* __restrict__ upcoming, long long upcoming_bytes) {
    if ((int)blockIdx.x >= n_out) {         // blocks beyond the rows: start the next kernel's weights into L2
        prefetch_l2_share(upcoming, upcoming_bytes, (long long)(blockIdx.x - n_out) * blockDim.x + threadIdx.x,
                          (long long)(gridDim.x - n_out) * blockDim.x);
        return;
    }
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ float row[];
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    int r = rows ? rows[i] : i;
    if (r < 0 || r >= n_rows_total) r = 0;
    float* res = residual + (size_t)r * H;
    const T* del = delta ? delta + (size_t)r * H : nullptr;
    float ss = 0.f;
    for (int j = threadIdx.x * 4; j < H; j += blockDim.x * 4) {
        float4 v = *reinterpret_cast<const float4*>(res + j);
        if (del) {
            const float4 dv = Vec4<T>::load(del + j);
            v.x += dv.x; v.y += dv.y; v.z += dv.z; v.w += dv.w;
            if (!rows) *reinterpret_cast<float4*>(res + j) = v;
        }
        *reinterpret_cast<float4*>(row + j) = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / (float)H + eps);
    T* o = out + (size_t)i * H;
    for (int j = threadIdx.x * 4; j < H; j += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(row + j);
        const float4 w = *reinterpret_cast<const float4*>(weight + j);
        Vec4<T>::store(o + j, make_float4(v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z, v.w * inv * w.w));
    }
}

constexpr int PREFETCH_BLOCKS = 64;

template <typename T>
static int launch_add_rmsnorm(float* residual, const void* delta, const float* weight, float eps, void* out,
                              const int* rows, int n_out, int H, int n_rows_total, const void* upcoming,
                              long long upcoming_bytes, cudaStream_t stream) {
    const int grid = n_out + (upcoming && upcoming_bytes > 0 ? PREFETCH_BLOCKS : 0);
    const size_t smem = (size_t)H * sizeof(float);
    const bool vec = H % 4 == 0;
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    cudaError_t err = cudaSuccess;
    if (vec) {
        if (smem > 48 * 1024)
            err = cudaFuncSetAttribute(add_rmsnorm_vec_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        FE_REQUIRE(err == cudaSuccess, "add_rmsnorm: %s", cudaGetErrorString(err));
        fe::launch(add_rmsnorm_vec_kernel<T>, grid, threads, smem, stream, residual, (const T*)delta, weight, eps, (T*)out,
                   rows, H, n_rows_total, n_out, upcoming, upcoming_bytes);
    } else {
        if (smem > 48 * 1024)
            err = cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        FE_REQUIRE(err == cudaSuccess, "add_rmsnorm: %s", cudaGetErrorString(err));
        fe::launch(add_rmsnorm_kernel<T>, grid, threads, smem, stream, residual, (const T*)delta, weight, eps, (T*)out, rows,
                   H, n_rows_total, n_out, upcoming, upcoming_bytes);
    }
    return fe_check_launch("add_rmsnorm");
}

// ``upcoming`` (may be null): memory that the next kernel will stream, ``upcoming_bytes`` of it; extra blocks ask for
// it to be brought into L2 while this kernel, which barely touches memory, runs.
extern "C" int fe_add_rmsnorm(float* residual, const void* delta, const float* weight, float eps, void* out,
                              const int* rows, int n_out, int H, int n_rows_total, int dtype, const void* upcoming,
                              long long upcoming_bytes, cudaStream_t stream) {
    FE_REQUIRE(n_out >= 0 && H > 0 && upcoming_bytes >= 0, "add_rmsnorm: bad sizes n=%d H=%d", n_out, H);
    if (n_out == 0) return 0;
    FE_REQUIRE((size_t)H * sizeof(float) <= 200 * 1024,
               "add_rmsnorm: hidden size %d needs %zu bytes of shared memory (limit 204800)", H, (size_t)H * sizeof(float));
    if (dtype == FE_F32)
        return launch_add_rmsnorm<float>(residual, delta, weight, eps, out, rows, n_out, H, n_rows_total, upcoming, upcoming_bytes, stream);
    if (dtype == FE_BF16)
        return launch_add_rmsnorm<bf16>(residual, delta, weight, eps, out, rows, n_out, H, n_rows_total, upcoming, upcoming_bytes, stream);
    FE_REQUIRE(false, "add_rmsnorm: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------------------
// grid (T, nq + 2 nkv): one block per (token, head).  Query heads: bias + rotation, written back
// in place.  Key heads: bias + rotation, written back and to the key pages.  Value heads: bias,
// written back and to the value pages.  Cache layout [pages, nkv, page_size, d]; slot = page *
// page_size + offset; a negative slot writes nothing.
// The projection is read from ``src`` as TI (the compute type, or float when the product was kept in 32-bit so that
// bias and rotation are added before the one rounding) and written to ``qkv`` as T; with TI = T the two may be the
// same buffer: every element is read before it is written, by the thread that writes it.
template <typename TI, typename T>
__global__ void qkv_bias_rope_cache_kernel(const TI* src, T* qkv, const float* __restrict__ bias,
                                           const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                           int rot, const int* __restrict__ slot_mapping, T* __restrict__ kc,
                                           T* __restrict__ vc, int nq, int nkv, int d, int ps, long long num_slots,
                                           int* __restrict__ status) {
    griddep_wait();
    griddep_launch_dependents();
    const int t = blockIdx.x, head = blockIdx.y;
    const int width = (nq + 2 * nkv) * d;
    T* x = qkv + (size_t)t * width + (size_t)head * d;
    const TI* xi = src + (size_t)t * width + (size_t)head * d;
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
            float a = to_float(xi[j]), c = to_float(xi[j + half]);
            if (b) { a += b[j]; c += b[j + half]; }
            float sn, cs;
            sincosf(pos * inv_freq[j], &sn, &cs);
            const T ra = from_float<T>(a * cs - c * sn), rc = from_float<T>(c * cs + a * sn);
            x[j] = ra; x[j + half] = rc;
            if (dst) { dst[j] = ra; dst[j + half] = rc; }
        }
        for (int j = rot + threadIdx.x; j < d; j += blockDim.x) {
            float a = to_float(xi[j]);
            if (b) a += b[j];
            const T ra = from_float<T>(a);
            x[j] = ra;
            if (dst) dst[j] = ra;
        }
    } else {
        for (int j = threadIdx.x; j < d; j += blockDim.x) {
            float a = to_float(xi[j]);
            if (b) a += b[j];
            const T ra = from_float<T>(a);
            x[j] = ra;
            if (dst) dst[j] = ra;
        }
    }
}

// The same for head sizes and rotary widths that are multiples of 16: one block per token; sine
// and cosine of the token's angles are computed once (they do not depend on the head) and
// every thread moves eight elements of each half at a time.
// eight consecutive floats from a 16-byte aligned address (bias, the table of cosines and sines)
__device__ __forceinline__ void load8f(const float* p, float* v) {
    const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 4);
    v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
}

template <typename TI, typename T>
__global__ void qkv_bias_rope_cache_vec_kernel(const TI* src, T* qkv, const float* __restrict__ bias,
                                               const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                               int rot, const int* __restrict__ slot_mapping, T* __restrict__ kc,
                                               T* __restrict__ vc, int nq, int nkv, int d, int ps,
                                               long long num_slots, int* __restrict__ status) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ __align__(16) float trig[];    // cos [rot/2], sin [rot/2]
    const int t = blockIdx.x;
    const int half = rot / 2;
    const bool rotary = inv_freq != nullptr && rot > 0;
    if (rotary) {
        const float pos = (float)positions[t];
        for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &trig[half + j], &trig[j]);
    }
    long long slot = slot_mapping ? slot_mapping[t] : -1;
    if (slot >= num_slots) {
        if (threadIdx.x == 0 && status) atomicOr(status, FE_STATUS_BAD_SLOT);
        slot = -1;
    }
    __syncthreads();
    const int heads = nq + 2 * nkv;
    const int width = heads * d;
    T* x = qkv + (size_t)t * width;
    const TI* xin = src + (size_t)t * width;
    // unit = (head, group of 8 elements of the first half of the rotated part, or of the rest)
    const int rot_units = rotary ? half / 8 : 0, rest_units = (d - (rotary ? rot : 0)) / 8;
    const int per_head = rot_units + rest_units;
    for (int u = threadIdx.x; u < heads * per_head; u += blockDim.x) {
        const int head = u / per_head, k = u - head * per_head;
        const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
        T* hx = x + (size_t)head * d;
        const TI* hi = xin + (size_t)head * d;
        const float* hb = bias ? bias + (size_t)head * d : nullptr;
        T* dst = nullptr;
        if (!is_q && slot >= 0) {
            const int kvh = is_k ? head - nq : head - nq - nkv;
            dst = (is_k ? kc : vc) + (((slot / ps) * nkv + kvh) * ps + (slot % ps)) * d;
        }
        if (k < rot_units && (is_q || is_k)) {
            const int j = k * 8;
            float a[8], c[8];
            load8<TI>(hi + j, a);
            load8<TI>(hi + j + half, c);
            float ra[8], rc[8];
            float cs[8], sn[8];
            load8f(trig + j, cs);
            load8f(trig + half + j, sn);
            if (hb) {
                float ba[8], bc[8];
                load8f(hb + j, ba);
                load8f(hb + j + half, bc);
#pragma unroll
                for (int e = 0; e < 8; ++e) { a[e] += ba[e]; c[e] += bc[e]; }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                ra[e] = a[e] * cs[e] - c[e] * sn[e];
                rc[e] = c[e] * cs[e] + a[e] * sn[e];
            }
            store8<T>(hx + j, ra);
            store8<T>(hx + j + half, rc);
            if (dst) { store8<T>(dst + j, ra); store8<T>(dst + j + half, rc); }
        } else {
            // a value head's "rotated" range, or the part of the head beyond the rotary width
            int j;
            if (k < rot_units) j = k * 8;
            else j = (rotary ? rot : 0) + (k - rot_units) * 8;
            for (int rep = 0; rep < ((k < rot_units) ? 2 : 1); ++rep, j += half) {
                float a[8];
                load8<TI>(hi + j, a);
                if (hb) {
                    float ba[8];
                    load8f(hb + j, ba);
#pragma unroll
                    for (int e = 0; e < 8; ++e) a[e] += ba[e];
                }
                store8<T>(hx + j, a);
                if (dst) store8<T>(dst + j, a);
            }
        }
    }
}

template <typename TI, typename T>
static int launch_rope(const void* src, void* qkv, const float* bias, const int* positions, const float* inv_freq, int rot,
                       const int* slot_mapping, void* kc, void* vc, int T_tokens, int nq, int nkv, int d, int ps,
                       long long num_slots, int* status, cudaStream_t stream) {
    if (d % 16 == 0 && rot % 16 == 0 && ((size_t)bias & 15) == 0) {
        const int units = (nq + 2 * nkv) * (d / 8 - (inv_freq && rot ? rot / 16 : 0));
        // as few passes over the units as 256 threads need, and then only as many threads as fill every pass
        const int passes = (units + 255) / 256;
        const int threads = max(64, ((units + passes - 1) / passes + 31) / 32 * 32);
        fe::launch(qkv_bias_rope_cache_vec_kernel<TI, T>, T_tokens, threads, (size_t)rot * sizeof(float), stream,
            (const TI*)src, (T*)qkv, bias, positions, inv_freq, rot, slot_mapping, (T*)kc, (T*)vc, nq, nkv, d, ps, num_slots, status);
    } else {
        const dim3 grid(T_tokens, nq + 2 * nkv);
        fe::launch(qkv_bias_rope_cache_kernel<TI, T>, grid, d / 2 >= 64 ? 64 : 32, 0, stream,
            (const TI*)src, (T*)qkv, bias, positions, inv_freq, rot, slot_mapping, (T*)kc, (T*)vc, nq, nkv, d, ps, num_slots, status);
    }
    return fe_check_launch("qkv_bias_rope_cache");
}

// ``src``: the projection, in the compute dtype (may be ``qkv`` itself) or, with ``src_float`` set, in float;
// ``qkv``: the result in the compute dtype ``dtype``.
extern "C" int fe_qkv_bias_rope_cache(const void* src, int src_float, void* qkv, const float* bias, const int* positions,
                                      const float* inv_freq, int rot, const int* slot_mapping, void* kc, void* vc, int T,
                                      int nq, int nkv, int d, int ps, long long num_slots, int dtype, int* status,
                                      cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && nq > 0 && nkv > 0 && d > 0 && ps > 0, "qkv_bias_rope_cache: bad sizes");
    FE_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "qkv_bias_rope_cache: rotary width %d does not fit head size %d", rot, d);
    if (T == 0) return 0;
    FE_REQUIRE(src != nullptr && qkv != nullptr, "qkv_bias_rope_cache: no source or destination");
    FE_REQUIRE(!(src_float && src == qkv), "qkv_bias_rope_cache: a float source cannot be rewritten in place as another type");
    if (dtype == FE_F32)
        return launch_rope<float, float>(src, qkv, bias, positions, inv_freq, rot, slot_mapping, kc, vc, T, nq, nkv, d, ps, num_slots, status, stream);
    if (dtype == FE_BF16 && src_float)
        return launch_rope<float, bf16>(src, qkv, bias, positions, inv_freq, rot, slot_mapping, kc, vc, T, nq, nkv, d, ps, num_slots, status, stream);
    if (dtype == FE_BF16)
        return launch_rope<bf16, bf16>(src, qkv, bias, positions, inv_freq, rot, slot_mapping, kc, vc, T, nq, nkv, d, ps, num_slots, status, stream);
    FE_REQUIRE(false, "qkv_bias_rope_cache: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long total, int I) {
    griddep_wait();
    griddep_launch_dependents();
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / I;
        const int i = (int)(idx % I);
        const float g = to_float(gate_up[t * 2 * I + i]);
        const float u = to_float(gate_up[t * 2 * I + I + i]);
        out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
    }
}

template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long units, int I) {
    griddep_wait();
    griddep_launch_dependents();
    const int per_row = I / 8;
    for (long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x; u < units; u += (long long)gridDim.x * blockDim.x) {
        const long long t = u / per_row;
        const int i = (int)(u - t * per_row) * 8;
        float g[8], up[8], r[8];
        load8<T>(gate_up + t * 2 * I + i, g);
        load8<T>(gate_up + t * 2 * I + I + i, up);
#pragma unroll
        for (int e = 0; e < 8; ++e) r[e] = g[e] / (1.f + expf(-g[e])) * up[e];
        store8<T>(out + t * I + i, r);
    }
}

extern "C" int fe_swiglu(const void* gate_up, void* out, int T, int I, int dtype, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && I > 0, "swiglu: bad sizes");
    if (T == 0) return 0;
    const bool vec = I % 8 == 0;
    const long long total = vec ? (long long)T * (I / 8) : (long long)T * I;
    const int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    const long long most = 16LL * fe_sm_count();
    if (blocks > most) blocks = most;
    if (dtype == FE_F32) {
        if (vec) fe::launch(swiglu_vec_kernel<float>, (int)blocks, threads, 0, stream, (const float*)gate_up, (float*)out, total, I);
        else fe::launch(swiglu_kernel<float>, (int)blocks, threads, 0, stream, (const float*)gate_up, (float*)out, total, I);
    } else if (dtype == FE_BF16) {
        if (vec) fe::launch(swiglu_vec_kernel<bf16>, (int)blocks, threads, 0, stream, (const bf16*)gate_up, (bf16*)out, total, I);
        else fe::launch(swiglu_kernel<bf16>, (int)blocks, threads, 0, stream, (const bf16*)gate_up, (bf16*)out, total, I);
    } else {
        FE_REQUIRE(false, "swiglu: unknown dtype %d", dtype);
    }
    return fe_check_launch("swiglu");
}
