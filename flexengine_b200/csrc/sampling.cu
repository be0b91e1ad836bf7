// Sampling on the device: one block per row of logits.
//
// temperature == 0: the lowest index of the maximum (reference: engine/sampling/sampler.py:12-13).
// otherwise: x = logits / T; when 0 < k < V keep the k largest (ties go to the lowest indices);
// p = softmax over the kept (float32, reference sampler.py:16-22); the draw is the inverse of the
// cumulative distribution taken in index order at u * total, u in [0, 1) from a counter-based
// generator keyed by (request seed, number of the draw), so that a request's tokens do not
// depend on what else is in the batch (reference: engine/scheduler/state.py:64-65).
#include <math_constants.h>

#include "common.cuh"

using namespace fe;

namespace {

constexpr int THREADS = 512;

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// order-preserving map from float to unsigned
__device__ __forceinline__ unsigned int ordered_key(float v) {
    const unsigned int b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float sanitize(float v) { return v != v ? -CUDART_INF_F : v; }

// exclusive scan over the block of one value per thread; returns the prefix of this thread and the
// block total through ``total``.  ``buf`` holds THREADS + 1 doubles-worth of floats.
template <typename V>
__device__ V block_exclusive_scan(V v, V* buf, V* total) {
    const int tid = threadIdx.x;
    __syncthreads();
    buf[tid] = v;
    __syncthreads();
    // Hillis-Steele over THREADS entries (log steps, deterministic order)
    for (int off = 1; off < THREADS; off <<= 1) {
        V add = tid >= off ? buf[tid - off] : (V)0;
        __syncthreads();
        buf[tid] += add;
        __syncthreads();
    }
    const V inclusive = buf[tid];
    *total = buf[THREADS - 1];
    return inclusive - v;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, long long ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const long long* __restrict__ seed,
              const long long* __restrict__ draw, int* __restrict__ out) {
    griddep_wait();
    griddep_launch_dependents();
    __shared__ float s_val[THREADS];
    __shared__ int s_idx[THREADS];
    __shared__ unsigned int hist[256];
    __shared__ unsigned int s_prefix, s_need;
    __shared__ float scan_f[THREADS];
    __shared__ int scan_i[THREADS];
    __shared__ int s_result;
    __shared__ float s_total;

    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)row * ld;
    const float temp = temperature[row];

    // ---- maximum and its lowest index (needed by both branches)
    float best = -CUDART_INF_F;
    int best_i = 0x7fffffff;
    if ((V & 3) == 0 && (reinterpret_cast<size_t>(x) & 15) == 0) {
        // four logits per load, two loads in flight per thread
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const int n4 = V >> 2;
        for (int i = tid; i < n4; i += 2 * THREADS) {
            const float4 a = x4[i];
            const int j = i + THREADS;
            const float4 b = j < n4 ? x4[j] : make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
            const float va[4] = {a.x, a.y, a.z, a.w}, vb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float v = sanitize(va[e]);
                if (v > best || (v == best && 4 * i + e < best_i)) { best = v; best_i = 4 * i + e; }
            }
            if (j < n4) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float v = sanitize(vb[e]);
                    if (v > best || (v == best && 4 * j + e < best_i)) { best = v; best_i = 4 * j + e; }
                }
            }
        }
    } else {
        for (int i = tid; i < V; i += THREADS) {
            const float v = sanitize(x[i]);
            if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
        }
    }
    s_val[tid] = best; s_idx[tid] = best_i;
    __syncthreads();
    for (int off = THREADS / 2; off > 0; off >>= 1) {
        if (tid < off) {
            const float v = s_val[tid + off]; const int i = s_idx[tid + off];
            if (v > s_val[tid] || (v == s_val[tid] && i < s_idx[tid])) { s_val[tid] = v; s_idx[tid] = i; }
        }
        __syncthreads();
    }
    const float max_logit = s_val[0];
    const int argmax = s_idx[0] == 0x7fffffff ? 0 : s_idx[0];
    if (temp == 0.f) {
        if (tid == 0) out[row] = argmax;
        return;
    }

    // ---- top-k threshold by radix select on the ordered keys of the logits (division by a
    //      positive temperature keeps the order)
    int k = top_k[row];
    const bool use_k = k > 0 && k < V;
    unsigned int thr_key = 0;      // keep keys > thr_key, and ``need`` of the keys == thr_key
    unsigned int need = 0;
    if (use_k) {
        if (tid == 0) { s_prefix = 0; s_need = (unsigned int)k; }
        __syncthreads();
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int b = tid; b < 256; b += THREADS) hist[b] = 0;
            __syncthreads();
            const unsigned int prefix = s_prefix;
            const unsigned int mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
            for (int i = tid; i < V; i += THREADS) {
                const unsigned int key = ordered_key(sanitize(x[i]));
                if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xffu], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned int remaining = s_need;
                int b = 255;
                for (; b > 0; --b) {
                    if (hist[b] >= remaining) break;
                    remaining -= hist[b];
                }
                s_prefix = prefix | ((unsigned int)b << shift);
                s_need = remaining;
            }
            __syncthreads();
        }
        thr_key = s_prefix;
        need = s_need;             // how many of the keys equal to the threshold are kept
    }

    // ---- each thread owns a contiguous segment of the vocabulary, so that index order is kept
    const int seg = (V + THREADS - 1) / THREADS;
    const int i0 = min(V, tid * seg), i1 = min(V, i0 + seg);

    // rank of threshold ties in index order
    int tie_base = 0;
    if (use_k) {
        int ties = 0;
        for (int i = i0; i < i1; ++i) ties += ordered_key(sanitize(x[i])) == thr_key;
        int total_ties;
        tie_base = block_exclusive_scan<int>(ties, scan_i, &total_ties);
    }

    const float inv_shift = max_logit / temp;
    float local = 0.f;
    {
        int tie_rank = tie_base;
        for (int i = i0; i < i1; ++i) {
            const float v = sanitize(x[i]);
            bool keep = true;
            if (use_k) {
                const unsigned int key = ordered_key(v);
                keep = key > thr_key || (key == thr_key && (unsigned int)(tie_rank++) < need);
            }
            if (keep) local += expf(v / temp - inv_shift);
        }
    }
    // prefix sums of the per-thread masses, accumulated by one thread in index order: the
    // sequence is nondecreasing, so the intervals [prefix[i], prefix[i+1]) tile [0, total)
    scan_f[tid] = local;
    __syncthreads();
    if (tid == 0) {
        float run = 0.f;
        for (int i = 0; i < THREADS; ++i) {
            const float v = scan_f[i];
            scan_f[i] = run;
            run += v;
        }
        s_total = run;
    }
    __syncthreads();
    const float total = s_total;
    const float before = scan_f[tid];
    const float upper = tid + 1 < THREADS ? scan_f[tid + 1] : total;

    const unsigned long long bits = splitmix64(splitmix64((unsigned long long)seed[row]) + (unsigned long long)draw[row]);
    const float u = (float)(bits >> 40) * (1.0f / 16777216.0f);
    float target = u * total;
    if (target >= total) target = nextafterf(total, 0.f);

    if (tid == 0) s_result = -1;
    __syncthreads();
    // the segment in which the cumulative sum first exceeds the target
    if (before <= target && target < upper) {
        float cum = before;
        int tie_rank = tie_base;
        int found = -1, last_kept = -1;
        for (int i = i0; i < i1; ++i) {
            const float v = sanitize(x[i]);
            bool keep = true;
            if (use_k) {
                const unsigned int key = ordered_key(v);
                keep = key > thr_key || (key == thr_key && (unsigned int)(tie_rank++) < need);
            }
            if (!keep) continue;
            last_kept = i;
            cum += expf(v / temp - inv_shift);
            if (cum > target) { found = i; break; }
        }
        if (found < 0) found = last_kept;          // rounding at the very end of the segment
        if (found >= 0) atomicMax(&s_result, found);
    }
    __syncthreads();
    if (tid == 0) out[row] = s_result >= 0 ? s_result : argmax;
}

}  // namespace

extern "C" int fe_sample(const float* logits, long long ld, int R, int V, const float* temperature,
                         const int* top_k, const long long* seed, const long long* draw, int* out,
                         cudaStream_t stream) {
    FE_REQUIRE(R >= 0 && V > 0 && ld >= V, "sample: bad sizes R=%d V=%d ld=%lld", R, V, ld);
    if (R == 0) return 0;
    fe::launch(sample_kernel, R, THREADS, 0, stream, logits, ld, V, temperature, top_k, seed, draw, out);
    return fe_check_launch("sample");
}
