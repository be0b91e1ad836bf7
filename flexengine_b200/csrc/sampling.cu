// Sampling on the device: one block per row of logits.
//
// temperature == 0: the lowest index of the maximum (reference: engine/sampling/sampler.py:12-13).
// otherwise: x = logits / T; when 0 < k < V keep the k largest (ties go to the lowest indices);
// p = softmax over the kept (float32, reference sampler.py:16-22); the draw is the inverse of the
// cumulative distribution taken in index order at u * total, u in [0, 1) from a counter-based
// generator keyed by (request seed, number of the draw), so that a request's tokens do not
// depend on what else is in the batch (reference: engine/scheduler/state.py:64-65).
//
// Every pass over a row is coalesced: warp w owns the contiguous segment [w S, (w + 1) S) of the vocabulary and
// walks it 32 indices at a time.  Mass is summed chunk by chunk (a fixed butterfly inside the chunk, then a running
// sum), warp totals are added up by one thread in index order, and the pass that looks for the token repeats the same
// arithmetic, so the intervals of the tokens tile [0, total) and the result is the same on every run.
#include <math_constants.h>

#define FE_PDL_CLASS 8      // FE_PDL_SAMPLING
#include "common.cuh"

using namespace fe;

namespace {

constexpr int THREADS = 1024;
constexpr int WARPS = THREADS / 32;
constexpr int RADIX_LOADS = 8;      // loads on their way at once in a pass of the radix select

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

__device__ __forceinline__ float warp_total(float v) {       // the same value in every lane, the same order every time
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, long long ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const long long* __restrict__ seed,
              const long long* __restrict__ draw, int* __restrict__ out) {
    griddep_wait();
    griddep_launch_dependents();
    __shared__ float s_val[THREADS];
    __shared__ int s_idx[THREADS];
    __shared__ unsigned int hist[256], suffix[256];
    __shared__ unsigned int warp_hist[WARPS][256];      // one histogram per warp: no two warps meet in a bin
    __shared__ unsigned int s_prefix, s_need;
    __shared__ float warp_mass[WARPS + 1];      // after the prefix: mass before warp w; [WARPS] = total
    __shared__ int warp_ties[WARPS];            // after the prefix: threshold ties before warp w, in index order
    __shared__ int s_result;

    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)row * ld;
    const float temp = temperature[row];

    // ---- maximum and its lowest index (needed by both branches)
    float best = -CUDART_INF_F;
    int best_i = 0x7fffffff;
    if ((V & 3) == 0 && (reinterpret_cast<size_t>(x) & 15) == 0) {
        // four logits per load, four loads in flight per thread: a row is read by one block, so what bounds this
        // pass is how many loads are on their way at once
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const int n4 = V >> 2;
        const float4 none = make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
        for (int i = tid; i < n4; i += 4 * THREADS) {
            float4 part[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) part[u] = i + u * THREADS < n4 ? x4[i + u * THREADS] : none;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int at = 4 * (i + u * THREADS);
                const float v4[4] = {part[u].x, part[u].y, part[u].z, part[u].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    // a thread meets its indices in rising order, so "greater" alone keeps the lowest index of its maximum
                    const float v = sanitize(v4[e]);
                    if (v > best) { best = v; best_i = at + e; }
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
            for (int b = tid; b < WARPS * 256; b += THREADS) (&warp_hist[0][0])[b] = 0;
            __syncthreads();
            const unsigned int prefix = s_prefix;
            const unsigned int mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
            auto count = [&](float raw) {
                const unsigned int key = ordered_key(sanitize(raw));
                if ((key & mask) == prefix) atomicAdd(&warp_hist[tid >> 5][(key >> shift) & 0xffu], 1u);
            };
            if ((V & 3) == 0 && (reinterpret_cast<size_t>(x) & 15) == 0) {
                // the order does not matter here: four logits per load, four loads on their way per thread
                const float4* x4 = reinterpret_cast<const float4*>(x);
                const int n4 = V >> 2;
                for (int i = tid; i < n4; i += 4 * THREADS) {
                    float4 part[4];
                    bool in[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        in[u] = i + u * THREADS < n4;
                        part[u] = in[u] ? x4[i + u * THREADS] : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (in[u]) { count(part[u].x); count(part[u].y); count(part[u].z); count(part[u].w); }
                }
            } else {
                for (int i0 = tid; i0 < V; i0 += RADIX_LOADS * THREADS) {
                    float v[RADIX_LOADS];
#pragma unroll
                    for (int u = 0; u < RADIX_LOADS; ++u) v[u] = i0 + u * THREADS < V ? x[i0 + u * THREADS] : 0.f;
#pragma unroll
                    for (int u = 0; u < RADIX_LOADS; ++u)
                        if (i0 + u * THREADS < V) count(v[u]);
                }
            }
            __syncthreads();
            if (tid < 256) {
                unsigned int sum = 0;
                for (int w = 0; w < WARPS; ++w) sum += warp_hist[w][tid];
                hist[tid] = sum;
            }
            __syncthreads();
            // the bin in which the count of larger keys passes what is still needed: thread b holds the number of keys
            // in bins above b (suffix sums by doubling), exactly one thread finds need within its own bin
            if (tid < 256) suffix[tid] = hist[tid];
            __syncthreads();
            for (int off = 1; off < 256; off <<= 1) {
                const unsigned int add = tid < 256 && tid + off < 256 ? suffix[tid + off] : 0u;
                __syncthreads();
                if (tid < 256) suffix[tid] += add;
                __syncthreads();
            }
            const unsigned int remaining = s_need;
            __syncthreads();
            if (tid < 256) {
                const unsigned int above = suffix[tid] - hist[tid];        // keys in bins above this one
                if (above < remaining && (suffix[tid] >= remaining || tid == 0)) {
                    s_prefix = prefix | ((unsigned int)tid << shift);
                    s_need = remaining - above;
                }
            }
            __syncthreads();
        }
        thr_key = s_prefix;
        need = s_need;             // how many of the keys equal to the threshold are kept
    }

    // ---- warp w owns the contiguous segment [seg0, seg1) of the vocabulary and walks it 32 indices at a time
    const int warp = tid >> 5, lane = tid & 31;
    const int S = ((V + WARPS - 1) / WARPS + 31) / 32 * 32;
    const int seg0 = min(V, warp * S), seg1 = min(V, seg0 + S);
    const unsigned int below = (1u << lane) - 1u;

    // Eight chunks (256 indices) are loaded at once, so that eight loads are on their way together: a row is read by
    // one block, and what bounds a pass is the latency of its loads.
    constexpr int GROUP = 8;
    auto load_group = [&](int base, float* v) {
#pragma unroll
        for (int c = 0; c < GROUP; ++c) {
            const int i = base + 32 * c + lane;
            v[c] = i < seg1 ? x[i] : 0.f;
        }
    };

    // threshold ties before this warp's segment, in index order
    if (use_k) {
        int ties = 0;
        for (int base = seg0; base < seg1; base += 32 * GROUP) {
            float v[GROUP];
            load_group(base, v);
#pragma unroll
            for (int c = 0; c < GROUP; ++c)
                ties += __popc(__ballot_sync(0xffffffffu, base + 32 * c + lane < seg1 && ordered_key(sanitize(v[c])) == thr_key));
        }
        if (lane == 0) warp_ties[warp] = ties;
        __syncthreads();
        if (tid == 0) {
            int run = 0;
            for (int w = 0; w < WARPS; ++w) { const int t = warp_ties[w]; warp_ties[w] = run; run += t; }
        }
        __syncthreads();
    }
    const int tie_base = use_k ? warp_ties[warp] : 0;
    const float inv_temp = 1.f / temp, inv_shift = max_logit * inv_temp;

    // the unnormalised probability of index ``i`` with logit ``raw`` (0 when it is cut off), and the running tie count
    auto mass_of = [&](int i, float raw, int& ties_seen) -> float {
        const bool in = i < seg1;
        const float v = sanitize(raw);
        bool keep = in;
        if (use_k) {
            const unsigned int key = ordered_key(v);
            const unsigned int tied = __ballot_sync(0xffffffffu, in && key == thr_key);
            const int rank = tie_base + ties_seen + __popc(tied & below);
            keep = in && (key > thr_key || (key == thr_key && (unsigned int)rank < need));
            ties_seen += __popc(tied);
        }
        return keep ? __expf(v * inv_temp - inv_shift) : 0.f;
    };

    // mass of the segment: per group, each lane adds its eight values in order, the lanes' sums are added by a fixed
    // butterfly, and the groups' sums are added up as the walk goes.  Lane g remembers where group g began (the sum
    // and the tie count before it), so that the search below can start at the right group.
    float began_at = 0.f;
    int ties_at = 0;
    {
        float cum = 0.f;
        int ties_seen = 0, g = 0;
        for (int base = seg0; base < seg1; base += 32 * GROUP, ++g) {
            if (lane == g) { began_at = cum; ties_at = ties_seen; }
            float v[GROUP];
            load_group(base, v);
            float part = 0.f;
#pragma unroll
            for (int c = 0; c < GROUP; ++c) part += mass_of(base + 32 * c + lane, v[c], ties_seen);
            cum += warp_total(part);
        }
        if (lane == 0) warp_mass[warp] = cum;
    }
    __syncthreads();
    if (tid == 0) {
        // accumulated by one thread in index order: nondecreasing, so the warps' intervals tile [0, total)
        float run = 0.f;
        for (int w = 0; w < WARPS; ++w) { const float m = warp_mass[w]; warp_mass[w] = run; run += m; }
        warp_mass[WARPS] = run;
        s_result = -1;
    }
    __syncthreads();
    const float total = warp_mass[WARPS];
    const unsigned long long bits = splitmix64(splitmix64((unsigned long long)seed[row]) + (unsigned long long)draw[row]);
    const float u = (float)(bits >> 40) * (1.0f / 16777216.0f);
    float target = u * total;
    if (target >= total) target = nextafterf(total, 0.f);

    // the warp into whose interval the target falls repeats its walk with the same arithmetic, stops at the group
    // that takes the running sum past the target, and looks for the token inside it chunk by chunk, lane by lane
    if (warp_mass[warp] <= target && target < warp_mass[warp + 1]) {
        float cum = warp_mass[warp];
        int ties_seen = 0, found = -1, last_kept = -1, first = seg0;
        const int groups = (seg1 - seg0 + 32 * GROUP - 1) / (32 * GROUP);
        if (groups <= 32) {
            // the last group that began at or below the target (sums are nondecreasing along the groups)
            const unsigned int at_or_below = __ballot_sync(0xffffffffu, lane < groups && warp_mass[warp] + began_at <= target);
            const int g = at_or_below ? 31 - __clz(at_or_below) : 0;
            cum += __shfl_sync(0xffffffffu, began_at, g);
            ties_seen = __shfl_sync(0xffffffffu, ties_at, g);
            first = seg0 + g * 32 * GROUP;
        }
        for (int base = first; base < seg1 && found < 0; base += 32 * GROUP) {
            float v[GROUP], p[GROUP];
            load_group(base, v);
            float part = 0.f;
#pragma unroll
            for (int c = 0; c < GROUP; ++c) {
                p[c] = mass_of(base + 32 * c + lane, v[c], ties_seen);
                part += p[c];
            }
            const float group = warp_total(part);
            const bool here = cum + group > target;
            float inside = cum;                       // the running sum inside the group, chunk by chunk
#pragma unroll
            for (int c = 0; c < GROUP; ++c) {
                const unsigned int kept = __ballot_sync(0xffffffffu, p[c] > 0.f);
                if (kept) last_kept = base + 32 * c + 31 - __clz(kept);
                if (here && found < 0) {
                    const float chunk = warp_total(p[c]);
                    if (inside + chunk > target) {
                        float incl = p[c];            // inclusive sums over the lanes of the chunk, in lane order
#pragma unroll
                        for (int off = 1; off < 32; off <<= 1) {
                            const float up = __shfl_up_sync(0xffffffffu, incl, off);
                            if (lane >= off) incl += up;
                        }
                        const unsigned int over = __ballot_sync(0xffffffffu, p[c] > 0.f && inside + incl > target);
                        found = over ? base + 32 * c + __ffs(over) - 1 : last_kept;      // else: rounding at the chunk's end
                    }
                    inside += chunk;
                }
            }
            if (here && found < 0) found = last_kept;  // rounding at the very end of the group
            cum += group;
        }
        if (found < 0) found = last_kept;              // rounding at the very end of the segment
        if (lane == 0 && found >= 0) atomicMax(&s_result, found);
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
