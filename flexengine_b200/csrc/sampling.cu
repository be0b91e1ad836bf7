// Sampling on the device: a thread-block cluster per row of logits (one to eight blocks of 1,024 threads, by how
// many rows there are), each block with a contiguous slice of the vocabulary; what the blocks have to know of one
// another (maxima, histograms, masses, tie counts) they read from each other's shared memory.
//
// temperature == 0: the lowest index of the maximum (reference: engine/sampling/sampler.py:12-13).
// otherwise: x = logits / T; when 0 < k < V keep the k largest (ties go to the lowest indices);
// p = softmax over the kept (float32, reference sampler.py:16-22); the draw is the inverse of the
// cumulative distribution taken in index order at u * total, u in [0, 1) from a counter-based
// generator keyed by (request seed, number of the draw), so that a request's tokens do not
// depend on what else is in the batch (reference: engine/scheduler/state.py:64-65).
//
// The vocabulary is cut into 256 segments of equal length, whatever the cluster size; a warp walks a segment 32
// indices at a time, so every pass is coalesced.  Mass is summed chunk by chunk (a fixed butterfly inside the chunk,
// then a running sum), the segments' masses are added up by one thread in index order, and the pass that looks for
// the token repeats the same arithmetic, so the intervals of the tokens tile [0, total) and the result is the same
// on every run, in every batch and with every cluster size.
#include <math_constants.h>

#define FE_PDL_CLASS 8      // FE_PDL_SAMPLING
#include "common.cuh"

using namespace fe;

namespace {

constexpr int THREADS = 1024;
constexpr int WARPS = THREADS / 32;
constexpr int RADIX_LOADS = 8;      // loads on their way at once in a pass of the radix select
constexpr int SEGMENTS = 256;       // of a row; a block of a cluster of C owns SEGMENTS / C of them, a warp SEGMENTS / C / 32
constexpr int MAX_CLUSTER = 8;

__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// the same 32-bit variable in the shared memory of block ``rank`` of this cluster
__device__ __forceinline__ unsigned int ld_peer(const void* own, unsigned rank) {
    unsigned remote, v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"((unsigned)__cvta_generic_to_shared(own)), "r"(rank));
    asm volatile("ld.shared::cluster.u32 %0, [%1];\n" : "=r"(v) : "r"(remote));
    return v;
}

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
              const long long* __restrict__ draw, int* __restrict__ out, const int C) {
    griddep_wait();
    griddep_launch_dependents();
    __shared__ float s_val[THREADS];
    __shared__ int s_idx[THREADS];
    __shared__ float blk_val;                           // this block's maximum and its lowest index
    __shared__ int blk_idx;
    __shared__ unsigned int hist[2][256], warp_above[8];      // hist: one per parity of the pass
    __shared__ unsigned int warp_hist[WARPS][256];      // one histogram per warp: no two warps meet in a bin
    __shared__ unsigned int s_prefix, s_need;
    __shared__ float seg_mass[SEGMENTS];                // of this block's segments (the first SEGMENTS / C entries)
    __shared__ int seg_ties[SEGMENTS];
    __shared__ float mass_before[SEGMENTS + 1];         // of every segment of the row: mass before it; [SEGMENTS] = total
    __shared__ int ties_before[SEGMENTS];               // threshold ties before it, in index order

    const int row = blockIdx.x / C, tid = threadIdx.x;
    const unsigned rank = blockIdx.x % C;               // of this block in its cluster
    const float* x = logits + (size_t)row * ld;
    const float temp = temperature[row];
    // segments of S indices (a multiple of 32); this block's slice of the row is its segments side by side
    const int S = ((V + SEGMENTS - 1) / SEGMENTS + 31) / 32 * 32;
    const int per_block = SEGMENTS / C, per_warp = per_block / WARPS;
    const int lo = (int)min((long long)V, (long long)rank * per_block * S), hi = (int)min((long long)V, (long long)(rank + 1) * per_block * S);

    // ---- maximum and its lowest index (needed by both branches)
    float best = -CUDART_INF_F;
    int best_i = 0x7fffffff;
    const bool vector = (V & 3) == 0 && (reinterpret_cast<size_t>(x) & 15) == 0;      // lo is a multiple of 32
    if (vector) {
        // four logits per load, four loads in flight per thread: what bounds this pass is how many loads are on
        // their way at once
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const int n4 = hi >> 2;                          // hi is V or a multiple of 32
        const float4 none = make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
        for (int i = (lo >> 2) + tid; i < n4; i += 4 * THREADS) {
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
        for (int i = lo + tid; i < hi; i += THREADS) {
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
    if (tid == 0) { blk_val = s_val[0]; blk_idx = s_idx[0]; }
    cluster_sync();
    float max_logit = -CUDART_INF_F;
    int argmax = 0x7fffffff;
    for (int c = 0; c < C; ++c) {                       // the blocks' slices are in index order
        const float v = __uint_as_float(ld_peer(&blk_val, c));
        const int i = (int)ld_peer(&blk_idx, c);
        if (v > max_logit || (v == max_logit && i < argmax)) { max_logit = v; argmax = i; }
    }
    if (argmax == 0x7fffffff) argmax = 0;
    if (rank == 0 && tid == 0) out[row] = argmax;       // the answer at temperature 0, and what stands if no mass is found
    if (temp == 0.f) {
        cluster_sync();                                 // no block leaves while another may still read its maximum
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
            if (vector) {
                // the order does not matter here: four logits per load, four loads on their way per thread
                const float4* x4 = reinterpret_cast<const float4*>(x);
                const int n4 = hi >> 2;
                for (int i = (lo >> 2) + tid; i < n4; i += 4 * THREADS) {
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
                for (int i0 = lo + tid; i0 < hi; i0 += RADIX_LOADS * THREADS) {
                    float v[RADIX_LOADS];
#pragma unroll
                    for (int u = 0; u < RADIX_LOADS; ++u) v[u] = i0 + u * THREADS < hi ? x[i0 + u * THREADS] : 0.f;
#pragma unroll
                    for (int u = 0; u < RADIX_LOADS; ++u)
                        if (i0 + u * THREADS < hi) count(v[u]);
                }
            }
            __syncthreads();
            if (tid < 256) {
                unsigned int sum = 0;
                for (int w = 0; w < WARPS; ++w) sum += warp_hist[w][tid];
                hist[pass & 1][tid] = sum;
            }
            // One cluster barrier a pass: the histograms alternate between two buffers, and a block that writes a buffer
            // again (two passes on) has passed the barrier of the pass between, which its peers reach only after
            // they have read the earlier one.
            cluster_sync();
            // every block adds up the blocks' histograms and finds the bin for itself: the same in all of them.
            // Thread b ends up with the number of keys in bins b and above: a suffix sum inside each warp of 32 bins by
            // shuffles, then the totals of the warps above.
            unsigned int mine = 0, at_and_above = 0;
            if (tid < 256) {
                for (int c = 0; c < C; ++c) mine += ld_peer(&hist[pass & 1][tid], c);
                at_and_above = mine;
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const unsigned int up = __shfl_down_sync(0xffffffffu, at_and_above, off);
                    if ((tid & 31) + off < 32) at_and_above += up;
                }
                if ((tid & 31) == 0) warp_above[tid >> 5] = at_and_above;
            }
            const unsigned int remaining = s_need;
            __syncthreads();
            if (tid < 256) {
                for (int w = (tid >> 5) + 1; w < 8; ++w) at_and_above += warp_above[w];
                const unsigned int above = at_and_above - mine;                  // keys in bins above this one
                // the bin in which the count of larger keys passes what is still needed: exactly one thread finds it
                if (above < remaining && (at_and_above >= remaining || tid == 0)) {
                    s_prefix = prefix | ((unsigned int)tid << shift);
                    s_need = remaining - above;
                }
            }
            __syncthreads();
        }
        thr_key = s_prefix;
        need = s_need;             // how many of the keys equal to the threshold are kept
    }

    // ---- warp w walks its segments, one after the other, 32 indices at a time
    const int warp = tid >> 5, lane = tid & 31;
    const unsigned int below = (1u << lane) - 1u;

    // Eight chunks (256 indices) are loaded at once, so that eight loads are on their way together.
    constexpr int GROUP = 8;
    auto load_group = [&](int base, int seg1, float* v) {
#pragma unroll
        for (int c = 0; c < GROUP; ++c) {
            const int i = base + 32 * c + lane;
            v[c] = i < seg1 ? x[i] : 0.f;
        }
    };
    auto bounds = [&](int segment, int& seg0, int& seg1) {      // of segment ``segment`` of the row
        seg0 = (int)min((long long)V, (long long)segment * S);
        seg1 = (int)min((long long)V, (long long)seg0 + S);
    };

    // threshold ties of every segment, and from them the ties before each, in index order
    if (use_k) {
        for (int j = 0; j < per_warp; ++j) {
            const int mine = warp * per_warp + j;
            int seg0, seg1;
            bounds((int)rank * per_block + mine, seg0, seg1);
            int ties = 0;
            for (int base = seg0; base < seg1; base += 32 * GROUP) {
                float v[GROUP];
                load_group(base, seg1, v);
#pragma unroll
                for (int c = 0; c < GROUP; ++c)
                    ties += __popc(__ballot_sync(0xffffffffu, base + 32 * c + lane < seg1 && ordered_key(sanitize(v[c])) == thr_key));
            }
            if (lane == 0) seg_ties[mine] = ties;
        }
        cluster_sync();
        if (tid < SEGMENTS) ties_before[tid] = (int)ld_peer(&seg_ties[tid % per_block], tid / per_block);
        __syncthreads();
        if (tid == 0) {
            int run = 0;
            for (int g = 0; g < SEGMENTS; ++g) { const int t = ties_before[g]; ties_before[g] = run; run += t; }
        }
        __syncthreads();
    }
    const float inv_temp = 1.f / temp, inv_shift = max_logit * inv_temp;

    // the unnormalised probability of index ``i`` with logit ``raw`` (0 when it is cut off), and the running tie count
    auto mass_of = [&](int i, int seg1, int tie_base, float raw, int& ties_seen) -> float {
        const bool in = i < seg1;
        const float v = sanitize(raw);
        bool keep = in;
        if (use_k) {
            const unsigned int key = ordered_key(v);
            const unsigned int tied = __ballot_sync(0xffffffffu, in && key == thr_key);
            const int rank_of_tie = tie_base + ties_seen + __popc(tied & below);
            keep = in && (key > thr_key || (key == thr_key && (unsigned int)rank_of_tie < need));
            ties_seen += __popc(tied);
        }
        return keep ? expf(v * inv_temp - inv_shift) : 0.f;
    };

    // mass of a segment: per group, each lane adds its eight values in order, the lanes' sums are added by a fixed
    // butterfly, and the groups' sums are added up as the walk goes
    for (int j = 0; j < per_warp; ++j) {
        const int mine = warp * per_warp + j, segment = (int)rank * per_block + mine;
        int seg0, seg1;
        bounds(segment, seg0, seg1);
        const int tie_base = use_k ? ties_before[segment] : 0;
        float cum = 0.f;
        int ties_seen = 0;
        for (int base = seg0; base < seg1; base += 32 * GROUP) {
            float v[GROUP];
            load_group(base, seg1, v);
            float part = 0.f;
#pragma unroll
            for (int c = 0; c < GROUP; ++c) part += mass_of(base + 32 * c + lane, seg1, tie_base, v[c], ties_seen);
            cum += warp_total(part);
        }
        if (lane == 0) seg_mass[mine] = cum;
    }
    cluster_sync();
    if (tid < SEGMENTS) mass_before[tid] = __uint_as_float(ld_peer(&seg_mass[tid % per_block], tid / per_block));
    __syncthreads();
    if (tid == 0) {
        // accumulated by one thread in index order: nondecreasing, so the segments' intervals tile [0, total)
        float run = 0.f;
        for (int g = 0; g < SEGMENTS; ++g) { const float m = mass_before[g]; mass_before[g] = run; run += m; }
        mass_before[SEGMENTS] = run;
    }
    cluster_sync();                                     // every block has read the others' masses (and ties): they may leave
    const float total = mass_before[SEGMENTS];
    const unsigned long long bits = splitmix64(splitmix64((unsigned long long)seed[row]) + (unsigned long long)draw[row]);
    const float u = (float)(bits >> 40) * (1.0f / 16777216.0f);
    float target = u * total;
    if (target >= total) target = nextafterf(total, 0.f);

    // the warp into whose segment the target falls repeats its walk with the same arithmetic, stops at the group
    // that takes the running sum past the target, and looks for the token inside it chunk by chunk, lane by lane
    for (int j = 0; j < per_warp; ++j) {
        const int segment = (int)rank * per_block + warp * per_warp + j;
        if (!(mass_before[segment] <= target && target < mass_before[segment + 1])) continue;
        int seg0, seg1;
        bounds(segment, seg0, seg1);
        const int tie_base = use_k ? ties_before[segment] : 0;
        float cum = mass_before[segment];
        int ties_seen = 0, found = -1, last_kept = -1;
        for (int base = seg0; base < seg1 && found < 0; base += 32 * GROUP) {
            float v[GROUP], p[GROUP];
            load_group(base, seg1, v);
            float part = 0.f;
#pragma unroll
            for (int c = 0; c < GROUP; ++c) {
                p[c] = mass_of(base + 32 * c + lane, seg1, tie_base, v[c], ties_seen);
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
        // exactly one segment of the row holds the target; block 0's argmax was written two cluster barriers ago
        if (lane == 0 && found >= 0) out[row] = found;
    }
}

}  // namespace

// How many clusters of ``blocks`` blocks of the kernel the device holds at once (a cluster lives inside one of the GPU's
// processing clusters); asked of the driver once per size and device.
static int clusters_resident(int blocks) {
    static int cached[64][4];
    int device = 0, slot = blocks == 8 ? 3 : blocks == 4 ? 2 : blocks == 2 ? 1 : 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
    if (cached[device][slot] == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)blocks);
        cfg.blockDim = dim3(THREADS);
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = blocks;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, sample_kernel, &cfg) != cudaSuccess) {
            cudaGetLastError();
            clusters = 0;
        }
        cached[device][slot] = clusters > 0 ? clusters : -1;
    }
    return cached[device][slot] > 0 ? cached[device][slot] : 0;
}

// How many blocks share a row: the most that still lets every row's cluster be resident at once (16 rows of eight
// blocks are 128 blocks on 148 SMs, but only 15 such clusters fit the processing clusters: a second round).
static int blocks_per_row(int R) {
    for (int c = MAX_CLUSTER; c > 1; c >>= 1)
        if (R <= clusters_resident(c)) return c;
    return 1;
}

extern "C" int fe_sample(const float* logits, long long ld, int R, int V, const float* temperature,
                         const int* top_k, const long long* seed, const long long* draw, int* out,
                         cudaStream_t stream) {
    FE_REQUIRE(R >= 0 && V > 0 && ld >= V, "sample: bad sizes R=%d V=%d ld=%lld", R, V, ld);
    FE_REQUIRE((long long)R * MAX_CLUSTER < (1LL << 31), "sample: too many rows");
    if (R == 0) return 0;
    const int C = blocks_per_row(R);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(R * C));
    cfg.blockDim = dim3(THREADS);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, sample_kernel, logits, ld, V, temperature, top_k, seed, draw, out, C);
    FE_REQUIRE(err == cudaSuccess, "sample (clusters of %d): %s", C, cudaGetErrorString(err));
    return fe_check_launch("sample");
}

// The same with a given number of blocks a row (1, 2, 4 or 8): the tokens are the same for every number.
extern "C" int fe_sample_blocks(const float* logits, long long ld, int R, int V, const float* temperature,
                                const int* top_k, const long long* seed, const long long* draw, int* out,
                                int blocks, cudaStream_t stream) {
    FE_REQUIRE(R >= 0 && V > 0 && ld >= V, "sample: bad sizes R=%d V=%d ld=%lld", R, V, ld);
    FE_REQUIRE(blocks == 1 || blocks == 2 || blocks == 4 || blocks == 8, "sample: %d blocks a row; 1, 2, 4 or 8", blocks);
    if (R == 0) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(R * blocks));
    cfg.blockDim = dim3(THREADS);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = blocks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, sample_kernel, logits, ld, V, temperature, top_k, seed, draw, out, blocks);
    FE_REQUIRE(err == cudaSuccess, "sample (clusters of %d): %s", blocks, cudaGetErrorString(err));
    return fe_check_launch("sample");
}
