// Shared helpers of the kernels: element conversion, warp and block reductions, error
// reporting.  Every kernel is templated on the element type (float for the true 32-bit
// path, __nv_bfloat16 for serving) and does its arithmetic in float.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// dtype codes of the C interface
#define FE_F32 0
#define FE_BF16 1

// bits a kernel may set in the device status word (it then skips the access)
#define FE_STATUS_BAD_TOKEN 1
#define FE_STATUS_BAD_PAGE 2
#define FE_STATUS_BAD_SLOT 4
#define FE_STATUS_WAIT_EXPIRED 8

namespace fe {

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the block; every thread gets the result.  ``scratch`` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                 // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float w = lane < warps ? scratch[lane] : 0.f;
        w = warp_sum(w);
        if (lane == 0) scratch[32] = w;
    }
    __syncthreads();
    return scratch[32];
}

// Load 8 consecutive elements (16-byte aligned for bf16, 32-byte span for float) as floats.
template <typename T> __device__ __forceinline__ void load8(const T* p, float* out);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* out) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, float* out) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// Store 8 consecutive elements from floats (same alignment as load8).
template <typename T> __device__ __forceinline__ void store8(T* p, const float* v);
template <> __device__ __forceinline__ void store8<float>(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<bf16>(bf16* p, const float* v) {
    uint4 raw;
    unsigned* w = reinterpret_cast<unsigned*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const unsigned*>(&pair);
    }
    *reinterpret_cast<uint4*>(p) = raw;
}

// Programmatic dependent launch: a kernel launched through fe::launch may begin while the kernel
// before it in the stream is still running.  Everything it reads that an earlier kernel wrote,
// and every write, must come after griddep_wait(); only data that no kernel writes (weights)
// may be touched before.  launch_dependents lets the next kernel start its own preamble; it is
// called after the wait, so that at most one kernel is resident ahead of the one that runs
// (called before, every later kernel of a graph piles onto the SMs and starves the running one).
// Without the launch attribute both are no-ops, and the attribute is off unless fe_set_pdl names classes of
// kernels: inside the CUDA graph of a decode step (28 layers, B200) a step took 3.24 ms without it; with it on the
// weight-streaming products alone 3.36 ms when they never trigger (the dependent starts as the last block exits),
// 4.25 ms with the trigger behind their main loop and 5.5 ms with the trigger first: the earlier the dependent's
// blocks become resident, the slower the step.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Worker ``w`` of ``workers`` threads asks for its share of the 128-byte lines of [base, base + bytes) to be brought
// into L2.  Used by kernels that leave the memory system idle (a norm over a few rows, decode attention) to start
// the weight matrix that the NEXT kernel streams: blocks beyond their own grid do nothing else.  A prefetch changes
// no data, so it needs no ordering with other kernels.
__device__ __forceinline__ void prefetch_l2_share(const void* base, long long bytes, long long w, long long workers) {
    const char* p = static_cast<const char*>(base);
    for (long long off = w * 128; off < bytes; off += workers * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p + off));
}

}  // namespace fe

// Host side: the last error message of this thread, and a checked launch epilogue.
void fe_set_error(const char* fmt, ...);
int fe_check_launch(const char* what);
int fe_pdl_enabled();
int fe_sm_count();      // multiprocessors of the current device (asked once per device)

// Classes of kernels for fe_set_pdl: a source file names its own before including this header.
#define FE_PDL_STREAMING_GEMM 1
#define FE_PDL_DECODE_ATTENTION 2
#define FE_PDL_ELEMENTWISE 4
#define FE_PDL_SAMPLING 8
#define FE_PDL_OTHER 128
#ifndef FE_PDL_CLASS
#define FE_PDL_CLASS FE_PDL_OTHER
#endif

namespace fe {
// Launch with the programmatic-stream-serialization attribute (when enabled for this file's class of kernels).
template <typename... KArgs, typename... Args>
inline void launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = (fe_pdl_enabled() & FE_PDL_CLASS) != 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);       // errors surface in fe_check_launch
}
}  // namespace fe

#define FE_REQUIRE(cond, ...)            \
    do {                                 \
        if (!(cond)) {                   \
            fe_set_error(__VA_ARGS__);   \
            return 1;                    \
        }                                \
    } while (0)
