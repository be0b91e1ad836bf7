// One decoder layer of the usual arrangement as ONE call from the host: pre-norm, attention with biased
// query/key/value projection and half-split rotation over the paged cache, SwiGLU feed-forward
// (x += out(attn(norm(x))); x += down(silu(gate(norm(x))) * up(norm(x))), as inference/models/qwen2.py:95-130 of
// the reference runs it module by module).
//
// Nothing new is computed here: the function launches the same kernels of this library, in the same order and with
// the same arguments, that the Python parts launch one by one for a step of more than a handful of tokens, and the
// same library products (cuBLAS, float accumulation).  What it saves is the host: a prompt portion of a 28-layer
// model is about 300 launches, each of which costs several microseconds through the interpreter, more than the
// device needs for a short portion.  With the layer as one call the host is out of the way.
//
// cuBLAS is looked up at run time in the process (the host application has loaded it already); when it cannot be
// found the function says so and the caller keeps launching kernel by kernel.
#include <cublas_v2.h>
#include <dlfcn.h>

#include "common.cuh"

// entry points of this library (elementwise.cu, attention_*.cu, gemm_tcgen05.cu)
extern "C" int fe_add_rmsnorm(float* residual, const void* delta, const float* weight, float eps, void* out, const int* rows,
                              int n_out, int H, int n_rows_total, int dtype, const void* upcoming, long long upcoming_bytes,
                              cudaStream_t stream);
extern "C" int fe_qkv_bias_rope_cache(const void* src, int src_float, void* qkv, const float* bias, const int* positions,
                                      const float* inv_freq, int rot, const int* slot_mapping, void* kc, void* vc, int T,
                                      int nq, int nkv, int d, int ps, long long num_slots, int dtype, int* status,
                                      cudaStream_t stream);
extern "C" int fe_swiglu(const void* gate_up, void* out, int T, int I, int dtype, cudaStream_t stream);
extern "C" int fe_gemm_tcgen05(const void* x, const void* W, void* out, int M, int N, int K, int epilogue, int* status,
                               cudaStream_t stream);
extern "C" int fe_paged_prefill_tcgen05(const void* q, long long q_stride, void* out, long long out_stride, const void* kc,
                                        const void* vc, const int* block_table, int bt_stride, const int* cu_q,
                                        const int* q_start, int requests, int max_q_len, int nq, int nkv, int d, int ps,
                                        int num_pages, float scale, int window, int splits, void* scratch,
                                        long long total_tokens, int* status, cudaStream_t stream);
extern "C" int fe_paged_prefill_mma(const void* q, long long q_stride, void* out, long long out_stride, const void* kc,
                                    const void* vc, const int* block_table, int bt_stride, const int* cu_q,
                                    const int* q_start, int requests, int max_q_len, int nq, int nkv, int d, int ps,
                                    int num_pages, float scale, int window, int* status, cudaStream_t stream);
extern "C" int fe_paged_decode_cluster(const void* q, long long q_stride, void* out, long long out_stride, const void* kc,
                                       const void* vc, const int* block_table, int bt_stride, const int* cu_q,
                                       const int* q_start, int requests, int nq, int nkv, int d, int ps, int num_pages,
                                       float scale, int window, int splits, int* status, cudaStream_t stream);
extern "C" int fe_paged_decode_mma(const void* q, long long q_stride, void* out, long long out_stride, void* scratch,
                                   const void* kc, const void* vc, const int* block_table, int bt_stride, const int* cu_q,
                                   const int* q_start, int requests, int nq, int nkv, int d, int ps, int num_pages,
                                   float scale, int window, int splits, int* status, cudaStream_t stream);

namespace {

typedef cublasStatus_t (*CreateFn)(cublasHandle_t*);
typedef cublasStatus_t (*SetStreamFn)(cublasHandle_t, cudaStream_t);
typedef cublasStatus_t (*SetMathModeFn)(cublasHandle_t, cublasMath_t);
typedef cublasStatus_t (*GemmExFn)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*, const void*,
                                   cudaDataType, int, const void*, cudaDataType, int, const void*, void*, cudaDataType, int,
                                   cublasComputeType_t, cublasGemmAlgo_t);

struct Blas {
    bool looked = false;
    CreateFn create = nullptr;
    SetStreamFn set_stream = nullptr;
    SetMathModeFn set_math_mode = nullptr;
    GemmExFn gemm_ex = nullptr;
    cublasHandle_t handle[64] = {};
};
Blas g_blas;

// The library's handle for the current device, or nullptr with the reason in fe_last_error().
cublasHandle_t blas_handle() {
    if (!g_blas.looked) {
        g_blas.looked = true;
        void* lib = dlopen("libcublas.so.12", RTLD_NOW | RTLD_GLOBAL);
        if (lib == nullptr) lib = dlopen("libcublas.so", RTLD_NOW | RTLD_GLOBAL);
        if (lib != nullptr) {
            g_blas.create = (CreateFn)dlsym(lib, "cublasCreate_v2");
            g_blas.set_stream = (SetStreamFn)dlsym(lib, "cublasSetStream_v2");
            g_blas.gemm_ex = (GemmExFn)dlsym(lib, "cublasGemmEx");
            g_blas.set_math_mode = (SetMathModeFn)dlsym(lib, "cublasSetMathMode");
        }
    }
    if (!g_blas.create || !g_blas.set_stream || !g_blas.gemm_ex) {
        fe_set_error("layer_forward: cuBLAS was not found in this process");
        return nullptr;
    }
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
        fe_set_error("layer_forward: no current device");
        return nullptr;
    }
    if (g_blas.handle[device] == nullptr) {
        if (g_blas.create(&g_blas.handle[device]) != CUBLAS_STATUS_SUCCESS) {
            g_blas.handle[device] = nullptr;
            fe_set_error("layer_forward: cublasCreate failed");
            return nullptr;
        }
        // A product split along K adds its partial sums up in float, not in bfloat16 (the library's default allows
        // the latter: errors of two to four times a bfloat16 rounding at K of a few thousand).
        if (g_blas.set_math_mode)
            g_blas.set_math_mode(g_blas.handle[device],
                                 (cublasMath_t)(CUBLAS_DEFAULT_MATH | CUBLAS_MATH_DISALLOW_REDUCED_PRECISION_REDUCTION));
    }
    return g_blas.handle[device];
}

// y[M, N] = x[M, K] w[N, K]^T, bfloat16 operands, float accumulation; y bfloat16 or float.
int product(cublasHandle_t handle, const void* x, const void* w, void* y, int M, int N, int K, bool y_float) {
    const float one = 1.f, zero = 0.f;
    const cublasStatus_t rc = g_blas.gemm_ex(handle, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &one, w, CUDA_R_16BF, K, x, CUDA_R_16BF, K,
                                             &zero, y, y_float ? CUDA_R_32F : CUDA_R_16BF, N, CUBLAS_COMPUTE_32F,
                                             CUBLAS_GEMM_DEFAULT_TENSOR_OP);
    FE_REQUIRE(rc == CUBLAS_STATUS_SUCCESS, "layer_forward: cublasGemmEx failed with status %d (M=%d N=%d K=%d)", (int)rc, M, N, K);
    return 0;
}

size_t align_up(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace

// What does not change from step to step: the layer's weights and sizes.
struct FeLayer {
    const float* input_norm;        // [H]
    const float* post_norm;         // [H]
    const void* qkv_weight;         // [(nq + 2 nkv) d, H] bfloat16
    const float* qkv_bias;          // [(nq + 2 nkv) d] or null
    const void* out_weight;         // [H, nq d]
    const void* gate_up_weight;     // [2 I, H]
    const void* down_weight;        // [H, I]
    const float* inv_freq;          // [rot / 2]
    float eps, scale;
    int hidden, nq, nkv, d, intermediate, rot, window;
};

// What a step brings: its index arrays on the device, sizes, and which attention kernel its shape takes.
struct FeStep {
    const int* positions;           // [T]
    const int* slot_mapping;        // [T] or null (a run entry that reads another entry's cache)
    const int* block_table;         // [R, bt_stride]
    const int* cu_q;                // [R + 1]
    const int* q_start;             // [R]
    float* residual;                // [T, H] float, updated in place
    void* workspace;                // fe_layer_workspace_bytes() bytes, 256-byte aligned
    void* attention_scratch;        // what the chosen attention kernel needs for its splits, or null
    int* status;
    long long workspace_bytes;
    int T, R, bt_stride, max_q_len;
    int page_size, num_pages;       // of the cache group the layer keeps its keys and values in
    int attention;                  // 0 decode, cluster; 1 decode, two kernels; 2 prefill, tcgen05; 3 prefill, mma.sync
    int splits;
    int gate_up_tcgen05;            // the fused tcgen05 product for gate/up + SwiGLU (many rows)
};

extern "C" long long fe_layer_workspace_bytes(int T, int hidden, int nq, int nkv, int d, int intermediate) {
    const size_t qkv = (size_t)(nq + 2 * nkv) * d;
    return (long long)(align_up((size_t)T * hidden * 2) + align_up((size_t)T * qkv * 4) + align_up((size_t)T * qkv * 2) +
                       align_up((size_t)T * nq * d * 2) + align_up((size_t)T * hidden * 2) +
                       align_up((size_t)T * 2 * intermediate * 2) + align_up((size_t)T * intermediate * 2));
}

// residual += attention branch; returns in ``pending_out`` [T, H] (bfloat16) the feed-forward branch's output, which the
// next norm adds.  ``pending_in`` (may be null): the output of the branch before this layer, not yet added.
// ``k_cache``, ``v_cache``: this layer's slot of the cache group, [num_pages, nkv, page_size, d] bfloat16 each.
extern "C" int fe_layer_forward(const FeLayer* layer, const FeStep* step, void* k_cache, void* v_cache, const void* pending_in,
                                void* pending_out, cudaStream_t stream) {
    FE_REQUIRE(layer != nullptr && step != nullptr && pending_out != nullptr && k_cache != nullptr && v_cache != nullptr,
               "layer_forward: a null argument");
    const FeLayer& L = *layer;
    const FeStep& S = *step;
    const int T = S.T, H = L.hidden, Wq = (L.nq + 2 * L.nkv) * L.d, I = L.intermediate;
    FE_REQUIRE(T > 0 && S.R > 0 && H > 0 && I > 0, "layer_forward: bad sizes");
    FE_REQUIRE(S.workspace_bytes >= fe_layer_workspace_bytes(T, H, L.nq, L.nkv, L.d, I), "layer_forward: the workspace is too small");
    cublasHandle_t handle = blas_handle();
    if (handle == nullptr) return 3;
    FE_REQUIRE(g_blas.set_stream(handle, stream) == CUBLAS_STATUS_SUCCESS, "layer_forward: cublasSetStream failed");

    char* at = static_cast<char*>(S.workspace);
    auto take = [&](size_t bytes) { char* p = at; at += align_up(bytes); return (void*)p; };
    void* h = take((size_t)T * H * 2);
    void* qkv32 = take((size_t)T * Wq * 4);
    void* qkv = take((size_t)T * Wq * 2);
    void* heads = take((size_t)T * L.nq * L.d * 2);
    void* mixed = take((size_t)T * H * 2);
    void* gate_up = take((size_t)T * 2 * I * 2);
    void* act = take((size_t)T * I * 2);

    // ---- attention branch ----
    if (fe_add_rmsnorm(S.residual, pending_in, L.input_norm, L.eps, h, nullptr, T, H, T, FE_BF16, nullptr, 0, stream)) return 1;
    if (product(handle, h, L.qkv_weight, qkv32, T, Wq, H, true)) return 1;
    const long long num_slots = (long long)S.num_pages * S.page_size;
    if (fe_qkv_bias_rope_cache(qkv32, 1, qkv, L.qkv_bias, S.positions, L.inv_freq, L.rot, S.slot_mapping, k_cache, v_cache,
                               T, L.nq, L.nkv, L.d, S.page_size, num_slots, FE_BF16, S.status, stream)) return 1;
    const long long out_stride = (long long)L.nq * L.d;
    int rc;
    switch (S.attention) {
        case 0:
            rc = fe_paged_decode_cluster(qkv, Wq, heads, out_stride, k_cache, v_cache, S.block_table, S.bt_stride, S.cu_q,
                                         S.q_start, S.R, L.nq, L.nkv, L.d, S.page_size, S.num_pages, L.scale, L.window, S.splits,
                                         S.status, stream);
            break;
        case 1:
            rc = fe_paged_decode_mma(qkv, Wq, heads, out_stride, S.attention_scratch, k_cache, v_cache, S.block_table,
                                     S.bt_stride, S.cu_q, S.q_start, S.R, L.nq, L.nkv, L.d, S.page_size, S.num_pages, L.scale,
                                     L.window, S.splits, S.status, stream);
            break;
        case 2:
            rc = fe_paged_prefill_tcgen05(qkv, Wq, heads, out_stride, k_cache, v_cache, S.block_table, S.bt_stride, S.cu_q,
                                          S.q_start, S.R, S.max_q_len, L.nq, L.nkv, L.d, S.page_size, S.num_pages, L.scale,
                                          L.window, S.splits, S.attention_scratch, T, S.status, stream);
            break;
        case 3:
            rc = fe_paged_prefill_mma(qkv, Wq, heads, out_stride, k_cache, v_cache, S.block_table, S.bt_stride, S.cu_q,
                                      S.q_start, S.R, S.max_q_len, L.nq, L.nkv, L.d, S.page_size, S.num_pages, L.scale, L.window,
                                      S.status, stream);
            break;
        default:
            FE_REQUIRE(false, "layer_forward: unknown attention kind %d", S.attention);
    }
    if (rc) return rc;
    if (product(handle, heads, L.out_weight, mixed, T, H, L.nq * L.d, false)) return 1;

    // ---- feed-forward branch ----
    if (fe_add_rmsnorm(S.residual, mixed, L.post_norm, L.eps, h, nullptr, T, H, T, FE_BF16, nullptr, 0, stream)) return 1;
    if (S.gate_up_tcgen05) {
        if (fe_gemm_tcgen05(h, L.gate_up_weight, act, T, 2 * I, H, 2, S.status, stream)) return 1;
    } else {
        if (product(handle, h, L.gate_up_weight, gate_up, T, 2 * I, H, false)) return 1;
        if (fe_swiglu(gate_up, act, T, I, FE_BF16, stream)) return 1;
    }
    return product(handle, act, L.down_weight, pending_out, T, H, I, false);
}
