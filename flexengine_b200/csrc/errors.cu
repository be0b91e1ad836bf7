// Error reporting shared by every entry point of the library.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

static thread_local char g_last_error[512] = "";

void fe_set_error(const char* fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, args);
    va_end(args);
}

int fe_check_launch(const char* what) {
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        fe_set_error("%s: %s", what, cudaGetErrorString(err));
        return 2;
    }
    return 0;
}

// The number of multiprocessors of the current device: the one place kernels' launch heuristics take it from.
int fe_sm_count() {
    static int cached[64] = {0};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 1;
    if (cached[device] == 0) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) return 1;
        cached[device] = sms;
    }
    return cached[device];
}

extern "C" int fe_device_sm_count() { return fe_sm_count(); }

static int g_pdl = 0;

int fe_pdl_enabled() { return g_pdl; }

// Which kernels may overlap their preamble with the tail of the kernel before them: a set of FE_PDL_* classes
// (0: none).  A file's kernels belong to the class it defines before it includes common.cuh.
extern "C" void fe_set_pdl(int classes) { g_pdl = classes; }

extern "C" const char* fe_last_error() { return g_last_error; }

extern "C" int fe_abi_version() { return 1; }
