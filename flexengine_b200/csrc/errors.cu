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

static int g_pdl = 1;

int fe_pdl_enabled() { return g_pdl; }

// 1: kernels may overlap their preamble with the tail of the kernel before them (default); 0: off.
extern "C" void fe_set_pdl(int on) { g_pdl = on ? 1 : 0; }

extern "C" const char* fe_last_error() { return g_last_error; }

extern "C" int fe_abi_version() { return 1; }
