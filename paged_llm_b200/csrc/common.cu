// Error reporting of the kernel library; compiled into every module.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

int pl_fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return 1;
}

PL_EXPORT const char* pl_last_error() { return g_error; }
PL_EXPORT int pl_abi_version() { return 1; }

// A plain asynchronous host-to-device copy on `stream` (the Python side uses it for the one
// metadata copy of a step; going through the tensor library costs several times the call).
PL_EXPORT int pl_copy_h2d(void* dst, const void* src, long long bytes, cudaStream_t stream) {
    PL_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, stream));
    return 0;
}
