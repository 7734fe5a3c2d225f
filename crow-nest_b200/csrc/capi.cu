// Library-wide pieces of the C ABI: the per-thread error message, the device status word and the
// version string.
#include <cstdarg>
#include <cstdio>
#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"

__device__ int g_cn_status = 0;

static thread_local char t_err[512] = "";

void cn_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof t_err, fmt, ap);
    va_end(ap);
}

cudaError_t cn_allow_smem(const void* kernel, int bytes) {
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, int> done;  // (kernel, device) -> largest size allowed so far
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(mu);
    int& have = done[std::make_pair(kernel, dev)];
    if (have >= bytes) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) have = bytes;
    return e;
}

extern "C" const char* cn_last_error_string(void) { return t_err; }

extern "C" const char* cn_version(void) { return "crownest_b200 sm_100a"; }

extern "C" int cn_device_status(int* code_out) {
    int code = 0, zero = 0;
    CN_CUDA(cudaDeviceSynchronize());
    CN_CUDA(cudaMemcpyFromSymbol(&code, g_cn_status, sizeof(int)));
    if (code) CN_CUDA(cudaMemcpyToSymbol(g_cn_status, &zero, sizeof(int)));
    if (code_out) *code_out = code;
    if (code) CN_FAIL(CN_ERR_DEVICE, "a kernel gave up a bounded wait (device code %d)", code);
    return CN_OK;
}
