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

// The book behind cn_allow_smem: the largest dynamic shared-memory size already allowed per (kernel, device). Returns 1
// when `bytes` is not covered yet (and records it when commit is set), 0 when it is. No CUDA call: testable without a GPU.
extern "C" int cn_smem_book(const void* kernel, int device, int bytes, int commit) {
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, int> done;
    std::lock_guard<std::mutex> lock(mu);
    int& have = done[std::make_pair(kernel, device)];
    if (have >= bytes) return 0;
    if (commit) have = bytes;
    return 1;
}

cudaError_t cn_allow_smem(const void* kernel, int bytes) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (!cn_smem_book(kernel, dev, bytes, 0)) return cudaSuccess;
    // the attribute belongs to the device that is current: every GPU of a process gets its own call
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) cn_smem_book(kernel, dev, bytes, 1);
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
