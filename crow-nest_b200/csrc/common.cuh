// Shared device/host helpers of the sm_100a kernels: status reporting, mbarrier and bulk-copy
// (TMA) PTX wrappers with bounded waits, NVFP4 decode primitives.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/crownest_ops.h"

// ---------------------------------------------------------------- host: errors
void cn_set_error(const char* fmt, ...);
#define CN_FAIL(code, ...)         \
    do {                           \
        cn_set_error(__VA_ARGS__); \
        return (code);             \
    } while (0)
#define CN_CUDA(expr)                                                                       \
    do {                                                                                    \
        cudaError_t e__ = (expr);                                                           \
        if (e__ != cudaSuccess) CN_FAIL(CN_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the CURRENT device only: remembered per (kernel, device),
// so that a process that drives several GPUs raises the limit on each of them (capi.cu).
cudaError_t cn_allow_smem(const void* kernel, int bytes);
#define CN_ALLOW_SMEM(kern, bytes) CN_CUDA(cn_allow_smem((const void*)(kern), (bytes)))

// ---------------------------------------------------------------- device: status word
// A wait that runs out of its iteration budget stores a code here (first writer wins) and the
// kernel returns; nothing traps and nothing spins without a limit.
extern __device__ int g_cn_status;
#define CN_DEV_WAIT_FULL 101
#define CN_DEV_WAIT_EMPTY 102
__device__ __forceinline__ void cn_dev_fail(int code) { atomicCAS(&g_cn_status, 0, code); }

// ---------------------------------------------------------------- device: mbarrier / bulk copy
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cta.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// the same with a suspend-time hint (ns): the thread may sleep in hardware until the phase completes or the
// hint runs out, instead of coming back to poll
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cta.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up (false) about one second after it started, far beyond any legitimate
// wait of these kernels (each try_wait itself blocks for a short hardware time slice).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try_wait_hint(bar, parity, 20000u)) return true;
        if (clock64() - t0 > 2000000000LL) return false;
    }
}
// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier. Both addresses
// 16-byte aligned, size a multiple of 16. No multicast.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// the same with an L2 evict-first hint: weights are streamed once per call
__device__ __forceinline__ void bulk_g2s_stream(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// programmatic dependent launch: wait for the producer grid's memory / let the consumer grid start
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launch with programmatic dependent launch allowed: the grid may be scheduled while its predecessor in the stream
// drains; the kernel calls pdl_wait() before it touches anything the predecessor wrote.
template <typename... KArgs, typename... Args>
inline cudaError_t cn_launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at, cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ---------------------------------------------------------------- device: NVFP4 decode
// UE4M3 scale byte -> f32 with the engine's reading: bit 7 ignored, e == 0 subnormal m * 2^-9,
// 0x7F -> 448 when `rule` (engine/src/cnq.rs:1287, engine/src/cpu_nvfp4.rs:88).
__device__ __forceinline__ float ue4m3_f32(uint32_t b, bool rule) {
    if (rule && b == 0x7Fu) b = 0x7Eu;
    const uint32_t e = (b >> 3) & 0xF, m = b & 7;
    return e == 0 ? (float)m * 1.953125e-3f : __uint_as_float(((e + 120u) << 23) | (m << 20));
}
// two E2M1 codes (one code byte; low nibble = even value) -> f16x2 (low half = low nibble);
// every E2M1 value is exact in f16
__device__ __forceinline__ uint32_t e2m1x2_to_f16x2(uint32_t byte) {
    uint32_t r;
    // the byte is taken with a vector mov: feeding cvt through cvt.u8.u32 gave wrong values when the source
    // register came straight from a byte load
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b0;\n\t}" : "=r"(r) : "r"(byte));
    return r;
}
// d = a * b + c with a, b f16 (exact product), c, d f32: one rounding
__device__ __forceinline__ float fma_f16_f32(uint16_t a, uint16_t b, float c) {
    float d;
    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(a), "h"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float f16lo_to_f32(uint32_t h2) { return __half2float(__ushort_as_half((uint16_t)(h2 & 0xffff))); }
__device__ __forceinline__ float f16hi_to_f32(uint32_t h2) { return __half2float(__ushort_as_half((uint16_t)(h2 >> 16))); }

// C (16 x 8, f32) += A (16 x 16, f16, row major) x B (16 x 8, f16, column major) on the warp's tensor cores.
// not volatile: a pure function of its operands, free to be scheduled between the shared-memory loads
__device__ __forceinline__ void mma16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// four code bytes of one word -> four f16x2 (byte i -> h[i]); the byte split is left to the
// assembler (vector mov), which measured 1.5x faster than shift-and-mask in front of each cvt
__device__ __forceinline__ void e2m1x8_to_f16x2(uint32_t word, uint32_t h[4]) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\tcvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
        : "r"(word));
}
// a0 += w.lo * x.lo, a1 += w.hi * x.hi for packed f16x2 w, x: products exact, f32 accumulate
__device__ __forceinline__ void fma2_f16_f32(float& a0, float& a1, uint32_t w, uint32_t x) {
    asm("{\n\t.reg .b16 wl, wh, xl, xh;\n\t"
        "mov.b32 {wl, wh}, %2;\n\tmov.b32 {xl, xh}, %3;\n\t"
        "fma.rn.f32.f16 %0, wl, xl, %0;\n\tfma.rn.f32.f16 %1, wh, xh, %1;\n\t}"
        : "+f"(a0), "+f"(a1)
        : "r"(w), "r"(x));
}
