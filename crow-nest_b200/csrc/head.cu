// The small operators either side of the GEMV chain: residual add + RMSNorm and the lm_head's argmax.
//
// add_rmsnorm supersedes add_rms_1k (engine/src/kernels_p2.rs:609-633; host call Engine::add_norm): h += y (when y is
// given), out = h * rsqrt(mean(h^2) + eps) * (1 + w), f32, one CTA of 1024 threads per row with the reference's summation
// order (strided per-thread sums, xor shuffles inside a warp, the 32 warp sums left to right).
// argmax supersedes argmax_k (engine/src/kernels.rs:4238-4261; call site engine/src/gen.rs:5638-5641): thread t scans
// logits t, t + 1024, .. keeping the first strict maximum, then a stride-halving tree in which the lower thread wins ties -
// the reference's tie rule, which is not "lowest index" across threads, reproduced as it is.
// lm_head + argmax = the vocabulary GEMV (cn_nvfp4_gemv, the largest matrix of a token) followed by the argmax of every row.
#include "common.cuh"
#include "nvfp4_gemv.cuh"

namespace {

__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ y, const float* __restrict__ w,
                                                           float* __restrict__ out, int hidden, float eps) {
    __shared__ float red[32];
    pdl_wait();
    float* hp = h + (size_t)blockIdx.x * hidden;
    const float* yp = y ? y + (size_t)blockIdx.x * hidden : nullptr;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += 1024) {
        float v = hp[i];
        if (yp) {
            v = __fadd_rn(v, yp[i]);
            hp[i] = v;
        }
        ss = __fadd_rn(ss, __fmul_rn(v, v));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; i++) ss = __fadd_rn(ss, red[i]);
    const float rms = rsqrtf(__fadd_rn(ss / (float)hidden, eps));
    float* op = out + (size_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += 1024) op[i] = __fmul_rn(__fmul_rn(hp[i], rms), __fadd_rn(1.0f, w[i]));
    pdl_launch_dependents();
}

template <int XT>
__global__ void __launch_bounds__(1024) argmax_kernel(const void* __restrict__ logits, int32_t* __restrict__ out, int n, size_t ld) {
    __shared__ float rb[1024];
    __shared__ int ri[1024];
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * ld;
    float best = -3.0e38f;
    int bi = 0;
    for (int i = threadIdx.x; i < n; i += 1024) {
        const float v = XT == 1 ? __bfloat162float(((const __nv_bfloat16*)logits)[base + i]) : ((const float*)logits)[base + i];
        if (v > best) best = v, bi = i;
    }
    rb[threadIdx.x] = best;
    ri[threadIdx.x] = bi;
    __syncthreads();
    for (int st = 512; st > 0; st >>= 1) {
        if (threadIdx.x < st && rb[threadIdx.x + st] > rb[threadIdx.x]) {
            rb[threadIdx.x] = rb[threadIdx.x + st];
            ri[threadIdx.x] = ri[threadIdx.x + st];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[blockIdx.x] = ri[0];
}

}  // namespace

extern "C" int cn_add_rmsnorm(float* h, const float* y, const float* w, float* out, int rows, int hidden, float eps, cn_stream_t stream) {
    if (!h || !w || !out || rows < 1 || hidden < 1) CN_FAIL(CN_ERR_SHAPE, "cn_add_rmsnorm: rows %d, hidden %d", rows, hidden);
    CN_CUDA(cn_launch_pdl(add_rmsnorm_kernel, dim3(rows), dim3(1024), 0, (cudaStream_t)stream, h, y, w, out, hidden, eps));
    return CN_OK;
}

extern "C" int cn_argmax(const void* logits, int32_t* out, int rows, int n, int ld, int dtype, cn_stream_t stream) {
    if (!logits || !out || rows < 1 || n < 1 || ld < n) CN_FAIL(CN_ERR_SHAPE, "cn_argmax: rows %d, n %d, ld %d", rows, n, ld);
    if (dtype == CN_BF16)
        CN_CUDA(cn_launch_pdl(argmax_kernel<1>, dim3(rows), dim3(1024), 0, (cudaStream_t)stream, logits, out, n, (size_t)ld));
    else if (dtype == CN_F32)
        CN_CUDA(cn_launch_pdl(argmax_kernel<0>, dim3(rows), dim3(1024), 0, (cudaStream_t)stream, logits, out, n, (size_t)ld));
    else
        CN_FAIL(CN_ERR_SHAPE, "cn_argmax: dtype %d is neither CN_F32 nor CN_BF16", dtype);
    return CN_OK;
}

extern "C" int cn_lm_head_argmax(const void* w, const float* gs, const void* x, void* logits, int32_t* tokens, int vocab, int k, int m, int dtype,
                                 cn_stream_t stream) {
    if (!tokens || !logits) CN_FAIL(CN_ERR_SHAPE, "cn_lm_head_argmax: null output");
    GemvCall a = {};
    a.w0 = w, a.gs0 = gs, a.x = x, a.y = logits, a.rows = vocab, a.k = k, a.m = m, a.ldy = vocab, a.dtype = dtype;
    if (int rc = cn_gemv_launch(a, (cudaStream_t)stream, "cn_lm_head_argmax")) return rc;
    return cn_argmax(logits, tokens, m, vocab, vocab, dtype, stream);
}
