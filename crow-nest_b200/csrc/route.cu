// MoE routing on the device: softmax top-k (Flash-Next) and sigmoid top-k (GLM), bit-exact
// indices against the host twins.
//
// Supersedes router_top10 (engine/src/kernels.rs:3109-3171; the residency bookkeeping of that
// kernel - cold mask, hit counters, pointer gather - is not part of this path: the MoE operator
// reads its pointer tables directly) and glm5_router_sig_topk (engine/src/kernels_glm5_moe.cu:44-96,
// host twin glm5_moe::route_from_logits, engine/src/glm5_moe.rs:196-236).
//
// One CTA per token row, one thread per expert slot (P = next power of two >= E, <= 1024).
// The softmax sum is the pairwise tree of the reference kernel (stride P/2, P/4, ..), so it rounds
// exactly as there; maxima and index minima do not depend on the order and are taken with warp
// shuffles (two barriers per selection round). exp() is taken in f64 and rounded once, which gives the
// correctly rounded f32 value the host twins' libm returns; selection is K rounds of "best value,
// lowest index on ties", as in both reference routers.
#include "common.cuh"

namespace {

__device__ __forceinline__ float exp_rn(float x) { return (float)exp((double)x); }

// max over the block's values (NaN operands are ignored, as fmaxf does in the reference's tree; the value does
// not depend on the order). buf: 32 floats; one barrier, the next use of `buf` must be a barrier later.
__device__ __forceinline__ float block_max(float v, float* buf, int e, int P) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((e & 31) == 0) buf[e >> 5] = v;
    __syncthreads();
    float r = (e & 31) < (P >> 5) ? buf[e & 31] : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
    return r;
}
__device__ __forceinline__ int block_min(int v, int* buf, int e, int P) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((e & 31) == 0) buf[e >> 5] = v;
    __syncthreads();
    int r = (e & 31) < (P >> 5) ? buf[e & 31] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r = min(r, __shfl_xor_sync(0xffffffffu, r, o));
    return r;
}

// One round of "best value, lowest index on ties" over the live slots: the best value, then the lowest slot that
// holds it (E when no live slot compares equal, i.e. a row of NaN). Two barriers; bmax / bmin: 32 words each.
__device__ __forceinline__ int pick_best(float* bmax, int* bmin, float mine, bool alive, int e, int P, int E) {
    const float best = block_max(alive ? mine : -INFINITY, bmax, e, P);
    return block_min((alive && mine == best) ? e : E, bmin, e, P);
}

// red[0..P) summed by the reference's stride-halving tree (red[e] += red[e + st], st = P/2, P/4, ..): strides of 32
// and more through shared memory, the last five inside warp 0 with the same pairs; every thread gets the sum
__device__ __forceinline__ float tree_sum(float* red, float* out, int e, int P) {
    for (int st = P >> 1; st >= 32; st >>= 1) {
        __syncthreads();
        if (e < st) red[e] = red[e] + red[e + st];
    }
    __syncthreads();
    if (e < 32) {
        float v = red[e];
#pragma unroll
        for (int st = 16; st > 0; st >>= 1) {
            const float o = __shfl_down_sync(0xffffffffu, v, st);
            if (e < st) v = v + o;
        }
        if (e == 0) *out = v;
    }
    __syncthreads();
    return *out;
}

__global__ void route_softmax_kernel(const float* __restrict__ logits, int32_t* __restrict__ ids, float* __restrict__ wts, int E, int K) {
    extern __shared__ float sm[];
    float* red = sm;               // [P]
    float* s_w = sm + blockDim.x;  // [K]
    __shared__ float bmax[32];
    __shared__ int bmin[32];
    __shared__ float s_den;
    const int P = blockDim.x, e = threadIdx.x, t = blockIdx.x;
    const bool in = e < E;
    const float l = in ? logits[(size_t)t * E + e] : -INFINITY;
    // missing leaves of a non-power-of-two E are absent from the trees: -inf for max, 0 for sum
    const float mx = block_max(l, bmax, e, P);
    const float ex = in ? exp_rn(l - mx) : 0.0f;
    red[e] = ex;
    const float den = tree_sum(red, &s_den, e, P);
    float p = in ? ex / den : -1.0f;
    bool alive = in;
    for (int j = 0; j < K; j++) {
        int pick = pick_best(bmax, bmin, p, alive, e, P, E);
        if (pick >= E) pick = 0;  // a row of NaN: keep indices valid
        if (e == pick) {
            s_w[j] = p;
            alive = false;
            ids[(size_t)t * K + j] = pick;
        }
    }
    __syncthreads();
    if (e == 0) {
        float sum = 0.0f;  // in pick order
        for (int j = 0; j < K; j++) sum += s_w[j];
        for (int j = 0; j < K; j++) wts[(size_t)t * K + j] = s_w[j] / sum;
    }
}

__global__ void route_sigmoid_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int32_t* __restrict__ ids,
                                     float* __restrict__ wts, int E, int K, float scale) {
    extern __shared__ float sm[];
    float* s_w = sm + blockDim.x;
    __shared__ float bmax[32];
    __shared__ int bmin[32];
    const int P = blockDim.x, e = threadIdx.x, t = blockIdx.x;
    const bool in = e < E;
    float s = 0.0f, c = -INFINITY;
    if (in) {
        s = 1.0f / (1.0f + exp_rn(-logits[(size_t)t * E + e]));
        const float v = s + (bias ? bias[e] : 0.0f);
        c = (v != v) ? -INFINITY : v;  // NaN never wins
    }
    bool alive = in;
    for (int j = 0; j < K; j++) {
        int pick = pick_best(bmax, bmin, c, alive, e, P, E);
        if (pick >= E) pick = 0;
        if (e == pick) {
            s_w[j] = s;
            alive = false;
            ids[(size_t)t * K + j] = pick;
        }
    }
    __syncthreads();
    if (e == 0) {
        float sum = 0.0f;
        for (int j = 0; j < K; j++) sum += s_w[j];
        const float den = sum + 1e-20f;
        for (int j = 0; j < K; j++) wts[(size_t)t * K + j] = (s_w[j] / den) * scale;
    }
}

int pow2_at_least(int n) {
    int p = 32;
    while (p < n) p <<= 1;
    return p;
}

int check(int tokens, int experts, int k, const char* who) {
    if (tokens < 1 || experts < 1 || experts > 1024 || k < 1 || k > experts || k > 64)
        CN_FAIL(CN_ERR_SHAPE, "%s: %d experts top-%d: the router takes 1 <= K <= 64, K <= E <= 1024", who, experts, k);
    return CN_OK;
}

}  // namespace

extern "C" int cn_route_softmax_topk(const float* logits, int32_t* ids, float* wts, int tokens, int experts, int k, cn_stream_t stream) {
    if (int rc = check(tokens, experts, k, "cn_route_softmax_topk")) return rc;
    const int P = pow2_at_least(experts);
    route_softmax_kernel<<<tokens, P, (P + k) * sizeof(float), (cudaStream_t)stream>>>(logits, ids, wts, experts, k);
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}

extern "C" int cn_route_sigmoid_topk(const float* logits, const float* bias, int32_t* ids, float* wts, int tokens, int experts, int k,
                                     float scale, cn_stream_t stream) {
    if (int rc = check(tokens, experts, k, "cn_route_sigmoid_topk")) return rc;
    const int P = pow2_at_least(experts);
    route_sigmoid_kernel<<<tokens, P, (P + k) * sizeof(float), (cudaStream_t)stream>>>(logits, bias, ids, wts, experts, k, scale);
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}
