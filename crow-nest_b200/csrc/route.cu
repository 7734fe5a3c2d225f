// MoE routing on the device: softmax top-k (Flash-Next) and sigmoid top-k (GLM), bit-exact
// indices against the host twins.
//
// Supersedes router_top10 (engine/src/kernels.rs:3109-3171; the residency bookkeeping of that
// kernel - cold mask, hit counters, pointer gather - is not part of this path: the MoE operator
// reads its pointer tables directly) and glm5_router_sig_topk (engine/src/kernels_glm5_moe.cu:44-96,
// host twin glm5_moe::route_from_logits, engine/src/glm5_moe.rs:196-236).
//
// One CTA per token row, one thread per expert slot (P = next power of two >= E, <= 1024).
// Reductions are the pairwise shared-memory trees of the reference kernel (stride P/2, P/4, ..),
// so sums round exactly as there. exp() is taken in f64 and rounded once, which gives the
// correctly rounded f32 value the host twins' libm returns; selection is K rounds of "best value,
// lowest index on ties", as in both reference routers.
#include "common.cuh"

namespace {

__device__ __forceinline__ float exp_rn(float x) { return (float)exp((double)x); }

// red[0] = max or sum over red[0..P) by the stride-halving tree; every thread calls it
template <bool MAX>
__device__ __forceinline__ float tree(float* red, int e, int P) {
    for (int st = P >> 1; st > 0; st >>= 1) {
        __syncthreads();
        if (e < st) red[e] = MAX ? fmaxf(red[e], red[e + st]) : red[e] + red[e + st];
    }
    __syncthreads();
    const float r = red[0];
    __syncthreads();
    return r;
}

// K rounds of argmax over score[] with ties to the lowest index; picks -> s_ids, returns nothing.
// `score` is private per thread (slot e), retired slots become -inf-like sentinels (`gone`).
__device__ __forceinline__ int pick_best(float* red, int* s_pick, float mine, bool alive, int e, int P, int E) {
    red[e] = alive ? mine : -INFINITY;
    const float best = tree<true>(red, e, P);
    if (e == 0) *s_pick = E;
    __syncthreads();
    if (alive && mine == best) atomicMin(s_pick, e);
    __syncthreads();
    int pick = *s_pick;
    __syncthreads();
    return pick;
}

__global__ void route_softmax_kernel(const float* __restrict__ logits, int32_t* __restrict__ ids, float* __restrict__ wts, int E, int K) {
    extern __shared__ float sm[];
    float* red = sm;           // [P]
    float* s_w = sm + blockDim.x;  // [K]
    __shared__ int s_pick;
    const int P = blockDim.x, e = threadIdx.x, t = blockIdx.x;
    const bool in = e < E;
    const float l = in ? logits[(size_t)t * E + e] : -INFINITY;
    // missing leaves of a non-power-of-two E are absent from the trees: -inf for max, 0 for sum
    red[e] = l;
    const float mx = tree<true>(red, e, P);
    const float ex = in ? exp_rn(l - mx) : 0.0f;
    red[e] = ex;
    const float den = tree<false>(red, e, P);
    float p = in ? ex / den : -1.0f;
    bool alive = in;
    float sum = 0.0f;  // kept by thread 0 in pick order
    for (int j = 0; j < K; j++) {
        int pick = pick_best(red, &s_pick, p, alive, e, P, E);
        if (pick >= E) pick = 0;  // a row of NaN: keep indices valid
        if (e == pick) {
            s_w[j] = p;
            alive = false;
        }
        __syncthreads();
        if (e == 0) {
            sum += s_w[j];
            ids[(size_t)t * K + j] = pick;
        }
    }
    __syncthreads();
    if (e == 0)
        for (int j = 0; j < K; j++) wts[(size_t)t * K + j] = s_w[j] / sum;
}

__global__ void route_sigmoid_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int32_t* __restrict__ ids,
                                     float* __restrict__ wts, int E, int K, float scale) {
    extern __shared__ float sm[];
    float* red = sm;
    float* s_w = sm + blockDim.x;
    __shared__ int s_pick;
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
        int pick = pick_best(red, &s_pick, c, alive, e, P, E);
        if (pick >= E) pick = 0;
        if (e == pick) {
            s_w[j] = s;
            alive = false;
        }
        __syncthreads();
        if (e == 0) ids[(size_t)t * K + j] = pick;
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
