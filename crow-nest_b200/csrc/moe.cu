// The routed-expert decode step over NVFP4 experts: grouped expert GEMVs after top-k routing, the
// shared expert, and the weighted combine.
//
// Supersedes the routed half of Engine::moe_run (engine/src/gen.rs:4168-4532): gemv_fp4_ptrb over
// the gate|up and down pointer tables (engine/src/kernels.rs:195-233), silu_mul_combo (:1562),
// acc_combo (:1583) and gate_shared (:1593); the operator shape follows GpuMoePlan
// (engine/src/glm5_moe.rs:518-793): a plan owns its scratch, run() only enqueues.
//
// B200 shape of the step: combos (token, rank) are sorted by expert on the device, so the CTAs
// that read one expert's matrices run back to back and every expert's bytes cross HBM once per
// step (repeats are L2 hits); gate, up and the activation are one launch; a null table entry
// skips the combo (the expert lives on another rank).
#include "common.cuh"
#include "nvfp4_gemv.cuh"

namespace {

// order[] = combos sorted by expert id (negative ids last); one CTA of 1024 threads, counting sort in shared memory
__global__ void moe_sort_kernel(const int32_t* __restrict__ ids, int32_t* __restrict__ order, int n, int E) {
    extern __shared__ int cnt[];  // [E + 2] counts, then start offsets; [n] the combos' bins
    int* bin = cnt + E + 2;
    __shared__ int wsum[32];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    for (int i = tid; i <= E + 1; i += blockDim.x) cnt[i] = 0;
    __syncthreads();
    for (int c = tid; c < n; c += blockDim.x) {
        const int e = ids[c];
        const int b = (e < 0 || e >= E) ? E : e;
        bin[c] = b;
        atomicAdd(&cnt[b], 1);
    }
    __syncthreads();
    // exclusive prefix sum over the E + 1 bins: every thread takes a contiguous run, the runs' totals are scanned
    // with warp shuffles
    const int per = (E + 1 + (int)blockDim.x - 1) / (int)blockDim.x;
    const int i0 = tid * per, i1 = min(i0 + per, E + 1);
    int mine = 0;
    for (int i = i0; i < i1; i++) mine += cnt[i];
    int inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
    }
    if (lane == 31) wsum[wid] = inc;
    __syncthreads();
    if (wid == 0) {
        int w = wsum[lane], winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += v;
        }
        wsum[lane] = winc - w;  // exclusive
    }
    __syncthreads();
    int run = wsum[wid] + inc - mine;
    for (int i = i0; i < i1; i++) {
        const int c = cnt[i];
        cnt[i] = run;
        run += c;
    }
    __syncthreads();
    // stable within an expert: each combo counts the earlier combos of its expert (n is small)
    for (int c = tid; c < n; c += blockDim.x) {
        const int b = bin[c];
        int before = 0;
        for (int d = 0; d < c; d++) before += bin[d] == b;
        order[cnt[b] + before] = c;
    }
}

// Sort the combos by expert and cut every expert's run into groups of up to gmax rows, gmax 4 or 8 (one CTA of 1024 threads):
//   order[]           the combos sorted by expert, stable; combos without a resident expert (id outside 0..E-1, or a
//                     null entry of `tab`) last and in no group
//   ga[] / counts[0]  positions (in order[]) of the one-row groups: an expert's single row, or the one left over after
//                     its groups of gmax
//   gb[], gbrows[] / counts[1]  first positions and row counts (2..gmax) of the other groups
//   gd[], gdrows[] / counts[2]  the same runs cut into groups of one or two rows (for f32 activations, which take two
//                     of the kernel's four row slots each: a high and a low f16 plane)
// Placement is done by one warp walking the combos in order (match.any finds the lanes of a step that share an expert),
// so the sort stays stable without ranking every combo against all others.
__global__ void __launch_bounds__(1024) moe_group_kernel(const int32_t* __restrict__ ids, const unsigned long long* __restrict__ tab, int n, int E,
                                                         int32_t* __restrict__ order, int* __restrict__ ga, int* __restrict__ gb,
                                                         int* __restrict__ gbrows, int* __restrict__ gd, int* __restrict__ gdrows,
                                                         int* __restrict__ counts, int gmax) {
    extern __shared__ int sm[];  // [E + 1] counts, [E + 1] starts, [E + 1] running, [n] bins
    int* cnt = sm;
    int* start = sm + (E + 1);
    int* run = sm + 2 * (E + 1);
    int* bin = sm + 3 * (E + 1);
    __shared__ int wsa[32], wsb[32], wsd[32];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int i = tid; i <= E; i += blockDim.x) cnt[i] = 0;
    __syncthreads();
    for (int c = tid; c < n; c += blockDim.x) {
        const int e = ids[c];
        const int b = (e < 0 || e >= E || (tab && tab[e] == 0ull)) ? E : e;
        bin[c] = b;
        atomicAdd(&cnt[b], 1);
    }
    __syncthreads();
    // per expert: one-row groups and larger groups, then three exclusive prefix sums over the experts (rows, a, b)
    const int per = (E + 1 + (int)blockDim.x - 1) / (int)blockDim.x;
    const int i0 = min(tid * per, E + 1), i1 = min(i0 + per, E + 1);
    int rows = 0, na = 0, nb = 0, nd = 0;
    for (int i = i0; i < i1; i++) {
        const int k = cnt[i];
        rows += k;
        if (i < E) na += (k % gmax) == 1, nb += k / gmax + ((k % gmax) >= 2), nd += (k + 1) >> 1;
    }
    int ir = rows, ia = na, ib = nb, id = nd;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int vr = __shfl_up_sync(0xffffffffu, ir, o), va = __shfl_up_sync(0xffffffffu, ia, o), vb = __shfl_up_sync(0xffffffffu, ib, o);
        const int vd = __shfl_up_sync(0xffffffffu, id, o);
        if (lane >= o) ir += vr, ia += va, ib += vb, id += vd;
    }
    __shared__ int wsr[32];
    if (lane == 31) wsr[wid] = ir, wsa[wid] = ia, wsb[wid] = ib, wsd[wid] = id;
    __syncthreads();
    if (wid == 0) {
        int r = wsr[lane], a = wsa[lane], b = wsb[lane], d = wsd[lane];
        const int r0 = r, a0 = a, b0 = b, d0 = d;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int vr = __shfl_up_sync(0xffffffffu, r, o), va = __shfl_up_sync(0xffffffffu, a, o), vb = __shfl_up_sync(0xffffffffu, b, o);
            const int vd = __shfl_up_sync(0xffffffffu, d, o);
            if (lane >= o) r += vr, a += va, b += vb, d += vd;
        }
        wsr[lane] = r - r0, wsa[lane] = a - a0, wsb[lane] = b - b0, wsd[lane] = d - d0;
        if (lane == 31) counts[0] = a, counts[1] = b, counts[2] = d;
    }
    __syncthreads();
    int pr = wsr[wid] + ir - rows, pa = wsa[wid] + ia - na, pb = wsb[wid] + ib - nb, pd = wsd[wid] + id - nd;
    for (int i = i0; i < i1; i++) {
        const int k = cnt[i];
        start[i] = pr;
        run[i] = pr;
        if (i < E) {
            for (int q = 0; q < k / gmax; q++) gb[pb] = pr + gmax * q, gbrows[pb] = gmax, pb++;
            const int rem = k % gmax, at = pr + k - rem;
            if (rem == 1) ga[pa++] = at;
            if (rem >= 2) gb[pb] = at, gbrows[pb] = rem, pb++;
            for (int q = 0; q < k; q += 2) gd[pd] = pr + q, gdrows[pd] = k - q >= 2 ? 2 : 1, pd++;
        }
        pr += k;
    }
    __syncthreads();
    if (wid == 0) {
        for (int c0 = 0; c0 < n; c0 += 32) {
            const int c = c0 + lane;
            const int b = c < n ? bin[c] : -1 - lane;  // lanes beyond the end match nobody
            const unsigned same = __match_any_sync(0xffffffffu, b);
            if (c < n) {
                const int base = run[b];
                order[base + __popc(same & ((1u << lane) - 1u))] = c;
            }
            __syncwarp();
            if (c < n && lane == __ffs(same) - 1) run[b] += __popc(same);
            __syncwarp();
        }
    }
}

// y[t][c] = base + sum_j w[t][j] * eo[t*K + j][c], j in pick order; base = shared[t][c]
// (times sigmoid(sgate[t]) when gated), 0 without a shared expert. A combo whose expert has no
// local matrix contributes nothing.
template <int YT>
__global__ void moe_combine_kernel(const float* __restrict__ eo, const float* __restrict__ wts, const int32_t* __restrict__ ids,
                                   const unsigned long long* __restrict__ tab, const float* __restrict__ shared,
                                   const float* __restrict__ sgate, void* __restrict__ y, int H, int K, int E) {
    // the token's K weights and "has a local matrix" flags once per CTA, so that the K loads of a column do not
    // wait on an id -> table -> value chain each
    constexpr int KC = 16;
    __shared__ float s_w[KC];
    __shared__ int s_ok[KC];
    const int c = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    float acc = 0.0f;
    for (int j0 = 0; j0 < K; j0 += KC) {
        const int kc = min(KC, K - j0);
        if (j0 > 0) __syncthreads();
        if ((int)threadIdx.x < kc) {
            const int e = ids[t * K + j0 + threadIdx.x];
            s_ok[threadIdx.x] = !(e < 0 || (E > 0 && e >= E) || (tab && tab[e] == 0ull));
            s_w[threadIdx.x] = wts[t * K + j0 + threadIdx.x];
        }
        __syncthreads();
        if (c < H) {
            float v[KC];
#pragma unroll
            for (int j = 0; j < KC; j++) v[j] = (j < kc && s_ok[j]) ? eo[((size_t)t * K + j0 + j) * H + c] : 0.0f;
#pragma unroll
            for (int j = 0; j < KC; j++)
                if (j < kc && s_ok[j]) acc = __fadd_rn(acc, __fmul_rn(s_w[j], v[j]));
        }
    }
    if (c >= H) return;
    float base = shared ? shared[(size_t)t * H + c] : 0.0f;
    if (shared && sgate) base = __fmul_rn(1.0f / (1.0f + expf(-sgate[t])), base);
    const float v = __fadd_rn(base, acc);
    if (YT == 1)
        ((__nv_bfloat16*)y)[(size_t)t * H + c] = __float2bfloat16_rn(v);
    else
        ((float*)y)[(size_t)t * H + c] = v;
}

struct MoePlan {
    int hidden, inter, experts, topk, max_tokens, device;
    float* h;        // [max_tokens * topk][inter]
    float* eo;       // [max_tokens * topk][hidden]
    float* hs;       // [max_tokens][shared inter <= inter_s]
    float* ys;       // [max_tokens][hidden]
    int32_t* order;  // [max_tokens * topk]
    int* groups;     // [5 * max_tokens * topk + 8]: the group lists of moe_group_kernel and their three counts
    int shared_inter;
    // the shared expert does not depend on the routed experts until the combine: it is enqueued on a side stream
    // between two events (fork after the caller's earlier work, join before the combine), also under stream capture
    cudaStream_t side;
    cudaEvent_t fork, join;
    bool shared_pending;  // cn_moe_nvfp4_shared_begin has enqueued the shared expert; the next finish joins it
};

}  // namespace

// the grouping step for other operators of the library (declared in nvfp4_gemv.cuh): lists of `combos` ints each, counts of 3
int cn_moe_group_launch(const int32_t* ids, const unsigned long long* tab, int combos, int experts, int32_t* order, int* ga, int* gb, int* gbrows,
                        int* gd, int* gdrows, int* counts, int gmax, cudaStream_t stream) {
    if (gmax != 4 && gmax != 8) CN_FAIL(CN_ERR_SHAPE, "grouping: groups of %d rows (4 or 8)", gmax);
    const size_t smem = (size_t)(3 * (experts + 1) + combos) * sizeof(int);
    if (smem > 160 * 1024) CN_FAIL(CN_ERR_LIMIT, "grouping %d combos over %d experts needs %zu B of shared memory", combos, experts, smem);
    CN_ALLOW_SMEM(moe_group_kernel, 160 * 1024);
    CN_CUDA(cn_launch_pdl(moe_group_kernel, dim3(1), dim3(1024), smem, stream, ids, tab, combos, experts, order, ga, gb, gbrows, gd, gdrows, counts, gmax));
    return CN_OK;
}

extern "C" int cn_moe_sort(const int32_t* ids, int32_t* order, int combos, int experts, cn_stream_t stream) {
    if (combos < 1 || experts < 1 || experts > 8192) CN_FAIL(CN_ERR_SHAPE, "cn_moe_sort: %d combos over %d experts", combos, experts);
    const size_t smem = (size_t)(experts + 2 + combos) * sizeof(int);
    if (smem > 48 * 1024) CN_FAIL(CN_ERR_LIMIT, "cn_moe_sort: %d combos over %d experts need %zu B of shared memory", combos, experts, smem);
    moe_sort_kernel<<<1, 1024, smem, (cudaStream_t)stream>>>(ids, order, combos, experts);
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}

extern "C" int cn_moe_combine(const float* eo, const float* wts, const int32_t* ids, const unsigned long long* table, const float* shared,
                              const float* sgate, void* y, int tokens, int hidden, int topk, int experts, int dtype, cn_stream_t stream) {
    if (tokens < 1 || hidden < 1 || topk < 1) CN_FAIL(CN_ERR_SHAPE, "cn_moe_combine: tokens %d hidden %d topk %d", tokens, hidden, topk);
    if (dtype != CN_F32 && dtype != CN_BF16) CN_FAIL(CN_ERR_SHAPE, "cn_moe_combine: dtype %d is neither CN_F32 nor CN_BF16", dtype);
    dim3 grid((hidden + 255) / 256, tokens);
    if (dtype == CN_BF16)
        moe_combine_kernel<1><<<grid, 256, 0, (cudaStream_t)stream>>>(eo, wts, ids, table, shared, sgate, y, hidden, topk, experts);
    else
        moe_combine_kernel<0><<<grid, 256, 0, (cudaStream_t)stream>>>(eo, wts, ids, table, shared, sgate, y, hidden, topk, experts);
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}

extern "C" int cn_moe_nvfp4_plan_destroy(void* plan);

extern "C" int cn_moe_nvfp4_plan_create(void** plan_out, int hidden, int inter, int shared_inter, int experts, int topk, int max_tokens) {
    if (!plan_out || hidden % 256 || inter % 256 || shared_inter % 256 || experts < 1 || topk < 1 || max_tokens < 1)
        CN_FAIL(CN_ERR_SHAPE, "cn_moe_nvfp4_plan_create: hidden %d, inter %d, shared inter %d must be multiples of 256", hidden, inter, shared_inter);
    MoePlan* p = new MoePlan();
    p->hidden = hidden, p->inter = inter, p->experts = experts, p->topk = topk, p->max_tokens = max_tokens, p->shared_inter = shared_inter;
    CN_CUDA(cudaGetDevice(&p->device));
    const size_t combos = (size_t)max_tokens * topk;
    // a failure part-way frees what the earlier steps got (the destroy call takes a half-built plan)
    cudaError_t e = cudaSuccess;
    auto step = [&](cudaError_t r) { if (e == cudaSuccess) e = r; };
    step(cudaMalloc(&p->h, combos * inter * sizeof(float)));
    step(cudaMalloc(&p->eo, combos * hidden * sizeof(float)));
    step(cudaMalloc(&p->hs, (size_t)max_tokens * (shared_inter > 0 ? shared_inter : 1) * sizeof(float)));
    step(cudaMalloc(&p->ys, (size_t)max_tokens * hidden * sizeof(float)));
    step(cudaMalloc(&p->order, combos * sizeof(int32_t)));
    step(cudaMalloc(&p->groups, (5 * combos + 8) * sizeof(int)));
    step(cudaStreamCreateWithFlags(&p->side, cudaStreamNonBlocking));
    step(cudaEventCreateWithFlags(&p->fork, cudaEventDisableTiming));
    step(cudaEventCreateWithFlags(&p->join, cudaEventDisableTiming));
    if (e != cudaSuccess) {
        cn_moe_nvfp4_plan_destroy(p);
        CN_FAIL(CN_ERR_CUDA, "cn_moe_nvfp4_plan_create: %s", cudaGetErrorString(e));
    }
    *plan_out = p;
    return CN_OK;
}

extern "C" int cn_moe_nvfp4_plan_destroy(void* plan) {
    MoePlan* p = (MoePlan*)plan;
    if (!p) return CN_OK;
    cudaFree(p->h), cudaFree(p->eo), cudaFree(p->hs), cudaFree(p->ys), cudaFree(p->order), cudaFree(p->groups);
    if (p->side) cudaStreamDestroy(p->side);
    if (p->fork) cudaEventDestroy(p->fork);
    if (p->join) cudaEventDestroy(p->join);
    delete p;
    return CN_OK;
}

namespace {

// the shared expert on every token, up to 8 rows per pass, on the plan's side stream between the fork and join events:
// whatever happens after the fork, the side stream is joined again (a capture of the caller's stream stays valid)
int shared_branch(MoePlan* p, const void* shared_gate, const void* shared_up, const void* shared_down, const float* shared_gs, const void* x,
                  int tokens, float limit, int dtype, cudaStream_t stream) {
    CN_CUDA(cudaEventRecord(p->fork, stream));
    CN_CUDA(cudaStreamWaitEvent(p->side, p->fork, 0));
    const size_t es = dtype == CN_BF16 ? 2 : 4;
    int rc = CN_OK;
    for (int t0 = 0; t0 < tokens && rc == CN_OK; t0 += CN_MAX_M) {
        const int m = tokens - t0 < CN_MAX_M ? tokens - t0 : CN_MAX_M;
        GemvCall g = {};
        g.w0 = shared_gate, g.w1 = shared_up, g.gs0 = shared_gs, g.gs1 = shared_gs + 1, g.x = (const char*)x + (size_t)t0 * p->hidden * es;
        g.y = p->hs + (size_t)t0 * p->shared_inter, g.rows = p->shared_inter, g.k = p->hidden, g.m = m, g.ldy = p->shared_inter;
        g.limit = limit, g.dtype = dtype, g.out_f32 = 1;
        rc = cn_gemv_launch(g, p->side, "cn_moe_nvfp4_run (shared gate/up)");
        if (rc != CN_OK) break;
        GemvCall s = {};
        s.w0 = shared_down, s.gs0 = shared_gs + 2, s.x = p->hs + (size_t)t0 * p->shared_inter, s.y = p->ys + (size_t)t0 * p->hidden;
        s.rows = p->hidden, s.k = p->shared_inter, s.m = m, s.ldy = p->hidden, s.dtype = CN_F32, s.out_f32 = 1, s.x_f16_ok = 0;
        rc = cn_gemv_launch(s, p->side, "cn_moe_nvfp4_run (shared down)");
    }
    CN_CUDA(cudaEventRecord(p->join, p->side));
    return rc;
}

// routed gate|up + activation, then routed down, one launch each over `combos` (token, pick) pairs: combo c reads
// activation row c / x_div and writes eo row c (or to eo_ptrs[c] when given: a row of another buffer, e.g. in a peer's memory)
int routed_experts(MoePlan* p, const unsigned long long* table_gu, const unsigned long long* table_up, const unsigned long long* table_dn,
                   const float* gs_gu, const float* gs_up, const float* gs_dn, const int32_t* ids, const void* x, float* eo,
                   const unsigned long long* eo_ptrs, int combos, int x_div, float limit, int dtype, cudaStream_t stream) {
    if (combos > 96 && combos >= 2 * p->experts) {
        // At least two combo slots per expert (a long batch, or the inbox of an expert-parallel rank, whose few resident
        // experts take all its rows): sort by expert, cut into groups of up to four rows of one expert, and stream every
        // expert once per group (persistent CTAs over a device-side group list; empty slots cost nothing). One-row
        // groups and larger groups are separate launches.
        const size_t smem = (size_t)(3 * (p->experts + 1) + combos) * sizeof(int);
        if (smem <= 160 * 1024) {
            int* ga = p->groups;
            int* gb = ga + combos;
            int* gbrows = gb + combos;
            int* gd = gbrows + combos;
            int* gdrows = gd + combos;
            int* counts = gdrows + combos;
            if (int rc = cn_moe_group_launch(ids, table_gu, combos, p->experts, p->order, ga, gb, gbrows, gd, gdrows, counts, 4, stream)) return rc;
            RoutedCall a = {};
            a.ids = ids, a.order = p->order, a.tab0 = table_gu, a.tab1 = table_up, a.fused_up_rows = table_up ? 0 : p->inter, a.gs0 = gs_gu;
            a.gs1 = gs_up ? gs_up : gs_gu, a.x = x, a.x_div = x_div, a.x_f32 = dtype == CN_F32, a.y = p->h, a.ldy = p->inter, a.rows = p->inter, a.k = p->hidden;
            a.limit = limit;
            RoutedCall d = {};
            d.ids = ids, d.order = p->order, d.tab0 = table_dn, d.gs0 = gs_dn, d.x = p->h, d.x_div = 1, d.x_f32 = 1, d.y = eo, d.yptrs = eo_ptrs, d.ldy = p->hidden;
            d.rows = p->hidden, d.k = p->inter;
            if (a.x_f32) {
                // f32 rows take two row slots each (high and low f16 plane): groups of one or two rows, one launch
                a.mt = 4, a.gcount = counts + 2, a.gpos = gd, a.grows = gdrows, a.max_groups = combos;
                if (int rc = cn_routed_launch(a, stream, "cn_moe_nvfp4 (gate/up, grouped)")) return rc;
            } else {
                for (int cls = 0; cls < 2; cls++) {
                    a.mt = cls ? 4 : 1, a.gcount = counts + cls, a.gpos = cls ? gb : ga, a.grows = cls ? gbrows : nullptr, a.max_groups = cls ? combos / 2 : combos;
                    if (int rc = cn_routed_launch(a, stream, "cn_moe_nvfp4 (gate/up, grouped)")) return rc;
                }
            }
            // the intermediate rows are f32
            d.mt = 4, d.gcount = counts + 2, d.gpos = gd, d.grows = gdrows, d.max_groups = combos;
            if (int rc = cn_routed_launch(d, stream, "cn_moe_nvfp4 (down, grouped)")) return rc;
            return CN_OK;
        }
    }
    // Few combos: one launch each for gate|up and down over the combos as they come (nearly every CTA of the step is
    // resident at once and L2 serves an expert's second reader).
    GemvCall a = {};
    a.gs0 = gs_gu, a.gs1 = gs_up ? gs_up : gs_gu, a.x = x, a.y = p->h, a.rows = p->inter, a.k = p->hidden, a.m = 1, a.ldy = p->inter;
    a.limit = limit, a.dtype = dtype, a.out_f32 = 1, a.ids = ids, a.order = nullptr, a.tab0 = table_gu, a.tab1 = table_up;
    a.fused_up_rows = table_up ? 0 : p->inter, a.x_div = x_div, a.combos = combos, a.experts = p->experts;
    if (int rc = cn_gemv_launch(a, stream, "cn_moe_nvfp4 (gate/up)")) return rc;
    GemvCall d = {};
    d.gs0 = gs_dn, d.x = p->h, d.y = eo, d.yptrs = eo_ptrs, d.rows = p->hidden, d.k = p->inter, d.m = 1, d.ldy = p->hidden, d.dtype = CN_F32, d.out_f32 = 1;
    d.x_f16_ok = 0, d.ids = ids, d.order = nullptr, d.tab0 = table_dn, d.x_div = 1, d.combos = combos, d.experts = p->experts;
    return cn_gemv_launch(d, stream, "cn_moe_nvfp4 (down)");
}

}  // namespace

extern "C" int cn_moe_nvfp4_experts(void* plan, const unsigned long long* table_gu, const unsigned long long* table_up,
                                    const unsigned long long* table_dn, const float* gs_gu, const float* gs_up, const float* gs_dn,
                                    const int32_t* ids, const void* x, float* eo, const unsigned long long* eo_ptrs, int combos, int x_div,
                                    float limit, int dtype, cn_stream_t stream) {
    MoePlan* p = (MoePlan*)plan;
    if (!p) CN_FAIL(CN_ERR_SHAPE, "cn_moe_nvfp4_experts: null plan");
    if (combos < 1 || combos > p->max_tokens * p->topk) CN_FAIL(CN_ERR_LIMIT, "cn_moe_nvfp4_experts: %d combos, the plan holds %d", combos, p->max_tokens * p->topk);
    if (x_div < 1) CN_FAIL(CN_ERR_SHAPE, "cn_moe_nvfp4_experts: x_div %d", x_div);
    if (dtype != CN_F32 && dtype != CN_BF16) CN_FAIL(CN_ERR_SHAPE, "cn_moe_nvfp4_experts: dtype %d is neither CN_F32 nor CN_BF16", dtype);
    if (!eo && !eo_ptrs) CN_FAIL(CN_ERR_SHAPE, "cn_moe_nvfp4_experts: no output");
    return routed_experts(p, table_gu, table_up, table_dn, gs_gu, gs_up, gs_dn, ids, x, eo, eo_ptrs, combos, x_div, limit, dtype, (cudaStream_t)stream);
}

extern "C" int cn_moe_nvfp4_shared_begin(void* plan, const void* shared_gate, const void* shared_up, const void* shared_down, const float* shared_gs,
                                         const void* x, int tokens, float limit, int dtype, cn_stream_t stream) {
    MoePlan* p = (MoePlan*)plan;
    if (!p || !shared_gate || !shared_up || !shared_down || !shared_gs) CN_FAIL(CN_ERR_SHAPE, "cn_moe_nvfp4_shared_begin: null argument");
    if (tokens < 1 || tokens > p->max_tokens) CN_FAIL(CN_ERR_LIMIT, "cn_moe_nvfp4_shared_begin: %d tokens, the plan holds %d", tokens, p->max_tokens);
    if (dtype != CN_F32 && dtype != CN_BF16) CN_FAIL(CN_ERR_SHAPE, "cn_moe_nvfp4_shared_begin: dtype %d is neither CN_F32 nor CN_BF16", dtype);
    const int rc = shared_branch(p, shared_gate, shared_up, shared_down, shared_gs, x, tokens, limit, dtype, (cudaStream_t)stream);
    p->shared_pending = true;  // also after a failure: the side stream was forked and must be joined
    return rc;
}

extern "C" int cn_moe_nvfp4_finish(void* plan, const void* shared_gate, const void* shared_up, const void* shared_down, const float* shared_gs,
                                   const float* sgate, const int32_t* ids, const float* wts, const unsigned long long* table, const void* x,
                                   const float* eo, void* y, int tokens, float limit, int dtype, cn_stream_t stream_) {
    MoePlan* p = (MoePlan*)plan;
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!p) CN_FAIL(CN_ERR_SHAPE, "cn_moe_nvfp4_finish: null plan");
    if (tokens < 1 || tokens > p->max_tokens) CN_FAIL(CN_ERR_LIMIT, "cn_moe_nvfp4_finish: %d tokens, the plan holds %d", tokens, p->max_tokens);
    if (dtype != CN_F32 && dtype != CN_BF16) CN_FAIL(CN_ERR_SHAPE, "cn_moe_nvfp4_finish: dtype %d is neither CN_F32 nor CN_BF16", dtype);
    const float* shared = nullptr;
    int rc = CN_OK;
    if (p->shared_pending) {
        p->shared_pending = false;
        CN_CUDA(cudaStreamWaitEvent(stream, p->join, 0));
        shared = p->ys;
    } else if (shared_gate) {
        rc = shared_branch(p, shared_gate, shared_up, shared_down, shared_gs, x, tokens, limit, dtype, stream);
        CN_CUDA(cudaStreamWaitEvent(stream, p->join, 0));
        shared = p->ys;
    }
    if (rc != CN_OK) return rc;
    return cn_moe_combine(eo, wts, ids, table, shared, sgate, y, tokens, p->hidden, p->topk, p->experts, dtype, stream_);
}

extern "C" int cn_moe_nvfp4_run(void* plan, const unsigned long long* table_gu, const unsigned long long* table_up,
                                const unsigned long long* table_dn, const float* gs_gu, const float* gs_up, const float* gs_dn,
                                const void* shared_gate, const void* shared_up, const void* shared_down, const float* shared_gs,
                                const float* sgate, const int32_t* ids, const float* wts, const void* x, void* y, int tokens, float limit,
                                int dtype, cn_stream_t stream_) {
    MoePlan* p = (MoePlan*)plan;
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!p) CN_FAIL(CN_ERR_SHAPE, "cn_moe_nvfp4_run: null plan");
    if (tokens < 1 || tokens > p->max_tokens) CN_FAIL(CN_ERR_LIMIT, "cn_moe_nvfp4_run: %d tokens, the plan holds %d", tokens, p->max_tokens);
    if (dtype != CN_F32 && dtype != CN_BF16 && dtype != CN_BF16_IN_F32_OUT) CN_FAIL(CN_ERR_SHAPE, "cn_moe_nvfp4_run: dtype %d", dtype);
    const int ydtype = dtype == CN_BF16 ? CN_BF16 : CN_F32;  // expert-parallel partial sums leave in f32
    if (dtype == CN_BF16_IN_F32_OUT) dtype = CN_BF16;
    const float* shared = nullptr;
    int rc = CN_OK;
    if (shared_gate) {
        rc = shared_branch(p, shared_gate, shared_up, shared_down, shared_gs, x, tokens, limit, dtype, stream);
        shared = p->ys;
    }
    if (rc == CN_OK)
        rc = routed_experts(p, table_gu, table_up, table_dn, gs_gu, gs_up, gs_dn, ids, x, p->eo, nullptr, tokens * p->topk, p->topk, limit, dtype, stream);
    if (shared) CN_CUDA(cudaStreamWaitEvent(stream, p->join, 0));
    if (rc != CN_OK) return rc;
    return cn_moe_combine(p->eo, wts, ids, table_dn, shared, sgate, y, tokens, p->hidden, p->topk, p->experts, ydtype, stream_);
}
