// FP8 (E4M3FN) GEMV for 1..8 activation rows on the tensor cores: persistent CTAs, a bulk-copy ring for the weight
// bytes, mma.sync.m16n8k16 (f16 x f16 -> f32) fed by cvt.rn.f16x2.e4m3x2. The reference has the FP8 codec only
// (engine/src/cnq.rs:1312-1376, converter/src/fp8.rs:19-82: E4M3FN bytes, one f32 scale per 128 x 128 tile); this GEMV is
// defined on that codec (see cn_fp8_gemv). Taken for cols % 128 == 0; other shapes stay on the warp-per-row kernel.
//
// A tile is 16 weight rows; a stage holds up to 1024 bytes of each of them (eight 128-column blocks), brought in by the
// producer warp as 16 bulk copies; consumer warp w takes block w of the stage. Inside a block the order of k is free as
// long as weights and activations agree, so it is chosen to make the loads wide: lane (g, t) reads 16 bytes of rows g and
// g + 8 at byte 16 t of a 64-byte piece (one LDS.128 each) and 16 activations at the same place, and MMA j of the piece
// multiplies bytes 4j .. 4j+3 of every lane: 4 loads, 16 cvt and 4 MMAs per 1024 weights. The eight columns of the MMA
// are the activation rows, so up to eight rows cost what one costs, and every row's sum is the same whatever the other
// columns hold (a row of an m-row call is bit-identical to a one-row call). A 128-column block shares one weight scale:
// its eight MMAs accumulate in the tensor core's f32 registers and are scaled once (weight scale x inverse activation
// scale) into the running sums; the eight warps' sums of a tile meet in shared memory and are added in warp order.
// Activations are staged once per CTA as f16 with a power-of-two scale per 128-column block (exact for bf16 input; f32 input
// is rounded to 11 bits there).
#include "common.cuh"

namespace {

constexpr int NW = 8;
constexpr int NTHREADS = (NW + 1) * 32;
constexpr int MAX_STAGES = 8;
constexpr int RED_DEPTH = 4;
constexpr int CB = 1024;           // bytes of a row per stage
constexpr int PS = CB + 64;        // padded row pitch: the two rows (g, g + 1) a quarter warp reads with 16-byte loads fall into different bank halves
constexpr int STAGE_BYTES = 16 * PS;
constexpr int TBAR_OFF = 128;
constexpr int RED_OFF = 256;       // [RED_DEPTH][NW][16 rows][8 tokens] f32
constexpr int XS_OFF = RED_OFF + RED_DEPTH * NW * 512;

struct Fp8Params {
    const uint8_t* w;
    const float* scale;
    const void* x;
    void* y;
    int rows, cols, m, ldy, x_bf16, stages;
    uint32_t xrow, stage_off;  // bytes of one staged activation row (padded); where the ring starts
};

// four E4M3 bytes -> two f16x2 (bytes 0,1 and bytes 2,3); every E4M3 value is exact in f16
__device__ __forceinline__ void e4m3x4_to_f16x2(uint32_t word, uint32_t& lo, uint32_t& hi) {
    asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}" : "=r"(lo), "=r"(hi) : "r"(word));
}

template <int CPS>
__global__ void __launch_bounds__(NTHREADS, CPS) fp8_gemv_tc_kernel(const Fp8Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = (uint64_t*)smem;
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* tbar = (uint64_t*)(smem + TBAR_OFF);
    float* red = (float*)(smem + RED_OFF);
    const int S = p.stages;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nkb = p.cols >> 7;                 // 128-column blocks per row
    const int nch = (p.cols + CB - 1) / CB;      // stages per tile
    const int ntiles = (p.rows + 15) >> 4;

    if (warp == NW) {
        if (lane == 0) {
            for (int s = 0; s < S; s++) {
                mbar_init(&full[s], 1);
                mbar_init(&empty[s], NW);
            }
            for (int i = 0; i < RED_DEPTH; i++) mbar_init(&tbar[i], NW);
            mbar_fence_init();
        }
        __syncwarp();
        asm volatile("bar.arrive 2, %0;" ::"n"(NTHREADS) : "memory");
        pdl_launch_dependents();
        // ------------------------------------------------------------ weight producer (the weights do not depend on the previous kernel)
        const uint64_t pol = l2_policy_evict_first();
        int s = 0;
        uint32_t par = 0;
        bool first_round = true;
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
            const int row = tile * 16 + lane;
            const uint8_t* src = (lane < 16 && row < p.rows) ? p.w + (size_t)row * p.cols : nullptr;
            const uint32_t nvalid = (uint32_t)__popc(__ballot_sync(0xffffffffu, src != nullptr));
            for (int c = 0; c < nch; c++) {
                const uint32_t piece = (uint32_t)min(CB, p.cols - c * CB);
                if (!first_round && !mbar_wait(&empty[s], par ^ 1u)) {
                    cn_dev_fail(CN_DEV_WAIT_EMPTY);
                    return;
                }
                uint8_t* dst = smem + p.stage_off + (size_t)s * STAGE_BYTES;
                if (lane == 0) {
                    mbar_expect_tx(&full[s], nvalid * piece);
                    mbar_arrive(&full[s]);
                }
                __syncwarp();
                if (src) bulk_g2s_stream(dst + (size_t)lane * PS, src + (size_t)c * CB, piece, &full[s], pol);
                if (++s == S) {
                    s = 0;
                    par ^= 1u;
                    first_round = false;
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumer warps: stage the activation rows
    pdl_launch_dependents();
    pdl_wait();
    uint8_t* xs0 = smem + XS_OFF;                                   // [m][xrow] f16
    float* xinv0 = (float*)(xs0 + (size_t)p.m * p.xrow);            // [8][nkb]; 1 for the rows beyond m (their sums are zero)
    for (int i = tid; i < (8 - p.m) * nkb; i += NW * 32) xinv0[p.m * nkb + i] = 1.0f;
    // a task = 8 consecutive values of one row (16 lanes per 128-column block); eight tasks of a thread have their loads in flight
    // together, so the staging costs a few trips to L2 whatever the row count
    {
        const int ntask = p.m * nkb * 16;
        constexpr int PF = 8;
        for (int t0 = tid; t0 < ntask; t0 += PF * NW * 32) {
            uint4 ra[PF], rb2[PF];
#pragma unroll
            for (int u = 0; u < PF; u++) {
                const int task = t0 + u * NW * 32;
                ra[u] = rb2[u] = make_uint4(0u, 0u, 0u, 0u);
                if (task >= ntask) continue;
                const int mrow = task / (nkb * 16), rem = task - mrow * nkb * 16;  // rem * 8 = first column of the task
                if (p.x_bf16) {
                    ra[u] = __ldcg((const uint4*)((const char*)p.x + ((size_t)mrow * p.cols + (size_t)rem * 8) * 2));
                } else {
                    const uint4* src = (const uint4*)((const char*)p.x + ((size_t)mrow * p.cols + (size_t)rem * 8) * 4);
                    ra[u] = __ldcg(src), rb2[u] = __ldcg(src + 1);
                }
            }
#pragma unroll
            for (int u = 0; u < PF; u++) {
                const int task = t0 + u * NW * 32;
                if (task >= ntask) break;  // uniform over every 16-lane group: ntask is a multiple of 16
                const int mrow = task / (nkb * 16), rem = task - mrow * nkb * 16;
                float v[8];
                if (p.x_bf16) {
                    const uint32_t w4[4] = {ra[u].x, ra[u].y, ra[u].z, ra[u].w};
#pragma unroll
                    for (int q = 0; q < 4; q++) v[2 * q] = __uint_as_float(w4[q] << 16), v[2 * q + 1] = __uint_as_float(w4[q] & 0xffff0000u);
                } else {
                    v[0] = __uint_as_float(ra[u].x), v[1] = __uint_as_float(ra[u].y), v[2] = __uint_as_float(ra[u].z), v[3] = __uint_as_float(ra[u].w);
                    v[4] = __uint_as_float(rb2[u].x), v[5] = __uint_as_float(rb2[u].y), v[6] = __uint_as_float(rb2[u].z), v[7] = __uint_as_float(rb2[u].w);
                }
                float amax = 0.0f;
#pragma unroll
                for (int q = 0; q < 8; q++) amax = fmaxf(amax, fabsf(v[q]));
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                uint32_t e = (__float_as_uint(amax) >> 23) & 0xFF;
                float mul = 1.0f, inv = 1.0f;
                if (amax > 0.0f && e < 255) {
                    e = e < 15 ? 15 : e;
                    mul = __uint_as_float((268u - e) << 23);
                    inv = __uint_as_float((e - 14u) << 23);
                }
                uint32_t h[4];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const __half2 hh = __floats2half2_rn(v[2 * q] * mul, v[2 * q + 1] * mul);
                    h[q] = *(const uint32_t*)&hh;
                }
                *(uint4*)(xs0 + (size_t)mrow * p.xrow + (size_t)rem * 16) = make_uint4(h[0], h[1], h[2], h[3]);
                if ((rem & 15) == 0) xinv0[mrow * nkb + (rem >> 4)] = inv;
            }
        }
    }
    asm volatile("bar.sync 2, %0;" ::"n"(NTHREADS) : "memory");  // staging done, and the ring's barriers exist

    const int g = lane >> 2, t = lane & 3;
    const uint8_t* xg = xs0 + (size_t)g * p.xrow;  // this lane's activation row (MMA column g)
    const bool xlive = g < p.m;
    int s = 0, rslot = 0;
    uint32_t par = 0, rpar = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};  // rows g, g + 8 of the tile x activation rows 2t, 2t + 1
        const float* srow = p.scale + (size_t)((tile * 16) >> 7) * nkb;
        for (int c = 0; c < nch; c++) {
            const int nb = min(CB, p.cols - c * CB) >> 7;  // 128-column blocks in this stage
            if (!mbar_wait(&full[s], par)) {
                cn_dev_fail(CN_DEV_WAIT_FULL);
                ok = false;
                break;
            }
            if (warp < nb) {
                const int kb = c * 8 + warp;
                const uint8_t* pa = smem + p.stage_off + (size_t)s * STAGE_BYTES + (size_t)g * PS + warp * 128 + 16 * t;
                const uint8_t* px = xg + (size_t)kb * 256 + 32 * t;
                const float ws = __ldg(srow + kb);  // asked for first, used after the MMAs
                float cc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int h = 0; h < 2; h++) {  // two 64-byte pieces of the block
                    const uint4 a = *(const uint4*)(pa + 64 * h), b = *(const uint4*)(pa + 8 * PS + 64 * h);
                    uint4 x0 = make_uint4(0u, 0u, 0u, 0u), x1 = x0;
                    if (xlive) x0 = *(const uint4*)(px + 128 * h), x1 = *(const uint4*)(px + 128 * h + 16);
                    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
                    const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        uint32_t a0, a2, a1, a3;
                        e4m3x4_to_f16x2(aw[j], a0, a2);
                        e4m3x4_to_f16x2(bw[j], a1, a3);
                        mma16816(cc, a0, a1, a2, a3, xw[2 * j], xw[2 * j + 1]);
                    }
                }
                const float s0 = ws * xinv0[(2 * t) * nkb + kb], s1 = ws * xinv0[(2 * t + 1) * nkb + kb];
                acc[0] = fmaf(cc[0], s0, acc[0]);
                acc[1] = fmaf(cc[1], s1, acc[1]);
                acc[2] = fmaf(cc[2], s0, acc[2]);
                acc[3] = fmaf(cc[3], s1, acc[3]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            if (++s == S) {
                s = 0;
                par ^= 1u;
            }
        }
        if (!ok) break;
        // the eight warps' blocks of K meet in shared memory; warp 0 adds them in warp order and stores
        float* rb = red + rslot * (NW * 128);
        rb[warp * 128 + g * 8 + 2 * t] = acc[0];
        rb[warp * 128 + g * 8 + 2 * t + 1] = acc[1];
        rb[warp * 128 + (g + 8) * 8 + 2 * t] = acc[2];
        rb[warp * 128 + (g + 8) * 8 + 2 * t + 1] = acc[3];
        __syncwarp();
        if (lane == 0) mbar_arrive(&tbar[rslot]);
        if (warp == 0) {
            if (!mbar_wait(&tbar[rslot], rpar)) {
                cn_dev_fail(CN_DEV_WAIT_FULL);
                ok = false;
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int e = i * 32 + lane;  // element (row e / 8, activation row e % 8)... stored row-major over rows
                    const int mrow = e >> 4, r = e & 15;  // lanes walk the 16 weight rows fastest: coalesced stores
                    float v = rb[r * 8 + mrow];
                    for (int ww = 1; ww < NW; ww++) v += rb[ww * 128 + r * 8 + mrow];
                    const int row = tile * 16 + r;
                    if (mrow < p.m && row < p.rows) {
                        if (p.x_bf16)
                            ((__nv_bfloat16*)p.y)[(size_t)mrow * p.ldy + row] = __float2bfloat16_rn(v);
                        else
                            ((float*)p.y)[(size_t)mrow * p.ldy + row] = v;
                    }
                }
            }
        }
        if (++rslot == RED_DEPTH) {
            rslot = 0;
            rpar ^= 1u;
        }
    }
}

}  // namespace

// returns CN_OK after a launch, or -1 when the shape is not one this kernel takes (the caller uses the warp-per-row kernel)
int cn_fp8_gemv_tc_launch(const void* w, const float* scale, const void* x, void* y, int rows, int cols, int m, int ldy, int dtype, cudaStream_t st) {
    if (cols % 128 != 0 || cols < 1024) return -1;
    const int nkb = cols / 128;
    const uint32_t xrow = (uint32_t)(cols * 2 + 16);  // + 16: the activation rows of a quarter warp's two quads land in different banks
    const uint32_t stage_off = (uint32_t)((XS_OFF + (size_t)m * xrow + 8 * (size_t)nkb * 4 + 127) & ~(size_t)127);
    const int nch = (cols + CB - 1) / CB;
    // two CTAs per SM when each still gets a ring of three stages (more warps to hide the shared-memory and barrier latencies)
    int cps = 2;
    int stages = (int)(((227 * 1024) / cps - 1024 - (long long)stage_off) / STAGE_BYTES);
    if (stages < 3) {
        cps = 1;
        stages = (int)((226 * 1024 - (long long)stage_off) / STAGE_BYTES);
    }
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages > (RED_DEPTH - 1) * nch) stages = (RED_DEPTH - 1) * nch;  // a warp runs at most `stages` stages ahead of warp 0: that many tile sums at most
    if (stages < 3) {
        // the staged activation rows leave no room for the ring: two calls over half the rows each (a row's sum does not
        // depend on its neighbours)
        if (m == 1) return -1;
        const int m0 = m / 2;
        const size_t es = dtype == CN_BF16 ? 2 : 4;
        const int rc = cn_fp8_gemv_tc_launch(w, scale, x, y, rows, cols, m0, ldy, dtype, st);
        if (rc != CN_OK) return rc;
        return cn_fp8_gemv_tc_launch(w, scale, (const char*)x + (size_t)m0 * cols * es, (char*)y + (size_t)m0 * ldy * es, rows, cols, m - m0, ldy, dtype, st);
    }
    int dev = 0, sms = 148;
    CN_CUDA(cudaGetDevice(&dev));
    CN_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int ntiles = (rows + 15) / 16;
    Fp8Params p;
    p.w = (const uint8_t*)w, p.scale = scale, p.x = x, p.y = y, p.rows = rows, p.cols = cols, p.m = m, p.ldy = ldy, p.x_bf16 = dtype == CN_BF16;
    p.stages = stages, p.xrow = xrow, p.stage_off = stage_off;
    const size_t smem = stage_off + (size_t)stages * STAGE_BYTES;
    const int grid = ntiles < sms * cps ? ntiles : sms * cps;
    if (cps == 2) {
        CN_ALLOW_SMEM(fp8_gemv_tc_kernel<2>, 113 * 1024);
        CN_CUDA(cn_launch_pdl(fp8_gemv_tc_kernel<2>, dim3(grid), dim3(NTHREADS), smem, st, p));
    } else {
        CN_ALLOW_SMEM(fp8_gemv_tc_kernel<1>, 226 * 1024);
        CN_CUDA(cn_launch_pdl(fp8_gemv_tc_kernel<1>, dim3(grid), dim3(NTHREADS), smem, st, p));
    }
    return CN_OK;
}
