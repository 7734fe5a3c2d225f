// Routed-expert NVFP4 GEMV over GROUPS of combos: the (token, expert) combos of a step are sorted by expert and cut
// into groups of up to four activation rows that share one expert, so an expert's weight bytes are streamed and
// decoded once per group instead of once per combo. Supersedes gemv_fp4_ptrb over the pointer tables
// (engine/src/kernels.rs:195-233, call sites engine/src/gen.rs:4499-4532) together with the grouping idea of the
// reference's prefill path (moe_count / moe_plan / moe_scatter, engine/src/kernels.rs:3334-3420).
//
// Persistent CTAs: the group list and its length live on the device (built by moe_group_kernel from the routing), the
// grid is fixed, and every CTA walks work items (group, part of the expert's row tiles) until the list ends: no CTA is
// launched for nothing when most slots of an expert-parallel inbox are empty. The producer warp streams the items'
// weight rows through one mbarrier ring without stopping between items; the consumer warps re-stage the (up to four)
// activation rows at every new group. Inner loops are those of the tensor-core GEMV (nvfp4_gemv_m1.cu): one row per
// group in "word" form, four rows in the packed-column form, summed so that a row's result does not depend on which
// group it rode in (bit-identical to a one-row call).
// Activations bf16 (exact as f16 x 2^e per 64-value block), or f32 held as TWO f16 planes - high part and the remainder
// times 2^11, 22 significant bits - that ride as two of the four row slots and are added at the end (the intermediate
// rows of the expert FFN); outputs f32. A row tile is 16 weight rows (8 gate + 8 up rows in the fused gate/up form); short rows
// (k = 512, 256) put two or four row tiles into one stage so that all eight consumer warps have a share.
#include "common.cuh"
#include "nvfp4_gemv.cuh"

namespace {

constexpr int NW = 8;
constexpr int NTHREADS = (NW + 1) * 32;
constexpr int MAX_STAGES = 8;
constexpr int RED_DEPTH = 10;
constexpr int XB = 128;
constexpr int TBAR_OFF = 128, ZERO_OFF = 224;
constexpr int ZERO2_OFF = ZERO_OFF + 2048;
constexpr int LUT_OFF = 2304;
constexpr int RED_OFF = LUT_OFF + 2048;  // [RED_DEPTH][NW][MT][16] f32
static_assert(ZERO2_OFF + 16 <= LUT_OFF && TBAR_OFF + RED_DEPTH * 8 <= ZERO_OFF, "header regions overlap");

struct RoutedParams {
    const int32_t* ids;    // [combos] expert of every combo
    const int32_t* order;  // [combos] combos sorted by expert
    const int* gcount;     // number of groups (device)
    const int* gpos;       // [groups] first position of the group in order[]
    const int* grows;      // [groups] rows of the group (null: one row each)
    const unsigned long long* tab0;
    const unsigned long long* tab1;
    int fused_up_rows;
    const float* gs0;
    const float* gs1;
    const void* x;
    int x_div, x_f32;
    float* y;
    const unsigned long long* yptrs;
    int ldy, rows, k;
    float limit;
    int stages, txb, rt;  // ring depth; blocks per row and stage; row tiles per stage
    uint32_t xs_off, stage_off;
};


// MT: row slots per group (1 or 4); TXB: 36-byte blocks per row and stage; RT: row tiles per stage
template <int MT, int TXB, int RT>
__global__ void __launch_bounds__(NTHREADS, MT == 1 ? 3 : 2) nvfp4_routed_kernel(const RoutedParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = (uint64_t*)smem;
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* tbar = (uint64_t*)(smem + TBAR_OFF);
    float* lut = (float*)(smem + LUT_OFF);
    float* red = (float*)(smem + RED_OFF);
    int* fail_s = (int*)(smem + 216);
    const int S = p.stages;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int bpr = p.k >> 6;
    constexpr int pstride = TXB * 36 + 16;
    constexpr int stage_bytes = RT * 16 * pstride;
    const int C = (bpr + TXB - 1) / TXB;  // chunks per row (1 when RT > 1)
    const size_t row_bytes = (size_t)bpr * 36;
    const bool gu = p.tab1 != nullptr || p.fused_up_rows > 0;
    const int per_tile = gu ? 8 : 16;                      // output rows per row tile
    const int T = (p.rows + per_tile - 1) / per_tile;      // row tiles of an expert
    const int ST = (T + RT - 1) / RT;                      // stages' worth of row tiles

    pdl_wait();  // the group list, ids and activations come from the kernels before this one
    // parts per group: about one and a half rounds of items for the grid, at least four stages per item; every CTA
    // computes the same
    const int ngroups = *p.gcount;
    int gx = ngroups > 0 ? (3 * (int)gridDim.x / 2 + ngroups - 1) / ngroups : 1;
    gx = gx > ST / 4 ? ST / 4 : gx;
    gx = gx < 1 ? 1 : gx;
    const int nitems = ngroups * gx;

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
        // ------------------------------------------------------------ weight producer
        const uint64_t pol = l2_policy_evict_first();
        int s = 0;
        uint32_t par = 0;
        bool first_round = true;
        // the pointer chain of an item (group -> position -> combo -> expert -> matrices) is four dependent loads: it is
        // resolved one item ahead, while the current item's copies are being issued
        auto resolve = [&](int w, const uint8_t*& w0, const uint8_t*& w1) {
            w0 = w1 = nullptr;
            if (w >= nitems) return;
            const int e = p.ids[p.order[p.gpos[w / gx]]];
            w0 = (const uint8_t*)p.tab0[e];
            w1 = p.tab1 ? (const uint8_t*)p.tab1[e] : (p.fused_up_rows > 0 ? w0 + (size_t)p.fused_up_rows * row_bytes : nullptr);
        };
        const uint8_t *nw0, *nw1;
        resolve(blockIdx.x, nw0, nw1);
        for (int w = blockIdx.x; w < nitems; w += gridDim.x) {
            const int g = w / gx, part = w - g * gx;
            const uint8_t *w0 = nw0, *w1 = nw1;
            resolve(w + gridDim.x, nw0, nw1);
            const int st0 = (int)(((long long)part * ST) / gx), st1 = (int)(((long long)(part + 1) * ST) / gx);
            for (int stt = st0; stt < st1; stt++) {
                for (int c = 0; c < C; c++) {
                    // lane l < 16: weight row slot l of row tile (stt * RT + r), r = 0 .. RT-1 in turn
                    const int nblk = min(TXB, bpr - c * TXB);
                    const uint32_t piece = (uint32_t)nblk * 36u;
                    uint32_t nvalid = 0;
                    const uint8_t* src[4];
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        src[r] = nullptr;
                        if (r < RT) {
                            const int tile = stt * RT + r;
                            const int row = gu ? tile * 8 + (lane & 7) : tile * 16 + lane;
                            const uint8_t* base = (gu && ((lane >> 3) & 1)) ? w1 : w0;
                            if (lane < 16 && tile < T && row < p.rows) src[r] = base + (size_t)row * row_bytes + (size_t)c * TXB * 36;
                            nvalid += (uint32_t)__popc(__ballot_sync(0xffffffffu, src[r] != nullptr));
                        }
                    }
                    if (!first_round && !mbar_wait(&empty[s], par ^ 1u)) {
                        cn_dev_fail(CN_DEV_WAIT_EMPTY);
                        return;
                    }
                    uint8_t* dst = smem + p.stage_off + (size_t)s * stage_bytes;
                    if (lane == 0) {
                        mbar_expect_tx(&full[s], nvalid * piece);
                        mbar_arrive(&full[s]);
                    }
                    __syncwarp();
#pragma unroll
                    for (int r = 0; r < 4; r++)
                        if (r < RT && src[r]) bulk_g2s_stream(dst + (size_t)(r * 16 + lane) * pstride, src[r], piece, &full[s], pol);
                    if (++s == S) {
                        s = 0;
                        par ^= 1u;
                        first_round = false;
                    }
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumer warps
    pdl_launch_dependents();
    const int g_ = lane >> 2, t = lane & 3;
    constexpr int gpr = TXB / 2;                       // groups (two 64-value blocks) per row tile and full stage
    constexpr int GPW = gpr >= NW ? gpr / NW : 1;      // groups per warp
    const int wrt = gpr >= NW ? 0 : warp / gpr;        // this warp's row tile inside a stage (RT > 1)
    const int wgr = gpr >= NW ? warp : warp % gpr;     // this warp's first group
    constexpr int gstep = gpr >= NW ? NW : gpr;        // distance between a warp's groups
    if (tid < 4) ((uint32_t*)(smem + ZERO_OFF))[tid] = 0u;
    if (tid >= 4 && tid < 8) ((uint32_t*)(smem + ZERO2_OFF))[tid - 4] = 0u;
    if (tid == 0) *fail_s = 0;
    {
        const float g0 = __ldg(p.gs0), g1 = gu ? __ldg(p.gs1) : g0;
        for (int b = tid; b < 256; b += NW * 32) {
            const float u = ue4m3_f32((uint32_t)b, true);
            lut[b] = u * g0;
            lut[256 + b] = u * g1;
        }
    }
    asm volatile("bar.sync 2, %0;" ::"n"(NTHREADS) : "memory");
    const float* lut_b = lut + (gu ? 256 : 0);
    uint8_t* xs0 = smem + p.xs_off;
    const uint32_t XS = (uint32_t)bpr * XB;
    float* xinv0 = (float*)(xs0 + (size_t)MT * XS);
    const uint32_t aoff = (uint32_t)((wrt * 16 + g_) * pstride + 4 * t + wgr * 72);
    const int sdelta = -4 * t + (t >> 1) * 36 + 2 * (t & 1);
    // one row: the lane's B registers of pair q come from its activations or from the zero chunk
    const int myq = ((g_ & 1) == (t >> 1)) ? (g_ >> 1) : -1;
    const int xb0 = 2 * wgr + (g_ >> 2);
    const uint32_t xoff_lane = p.xs_off + (uint32_t)(xb0 * XB + (((2 * (g_ & 3) + (t & 1)) ^ (xb0 & 7)) << 4));
    // four rows, packed columns: column g_ = activation row g_ >> 1, sub-block g_ & 1 of the pair in hand
    const bool live = MT > 1 && (t >> 1) == (g_ & 1) && (g_ >> 1) < MT;
    uint32_t xq_lane[4];
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const int blk = 2 * wgr + (q >> 1);
        xq_lane[q] = live ? p.xs_off + (uint32_t)((g_ >> 1) * XS + blk * XB + (((4 * (q & 1) + t) ^ (blk & 7)) << 4)) : (uint32_t)ZERO_OFF;
    }
    constexpr uint32_t jstep = (uint32_t)(gstep * 2 * XB);  // activation bytes between a warp's groups
    const int mrow = t < MT ? t : MT - 1;

    int s = 0, rslot = 0;
    uint32_t par = 0, rpar = 0;
    bool ok = true;
    int cur_group = -1;
    int mlive = 1;
    int combo[MT];
    for (int w = blockIdx.x; w < nitems && ok; w += gridDim.x) {
        const int g = w / gx, part = w - g * gx;
        if (g != cur_group) {
            cur_group = g;
            const int pos0 = p.gpos[g];
            mlive = p.grows ? p.grows[g] : 1;  // rows of the group (at most two when they are f32: two slots each)
#pragma unroll
            for (int m = 0; m < MT; m++) combo[m] = m < mlive ? p.order[pos0 + m] : -1;
            // ---- stage the group's activation rows (everybody has left the previous group's)
            asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
            if (*(volatile int*)fail_s) break;
            const int ntask = MT * bpr * 8;
            const bool split = MT > 1 && p.x_f32;  // row slot m = plane (m & 1) of the group's row m >> 1
            constexpr int PF = 4;  // tasks of a thread whose loads fly together
            for (int task0 = tid; task0 < ntask; task0 += PF * NW * 32) {
                uint4 ra[PF], rb2[PF];
#pragma unroll
                for (int pf = 0; pf < PF; pf++) {
                    const int task = task0 + pf * NW * 32;
                    ra[pf] = rb2[pf] = make_uint4(0u, 0u, 0u, 0u);
                    if (task >= ntask) continue;
                    const int b = task >> 3, i = task & 7;
                    const int m = MT == 1 ? 0 : b / bpr, blk = MT == 1 ? b : b - m * bpr;
                    const int mreal = split ? m >> 1 : m;
                    int c_m = combo[0];
#pragma unroll
                    for (int mm = 1; mm < MT; mm++) c_m = (mreal == mm) ? combo[mm] : c_m;
                    if (c_m < 0) continue;
                    if (p.x_f32) {
                        const uint4* src = (const uint4*)((const char*)p.x + ((size_t)(c_m / p.x_div) * p.k + (size_t)blk * 64 + i * 8) * 4);
                        ra[pf] = __ldcg(src), rb2[pf] = __ldcg(src + 1);
                    } else {
                        ra[pf] = __ldcg((const uint4*)((const char*)p.x + ((size_t)(c_m / p.x_div) * p.k + (size_t)blk * 64 + i * 8) * 2));
                    }
                }
#pragma unroll
                for (int pf = 0; pf < PF; pf++) {
                    const int task = task0 + pf * NW * 32;
                    if (task >= ntask) break;  // uniform over the warp: ntask is a multiple of 8 and tasks of a warp are consecutive
                    const int b = task >> 3, i = task & 7;
                    const int m = MT == 1 ? 0 : b / bpr, blk = MT == 1 ? b : b - m * bpr;
                    float v[8];
                    if (p.x_f32) {
                        v[0] = __uint_as_float(ra[pf].x), v[1] = __uint_as_float(ra[pf].y), v[2] = __uint_as_float(ra[pf].z), v[3] = __uint_as_float(ra[pf].w);
                        v[4] = __uint_as_float(rb2[pf].x), v[5] = __uint_as_float(rb2[pf].y), v[6] = __uint_as_float(rb2[pf].z), v[7] = __uint_as_float(rb2[pf].w);
                    } else {
                        const uint32_t u[4] = {ra[pf].x, ra[pf].y, ra[pf].z, ra[pf].w};
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            v[2 * q] = __uint_as_float(u[q] << 16);
                            v[2 * q + 1] = __uint_as_float(u[q] & 0xffff0000u);
                        }
                    }
                    float amax = 0.0f;
#pragma unroll
                    for (int q = 0; q < 8; q++) amax = fmaxf(amax, fabsf(v[q]));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
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
                        float a0 = v[2 * q] * mul, a1 = v[2 * q + 1] * mul;
                        __half2 hh = __floats2half2_rn(a0, a1);
                        if (split && (m & 1)) {
                            // low plane: what the high plane left (exact in f32), times 2^11
                            a0 = (a0 - __low2float(hh)) * 2048.0f, a1 = (a1 - __high2float(hh)) * 2048.0f;
                            hh = __floats2half2_rn(a0, a1);
                        }
                        h[q] = *(const uint32_t*)&hh;
                    }
                    ((uint4*)(xs0 + (size_t)b * XB))[i ^ (blk & 7)] = make_uint4(h[0], h[1], h[2], h[3]);
                    if (i == 0) xinv0[b] = (split && (m & 1)) ? inv * (1.0f / 2048.0f) : inv;
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
        }
        const int st0 = (int)(((long long)part * ST) / gx), st1 = (int)(((long long)(part + 1) * ST) / gx);
        for (int stt = st0; stt < st1 && ok; stt++) {
            float acc0 = 0.0f, acc1 = 0.0f;     // one row: weight rows g_ and g_ + 8, this lane's two columns
            float pk0[4], pk1[4];               // four rows: activation row t, per pair
#pragma unroll
            for (int q = 0; q < 4; q++) pk0[q] = pk1[q] = 0.0f;
            for (int c = 0; c < C; c++) {
                const int ng = min(TXB, bpr - c * TXB) >> 1;
                if (!mbar_wait(&full[s], par)) {
                    cn_dev_fail(CN_DEV_WAIT_FULL);
                    ok = false;
                    break;
                }
                const uint8_t* pa0 = smem + p.stage_off + (size_t)s * stage_bytes + aoff;
#pragma unroll
                for (int j = 0; j < GPW; j++) {
                    if (wgr + gstep * j >= ng) break;
                    const uint8_t* pa = pa0 + j * (gstep * 72);
                    const uint8_t* pb = pa + 8 * pstride;
                    const uint32_t xadd = (uint32_t)(c * TXB * XB) + j * jstep;
                    if constexpr (MT == 1) {
                        float cc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const int off = (q >> 1) * 36 + 4 + 16 * (q & 1);
                            uint32_t ha[4], hb[4];
                            e2m1x8_to_f16x2(*(const uint32_t*)(pa + off), ha);
                            e2m1x8_to_f16x2(*(const uint32_t*)(pb + off), hb);
                            // the zero chunks sit where any group offset of a warp lands on zeros as well
                            const uint4 xv = myq == q ? *(const uint4*)(smem + xoff_lane + xadd) : make_uint4(0u, 0u, 0u, 0u);
                            mma16816(cc, ha[0], hb[0], ha[1], hb[1], xv.x, xv.y);
                            mma16816(cc, ha[2], hb[2], ha[3], hb[3], xv.z, xv.w);
                        }
                        const uint8_t* sc = pa + sdelta;
                        const float s0 = lut[sc[0]], s1 = lut[sc[1]], s2 = lut_b[sc[8 * pstride]], s3 = lut_b[sc[8 * pstride + 1]];
                        const float xi = xinv0[c * TXB + 2 * (wgr + gstep * j) + (t >> 1)];
                        acc0 = fmaf(fmaf(cc[1], s1, cc[0] * s0), xi, acc0);
                        acc1 = fmaf(fmaf(cc[3], s3, cc[2] * s2), xi, acc1);
                    } else {
                        const uint8_t* sr = pa - 4 * t;
                        const uint32_t sw0[2] = {*(const uint32_t*)sr, *(const uint32_t*)(sr + 36)};
                        const uint32_t sw1[2] = {*(const uint32_t*)(sr + 8 * pstride), *(const uint32_t*)(sr + 8 * pstride + 36)};
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const int off = (q >> 1) * 36 + 4 + 16 * (q & 1);
                            uint32_t ha[4], hb[4];
                            e2m1x8_to_f16x2(*(const uint32_t*)(pa + off), ha);
                            e2m1x8_to_f16x2(*(const uint32_t*)(pb + off), hb);
                            const uint32_t wa = sw0[q >> 1], wb = sw1[q >> 1];
                            const uint32_t o0 = (q & 1) ? (wa >> 14) & 0x3fcu : (wa << 2) & 0x3fcu, o1 = (q & 1) ? (wa >> 22) & 0x3fcu : (wa >> 6) & 0x3fcu;
                            const uint32_t o2 = (q & 1) ? (wb >> 14) & 0x3fcu : (wb << 2) & 0x3fcu, o3 = (q & 1) ? (wb >> 22) & 0x3fcu : (wb >> 6) & 0x3fcu;
                            const float s0 = *(const float*)((const char*)lut + o0), s1 = *(const float*)((const char*)lut + o1);
                            const float s2 = *(const float*)((const char*)lut_b + o2), s3 = *(const float*)((const char*)lut_b + o3);
                            const uint4 xv = live ? *(const uint4*)(smem + xq_lane[q] + xadd) : make_uint4(0u, 0u, 0u, 0u);
                            float cc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                            mma16816(cc, ha[0], hb[0], ha[1], hb[1], xv.x, xv.y);
                            mma16816(cc, ha[2], hb[2], ha[3], hb[3], xv.z, xv.w);
                            const float xi = xinv0[mrow * bpr + c * TXB + 2 * (wgr + gstep * j) + (q >> 1)];
                            pk0[q] = fmaf(fmaf(cc[1], s1, cc[0] * s0), xi, pk0[q]);
                            pk1[q] = fmaf(fmaf(cc[3], s3, cc[2] * s2), xi, pk1[q]);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
                if (++s == S) {
                    s = 0;
                    par ^= 1u;
                }
            }
            if (!ok) break;
            // the warps' K ranges (and, with several row tiles per stage, the row tiles) meet in shared memory
            float* rb = red + rslot * (NW * MT * 16);
            if constexpr (MT == 1) {
                float a = acc0, b = acc1;
                a += __shfl_xor_sync(0xffffffffu, a, 1);
                b += __shfl_xor_sync(0xffffffffu, b, 1);
                a += __shfl_xor_sync(0xffffffffu, a, 2);
                b += __shfl_xor_sync(0xffffffffu, b, 2);
                if (t == 0) {
                    rb[warp * 16 + g_] = a;
                    rb[warp * 16 + g_ + 8] = b;
                }
            } else {
                if (t < MT) {
                    rb[(warp * MT + t) * 16 + g_] = (pk0[0] + pk0[1]) + (pk0[2] + pk0[3]);
                    rb[(warp * MT + t) * 16 + g_ + 8] = (pk1[0] + pk1[1]) + (pk1[2] + pk1[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&tbar[rslot]);
            if (warp == 0) {
                if (!mbar_wait(&tbar[rslot], rpar)) {
                    cn_dev_fail(CN_DEV_WAIT_FULL);
                    *fail_s = 1;
                } else {
                    constexpr int nwr = gpr >= NW ? NW : gpr;  // warps that share one row tile
                    for (int r = 0; r < RT; r++) {
                        const int tile = stt * RT + r;
                        if (tile >= T) break;
                        const int wbase = gpr >= NW ? 0 : r * gpr;
                        const bool split = MT > 1 && p.x_f32;
#pragma unroll
                        for (int m = 0; m < MT; m++) {
                            if (m >= mlive) break;
                            float v = 0.0f;
                            if (lane < 16) {
                                if (split) {
                                    // high plane over the warps in order, then the low plane the same way, then their sum
                                    float lo = rb[((wbase)*MT + 2 * m + 1) * 16 + lane];
                                    v = rb[((wbase)*MT + 2 * m) * 16 + lane];
                                    for (int ww = 1; ww < nwr; ww++) {
                                        v += rb[((wbase + ww) * MT + 2 * m) * 16 + lane];
                                        lo += rb[((wbase + ww) * MT + 2 * m + 1) * 16 + lane];
                                    }
                                    v += lo;
                                } else {
                                    v = rb[((wbase)*MT + m) * 16 + lane];
                                    for (int ww = 1; ww < nwr; ww++) v += rb[((wbase + ww) * MT + m) * 16 + lane];
                                }
                            }
                            const float up = __shfl_down_sync(0xffffffffu, v, 8);
                            const int row = tile * per_tile + lane;
                            if (lane < per_tile && row < p.rows) {
                                const float rr = gu ? act_gu(v, up, p.limit) : v;
                                float* yb = p.yptrs ? (float*)(uintptr_t)p.yptrs[combo[m]] : p.y + (size_t)combo[m] * p.ldy;
                                yb[row] = rr;
                            }
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
}

}  // namespace

// One class of groups (all one-row groups, or all groups of two to four rows) as one persistent launch.
int cn_routed_launch(const RoutedCall& a, cudaStream_t stream, const char* who) {
    if (a.rows <= 0 || a.k <= 0 || a.k % 256 != 0) CN_FAIL(CN_ERR_SHAPE, "%s: k = %d must be a positive multiple of 256", who, a.k);
    if (a.mt != 1 && a.mt != 4) CN_FAIL(CN_ERR_SHAPE, "%s: groups of %d rows", who, a.mt);
    if (a.x_f32 && a.mt != 4) CN_FAIL(CN_ERR_SHAPE, "%s: f32 rows ride two row slots each and need the four-slot kernel", who);
    const int bpr = a.k / 64;
    // blocks per row and stage / row tiles per stage: long rows in chunks of 32 blocks, short ones several tiles at once
    int txb = 32, rt = 1;
    if (bpr == 8) txb = 8, rt = 2;
    if (bpr == 4) txb = 4, rt = 4;
    if (bpr == 16) txb = 16;
    const int pstride = txb * 36 + 16;
    const size_t stage_bytes = (size_t)rt * 16 * pstride;
    const int cps = a.mt == 1 ? 3 : 2;
    const uint32_t xs_off = (uint32_t)(RED_OFF + RED_DEPTH * NW * a.mt * 64);
    const uint32_t stage_off = (uint32_t)((xs_off + (size_t)a.mt * bpr * XB + (size_t)a.mt * bpr * 4 + 127) & ~(size_t)127);
    int stages = (int)(((227 * 1024) / cps - 1024 - (long long)stage_off) / (long long)stage_bytes);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) CN_FAIL(CN_ERR_LIMIT, "%s: k = %d leaves no room for a weight ring beside %d activation rows", who, a.k, a.mt);
    const bool gu = a.tab1 != nullptr || a.fused_up_rows > 0;
    const int T = (a.rows + (gu ? 8 : 16) - 1) / (gu ? 8 : 16), ST = (T + rt - 1) / rt;
    // a full machine of persistent CTAs unless even the longest possible group list cannot feed it
    int dev = 0, sms = 148;
    CN_CUDA(cudaGetDevice(&dev));
    CN_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    long long grid = (long long)a.max_groups * (ST / 4 > 0 ? ST / 4 : 1);
    if (grid > sms * cps) grid = sms * cps;
    if (grid < 1) grid = 1;
    RoutedParams p = {};
    p.ids = a.ids, p.order = a.order, p.gcount = a.gcount, p.gpos = a.gpos, p.grows = a.grows, p.tab0 = a.tab0, p.tab1 = a.tab1;
    p.fused_up_rows = a.fused_up_rows, p.gs0 = a.gs0, p.gs1 = a.gs1 ? a.gs1 : a.gs0, p.x = a.x, p.x_div = a.x_div, p.x_f32 = a.x_f32, p.y = a.y;
    p.yptrs = a.yptrs, p.ldy = a.ldy, p.rows = a.rows, p.k = a.k, p.limit = a.limit, p.stages = stages, p.txb = txb, p.rt = rt;
    p.xs_off = xs_off, p.stage_off = stage_off;
    const size_t smem = stage_off + (size_t)stages * stage_bytes;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid), cfg.blockDim = dim3(NTHREADS), cfg.dynamicSmemBytes = smem, cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at, cfg.numAttrs = 1;
#define CN_ROUTED_CASE(MTV, TXV, RTV)                                                   \
    if (a.mt == MTV && txb == TXV && rt == RTV) {                                       \
        CN_ALLOW_SMEM((nvfp4_routed_kernel<MTV, TXV, RTV>), 226 * 1024);                \
        CN_CUDA(cudaLaunchKernelEx(&cfg, nvfp4_routed_kernel<MTV, TXV, RTV>, p));       \
        return CN_OK;                                                                   \
    }
    CN_ROUTED_CASE(1, 32, 1) CN_ROUTED_CASE(1, 16, 1) CN_ROUTED_CASE(1, 8, 2) CN_ROUTED_CASE(1, 4, 4)
    CN_ROUTED_CASE(4, 32, 1) CN_ROUTED_CASE(4, 16, 1) CN_ROUTED_CASE(4, 8, 2) CN_ROUTED_CASE(4, 4, 4)
#undef CN_ROUTED_CASE
    CN_FAIL(CN_ERR_SHAPE, "%s: no kernel for %d row slots, %d blocks per stage", who, a.mt, txb);
}
