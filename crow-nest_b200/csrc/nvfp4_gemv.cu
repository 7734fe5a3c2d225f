// NVFP4 GEMV for M = 1..8 activation rows on sm_100a: the decode projection of the dense family
// and its small-M (speculative verify) form, plain or with the fused gate/up activation.
//
// Supersedes gemv_nvfp4_w / _gu / _wm / _gum (engine/src/kernels_p2.rs:355-530) and the record
// kernels gemv_fp4(_b) (engine/src/kernels.rs:118-189), glm5_gemv_fp4 (engine/src/kernels_glm5_moe.cu:284).
//
// Shape of the kernel (HBM-bound; the container layout is consumed as it lies, no repack):
//   - a CTA owns ROWS output rows over the whole K. A producer warp streams the rows' bytes
//     through a ring of shared-memory stages with 1-D bulk copies (TMA, completion counted on an
//     mbarrier), one piece of TX 36-byte blocks per row and stage; it never waits for anything
//     but a free stage, so the weight stream runs ahead of the arithmetic;
//   - a second helper warp stages the matching slice of the M activation rows, converted once
//     per CTA: bf16 -> f16 with a power-of-two scale per 64-value block (exact; the inverse is
//     applied with the block's partial sum), or f32 kept as f32;
//   - consumer warps: lane (ry, tx) owns k-block tx of the stage for RT rows; the nine words of a
//     block are read with conflict-free 4-byte loads (36-byte stride), codes are decoded in
//     registers (cvt.rn.f16x2.e2m1x2: every E2M1 value is exact in f16) and multiplied with
//     fma.rn.f32.f16 (f16 x f16 product exact, f32 accumulate; measured at the FFMA rate on
//     B200), each 16-value sub-block's partial sum is multiplied by its UE4M3 scale * tensor
//     scale (a 256-entry table, the reference's scale_lut) and accumulated in f32; the K split
//     over the TX lanes is reduced with xor shuffles in a fixed order.
// Each (row, m) pair runs the same instruction sequence whatever M is, so row m of an M-row call
// is bit-identical to a one-row call (the batch invariance of engine/src/kernels_p2.rs:391-396).
#include <cstdarg>
#include <cstdio>

#include "common.cuh"
#include "nvfp4_gemv.cuh"

namespace {

constexpr int NW = 4;  // consumer warps
constexpr int NTHREADS = (NW + 1) * 32;
constexpr int MAX_STAGES = 8;
constexpr int XB_F16 = 144;  // bytes of one k-block's 64 activations as f16, padded: conflict-free 16-byte loads
constexpr int XB_F32 = 272;  // the same as f32
constexpr int XB_SWZ = 128;  // bf16 rows staged by TMA, converted in place: 16-byte chunks XOR-swizzled instead of padded
constexpr int HDR_BYTES = 256 + 2048;  // barriers, two scale tables

// one load group of eight activation values: raw words in flight, widened exactly to f32 on use
template <int XT>
struct XRaw {
    uint4 a;
    uint4 b;  // f32 input only
};
template <int XT>
__device__ __forceinline__ void load_x8(const void* x, size_t at, XRaw<XT>& r) {
    if (XT == 1) {
        r.a = *(const uint4*)((const __nv_bfloat16*)x + at);
    } else {
        r.a = *(const uint4*)((const float*)x + at);
        r.b = *(const uint4*)((const float*)x + at + 4);
    }
}
template <int XT>
__device__ __forceinline__ void widen_x8(const XRaw<XT>& r, float v[8]) {
    if (XT == 1) {
        const uint32_t u[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            v[2 * i] = __uint_as_float(u[i] << 16);
            v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
        }
    } else {
        v[0] = __uint_as_float(r.a.x), v[1] = __uint_as_float(r.a.y), v[2] = __uint_as_float(r.a.z), v[3] = __uint_as_float(r.a.w);
        v[4] = __uint_as_float(r.b.x), v[5] = __uint_as_float(r.b.y), v[6] = __uint_as_float(r.b.z), v[7] = __uint_as_float(r.b.w);
    }
}

// XT: 0 = f32 activations/outputs, 1 = bf16. MP: activation rows compiled in (1, 2, 4, 8).
// RT: rows per consumer thread. MODE: 0 = f32 FMA, 1 = f16 x f16 + f32 mixed FMA (bf16 input only).
template <int XT, int MP, int RT, int MODE>
__global__ void __launch_bounds__(NTHREADS, (MP <= 2 ? 4 : 1)) nvfp4_gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr bool SWZ = XT == 1 && MODE == 1;
    constexpr int XB = SWZ ? XB_SWZ : (MODE == 1 ? XB_F16 : XB_F32);
    const int TX = p.tx;
    const int G = NW * (32 / TX);  // row groups per CTA
    const int ROWS = G * RT;       // row slots per stage
    const int piece = TX * 36;     // bytes of one row's share of a stage
    const int bpr = p.k >> 6;
    const size_t row_bytes = (size_t)bpr * 36;
    const int nchunks = bpr / TX;
    const int S = p.stages;
    const uint8_t* w0 = p.w0;
    const uint8_t* w1 = p.w1;
    const char* xbase = (const char*)p.x;
    char* ybase = (char*)p.y;
    if (p.ids) {
        // ids, order and tables may come from the kernels just before this one, and a CTA whose expert is not resident
        // returns at once: wait for the predecessor grid first, so that even a grid whose CTAs all return early
        // completes only after its predecessor has
        pdl_wait();
        const int c = p.order ? p.order[blockIdx.y] : (int)blockIdx.y;
        const int e = p.ids[c];
        if (e < 0 || (p.experts > 0 && e >= p.experts)) return;  // uniform over the CTA, before any barrier
        w0 = (const uint8_t*)p.tab0[e];
        if (!w0) return;  // the expert is not resident here: nothing to read or write
        w1 = p.tab1 ? (const uint8_t*)p.tab1[e] : (p.fused_up_rows > 0 ? w0 + (size_t)p.fused_up_rows * row_bytes : nullptr);
        xbase += (size_t)(c / p.x_div) * p.k * (XT == 1 ? 2 : 4);
        ybase = p.yptrs ? (char*)p.yptrs[c] : ybase + (size_t)c * p.ldy * ((XT == 1 && !p.out_f32) ? 2 : 4);
    }
    const bool gu = w1 != nullptr;

    uint64_t* full = (uint64_t*)smem;
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* xbar = empty + MAX_STAGES;  // the activation rows have landed
    float* lut = (float*)(smem + 256);    // [2][256]
    uint8_t* xs0 = smem + HDR_BYTES;                              // [MP][bpr][XB] staged activations
    float* xinv0 = (float*)(xs0 + (size_t)MP * bpr * XB);         // [MP][bpr] inverse block scales
    uint8_t* stage0 = (uint8_t*)(xinv0 + ((MP * bpr + 3) & ~3));  // the weight ring
    const int stage_bytes = ROWS * piece;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // output rows of this CTA: plain ROWS consecutive rows; gate/up ROWS/2 consecutive indices
    const int per_cta = gu ? ROWS / 2 : ROWS;
    const int row0 = blockIdx.x * per_cta;

    if (tid == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(&full[s], 1);  // the producer's expect_tx arrive; the copies count bytes
            mbar_init(&empty[s], NW);
        }
        mbar_init(xbar, 1);
        mbar_fence_init();
    }
    // scale tables: ue4m3(rule(byte)) * gs, the product the reference tabulates (cpu_nvfp4.rs:98)
    {
        const float g0 = p.gs0[0], g1 = gu ? p.gs1[0] : g0;
        for (int b = tid; b < 256; b += NTHREADS) {
            const float u = ue4m3_f32((uint32_t)b, true);
            lut[b] = u * g0;
            lut[256 + b] = u * g1;
        }
    }
    __syncthreads();
    // let the next kernel of the stream begin its own weight prefetch while this one drains
    pdl_launch_dependents();

    if (warp == NW) {
        // ------------------------------------------------------------ weight producer warp
        // source row of slot sl = j*G + g: plain row0 + sl; gate/up: matrix j & 1, index row0 + (j>>1)*G + g
        const uint64_t pol = l2_policy_evict_first();
        const uint8_t* src[4];
        uint32_t total = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int sl = lane + 32 * i;
            src[i] = nullptr;
            if (sl < ROWS) {
                const int j = sl / G, g = sl % G;
                const int r = gu ? row0 + (j >> 1) * G + g : row0 + sl;
                const uint8_t* base = (gu && (j & 1)) ? w1 : w0;
                if (r < p.rows) src[i] = base + (size_t)r * row_bytes;
            }
            total += src[i] ? piece : 0;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        for (int c = 0; c < nchunks; c++) {
            const int s = c % S;
            if (c >= S && !mbar_wait(&empty[s], ((c / S) - 1) & 1)) {
                cn_dev_fail(CN_DEV_WAIT_EMPTY);
                return;
            }
            uint8_t* st = stage0 + (size_t)s * stage_bytes;
            if (lane == 0) {
                mbar_expect_tx(&full[s], total);
                mbar_arrive(&full[s]);
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; i++)
                if (src[i]) bulk_g2s_stream(st + (size_t)(lane + 32 * i) * piece, src[i] + (size_t)c * piece, piece, &full[s], pol);
        }
        return;
    }

    // ---------------------------------------------------------------- consumer warps
    // First the activations: every row, the whole K, staged once per CTA while the producer fills
    // the weight ring. Groups of 8 values; lane & 7 = position in the 64-value block, so the 8
    // lanes of a block sit side by side. All loads of a batch are in flight before the first
    // conversion (one L2 round trip per batch, not per group).
    if (SWZ) {
        // bf16 rows: one bulk copy per row into shared memory, then an in-place conversion to f16 with a
        // power-of-two scale per 64-value block. A thread owns whole 128-byte blocks (no exchange) and
        // writes the eight 16-byte chunks of block b at chunk index i ^ (b & 7): conflict-free 16-byte
        // loads for eight lanes reading eight consecutive blocks, without padding.
        if (tid == 0) {
            pdl_wait();  // activations may come from the previous kernel of the stream
            mbar_expect_tx(xbar, (uint32_t)p.m * (uint32_t)p.k * 2u);
            mbar_arrive(xbar);
            for (int m = 0; m < p.m; m++) bulk_g2s(xs0 + (size_t)m * bpr * XB, xbase + (size_t)m * p.k * 2, (uint32_t)p.k * 2u, xbar);
        }
        if (!mbar_wait(xbar, 0)) {
            cn_dev_fail(CN_DEV_WAIT_FULL);
            return;
        }
        for (int b = tid; b < MP * bpr; b += NW * 32) {
            const int m = b / bpr;
            uint4* blkp = (uint4*)(xs0 + (size_t)b * XB);
            uint4 raw[8];
#pragma unroll
            for (int i = 0; i < 8; i++) raw[i] = m < p.m ? blkp[i] : make_uint4(0, 0, 0, 0);
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t u[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    amax = fmaxf(amax, fabsf(__uint_as_float(u[q] << 16)));
                    amax = fmaxf(amax, fabsf(__uint_as_float(u[q] & 0xffff0000u)));
                }
            }
            uint32_t e = (__float_as_uint(amax) >> 23) & 0xFF;
            float mul = 1.0f, inv = 1.0f;
            if (amax > 0.0f && e < 255) {
                e = e < 15 ? 15 : e;
                mul = __uint_as_float((268u - e) << 23);
                inv = __uint_as_float((e - 14u) << 23);
            }
            const int sw = (b % bpr) & 7;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t u[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
                uint32_t h[4];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const __half2 hh = __floats2half2_rn(__uint_as_float(u[q] << 16) * mul, __uint_as_float(u[q] & 0xffff0000u) * mul);
                    h[q] = *(const uint32_t*)&hh;
                }
                blkp[i ^ sw] = make_uint4(h[0], h[1], h[2], h[3]);
            }
            xinv0[b] = inv;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
    } else {
        pdl_wait();  // activations may come from the previous kernel of the stream
        constexpr int BATCH = 4;
        const int groups = MP * bpr * 8;
        for (int g0 = 0; g0 < groups; g0 += BATCH * NW * 32) {
            XRaw<XT> raw[BATCH];
#pragma unroll
            for (int b = 0; b < BATCH; b++) {
                const int gq = g0 + b * NW * 32 + tid;
                const int m = gq / (bpr * 8), gi = gq % (bpr * 8);
                raw[b].a = make_uint4(0, 0, 0, 0);
                raw[b].b = make_uint4(0, 0, 0, 0);
                if (gq < groups && m < p.m) load_x8<XT>(xbase, (size_t)m * p.k + (size_t)gi * 8, raw[b]);
            }
#pragma unroll
            for (int b = 0; b < BATCH; b++) {
                const int gq = g0 + b * NW * 32 + tid;
                const int m = gq / (bpr * 8), gi = gq % (bpr * 8), kb = gi >> 3, wi = gi & 7;
                const bool live = gq < groups;  // uniform over each aligned group of 8 lanes
                uint8_t* dst = xs0 + (size_t)(m * bpr + kb) * XB;
                float vv[8];
                widen_x8<XT>(raw[b], vv);
                if (MODE == 1) {
                    // power-of-two scale per 64-value block: |x| * mul < 2^15, exact in f16
                    float amax = 0.0f;
#pragma unroll
                    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(vv[i]));
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
                    if (live) {
                        uint32_t h[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const __half2 hh = __floats2half2_rn(vv[2 * i] * mul, vv[2 * i + 1] * mul);
                            h[i] = *(const uint32_t*)&hh;
                        }
                        *(uint4*)(dst + wi * 16) = make_uint4(h[0], h[1], h[2], h[3]);
                        if (wi == 0) xinv0[m * bpr + kb] = inv;
                    }
                } else if (live) {
                    *(float4*)(dst + wi * 32) = make_float4(vv[0], vv[1], vv[2], vv[3]);
                    *(float4*)(dst + wi * 32 + 16) = make_float4(vv[4], vv[5], vv[6], vv[7]);
                }
            }
        }
        // the consumer warps only (the producer warp is streaming): named barrier 1
        asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
    }
    const int txi = lane % TX, ry = lane / TX;
    const int g = warp * (32 / TX) + ry;
    float acc[RT][MP];
#pragma unroll
    for (int r = 0; r < RT; r++)
#pragma unroll
        for (int m = 0; m < MP; m++) acc[r][m] = 0.0f;

    for (int c = 0; c < nchunks; c++) {
        const int s = c % S;
        if (!mbar_wait(&full[s], (c / S) & 1)) {
            cn_dev_fail(CN_DEV_WAIT_FULL);
            return;
        }
        const uint8_t* st = stage0 + (size_t)s * stage_bytes;
        uint32_t wv[RT][9];
#pragma unroll
        for (int r = 0; r < RT; r++) {
            const uint32_t* wp = (const uint32_t*)(st + (size_t)(r * G + g) * piece + txi * 36);
#pragma unroll
            for (int i = 0; i < 9; i++) wv[r][i] = wp[i];
        }
        const uint8_t* xs = xs0 + (size_t)(c * TX + txi) * XB;
        float blk[RT][MP];
#pragma unroll
        for (int r = 0; r < RT; r++)
#pragma unroll
            for (int m = 0; m < MP; m++) blk[r][m] = 0.0f;
#pragma unroll
        for (int sb = 0; sb < 4; sb++) {
            if (MODE == 1) {
                uint4 xa[MP], xb[MP];
#pragma unroll
                for (int m = 0; m < MP; m++) {
                    const uint4* xp = (const uint4*)(xs + (size_t)m * bpr * XB);
                    if (SWZ) {
                        const int sw = (c * TX + txi) & 7;
                        xa[m] = xp[(2 * sb) ^ sw];
                        xb[m] = xp[(2 * sb + 1) ^ sw];
                    } else {
                        xa[m] = xp[2 * sb];
                        xb[m] = xp[2 * sb + 1];
                    }
                }
#pragma unroll
                for (int r = 0; r < RT; r++) {
                    const float sc = lut[((gu && (r & 1)) ? 256 : 0) + ((wv[r][0] >> (8 * sb)) & 0xFF)];
                    const uint32_t c0 = wv[r][1 + 2 * sb], c1 = wv[r][2 + 2 * sb];
                    uint32_t h[8];
                    e2m1x8_to_f16x2(c0, h);
                    e2m1x8_to_f16x2(c1, h + 4);
#pragma unroll
                    for (int m = 0; m < MP; m++) {
                        const uint32_t xv[8] = {xa[m].x, xa[m].y, xa[m].z, xa[m].w, xb[m].x, xb[m].y, xb[m].z, xb[m].w};
                        float p0 = 0.0f, p1 = 0.0f;  // even / odd values: two independent chains
#pragma unroll
                        for (int i = 0; i < 8; i++) fma2_f16_f32(p0, p1, h[i], xv[i]);
                        blk[r][m] = fmaf(p0 + p1, sc, blk[r][m]);
                    }
                }
            } else {
                float xv[MP][16];
#pragma unroll
                for (int m = 0; m < MP; m++) {
                    const float4* xp = (const float4*)(xs + (size_t)m * bpr * XB + sb * 64);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float4 t = xp[i];
                        xv[m][4 * i] = t.x, xv[m][4 * i + 1] = t.y, xv[m][4 * i + 2] = t.z, xv[m][4 * i + 3] = t.w;
                    }
                }
#pragma unroll
                for (int r = 0; r < RT; r++) {
                    const float sc = lut[((gu && (r & 1)) ? 256 : 0) + ((wv[r][0] >> (8 * sb)) & 0xFF)];
                    const uint32_t c0 = wv[r][1 + 2 * sb], c1 = wv[r][2 + 2 * sb];
                    float wf[16];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const uint32_t h0 = e2m1x2_to_f16x2((c0 >> (8 * i)) & 0xFF), h1 = e2m1x2_to_f16x2((c1 >> (8 * i)) & 0xFF);
                        wf[2 * i] = f16lo_to_f32(h0), wf[2 * i + 1] = f16hi_to_f32(h0);
                        wf[8 + 2 * i] = f16lo_to_f32(h1), wf[8 + 2 * i + 1] = f16hi_to_f32(h1);
                    }
#pragma unroll
                    for (int m = 0; m < MP; m++) {
                        float p0 = 0.0f, p1 = 0.0f;
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            p0 = fmaf(wf[2 * i], xv[m][2 * i], p0);
                            p1 = fmaf(wf[2 * i + 1], xv[m][2 * i + 1], p1);
                        }
                        blk[r][m] = fmaf(p0 + p1, sc, blk[r][m]);
                    }
                }
            }
        }
        if (MODE == 1) {
#pragma unroll
            for (int m = 0; m < MP; m++) {
                const float inv = xinv0[m * bpr + c * TX + txi];
#pragma unroll
                for (int r = 0; r < RT; r++) acc[r][m] = fmaf(blk[r][m], inv, acc[r][m]);
            }
        } else {
#pragma unroll
            for (int r = 0; r < RT; r++)
#pragma unroll
                for (int m = 0; m < MP; m++) acc[r][m] += blk[r][m];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }

    // K split over the TX lanes: xor-shuffle tree, fixed order
#pragma unroll
    for (int r = 0; r < RT; r++)
#pragma unroll
        for (int m = 0; m < MP; m++) {
            float v = acc[r][m];
            for (int o = TX >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            acc[r][m] = v;
        }
    if (txi == 0) {
        if (!gu) {
#pragma unroll
            for (int r = 0; r < RT; r++) {
                const int row = row0 + r * G + g;
                if (row < p.rows) {
#pragma unroll
                    for (int m = 0; m < MP; m++)
                        if (m < p.m) {
                            if (XT == 1 && !p.out_f32)
                                ((__nv_bfloat16*)ybase)[(size_t)m * p.ldy + row] = __float2bfloat16_rn(acc[r][m]);
                            else
                                ((float*)ybase)[(size_t)m * p.ldy + row] = acc[r][m];
                        }
                }
            }
        } else {
#pragma unroll
            for (int r = 0; r + 1 < RT; r += 2) {
                const int row = row0 + (r >> 1) * G + g;
                if (row < p.rows) {
#pragma unroll
                    for (int m = 0; m < MP; m++)
                        if (m < p.m) {
                            const float h = act_gu(acc[r][m], acc[r + 1][m], p.limit);
                            if (XT == 1 && !p.out_f32)
                                ((__nv_bfloat16*)ybase)[(size_t)m * p.ldy + row] = __float2bfloat16_rn(h);
                            else
                                ((float*)ybase)[(size_t)m * p.ldy + row] = h;
                        }
                }
            }
        }
    }
}

// out[r][c] = e2m1(code) * (ue4m3(byte) * gs): one thread per 8 values (one code word)
__global__ void nvfp4_dequant_kernel(const uint8_t* __restrict__ w, const float* __restrict__ gs, float* __restrict__ out,
                                     long long nwords, int rule) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nwords) return;
    const long long blk = i >> 3;
    const int wi = (int)(i & 7);
    const uint8_t* b = w + blk * 36;
    const float s = ue4m3_f32(b[wi >> 1], rule != 0) * gs[0];
    const uint32_t cw = *(const uint32_t*)(b + 4 + 4 * wi);
    float* o = out + blk * 64 + wi * 8;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t h = e2m1x2_to_f16x2((cw >> (8 * j)) & 0xFF);
        o[2 * j] = f16lo_to_f32(h) * s;
        o[2 * j + 1] = f16hi_to_f32(h) * s;
    }
}

template <int XT, int MP, int RT, int MODE>
int launch_one(const GemvParams& p, int grid, int gy, size_t smem, cudaStream_t stream) {
    auto kern = nvfp4_gemv_kernel<XT, MP, RT, MODE>;
    CN_ALLOW_SMEM(kern, 200 * 1024);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, (unsigned)gy);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    CN_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
    return CN_OK;
}

template <int XT, int MODE>
int launch_m(const GemvParams& p, int mp, int rt, int grid, int gy, size_t smem, cudaStream_t stream) {
#define CN_CASE(MPV, RTV) \
    if (mp == MPV && rt == RTV) return launch_one<XT, MPV, RTV, MODE>(p, grid, gy, smem, stream);
    CN_CASE(1, 2) CN_CASE(1, 4) CN_CASE(2, 2) CN_CASE(2, 4) CN_CASE(4, 2) CN_CASE(4, 4) CN_CASE(8, 2) CN_CASE(8, 4)
#undef CN_CASE
    CN_FAIL(CN_ERR_SHAPE, "nvfp4 gemv: no kernel for m %d, rows per thread %d", mp, rt);
}

}  // namespace

// One launch of the GEMV family (declared in nvfp4_gemv.cuh for the MoE operator).
int cn_gemv_launch(const GemvCall& a, cudaStream_t stream, const char* who) {
    const int rows = a.rows, k = a.k, m = a.m;
    if (rows <= 0 || k <= 0 || k % 256 != 0) CN_FAIL(CN_ERR_SHAPE, "%s: k = %d must be a positive multiple of 256 (rows of 16-byte multiples)", who, k);
    if (m < 1 || m > CN_MAX_M) CN_FAIL(CN_ERR_LIMIT, "%s: m = %d, the kernel takes 1..%d activation rows", who, m, CN_MAX_M);
    if (a.ldy < rows) CN_FAIL(CN_ERR_SHAPE, "%s: ldy %d < rows %d", who, a.ldy, rows);
    if (a.dtype != CN_F32 && a.dtype != CN_BF16) CN_FAIL(CN_ERR_SHAPE, "%s: dtype %d is neither CN_F32 nor CN_BF16", who, a.dtype);
    if (((uintptr_t)a.w0 & 15) || ((uintptr_t)a.w1 & 15) || ((uintptr_t)a.x & 15))
        CN_FAIL(CN_ERR_SHAPE, "%s: weight and activation pointers must be 16-byte aligned", who);
    const bool routed = a.ids != nullptr;
    if (routed && (m != 1 || a.combos < 1 || a.x_div < 1)) CN_FAIL(CN_ERR_SHAPE, "%s: the routed form takes one row per combo", who);
    // bf16 activations: the tensor-core kernel
    if (a.dtype == CN_BF16) return cn_gemv_m1_launch(a, stream, who);
    if (a.line_bases) CN_FAIL(CN_ERR_SHAPE, "%s: line output takes bf16 activations", who);
    const bool gu = a.w1 != nullptr || a.tab1 != nullptr || a.fused_up_rows > 0;
    const int bpr = k / 64;
    const int tx = bpr % 16 == 0 ? 16 : (bpr % 8 == 0 ? 8 : 4);
    const int mp = m == 1 ? 1 : (m == 2 ? 2 : (m <= 4 ? 4 : 8));
    // f32 activations keep exact f32 arithmetic unless the caller allows rounding them to f16 at staging
    const int mode = (a.dtype == CN_BF16 || a.x_f16_ok) ? 1 : 0;
    const int G = NW * (32 / tx);
    int rt = 4;
    const long long slots = (long long)rows * (gu ? 2 : 1) * (routed ? a.combos : 1);
    if (slots / (G * 4) < 2 * 148) rt = 2;
    const int ROWS = G * rt;
    const int per_cta = gu ? ROWS / 2 : ROWS;
    const int grid = (rows + per_cta - 1) / per_cta;
    const int xb = (mode == 1 && a.dtype == CN_BF16) ? XB_SWZ : (mode == 1 ? XB_F16 : XB_F32);
    const size_t stage_bytes = (size_t)ROWS * tx * 36;
    const size_t xbytes = (size_t)mp * bpr * xb + (size_t)((mp * bpr + 3) & ~3) * 4;
    const int nchunks = bpr / tx;
    // ring depth: enough bytes in flight per SM to cover the HBM latency (about 96 KB), shared between
    // the CTAs that will be resident together (at most four, fewer when the grid is small)
    const long long total_ctas = (long long)grid * (routed ? a.combos : 1);
    int resident = (int)((total_ctas + 147) / 148);
    resident = resident < 1 ? 1 : (resident > 4 ? 4 : resident);
    long long want = (96 * 1024) / resident;                                         // in-flight bytes per CTA
    long long cap = (208 * 1024) / resident - (long long)HDR_BYTES - (long long)xbytes;  // what fits beside the activations
    if (want > cap) want = cap;
    int stages = (int)((want + (long long)stage_bytes - 1) / (long long)stage_bytes);
    stages = stages < 2 ? 2 : (stages > MAX_STAGES ? MAX_STAGES : stages);
    if (stages > nchunks) stages = nchunks < 1 ? 1 : nchunks;
    const size_t smem = HDR_BYTES + xbytes + stages * stage_bytes;
    if (smem > 200 * 1024) {
        // the staged activations of all m rows do not fit one CTA: two calls over half the rows each
        // (each row's arithmetic is the same whatever the split, so results do not change)
        if (m == 1) CN_FAIL(CN_ERR_LIMIT, "%s: k = %d needs %zu B of shared memory per block", who, k, smem);
        const int m0 = m / 2;
        const size_t es = a.dtype == CN_BF16 ? 2 : 4, eso = (a.dtype == CN_BF16 && !a.out_f32) ? 2 : 4;
        GemvCall lo = a, hi = a;
        lo.m = m0;
        hi.m = m - m0;
        hi.x = (const char*)a.x + (size_t)m0 * k * es;
        hi.y = (char*)a.y + (size_t)m0 * a.ldy * eso;
        int rc = cn_gemv_launch(lo, stream, who);
        return rc ? rc : cn_gemv_launch(hi, stream, who);
    }
    GemvParams p;
    p.w0 = (const uint8_t*)a.w0, p.w1 = (const uint8_t*)a.w1, p.gs0 = a.gs0, p.gs1 = a.gs1 ? a.gs1 : a.gs0, p.x = a.x, p.y = a.y;
    p.rows = rows, p.k = k, p.m = m, p.ldy = a.ldy, p.limit = a.limit, p.tx = tx, p.stages = stages, p.out_f32 = a.out_f32;
    p.ids = a.ids, p.order = a.order, p.tab0 = a.tab0, p.tab1 = a.tab1, p.fused_up_rows = a.fused_up_rows, p.x_div = a.x_div;
    p.experts = a.experts, p.yptrs = a.yptrs;
    const int gy = routed ? a.combos : 1;
    if (a.dtype == CN_BF16) return mode == 1 ? launch_m<1, 1>(p, mp, rt, grid, gy, smem, stream) : launch_m<1, 0>(p, mp, rt, grid, gy, smem, stream);
    return mode == 1 ? launch_m<0, 1>(p, mp, rt, grid, gy, smem, stream) : launch_m<0, 0>(p, mp, rt, grid, gy, smem, stream);
}

extern "C" int cn_nvfp4_gemv(const void* w, const float* gs, const void* x, void* y, int rows, int k, int m, int ldy, int dtype,
                             cn_stream_t stream) {
    GemvCall a = {};
    a.w0 = w, a.gs0 = gs, a.x = x, a.y = y, a.rows = rows, a.k = k, a.m = m, a.ldy = ldy, a.dtype = dtype;
    return cn_gemv_launch(a, (cudaStream_t)stream, "cn_nvfp4_gemv");
}

extern "C" int cn_nvfp4_gemv_gu(const void* wg, const void* wu, const float* gs_g, const float* gs_u, const void* x, void* h, int inter,
                                int k, int m, int ldh, float limit, int dtype, cn_stream_t stream) {
    if (!wu) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_gemv_gu: the up matrix is null");
    GemvCall a = {};
    a.w0 = wg, a.w1 = wu, a.gs0 = gs_g, a.gs1 = gs_u, a.x = x, a.y = h, a.rows = inter, a.k = k, a.m = m, a.ldy = ldh, a.limit = limit,
    a.dtype = dtype;
    return cn_gemv_launch(a, (cudaStream_t)stream, "cn_nvfp4_gemv_gu");
}

extern "C" int cn_nvfp4_gemv_lines(const void* w, const float* gs, const void* x, void* y, int rows, int k, const unsigned long long* line_bases,
                                   int world, int row0, size_t line_stride, const unsigned int* epoch, int tag, int buf, int flip, cn_stream_t stream) {
    if (!line_bases || !epoch) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_gemv_lines: null line buffers or step counter");
    GemvCall a = {};
    a.w0 = w, a.gs0 = gs, a.x = x, a.y = y, a.rows = rows, a.k = k, a.m = 1, a.ldy = rows, a.dtype = CN_BF16;
    a.line_bases = line_bases, a.line_world = world, a.line_row0 = row0, a.line_stride = line_stride, a.line_epoch = epoch;
    a.line_tag = tag, a.line_buf = buf, a.line_flip = flip;
    return cn_gemv_launch(a, (cudaStream_t)stream, "cn_nvfp4_gemv_lines");
}

extern "C" int cn_nvfp4_gemv_gu_lines(const void* wg, const void* wu, const float* gs_g, const float* gs_u, const void* x, void* h, int inter, int k,
                                      float limit, const unsigned long long* line_bases, int world, int row0, size_t line_stride,
                                      const unsigned int* epoch, int tag, int buf, int flip, cn_stream_t stream) {
    if (!wu) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_gemv_gu_lines: the up matrix is null");
    if (!line_bases || !epoch) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_gemv_gu_lines: null line buffers or step counter");
    GemvCall a = {};
    a.w0 = wg, a.w1 = wu, a.gs0 = gs_g, a.gs1 = gs_u, a.x = x, a.y = h, a.rows = inter, a.k = k, a.m = 1, a.ldy = inter, a.limit = limit,
    a.dtype = CN_BF16;
    a.line_bases = line_bases, a.line_world = world, a.line_row0 = row0, a.line_stride = line_stride, a.line_epoch = epoch;
    a.line_tag = tag, a.line_buf = buf, a.line_flip = flip;
    return cn_gemv_launch(a, (cudaStream_t)stream, "cn_nvfp4_gemv_gu_lines");
}

extern "C" int cn_nvfp4_dequant(const void* w, const float* gs, float* out, int rows, int k, int rule, cn_stream_t stream) {
    if (rows <= 0 || k <= 0 || k % 64 != 0) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_dequant: %d columns are not whole 64-value NVFP4 blocks", k);
    const long long nwords = (long long)rows * (k / 64) * 8;
    const int threads = 256;
    const long long blocks = (nwords + threads - 1) / threads;
    nvfp4_dequant_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>((const uint8_t*)w, gs, out, nwords, rule);
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}
