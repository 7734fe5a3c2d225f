// NVFP4 GEMV for bf16 activations, M = 1..8, with the warp-level tensor-core instruction as the
// multiply-accumulate engine. Same operator, layout and pipeline as nvfp4_gemv.cu (bulk-copy weight
// ring, activations staged once per CTA as f16 with a power-of-two scale per 64-value block); what
// changes is the inner loop, which on the CUDA-core path spent 3.2 issue slots per weight (ncu) and
// ran out of issue slots at 37 % of the HBM rate.
//
// mma.sync.m16n8k16 (f16 x f16 -> f32) consumes the f16x2 registers that cvt.rn.f16x2.e2m1x2 makes,
// as they are: A = 16 weight rows x one 16-value sub-block (every E2M1 value is exact in f16), B =
// the matching 16 activations. The k order inside an MMA is free as long as A and B agree, so slot
// pairs (2t, 2t+1) / (2t+8, 2t+9) of thread t are bound to code bytes 2t and 2t+1 of the sub-block:
// one 16-bit shared-memory load per row and sub-block feeds two cvt and nothing else.
//   M = 1 ("column" form): the eight columns of B hold eight consecutive sub-blocks (column j = the
//     activations of sub-block j, zero elsewhere), eight MMAs accumulate into one C tile, and the
//     UE4M3 scale * tensor scale * inverse activation scale is applied once per eight sub-blocks.
//   M = 2..8 ("token" form): the columns are the activation rows and the scale is applied per MMA.
// Products are exact, accumulation is the tensor core's f32; each output element depends only on
// its own column, so row m of an M-row call equals a one-row call in the token form bit for bit.
#include "common.cuh"
#include "nvfp4_gemv.cuh"

namespace {

constexpr int NW = 4;  // consumer warps: the K range of a stage split four ways
constexpr int NTHREADS = (NW + 1) * 32;
constexpr int MAX_STAGES = 8;
constexpr int XB = 128;        // one 64-value block of f16 activations, 16-byte chunks XOR-swizzled
constexpr int HDR = 256 + 2048;
constexpr int ROWS = 16;  // row slots per CTA: one MMA row tile
#ifndef MINB
#define MINB 3
#endif

__device__ __forceinline__ void mma16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// two code bytes (a 16-bit unit of a sub-block) -> two f16x2. Each byte is loaded on its own so that it sits
// in the low byte of its register, where cvt takes it without a shift.
__device__ __forceinline__ void cvt_unit(const uint8_t* p2, uint32_t& lo, uint32_t& hi) {
    lo = e2m1x2_to_f16x2(p2[0]);
    hi = e2m1x2_to_f16x2(p2[1]);
}

// COLS: true = M == 1 column form, false = token form (MP activation rows, <= 8)
// TX: 36-byte blocks per row and stage (16 or 8), a template parameter so that every shared-memory offset
// of the unrolled inner loop is an immediate
template <bool COLS, int TX>
__global__ void __launch_bounds__(NTHREADS, MINB) nvfp4_gemv_mma_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int piece = TX * 36;       // payload bytes of one row's share of a stage
    constexpr int pstride = piece + 16;  // padded so that 8 rows x 2 words hit 16 banks
    const int bpr = p.k >> 6;
    const size_t row_bytes = (size_t)bpr * 36;
    const int nchunks = bpr / TX;
    const int S = p.stages;
    const int MP = COLS ? 1 : p.m;
    const uint8_t* w0 = p.w0;
    const uint8_t* w1 = p.w1;
    const char* xbase = (const char*)p.x;
    char* ybase = (char*)p.y;
    if (p.ids) {
        const int c = p.order ? p.order[blockIdx.y] : (int)blockIdx.y;
        const int e = p.ids[c];
        if (e < 0) return;  // uniform over the CTA, before any barrier
        w0 = (const uint8_t*)p.tab0[e];
        if (!w0) return;
        w1 = p.tab1 ? (const uint8_t*)p.tab1[e] : (p.fused_up_rows > 0 ? w0 + (size_t)p.fused_up_rows * row_bytes : nullptr);
        xbase += (size_t)(c / p.x_div) * p.k * 2;
        ybase += (size_t)c * p.ldy * (p.out_f32 ? 4 : 2);
    }
    const bool gu = w1 != nullptr;

    uint64_t* full = (uint64_t*)smem;
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* xbar = empty + MAX_STAGES;
    float* lut = (float*)(smem + 256);                             // [2][256] ue4m3 * gs
    uint8_t* xs0 = smem + HDR;                                     // [MP][bpr][128] f16 activations
    float* xinv0 = (float*)(xs0 + (size_t)MP * bpr * XB);          // [MP][bpr]
    uint8_t* stage0 = (uint8_t*)(xinv0 + ((MP * bpr + 3) & ~3));
    const int stage_bytes = ROWS * pstride;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // plain: 16 consecutive rows per CTA; gate/up: 8 indices, row slots 0-7 gate, 8-15 up
    const int per_cta = gu ? ROWS / 2 : ROWS;
    const int row0 = blockIdx.x * per_cta;

    if (tid == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], NW);
        }
        mbar_init(xbar, 1);
        mbar_fence_init();
    }
    {
        const float g0 = p.gs0[0], g1 = gu ? p.gs1[0] : g0;
        for (int b = tid; b < 256; b += NTHREADS) {
            const float u = ue4m3_f32((uint32_t)b, true);
            lut[b] = u * g0;
            lut[256 + b] = u * g1;
        }
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == NW) {
        // ------------------------------------------------------------ weight producer warp
        const uint64_t pol = l2_policy_evict_first();
        const uint8_t* src[1];
        uint32_t total = 0;
        {
            const int row = gu ? row0 + (lane & 7) : row0 + lane;
            const uint8_t* base = (gu && (lane >> 3)) ? w1 : w0;
            src[0] = (lane < ROWS && row < p.rows) ? base + (size_t)row * row_bytes : nullptr;
            total += src[0] ? piece : 0;
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
            if (src[0]) bulk_g2s_stream(st + (size_t)lane * pstride, src[0] + (size_t)c * piece, piece, &full[s], pol);
        }
        return;
    }

    // ---------------------------------------------------------------- consumer warps: activations first
    if (tid == 0) {
        pdl_wait();  // activations may come from the previous kernel of the stream
        mbar_expect_tx(xbar, (uint32_t)MP * (uint32_t)p.k * 2u);
        mbar_arrive(xbar);
        for (int m = 0; m < MP; m++) bulk_g2s(xs0 + (size_t)m * bpr * XB, xbase + (size_t)m * p.k * 2, (uint32_t)p.k * 2u, xbar);
    }
    if (!mbar_wait(xbar, 0)) {
        cn_dev_fail(CN_DEV_WAIT_FULL);
        return;
    }
    // in place bf16 -> f16 * 2^e per 64-value block, chunk i of block b stored at chunk i ^ (b & 7)
    for (int b = tid; b < MP * bpr; b += NW * 32) {
        uint4* blkp = (uint4*)(xs0 + (size_t)b * XB);
        const int sw = (b % bpr) & 7;
        uint4 raw[8];  // raw[i] = chunk i ^ sw, so that eight threads on eight blocks hit eight bank groups
#pragma unroll
        for (int i = 0; i < 8; i++) raw[i] = blkp[i];
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

    // ---------------------------------------------------------------- main loop
    // The CTA owns 16 rows; the K range of every stage is split over the four consumer warps (warp w
    // takes blocks w * TX/4 .. of the stage), partial sums meet in shared memory at the end.
    const int g = lane >> 2, t = lane & 3;
    const float* lut_b = lut + (gu ? 256 : 0);  // gate/up: rows 8-15 are up rows
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};    // COLS: [0] row g, [1] row g+8; else row g tok 2t, 2t+1, row g+8 tok 2t, 2t+1
    constexpr int nb = TX / NW;                  // blocks per warp and stage: 4 or 2
    uint32_t colmask[8];                         // all ones in the MMA whose column this lane's activations fill
#pragma unroll
    for (int j = 0; j < 8; j++) colmask[j] = g == j ? 0xffffffffu : 0u;

    for (int c = 0; c < nchunks; c++) {
        const int s = c % S;
        if (!mbar_wait(&full[s], (c / S) & 1)) {
            cn_dev_fail(CN_DEV_WAIT_FULL);
            break;  // every consumer warp waits on the same phase and gives up alike; the barriers below still meet
        }
        const uint8_t* st = stage0 + (size_t)s * stage_bytes;
        const uint8_t* pa = st + g * pstride + warp * (nb * 36) + 2 * t;  // this warp's blocks, this thread's 16-bit unit
        const uint8_t* pb = pa + 8 * pstride;
        if (COLS) {
            // groups of two blocks = eight sub-blocks = the eight columns of one C tile; two groups in
            // flight when the warp has four blocks, so that the MMA chains overlap
#pragma unroll
            for (int q0 = 0; q0 < nb / 2; q0 += 2) {
                constexpr int ng = nb / 2 >= 2 ? 2 : 1;
                float cc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
                uint2 xv[2];
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    if (u < ng) {
                        // this thread's column: sub-block g of the group, four activations starting at 4t
                        const int gbx = c * TX + warp * nb + 2 * (q0 + u) + (g >> 2);
                        xv[u] = *(const uint2*)(xs0 + (size_t)gbx * XB + ((((g & 3) * 2 + (t >> 1)) ^ (gbx & 7)) << 4) + ((t & 1) << 3));
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; j++) {
#pragma unroll
                    for (int u = 0; u < 2; u++) {
                        if (u < ng) {
                            const int off = (2 * (q0 + u) + (j >> 2)) * 36 + 4 + (j & 3) * 8;
                            uint32_t a0, a1, a2, a3;
                            cvt_unit(pa + off, a0, a2);
                            cvt_unit(pb + off, a1, a3);
                            mma16816(cc[u], a0, a1, a2, a3, xv[u].x & colmask[j], xv[u].y & colmask[j]);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    if (u < ng) {
                        // columns 2t, 2t + 1 of C are sub-blocks 2t, 2t + 1 of the group: block + (t >> 1), scale bytes 2(t & 1), +1
                        const int bs = 2 * (q0 + u) + (t >> 1);  // relative to the warp's first block
                        const float xi = xinv0[c * TX + warp * nb + bs];
                        const int so = bs * 36 + 2 * (t & 1) - 2 * t;
                        const uint32_t sa = *(const uint16_t*)(pa + so), sb = *(const uint16_t*)(pb + so);
                        acc[0] = fmaf(cc[u][0], lut[sa & 0xFF] * xi, acc[0]);
                        acc[0] = fmaf(cc[u][1], lut[sa >> 8] * xi, acc[0]);
                        acc[1] = fmaf(cc[u][2], lut_b[sb & 0xFF] * xi, acc[1]);
                        acc[1] = fmaf(cc[u][3], lut_b[sb >> 8] * xi, acc[1]);
                    }
                }
            }
        } else {
#pragma unroll
            for (int bi = 0; bi < nb; bi++) {
                const int gbx = c * TX + warp * nb + bi;
                const uint32_t swa = *(const uint32_t*)(pa + bi * 36 - 2 * t), swb = *(const uint32_t*)(pb + bi * 36 - 2 * t);
                const float xi0 = 2 * t < MP ? xinv0[(2 * t) * bpr + gbx] : 0.0f, xi1 = 2 * t + 1 < MP ? xinv0[(2 * t + 1) * bpr + gbx] : 0.0f;
                const uint8_t* xrow = xs0 + ((size_t)(g < MP ? g : 0) * bpr + gbx) * XB;
                float cc[4][4];
#pragma unroll
                for (int sbi = 0; sbi < 4; sbi++) {
                    uint2 xv = *(const uint2*)(xrow + (((sbi * 2 + (t >> 1)) ^ (gbx & 7)) << 4) + ((t & 1) << 3));
                    if (g >= MP) xv = make_uint2(0u, 0u);
                    const int off = bi * 36 + 4 + sbi * 8;
                    uint32_t a0, a1, a2, a3;
                    cvt_unit(pa + off, a0, a2);
                    cvt_unit(pb + off, a1, a3);
                    cc[sbi][0] = cc[sbi][1] = cc[sbi][2] = cc[sbi][3] = 0.0f;
                    mma16816(cc[sbi], a0, a1, a2, a3, xv.x, xv.y);
                }
#pragma unroll
                for (int sbi = 0; sbi < 4; sbi++) {
                    const float sa = lut[(swa >> (8 * sbi)) & 0xFF], sb = lut_b[(swb >> (8 * sbi)) & 0xFF];
                    acc[0] = fmaf(cc[sbi][0], sa * xi0, acc[0]);
                    acc[1] = fmaf(cc[sbi][1], sa * xi1, acc[1]);
                    acc[2] = fmaf(cc[sbi][2], sb * xi0, acc[2]);
                    acc[3] = fmaf(cc[sbi][3], sb * xi1, acc[3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }

    // ---------------------------------------------------------------- K-split reduction and epilogue
    if (COLS) {
        // the four lanes of a row pair hold two sub-block columns each: xor-shuffle tree, fixed order
        acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 1);
        acc[1] += __shfl_xor_sync(0xffffffffu, acc[1], 1);
        acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 2);
        acc[1] += __shfl_xor_sync(0xffffffffu, acc[1], 2);
    }
    float* red = (float*)stage0;  // the ring is drained: every stage was consumed before this point
    asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
#pragma unroll
    for (int i = 0; i < 4; i++) red[(warp * 32 + lane) * 4 + i] = acc[i];
    asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
    if (warp != 0) return;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float v = red[lane * 4 + i];
        for (int w = 1; w < NW; w++) v += red[(w * 32 + lane) * 4 + i];  // warps in order: deterministic
        acc[i] = v;
    }
    auto store = [&](int m, int row, float v) {
        if (p.out_f32)
            ((float*)ybase)[(size_t)m * p.ldy + row] = v;
        else
            ((__nv_bfloat16*)ybase)[(size_t)m * p.ldy + row] = __float2bfloat16_rn(v);
    };
    const int ra = row0 + g, rb = row0 + g + 8;  // plain rows; gate/up: index row0 + g, gate in a, up in b
    if (COLS) {
        if (t == 0) {
            if (gu) {
                if (ra < p.rows) store(0, ra, act_gu(acc[0], acc[1], p.limit));
            } else {
                if (ra < p.rows) store(0, ra, acc[0]);
                if (rb < p.rows) store(0, rb, acc[1]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int m = 2 * t + i;
            if (m < MP) {
                if (gu) {
                    if (ra < p.rows) store(m, ra, act_gu(acc[i], acc[2 + i], p.limit));
                } else {
                    if (ra < p.rows) store(m, ra, acc[i]);
                    if (rb < p.rows) store(m, rb, acc[2 + i]);
                }
            }
        }
    }
}

int g_mma_stages = 0;

}  // namespace

void cn_gemv_mma_set_stages(int s) { g_mma_stages = s; }

int cn_gemv_mma_launch(const GemvCall& a, cudaStream_t stream, const char* who) {
    const int rows = a.rows, k = a.k, m = a.m;
    const bool routed = a.ids != nullptr;
    const bool gu = a.w1 != nullptr || a.tab1 != nullptr || a.fused_up_rows > 0;
    const int bpr = k / 64;
    const int tx = bpr % 16 == 0 ? 16 : 8;  // the caller sends k % 512 != 0 to the CUDA-core kernel
    const int mp = m;
    const int pstride = tx * 36 + 16;
    const size_t stage_bytes = (size_t)ROWS * pstride;
    const size_t xbytes = (size_t)mp * bpr * XB + (size_t)((mp * bpr + 3) & ~3) * 4;
    const int nchunks = bpr / tx;
    long long room = 48 * 1024 - (long long)HDR - (long long)xbytes;
    int stages = (int)(room / (long long)stage_bytes);
    if (g_mma_stages > 0) stages = g_mma_stages;
    stages = stages < 2 ? 2 : (stages > MAX_STAGES ? MAX_STAGES : stages);
    if (stages > nchunks) stages = nchunks < 1 ? 1 : nchunks;
    const size_t smem = HDR + xbytes + stages * stage_bytes;
    if (smem > 200 * 1024) {
        if (m == 1) CN_FAIL(CN_ERR_LIMIT, "%s: k = %d needs %zu B of shared memory per block", who, k, smem);
        GemvCall lo = a, hi = a;
        const int m0 = m / 2;
        lo.m = m0, hi.m = m - m0;
        hi.x = (const char*)a.x + (size_t)m0 * k * 2;
        hi.y = (char*)a.y + (size_t)m0 * a.ldy * (a.out_f32 ? 4 : 2);
        int rc = cn_gemv_mma_launch(lo, stream, who);
        return rc ? rc : cn_gemv_mma_launch(hi, stream, who);
    }
    GemvParams p;
    p.w0 = (const uint8_t*)a.w0, p.w1 = (const uint8_t*)a.w1, p.gs0 = a.gs0, p.gs1 = a.gs1 ? a.gs1 : a.gs0, p.x = a.x, p.y = a.y;
    p.rows = rows, p.k = k, p.m = m, p.ldy = a.ldy, p.limit = a.limit, p.tx = tx, p.stages = stages, p.out_f32 = a.out_f32;
    p.ids = a.ids, p.order = a.order, p.tab0 = a.tab0, p.tab1 = a.tab1, p.fused_up_rows = a.fused_up_rows, p.x_div = a.x_div;
    const int per_cta = gu ? ROWS / 2 : ROWS;
    static bool attr = false;
    if (!attr) {
        CN_CUDA(cudaFuncSetAttribute(nvfp4_gemv_mma_kernel<true, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        CN_CUDA(cudaFuncSetAttribute(nvfp4_gemv_mma_kernel<false, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        CN_CUDA(cudaFuncSetAttribute(nvfp4_gemv_mma_kernel<true, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        CN_CUDA(cudaFuncSetAttribute(nvfp4_gemv_mma_kernel<false, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((rows + per_cta - 1) / per_cta), (unsigned)(routed ? a.combos : 1));
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (m == 1 && tx == 16)
        CN_CUDA(cudaLaunchKernelEx(&cfg, nvfp4_gemv_mma_kernel<true, 16>, p));
    else if (m == 1)
        CN_CUDA(cudaLaunchKernelEx(&cfg, nvfp4_gemv_mma_kernel<true, 8>, p));
    else if (tx == 16)
        CN_CUDA(cudaLaunchKernelEx(&cfg, nvfp4_gemv_mma_kernel<false, 16>, p));
    else
        CN_CUDA(cudaLaunchKernelEx(&cfg, nvfp4_gemv_mma_kernel<false, 8>, p));
    return CN_OK;
}
