// NVFP4 GEMM for M >= 9 activation rows (prefill / batched verify): Y[t][n] = gs * sum_k X[t][k] * W[n][k],
// on the fifth-generation tensor cores: tcgen05.mma (kind::f16) with the accumulator in tensor memory.
//
// Supersedes the reference's prompt GEMMs gemm_fp4_dense (engine/src/kernels.rs:533) and
// glm5_gemm_fp4_tc (engine/src/kernels_glm5_moe.cu:349: "NVFP4 decoded losslessly to f16 in shared
// memory, x rounded to f16, f32 accumulate"), whose arithmetic this kernel keeps: the weights are
// consumed in the container layout and widened in flight, nothing is re-quantised.
//
// Arithmetic. A = w * s as f16: an E2M1 code times a UE4M3 scale has at most 5 significant bits and
// lies in [2^-10, 2688], so the product is exact in f16. B = x * 2^k as f16 with one power of two per
// activation row (row amax brought to [2^13, 2^14)): exact for bf16 input down to 2^-27 of the row
// maximum. Products are exact in the tensor core, accumulation is f32 in tensor memory, the epilogue
// multiplies by gs * 2^-k once.
//
// One CTA = 128 weight rows x TN activation rows (128, or 256 when more than 128 rows are given), K walked
// 64 at a time through a 3- or 4-stage ring:
//   warps 0-7   A producers: thread (r, h) owns half of weight row r's 36-byte block per step (prefetched three
//               steps ahead), cvt.rn.f16x2.e2m1x2 + one HMUL2 per pair, four 16-byte stores into the canonical
//               K-major 128-byte-swizzle tile (row r at r * 128, chunk c at c ^ (r & 7));
//   warps 8-11  B producers: cp.async of the activation rows' 128 bytes per step into the same tile form, the
//               stage's mbarrier counting the copies as they land, so the threads run ahead of the data;
//   warp 12     one lane issues four tcgen05.mma (M 128, N TN, K 16) per stage and commits the stage's "empty"
//               mbarrier; after the last step it commits the accumulator barrier;
//   warps 0-7   then read the accumulator (tcgen05.ld 32x32b: lane = weight row, 32 activation rows per load),
//               scale, and store y[t][n] (for one t the 32 lanes write 32 consecutive n).
// Every wait is bounded; tensor memory (TN columns) is allocated by warp 12 and freed by it after the CTA has
// met again, whatever happened in between.
#include "common.cuh"

namespace {

constexpr int TM = 128, TK = 64;
constexpr int A_BYTES = TM * 128;
constexpr int A_WARPS = 8, B_WARPS = 4;  // producers; one more warp issues the MMAs
constexpr int GEMM_THREADS = (A_WARPS + B_WARPS + 1) * 32;
// TN activation rows per CTA: 128 (3 stages, two CTAs per SM) or 256 (4 stages, one CTA per SM, half the weight
// decoding per MMA)
__host__ __device__ constexpr int stages_of(int tn) { return tn == 256 ? 4 : 3; }
__host__ __device__ constexpr int smem_of(int tn) { return 2048 + stages_of(tn) * (A_BYTES + tn * 128) + 1024; }  // header (barriers, scale table) + ring + alignment slack
// instruction descriptor, kind::f16: D f32 (bit 4), A and B f16 K-major (0), N >> 3 at bit 17, M >> 4 at bit 24
__host__ __device__ constexpr uint32_t idesc_of(int tn) { return (1u << 4) | ((uint32_t)(tn >> 3) << 17) | ((uint32_t)(TM >> 4) << 24); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// this thread's arrival on the barrier, made when its earlier cp.async copies have landed
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: start address >> 4, leading byte
// offset 1 (unused by swizzled K-major tiles), stride byte offset = 8 rows * 128 B, descriptor version 1, layout 2
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t v[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,"
        "%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
          "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
          "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
          "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// activation rows -> f16 * 2^k (k per row), and the rows' 2^-k. grid (M), block 256.
template <int XT>
__global__ void gemm_prep_x_kernel(const void* __restrict__ x, uint16_t* __restrict__ xh, float* __restrict__ rs, int k) {
    __shared__ float amax_w[8];
    const size_t row = blockIdx.x;
    auto at = [&](int i) -> float {
        return XT == 1 ? __bfloat162float(((const __nv_bfloat16*)x)[row * k + i]) : ((const float*)x)[row * k + i];
    };
    float amax = 0.0f;
    for (int i = threadIdx.x; i < k; i += blockDim.x) amax = fmaxf(amax, fabsf(at(i)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) amax_w[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = 0.0f;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) amax = fmaxf(amax, amax_w[w]);
    // amax * mul in [2^13, 2^14): two binades under the largest f16; zero, NaN and infinite rows are left unscaled
    uint32_t e = (__float_as_uint(amax) >> 23) & 0xFF;
    float mul = 1.0f, inv = 1.0f;
    if (amax > 0.0f && e < 255 && e > 14 && e < 240) {
        mul = __uint_as_float((127u + 13u + 127u - e) << 23);
        inv = __uint_as_float((e - 13u) << 23);
    }
    for (int i = threadIdx.x; i < k; i += blockDim.x) xh[row * k + i] = __half_as_ushort(__float2half_rn(at(i) * mul));
    if (threadIdx.x == 0) rs[row] = inv;
}

struct GemmParams {
    const uint8_t* w;
    const float* gs;
    const uint16_t* xh;
    const float* rs;
    void* y;
    int rows, k, m, ldy, out_bf16;
    // K shared between `ksplits` CTAs of a tile (blockIdx.y, when m <= 128 and the row tiles alone do not fill the
    // machine): each writes its raw f32 sums to part[split][m][rows], a second kernel adds them in split order
    int ksplits;
    float* part;
};

template <int TN>
__global__ void __launch_bounds__(GEMM_THREADS, TN == 256 ? 1 : 2) nvfp4_gemm_tc5_kernel(const GemmParams p) {
    constexpr int STAGES = stages_of(TN), B_BYTES = TN * 128;
    constexpr uint32_t IDESC = idesc_of(TN);
    extern __shared__ uint8_t smem_raw[];
    // header in the first 1024 bytes as the runtime gives them; the ring starts at the next 1024-byte boundary
    uint64_t* full = (uint64_t*)smem_raw;
    uint64_t* empty = full + STAGES;
    uint64_t* accbar = empty + STAGES;
    uint32_t* tmem_slot = (uint32_t*)(accbar + 1);
    volatile int* failed = (volatile int*)(tmem_slot + 1);
    uint32_t* slut = (uint32_t*)(smem_raw + 1024);  // [256] UE4M3 scale byte -> f16x2 (both halves), 0x7F read as 0x7E
    const uint32_t ring_addr = (smem_u32(smem_raw) + 2048u + 1023u) & ~1023u;
    uint8_t* ring = smem_raw + (ring_addr - smem_u32(smem_raw));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int KSP = p.ksplits, ksi = KSP > 1 ? (int)blockIdx.y : 0;
    const int row0 = blockIdx.x * TM, tok0 = KSP > 1 ? 0 : (int)blockIdx.y * TN;
    const int bpr_all = p.k >> 6;
    const int kbeg = (int)((long long)bpr_all * ksi / KSP), bpr = (int)((long long)bpr_all * (ksi + 1) / KSP) - kbeg;  // this CTA's blocks
    const size_t row_bytes = (size_t)bpr_all * 36;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], (A_WARPS + B_WARPS) * 32);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accbar, 1);
        mbar_fence_init();
        *failed = 0;
    }
    if (tid < 256) {
        const __half2 h2 = __half2half2(__float2half_rn(ue4m3_f32((uint32_t)tid, true)));
        slut[tid] = *(const uint32_t*)&h2;
    }
    if (warp == A_WARPS + B_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)TN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp < A_WARPS) {
        // ------------------------------------------------------------ A producers: unit (row, chunk c) = one code word = eight
        // weights -> one 16-byte chunk of the tile. Eight consecutive lanes take the eight words of one row's block, so a
        // warp's load touches four rows' 36 contiguous bytes, and its store fills four whole 128-byte tile rows.
        constexpr int UNITS = TM * 8 / (A_WARPS * 32);  // 4 per thread and stage
        constexpr int PF = 3;                           // stages of container words in flight per thread
        const int c = tid & 7;
        const uint32_t* src[UNITS];
        bool live[UNITS];
#pragma unroll
        for (int u = 0; u < UNITS; u++) {
            const int r = (u * (A_WARPS * 32) + tid) >> 3;
            live[u] = row0 + r < p.rows;
            src[u] = (const uint32_t*)(p.w + (size_t)(live[u] ? row0 + r : 0) * row_bytes + (size_t)kbeg * 36);
        }
        uint32_t code[PF][UNITS], scl[PF][UNITS];
        auto fetch = [&](int d, int kb) {
#pragma unroll
            for (int u = 0; u < UNITS; u++) {
                scl[d][u] = live[u] ? __ldg(src[u] + (size_t)kb * 9) : 0u;
                code[d][u] = live[u] ? __ldg(src[u] + (size_t)kb * 9 + 1 + c) : 0u;
            }
        };
#pragma unroll
        for (int d = 0; d < PF; d++) {
            if (d < bpr) {
                fetch(d, d);
            } else {
#pragma unroll
                for (int u = 0; u < UNITS; u++) scl[d][u] = code[d][u] = 0u;
            }
        }
        bool ok = true;
        for (int kb0 = 0; kb0 < bpr && ok; kb0 += PF) {
#pragma unroll
            for (int d = 0; d < PF; d++) {
                const int kb = kb0 + d;
                if (kb >= bpr || !ok) break;
                const int s = kb % STAGES;
                uint32_t cw[UNITS], sw[UNITS];
#pragma unroll
                for (int u = 0; u < UNITS; u++) cw[u] = code[d][u], sw[u] = scl[d][u];
                if (kb + PF < bpr) fetch(d, kb + PF);
                if (kb >= STAGES && !mbar_wait(&empty[s], ((kb / STAGES) - 1) & 1)) {
                    cn_dev_fail(CN_DEV_WAIT_EMPTY);
                    *failed = 1;
                    ok = false;
                    break;
                }
                uint8_t* tile = ring + (size_t)s * (A_BYTES + B_BYTES);
#pragma unroll
                for (int u = 0; u < UNITS; u++) {
                    const int r = (u * (A_WARPS * 32) + tid) >> 3;
                    // the chunk's sub-block is c >> 1: its scale in both halves of an f16x2
                    const uint32_t sbits = slut[(sw[u] >> (8 * (c >> 1))) & 0xFFu];
                    const __half2 s2 = *(const __half2*)&sbits;
                    uint32_t f[4];
                    e2m1x8_to_f16x2(cw[u], f);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const __half2 v = __hmul2(*(const __half2*)&f[q], s2);
                        f[q] = *(const uint32_t*)&v;
                    }
                    *(uint4*)(tile + (size_t)r * 128 + ((c ^ (r & 7)) << 4)) = make_uint4(f[0], f[1], f[2], f[3]);
                }
                fence_proxy_async();
                mbar_arrive(&full[s]);
            }
        }
    } else if (warp < A_WARPS + B_WARPS) {
        // ------------------------------------------------------------ B producers: activation rows j, j + 128 .. of the tile,
        // copied asynchronously (cp.async) so that this thread runs as far ahead as the ring has free stages
        const int j = tid - A_WARPS * 32;
        bool ok = true;
        for (int kb = 0; kb < bpr && ok; kb++) {
            const int s = kb % STAGES;
            if (kb >= STAGES && !mbar_wait(&empty[s], ((kb / STAGES) - 1) & 1)) {
                cn_dev_fail(CN_DEV_WAIT_EMPTY);
                *failed = 1;
                ok = false;
                break;
            }
            // eight consecutive lanes copy the eight 16-byte chunks of one activation row: whole 128-byte lines per request
#pragma unroll
            for (int it = 0; it < TN * 8 / (B_WARPS * 32); it++) {
                const int idx = it * (B_WARPS * 32) + j, jr = idx >> 3, c = idx & 7, tok = tok0 + jr;
                uint8_t* dst = ring + (size_t)s * (A_BYTES + B_BYTES) + A_BYTES + (size_t)jr * 128 + ((c ^ (jr & 7)) << 4);
                if (tok < p.m)
                    cp_async16(smem_u32(dst), (const uint4*)(p.xh + (size_t)tok * p.k) + (size_t)(kbeg + kb) * 8 + c);
                else
                    *(uint4*)dst = make_uint4(0u, 0u, 0u, 0u);
            }
            fence_proxy_async();       // the plain zero stores, if any
            cp_async_arrive(&full[s]);  // counts as this thread's arrival once its copies have landed
        }
    } else if (lane == 0) {
        // ------------------------------------------------------------ MMA issuer
        bool ok = true;
        for (int kb = 0; kb < bpr && ok; kb++) {
            const int s = kb % STAGES;
            if (!mbar_wait(&full[s], (kb / STAGES) & 1)) {
                cn_dev_fail(CN_DEV_WAIT_FULL);
                *failed = 1;
                ok = false;
                break;
            }
            fence_proxy_async();  // the producers' shared-memory writes (plain stores and cp.async), before the tensor core reads them
            tc_fence_after();
            const uint32_t a_addr = ring_addr + (uint32_t)s * (A_BYTES + B_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
            for (int kk = 0; kk < TK / 16; kk++)  // 16 f16 = 32 bytes further along K inside the swizzled row
                umma_f16(tmem, umma_desc(a_addr + 32u * kk), umma_desc(b_addr + 32u * kk), IDESC, (kb > 0 || kk > 0) ? 1u : 0u);
            umma_commit(&empty[s]);  // arrives when the MMAs above have read the stage
        }
        if (ok) umma_commit(accbar);
    }

    if (warp < A_WARPS) {
        // ------------------------------------------------------------ epilogue: lane = weight row (the warp's quarter of the
        // accumulator's 128 lanes is warp % 4), 32 activation rows per load; warps 4-7 take the upper half of the columns
        bool ok = !*failed;
        if (ok && !mbar_wait(accbar, 0)) {
            cn_dev_fail(CN_DEV_WAIT_FULL);
            ok = false;
        }
        if (ok) {
            tc_fence_after();
            const int q = warp & 3, half = warp >> 2;
            const int row = row0 + 32 * q + lane;
            const float gs = p.gs[0];
            for (int c0 = half * (TN / 2); c0 < (half + 1) * (TN / 2); c0 += 32) {
                if (tok0 + c0 >= p.m) break;  // uniform
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    const int tok = tok0 + c0 + i;
                    if (tok < p.m && row < p.rows) {
                        if (KSP > 1) {
                            p.part[((size_t)ksi * p.m + tok) * p.rows + row] = __uint_as_float(v[i]);
                            continue;
                        }
                        const float r = __uint_as_float(v[i]) * (gs * p.rs[tok]);
                        if (p.out_bf16)
                            ((__nv_bfloat16*)p.y)[(size_t)tok * p.ldy + row] = __float2bfloat16_rn(r);
                        else
                            ((float*)p.y)[(size_t)tok * p.ldy + row] = r;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == A_WARPS + B_WARPS) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TN) : "memory");
}

// y[t][n] = (sum over splits, in order, of part[s][t][n]) * gs * rs[t]
__global__ void gemm_splitk_reduce_kernel(const float* __restrict__ part, const float* __restrict__ gs, const float* __restrict__ rs,
                                          void* __restrict__ y, int rows, int m, int ldy, int ksplits, int out_bf16) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (n >= rows) return;
    float v = part[(size_t)t * rows + n];
    for (int s = 1; s < ksplits; s++) v += part[((size_t)s * m + t) * rows + n];
    v *= gs[0] * rs[t];
    if (out_bf16)
        ((__nv_bfloat16*)y)[(size_t)t * ldy + n] = __float2bfloat16_rn(v);
    else
        ((float*)y)[(size_t)t * ldy + n] = v;
}

constexpr int MAX_KSPLITS = 8;

// K splits for m <= 128: enough CTAs for two per SM, at least eight 64-wide steps each
int gemm_ksplits(int rows, int k, int m) {
    if (m > 128) return 1;
    const int tiles = (rows + TM - 1) / TM, bpr = k / 64;
    int ks = (2 * 148 + tiles - 1) / tiles;
    if (ks > MAX_KSPLITS) ks = MAX_KSPLITS;
    if (ks > bpr / 8) ks = bpr / 8;
    return ks < 1 ? 1 : ks;
}

}  // namespace

extern "C" size_t cn_nvfp4_gemm_workspace_bytes(int k, int m) {
    if (k <= 0 || m <= 0) return 0;
    // widened activations, row scales, and (m <= 128) room for the partial sums of up to 8 K splits of 2^15 rows
    const size_t part = m <= 128 ? (size_t)MAX_KSPLITS * m * 32768 * 4 : 0;
    return (size_t)m * k * 2 + (((size_t)m * 4 + 255) & ~(size_t)255) + 256 + part;
}

extern "C" int cn_nvfp4_gemm(const void* w, const float* gs, const void* x, void* y, int rows, int k, int m, int ldy, int dtype, void* workspace,
                             size_t workspace_bytes, cn_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (rows <= 0 || k <= 0 || k % 256 != 0) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_gemm: k = %d must be a positive multiple of 256", k);
    if (m < 1) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_gemm: m = %d", m);
    if (ldy < rows) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_gemm: ldy %d < rows %d", ldy, rows);
    if (dtype != CN_F32 && dtype != CN_BF16) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_gemm: dtype %d is neither CN_F32 nor CN_BF16", dtype);
    if (((uintptr_t)w & 15) || ((uintptr_t)x & 15) || ((uintptr_t)workspace & 255))
        CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_gemm: weights and activations must be 16-byte aligned, the workspace 256-byte aligned");
    if (!workspace || workspace_bytes < cn_nvfp4_gemm_workspace_bytes(k, m))
        CN_FAIL(CN_ERR_LIMIT, "cn_nvfp4_gemm: workspace of %zu B, %zu B needed", workspace_bytes, cn_nvfp4_gemm_workspace_bytes(k, m));
    uint16_t* xh = (uint16_t*)workspace;
    float* rs = (float*)((char*)workspace + (((size_t)m * k * 2 + 255) & ~(size_t)255));
    if (dtype == CN_BF16)
        gemm_prep_x_kernel<1><<<m, 256, 0, stream>>>(x, xh, rs, k);
    else
        gemm_prep_x_kernel<0><<<m, 256, 0, stream>>>(x, xh, rs, k);
    CN_CUDA(cudaGetLastError());
    CN_ALLOW_SMEM(nvfp4_gemm_tc5_kernel<128>, (int)smem_of(128));
    CN_ALLOW_SMEM(nvfp4_gemm_tc5_kernel<256>, (int)smem_of(256));
    GemmParams p;
    p.w = (const uint8_t*)w, p.gs = gs, p.xh = xh, p.rs = rs, p.y = y, p.rows = rows, p.k = k, p.m = m, p.ldy = ldy, p.out_bf16 = dtype == CN_BF16;
    p.ksplits = 1, p.part = nullptr;
    if (m > 128) {
        dim3 grid((unsigned)((rows + TM - 1) / TM), (unsigned)((m + 255) / 256));
        nvfp4_gemm_tc5_kernel<256><<<grid, GEMM_THREADS, smem_of(256), stream>>>(p);
    } else {
        int ks = gemm_ksplits(rows, k, m);
        if (rows > 32768) ks = 1;  // the workspace holds partial sums for up to 2^15 rows
        p.ksplits = ks;
        p.part = (float*)((char*)workspace + (((size_t)m * k * 2 + 255) & ~(size_t)255) + (((size_t)m * 4 + 255) & ~(size_t)255));
        dim3 grid((unsigned)((rows + TM - 1) / TM), (unsigned)ks);
        nvfp4_gemm_tc5_kernel<128><<<grid, GEMM_THREADS, smem_of(128), stream>>>(p);
        if (ks > 1) {
            CN_CUDA(cudaGetLastError());
            gemm_splitk_reduce_kernel<<<dim3((unsigned)((rows + 255) / 256), (unsigned)m), 256, 0, stream>>>(p.part, gs, rs, y, rows, m, ldy, ks,
                                                                                                         p.out_bf16);
        }
    }
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}
