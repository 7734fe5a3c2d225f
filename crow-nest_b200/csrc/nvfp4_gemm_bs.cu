// Batched NVFP4 GEMM on the block-scaled FP4 tensor-core path: tcgen05.mma kind::mxf4nvf4 (E2M1 x E2M1, one UE4M3 scale
// per 16 values on both operands, f32 accumulation in tensor memory). Supersedes gemm_fp4_dense / gemm_fp4_dense_b
// (engine/src/kernels.rs:533, :642; MMA shape :362-372, launched by launch_mma_d, engine/src/gen.rs:2491) and the activation
// cascade that feeds them (quant_row_prescaled, engine/src/kernels.rs:264-350; host twin act_cascade, :5354-5475).
//
// Both operands of this MMA are FP4, so the activations are re-quantised: every row becomes a per-row power of two times a
// sum of LEVELS NVFP4 "levels", each level coding what the levels before it left (the reference's cascade, which stops at
// three levels; five are used here - each level buys a factor of about 16, and the output contract of 2 bf16 ulp needs
// the activation error near 1e-5, see tests/test_oracle_cascade.py). The levels of a token ride as separate columns of the
// MMA's N dimension and are added in the epilogue; products and scales are exact, the accumulator is f32.
//
// Layouts (made once per matrix by cn_nvfp4_bs_repack, per call for the activations by the cascade kernel), both stored
// as the exact shared-memory image of a stage so that one 1-D bulk copy brings a stage in:
//   weights   per (128-row tile, 256-column tile): [128 rows x 128 B, 16-byte chunks XOR-swizzled by row & 7] then the
//             scale bytes of the four 64-column MMAs as [4][32][16] (row r at (r % 32) * 16 + (r / 32) * 4 + sub-block),
//             0x7F -> 0x7E and bit 7 cleared (the tensor core reads 0x7F as NaN; engine/src/residency.rs:119-137)
//   cascade   per (32-token block, 256-column tile): [160 rows x 128 B] the same way, row = level * 32 + token, then the
//             scale bytes as [4][2][32][16]
// A CTA owns one 128-row tile and one or two token blocks over a range of column tiles: warp 4 brings the stages in,
// one lane of warp 5 copies the scale chunks to tensor memory (tcgen05.cp) and issues the MMAs, warps 0-3 read the
// accumulator (tcgen05.ld), add the five levels of every token and store. When the row tiles alone cannot fill the GPU the
// column range is split over blockIdx.z and a second kernel adds the partial sums in split order.
#include "common.cuh"

namespace {

constexpr int LEVELS = 5;
constexpr int TB = 32;                    // tokens per token block
constexpr int NCOL = LEVELS * TB;         // MMA N per token block: 160
constexpr int KT = 256;                   // columns per stage (four MMAs of K = 64)
constexpr int A_IMG = 128 * 128, A_SF = 4 * 512, A_STAGE = A_IMG + A_SF;       // 18432
constexpr int B_IMG = NCOL * 128, B_SF = 4 * 2 * 512, B_STAGE = B_IMG + B_SF;  // 24576
constexpr int BS_THREADS = 192;
constexpr int TMEM_COLS = 512;
__host__ __device__ constexpr int stage_bytes(int nb) { return A_STAGE + nb * B_STAGE; }
__host__ __device__ constexpr int stages_of(int nb) { return nb == 2 ? 3 : 5; }
__host__ __device__ constexpr int smem_of(int nb) { return 2048 + 1024 + stages_of(nb) * stage_bytes(nb); }

// ---------------------------------------------------------------- the reference's quantiser, operation for operation
// engine/src/kernels.rs:238-249 (round to nearest onto {0,.5,1,1.5,2,3,4,6}, ties to the even mantissa): the if-chain of the
// reference as a count of passed thresholds
__device__ __forceinline__ uint32_t q_e2m1(float v) {
    const float r = fabsf(v);
    const uint32_t c = (uint32_t)(r > 0.25f) + (uint32_t)(r >= 0.75f) + (uint32_t)(r > 1.25f) + (uint32_t)(r >= 1.75f) + (uint32_t)(r > 2.5f) +
                       (uint32_t)(r >= 3.5f) + (uint32_t)(r > 5.0f);
    // an all-zero sub-block has scale 0 and v = 0 * inf = NaN here: the reference's chain of comparisons then falls through
    // to its last code (6 x scale 0 = 0), and so does this
    return (r != r ? 7u : c) | (v < 0.0f ? 8u : 0u);
}
__device__ __forceinline__ float e2m1_f32(uint32_t n) {
    const uint32_t c = n & 7u;
    const float v = c < 2u ? 0.5f * (float)c : __uint_as_float(((126u + (c >> 1)) << 23) | ((c & 1u) << 22));
    return (n & 8u) ? -v : v;
}
// engine/src/kernels.rs:254-263: the smallest UE4M3 value >= s, saturating at 0x7E. The reference tries the exponents
// e = 0 .. 15 in turn and takes the first whose mantissa ceil(s * 2^(10 - e)) - 8 fits (ceil(s * 512) at e = 0); with
// t = s * 512 = f * 2^x that first exponent is 0 for t <= 7, else 1 + max(0, x - 3 + (8 f > 15)). All products are by powers
// of two, hence exact, and the result is the reference's byte for every s (checked against its host twin).
__device__ __forceinline__ uint32_t enc_ue4m3_up(float s) {
    if (!(s > 0.0f)) return 0;
    const float t = s * 512.0f;
    if (t <= 7.0f) return (uint32_t)ceilf(t);
    if (!(t < 3.0e38f)) return 0x7E;
    const int x = (int)((__float_as_uint(t) >> 23) & 0xFFu) - 127;
    const float f8 = t * __uint_as_float((uint32_t)(127 + 3 - x) << 23);  // in [8, 16)
    int j = x - 3 + (f8 > 15.0f ? 1 : 0);
    j = j < 0 ? 0 : j;
    if (j > 14) return 0x7E;
    const int m = (int)ceilf(t * __uint_as_float((uint32_t)(127 - j) << 23)) - 8;
    const int e = 1 + j;
    if (e == 15 && m > 6) return 0x7E;
    return (uint32_t)((e << 3) | m);
}
// engine/src/kernels.rs:298-304
__device__ __forceinline__ int row_prescale_k(float amax) {
    if (!(amax > 0.0f) || !(amax <= 3.402823466e38f)) return 0;
    const uint32_t bits = __float_as_uint(amax);
    const int ef = (int)((bits >> 23) & 0xFFu);
    const int e = ef ? ef - 126 : (31 - __clz((int)(bits & 0x7FFFFFu))) - 148;
    return max(-64, min(64, 11 - e));
}
// engine/src/kernels.rs:305-322: one 16-value sub-block -> scale byte, 8 code bytes, residual (in place)
__device__ __forceinline__ void quant_level(float v[16], uint32_t& sc_out, uint32_t code[2]) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; j++) amax = fmaxf(amax, fabsf(v[j]));
    const uint32_t sc = enc_ue4m3_up(amax * (1.0f / 6.0f));
    const float scf = ue4m3_f32(sc, false);
    const float inv = 1.0f / scf;
    sc_out = sc;
    code[0] = code[1] = 0u;
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const uint32_t n = q_e2m1(v[j] * inv);
        code[j >> 3] |= n << (4 * (j & 7));
        v[j] = v[j] - e2m1_f32(n) * scf;
    }
}
template <int XT>
__device__ __forceinline__ float load_act(const void* x, size_t i) {
    return XT == 1 ? __bfloat162float(((const __nv_bfloat16*)x)[i]) : ((const float*)x)[i];
}
__device__ __forceinline__ float block_amax(float amax, float* buf) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) buf[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = 0.0f;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) amax = fmaxf(amax, buf[w]);
    return amax;
}

// The cascade in the reference's own byte layout (engine/src/kernels.rs:275-283, with `levels` in place of three):
// per row levels * bpr * 36 bytes, level L at L * bpr * 36 in the container's block layout, then the f32 factor 2^-k.
// grid (rows), block 128 (quant_x_fp4, engine/src/kernels.rs:351).
template <int XT>
__global__ void act_cascade_kernel(const void* __restrict__ x, uint8_t* __restrict__ out, int k, int levels) {
    __shared__ float amax_w[32];
    const size_t row = blockIdx.x;
    const int bpr = k / 64;
    float amax = 0.0f;
    for (int i = threadIdx.x; i < k; i += blockDim.x) amax = fmaxf(amax, fabsf(load_act<XT>(x, row * k + i)));
    amax = block_amax(amax, amax_w);
    const int kk = row_prescale_k(amax);
    const float up = __uint_as_float((uint32_t)(127 + kk) << 23);
    uint8_t* op = out + row * ((size_t)levels * bpr * 36 + 4);
    for (int sb = threadIdx.x; sb < bpr * 4; sb += blockDim.x) {
        const int b = sb >> 2, s = sb & 3;
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; j++) v[j] = load_act<XT>(x, row * k + (size_t)b * 64 + s * 16 + j) * up;
        for (int lv = 0; lv < levels; lv++) {
            uint32_t sc, code[2];
            quant_level(v, sc, code);
            uint8_t* base = op + (size_t)lv * bpr * 36 + (size_t)b * 36;
            base[s] = (uint8_t)sc;
            *(uint32_t*)(base + 4 + s * 8) = code[0];
            *(uint32_t*)(base + 8 + s * 8) = code[1];
        }
    }
    if (threadIdx.x == 0) {
        const float f = __uint_as_float((uint32_t)(127 - kk) << 23);
        memcpy(op + (size_t)levels * bpr * 36, &f, 4);
    }
}

// rs[tok] = 2^-k of every activation row (1 for rows beyond m). grid (token blocks * TB), block 256.
template <int XT>
__global__ void bs_rowscale_kernel(const void* __restrict__ x, float* __restrict__ rs, int k, int m) {
    __shared__ float amax_w[32];
    const int tok = blockIdx.x;
    float amax = 0.0f;
    if (tok < m)
        for (int i = threadIdx.x; i < k; i += blockDim.x) amax = fmaxf(amax, fabsf(load_act<XT>(x, (size_t)tok * k + i)));
    amax = block_amax(amax, amax_w);
    if (threadIdx.x == 0) rs[tok] = __uint_as_float((uint32_t)(127 - row_prescale_k(amax)) << 23);
}

// The same cascade (LEVELS levels) written as the stage images of the GEMM: one thread per 16-value sub-block of a row.
// grid (tokens rounded up to whole token blocks, k / 16 / 128 rounded up), block 128; rows beyond m are zero rows.
template <int XT>
__global__ void bs_cascade_kernel(const void* __restrict__ x, uint8_t* __restrict__ ws, const float* __restrict__ rs, int k, int m) {
    const int tok = blockIdx.x, tb = tok / TB, tt = tok % TB;
    const int kts = k / KT;
    const int sb = blockIdx.y * blockDim.x + threadIdx.x;
    if (sb >= k / 16) return;
    const bool live = tok < m;
    const float up = 1.0f / rs[tok];  // a power of two: exact
    const int kt = sb >> 4, sub = sb & 15;  // column tile, sub-block inside it: MMA sub >> 2, scale slot sub & 3
    float v[16];
    if (live) {
        if (XT == 1) {
            const uint4* src = (const uint4*)((const char*)x + ((size_t)tok * k + (size_t)sb * 16) * 2);
            const uint4 a = src[0], b = src[1];
            const uint32_t u[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int j = 0; j < 8; j++) v[2 * j] = __uint_as_float(u[j] << 16) * up, v[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u) * up;
        } else {
            const float4* src = (const float4*)((const char*)x + ((size_t)tok * k + (size_t)sb * 16) * 4);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float4 a = src[j];
                v[4 * j] = a.x * up, v[4 * j + 1] = a.y * up, v[4 * j + 2] = a.z * up, v[4 * j + 3] = a.w * up;
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 16; j++) v[j] = 0.0f;
    }
    uint8_t* img = ws + ((size_t)tb * kts + kt) * B_STAGE;
#pragma unroll
    for (int lv = 0; lv < LEVELS; lv++) {
        uint32_t sc, code[2];
        quant_level(v, sc, code);
        const int n = lv * TB + tt;
        const int c = sub >> 1;
        *(uint2*)(img + (size_t)n * 128 + ((c ^ (n & 7)) << 4) + (sub & 1) * 8) = make_uint2(code[0], code[1]);
        img[B_IMG + ((sub >> 2) * 2 + (n >> 7)) * 512 + ((n & 127) & 31) * 16 + ((n & 127) >> 5) * 4 + (sub & 3)] = (uint8_t)sc;
    }
}

// container -> stage images of the weights. One thread per 16-byte chunk of the image (32 codes = half a container block)
// and one per scale byte.
__global__ void bs_repack_kernel(const uint8_t* __restrict__ w, uint8_t* __restrict__ out, int rows, int k) {
    const int kts = k / KT, bpr = k / 64;
    const long long tile = blockIdx.x;  // (row tile, column tile)
    const int rt = (int)(tile / kts), kt = (int)(tile % kts);
    uint8_t* img = out + (size_t)tile * A_STAGE;
    for (int u = threadIdx.x; u < 128 * 8; u += blockDim.x) {
        const int r = u >> 3, c = u & 7;
        const int row = rt * 128 + r;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < rows) {
            const uint8_t* src = w + ((size_t)row * bpr + kt * 4 + (c >> 1)) * 36 + 4 + (c & 1) * 16;
            const uint32_t* s4 = (const uint32_t*)src;  // container blocks are 4-byte aligned
            v = make_uint4(s4[0], s4[1], s4[2], s4[3]);
        }
        *(uint4*)(img + (size_t)r * 128 + ((c ^ (r & 7)) << 4)) = v;
    }
    for (int u = threadIdx.x; u < 128 * 16; u += blockDim.x) {
        const int r = u >> 4, sub = u & 15;  // MMA sub >> 2, scale slot sub & 3
        const int row = rt * 128 + r;
        uint32_t s = 0;
        if (row < rows) {
            s = w[((size_t)row * bpr + kt * 4 + (sub >> 2)) * 36 + (sub & 3)] & 0x7Fu;
            if (s == 0x7Fu) s = 0x7Eu;
        }
        img[A_IMG + (sub >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (sub & 3)] = (uint8_t)s;
    }
}

// ---------------------------------------------------------------- tcgen05 wrappers
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
// K-major tile with 128-byte swizzle: start >> 4, leading offset 1 (unused), stride 8 rows * 128 B, version 1, layout 2
__device__ __forceinline__ uint64_t desc_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// a scale chunk: 32 rows of 16 bytes, no swizzle: 8-row groups 128 B apart
__device__ __forceinline__ uint64_t desc_sf(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}
// instruction descriptor, kind::mxf4nvf4: A and B E2M1 (format 1) K-major, UE4M3 scales (0), N >> 3 at bit 17, M >> 4 at bit 24
__host__ __device__ constexpr uint32_t idesc_bs(int n) { return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24); }
__device__ __forceinline__ void cp_sf(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_bs(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
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

struct BsParams {
    const uint8_t* wp;  // repacked weights
    const uint8_t* xq;  // cascade images
    const float* gs;
    const float* rs;    // [token blocks * TB] the rows' 2^-k
    void* y;
    float* part;        // [ksplits][m][rows] raw sums when ksplits > 1
    int rows, k, m, ldy, out_bf16, ksplits;
};

// grid (row tiles, token blocks / NB, ksplits)
template <int NB>
__global__ void __launch_bounds__(BS_THREADS, 1) nvfp4_gemm_bs_kernel(const BsParams p) {
    constexpr int STAGES = stages_of(NB), STAGE = stage_bytes(NB);
    constexpr uint32_t IDESC = idesc_bs(NCOL);
    constexpr uint32_t SFA_COL = NB * NCOL, SFB_COL = SFA_COL + 16;  // tensor-memory columns behind the accumulators
    static_assert(SFB_COL + NB * 32 <= TMEM_COLS, "tensor memory columns");
    extern __shared__ uint8_t smem_raw[];
    uint64_t* full = (uint64_t*)smem_raw;
    uint64_t* empty = full + STAGES;
    uint64_t* accbar = empty + STAGES;
    uint32_t* tmem_slot = (uint32_t*)(accbar + 1);
    volatile int* failed = (volatile int*)(tmem_slot + 1);
    const uint32_t ring_addr = (smem_u32(smem_raw) + 2048u + 1023u) & ~1023u;
    uint8_t* ring = smem_raw + (ring_addr - smem_u32(smem_raw));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kts = p.k / KT;
    const int rt = blockIdx.x, tb0 = blockIdx.y * NB;
    const int ntb = (p.m + TB - 1) / TB;
    const int ksi = blockIdx.z;
    const int kt0 = (int)(((long long)ksi * kts) / p.ksplits), kt1 = (int)(((long long)(ksi + 1) * kts) / p.ksplits);
    const int nst = kt1 - kt0;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accbar, 1);
        mbar_fence_init();
        *failed = 0;
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 4) {
        // ------------------------------------------------------------ producer: one bulk copy per operand and stage
        if (lane == 0) {
            for (int i = 0; i < nst; i++) {
                const int s = i % STAGES;
                if (i >= STAGES && !mbar_wait(&empty[s], ((i / STAGES) - 1) & 1)) {
                    cn_dev_fail(CN_DEV_WAIT_EMPTY);
                    *failed = 1;
                    break;
                }
                uint8_t* dst = ring + (size_t)s * STAGE;
                int nbl = 0;
                for (int nb = 0; nb < NB; nb++) nbl += (tb0 + nb) < ntb;
                mbar_expect_tx(&full[s], (uint32_t)(A_STAGE + nbl * B_STAGE));
                mbar_arrive(&full[s]);
                bulk_g2s(dst, p.wp + ((size_t)rt * kts + kt0 + i) * A_STAGE, A_STAGE, &full[s]);
                for (int nb = 0; nb < NB; nb++)
                    if (tb0 + nb < ntb) bulk_g2s(dst + A_STAGE + nb * B_STAGE, p.xq + ((size_t)(tb0 + nb) * kts + kt0 + i) * B_STAGE, B_STAGE, &full[s]);
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ scale copies and MMAs, one lane
        if (lane == 0) {
            bool ok = true;
            for (int i = 0; i < nst && ok; i++) {
                const int s = i % STAGES;
                if (!mbar_wait(&full[s], (i / STAGES) & 1)) {
                    cn_dev_fail(CN_DEV_WAIT_FULL);
                    *failed = 1;
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = ring_addr + (uint32_t)s * STAGE;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    cp_sf(tmem + SFA_COL + 4 * j, desc_sf(a_addr + A_IMG + 512 * j));
#pragma unroll
                    for (int nb = 0; nb < NB; nb++) {
                        if (tb0 + nb >= ntb) continue;
                        const uint32_t b_addr = a_addr + A_STAGE + nb * B_STAGE;
                        cp_sf(tmem + SFB_COL + nb * 32 + 8 * j, desc_sf(b_addr + B_IMG + (2 * j) * 512));
                        cp_sf(tmem + SFB_COL + nb * 32 + 8 * j + 4, desc_sf(b_addr + B_IMG + (2 * j + 1) * 512));
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
#pragma unroll
                    for (int nb = 0; nb < NB; nb++) {
                        if (tb0 + nb >= ntb) continue;
                        const uint32_t b_addr = a_addr + A_STAGE + nb * B_STAGE;
                        umma_bs(tmem + nb * NCOL, desc_sw128(a_addr + 32u * j), desc_sw128(b_addr + 32u * j), IDESC, tmem + SFA_COL + 4 * j,
                                tmem + SFB_COL + nb * 32 + 8 * j, (i > 0 || j > 0) ? 1u : 0u);
                    }
                }
                umma_commit(&empty[s]);
            }
            if (ok) umma_commit(accbar);
        }
    } else {
        // ------------------------------------------------------------ epilogue: lane = weight row, the five levels of a token added
        bool ok = true;
        if (!mbar_wait(accbar, 0)) {
            if (!*failed) cn_dev_fail(CN_DEV_WAIT_FULL);
            ok = false;
        }
        if (ok && nst > 0) {
            tc_fence_after();
            const int q = warp & 3;
            const int row = rt * 128 + 32 * q + lane;
            const float gs = p.gs[0];
            for (int nb = 0; nb < NB; nb++) {
                if (tb0 + nb >= ntb) break;
                float acc[TB];
#pragma unroll
                for (int i = 0; i < TB; i++) acc[i] = 0.0f;
#pragma unroll
                for (int lv = 0; lv < LEVELS; lv++) {
                    uint32_t v[32];
                    tmem_ld32(tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(nb * NCOL + lv * TB), v);
#pragma unroll
                    for (int i = 0; i < TB; i++) acc[i] += __uint_as_float(v[i]);
                }
#pragma unroll
                for (int i = 0; i < TB; i++) {
                    const int tok = (tb0 + nb) * TB + i;
                    if (tok < p.m && row < p.rows) {
                        if (p.ksplits > 1) {
                            p.part[((size_t)ksi * p.m + tok) * p.rows + row] = acc[i];
                        } else {
                            const float r = acc[i] * (gs * p.rs[tok]);
                            if (p.out_bf16)
                                ((__nv_bfloat16*)p.y)[(size_t)tok * p.ldy + row] = __float2bfloat16_rn(r);
                            else
                                ((float*)p.y)[(size_t)tok * p.ldy + row] = r;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
}

// y[t][n] = (sum over splits, in order, of part[s][t][n]) * gs * rs[t]
__global__ void bs_splitk_reduce_kernel(const float* __restrict__ part, const float* __restrict__ gs, const float* __restrict__ rs,
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

int ksplits_for(int rows, int k, int m) {
    const int rts = (rows + 127) / 128, ntb = (m + TB - 1) / TB, kts = k / KT;
    const int ctas = rts * ((ntb + 1) / 2);
    int ks = 1;
    if (ctas < 120) {
        ks = 148 / ctas;
        if (ks > kts / 4) ks = kts / 4;
        if (ks < 1) ks = 1;
    }
    return ks;
}

}  // namespace

extern "C" size_t cn_nvfp4_bs_packed_bytes(int rows, int k) {
    if (rows <= 0 || k <= 0 || k % KT) return 0;
    return (size_t)((rows + 127) / 128) * (k / KT) * A_STAGE;
}

extern "C" int cn_nvfp4_bs_repack(const void* w, void* packed, int rows, int k, cn_stream_t stream) {
    if (rows <= 0 || k <= 0 || k % KT) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_bs_repack: k = %d must be a positive multiple of 256", k);
    if (!w || !packed || ((uintptr_t)w & 3) || ((uintptr_t)packed & 15)) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_bs_repack: null or misaligned buffer");
    const long long tiles = (long long)((rows + 127) / 128) * (k / KT);
    bs_repack_kernel<<<(unsigned)tiles, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)w, (uint8_t*)packed, rows, k);
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}

extern "C" size_t cn_nvfp4_bs_workspace_bytes(int rows, int k, int m) {
    if (rows <= 0 || k <= 0 || k % KT || m <= 0) return 0;
    const size_t ntb = (size_t)(m + TB - 1) / TB;
    const int ks = ksplits_for(rows, k, m);
    return ntb * (k / KT) * B_STAGE + ntb * TB * 4 + 256 + (ks > 1 ? (size_t)ks * m * rows * 4 : 0);
}

extern "C" int cn_nvfp4_bs_gemm(const void* packed, const float* gs, const void* x, void* y, int rows, int k, int m, int ldy, int dtype,
                                void* workspace, size_t workspace_bytes, cn_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (rows <= 0 || k <= 0 || k % KT) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_bs_gemm: k = %d must be a positive multiple of 256", k);
    if (m < 1) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_bs_gemm: m = %d", m);
    if (ldy < rows) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_bs_gemm: ldy %d < rows %d", ldy, rows);
    if (dtype != CN_F32 && dtype != CN_BF16) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_bs_gemm: dtype %d is neither CN_F32 nor CN_BF16", dtype);
    if (!workspace || ((uintptr_t)workspace & 255) || workspace_bytes < cn_nvfp4_bs_workspace_bytes(rows, k, m))
        CN_FAIL(CN_ERR_LIMIT, "cn_nvfp4_bs_gemm: the workspace must be 256-byte aligned and at least %zu B", cn_nvfp4_bs_workspace_bytes(rows, k, m));
    const int ntb = (m + TB - 1) / TB, kts = k / KT;
    uint8_t* xq = (uint8_t*)workspace;
    float* rs = (float*)(xq + (size_t)ntb * kts * B_STAGE);
    float* part = rs + (size_t)ntb * TB + 64;
    if (((uintptr_t)x & 15)) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_bs_gemm: x must be 16-byte aligned");
    const dim3 cgrid(ntb * TB, (k / 16 + 127) / 128);
    if (dtype == CN_BF16) {
        bs_rowscale_kernel<1><<<ntb * TB, 256, 0, stream>>>(x, rs, k, m);
        bs_cascade_kernel<1><<<cgrid, 128, 0, stream>>>(x, xq, rs, k, m);
    } else {
        bs_rowscale_kernel<0><<<ntb * TB, 256, 0, stream>>>(x, rs, k, m);
        bs_cascade_kernel<0><<<cgrid, 128, 0, stream>>>(x, xq, rs, k, m);
    }
    CN_CUDA(cudaGetLastError());
    BsParams p;
    p.wp = (const uint8_t*)packed, p.xq = xq, p.gs = gs, p.rs = rs, p.y = y, p.rows = rows, p.k = k, p.m = m, p.ldy = ldy, p.out_bf16 = dtype == CN_BF16;
    p.ksplits = ksplits_for(rows, k, m), p.part = p.ksplits > 1 ? part : nullptr;
    const int rts = (rows + 127) / 128;
    if (ntb >= 2) {
        CN_ALLOW_SMEM(nvfp4_gemm_bs_kernel<2>, smem_of(2));
        nvfp4_gemm_bs_kernel<2><<<dim3(rts, (ntb + 1) / 2, p.ksplits), BS_THREADS, smem_of(2), stream>>>(p);
    } else {
        CN_ALLOW_SMEM(nvfp4_gemm_bs_kernel<1>, smem_of(1));
        nvfp4_gemm_bs_kernel<1><<<dim3(rts, 1, p.ksplits), BS_THREADS, smem_of(1), stream>>>(p);
    }
    CN_CUDA(cudaGetLastError());
    if (p.ksplits > 1) {
        bs_splitk_reduce_kernel<<<dim3((rows + 255) / 256, m), 256, 0, stream>>>(part, gs, rs, y, rows, m, ldy, p.ksplits, p.out_bf16);
        CN_CUDA(cudaGetLastError());
    }
    return CN_OK;
}

extern "C" int cn_nvfp4_act_cascade(const void* x, void* out, int rows, int k, int levels, int dtype, cn_stream_t stream) {
    if (rows < 1 || k <= 0 || k % 64) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_act_cascade: [%d, %d] is not whole 64-value blocks", rows, k);
    if (levels < 1 || levels > 8) CN_FAIL(CN_ERR_LIMIT, "cn_nvfp4_act_cascade: %d levels (1..8)", levels);
    if (dtype != CN_F32 && dtype != CN_BF16) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_act_cascade: dtype %d is neither CN_F32 nor CN_BF16", dtype);
    if (dtype == CN_BF16)
        act_cascade_kernel<1><<<rows, 128, 0, (cudaStream_t)stream>>>(x, (uint8_t*)out, k, levels);
    else
        act_cascade_kernel<0><<<rows, 128, 0, (cudaStream_t)stream>>>(x, (uint8_t*)out, k, levels);
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}
