// FP8 (E4M3FN) GEMV for M = 1..8 activation rows: y[m][r] = sum over 128-column tiles of
// (sum_k e4m3(q[r][k]) * x[m][k]) * scale[r/128][k/128].
//
// The reference engine has an FP8 codec only (engine/src/cnq.rs:1312-1376, converter/src/fp8.rs:19-82:
// E4M3FN bytes with one f32 scale per 128x128 tile); this GEMV is defined on that codec so that
// FP8-stored projections can be served without a conversion pass.
//
// HBM-bound at one byte per weight. One warp per output row, lanes stride the row in 16-byte
// groups (coalesced 128-bit loads, four in flight per lane); codes are widened with
// cvt.rn.f16x2.e4m3x2 (every E4M3 value is exact in f16) and multiplied with the f16 x f16 -> f32
// mixed FMA against activations staged once per CTA in shared memory as f16 with a power-of-two
// scale per 128-column tile (exact for bf16 input); the tile's weight scale and the inverse
// activation scale are applied to each 16-value partial sum. Lanes are reduced with xor shuffles.
#include "common.cuh"

int cn_fp8_gemv_tc_launch(const void* w, const float* scale, const void* x, void* y, int rows, int cols, int m, int ldy, int dtype, cudaStream_t st);

namespace {

constexpr int WARPS = 8;

template <int XT, int MP>
__global__ void __launch_bounds__(WARPS * 32) fp8_gemv_kernel(const uint8_t* __restrict__ w, const float* __restrict__ scale,
                                                              const void* __restrict__ x, void* __restrict__ y, int rows, int cols, int m_live,
                                                              int ldy) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int tiles = (cols + 127) / 128;
    uint16_t* xs = (uint16_t*)smem;                      // [MP][cols] f16
    float* xinv = (float*)(xs + (size_t)MP * cols);      // [MP][tiles]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_launch_dependents();
    pdl_wait();
    // stage the activations: one 128-column tile per warp pass, 4 values per lane
    for (int i = warp; i < MP * tiles; i += WARPS) {
        const int m = i / tiles, tl = i - m * tiles, c0 = tl * 128 + lane * 4;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (m < m_live) {
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (c0 + j < cols)
                    v[j] = XT == 1 ? __bfloat162float(((const __nv_bfloat16*)x)[(size_t)m * cols + c0 + j]) : ((const float*)x)[(size_t)m * cols + c0 + j];
        }
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        uint32_t e = (__float_as_uint(amax) >> 23) & 0xFF;
        float mul = 1.0f, inv = 1.0f;
        if (amax > 0.0f && e < 255) {
            e = e < 15 ? 15 : e;
            mul = __uint_as_float((268u - e) << 23);
            inv = __uint_as_float((e - 14u) << 23);
        }
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (c0 + j < cols) xs[(size_t)m * cols + c0 + j] = __half_as_ushort(__float2half_rn(v[j] * mul));
        if (lane == 0) xinv[m * tiles + tl] = inv;
    }
    __syncthreads();

    const int groups = cols / 16;  // 16-byte groups per row
    for (int row = blockIdx.x * WARPS + warp; row < rows; row += gridDim.x * WARPS) {
        const uint4* wr = (const uint4*)(w + (size_t)row * cols);
        const float* srow = scale + (size_t)(row / 128) * tiles;
        float acc[MP];
#pragma unroll
        for (int m = 0; m < MP; m++) acc[m] = 0.0f;
        for (int g0 = lane; g0 < groups; g0 += 128) {
            uint4 q[4];
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (g0 + 32 * u < groups) q[u] = __ldg(wr + g0 + 32 * u);
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int g = g0 + 32 * u;
                if (g < groups) {
                    const uint32_t qq[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
                    uint32_t h[8];
#pragma unroll
                    for (int i = 0; i < 4; i++)
                        asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, lo;\n\tcvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
                            : "=r"(h[2 * i]), "=r"(h[2 * i + 1])
                            : "r"(qq[i]));
                    const int tl = g >> 3;
                    const float ws = srow[tl];
#pragma unroll
                    for (int m = 0; m < MP; m++) {
                        const uint4* xp = (const uint4*)(xs + (size_t)m * cols + (size_t)g * 16);
                        const uint4 xa = xp[0], xb = xp[1];
                        const uint32_t xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
                        float p0 = 0.0f, p1 = 0.0f;
#pragma unroll
                        for (int i = 0; i < 8; i++) fma2_f16_f32(p0, p1, h[i], xv[i]);
                        acc[m] = fmaf(p0 + p1, ws * xinv[m * tiles + tl], acc[m]);
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MP; m++) {
            float v = acc[m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && m < m_live) {
                if (XT == 1)
                    ((__nv_bfloat16*)y)[(size_t)m * ldy + row] = __float2bfloat16_rn(v);
                else
                    ((float*)y)[(size_t)m * ldy + row] = v;
            }
        }
    }
}

template <int XT>
int launch(const void* w, const float* scale, const void* x, void* y, int rows, int cols, int m, int ldy, cudaStream_t st) {
    const int mp = m == 1 ? 1 : (m == 2 ? 2 : (m <= 4 ? 4 : 8));
    const int tiles = (cols + 127) / 128;
    const size_t smem = (size_t)mp * cols * 2 + (size_t)mp * tiles * 4 + 16;
    if (smem > 200 * 1024) {
        // the staged activations of all m rows do not fit one CTA: two calls over half the rows each
        if (m == 1) CN_FAIL(CN_ERR_LIMIT, "cn_fp8_gemv: %d activations need %zu B of shared memory", cols, smem);
        const int m0 = m / 2;
        const size_t es = XT == 1 ? 2 : 4;
        if (int rc = launch<XT>(w, scale, x, y, rows, cols, m0, ldy, st)) return rc;
        return launch<XT>(w, scale, (const char*)x + (size_t)m0 * cols * es, (char*)y + (size_t)m0 * ldy * es, rows, cols, m - m0, ldy, st);
    }
    int grid = (rows + WARPS - 1) / WARPS;
    if (grid > 148 * 8) grid = 148 * 8;
#define CN_FP8_CASE(MPV)                                                                                                  \
    if (mp == MPV) {                                                                                                      \
        CN_ALLOW_SMEM((fp8_gemv_kernel<XT, MPV>), 200 * 1024);                                                            \
        fp8_gemv_kernel<XT, MPV><<<grid, WARPS * 32, smem, st>>>((const uint8_t*)w, scale, x, y, rows, cols, m, ldy);    \
    }
    CN_FP8_CASE(1) CN_FP8_CASE(2) CN_FP8_CASE(4) CN_FP8_CASE(8)
#undef CN_FP8_CASE
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}

}  // namespace

extern "C" int cn_fp8_gemv(const void* w, const float* scale, const void* x, void* y, int rows, int cols, int m, int ldy, int dtype,
                           cn_stream_t stream) {
    if (rows <= 0 || cols <= 0 || cols % 16 != 0) CN_FAIL(CN_ERR_SHAPE, "cn_fp8_gemv: %d columns must be a positive multiple of 16", cols);
    if (m < 1 || m > CN_MAX_M) CN_FAIL(CN_ERR_LIMIT, "cn_fp8_gemv: m = %d, the kernel takes 1..%d activation rows", m, CN_MAX_M);
    if (ldy < rows) CN_FAIL(CN_ERR_SHAPE, "cn_fp8_gemv: ldy %d < rows %d", ldy, rows);
    if (((uintptr_t)w & 15) || ((uintptr_t)x & 15)) CN_FAIL(CN_ERR_SHAPE, "cn_fp8_gemv: weight and activation pointers must be 16-byte aligned");
    if (dtype != CN_BF16 && dtype != CN_F32) CN_FAIL(CN_ERR_SHAPE, "cn_fp8_gemv: dtype %d is neither CN_F32 nor CN_BF16", dtype);
    // whole 128-column blocks: the tensor-core kernel (fp8_gemv_tc.cu); ragged rows stay on the warp-per-row kernel below
    {
        const int rc = cn_fp8_gemv_tc_launch(w, scale, x, y, rows, cols, m, ldy, dtype, (cudaStream_t)stream);
        if (rc >= 0) return rc;
    }
    if (dtype == CN_BF16) return launch<1>(w, scale, x, y, rows, cols, m, ldy, (cudaStream_t)stream);
    if (dtype == CN_F32) return launch<0>(w, scale, x, y, rows, cols, m, ldy, (cudaStream_t)stream);
    CN_FAIL(CN_ERR_SHAPE, "cn_fp8_gemv: dtype %d is neither CN_F32 nor CN_BF16", dtype);
}
