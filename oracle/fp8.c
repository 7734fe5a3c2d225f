/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement of the reference's FP8 E4M3 codec (the reference has a codec only, no FP8
 * GEMV) plus the FP8 GEMV this library defines on top of it, used only as the checker for the
 * CUDA kernels and as a timed CPU baseline.
 *
 * Parity pins: the reference's golden table of all 256 codes (torch float8_e4m3fn) and the two
 * sha256 digests of block-dequantised synthetic tensors (converter/tests/fixtures/fp8-*.tsv),
 * committed under tests/golden.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

/* converter/src/fp8.rs:19-33 (`e4m3fn_to_f32`), engine/src/cnq.rs:1363-1376 (`e4m3_to_f32`):
 * bias 7, S.1111.111 is NaN, subnormals m * 2^-9 */
float cn_o_e4m3_to_f32(uint8_t b) {
    int e = (b >> 3) & 0xF;
    float m = (float)(b & 0x7);
    float v;
    if (e == 15 && (b & 0x7) == 7)
        v = NAN;
    else if (e == 0)
        v = m * ldexpf(1.0f, -9);
    else
        v = (1.0f + m / 8.0f) * ldexpf(1.0f, e - 7);
    return (b & 0x80) ? -v : v;
}

/* engine/src/cnq.rs:1310-1361 (`f32_to_e4m3`): round to nearest even, saturating at 448,
 * 0x7F / 0xFF only for NaN inputs */
uint8_t cn_o_f32_to_e4m3(float v) {
    if (isnan(v)) return signbit(v) ? 0xFF : 0x7F;
    uint8_t s = signbit(v) ? 0x80 : 0;
    float f = fabsf(v);
    if (isinf(f)) return s | 0x7E;
    if (f == 0.0f) return s;
    if (f >= 464.0f) return s | 0x7E;
    if (f < ldexpf(1.0f, -6)) {
        float m = nearbyintf(f / ldexpf(1.0f, -9)); /* default rounding mode: ties to even */
        if (m >= 8.0f) return s | (1u << 3);
        return s | ((uint8_t)m & 0x7);
    }
    int e_i = (int)floorf(log2f(f));
    while (ldexpf(1.0f, e_i) > f) e_i--;
    while (ldexpf(1.0f, e_i + 1) <= f) e_i++;
    int exp_field = e_i + 7;
    if (exp_field > 15) return s | 0x7E;
    float q = nearbyintf(f / ldexpf(1.0f, e_i - 3));
    if (q >= 16.0f) {
        int exp2 = e_i + 8;
        if (exp2 > 15) return s | 0x7E;
        return s | (uint8_t)(exp2 << 3);
    }
    return s | (uint8_t)(exp_field << 3) | ((uint8_t)q & 0x7);
}

/* converter/src/fp8.rs:60-82 (`dequant_fp8_block`): out[r][c] = lut[q] * scale[r/128][c/128],
 * row-major ceil grid, partial edge tiles allowed. Returns 0, -1 on a NaN code (refused). */
int cn_o_fp8_dequant(const uint8_t* q, int64_t rows, int64_t cols, const float* scale, float* out) {
    int64_t sc = (cols + 127) / 128;
    for (int64_t r = 0; r < rows; r++)
        for (int64_t c = 0; c < cols; c++) {
            uint8_t b = q[r * cols + c];
            if ((b & 0x7F) == 0x7F) return -1;
            out[r * cols + c] = cn_o_e4m3_to_f32(b) * scale[(r / 128) * sc + c / 128];
        }
    return 0;
}

/* The FP8 GEMV this library defines (no counterpart in the reference, which stops at the codec):
 * W is [rows][cols] E4M3FN bytes with one f32 scale per 128x128 tile (the codec's grid);
 * y[t][r] = sum over column tiles cb of (sum_{k in tile} e4m3(q[r][k]) * x[t][k]) * scale[r/128][cb],
 * all in f32, each tile's inner sum taken left to right. x [T][cols], y [T][rows]. */
int cn_o_fp8_gemv(const uint8_t* q, int64_t rows, int64_t cols, const float* scale, const float* x, int64_t tokens,
                  float* y) {
    int64_t sc = (cols + 127) / 128;
    float lut[256];
    for (int i = 0; i < 256; i++) lut[i] = cn_o_e4m3_to_f32((uint8_t)i);
    for (int64_t t = 0; t < tokens; t++)
        for (int64_t r = 0; r < rows; r++) {
            float acc = 0.0f;
            for (int64_t cb = 0; cb < sc; cb++) {
                int64_t c1 = (cb + 1) * 128 < cols ? (cb + 1) * 128 : cols;
                float part = 0.0f;
                for (int64_t c = cb * 128; c < c1; c++) part += lut[q[r * cols + c]] * x[t * cols + c];
                acc += part * scale[(r / 128) * sc + cb];
            }
            y[t * rows + r] = acc;
        }
    return 0;
}
