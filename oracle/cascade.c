/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement of the reference's activation cascade: an f32 activation row is re-quantised
 * into several NVFP4 levels, each level coding the residual the previous ones left, behind one
 * power-of-two factor per row. The block-scaled FP4 tensor-core GEMM consumes activations in this
 * form; this file is the checker for the device-side quantiser and the tool that measures how many
 * levels the accuracy contract needs.
 *
 * Follows engine/src/kernels.rs:236-350 (device text: q_e2m1, enc_ue4m3_up, row_prescale_k,
 * quant_level, quant_row_prescaled) and its host twin `act_cascade`, engine/src/kernels.rs:5354-5475.
 * The reference fixes three levels; the level count is a parameter here (1..8), three giving the
 * reference's bytes. Parity pin: the reference's own assertions on the twin
 * (engine/src/kernels.rs:5546-5568, :5608-5633), restated in tests/test_oracle_cascade.py.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

float cn_o_e2m1(uint32_t nibble);
float cn_o_ue4m3(uint32_t byte);

/* engine/src/kernels.rs:238-249 (`q_e2m1`): round to nearest onto {0,.5,1,1.5,2,3,4,6}, ties to the even mantissa */
uint32_t cn_o_q_e2m1(float v) {
    const uint32_t s = v < 0.0f ? 8u : 0u;
    const float r = fabsf(v);
    if (r <= 0.25f) return s;
    if (r < 0.75f) return s | 1;
    if (r <= 1.25f) return s | 2;
    if (r < 1.75f) return s | 3;
    if (r <= 2.5f) return s | 4;
    if (r < 3.5f) return s | 5;
    if (r <= 5.0f) return s | 6;
    return s | 7;
}

/* engine/src/kernels.rs:254-263 (`enc_ue4m3_up`): the smallest UE4M3 value >= s; 0 iff s <= 0; saturates at 0x7E */
uint8_t cn_o_enc_ue4m3_up(float s) {
    if (!(s > 0.0f)) return 0;
    for (int e = 0; e < 16; e++) {
        const float mul = e == 0 ? 512.0f : ldexpf(1.0f, 10 - e);
        const float m = ceilf(s * mul) - (e == 0 ? 0.0f : 8.0f);
        const float m_max = e == 15 ? 6.0f : 7.0f;
        if (m >= 0.0f && m <= m_max) return (uint8_t)((e << 3) | (int)m);
    }
    return 0x7E;
}

/* engine/src/kernels.rs:298-304 (`row_prescale_k`): k with amax * 2^k in [1024, 2048), clamped to +-64; 0 for a
 * zero, NaN or infinite amax */
int cn_o_row_prescale_k(float amax) {
    if (!(amax > 0.0f) || !(amax <= 3.402823466e38f)) return 0;
    uint32_t bits;
    memcpy(&bits, &amax, 4);
    const int ef = (int)((bits >> 23) & 0xFFu);
    int e;
    if (ef) {
        e = ef - 126;
    } else {
        const uint32_t m = bits & 0x7FFFFFu;
        e = (31 - __builtin_clz(m)) - 148;
    }
    int k = 11 - e;
    if (k < -64) k = -64;
    if (k > 64) k = 64;
    return k;
}

/* engine/src/kernels.rs:305-322 (`quant_level`): one 16-value sub-block; writes its scale byte and 8 code bytes,
 * returns the residual in r */
static void quant_level(const float* p, float* r, uint8_t* sc_dst, uint8_t* d_dst) {
    float amax = 0.0f;
    for (int j = 0; j < 16; j++) amax = fmaxf(amax, fabsf(p[j]));
    const uint8_t sc = cn_o_enc_ue4m3_up(amax * (1.0f / 6.0f));
    const float scf = cn_o_ue4m3(sc);
    const float inv = 1.0f / scf;
    *sc_dst = sc;
    for (int j = 0; j < 8; j++) {
        const uint32_t n0 = cn_o_q_e2m1(p[2 * j] * inv), n1 = cn_o_q_e2m1(p[2 * j + 1] * inv);
        d_dst[j] = (uint8_t)(n0 | (n1 << 4));
        r[2 * j] = p[2 * j] - cn_o_e2m1(n0) * scf;
        r[2 * j + 1] = p[2 * j + 1] - cn_o_e2m1(n1) * scf;
    }
}

/* engine/src/kernels.rs:5418-5437 (`quant_row_with`) with `levels` in place of the fixed three: out holds
 * levels * bpr * 36 bytes (level L at L * bpr * 36, container block layout) and then the f32 factor 2^-k.
 * `level_shift` (0 in the reference): level L codes the residual times 2^(level_shift * L), so that deep levels stay
 * inside the UE4M3 range; its dequantised value is divided by the same power. */
void cn_o_act_cascade(const float* x, int64_t k_dim, int levels, int prescale, int level_shift, uint8_t* out) {
    const int64_t bpr = k_dim / 64;
    float amax = 0.0f;
    for (int64_t i = 0; i < k_dim; i++) amax = fmaxf(amax, fabsf(x[i]));
    const int k = prescale ? cn_o_row_prescale_k(amax) : 0;
    const float up = ldexpf(1.0f, k), lup = ldexpf(1.0f, level_shift);
    for (int64_t b = 0; b < bpr; b++)
        for (int s = 0; s < 4; s++) {
            float src[16], res[16];
            for (int j = 0; j < 16; j++) src[j] = x[b * 64 + s * 16 + j] * up;
            for (int lv = 0; lv < levels; lv++) {
                uint8_t* base = out + (int64_t)lv * bpr * 36 + b * 36;
                quant_level(src, res, base + s, base + 4 + s * 8);
                for (int j = 0; j < 16; j++) src[j] = res[j] * lup;
            }
        }
    const float f = ldexpf(1.0f, -k);
    memcpy(out + (int64_t)levels * bpr * 36, &f, 4);
}

/* engine/src/kernels.rs:5446-5474 (`dequant_level`, `dequant_row`): the value the MMA consumers see */
void cn_o_act_cascade_dequant(const uint8_t* q, int64_t k_dim, int levels, int level_shift, float* out) {
    const int64_t bpr = k_dim / 64;
    for (int64_t i = 0; i < k_dim; i++) out[i] = 0.0f;
    for (int lv = 0; lv < levels; lv++) {
        const float down = ldexpf(1.0f, -level_shift * lv);
        for (int64_t b = 0; b < bpr; b++) {
            const uint8_t* blk = q + (int64_t)lv * bpr * 36 + b * 36;
            for (int idx = 0; idx < 64; idx++) {
                const uint32_t byte = blk[4 + (idx >> 1)];
                const uint32_t nib = (idx & 1) ? byte >> 4 : byte & 0xF;
                out[b * 64 + idx] += cn_o_e2m1(nib) * cn_o_ue4m3(blk[idx >> 4]) * down;
            }
        }
    }
    float f;
    memcpy(&f, q + (int64_t)levels * bpr * 36, 4);
    for (int64_t i = 0; i < k_dim; i++) out[i] *= f;
}
