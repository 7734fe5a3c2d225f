/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement of the reference's EXL3 "MUL1" trellis codec and its exact-order CPU GEMV /
 * expert FFN, used only as the checker for the CUDA kernels and as the timed CPU baseline.
 * The reference implementation is Rust (not buildable here: no Rust toolchain), so this is a
 * port; every function names the reference lines it follows.
 *
 * Parity pins: the sha256 digests of exllamav3's own `reconstruct` output for seven experts
 * (converter/tests/fixtures/exl3-mul1-decode.tsv, four of them real quantizer records), the
 * all-65,536-state weight table, and the HF-computed MoE golden of engine/tests/fixtures/glm5/moe
 * (see tests/golden).
 *
 * Format (converter/src/mul1.rs:10-34, engine/src/cpu_mul1.rs:7-33): a linear [k = in, n = out]
 * is (k/16)(n/16) tiles of `wpt` u16 words (wpt = 16 K, +8 for half bitrates); tile (kb, nb) is
 * tile kb * n/16 + nb. A tile is a circular MSB-first bit stream over u32 words u16[2i] |
 * u16[2i+1] << 16; position p's 16-bit state is the window ending at bit end_bit(p). Position
 * 8 L + j sits at row 2 (L % 4) + {0,1,8,9}[j % 4], column L / 4 + 8 (j / 4).
 */
#include <math.h>
#include <pthread.h>
#include <stddef.h>

void cn_o_pool_run(void* (*fn)(void*), void* jobs, size_t stride, int n);
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define HAD 128
#define MUL1_MULT 0x83DCD12Du
static const int ROW_OFF[4] = {0, 1, 8, 9};

/* ---- bitrate (converter/src/mul1.rs:57-93, engine/src/cpu_mul1.rs:98-141) ---- */
/* bits = integer part, half = 1 for K + 0.5 */
int cn_o_mul1_words_per_tile(int bits, int half) { return 16 * bits + (half ? 8 : 0); }

int cn_o_mul1_end_bit(int bits, int half, int t) {
    if (!half) return (t + 1) * bits;
    if (t % 2 == 1) return (t / 2 + 1) * (2 * bits + 1);
    return (t / 2) * (2 * bits + 1) + bits;
}

/* ---- fp16 helpers (converter/src/mul1.rs:95-133, engine/src/cpu_mul1.rs:154-172) ---- */
static double f16_to_f64(uint16_t h) {
    double sign = (h & 0x8000) ? -1.0 : 1.0;
    int e = (h >> 10) & 0x1f;
    double m = (double)(h & 0x3ff);
    if (e == 0) return sign * m * ldexp(1.0, -24);
    if (e == 31) return m == 0.0 ? sign * INFINITY : NAN;
    return sign * (1024.0 + m) * ldexp(1.0, e - 25);
}

float cn_o_f16_to_f32(uint16_t h) { return (float)f16_to_f64(h); /* every fp16 value is exact in f32 */ }

static uint16_t f64_to_f16(double x) {
    uint16_t sign = signbit(x) ? 0x8000 : 0;
    double a = fabs(x);
    if (a == 0.0) return sign;
    if (a < ldexp(1.0, -14)) return sign | (uint16_t)nearbyint(a * ldexp(1.0, 24));
    int e;
    frexp(a, &e);
    e -= 1; /* a = f * 2^e with f in [1, 2) */
    uint32_t q = (uint32_t)nearbyint(a * ldexp(1.0, 10 - e));
    if (q == 2048) {
        q = 1024;
        e += 1;
    }
    if (e + 15 >= 31) return sign | 0x7c00;
    return sign | (uint16_t)((e + 15) << 10) | (uint16_t)(q - 1024);
}

uint16_t cn_o_f32_to_f16(float x) { return f64_to_f16((double)x); }

/* ---- codec (converter/src/mul1.rs:135-195) ---- */
/* `mul1_decode`: fp16 bits of one 16-bit state; x = state * 0x83DCD12D, sum = 0x6400 + the four
 * bytes, w = fma(half(sum), half(0x1eee), half(0xc931)) with one rounding */
uint16_t cn_o_mul1_decode(uint16_t state) {
    uint32_t x = (uint32_t)state * MUL1_MULT;
    uint32_t sum = 0x6400u + (x & 0xff) + ((x >> 8) & 0xff) + ((x >> 16) & 0xff) + (x >> 24);
    double h = f16_to_f64((uint16_t)sum);
    return f64_to_f16(h * f16_to_f64(0x1eee) + f16_to_f64(0xc931));
}

static int tile_index(int p) {
    int lane = p / 8, j = p % 8;
    int row = 2 * (lane % 4) + ROW_OFF[j % 4];
    int col = lane / 4 + 8 * (j / 4);
    return row * 16 + col;
}

static inline uint32_t state_at_words(const uint16_t* words, int n32, int lo) {
    int i = lo / 32, o = lo % 32, i1 = (i + 1) % n32;
    uint64_t a = (uint32_t)words[2 * i] | ((uint32_t)words[2 * i + 1] << 16);
    uint64_t b = (uint32_t)words[2 * i1] | ((uint32_t)words[2 * i1 + 1] << 16);
    return (uint32_t)((((a << 32) | b) >> (48 - o)) & 0xffff);
}

/* `decode_tile`: 256 fp16 bit patterns, row major */
void cn_o_mul1_decode_tile(const uint16_t* words, int bits, int half, uint16_t out[256]) {
    int wpt = cn_o_mul1_words_per_tile(bits, half), n32 = wpt / 2, s = wpt * 16;
    for (int p = 0; p < 256; p++) {
        int lo = (cn_o_mul1_end_bit(bits, half, p) + s - 16) % s;
        out[tile_index(p)] = cn_o_mul1_decode((uint16_t)state_at_words(words, n32, lo));
    }
}

/* `reconstruct`: the rotated weight W_hat [k][n] as fp16 bits, row major */
void cn_o_mul1_reconstruct(const uint16_t* trellis, int64_t k, int64_t n, int bits, int half, uint16_t* w) {
    int wpt = cn_o_mul1_words_per_tile(bits, half);
    uint16_t tile[256];
    for (int64_t kb = 0; kb < k / 16; kb++)
        for (int64_t nb = 0; nb < n / 16; nb++) {
            cn_o_mul1_decode_tile(trellis + (kb * (n / 16) + nb) * wpt, bits, half, tile);
            for (int r = 0; r < 16; r++) memcpy(w + (kb * 16 + r) * n + nb * 16, tile + r * 16, 32);
        }
}

/* `synth_words` of the fixtures (converter/src/mul1.rs:317-328) */
void cn_o_mul1_synth_words(uint16_t* out, int64_t count, uint32_t seed) {
    for (uint32_t i = 0; i < (uint32_t)count; i++) {
        uint32_t x = i * 0x9E3779B1u + seed * 0x85EBCA6Bu;
        x ^= x >> 15;
        x *= 0x2C1B3C6Du;
        x ^= x >> 12;
        out[i] = (uint16_t)(x & 0xffff);
    }
}

/* ---- the exact-order GEMV (engine/src/cpu_mul1.rs:35-48) ---- */
#define KINV (1774.0f / 262144.0f) /* fp16 0x1eee */
#define CAFF (-3.453125f)          /* 1024 * k_inv + fp16(0xc931) */

/* engine/src/cpu_mul1.rs:174-183 (`rne16`): one RNE rounding to fp16 precision */
static float rne16(float v) {
    double a = fabs((double)v);
    if (a == 0.0) return v;
    int e;
    frexp(a, &e);
    e -= 1;
    if (e < -14) e = -14;
    double ulp = ldexp(1.0, e - 10);
    return (float)(nearbyint((double)v / ulp) * ulp);
}

static float WEIGHT_LUT[1021];
static pthread_once_t weight_once = PTHREAD_ONCE_INIT;
static void weight_lut_init(void) {
    /* engine/src/cpu_mul1.rs:185-195 (`weight_lut`) */
    for (int s = 0; s <= 1020; s++) WEIGHT_LUT[s] = rne16((float)s * KINV + CAFF);
}

static inline int bytesum(uint32_t state) {
    uint32_t x = state * MUL1_MULT;
    return (int)((x & 0xff) + ((x >> 8) & 0xff) + ((x >> 16) & 0xff) + (x >> 24));
}

/* engine/src/cpu_mul1.rs:203-206 (`weight`): the codec weight as the scalar path decodes it */
float cn_o_mul1_weight(uint16_t state) {
    pthread_once(&weight_once, weight_lut_init);
    return WEIGHT_LUT[bytesum(state)];
}

/* engine/src/cpu_mul1.rs:457-474 (`fwht128`): natural order, stages h = 1..64, (a+b, a-b) */
void cn_o_fwht128(float* v) {
    for (int h = 1; h < HAD; h *= 2)
        for (int i = 0; i < HAD; i += 2 * h)
            for (int j = i; j < i + h; j++) {
                float a = v[j], b = v[j + h];
                v[j] = a + b;
                v[j + h] = a - b;
            }
}

typedef struct {
    const uint8_t* trellis; /* bytes of (k/16)(n/16) tiles */
    const uint8_t *suh, *svh; /* fp16 LE */
    int64_t k, n;
    int bits, half;
} mul1_mat;

static inline float scale_at(const uint8_t* v, int64_t i) {
    return cn_o_f16_to_f32((uint16_t)(v[2 * i] | (v[2 * i + 1] << 8)));
}

static inline uint32_t rd32(const uint8_t* t, int i) {
    return (uint32_t)t[4 * i] | ((uint32_t)t[4 * i + 1] << 8) | ((uint32_t)t[4 * i + 2] << 16) | ((uint32_t)t[4 * i + 3] << 24);
}

/* engine/src/cpu_mul1.rs:213-220 (`state_at`) */
static inline uint32_t state_at(const uint8_t* tile, int n32, int lo) {
    int i = lo >> 5, o = lo & 31;
    uint64_t a = rd32(tile, i), b = rd32(tile, i + 1 == n32 ? 0 : i + 1);
    return (uint32_t)((((a << 32) | b) >> (48 - o)) & 0xffff);
}

/* engine/src/cpu_mul1.rs:1503-1514 (`prep_block`) + :1489-1501 (`permute_block`):
 * xp[t][kb][q][j] = H(x * suh)[16 kb + 2 q + ROW_OFF[j % 4]] */
static void prep_all(const mul1_mat* m, const float* x, int64_t tokens, float* xp) {
    int64_t tk = m->k / 16;
    float v[HAD];
    for (int64_t t = 0; t < tokens; t++)
        for (int64_t b = 0; b < m->k / HAD; b++) {
            for (int r = 0; r < HAD; r++) v[r] = x[t * m->k + b * HAD + r] * scale_at(m->suh, b * HAD + r);
            cn_o_fwht128(v);
            for (int kl = 0; kl < 8; kl++)
                for (int q = 0; q < 4; q++)
                    for (int j = 0; j < 8; j++)
                        xp[(t * tk + b * 8 + kl) * 32 + q * 8 + j] = v[16 * kl + 2 * q + ROW_OFF[j % 4]];
        }
}

/* engine/src/cpu_mul1.rs:549-592 (`fold`, `unit_scalar`) for one tile column nb and every
 * token: per token 8 x 8 accumulators acc[C][j]; kb ascending, C 0..8, q 0..4, trellis lane
 * g = 4 C + q: acc[C][j] += w[j] * xp[t][kb][q][j] (product and sum rounded on their own);
 * column 16 nb + C = (a0 + a1) + (a2 + a3), column 16 nb + C + 8 the same over j = 4..7. */
static void tile_column(const mul1_mat* m, const int* lo, const float* xp, int64_t tokens, int64_t nb, float* raw) {
    int64_t tk = m->k / 16, tn = m->n / 16;
    int wpt = cn_o_mul1_words_per_tile(m->bits, m->half), tb = 2 * wpt, n32 = wpt / 2;
    float* acc = (float*)calloc((size_t)tokens * 64, sizeof(float));
    for (int64_t kb = 0; kb < tk; kb++) {
        const uint8_t* tile = m->trellis + (kb * tn + nb) * tb;
        for (int c = 0; c < 8; c++)
            for (int q = 0; q < 4; q++) {
                int g = 4 * c + q;
                float w[8];
                for (int j = 0; j < 8; j++) w[j] = WEIGHT_LUT[bytesum(state_at(tile, n32, lo[8 * g + j]))];
                for (int64_t t = 0; t < tokens; t++) {
                    const float* xv = xp + (t * tk + kb) * 32 + q * 8;
                    float* a = acc + t * 64 + c * 8;
                    for (int j = 0; j < 8; j++) a[j] += w[j] * xv[j];
                }
            }
    }
    for (int64_t t = 0; t < tokens; t++)
        for (int c = 0; c < 8; c++) {
            const float* a = acc + t * 64 + c * 8;
            raw[t * m->n + nb * 16 + c] = (a[0] + a[1]) + (a[2] + a[3]);
            raw[t * m->n + nb * 16 + c + 8] = (a[4] + a[5]) + (a[6] + a[7]);
        }
    free(acc);
}

typedef struct {
    const mul1_mat* m;
    const int* lo;
    const float* xp;
    int64_t tokens, nb0, nb1;
    float* raw;
} col_job;

static void* col_worker(void* p) {
    col_job* j = (col_job*)p;
    for (int64_t nb = j->nb0; nb < j->nb1; nb++) tile_column(j->m, j->lo, j->xp, j->tokens, nb, j->raw);
    return NULL;
}

/* engine/src/cpu_mul1.rs:1626-1663 (`gemv`): y[t] = x[t] W, W = diag(suh) H W_hat H diag(svh) /
 * 128. Input transform per 128-block, the tile columns (threads split columns, never a sum, so
 * the bits do not depend on the thread count), then per 128 outputs the FWHT, * 2^-7, * svh
 * (:1473-1487 `had_out_block`). x [T][k], y [T][n], f32. */
static int gemv_mat(const mul1_mat* m, const float* x, int64_t tokens, float* y, int threads) {
    if (m->k <= 0 || m->n <= 0 || m->k % HAD || m->n % HAD) return -1;
    pthread_once(&weight_once, weight_lut_init);
    int wpt = cn_o_mul1_words_per_tile(m->bits, m->half), s = wpt * 16;
    int lo[256];
    for (int p = 0; p < 256; p++) lo[p] = (cn_o_mul1_end_bit(m->bits, m->half, p) + s - 16) % s;
    int64_t tk = m->k / 16, tn = m->n / 16;
    float* xp = (float*)malloc(sizeof(float) * (size_t)(tokens * tk * 32));
    float* raw = (float*)malloc(sizeof(float) * (size_t)(tokens * m->n));
    prep_all(m, x, tokens, xp);
    int k = threads < 1 ? 1 : threads;
    if (k > tn) k = (int)tn;
    if (k > 257) k = 257; /* the pool's size */
    col_job* jobs = (col_job*)malloc(sizeof(col_job) * (size_t)k);
    for (int i = 0; i < k; i++) {
        col_job j = {m, lo, xp, tokens, tn * i / k, tn * (i + 1) / k, raw};
        jobs[i] = j;
    }
    /* parked workers (the reference's persistent pool, engine/src/cpu_mul1.rs:2114-2318), not a thread start per call */
    cn_o_pool_run(col_worker, jobs, sizeof(col_job), k);
    float v[HAD];
    for (int64_t t = 0; t < tokens; t++)
        for (int64_t b = 0; b < m->n / HAD; b++) {
            memcpy(v, raw + t * m->n + b * HAD, sizeof v);
            cn_o_fwht128(v);
            for (int i = 0; i < HAD; i++) y[t * m->n + b * HAD + i] = (v[i] * (1.0f / 128.0f)) * scale_at(m->svh, b * HAD + i);
        }
    free(jobs);
    free(xp);
    free(raw);
    return 0;
}

int cn_o_mul1_gemv(const uint8_t* trellis, const uint8_t* suh, const uint8_t* svh, int64_t k, int64_t n, int bits,
                   int half, const float* x, int64_t tokens, float* y, int threads) {
    mul1_mat m = {trellis, suh, svh, k, n, bits, half};
    return gemv_mat(&m, x, tokens, y, threads);
}

/* bytes of one record: three trellis + six fp16 scale vectors, rounded up to 4096
 * (converter/src/mul1.rs:221-231 `RecordLayout::new`, engine/src/cpu_mul1.rs:415-419) */
int64_t cn_o_mul1_trellis_bytes(int64_t k, int64_t n, int bits, int half) {
    return k / 16 * (n / 16) * 2 * cn_o_mul1_words_per_tile(bits, half);
}

int64_t cn_o_mul1_record_payload(int64_t hidden, int64_t inter, int bits, int half) {
    return 3 * cn_o_mul1_trellis_bytes(hidden, inter, bits, half) + 6 * (hidden + inter);
}

int64_t cn_o_mul1_record_bytes(int64_t hidden, int64_t inter, int bits, int half) {
    int64_t p = cn_o_mul1_record_payload(hidden, inter, bits, half);
    return (p + 4095) / 4096 * 4096;
}

extern float cn_o_silu_mul(float g, float u);
extern float cn_o_swiglu_clamp(float g, float u, float l);

/* One routed expert from its record (engine/src/cpu_mul1.rs:431-455 `from_record`: trellis of
 * gate, up, down, then gate.suh, gate.svh, up.suh, up.svh, down.suh, down.svh):
 * y = down(act(gate x, up x)), act = silu(g) * u (engine/src/cpu_mul1.rs:1665-1681
 * `expert_ffn`) or the clamped SwiGLU when limit > 0 (engine/src/glm5_moe.rs:280-290
 * `expert_ffn_mul1_cpu`). gate, up are [hidden -> inter], down [inter -> hidden]. */
int cn_o_mul1_expert_ffn(const uint8_t* rec, int64_t hidden, int64_t inter, int bits, int half, float limit,
                         const float* x, int64_t tokens, float* y, int threads) {
    int64_t tb = cn_o_mul1_trellis_bytes(hidden, inter, bits, half);
    const uint8_t* at = rec + 3 * tb;
    const uint8_t* gs = at; at += 2 * hidden;
    const uint8_t* gv = at; at += 2 * inter;
    const uint8_t* us = at; at += 2 * hidden;
    const uint8_t* uv = at; at += 2 * inter;
    const uint8_t* ds = at; at += 2 * inter;
    const uint8_t* dv = at;
    mul1_mat gate = {rec, gs, gv, hidden, inter, bits, half};
    mul1_mat up = {rec + tb, us, uv, hidden, inter, bits, half};
    mul1_mat down = {rec + 2 * tb, ds, dv, inter, hidden, bits, half};
    float* g = (float*)malloc(sizeof(float) * (size_t)(tokens * inter));
    float* u = (float*)malloc(sizeof(float) * (size_t)(tokens * inter));
    int rc = gemv_mat(&gate, x, tokens, g, threads);
    if (!rc) rc = gemv_mat(&up, x, tokens, u, threads);
    if (!rc) {
        for (int64_t i = 0; i < tokens * inter; i++)
            g[i] = limit > 0.0f ? cn_o_swiglu_clamp(g[i], u[i], limit) : cn_o_silu_mul(g[i], u[i]);
        rc = gemv_mat(&down, g, tokens, y, threads);
    }
    free(g);
    free(u);
    return rc;
}
