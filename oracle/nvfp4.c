/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement of the reference engine's NVFP4 path, used only as the checker for the CUDA
 * kernels (tests, the smoke check) and as the timed CPU baseline of the benchmark. Nothing the
 * library ships calls into this file.
 *
 * The reference implementation is Rust and cannot be compiled in this environment (no Rust
 * toolchain), so this is a port: every function names the reference lines it follows.
 * Parity pins: the reference's Python block decoder (oracle/cnq_weights.py) run on the
 * reference's own container fixture, and the HF-computed dense-FFN golden of
 * engine/tests/fixtures/glm5/moe (see tests/golden).
 *
 * Format (engine/src/cpu_nvfp4.rs:8-15): an NVFP4 matrix [rows][cols] is rows * cols / 64 blocks
 * of 36 bytes, row-major. A block is 4 UE4M3 scale bytes (one per 16 values) followed by 32 code
 * bytes; value idx sits in byte 4 + idx / 2, low nibble for even idx.
 *
 * Build: see oracle/Makefile (-ffp-contract=off: the reference never contracts a*b+c).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(__AVX2__)
#include <immintrin.h>
#endif

void cn_o_pool_run(void* (*fn)(void*), void* jobs, size_t stride, int n);

#define CN_BLOCK_BYTES 36
#define CN_BLOCK_VALUES 64
#define CN_TOK_TILE 4

/* engine/src/cnq.rs:1241-1245 (`e2m1`) and engine/src/cpu_nvfp4.rs:52 (table) */
static const float E2M1_TABLE[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                     -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

float cn_o_e2m1(uint32_t nibble) { return E2M1_TABLE[nibble & 0xF]; }

/* engine/src/cnq.rs:1287-1295 (`ue4m3`): bit 7 is ignored, e == 0 is the subnormal m * 2^-9 */
float cn_o_ue4m3(uint32_t byte) {
    uint32_t e = (byte >> 3) & 0xF, m = byte & 0x7;
    if (e == 0) return (float)m * 1.953125e-3f;
    return (1.0f + (float)m / 8.0f) * ldexpf(1.0f, (int)e - 7);
}

/* engine/src/cpu_nvfp4.rs:88-96 (`scale_rule`): 0x7F (the E4M3 NaN code) reads as 0x7E (448) */
uint8_t cn_o_scale_rule(uint8_t byte) { return byte == 0x7F ? 0x7E : byte; }

/* engine/src/cpu_nvfp4.rs:98-105 (`scale_lut`) */
void cn_o_scale_lut(float gs, float lut[256]) {
    for (int b = 0; b < 256; b++) lut[b] = cn_o_ue4m3(cn_o_scale_rule((uint8_t)b)) * gs;
}

/* engine/src/cnq.rs:1298-1308 (`dequant_block`): raw scale bytes, no 0x7F rule */
void cn_o_dequant_block(const uint8_t* blk, float gs, float out[64]) {
    for (int sb = 0; sb < 4; sb++) {
        float s = cn_o_ue4m3(blk[sb]) * gs;
        for (int j = 0; j < 16; j++) {
            int idx = sb * 16 + j;
            uint8_t byte = blk[4 + (idx >> 1)];
            uint32_t nib = (idx & 1) ? ((byte >> 4) & 0xF) : (byte & 0xF);
            out[idx] = cn_o_e2m1(nib) * s;
        }
    }
}

/* Whole-matrix dequant: `dequant_block` over every block; `rule` != 0 applies the 0x7F -> 0x7E
 * rule first (what the GEMV reads, engine/src/cpu_nvfp4.rs:12-15). out is [rows][cols] f32. */
void cn_o_nvfp4_dequant(const uint8_t* w, int64_t rows, int64_t cols, float gs, int rule, float* out) {
    int64_t nblk = rows * (cols / CN_BLOCK_VALUES);
    for (int64_t b = 0; b < nblk; b++) {
        uint8_t tmp[CN_BLOCK_BYTES];
        memcpy(tmp, w + b * CN_BLOCK_BYTES, CN_BLOCK_BYTES);
        if (rule)
            for (int i = 0; i < 4; i++) tmp[i] = cn_o_scale_rule(tmp[i]);
        cn_o_dequant_block(tmp, gs, out + b * CN_BLOCK_VALUES);
    }
}

/* engine/src/cpu_nvfp4.rs:182-197 (`lane_pos`, `permute`): per 16 values, evens then odds */
static inline int64_t lane_pos(int64_t j) {
    int64_t k = j & 15;
    return (j & ~(int64_t)15) | ((k & 1) == 0 ? (k >> 1) : 8 + (k >> 1));
}

static float* permute_x(const float* x, int64_t tokens, int64_t cols) {
    float* xp = (float*)malloc(sizeof(float) * (size_t)(tokens * cols));
    for (int64_t t = 0; t < tokens; t++)
        for (int64_t j = 0; j < cols; j++) xp[t * cols + lane_pos(j)] = x[t * cols + j];
    return xp;
}

/* engine/src/cpu_nvfp4.rs:205-235 (`row_scalar`): 8 lane accumulators per token; per 16-value
 * sub-block p = lo * x[l] + hi * x[8 + l] then acc[l] += p * s, every operation rounded on its
 * own; the row result is acc[0] + ... + acc[7] left to right. */
static void row_scalar(const uint8_t* row, const float* lut, const float* xp, int64_t cols, int64_t t0, int nt,
                       float* out) {
    float acc[CN_TOK_TILE][8];
    memset(acc, 0, sizeof acc);
    int64_t bpr = cols / CN_BLOCK_VALUES;
    for (int64_t b = 0; b < bpr; b++) {
        const uint8_t* blk = row + b * CN_BLOCK_BYTES;
        for (int sb = 0; sb < 4; sb++) {
            float s = lut[blk[sb]];
            const uint8_t* codes = blk + 4 + sb * 8;
            float lo[8], hi[8];
            for (int l = 0; l < 8; l++) {
                lo[l] = E2M1_TABLE[codes[l] & 0xF];
                hi[l] = E2M1_TABLE[codes[l] >> 4];
            }
            int64_t base = b * CN_BLOCK_VALUES + sb * 16;
            for (int t = 0; t < nt; t++) {
                const float* x = xp + (t0 + t) * cols + base;
                for (int l = 0; l < 8; l++) {
                    float p = lo[l] * x[l] + hi[l] * x[8 + l];
                    acc[t][l] += p * s;
                }
            }
        }
    }
    for (int t = 0; t < nt; t++) {
        float r = 0.0f;
        for (int l = 0; l < 8; l++) r += acc[t][l];
        out[t] = r;
    }
}

#if defined(__AVX2__)
/* The same operations as `row_scalar`, eight lanes at a time (engine/src/cpu_nvfp4.rs:237-287
 * is the reference's AVX2 arm; the contract is bit-identity with the scalar arm). Magnitudes come
 * from an 8-entry register table, the sign from code bit 3. */
static void row_avx2(const uint8_t* row, const float* lut, const float* xp, int64_t cols, int64_t t0, int nt,
                     float* out) {
    const __m256 mags = _mm256_setr_ps(0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f);
    const __m256i nib_mask = _mm256_set1_epi32(0xF), sign_bit = _mm256_set1_epi32(0x8);
    __m256 acc[CN_TOK_TILE];
    for (int t = 0; t < CN_TOK_TILE; t++) acc[t] = _mm256_setzero_ps();
    int64_t bpr = cols / CN_BLOCK_VALUES;
    for (int64_t b = 0; b < bpr; b++) {
        const uint8_t* blk = row + b * CN_BLOCK_BYTES;
        for (int sb = 0; sb < 4; sb++) {
            __m256 s = _mm256_set1_ps(lut[blk[sb]]);
            __m256i c = _mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i*)(blk + 4 + sb * 8)));
            __m256i nlo = _mm256_and_si256(c, nib_mask), nhi = _mm256_srli_epi32(c, 4);
            __m256 wlo = _mm256_xor_ps(_mm256_permutevar8x32_ps(mags, nlo),
                                       _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_and_si256(nlo, sign_bit), 28)));
            __m256 whi = _mm256_xor_ps(_mm256_permutevar8x32_ps(mags, nhi),
                                       _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_and_si256(nhi, sign_bit), 28)));
            int64_t base = b * CN_BLOCK_VALUES + sb * 16;
            for (int t = 0; t < nt; t++) {
                const float* x = xp + (t0 + t) * cols + base;
                __m256 p = _mm256_add_ps(_mm256_mul_ps(wlo, _mm256_loadu_ps(x)), _mm256_mul_ps(whi, _mm256_loadu_ps(x + 8)));
                acc[t] = _mm256_add_ps(acc[t], _mm256_mul_ps(p, s));
            }
        }
    }
    for (int t = 0; t < nt; t++) {
        float lanes[8];
        _mm256_storeu_ps(lanes, acc[t]);
        float r = 0.0f;
        for (int l = 0; l < 8; l++) r += lanes[l];
        out[t] = r;
    }
}
#endif

/* path: 0 = scalar, 1 = AVX2 when compiled in (engine/src/cpu_nvfp4.rs:55-63 `Path`) */
int cn_o_have_avx2(void) {
#if defined(__AVX2__)
    return __builtin_cpu_supports("avx2") ? 1 : 0;
#else
    return 0;
#endif
}

static void row_dot(int path, const uint8_t* row, const float* lut, const float* xp, int64_t cols, int64_t t0, int nt,
                    float* out) {
#if defined(__AVX2__)
    if (path == 1) {
        row_avx2(row, lut, xp, cols, t0, nt, out);
        return;
    }
#endif
    (void)path;
    row_scalar(row, lut, xp, cols, t0, nt, out);
}

/* engine/src/cpu_nvfp4.rs:330-345 (`rows_into`): out[t * rows + r] */
static void rows_into(int path, const uint8_t* w, int64_t rows, int64_t cols, const float* lut, const float* xp,
                      int64_t tokens, int64_t r0, int64_t r1, float* out) {
    int64_t rb = cols / CN_BLOCK_VALUES * CN_BLOCK_BYTES;
    float tmp[CN_TOK_TILE];
    for (int64_t r = r0; r < r1; r++) {
        for (int64_t t0 = 0; t0 < tokens; t0 += CN_TOK_TILE) {
            int nt = (int)((tokens - t0) < CN_TOK_TILE ? (tokens - t0) : CN_TOK_TILE);
            row_dot(path, w + r * rb, lut, xp, cols, t0, nt, tmp);
            for (int t = 0; t < nt; t++) out[(t0 + t) * rows + r] = tmp[t];
        }
    }
}

typedef struct {
    int path;
    const uint8_t* w;
    int64_t rows, cols, tokens, r0, r1;
    const float *lut, *xp;
    float* out;
} gemv_job;

static void* gemv_worker(void* p) {
    gemv_job* j = (gemv_job*)p;
    rows_into(j->path, j->w, j->rows, j->cols, j->lut, j->xp, j->tokens, j->r0, j->r1, j->out);
    return NULL;
}

/* rows split over `threads` workers, worker w takes rows n*w/k .. n*(w+1)/k
 * (engine/src/cpu_nvfp4.rs:199-203 `split`, :349-373 `gemv`). Threads never split a sum, so the
 * bits do not depend on the thread count. */
static void gemv_xp(int path, const uint8_t* w, int64_t rows, int64_t cols, const float* lut, const float* xp,
                    int64_t tokens, float* y, int threads) {
    int k = threads < 1 ? 1 : threads;
    if (k > rows) k = rows > 0 ? (int)rows : 1;
    if (k == 1) {
        rows_into(path, w, rows, cols, lut, xp, tokens, 0, rows, y);
        return;
    }
    if (k > 257) k = 257; /* the pool's size */
    gemv_job* jobs = (gemv_job*)malloc(sizeof(gemv_job) * (size_t)k);
    for (int i = 0; i < k; i++) {
        gemv_job j = {path, w, rows, cols, tokens, rows * i / k, rows * (i + 1) / k, lut, xp, y};
        jobs[i] = j;
    }
    cn_o_pool_run(gemv_worker, jobs, sizeof(gemv_job), k); /* parked workers, not a thread start per call */
    free(jobs);
}

/* engine/src/cpu_nvfp4.rs:347-373 (`gemv`): y[t][r] = sum_k W[r][k] x[t][k]; x [T][cols] f32,
 * y [T][rows] f32. Returns 0, or -1 when cols is not whole 64-value blocks (the reference's
 * `Nvfp4Matrix::new` refusal, :122-131). */
int cn_o_nvfp4_gemv(const uint8_t* w, int64_t rows, int64_t cols, float gs, const float* x, int64_t tokens, float* y,
                    int threads, int path) {
    if (cols <= 0 || cols % CN_BLOCK_VALUES != 0) return -1;
    float lut[256];
    cn_o_scale_lut(gs, lut);
    float* xp = permute_x(x, tokens, cols);
    gemv_xp(path, w, rows, cols, lut, xp, tokens, y, threads);
    free(xp);
    return 0;
}

/* silu(g) * u = g / (1 + exp(-g)) * u  (engine/src/cpu_nvfp4.rs:19-20, :404) */
float cn_o_silu_mul(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

/* engine/src/glm5_moe.rs:138-151 (`swiglu_clamp`): gate clamped from above, up on both sides,
 * NaN kept (comparisons with NaN are false) */
float cn_o_swiglu_clamp(float g, float u, float l) {
    g = g > l ? l : g;
    u = u > l ? l : (u < -l ? -l : u);
    return (g / (1.0f + expf(-g))) * u;
}

/* engine/src/cpu_nvfp4.rs:375-427 (`expert_ffn`) with limit <= 0, and engine/src/glm5_moe.rs:
 * 269-278 (`ffn_nvfp4_cpu`, clamped SwiGLU) with limit > 0. gate, up [inter][hidden], down
 * [hidden][inter], each with its own global scale; x, y [T][hidden]. The fused and the staged
 * form are bit-identical in the reference (its test at :645), so this is the staged form. */
int cn_o_nvfp4_ffn(const uint8_t* gate, const uint8_t* up, const uint8_t* down, int64_t hidden, int64_t inter,
                   float gs_gate, float gs_up, float gs_down, float limit, const float* x, int64_t tokens, float* y,
                   int threads, int path) {
    if (hidden % CN_BLOCK_VALUES || inter % CN_BLOCK_VALUES) return -1;
    float* g = (float*)malloc(sizeof(float) * (size_t)(tokens * inter));
    float* u = (float*)malloc(sizeof(float) * (size_t)(tokens * inter));
    cn_o_nvfp4_gemv(gate, inter, hidden, gs_gate, x, tokens, g, threads, path);
    cn_o_nvfp4_gemv(up, inter, hidden, gs_up, x, tokens, u, threads, path);
    for (int64_t i = 0; i < tokens * inter; i++)
        g[i] = limit > 0.0f ? cn_o_swiglu_clamp(g[i], u[i], limit) : cn_o_silu_mul(g[i], u[i]);
    cn_o_nvfp4_gemv(down, hidden, inter, gs_down, g, tokens, y, threads, path);
    free(g);
    free(u);
    return 0;
}

/* The f64 reference of the reference's own tests (engine/src/cpu_nvfp4.rs:491-514): dequantize
 * with the f32 scale, accumulate w * x in f64; also returns sum |w x| for the Higham bound. */
void cn_o_nvfp4_gemv_f64(const uint8_t* w, int64_t rows, int64_t cols, float gs, int rule, const float* x,
                         int64_t tokens, double* y, double* yabs) {
    int64_t bpr = cols / CN_BLOCK_VALUES;
    for (int64_t r = 0; r < rows; r++) {
        for (int64_t t = 0; t < tokens; t++) {
            double s1 = 0.0, s2 = 0.0;
            for (int64_t b = 0; b < bpr; b++) {
                const uint8_t* blk = w + (r * bpr + b) * CN_BLOCK_BYTES;
                for (int idx = 0; idx < 64; idx++) {
                    uint8_t sbyte = blk[idx / 16];
                    if (rule) sbyte = cn_o_scale_rule(sbyte);
                    float s = cn_o_ue4m3(sbyte) * gs;
                    uint32_t nib = (blk[4 + idx / 2] >> (4 * (idx % 2))) & 0xF;
                    double p = (double)cn_o_e2m1(nib) * (double)s * (double)x[t * cols + b * 64 + idx];
                    s1 += p;
                    s2 += fabs(p);
                }
            }
            y[t * rows + r] = s1;
            if (yabs) yabs[t * rows + r] = s2;
        }
    }
}
