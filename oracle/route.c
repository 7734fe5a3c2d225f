/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement of the reference's MoE routing and combine steps, used only as the checker for
 * the CUDA kernels and inside the timed CPU baseline.
 *
 * Parity pins: the sigmoid router is pinned by the HF-computed goldens of
 * engine/tests/fixtures/glm5/moe (router-ids / router-weights, 64 + 4 rows) and by the
 * reference's tie / NaN / bias unit cases, all restated in tests. The softmax top-k router has
 * no CPU twin and no reproducible golden in the reference ("parity unpinned"): it restates the
 * device kernel's text.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

/* engine/src/glm5_moe.rs:132-136 (`sigmoid`) */
static inline float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

/* engine/src/glm5_moe.rs:196-236 (`route_from_logits`), device twin
 * engine/src/kernels_glm5_moe.cu:44-96: s = sigmoid(l); c = s + bias with NaN -> -inf; K times
 * the best untaken c, ties (and a row of -inf) to the lowest expert; w = s / (sum_picked s +
 * 1e-20) * scale, the sum taken in pick order. ids, wts are [T][K] in pick order. */
void cn_o_route_sigmoid_topk(const float* logits, const float* bias, int64_t tokens, int experts, int topk, float scale,
                             int32_t* ids, float* wts) {
    float* s = (float*)malloc(sizeof(float) * (size_t)experts);
    float* c = (float*)malloc(sizeof(float) * (size_t)experts);
    uint8_t* taken = (uint8_t*)malloc((size_t)experts);
    float* w = (float*)malloc(sizeof(float) * (size_t)topk);
    for (int64_t t = 0; t < tokens; t++) {
        const float* row = logits + t * experts;
        for (int i = 0; i < experts; i++) {
            s[i] = sigmoidf_(row[i]);
            float v = s[i] + (bias ? bias[i] : 0.0f);
            c[i] = isnan(v) ? -INFINITY : v;
            taken[i] = 0;
        }
        for (int j = 0; j < topk; j++) {
            int best = -1;
            for (int i = 0; i < experts; i++)
                if (!taken[i] && (best < 0 || c[i] > c[best])) best = i;
            taken[best] = 1;
            ids[t * topk + j] = best;
            w[j] = s[best];
        }
        float sum = 0.0f;
        for (int j = 0; j < topk; j++) sum += w[j];
        float den = sum + 1e-20f;
        for (int j = 0; j < topk; j++) wts[t * topk + j] = (w[j] / den) * scale;
    }
    free(s);
    free(c);
    free(taken);
    free(w);
}

/* The pairwise tree of the device reductions (engine/src/kernels.rs:3129-3132, :3143-3146):
 * for st = E/2, E/4, .., 1: red[e] op= red[e + st] for e < st. E is a power of two there; for
 * any other E the tree runs over the next power of two with the missing leaves absent. */
static float tree_reduce(float* red, int n, int is_max) {
    int p = 1;
    while (p < n) p <<= 1;
    for (int st = p / 2; st > 0; st >>= 1)
        for (int e = 0; e < st; e++)
            if (e + st < n) red[e] = is_max ? fmaxf(red[e], red[e + st]) : red[e] + red[e + st];
    return red[0];
}

/* engine/src/kernels.rs:3109-3171 (`router_top10`): p = exp(l - max) / sum (tree sums), then K
 * times: best = max p, pick = lowest index with p == best, retire it; w_j = p_j / (p_0 + .. +
 * p_{K-1}) with the sum taken in pick order. ids, wts are [T][K] in pick order. */
void cn_o_route_softmax_topk(const float* logits, int64_t tokens, int experts, int topk, int32_t* ids, float* wts) {
    float* p = (float*)malloc(sizeof(float) * (size_t)experts);
    float* red = (float*)malloc(sizeof(float) * (size_t)experts);
    float* ws = (float*)malloc(sizeof(float) * (size_t)topk);
    for (int64_t t = 0; t < tokens; t++) {
        const float* row = logits + t * experts;
        for (int i = 0; i < experts; i++) red[i] = row[i];
        float mx = tree_reduce(red, experts, 1);
        for (int i = 0; i < experts; i++) {
            p[i] = expf(row[i] - mx);
            red[i] = p[i];
        }
        float den = tree_reduce(red, experts, 0);
        for (int i = 0; i < experts; i++) p[i] = p[i] / den;
        float sum = 0.0f;
        for (int j = 0; j < topk; j++) {
            for (int i = 0; i < experts; i++) red[i] = p[i];
            float best = tree_reduce(red, experts, 1);
            int pick = experts;
            for (int i = 0; i < experts; i++)
                if (p[i] == best) {
                    pick = i;
                    break;
                }
            if (pick == experts) pick = 0; /* a NaN row: the device leaves the sentinel; keep indices valid */
            ids[t * topk + j] = pick;
            ws[j] = p[pick];
            sum += p[pick];
            p[pick] = -1.0f;
        }
        for (int j = 0; j < topk; j++) wts[t * topk + j] = ws[j] / sum;
    }
    free(p);
    free(red);
    free(ws);
}

/* engine/src/glm5_moe.rs:305-317 (`combine`, device `glm5_moe_combine`): y[t] = (sum_k w[t][k] *
 * ye[t*K + k]) + ys[t], k in pick order, the shared expert added last. ys may be NULL. */
void cn_o_moe_combine(int topk, int64_t tokens, int64_t hidden, const float* ye, const float* weights, const float* ys,
                      float* y) {
    for (int64_t t = 0; t < tokens; t++)
        for (int64_t j = 0; j < hidden; j++) {
            float acc = 0.0f;
            for (int k = 0; k < topk; k++) acc += weights[t * topk + k] * ye[(t * topk + k) * hidden + j];
            y[t * hidden + j] = ys ? acc + ys[t * hidden + j] : acc;
        }
}

/* The Flash-Next order (engine/src/kernels.rs:1583-1599, call sites engine/src/gen.rs:4360-4364,
 * :4531): the shared expert is the first writer, y = g * shared with g = sigmoid(sgate[t]) when a
 * gate is given (else y = shared), then y += sum_k w[t][k] * eo[t*K + k] in pick order. */
void cn_o_moe_acc_combo(int topk, int64_t tokens, int64_t hidden, const float* eo, const float* weights,
                        const float* shared, const float* sgate, float* y) {
    for (int64_t t = 0; t < tokens; t++)
        for (int64_t j = 0; j < hidden; j++) {
            float base = shared ? shared[t * hidden + j] : 0.0f;
            if (shared && sgate) base = (1.0f / (1.0f + expf(-sgate[t]))) * base;
            float acc = 0.0f;
            for (int k = 0; k < topk; k++) acc += weights[t * topk + k] * eo[(t * topk + k) * hidden + j];
            y[t * hidden + j] = base + acc;
        }
}

/* engine/src/kernels.rs:4238-4261 (`argmax_k`): 1024 workers, worker t scans i = t, t + 1024, .. keeping the first strict
 * maximum (start -3e38 at index 0), then a stride-halving tree where the upper worker's candidate replaces the lower one
 * only when strictly larger. NaN never compares larger. */
int32_t cn_o_argmax(const float* logits, int64_t n) {
    float rb[1024];
    int32_t ri[1024];
    for (int t = 0; t < 1024; t++) {
        float best = -3.0e38f;
        int32_t bi = 0;
        for (int64_t i = t; i < n; i += 1024)
            if (logits[i] > best) best = logits[i], bi = (int32_t)i;
        rb[t] = best, ri[t] = bi;
    }
    for (int st = 512; st > 0; st >>= 1)
        for (int t = 0; t < st; t++)
            if (rb[t + st] > rb[t]) rb[t] = rb[t + st], ri[t] = ri[t + st];
    return ri[0];
}

/* engine/src/kernels_p2.rs:609-633 (`add_rms_1k`): h += y (y may be null), out = h * rsqrt(mean(h^2) + eps) * (1 + w); the sum
 * of squares in the kernel's order: 1024 strided partial sums, xor-shuffle tree inside each group of 32, the 32 group sums
 * left to right. 1 / sqrtf stands in for the device's rsqrtf (2 ulp apart at most). */
void cn_o_add_rmsnorm(float* h, const float* y, const float* w, float* out, int64_t rows, int64_t hidden, float eps) {
    for (int64_t r = 0; r < rows; r++) {
        float* hp = h + r * hidden;
        float part[1024];
        for (int t = 0; t < 1024; t++) {
            float ss = 0.0f;
            for (int64_t i = t; i < hidden; i += 1024) {
                float v = hp[i];
                if (y) {
                    v = v + y[r * hidden + i];
                    hp[i] = v;
                }
                ss = ss + v * v;
            }
            part[t] = ss;
        }
        float red[32];
        for (int g = 0; g < 32; g++) {
            float v[32];
            for (int l = 0; l < 32; l++) v[l] = part[g * 32 + l];
            for (int o = 16; o > 0; o >>= 1) {
                float nv[32];
                for (int l = 0; l < 32; l++) nv[l] = v[l] + v[l ^ o];
                for (int l = 0; l < 32; l++) v[l] = nv[l];
            }
            red[g] = v[0];
        }
        float ss = 0.0f;
        for (int g = 0; g < 32; g++) ss = ss + red[g];
        const float rms = 1.0f / sqrtf(ss / (float)hidden + eps);
        for (int64_t i = 0; i < hidden; i++) out[r * hidden + i] = (hp[i] * rms) * (1.0f + w[i]);
    }
}
