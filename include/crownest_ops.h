/*
 * crownest_ops.h - C ABI of the B200 (sm_100a) quantized GEMV / MoE decode kernels.
 *
 * Drop-in boundary for the reference engine's L3 operator layer: every entry point below replaces
 * one family of NVRTC kernels that the Rust host code launches through
 * `launch_v(f, gx, gy, gz, bx, &[u64])` (engine/src/kernels.rs:5296-5348). The conventions of
 * that boundary are kept:
 *   - every buffer argument is a DEVICE pointer owned by the caller; weights are borrowed;
 *   - work is enqueued on the caller's stream and the call returns at once: no allocation, no
 *     synchronisation, no host access to the buffers (so calls can be captured in a CUDA graph);
 *   - outputs are assigned, never accumulated into, unless stated.
 * Differences: shapes are plain ints instead of device int buffers, kernels are compiled ahead of
 * time for sm_100a, and errors come back as a status code (0 = ok) with a message in
 * cn_last_error_string() instead of a panic.
 *
 * NVFP4 matrix layout (engine/src/cpu_nvfp4.rs:8-15, engine/src/cnq.rs:1298-1308): [rows][k/64]
 * blocks of 36 bytes, row-major; a block is 4 UE4M3 scale bytes (one per 16 values) then 32 code
 * bytes, value idx in byte 4 + idx/2, low nibble = even idx. A scale byte 0x7F reads as 0x7E
 * (448) and bit 7 is ignored (engine/src/cpu_nvfp4.rs:88-105). k must be a multiple of 256 (rows
 * are then 16-byte multiples, the rule of engine/src/kernels_p2.rs:302-303) and `w` 16-byte
 * aligned.
 */
#ifndef CROWNEST_OPS_H
#define CROWNEST_OPS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* activation / output element type of a call */
#define CN_F32 0  /* the reference's own dtype (f32 in, f32 out) */
#define CN_BF16 1 /* bf16 in, bf16 out, f32 accumulation */
#define CN_BF16_IN_F32_OUT 2 /* cn_moe_nvfp4_run only: bf16 in, f32 out (partial sums of an expert-parallel rank) */

/* status codes */
#define CN_OK 0
#define CN_ERR_SHAPE 1   /* a shape or alignment the kernels do not take */
#define CN_ERR_CUDA 2    /* a CUDA runtime call failed; see cn_last_error_string() */
#define CN_ERR_LIMIT 3   /* a size beyond a documented maximum */
#define CN_ERR_DEVICE 4  /* a kernel reported a failed bounded wait (see cn_device_status) */

/* most activation rows one small-M call takes (reference: NVFP4_MMAX 4 for NVFP4,
 * engine/src/kernels_p2.rs:397; MUL1_MAXT 8, engine/src/kernels_mul1.cu:40) */
#define CN_MAX_M 8

typedef void* cn_stream_t; /* a cudaStream_t */

/* message of the last failing call on this thread ("" if none) */
const char* cn_last_error_string(void);

/* library build info, e.g. "crownest_b200 sm_100a" */
const char* cn_version(void);

/* Device-side error word: kernels never trap or spin for ever; a wait that runs out of its
 * iteration budget records a code here and the kernel returns. Reads and clears the word
 * (synchronises the device). 0 = no error. */
int cn_device_status(int* code_out);
/* Bookkeeping of the per-device kernel attribute (large dynamic shared memory) that every launch path consults: 1 when
 * (kernel, device) has not been allowed `bytes` yet (recorded when commit != 0), else 0. Makes no CUDA call; exported so
 * that the per-device rule can be checked without a GPU. */
int cn_smem_book(const void* kernel, int device, int bytes, int commit);

/* ---------------------------------------------------------------- NVFP4 GEMV, M = 1..8
 * y[m][r] = sum_k W[r][k] * x[m][k], m < M.
 * Replaces gemv_nvfp4_w (engine/src/kernels_p2.rs:355), its small-M form gemv_nvfp4_wm (:472,
 * reached through Engine::proj_m, engine/src/gen.rs:5455) and the record kernels gemv_fp4 /
 * gemv_fp4_b (engine/src/kernels.rs:118, :154) and glm5_gemv_fp4 (engine/src/kernels_glm5_moe.cu:284);
 * call sites PW::launch_gemv (engine/src/gen.rs:234-266), Engine::dense_proj (:3915).
 * x row m at x + m*k elements, y row m at y + m*ldy elements (ldy >= rows). gs: device pointer to
 * the f32 tensor scale. Row m of a call with M rows is bit-identical to a call with M = 1 on that
 * row (the batch invariance of engine/src/kernels_p2.rs:391-396). */
int cn_nvfp4_gemv(const void* w, const float* gs, const void* x, void* y, int rows, int k, int m, int ldy, int dtype,
                  cn_stream_t stream);

/* Fused gate/up GEMV + activation: h[m][i] = act(gs_g <gate_i, x_m>, gs_u <up_i, x_m>).
 * Replaces gemv_nvfp4_gu / gemv_nvfp4_gum (engine/src/kernels_p2.rs:372, :499; call sites
 * Engine::dense_ffn_w engine/src/gen.rs:3974, verify_kernels :5632).
 * act: limit <= 0 -> silu(g) * u; limit > 0 -> the clamped SwiGLU silu(min(g, l)) * clamp(u, -l, l)
 * (glm5_swiglu_clamp, engine/src/kernels_glm5_moe.cu:113). wg, wu: [inter][k] NVFP4. h row m at
 * h + m*ldh. */
int cn_nvfp4_gemv_gu(const void* wg, const void* wu, const float* gs_g, const float* gs_u, const void* x, void* h,
                     int inter, int k, int m, int ldh, float limit, int dtype, cn_stream_t stream);

/* A chain of one-row (bf16) NVFP4 GEMV steps in ONE persistent launch: the fused form of the decode step's
 * projection chain. Replaces the launch sequence of Engine::dense_ffn_w (engine/src/gen.rs:3974-3990: gemv_nvfp4_gu then
 * gemv_nvfp4_w), the FusedFfn operator (engine/src/kernels.rs:6777-6840) and, for a stack of projections, the launches of
 * Engine::decode_step (engine/src/gen.rs:6117-6190). The CTAs stay resident over all steps: weights of the next step are
 * already streaming while a step finishes, and every step's work is dealt to the CTAs in equal shares whatever its row
 * count. Step i: y = W x, or h = act(W x, W_up x) when w_up != null (limit as in cn_nvfp4_gemv_gu); x bf16 [k], y bf16
 * [rows] (f32 when out_f32). `after`: index of the earlier step whose output this step reads (it starts reading x only
 * once that step is complete on every CTA), -1 when x is ready before the launch. A step that overwrites a buffer an
 * earlier step reads must be ordered after it through `after` links. k a multiple of 256, k >= 2048.
 * The plan copies the descriptors to the device and owns the hand-over scratch (the only allocation; run() allocates
 * nothing and does not synchronise; the launch is cooperative). One run at a time per plan. After a device-side wait
 * has failed (cn_device_status) the plan's counters are undefined: destroy it. */
typedef struct cn_gemv_step {
    const void* w;      /* [rows][k] NVFP4, or gate */
    const void* w_up;   /* up (fused gate/up + activation), else null */
    const float* gs;    /* device f32 tensor scale of w */
    const float* gs_up; /* of w_up (null: gs) */
    const void* x;      /* bf16 [k] */
    void* y;            /* bf16 (or f32) [rows] */
    int rows, k;
    float limit;
    int after;
    int out_f32;
} cn_gemv_step;
int cn_nvfp4_seq_create(void** plan_out, const cn_gemv_step* steps, int nsteps);
int cn_nvfp4_seq_run(void* plan, cn_stream_t stream);
int cn_nvfp4_seq_destroy(void* plan);

/* Residual add + RMSNorm between the projections: h[r] += y[r] (y may be null), out[r] = h[r] * rsqrt(mean(h[r]^2) + eps) *
 * (1 + w). Replaces add_rms_1k (engine/src/kernels_p2.rs:609-633, Engine::add_norm). All f32; h is updated in place. */
int cn_add_rmsnorm(float* h, const float* y, const float* w, float* out, int rows, int hidden, float eps, cn_stream_t stream);

/* Token id of the largest logit per row, with the tie rule of argmax_k (engine/src/kernels.rs:4238-4261): 1024 strided
 * scanners keeping their first strict maximum, then a tree in which the lower scanner wins ties. logits [rows][ld >= n] in
 * `dtype`. cn_lm_head_argmax: the vocabulary GEMV (cn_nvfp4_gemv over w [vocab][k], m <= CN_MAX_M rows, logits [m][vocab] in
 * `dtype` kept for the caller's sampler) followed by that argmax (engine/src/gen.rs:5638-5641). */
int cn_argmax(const void* logits, int32_t* out, int rows, int n, int ld, int dtype, cn_stream_t stream);
int cn_lm_head_argmax(const void* w, const float* gs, const void* x, void* logits, int32_t* tokens, int vocab, int k, int m, int dtype,
                      cn_stream_t stream);

/* Bit-exact dequantisation self-check: out[r][c] f32 = e2m1(code) * (ue4m3(scale byte) * gs).
 * Replaces dequant_fp4_flat (engine/src/kernels.rs:1460), host twin cnq::dequant_block
 * (engine/src/cnq.rs:1298). rule != 0 reads 0x7F as 0x7E first (the GEMV's reading). */
int cn_nvfp4_dequant(const void* w, const float* gs, float* out, int rows, int k, int rule, cn_stream_t stream);

/* ---------------------------------------------------------------- MoE routing
 * Softmax top-k (Flash-Next): p = softmax(logits[t]); k rounds of "largest p, lowest index on
 * ties"; wts = p_j / (sum of the picked p, in pick order). Replaces the selection half of
 * router_top10 (engine/src/kernels.rs:3109-3171). logits [tokens][experts] f32; ids, wts
 * [tokens][k] in pick order. experts <= 1024, k <= 64. */
int cn_route_softmax_topk(const float* logits, int32_t* ids, float* wts, int tokens, int experts, int k, cn_stream_t stream);

/* Sigmoid top-k (GLM): s = sigmoid(logit); choice = s + bias (NaN -> -inf; bias may be null);
 * wts = s / (sum_picked s + 1e-20) * scale. Replaces glm5_router_sig_topk
 * (engine/src/kernels_glm5_moe.cu:44-96), host twin glm5_moe::route_from_logits
 * (engine/src/glm5_moe.rs:196-236). */
int cn_route_sigmoid_topk(const float* logits, const float* bias, int32_t* ids, float* wts, int tokens, int experts, int k,
                          float scale, cn_stream_t stream);

/* ---------------------------------------------------------------- routed NVFP4 experts
 * order[] = the combos 0..combos-1 sorted by expert id (stable; ids outside 0..experts-1 last).
 * The grouping step in front of the routed GEMVs; the reference's analogue is moe_count / moe_plan /
 * moe_scatter of its prefill path (engine/src/kernels.rs:3334-3420). */
int cn_moe_sort(const int32_t* ids, int32_t* order, int combos, int experts, cn_stream_t stream);

/* y[t] = base[t] + sum_j wts[t][j] * eo[t*topk + j], j in pick order; base = shared[t] (times
 * sigmoid(sgate[t]) when sgate != null), 0 when shared == null. A combo whose table entry is null
 * adds nothing (table may be null: every combo counts), and so does an id outside 0..experts-1 (experts = entries
 * of table; 0 = not checked). Replaces acc_combo + gate_shared
 * (engine/src/kernels.rs:1583-1599) and glm5_moe_combine (engine/src/kernels_glm5_moe.cu:141).
 * eo, shared f32; y in `dtype`. */
int cn_moe_combine(const float* eo, const float* wts, const int32_t* ids, const unsigned long long* table, const float* shared,
                   const float* sgate, void* y, int tokens, int hidden, int topk, int experts, int dtype, cn_stream_t stream);

/* The routed-expert decode step, GpuMoePlan-shaped (engine/src/glm5_moe.rs:518-793; Flash-Next call
 * site Engine::moe_run, engine/src/gen.rs:4168-4532). The plan owns the scratch (the only
 * allocation; run() allocates nothing and does not synchronise). The plan also owns one side stream
 * and two events: run() enqueues the shared expert there between a fork event recorded on `stream`
 * and a join event `stream` waits for before the combine, so everything is ordered with the caller's
 * stream as if it ran on it (a capture of `stream` takes the side branch in). cn_mul1_ffn and
 * cn_moe_mul1_run do the same with the up projection.
 * Tables are device arrays [experts] of device addresses (0 = expert not resident: its combos are
 * skipped, the contract of engine/src/kernels_mul1.cu:118-119; so are ids outside 0..experts-1). ids, order and the
 * tables must be complete when the call is enqueued or be written by earlier work on `stream`. table_gu = gate [inter][hidden], or
 * the fused gate|up slab [2*inter][hidden] when table_up == null; table_dn = down [hidden][inter].
 * gs_gu / gs_up / gs_dn: device f32 tensor scales shared by all experts (gs_up may be null = gs_gu).
 * shared_*: the shared expert's matrices (null = none) with shared_gs a device f32[3] (gate, up,
 * down); sgate: optional device f32 [tokens] gate logits of the shared expert (engine/src/kernels.rs:1593).
 * ids, wts [tokens][topk] from a router above; x, y [tokens][hidden] in `dtype`; CN_BF16_IN_F32_OUT
 * reads bf16 x and writes f32 y, for a rank that holds part of the experts (the other table entries
 * null) and hands its partial sums to a reduction across ranks. */
int cn_moe_nvfp4_plan_create(void** plan_out, int hidden, int inter, int shared_inter, int experts, int topk, int max_tokens);
int cn_moe_nvfp4_plan_destroy(void* plan);
int cn_moe_nvfp4_run(void* plan, const unsigned long long* table_gu, const unsigned long long* table_up,
                     const unsigned long long* table_dn, const float* gs_gu, const float* gs_up, const float* gs_dn,
                     const void* shared_gate, const void* shared_up, const void* shared_down, const float* shared_gs,
                     const float* sgate, const int32_t* ids, const float* wts, const void* x, void* y, int tokens, float limit,
                     int dtype, cn_stream_t stream);

/* The two halves of cn_moe_nvfp4_run for callers that put something between them (expert parallelism: the rows come from
 * other ranks and the results go back to them). cn_moe_nvfp4_experts: routed gate|up + activation and routed down over
 * `combos` rows, combo c reading activation row c / x_div of x and writing f32 row c of eo - or to the address eo_ptrs[c]
 * when eo_ptrs != null (a row of any device-visible buffer, a peer GPU's included); ids[c] < 0, beyond the tables or with
 * a null table entry skips the combo. The plan needs max_tokens * topk >= combos. cn_moe_nvfp4_finish: the shared expert
 * on x (when given) and y[t] = shared[t] + sum_j wts[t][j] * eo[t * topk + j] over the plan's top-k, `table` as in
 * cn_moe_combine (null: every combo counts). cn_moe_nvfp4_shared_begin enqueues the shared expert early, on the plan's
 * side stream, so that it runs beside whatever the caller puts on `stream` next (an exchange between ranks); the next
 * cn_moe_nvfp4_finish on the plan then joins it instead of computing it (its shared_* arguments are ignored). */
int cn_moe_nvfp4_shared_begin(void* plan, const void* shared_gate, const void* shared_up, const void* shared_down, const float* shared_gs,
                              const void* x, int tokens, float limit, int dtype, cn_stream_t stream);
int cn_moe_nvfp4_experts(void* plan, const unsigned long long* table_gu, const unsigned long long* table_up,
                         const unsigned long long* table_dn, const float* gs_gu, const float* gs_up, const float* gs_dn,
                         const int32_t* ids, const void* x, float* eo, const unsigned long long* eo_ptrs, int combos, int x_div, float limit,
                         int dtype, cn_stream_t stream);
int cn_moe_nvfp4_finish(void* plan, const void* shared_gate, const void* shared_up, const void* shared_down, const float* shared_gs,
                        const float* sgate, const int32_t* ids, const float* wts, const unsigned long long* table, const void* x,
                        const float* eo, void* y, int tokens, float limit, int dtype, cn_stream_t stream);

/* ---------------------------------------------------------------- NVFP4 GEMM (prefill / batched rows)
 * Y[t][n] = gs * sum_k X[t][k] * W[n][k] for any m >= 1 activation rows (meant for m > 8; up to 8 rows
 * cn_nvfp4_gemv streams the weights once and is faster), on tcgen05 tensor cores with the accumulator in
 * tensor memory. Replaces gemm_fp4_dense (engine/src/kernels.rs:533, launched by launch_mma_d,
 * engine/src/gen.rs:2491) and glm5_gemm_fp4_tc (engine/src/kernels_glm5_moe.cu:349), with the latter's
 * arithmetic: weights widened losslessly to f16 (code x block scale), activations as f16 x 2^k per row,
 * exact products, f32 accumulation. w is the container layout, unchanged. The call allocates nothing:
 * `workspace` (device, 256-byte aligned) holds the widened activations and must be at least
 * cn_nvfp4_gemm_workspace_bytes(k, m) bytes; it may be reused by the next call on the same stream. */
size_t cn_nvfp4_gemm_workspace_bytes(int k, int m);
int cn_nvfp4_gemm(const void* w, const float* gs, const void* x, void* y, int rows, int k, int m, int ldy, int dtype, void* workspace,
                  size_t workspace_bytes, cn_stream_t stream);

/* The same product on the block-scaled FP4 tensor-core path: tcgen05.mma kind::mxf4nvf4 (both operands E2M1 with one
 * UE4M3 scale per 16 values, f32 accumulation in tensor memory). Replaces gemm_fp4_dense / gemm_fp4_dense_b
 * (engine/src/kernels.rs:533, :642) and quant_x_fp4 / quant_row_prescaled (:264-351, host twin act_cascade :5354-5475).
 * The weights are re-laid once at load (cn_nvfp4_bs_repack into cn_nvfp4_bs_packed_bytes bytes, 16-byte aligned: tiles of
 * 128 rows x 256 columns in the tensor core's shared-memory layout, scale byte 0x7F -> 0x7E and bit 7 cleared as the
 * reference does at load, engine/src/residency.rs:119-137). The activations of every call go through the reference's
 * cascade - a per-row power of two times a sum of NVFP4 levels, each coding the residual of the ones before - with five
 * levels instead of the reference's three (three leave 8e-4 relative L2, inside 1e-3 but tens of bf16 ulp on small outputs;
 * each level buys a factor of about 16). The levels of a token ride as columns of the MMA and are added in the epilogue.
 * k a multiple of 256; workspace (256-byte aligned, cn_nvfp4_bs_workspace_bytes) holds the cascade and, for few rows, the
 * partial sums of a split K range. Meant for 16 < m <= a few hundred rows, where it streams the weights near HBM speed;
 * for thousands of rows cn_nvfp4_gemm is as fast. cn_nvfp4_act_cascade exposes the cascade alone in the reference's byte
 * layout ([rows][levels * k/64 * 36 + 4]; level L at L * k/64 * 36, then the f32 factor 2^-k), bit-identical to the
 * reference's host twin; levels 1..8. */
size_t cn_nvfp4_bs_packed_bytes(int rows, int k);
int cn_nvfp4_bs_repack(const void* w, void* packed, int rows, int k, cn_stream_t stream);
size_t cn_nvfp4_bs_workspace_bytes(int rows, int k, int m);
int cn_nvfp4_bs_gemm(const void* packed, const float* gs, const void* x, void* y, int rows, int k, int m, int ldy, int dtype, void* workspace,
                     size_t workspace_bytes, cn_stream_t stream);
int cn_nvfp4_act_cascade(const void* x, void* out, int rows, int k, int levels, int dtype, cn_stream_t stream);

/* ---------------------------------------------------------------- EXL3 "MUL1" trellis experts
 * A record holds one expert (converter/src/mul1.rs:30-34, engine/src/cpu_mul1.rs:7-12):
 * [gate.trellis][up.trellis][down.trellis][gate.suh][gate.svh][up.suh][up.svh][down.suh][down.svh],
 * gate/up [hidden -> inter], down [inter -> hidden], bitrate K = bits (+0.5 when half), records
 * 16-byte aligned. ptrs: device array [slots] of record addresses, 0 = skip the slot
 * (engine/src/kernels_mul1.cu:118-119). The plan owns the scratch (transformed activations and the
 * k-split partial sums); run calls allocate nothing. Replaces mul1::GemvPlan / FfnPlan / FusedFfn
 * (engine/src/kernels.rs:6644-6850) and their kernels (engine/src/kernels_mul1.cu:114-700). */
int cn_mul1_plan_create(void** plan_out, int hidden, int inter, int bits, int half, int max_slots, int max_t);
int cn_mul1_plan_destroy(void* plan);

/* y[slot][t] = x[slot / x_div][t] W for matrix `which` of each slot's record (0 gate, 1 up, 2 down);
 * x [slots / x_div][t][k], y [slots][t][n] in `dtype`; t <= 8. GemvPlan::run_slots
 * (engine/src/kernels.rs:6683-6717), CPU twin cpu_mul1::gemv (engine/src/cpu_mul1.rs:1626). */
int cn_mul1_gemv(void* plan, int which, const unsigned long long* ptrs, const void* x, void* y, int slots, int t, int x_div,
                 int dtype, cn_stream_t stream);

/* y[slot][t] = down(act(gate x, up x)), act = silu(g) * u, or the clamped SwiGLU when limit > 0.
 * FfnPlan / FusedFfn (engine/src/kernels.rs:6731-6850), CPU twin cpu_mul1::expert_ffn
 * (engine/src/cpu_mul1.rs:1665) / glm5_moe::expert_ffn_mul1_cpu (engine/src/glm5_moe.rs:280). */
int cn_mul1_ffn(void* plan, const unsigned long long* ptrs, const void* x, void* y, int slots, int t, int x_div, float limit,
                int dtype, cn_stream_t stream);

/* The GLM-style routed step over MUL1 experts: ptrs[c] = table[ids[c]] (glm5_moe_gather), one slot
 * per (token, rank) combo, the FFN of every slot, then y[t] = sum_j wts[t][j] * eo[t*topk + j] +
 * shared[t] (shared: optional f32 [tokens][hidden], e.g. the NVFP4 shared expert's output).
 * GpuMoePlan::experts (engine/src/glm5_moe.rs:741-793). The plan needs max_slots >= tokens * topk. experts = entries of
 * table: an id outside 0..experts-1 is skipped like a null entry (0 = ids are not checked). */
int cn_moe_mul1_run(void* plan, const unsigned long long* table, const int32_t* ids, const float* wts, const float* shared,
                    const void* x, void* y, int tokens, int topk, int experts, float limit, int dtype, cn_stream_t stream);

/* The expert half of cn_moe_mul1_run alone: eo[c] (f32 [combos][hidden], caller's buffer) = FFN of expert ids[c] on
 * activation row c / x_div; the combine is cn_moe_combine. For expert parallelism (rows from other ranks). */
int cn_moe_mul1_experts(void* plan, const unsigned long long* table, const int32_t* ids, const void* x, float* eo, int combos, int x_div,
                        int experts, float limit, int dtype, cn_stream_t stream);

/* The MUL1 GEMV of cn_mul1_gemv without a plan and without any allocation: for a caller that cannot
 * allocate device memory where it makes the call (a decode loop that must not hit the device-wide
 * synchronisation an allocation implies, a host that hands out all device memory at start-up, a
 * plugin sandbox that forbids it). Its scratch is a fixed array of about 2.2 MB inside the library
 * image, which every GPU that loads the library keeps until the process exits.
 * This entry point has no counterpart in the reference (there every plan allocates its scratch,
 * engine/src/kernels.rs:6664).
 * Limits, refused with CN_ERR_LIMIT beyond them: slots * t <= CN_MUL1_STATIC_ROWS activation rows,
 * hidden and inter <= CN_MUL1_STATIC_DIM. Same arguments and results as cn_mul1_gemv (bit for bit).
 * The first call on each device looks up the array's device address (with that device current); make
 * that first call outside any stream capture. All calls on a device share the one array, which keeps
 * the previous call's contents (each call overwrites what it reads, nothing needs clearing): two calls
 * whose kernels can overlap on the GPU - different streams without ordering - race on it. */
#define CN_MUL1_STATIC_ROWS 8
#define CN_MUL1_STATIC_DIM 4096
int cn_mul1_gemv_noalloc(int which, int hidden, int inter, int bits, int half, const unsigned long long* ptrs, const void* x, void* y,
                         int slots, int t, int x_div, int dtype, cn_stream_t stream);

/* W_hat [k][n] as fp16 bits from a trellis (the codec self-check; converter/src/mul1.rs:177-195
 * `reconstruct`, GPU test mul1_gpu_weight_equals_codec engine/src/kernels.rs:7076). */
int cn_mul1_reconstruct(const void* trellis, void* w_out, int k, int n, int bits, int half, cn_stream_t stream);

/* ---------------------------------------------------------------- FP8 (E4M3FN) GEMV, M = 1..8
 * y[m][r] = sum over 128-column tiles cb of (sum_{k in tile} e4m3(q[r][k]) * x[m][k]) * scale[r/128][cb].
 * w: [rows][cols] E4M3FN bytes; scale: f32 [ceil(rows/128)][ceil(cols/128)], the codec's block grid
 * (converter/src/fp8.rs:44-82 `dequant_fp8_block`; byte decode engine/src/cnq.rs:1363-1376). The
 * reference has this codec but no FP8 GEMV; this entry point defines one on it. cols % 16 == 0.
 * f32 activations are rounded to f16 (11 bits) when staged; bf16 activations are exact. */
int cn_fp8_gemv(const void* w, const float* scale, const void* x, void* y, int rows, int cols, int m, int ldy, int dtype,
                cn_stream_t stream);

/* ---------------------------------------------------------------- expert-parallel token exchange over peer memory
 * No counterpart in the reference (single GPU); it stands where glm5_moe_gather / glm5_moe_combine
 * (engine/src/kernels_glm5_moe.cu:101-156) gather rows for the expert kernels and sum their outputs. Expert e lives on rank
 * e / (experts / world). Every rank holds one buffer of the same layout, opened by all peers (cn_peer_export / cn_peer_open),
 * zero before the first use:
 *   inbox_x    [world][cap][hidden] bf16, inbox_meta [world][cap] {i32, i32}, ret [cap][hidden] f32, flags cn_ep_flag_bytes()
 * cap = the most combos a rank sends per step (its tokens x top-k; the same on every rank).
 * cn_ep_dispatch: all-to-all dispatch. Pushes activation row c / topk (bf16) of every local combo c to the rank that owns
 * expert ids[c] (order = the combos sorted by expert, from cn_moe_sort), meets the other ranks, and fills for the routed
 * kernels ids_in [world * cap] (expert of every inbox slot, -1 = empty) and out_ptrs [world * cap] (where that slot's
 * result goes: row c of the source rank's ret). The inbox rows are then the x of cn_moe_nvfp4_experts / cn_moe_mul1_experts
 * with x_div = 1.
 * cn_ep_return: all-to-all return. With eo != null copies result row i of eo [world * cap][hidden] f32 to out_ptrs[i] first
 * (not needed when the expert kernel stored there itself); then meets the other ranks: afterwards ret holds the f32 output of
 * every local combo, ready for cn_moe_combine / cn_moe_nvfp4_finish with the rank's own ids and weights - the same sum in
 * the same order as on one GPU. Two launches per call at most, graph-capturable, bounded waits; world <= 8. */
size_t cn_ep_flag_bytes(void);
int cn_ep_dispatch(const void* const* peer_bases, int rank, int world, int cap, int hidden, size_t inbox_x, size_t inbox_meta, size_t ret,
                   size_t flags, const int32_t* ids, const int32_t* order, const void* x, int combos, int topk, int experts,
                   int32_t* ids_in, unsigned long long* out_ptrs, cn_stream_t stream);
int cn_ep_return(const void* const* peer_bases, int rank, int world, int cap, int hidden, size_t inbox_x, size_t inbox_meta, size_t ret,
                 size_t flags, const float* eo, const int32_t* ids_in, const unsigned long long* out_ptrs, cn_stream_t stream);

/* ---------------------------------------------------------------- tensor-parallel exchange over peer memory
 * No counterpart in the reference (it is single-GPU). Every rank holds one buffer of the same layout; a rank
 * exports its buffer (cn_peer_export: a 64-byte CUDA IPC handle of the allocation and the buffer's offset in it),
 * the others open it (cn_peer_open) and pass all base pointers, their own included, to cn_tp_allgather:
 * the rank's slice [data_off + rank * slice_bytes, + slice_bytes) is stored into every peer's buffer at the same
 * place, then the ranks meet on the arrival counters at flag_off (36 bytes, zero before the first use, one flag
 * block per exchange point). One launch, graph-capturable; the wait is bounded. Offsets and sizes in multiples of
 * 16 bytes; world <= 8. */
int cn_peer_export(const void* ptr, void* handle64, size_t* offset);
int cn_peer_open(const void* handle64, size_t offset, void** ptr);
int cn_peer_close(void* ptr, size_t offset);
int cn_tp_allgather(const void* const* peer_bases, int rank, int world, size_t data_off, size_t slice_bytes, size_t flag_off,
                    cn_stream_t stream);
/* The same exchange as 16-byte lines {word, sequence number, word, sequence number} through a line buffer at line_off
 * (2 x world x 2 x slice_bytes bytes in every rank's buffer, zero before the first use): no flag has to wait for the
 * data to be acknowledged, so an exchange is one trip over NVLink; meant for slices of a few KB. The result in [data_off, + world * slice_bytes) is the same
 * bytes; flag_off as above (only its sequence counter is used). */
int cn_tp_allgather_ll(const void* const* peer_bases, int rank, int world, size_t data_off, size_t slice_bytes, size_t line_off,
                       size_t flag_off, cn_stream_t stream);
/* The exchange fused into the GEMV that produces the slice (no counterpart in the reference). cn_nvfp4_gemv_lines /
 * cn_nvfp4_gemv_gu_lines are cn_nvfp4_gemv / cn_nvfp4_gemv_gu for one bf16 activation row (y / h hold `rows` / `inter`
 * values) whose epilogue also stores the output rows as lines into the other ranks' line buffers: line_bases[r] is the
 * device address of rank r's line buffers of this vector (0 for the calling rank), row0 the global index of the call's
 * first output row (rows and row0 multiples of 4), line_stride the bytes between a rank's two line buffers
 * (world x 2 x slice_bytes). The number a line carries is *epoch x 4096 + tag: epoch is the rank's step counter, which
 * cn_tp_epoch_advance increments once at the start of every step (all ranks run the same steps), tag (1..4095) names the
 * exchange within the step and is the same on every rank. The lines go to buffer buf ^ (flip & *epoch & 1): consecutive
 * exchanges of a vector must alternate between its two buffers (a peer can be one exchange ahead, never two), also across
 * steps, so a vector that is exchanged an odd number of times per step passes flip = 1.
 * cn_tp_recv_lines is the receiving half on every rank, with the same tag / buf / flip: it polls the rank's own line
 * buffer for the peers' slices and writes them into [data_off, ...). It lets its successor in the stream start at once
 * and waits for its predecessor only before it ends, so it is enqueued right behind the producing GEMV; the wait for the
 * peers is bounded. */
int cn_tp_epoch_advance(void* epoch, cn_stream_t stream);
int cn_nvfp4_gemv_lines(const void* w, const float* gs, const void* x, void* y, int rows, int k, const unsigned long long* line_bases, int world,
                        int row0, size_t line_stride, const unsigned int* epoch, int tag, int buf, int flip, cn_stream_t stream);
int cn_nvfp4_gemv_gu_lines(const void* wg, const void* wu, const float* gs_g, const float* gs_u, const void* x, void* h, int inter, int k,
                           float limit, const unsigned long long* line_bases, int world, int row0, size_t line_stride,
                           const unsigned int* epoch, int tag, int buf, int flip, cn_stream_t stream);
int cn_tp_recv_lines(void* base, int rank, int world, size_t data_off, size_t slice_bytes, size_t line_off, const void* epoch, int tag,
                     int buf, int flip, cn_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
