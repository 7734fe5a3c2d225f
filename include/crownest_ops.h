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

/* Bit-exact dequantisation self-check: out[r][c] f32 = e2m1(code) * (ue4m3(scale byte) * gs).
 * Replaces dequant_fp4_flat (engine/src/kernels.rs:1460), host twin cnq::dequant_block
 * (engine/src/cnq.rs:1298). rule != 0 reads 0x7F as 0x7E first (the GEMV's reading). */
int cn_nvfp4_dequant(const void* w, const float* gs, float* out, int rows, int k, int rule, cn_stream_t stream);

/* diagnostics: select an inner-loop variant of the NVFP4 GEMV for A/B timing (0 = default) */
void cn_set_tuning(int key, int value);
#define CN_TUNE_GEMV_MODE 1 /* 0 default, 1 force f32 FMA path, 2 force f16 mixed-FMA path */
#define CN_TUNE_GEMV_RT 2   /* rows per thread: 0 heuristic, else 1, 2 or 4 */
#define CN_TUNE_GEMV_STAGES 3

#ifdef __cplusplus
}
#endif
#endif
