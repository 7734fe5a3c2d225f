// Host-side launch descriptor of the NVFP4 GEMV family, shared by the C entry points and the MoE operator.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

struct GemvCall {
    const void* w0;  // plain matrix, or gate
    const void* w1;  // up (fused gate/up form), else null
    const float* gs0;
    const float* gs1;
    const void* x;
    void* y;
    int rows, k, m, ldy;
    float limit;   // > 0: clamped SwiGLU in the gate/up form
    int dtype;     // CN_F32 or CN_BF16 activations
    int out_f32;   // store f32 whatever the activation type
    int x_f16_ok;  // f32 activations may be rounded to f16 (11 bits) at staging: the fast arithmetic path
    // routed-expert form: one launch over `combos` (token, rank) pairs, matrices from device pointer tables
    const int32_t* ids;
    const int32_t* order;
    const unsigned long long* tab0;
    const unsigned long long* tab1;
    int fused_up_rows, x_div, combos;
    int experts;  // entries of the tables (0 = unknown: ids are trusted); an id beyond them skips the combo
    const unsigned long long* yptrs;  // routed form: output row address per combo (null: y + combo * ldy); may name peer memory
    // Tensor-parallel line output (one bf16 activation row, plain or gate/up form): besides y, the output rows go out as
    // 16-byte lines {two rows, number, two rows, number} to the line buffers of the other ranks, where number =
    // *line_epoch * 4096 + line_tag and the buffer used is line_buf ^ (line_flip & *line_epoch & 1).
    // line_bases: host array [line_world] of device addresses (0 = this rank).
    const unsigned long long* line_bases;
    int line_world, line_row0;        // ranks; global index of output row 0 (a multiple of 4)
    size_t line_stride;               // bytes between the two line buffers of a rank
    const unsigned int* line_epoch;   // this rank's step counter (cn_tp_epoch_advance)
    int line_tag, line_buf, line_flip;
};

int cn_gemv_launch(const GemvCall& a, cudaStream_t stream, const char* who);

// One class of routed-expert groups (nvfp4_routed.cu): combos sorted by expert (order), groups of `mt` = 1 or up to 4
// consecutive positions of one expert (gpos, grows; grows null for one-row groups), their number on the device (gcount).
struct RoutedCall {
    const int32_t* ids;
    const int32_t* order;
    const int* gcount;
    const int* gpos;
    const int* grows;
    const unsigned long long* tab0;
    const unsigned long long* tab1;
    int fused_up_rows;
    const float* gs0;
    const float* gs1;
    const void* x;  // activation row of combo c: row c / x_div, bf16 (or f32 when x_f32)
    int x_div, x_f32;
    float* y;  // f32 row of combo c at y + c * ldy, or at yptrs[c]
    const unsigned long long* yptrs;
    int ldy, rows, k;
    float limit;
    int mt, max_groups;
};
int cn_routed_launch(const RoutedCall& a, cudaStream_t stream, const char* who);

// Sort combos by expert and cut every expert's run into groups (moe.cu): order [combos]; ga = positions (in order) of the
// one-row groups, counts[0] of them; gb / gbrows = positions and row counts (2..gmax, gmax 4 or 8) of the larger groups,
// counts[1]; gd / gdrows = the same runs cut into groups of one or two rows, counts[2]. Combos without a resident expert
// are in no group.
int cn_moe_group_launch(const int32_t* ids, const unsigned long long* tab, int combos, int experts, int32_t* order, int* ga, int* gb, int* gbrows,
                        int* gd, int* gdrows, int* counts, int gmax, cudaStream_t stream);

// Kernel-side parameters shared by the CUDA-core and the tensor-core GEMV kernels.
struct GemvParams {
    const uint8_t* w0;  // plain: the matrix; gate/up: gate
    const uint8_t* w1;  // gate/up: up (else null)
    const float* gs0;
    const float* gs1;
    const void* x;
    void* y;
    int rows;  // output rows (gate/up: inter)
    int k;
    int m;  // live activation rows (<= MP)
    int ldy;
    float limit;
    int tx;      // lanes across K per row: 16, 8 or 4
    int stages;  // ring depth
    int out_f32;  // store f32 whatever the activation type (MoE intermediates)
    // routed-expert form (ids != null): blockIdx.y walks the combos, combo c = t * topk + j reads the
    // matrix of expert ids[c] from a device pointer table (a null entry skips the combo), activation
    // row c / x_div, output row c
    const int32_t* ids;
    const int32_t* order;           // combos sorted by expert (null: identity)
    const unsigned long long* tab0;  // [experts] plain matrix or gate (or the fused gate|up slab)
    const unsigned long long* tab1;  // [experts] up (null with a fused slab or a plain matrix)
    int fused_up_rows;               // > 0: up = gate + fused_up_rows rows of the same slab
    int x_div;
    int experts;  // entries of tab0 / tab1 (0 = unknown); ids outside 0..experts-1 skip the combo
    const unsigned long long* yptrs;  // output row address per combo (null: y + combo * ldy)
    int red_depth;  // multi-row tensor-core kernel: tile-sum slots in flight
    int ksplit;     // 2: launched as two-CTA clusters, each CTA of a pair over half of K (one activation row only)
    // tensor-parallel line output (see GemvCall): line buffer of every rank (0 = none), first global row, the counter
    unsigned long long yl[8];
    int yl_world, yl_row0;
    unsigned long long yl_stride;
    const unsigned int* yl_epoch;
    int yl_tag, yl_buf, yl_flip;
#ifdef CN_M1_TRACE
    unsigned long long* trace;  // [8] globaltimer stamps per CTA of this launch (diagnostic build only), or null
#endif
};

__device__ __forceinline__ float act_gu(float g, float u, float limit) {
    if (limit > 0.0f) {
        g = g > limit ? limit : g;
        u = u > limit ? limit : (u < -limit ? -limit : u);
    }
    return (g / (1.0f + expf(-g))) * u;
}


// bf16 activation rows (1..8): persistent CTAs, tensor-core inner loop in word form (nvfp4_gemv_m1.cu)
int cn_gemv_m1_launch(const GemvCall& a, cudaStream_t stream, const char* who);
