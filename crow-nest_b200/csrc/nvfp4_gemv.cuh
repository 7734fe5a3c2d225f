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
};

int cn_gemv_launch(const GemvCall& a, cudaStream_t stream, const char* who);
