// EXL3 "MUL1" trellis GEMV / expert FFN on sm_100a: y = x W with W = diag(suh) H W_hat H diag(svh) / 128,
// W_hat decoded from the 16-bit trellis states in the inner loop.
//
// Supersedes mul1_had_in / mul1_gemv / mul1_gemv2 / mul1_had_out / mul1_act_had_in
// (engine/src/kernels_mul1.cu:114, :280, :553, :669, :688) behind the plan interface of
// kernels::mul1::GemvPlan / FfnPlan (engine/src/kernels.rs:6644-6850); CPU twin cpu_mul1::gemv
// (engine/src/cpu_mul1.rs:1626). Format: converter/src/mul1.rs:10-34.
//
// Three steps per GEMV, none of which writes a dequantised weight:
//   had_in   xh = H128(x * suh) per 128-block, stored f16 with a power-of-two scale per block
//   gemv     y' = xh W_hat over a k-split: each CTA owns 8 adjacent tile columns (128 outputs) and
//            k/(16 S) tile rows; the 768-byte run of 8 tiles per tile row arrives by 1-D bulk copy
//            (TMA) into a shared-memory ring; warp w decodes tile column w: lane g extracts its 8
//            states from a 64-bit window (compile-time shifts at K = 3), multiplies by 0x83DCD12D,
//            sums the bytes with dp4a (+0x6400 = the f16 pattern of 1024 + s), maps pairs through
//            one HFMA2 to the codec's f16 weights (bit-exact) and accumulates with f16 x f16 -> f32
//            mixed FMAs; partial sums of the k-split go to scratch
//   had_out  y = H128(sum of partials) / 128 * svh
// The inner loop is instruction-bound, not HBM-bound: about 7 issue slots per 3-bit weight.
// Three helpers restate reference text because their operation order defines the bits the parity contract asks for:
// fwht128 follows mul1_fwht128 (engine/src/kernels_mul1.cu:74-88: the stage order and the a+b / a-b pairing), out_block
// follows mul1_out_block (:98-110: partial sums left to right, then the transform, 1/128 and the scale), mul1_pair follows
// the first half of mul1_w2 (:500-510: the multiply-hash byte sum and the f16 FMA constants of the codec).
#include "common.cuh"
#include "nvfp4_gemv.cuh"

namespace {

constexpr int MUL1_MAXT = CN_MAX_M;  // activation rows per slot
constexpr int MUL1_GT = 8;           // most rows of a group when the MoE step bundles the combos of an expert (groups of 4 or 8)
constexpr int RING = 4;              // stages of the tile ring
constexpr int UROWS = 4;             // tile rows per stage
constexpr int XPAD = 8;              // f16 elements added to the pitch of a staged activation row

struct Mul1Spec {
    int k, n;        // in, out
    int bits, half;  // bitrate
    int n32;         // u32 words per tile
    long long tr_off, suh_off, svh_off;  // byte offsets into the record
};

__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// natural-order FWHT of 128 values over one warp, element 4*lane + j in v[j]; stages (a+b, a-b)
__device__ __forceinline__ void fwht128(float v[4], int lane) {
    const float a0 = __fadd_rn(v[0], v[1]), a1 = __fsub_rn(v[0], v[1]), a2 = __fadd_rn(v[2], v[3]), a3 = __fsub_rn(v[2], v[3]);
    v[0] = __fadd_rn(a0, a2), v[1] = __fadd_rn(a1, a3), v[2] = __fsub_rn(a0, a2), v[3] = __fsub_rn(a1, a3);
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float o = __shfl_xor_sync(0xffffffffu, v[j], m);
            v[j] = (lane & m) ? __fsub_rn(o, v[j]) : __fadd_rn(v[j], o);
        }
    }
}

// power-of-two scale of a 128-block so that |v| * mul < 2^15 (f16 exact range); returns mul, sets inv
__device__ __forceinline__ float block_scale(float amax, float& inv) {
    uint32_t e = (__float_as_uint(amax) >> 23) & 0xFF;
    inv = 1.0f;
    if (!(amax > 0.0f) || e == 255) return 1.0f;
    e = e < 15 ? 15 : e;
    inv = __uint_as_float((e - 14u) << 23);
    return __uint_as_float((268u - e) << 23);
}

// Four scaled values as two f16 planes: hi = f16(v * mul), lo = f16((v * mul - hi) * 2^11). hi + lo * 2^-11
// carries 22 significand bits, so the f16 x f16 products lose nothing that an f32 activation would keep.
__device__ __forceinline__ void store_hi_lo(uint16_t* xh, size_t plane, size_t at, const float v[4], float mul) {
    uint16_t hi[4], lo[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float s = v[j] * mul;
        const __half h = __float2half_rn(s);
        hi[j] = __half_as_ushort(h);
        lo[j] = __half_as_ushort(__float2half_rn((s - __half2float(h)) * 2048.0f));
    }
    *(uint2*)(xh + at) = make_uint2(hi[0] | ((uint32_t)hi[1] << 16), hi[2] | ((uint32_t)hi[3] << 16));
    *(uint2*)(xh + plane + at) = make_uint2(lo[0] | ((uint32_t)lo[1] << 16), lo[2] | ((uint32_t)lo[3] << 16));
}

// xh16[slot][t][k] = the hi / lo planes of H128(x * suh) * mul, xinv[slot][t][k/128] = 1/mul.
// grid (k/128, 1, slots), block 32 T (warp t = activation row t). XT: 0 f32, 1 bf16 input. x row of slot: x + (slot / x_div) * T * k.
// rowsrc (optional): the x row of (slot, t) as an index into x [rows][k], negative = an unused row slot (stored as zeros)
template <int XT>
__global__ void mul1_had_in_kernel(const unsigned long long* __restrict__ ptrs, const void* __restrict__ x, uint16_t* __restrict__ xh,
                                   float* __restrict__ xinv, int k, int T, long long suh_off, int x_div, size_t plane,
                                   const int* __restrict__ rowsrc) {
    pdl_launch_dependents();
    pdl_wait();  // everything below may read what earlier kernels of the stream wrote
    const int slot = blockIdx.z, t = threadIdx.x >> 5, blk = blockIdx.x, lane = threadIdx.x & 31;  // one warp per activation row
    if (ptrs[slot] == 0ull) return;  // a null record: nothing to read or write
    const uint16_t* suh = (const uint16_t*)(ptrs[slot] + (unsigned long long)suh_off);
    const int src = rowsrc ? rowsrc[slot * T + t] : 0;
    const size_t xrow = rowsrc ? (size_t)(src < 0 ? 0 : src) * k : ((size_t)(slot / x_div) * T + t) * k, row = ((size_t)slot * T + t) * k;
    const int c0 = blk * 128 + 4 * lane;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        float xv = XT == 1 ? __bfloat162float(((const __nv_bfloat16*)x)[xrow + c0 + j]) : ((const float*)x)[xrow + c0 + j];
        if (src < 0) xv = 0.0f;
        v[j] = __fmul_rn(xv, h2f(suh[c0 + j]));
    }
    fwht128(v, lane);
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float inv;
    const float mul = block_scale(amax, inv);
    store_hi_lo(xh, plane, row + c0, v, mul);
    if (lane == 0) xinv[((size_t)slot * T + t) * (k / 128) + blk] = inv;
}

// the codec's f16 weights of two states (bit-exact): sum16 = 0x6400 + bytesum(state * 0x83DCD12D) is the
// f16 pattern of 1024 + s; w = fma(sum16, 0x1eee, 0xc931) in f16 with one rounding (converter/src/mul1.rs:135-143)
__device__ __forceinline__ uint32_t mul1_pair(uint32_t s0, uint32_t s1) {
    const uint32_t a = __dp4a(s0 * 0x83DCD12Du, 0x01010101u, 0x6400u), b = __dp4a(s1 * 0x83DCD12Du, 0x01010101u, 0x6400u);
    const uint32_t packed = __byte_perm(a, b, 0x5410);
    uint32_t w;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(w) : "r"(packed), "r"(0x1eee1eeeu), "r"(0xc931c931u));
    return w;
}

// Lane g's eight 16-bit states of one tile. K3: bits = 3, whole bitrate, every shift a constant after the
// window is aligned to the lane's first bit. Otherwise the general circular extraction.
template <bool K3>
__device__ __forceinline__ void lane_states(const uint32_t* tile, int n32, const int lo[8], int wi0, int sh0, uint32_t st[8]) {
    if (K3) {
        // words wi0, wi0+1, wi0+2 (circular) hold bits [24g - 13, 24g + 24); align the window to bit 0
        const uint32_t w0 = tile[wi0], w1 = tile[wi0 + 1 >= n32 ? wi0 + 1 - n32 : wi0 + 1], w2 = tile[wi0 + 2 >= n32 ? wi0 + 2 - n32 : wi0 + 2];
        const uint32_t hi = __funnelshift_l(w1, w0, sh0), lw = __funnelshift_l(w2, w1, sh0);
        // state j = bits [3j, 3j + 16) of the 64-bit window hi:lw (MSB first)
        st[0] = hi >> 16;
        st[1] = (hi >> 13) & 0xffffu;
        st[2] = (hi >> 10) & 0xffffu;
        st[3] = (hi >> 7) & 0xffffu;
        st[4] = (hi >> 4) & 0xffffu;
        st[5] = (hi >> 1) & 0xffffu;
        st[6] = __funnelshift_l(lw, hi, 18) >> 16;
        st[7] = __funnelshift_l(lw, hi, 21) >> 16;
    } else {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int i = lo[j] >> 5, o = lo[j] & 31, i1 = i + 1 == n32 ? 0 : i + 1;
            st[j] = __funnelshift_l(tile[i1], tile[i], o) >> 16;
        }
    }
}

// y' partials of one k-split. grid (n/128, S, slots), block 288 = 8 decode warps + 1 copy warp.
// part[slot][sp][t][n]; xh16 [slot][T][k] f16, xinv [slot][T][k/128].
// MT: activation rows the register allocation is built for (1, 2, 4 or 8; T <= MT of them live)
template <bool K3, int MT>
__global__ void __launch_bounds__(288, 4) mul1_gemv_kernel(const unsigned long long* __restrict__ ptrs, const uint16_t* __restrict__ xh,
                                                        const float* __restrict__ xinv, float* __restrict__ part, Mul1Spec sp_, int S, int T,
                                                        size_t plane, int SPC) {
    pdl_launch_dependents();
    pdl_wait();  // everything below may read what earlier kernels of the stream wrote
    // SPC consecutive k-splits per CTA (blockIdx.y walks groups of SPC): the splits keep their own partial sums, so
    // the arithmetic does not depend on SPC; a CTA that takes several streams them through one ring without a drain
    extern __shared__ __align__(128) uint8_t smem[];
    const int slot = blockIdx.z, sp0 = blockIdx.y * SPC;
    const unsigned long long rec = ptrs[slot];
    if (rec == 0ull) return;  // uniform, before any barrier
    const int k = sp_.k, n = sp_.n, n32 = sp_.n32;
    const int tiles_n = n >> 4, tps = (k >> 4) / S, kb0 = sp0 * tps, rows = SPC * tps * 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb0 = blockIdx.x * 8;
    const int run_bytes = 32 * n32;  // 8 tiles of one tile row
    uint64_t* full = (uint64_t*)smem;
    uint64_t* empty = full + RING;
    uint32_t* ring = (uint32_t*)(smem + 128);                                   // [RING][UROWS][8][n32]
    // [2][T][pitch] f16: hi plane, lo plane; a row pitch of 16 bytes more than a multiple of 256 keeps the eight rows
    // the lanes of a warp read at once on distinct banks
    const int pitch = rows + XPAD;
    uint16_t* xs = (uint16_t*)(smem + 128 + (size_t)RING * UROWS * run_bytes);
    float* xi = (float*)(xs + (size_t)2 * T * pitch);  // [T][rows/128]
    if (threadIdx.x == 0) {
        for (int s = 0; s < RING; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 8);
        }
        mbar_fence_init();
    }
    __syncthreads();
    const int nst1 = (tps + UROWS - 1) / UROWS;  // stages of one split
    const int nst = SPC * nst1;
    if (warp == 8) {
        const uint8_t* base = (const uint8_t*)(rec + (unsigned long long)sp_.tr_off);
        if (((uintptr_t)base & 15) != 0) {
            cn_dev_fail(103);  // a trellis that is not 16-byte aligned cannot be bulk-copied
            return;
        }
        for (int c = 0; c < nst; c++) {
            const int s = c % RING;
            if (c >= RING && !mbar_wait(&empty[s], ((c / RING) - 1) & 1)) {
                cn_dev_fail(CN_DEV_WAIT_EMPTY);
                return;
            }
            const int spi = c / nst1, cs = c - spi * nst1;  // split within the CTA, stage within the split
            const int live = min(UROWS, tps - cs * UROWS);
            if (lane == 0) {
                mbar_expect_tx(&full[s], (uint32_t)(live * run_bytes));
                mbar_arrive(&full[s]);
            }
            __syncwarp();
            if (lane < live) {
                const size_t off = ((size_t)(kb0 + spi * tps + cs * UROWS + lane) * tiles_n + nb0) * n32 * 4;
                bulk_g2s((uint8_t*)ring + ((size_t)s * UROWS + lane) * run_bytes, base + off, (uint32_t)run_bytes, &full[s]);
            }
        }
        return;
    }
    // the activation rows of this k-split, and their block scales
    for (int i = threadIdx.x; i < T * rows / 2; i += 256) {
        const int t = i / (rows / 2), r = i - t * (rows / 2);
        const size_t at = ((size_t)slot * T + t) * k + (size_t)kb0 * 16;
        ((uint32_t*)(xs + (size_t)t * pitch))[r] = ((const uint32_t*)(xh + at))[r];
        ((uint32_t*)(xs + (size_t)(T + t) * pitch))[r] = ((const uint32_t*)(xh + plane + at))[r];
    }
    const int nblk = rows / 128;
    for (int i = threadIdx.x; i < T * nblk; i += 256) {
        const int t = i / nblk, b = i - t * nblk;
        xi[i] = xinv[((size_t)slot * T + t) * (k / 128) + kb0 / 8 + b];
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");

    int lo[8];
    const int sbits = n32 * 32;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int tpos = 8 * lane + j;
        const int eb = !sp_.half ? (tpos + 1) * sp_.bits : ((tpos & 1) ? (tpos / 2 + 1) * (2 * sp_.bits + 1) : (tpos / 2) * (2 * sp_.bits + 1) + sp_.bits);
        lo[j] = (eb - 16 + sbits) % sbits;
    }
    const int wi0 = lo[0] >> 5, sh0 = lo[0] & 31;
    // Multiply-accumulate on the tensor cores. The eight weights a lane decodes from a tile are the A fragment of one
    // mma.m16n8k16 as they stand (MMA row = output column g / g + 8 of the tile, MMA k = the tile's k): w01 | w45 | w23 |
    // w67. Column c of the B operand is activation row c >> 1, plane c & 1 (hi, lo), so one MMA serves four activation
    // rows and a lane (g, t) ends up with the hi and lo sums of activation row t for outputs g and g + 8: nothing is
    // exchanged between lanes. Columns of rows beyond T repeat the last live row and are never stored.
    const int g = lane >> 2, t4 = lane & 3;
    constexpr int NM = MT > 4 ? 2 : 1;  // MMAs per tile: four activation rows each
    const uint16_t* xb[NM];
    const float* xil[NM];
#pragma unroll
    for (int i = 0; i < NM; i++) {
        const int rb = min(4 * i + (g >> 1), T - 1), rc = min(4 * i + t4, T - 1);
        xb[i] = xs + ((size_t)(g & 1) * T + rb) * pitch + 2 * t4;
        xil[i] = xi + rc * nblk;
    }
    float acc[NM][4], tot0[NM], tot1[NM];
#pragma unroll
    for (int i = 0; i < NM; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = tot0[i] = tot1[i] = 0.0f;
    // Everything a tile needs beyond its own words is a constant offset from pointers that move once per stage: at
    // K = 3 a tile is 24 words, and a split is a whole number of stages and of 128-row blocks (tps % 8 == 0, which
    // the launcher guarantees), so the loop carries no division, no bounds test and no address arithmetic per tile.
    constexpr int TW = K3 ? 24 : 0;  // words of a tile when known at compile time
    const int tw = K3 ? TW : n32;
    const int o1 = wi0 + 1 >= tw ? wi0 + 1 - tw : wi0 + 1, o2 = wi0 + 2 >= tw ? wi0 + 2 - tw : wi0 + 2;
    const uint32_t* lane_tile = ring + (size_t)warp * tw;  // this warp's tile of the ring's first tile row
    int s = 0, cs = 0, spi = 0, blk = 0;
    uint32_t ph = 0;
    for (int c = 0; c < nst; c++) {
        if (!mbar_wait(&full[s], ph)) {
            cn_dev_fail(CN_DEV_WAIT_FULL);
            return;
        }
        const uint32_t* tb = lane_tile + (size_t)s * (UROWS * 8) * tw;
        const int kx = (spi * tps + cs * UROWS) * 16;  // first k of the stage within the staged activations
#pragma unroll
        for (int u = 0; u < UROWS; u++) {
            uint32_t st[8];
            if (K3) {
                // words wi0, wi0 + 1, wi0 + 2 (circular) hold bits [24 g - 13, 24 g + 24) of the tile; the window is
                // aligned to the lane's first bit and state j = bits [3 j, 3 j + 16) of it, most significant bit first
                const uint32_t* tl = tb + u * 8 * TW;
                const uint32_t w0 = tl[wi0], w1 = tl[o1], w2 = tl[o2];
                const uint32_t hi = __funnelshift_l(w1, w0, sh0), lw = __funnelshift_l(w2, w1, sh0);
                st[0] = hi >> 16;
                st[1] = (hi >> 13) & 0xffffu;
                st[2] = (hi >> 10) & 0xffffu;
                st[3] = (hi >> 7) & 0xffffu;
                st[4] = (hi >> 4) & 0xffffu;
                st[5] = (hi >> 1) & 0xffffu;
                st[6] = __funnelshift_l(lw, hi, 18) >> 16;
                st[7] = __funnelshift_l(lw, hi, 21) >> 16;
            } else {
                lane_states<false>(tb + (size_t)u * 8 * tw, n32, lo, wi0, sh0, st);
            }
            const uint32_t w01 = mul1_pair(st[0], st[1]), w23 = mul1_pair(st[2], st[3]);
            const uint32_t w45 = mul1_pair(st[4], st[5]), w67 = mul1_pair(st[6], st[7]);
#pragma unroll
            for (int i = 0; i < NM; i++) {
                const uint32_t* xr = (const uint32_t*)(xb[i] + kx + u * 16);
                mma16816(acc[i], w01, w45, w23, w67, xr[0], xr[4]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
        if (++s == RING) s = 0, ph ^= 1u;
        if (cs & 1) {
            // end of a 128-row block (two stages): hi + lo * 2^-11, then the block's activation scale
#pragma unroll
            for (int i = 0; i < NM; i++) {
                const float inv = xil[i][blk];
                tot0[i] = fmaf(fmaf(acc[i][1], 4.8828125e-4f, acc[i][0]), inv, tot0[i]);
                tot1[i] = fmaf(fmaf(acc[i][3], 4.8828125e-4f, acc[i][2]), inv, tot1[i]);
                acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
            }
            blk++;
        }
        if (++cs == nst1) {
            // end of a split: lane (g, t) stores outputs g and g + 8 of its tile column for activation row t (+ 4)
#pragma unroll
            for (int i = 0; i < NM; i++) {
                const int t = 4 * i + t4;
                if (t < T) {
                    float* pp = part + (((size_t)slot * S + sp0 + spi) * T + t) * n + (size_t)(nb0 + warp) * 16 + g;
                    pp[0] = tot0[i];
                    pp[8] = tot1[i];
                }
                tot0[i] = tot1[i] = 0.0f;
            }
            cs = 0;
            spi++;
        }
    }
}

// v = H128(sum_sp part[slot][sp][t][blk*128 ..]) / 128 * svh
__device__ __forceinline__ void out_block(float v[4], const float* __restrict__ part, const uint16_t* __restrict__ svh, int slot, int S, int T,
                                          int t, int n, int blk, int lane) {
    const int c0 = blk * 128 + 4 * lane;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        float s = part[(((size_t)slot * S + 0) * T + t) * n + c0 + j];
        for (int q = 1; q < S; q++) s = __fadd_rn(s, part[(((size_t)slot * S + q) * T + t) * n + c0 + j]);
        v[j] = s;
    }
    fwht128(v, lane);
#pragma unroll
    for (int j = 0; j < 4; j++) v[j] = __fmul_rn(__fmul_rn(v[j], 0.0078125f), h2f(svh[c0 + j]));
}

// grid (n/128, 1, slots), block 32 T (warp t = activation row t). YT: 0 f32, 1 bf16 output; y row = slot * T + t
// rowdst (optional): the y row of (slot, t) as an index into y [rows][n], negative = nothing to store
template <int YT>
__global__ void mul1_had_out_kernel(const unsigned long long* __restrict__ ptrs, const float* __restrict__ part, void* __restrict__ y, int n,
                                    int S, int T, long long svh_off, const int* __restrict__ rowdst) {
    pdl_launch_dependents();
    pdl_wait();  // everything below may read what earlier kernels of the stream wrote
    const int slot = blockIdx.z, t = threadIdx.x >> 5, blk = blockIdx.x, lane = threadIdx.x & 31;  // one warp per activation row
    if (ptrs[slot] == 0ull) return;
    const int dst = rowdst ? rowdst[slot * T + t] : 0;
    if (dst < 0) return;
    float v[4];
    out_block(v, part, (const uint16_t*)(ptrs[slot] + (unsigned long long)svh_off), slot, S, T, t, n, blk, lane);
    const size_t at = (rowdst ? (size_t)dst : (size_t)slot * T + t) * n + blk * 128 + 4 * lane;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        if (YT == 1)
            ((__nv_bfloat16*)y)[at + j] = __float2bfloat16_rn(v[j]);
        else
            ((float*)y)[at + j] = v[j];
    }
}

// The middle of the FFN in one launch: had_out of gate and of up, h = act(g, u), had_in of down.
// grid (inter/128, 1, slots), block 32 T (warp t = activation row t).
__global__ void mul1_act_had_in_kernel(const unsigned long long* __restrict__ ptrs, const float* __restrict__ part_g,
                                       const float* __restrict__ part_u, uint16_t* __restrict__ xh_d, float* __restrict__ xinv_d, int inter, int S,
                                       int T, long long svh_g, long long svh_u, long long suh_d, float limit, size_t plane) {
    pdl_launch_dependents();
    pdl_wait();  // everything below may read what earlier kernels of the stream wrote
    const int slot = blockIdx.z, t = threadIdx.x >> 5, blk = blockIdx.x, lane = threadIdx.x & 31;  // one warp per activation row
    if (ptrs[slot] == 0ull) return;
    float g[4], u[4], v[4];
    out_block(g, part_g, (const uint16_t*)(ptrs[slot] + (unsigned long long)svh_g), slot, S, T, t, inter, blk, lane);
    out_block(u, part_u, (const uint16_t*)(ptrs[slot] + (unsigned long long)svh_u), slot, S, T, t, inter, blk, lane);
    const uint16_t* suh = (const uint16_t*)(ptrs[slot] + (unsigned long long)suh_d);
    const int c0 = blk * 128 + 4 * lane;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        float gv = g[j], uv = u[j];
        if (limit > 0.0f) {
            gv = gv > limit ? limit : gv;
            uv = uv > limit ? limit : (uv < -limit ? -limit : uv);
        }
        const float h = __fmul_rn(gv / (1.0f + expf(-gv)), uv);
        v[j] = __fmul_rn(h, h2f(suh[c0 + j]));
    }
    fwht128(v, lane);
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float inv;
    const float mul = block_scale(amax, inv);
    const size_t row = ((size_t)slot * T + t) * inter;
    store_hi_lo(xh_d, plane, row + c0, v, mul);
    if (lane == 0) xinv_d[((size_t)slot * T + t) * (inter / 128) + blk] = inv;
}

// W_hat as fp16 bits, row major [k][n]: one thread per (tile, position) - the codec self-check
__global__ void mul1_reconstruct_kernel(const uint32_t* __restrict__ trellis, uint16_t* __restrict__ w, int k, int n, int bits, int half, int n32) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)(k / 16) * (n / 16) * 256;
    if (i >= total) return;
    const int p = (int)(i & 255);
    const long long tile = i >> 8;
    const int kb = (int)(tile / (n / 16)), nb = (int)(tile % (n / 16));
    const int sbits = n32 * 32;
    const int eb = !half ? (p + 1) * bits : ((p & 1) ? (p / 2 + 1) * (2 * bits + 1) : (p / 2) * (2 * bits + 1) + bits);
    const int lo = (eb - 16 + sbits) % sbits;
    const uint32_t* t = trellis + tile * n32;
    const int wi = lo >> 5, o = lo & 31, w1 = wi + 1 == n32 ? 0 : wi + 1;
    const uint32_t st = __funnelshift_l(t[w1], t[wi], o) >> 16;
    const uint32_t pr = mul1_pair(st, st);
    const int lane = p >> 3, j = p & 7;
    const int off[4] = {0, 1, 8, 9};
    const int row = 2 * (lane & 3) + off[j & 3], col = (lane >> 2) + 8 * (j >> 2);
    w[(size_t)(kb * 16 + row) * n + nb * 16 + col] = (uint16_t)(pr & 0xffff);
}

}  // namespace

// ---------------------------------------------------------------- host side
namespace {

struct Mul1Plan {
    int hidden, inter, bits, half, n32, max_slots, max_t;
    size_t kmax;
    uint16_t *xh_a, *xh_b;  // [2 planes][slots][T][kmax] f16
    size_t plane;           // elements of one plane
    float *xinv_a, *xinv_b;  // [slots][T][kmax/128]
    float *part_a, *part_b;  // [slots][16][T][kmax]
    unsigned long long* ptrs;  // [slots] gathered record addresses (MoE form)
    int32_t* order;            // [slots] combos sorted by expert (grouped MoE form)
    int* groups;               // [5 * slots + 8] the group lists and counts of cn_moe_group_launch
    int* rowsrc;               // [slots * MUL1_GT] x row of every (group slot, row), -1 = unused
    int* rowdst;               // [slots * MUL1_GT] combo (output row) of every (group slot, row), -1 = unused
    int grp_rows;              // rows the scratch holds per slot: max(max_t, 4)
    float* eo;                 // [slots][T][hidden] expert outputs (MoE form)
    // the up projection does not depend on the gate projection: it runs on a side stream between two events
    cudaStream_t side;
    cudaEvent_t fork, join;
};

int ksplit(int k) {
    // the largest divisor of k/128 that is <= 16: k-splits end on Hadamard blocks
    const int blocks = k / 128;
    for (int s = 16; s >= 1; s--)
        if (blocks % s == 0) return s;
    return 1;
}

long long trellis_bytes(int k, int n, int n32) { return (long long)(k / 16) * (n / 16) * n32 * 4; }

Mul1Spec spec_of(const Mul1Plan* p, int which) {
    const long long tb = trellis_bytes(p->hidden, p->inter, p->n32), h2 = 2LL * p->hidden, i2 = 2LL * p->inter;
    Mul1Spec s;
    s.bits = p->bits, s.half = p->half, s.n32 = p->n32;
    if (which == 0) s.k = p->hidden, s.n = p->inter, s.tr_off = 0, s.suh_off = 3 * tb, s.svh_off = 3 * tb + h2;
    if (which == 1) s.k = p->hidden, s.n = p->inter, s.tr_off = tb, s.suh_off = 3 * tb + h2 + i2, s.svh_off = 3 * tb + 2 * h2 + i2;
    if (which == 2) s.k = p->inter, s.n = p->hidden, s.tr_off = 2 * tb, s.suh_off = 3 * tb + 2 * h2 + 2 * i2, s.svh_off = 3 * tb + 2 * h2 + 3 * i2;
    return s;
}

int launch_had_in(const unsigned long long* ptrs, const void* x, uint16_t* xh, float* xinv, const Mul1Spec& s, int slots, int T, int x_div,
                  int dtype, size_t plane, cudaStream_t st, const int* rowsrc = nullptr) {
    dim3 grid(s.k / 128, 1, slots);
    if (dtype == CN_BF16)
        CN_CUDA(cn_launch_pdl((mul1_had_in_kernel<1>), dim3(grid), dim3(32 * T), 0, st, ptrs, x, xh, xinv, s.k, T, s.suh_off, x_div, plane, rowsrc));
    else
        CN_CUDA(cn_launch_pdl((mul1_had_in_kernel<0>), dim3(grid), dim3(32 * T), 0, st, ptrs, x, xh, xinv, s.k, T, s.suh_off, x_div, plane, rowsrc));
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}

// live: how many of the slots are expected to hold a record (the grouped MoE form launches more slots than it fills)
int launch_gemv(const unsigned long long* ptrs, const uint16_t* xh, const float* xinv, float* part, const Mul1Spec& s, int slots, int T,
                size_t plane, cudaStream_t st, int live = 0) {
    if (live < 1 || live > slots) live = slots;
    const int S = ksplit(s.k), tps = (s.k / 16) / S;
    if (tps % 8 != 0) CN_FAIL(CN_ERR_SHAPE, "mul1 gemv: k = %d does not split into whole 128-row blocks", s.k);  // the kernel's stage / block counters rely on it
    // k-splits per CTA: as many as still leave about four CTAs per SM (the splits keep separate partial sums, so
    // this only moves work between CTAs) and fit the staged activations
    int spc = 1;
    for (int c = S; c > 1; c--) {
        if (S % c) continue;
        const long long ctas = (long long)(s.n / 128) * (S / c) * live;
        const size_t need = 128 + (size_t)RING * UROWS * 32 * s.n32 + (size_t)2 * T * (c * tps * 16 + XPAD) * 2 + 8 + (size_t)T * (c * tps / 8) * 4;
        if (ctas >= 592 && need <= 160 * 1024) {
            spc = c;
            break;
        }
    }
    const int rows = spc * tps * 16;
    const size_t smem = 128 + (size_t)RING * UROWS * 32 * s.n32 + (size_t)2 * T * (rows + XPAD) * 2 + 8 + (size_t)T * (rows / 128) * 4;
    dim3 grid(s.n / 128, S / spc, slots);
    if (smem > 160 * 1024) CN_FAIL(CN_ERR_LIMIT, "mul1 gemv: %zu B of shared memory per block", smem);
    const bool k3 = s.bits == 3 && !s.half;
    const int mt = T == 1 ? 1 : (T == 2 ? 2 : (T <= 4 ? 4 : 8));
#define CN_MUL1_CASE(K3V, MTV)                                                                                                      \
    if (k3 == K3V && mt == MTV) {                                                                                                   \
        CN_ALLOW_SMEM((mul1_gemv_kernel<K3V, MTV>), 160 * 1024);                                                                    \
        CN_CUDA(cn_launch_pdl((mul1_gemv_kernel<K3V, MTV>), grid, dim3(288), smem, st, ptrs, xh, xinv, part, s, S, T, plane, spc));        \
    }
    CN_MUL1_CASE(true, 1) CN_MUL1_CASE(true, 2) CN_MUL1_CASE(true, 4) CN_MUL1_CASE(true, 8)
    CN_MUL1_CASE(false, 1) CN_MUL1_CASE(false, 2) CN_MUL1_CASE(false, 4) CN_MUL1_CASE(false, 8)
#undef CN_MUL1_CASE
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}

int check_run(const Mul1Plan* p, int slots, int T, const char* who) {
    if (!p) CN_FAIL(CN_ERR_SHAPE, "%s: null plan", who);
    if (slots < 1 || slots > p->max_slots || T < 1 || T > p->max_t)
        CN_FAIL(CN_ERR_LIMIT, "%s: %d slots x %d rows, the plan holds %d x %d", who, slots, T, p->max_slots, p->max_t);
    return CN_OK;
}

__global__ void mul1_gather_kernel(const unsigned long long* __restrict__ table, const int32_t* __restrict__ ids, unsigned long long* ptrs, int n,
                                   int experts) {
    pdl_launch_dependents();
    pdl_wait();  // everything below may read what earlier kernels of the stream wrote
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < n) ptrs[c] = (ids[c] < 0 || (experts > 0 && ids[c] >= experts)) ? 0ull : table[ids[c]];
}

// Slot s of the grouped MoE form (gt rows per slot, 4 or 8): the groups of two or more rows first, then the one-row
// groups, then empty slots (null record). Fills the slot's record address and, per row, where its x row comes from and
// which combo's output row it is.
__global__ void mul1_slots_kernel(const unsigned long long* __restrict__ table, const int32_t* __restrict__ ids, const int32_t* __restrict__ order,
                                  const int* __restrict__ ga, const int* __restrict__ gb, const int* __restrict__ gbrows, const int* __restrict__ counts,
                                  unsigned long long* __restrict__ ptrs, int* __restrict__ rowsrc, int* __restrict__ rowdst, int slots, int x_div, int gt) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= slots) return;
    const int na = counts[0], nb = counts[1];
    int pos = -1, rows = 0;
    if (s < nb) pos = gb[s], rows = gbrows[s];
    else if (s < nb + na) pos = ga[s - nb], rows = 1;
    ptrs[s] = pos < 0 ? 0ull : table[ids[order[pos]]];
    for (int t = 0; t < gt; t++) {
        const int c = t < rows ? order[pos + t] : -1;
        rowsrc[s * gt + t] = c < 0 ? -1 : c / x_div;
        rowdst[s * gt + t] = c;
    }
}

}  // namespace

extern "C" int cn_mul1_plan_destroy(void* plan);

extern "C" int cn_mul1_plan_create(void** plan_out, int hidden, int inter, int bits, int half, int max_slots, int max_t) {
    if (!plan_out || hidden <= 0 || inter <= 0 || hidden % 128 || inter % 128)
        CN_FAIL(CN_ERR_SHAPE, "cn_mul1_plan_create: [%d, %d] is not a positive multiple of 128 on both sides", hidden, inter);
    if (bits < 1 || bits > 8 || (half && bits > 3)) CN_FAIL(CN_ERR_SHAPE, "cn_mul1_plan_create: unsupported bitrate %d%s", bits, half ? ".5" : "");
    if (max_slots < 1 || max_t < 1 || max_t > MUL1_MAXT) CN_FAIL(CN_ERR_LIMIT, "cn_mul1_plan_create: %d slots, %d rows (rows <= %d)", max_slots, max_t, MUL1_MAXT);
    Mul1Plan* p = new Mul1Plan();
    p->hidden = hidden, p->inter = inter, p->bits = bits, p->half = half, p->n32 = 8 * bits + (half ? 4 : 0), p->max_slots = max_slots, p->max_t = max_t;
    p->kmax = hidden > inter ? hidden : inter;
    // the grouped MoE form runs its slots with four or eight rows: the scratch holds four rows per slot, which covers
    // eight-row groups whenever there are few enough of them (see cn_moe_mul1_experts)
    p->grp_rows = max_t > 4 ? max_t : 4;
    const size_t rows = (size_t)max_slots * p->grp_rows;
    p->plane = rows * p->kmax;
    // a failure part-way frees what the earlier steps got (the destroy call takes a half-built plan)
    cudaError_t e = cudaSuccess;
    auto step = [&](cudaError_t r) { if (e == cudaSuccess) e = r; };
    step(cudaMalloc(&p->xh_a, 2 * p->plane * 2));
    step(cudaMalloc(&p->xh_b, 2 * p->plane * 2));
    step(cudaMalloc(&p->xinv_a, rows * (p->kmax / 128) * 4));
    step(cudaMalloc(&p->xinv_b, rows * (p->kmax / 128) * 4));
    step(cudaMalloc(&p->part_a, rows * 16 * p->kmax * 4));
    step(cudaMalloc(&p->part_b, rows * 16 * p->kmax * 4));
    step(cudaMalloc(&p->ptrs, (size_t)max_slots * 8));
    step(cudaMalloc(&p->order, (size_t)max_slots * 4));
    step(cudaMalloc(&p->groups, ((size_t)5 * max_slots + 8) * 4));
    step(cudaMalloc(&p->rowsrc, (size_t)max_slots * MUL1_GT * 4));
    step(cudaMalloc(&p->rowdst, (size_t)max_slots * MUL1_GT * 4));
    step(cudaMalloc(&p->eo, rows * hidden * 4));
    step(cudaStreamCreateWithFlags(&p->side, cudaStreamNonBlocking));
    step(cudaEventCreateWithFlags(&p->fork, cudaEventDisableTiming));
    step(cudaEventCreateWithFlags(&p->join, cudaEventDisableTiming));
    if (e != cudaSuccess) {
        cn_mul1_plan_destroy(p);
        CN_FAIL(CN_ERR_CUDA, "cn_mul1_plan_create: %s", cudaGetErrorString(e));
    }
    *plan_out = p;
    return CN_OK;
}

extern "C" int cn_mul1_plan_destroy(void* plan) {
    Mul1Plan* p = (Mul1Plan*)plan;
    if (!p) return CN_OK;
    cudaFree(p->xh_a), cudaFree(p->xh_b), cudaFree(p->xinv_a), cudaFree(p->xinv_b), cudaFree(p->part_a), cudaFree(p->part_b), cudaFree(p->ptrs),
        cudaFree(p->eo), cudaFree(p->order), cudaFree(p->groups), cudaFree(p->rowsrc), cudaFree(p->rowdst);
    if (p->side) cudaStreamDestroy(p->side);
    if (p->fork) cudaEventDestroy(p->fork);
    if (p->join) cudaEventDestroy(p->join);
    delete p;
    return CN_OK;
}

extern "C" int cn_mul1_gemv(void* plan, int which, const unsigned long long* ptrs, const void* x, void* y, int slots, int t, int x_div, int dtype,
                            cn_stream_t stream) {
    Mul1Plan* p = (Mul1Plan*)plan;
    if (int rc = check_run(p, slots, t, "cn_mul1_gemv")) return rc;
    if (which < 0 || which > 2 || x_div < 1) CN_FAIL(CN_ERR_SHAPE, "cn_mul1_gemv: matrix %d (0 gate, 1 up, 2 down), x_div %d", which, x_div);
    if (dtype != CN_F32 && dtype != CN_BF16) CN_FAIL(CN_ERR_SHAPE, "cn_mul1_gemv: dtype %d is neither CN_F32 nor CN_BF16", dtype);
    cudaStream_t st = (cudaStream_t)stream;
    const Mul1Spec s = spec_of(p, which);
    if (int rc = launch_had_in(ptrs, x, p->xh_a, p->xinv_a, s, slots, t, x_div, dtype, p->plane, st)) return rc;
    if (int rc = launch_gemv(ptrs, p->xh_a, p->xinv_a, p->part_a, s, slots, t, p->plane, st)) return rc;
    dim3 grid(s.n / 128, 1, slots);
    if (dtype == CN_BF16)
        CN_CUDA(cn_launch_pdl((mul1_had_out_kernel<1>), dim3(grid), dim3(32 * t), 0, st, ptrs, p->part_a, y, s.n, ksplit(s.k), t, s.svh_off, (const int*)nullptr));
    else
        CN_CUDA(cn_launch_pdl((mul1_had_out_kernel<0>), dim3(grid), dim3(32 * t), 0, st, ptrs, p->part_a, y, s.n, ksplit(s.k), t, s.svh_off, (const int*)nullptr));
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}

// y[slot][t] = down(act(gate x, up x)) as f32 when out_f32, else in `dtype`
static int mul1_ffn(Mul1Plan* p, const unsigned long long* ptrs, const void* x, void* y, int slots, int t, int x_div, float limit, int dtype,
                    int out_f32, cudaStream_t st, const int* rowsrc = nullptr, const int* rowdst = nullptr, int live = 0) {
    const Mul1Spec g = spec_of(p, 0), u = spec_of(p, 1), d = spec_of(p, 2);
    // up branch on the side stream; it is joined again on every path, so a capture of `st` stays valid
    CN_CUDA(cudaEventRecord(p->fork, st));
    CN_CUDA(cudaStreamWaitEvent(p->side, p->fork, 0));
    int rc = launch_had_in(ptrs, x, p->xh_b, p->xinv_b, u, slots, t, x_div, dtype, p->plane, p->side, rowsrc);
    if (rc == CN_OK) rc = launch_gemv(ptrs, p->xh_b, p->xinv_b, p->part_b, u, slots, t, p->plane, p->side, live);
    CN_CUDA(cudaEventRecord(p->join, p->side));
    if (rc == CN_OK) rc = launch_had_in(ptrs, x, p->xh_a, p->xinv_a, g, slots, t, x_div, dtype, p->plane, st, rowsrc);
    if (rc == CN_OK) rc = launch_gemv(ptrs, p->xh_a, p->xinv_a, p->part_a, g, slots, t, p->plane, st, live);
    CN_CUDA(cudaStreamWaitEvent(st, p->join, 0));
    if (rc != CN_OK) return rc;
    CN_CUDA(cn_launch_pdl(mul1_act_had_in_kernel, dim3(p->inter / 128, 1, slots), dim3(32 * t), 0, st, ptrs, p->part_a, p->part_b, p->xh_a, p->xinv_a, p->inter, ksplit(p->hidden), t,
                                                                         g.svh_off, u.svh_off, d.suh_off, limit, p->plane));
    CN_CUDA(cudaGetLastError());
    if (int rc = launch_gemv(ptrs, p->xh_a, p->xinv_a, p->part_a, d, slots, t, p->plane, st, live)) return rc;
    dim3 grid(d.n / 128, 1, slots);
    if (dtype == CN_BF16 && !out_f32)
        CN_CUDA(cn_launch_pdl((mul1_had_out_kernel<1>), dim3(grid), dim3(32 * t), 0, st, ptrs, p->part_a, y, d.n, ksplit(d.k), t, d.svh_off, rowdst));
    else
        CN_CUDA(cn_launch_pdl((mul1_had_out_kernel<0>), dim3(grid), dim3(32 * t), 0, st, ptrs, p->part_a, y, d.n, ksplit(d.k), t, d.svh_off, rowdst));
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}

extern "C" int cn_mul1_ffn(void* plan, const unsigned long long* ptrs, const void* x, void* y, int slots, int t, int x_div, float limit, int dtype,
                           cn_stream_t stream) {
    Mul1Plan* p = (Mul1Plan*)plan;
    if (int rc = check_run(p, slots, t, "cn_mul1_ffn")) return rc;
    if (x_div < 1) CN_FAIL(CN_ERR_SHAPE, "cn_mul1_ffn: x_div %d", x_div);
    if (dtype != CN_F32 && dtype != CN_BF16) CN_FAIL(CN_ERR_SHAPE, "cn_mul1_ffn: dtype %d is neither CN_F32 nor CN_BF16", dtype);
    return mul1_ffn(p, ptrs, x, y, slots, t, x_div, limit, dtype, 0, (cudaStream_t)stream);
}

extern "C" int cn_moe_combine(const float* eo, const float* wts, const int32_t* ids, const unsigned long long* table, const float* shared,
                              const float* sgate, void* y, int tokens, int hidden, int topk, int experts, int dtype, cn_stream_t stream);

extern "C" int cn_moe_mul1_experts(void* plan, const unsigned long long* table, const int32_t* ids, const void* x, float* eo, int combos, int x_div,
                                   int experts, float limit, int dtype, cn_stream_t stream) {
    Mul1Plan* p = (Mul1Plan*)plan;
    if (int rc = check_run(p, combos, 1, "cn_moe_mul1_experts")) return rc;
    if (x_div < 1 || !eo) CN_FAIL(CN_ERR_SHAPE, "cn_moe_mul1_experts: x_div %d, eo %p", x_div, (void*)eo);
    if (dtype != CN_F32 && dtype != CN_BF16) CN_FAIL(CN_ERR_SHAPE, "cn_moe_mul1_experts: dtype %d is neither CN_F32 nor CN_BF16", dtype);
    cudaStream_t st = (cudaStream_t)stream;
    if (experts > 0 && 2 * combos >= experts) {
        // Enough combos that experts repeat: the combos are sorted by expert and bundled into groups that share one
        // decode of the expert's trellis (a group of up to four rows is one MMA per tile like a single row, eight rows
        // are two). Groups of eight when the batch is long (four combo slots per expert or more) and the plan's scratch
        // holds them; the slots launched are bounded by experts + combos / rows, the rest of the combo slots do not exist.
        const long long cap_rows = (long long)p->max_slots * p->grp_rows;
        int gt = 4;
        if (combos >= 4 * experts && ((long long)experts + combos / 8) * 8 <= cap_rows) gt = 8;
        long long ng = (long long)experts + combos / gt;  // every expert ends in at most one short group
        if (ng > combos) ng = combos;
        if (ng * gt <= cap_rows && ng <= p->max_slots) {
            int* ga = p->groups;
            int* gb = ga + combos;
            int* gbrows = gb + combos;
            int* gd = gbrows + combos;
            int* gdrows = gd + combos;
            int* counts = gdrows + combos;
            if (int rc = cn_moe_group_launch(ids, table, combos, experts, p->order, ga, gb, gbrows, gd, gdrows, counts, gt, st)) return rc;
            CN_CUDA(cn_launch_pdl(mul1_slots_kernel, dim3(((int)ng + 127) / 128), dim3(128), 0, st, table, ids, p->order, ga, gb, gbrows, counts, p->ptrs,
                                  p->rowsrc, p->rowdst, (int)ng, x_div, gt));
            // a slot beyond the groups is a null record, which all kernels skip; a group's unused rows are zero rows
            // (the work per CTA is sized as if a quarter of the launched slots were filled: measured best at 45 of 64 and at 8 of 128)
            return mul1_ffn(p, p->ptrs, x, eo, (int)ng, gt, 1, limit, dtype, 1, st, p->rowsrc, p->rowdst, (int)((ng + 3) / 4));
        }
    }
    CN_CUDA(cn_launch_pdl(mul1_gather_kernel, dim3((combos + 127) / 128), dim3(128), 0, st, table, ids, p->ptrs, combos, experts));
    CN_CUDA(cudaGetLastError());
    return mul1_ffn(p, p->ptrs, x, eo, combos, 1, x_div, limit, dtype, 1, st);
}

extern "C" int cn_moe_mul1_run(void* plan, const unsigned long long* table, const int32_t* ids, const float* wts, const float* shared, const void* x,
                               void* y, int tokens, int topk, int experts, float limit, int dtype, cn_stream_t stream) {
    Mul1Plan* p = (Mul1Plan*)plan;
    if (int rc = cn_moe_mul1_experts(plan, table, ids, x, p ? p->eo : nullptr, tokens * topk, topk, experts, limit, dtype, stream)) return rc;
    return cn_moe_combine(p->eo, wts, ids, table, shared, nullptr, y, tokens, p->hidden, topk, experts, dtype, stream);
}

extern "C" int cn_mul1_reconstruct(const void* trellis, void* w_out, int k, int n, int bits, int half, cn_stream_t stream) {
    if (k <= 0 || n <= 0 || k % 16 || n % 16) CN_FAIL(CN_ERR_SHAPE, "cn_mul1_reconstruct: [%d, %d] is not a multiple of 16", k, n);
    const int n32 = 8 * bits + (half ? 4 : 0);
    const long long total = (long long)(k / 16) * (n / 16) * 256;
    mul1_reconstruct_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint32_t*)trellis, (uint16_t*)w_out, k, n, bits, half, n32);
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}

// ---------------------------------------------------------------- allocation-free MUL1 GEMV
// For callers that may not allocate device memory at the point of the call - an engine thread that
// already runs inside a latency-critical decode loop, a plugin host that forbids cudaMalloc after
// start-up because an allocation synchronises the whole device, or code that holds a memory budget
// it has fully handed out. The scratch of the GEMV (the transformed activations and the k-split
// partial sums) lives in a fixed array inside the library image instead of a plan.
//
// Limits: slots * t <= CN_MUL1_STATIC_ROWS (8) activation rows per call, hidden and inter <=
// CN_MUL1_STATIC_DIM (4096). The array is about 2.2 MB and every GPU that loads the library holds
// it until the process exits.
namespace {

constexpr size_t NA_ROWS = 8, NA_DIM = 4096, NA_SPLITS = 16;
constexpr size_t NA_XH_BYTES = 2 * NA_ROWS * NA_DIM * 2;             // hi and lo f16 planes
constexpr size_t NA_XINV_BYTES = NA_ROWS * (NA_DIM / 128) * 4;       // one f32 per 128-block
constexpr size_t NA_PART_BYTES = NA_ROWS * NA_SPLITS * NA_DIM * 4;   // f32 partial sums of the k-split
constexpr size_t NA_BYTES = NA_XH_BYTES + NA_XINV_BYTES + NA_PART_BYTES;

// File-scope device array: in host code this name is only a handle for the runtime, never an
// address a kernel may be given; the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_mul1_static_scratch[NA_BYTES];

constexpr int NA_MAX_DEVICES = 64;
unsigned char* g_static_ptr[NA_MAX_DEVICES] = {};

// The device address of the scratch array on the current device, looked up once per device.
int static_scratch(unsigned char** out) {
    int dev = -1;
    CN_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= NA_MAX_DEVICES) CN_FAIL(CN_ERR_LIMIT, "cn_mul1_gemv_noalloc: device ordinal %d beyond %d", dev, NA_MAX_DEVICES);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_mul1_static_scratch);
        if (e != cudaSuccess || !p) CN_FAIL(CN_ERR_CUDA, "cn_mul1_gemv_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_static_ptr[dev] = (unsigned char*)p;
    }
    *out = g_static_ptr[dev];
    return CN_OK;
}

}  // namespace

extern "C" int cn_mul1_gemv_noalloc(int which, int hidden, int inter, int bits, int half, const unsigned long long* ptrs, const void* x, void* y,
                                    int slots, int t, int x_div, int dtype, cn_stream_t stream) {
    if (hidden <= 0 || inter <= 0 || hidden % 128 || inter % 128)
        CN_FAIL(CN_ERR_SHAPE, "cn_mul1_gemv_noalloc: [%d, %d] is not a positive multiple of 128 on both sides", hidden, inter);
    if (bits < 1 || bits > 8 || (half && bits > 3)) CN_FAIL(CN_ERR_SHAPE, "cn_mul1_gemv_noalloc: unsupported bitrate %d%s", bits, half ? ".5" : "");
    if (which < 0 || which > 2 || x_div < 1) CN_FAIL(CN_ERR_SHAPE, "cn_mul1_gemv_noalloc: matrix %d (0 gate, 1 up, 2 down), x_div %d", which, x_div);
    if (slots < 1 || t < 1 || t > MUL1_MAXT || (size_t)slots * t > NA_ROWS)
        CN_FAIL(CN_ERR_LIMIT, "cn_mul1_gemv_noalloc: %d slots x %d rows; the fixed scratch holds %zu rows in all (use a plan for more)", slots, t, NA_ROWS);
    if ((size_t)hidden > NA_DIM || (size_t)inter > NA_DIM)
        CN_FAIL(CN_ERR_LIMIT, "cn_mul1_gemv_noalloc: hidden %d / inter %d beyond the fixed scratch's %zu (use a plan for more)", hidden, inter, NA_DIM);
    // before the first launch: the kernels read x in this type
    if (dtype != CN_F32 && dtype != CN_BF16) CN_FAIL(CN_ERR_SHAPE, "cn_mul1_gemv_noalloc: dtype %d is neither CN_F32 nor CN_BF16", dtype);
    unsigned char* base = nullptr;
    if (int rc = static_scratch(&base)) return rc;
    Mul1Plan view = {};
    view.hidden = hidden, view.inter = inter, view.bits = bits, view.half = half, view.n32 = 8 * bits + (half ? 4 : 0);
    const Mul1Spec s = spec_of(&view, which);
    uint16_t* xh = (uint16_t*)base;
    float* xinv = (float*)(base + NA_XH_BYTES);
    float* part = (float*)(base + NA_XH_BYTES + NA_XINV_BYTES);
    const size_t plane = NA_ROWS * NA_DIM;  // the lo plane starts one full plane after the hi plane
    cudaStream_t st = (cudaStream_t)stream;
    // every region is written before it is read within one call (had_in fills xh / xinv of the live
    // slots, the GEMV fills every partial that had_out sums), so nothing has to start at zero
    if (int rc = launch_had_in(ptrs, x, xh, xinv, s, slots, t, x_div, dtype, plane, st)) return rc;
    if (int rc = launch_gemv(ptrs, xh, xinv, part, s, slots, t, plane, st)) return rc;
    dim3 grid(s.n / 128, 1, slots);
    if (dtype == CN_BF16)
        CN_CUDA(cn_launch_pdl((mul1_had_out_kernel<1>), dim3(grid), dim3(32 * t), 0, st, ptrs, part, y, s.n, ksplit(s.k), t, s.svh_off, (const int*)nullptr));
    else
        CN_CUDA(cn_launch_pdl((mul1_had_out_kernel<0>), dim3(grid), dim3(32 * t), 0, st, ptrs, part, y, s.n, ksplit(s.k), t, s.svh_off, (const int*)nullptr));
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}
