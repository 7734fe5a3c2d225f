// A chain of NVFP4 GEMV steps (one bf16 activation row) run by ONE persistent launch: the fused form of the
// decode step's projection chain. Supersedes the launch sequences of Engine::dense_ffn_w (engine/src/gen.rs:3974-3990:
// gemv_nvfp4_gu then gemv_nvfp4_w), the FusedFfn operator (engine/src/kernels.rs:6777-6840) and, for a stack of
// projections, the per-projection launches of Engine::decode_step (engine/src/gen.rs:6117-6190).
//
// Why one launch. A decode GEMV streams 15 - 100 MB; at HBM speed that is 2 - 15 us, and a kernel boundary costs
// 2 - 3 us of it (drain, launch, barrier set-up, first bytes). Here the CTAs stay resident for the whole chain:
//   - the producer warp of every CTA walks the weight bytes of ALL steps through one mbarrier ring and never stops at
//     a step boundary (weights do not depend on activations), so the ring is full when the consumers arrive;
//   - a step is cut into units of (16-row tile, 2048-column chunk) and every CTA takes an equal, contiguous share of
//     the units, whatever the row count: no wave quantisation. A tile cut between CTAs is finished by the CTA that
//     holds its first chunk; the others hand their 16 partial sums over through global memory, posted at the START of
//     their share and collected at the END of the owner's, in a fixed order (run-to-run identical bits);
//   - a step that reads what an earlier step wrote waits on that step's arrival counter (every CTA arrives once per
//     step) before it stages its activation row. Counters only grow (run number x CTAs), so a captured graph replays.
// All waits are bounded and report through the device status word. The launch is cooperative (all CTAs resident).
//
// Inner loop and activation staging are those of the one-row tensor-core GEMV (nvfp4_gemv_m1.cu): mma.sync.m16n8k16
// f16 in "word" form, activations as f16 x 2^e per 64-value block (exact for bf16), UE4M3 x tensor scale applied once
// per 16-value sub-block and row, f32 accumulation.
#include <vector>

#include "common.cuh"
#include "nvfp4_gemv.cuh"

namespace {

constexpr int NW = 8;  // consumer warps
constexpr int NTHREADS = (NW + 1) * 32;
constexpr int MAX_STAGES = 8;
constexpr int RED_DEPTH = 10;
constexpr int XB = 128;
constexpr int TX = 32;  // 36-byte blocks per row and stage
constexpr int TBAR_OFF = 128, ZERO_OFF = 224;
constexpr int ZERO2_OFF = ZERO_OFF + 2048;
constexpr int LUT_OFF = 2304;
constexpr int RED_OFF = LUT_OFF + 2048;  // [RED_DEPTH][NW][16] f32
constexpr int XS_OFF = RED_OFF + RED_DEPTH * NW * 64;
constexpr int ROWS = 16;
constexpr int PSTRIDE = TX * 36 + 16;
constexpr int STAGE_BYTES = ROWS * PSTRIDE;
static_assert(ZERO2_OFF + 16 <= LUT_OFF && TBAR_OFF + RED_DEPTH * 8 <= ZERO_OFF, "header regions overlap");

#define CN_DEV_WAIT_STEP 103
#define CN_DEV_WAIT_PART 104

struct SeqStepDev {
    const uint8_t* w0;
    const uint8_t* w1;
    const float* gs0;
    const float* gs1;
    const void* x;
    void* y;
    int rows, k;
    float limit;
    int after;    // index of the step whose completion this step waits for before it reads x (-1: none)
    int out_f32;
    int pad;
};

struct SeqParams {
    const SeqStepDev* steps;
    int nsteps;
    int stages;
    uint32_t stage_off;   // byte offset of the weight ring in shared memory (behind the longest activation row)
    int pdl;              // launched with programmatic dependent launch (a single step): wait for the predecessor grid before x is read
    unsigned int* done;   // [nsteps] arrivals: after run r every entry is (r + 1) * gridDim.x
    unsigned int* pflag;  // [nsteps][grid] run number + 1 of the last partial posted by that CTA in that step
    float* part;          // [nsteps][grid][16]
    unsigned int* runs;   // [0] completed runs, [1] exit tickets of the current run
#ifdef CN_SEQ_TRACE
    unsigned long long* trace;  // [nsteps][grid][6] globaltimer stamps of every CTA (diagnostic build only)
#endif
};

#ifdef CN_SEQ_TRACE
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define CN_STAMP(i) if (tid == 0 && p.trace) p.trace[((size_t)st * ncta + cid) * 6 + (i)] = gtime()
#else
#define CN_STAMP(i)
#endif

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, unsigned int v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// bounded wait until *p has reached `target` (counters only grow; wrap-safe compare)
__device__ __forceinline__ bool wait_reached(const unsigned int* p, unsigned int target) {
    if ((int)(ld_acquire_gpu(p) - target) >= 0) return true;
    const long long t0 = clock64();
    for (;;) {
        if ((int)(ld_acquire_gpu(p) - target) >= 0) return true;
        // about a second; at once when another CTA has already given up (nothing will arrive any more)
        if (clock64() - t0 > 2000000000LL || *(volatile int*)&g_cn_status != 0) return false;
        __nanosleep(40);
    }
}
// first unit of CTA c when U units are dealt to n CTAs in contiguous, equal shares
__device__ __forceinline__ int share_start(int c, int U, int n) { return (int)(((long long)c * U) / n); }

template <int CPS>
__global__ void __launch_bounds__(NTHREADS, CPS) nvfp4_gemv_seq_kernel(const SeqParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = (uint64_t*)smem;
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* tbar = (uint64_t*)(smem + TBAR_OFF);
    float* lut = (float*)(smem + LUT_OFF);
    float* red = (float*)(smem + RED_OFF);
    const int S = p.stages;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cid = blockIdx.x, ncta = gridDim.x;

    if (warp == NW) {
        if (lane == 0) {
            for (int s = 0; s < S; s++) {
                mbar_init(&full[s], 1);
                mbar_init(&empty[s], NW);
            }
            for (int i = 0; i < RED_DEPTH; i++) mbar_init(&tbar[i], NW);
            mbar_fence_init();
        }
        __syncwarp();
        asm volatile("bar.arrive 2, %0;" ::"n"(NTHREADS) : "memory");
        pdl_launch_dependents();
        // ------------------------------------------------------------ weight producer: every step, back to back
        const uint64_t pol = l2_policy_evict_first();
        int s = 0;
        uint32_t par = 0;
        bool first_round = true;
        for (int st = 0; st < p.nsteps; st++) {
            const SeqStepDev d = p.steps[st];
            const bool gu = d.w1 != nullptr;
            const int bpr = d.k >> 6, HC = (bpr + 15) >> 4;  // half chunks (16 blocks, the last may be shorter) per row: the unit the shares are dealt in
            const size_t row_bytes = (size_t)bpr * 36;
            const int per_cta = gu ? ROWS / 2 : ROWS;
            const int T = (d.rows + per_cta - 1) / per_cta, U = T * HC;
            const int u0 = share_start(cid, U, ncta), u1 = share_start(cid + 1, U, ncta);
            int tile = u0 / HC, hc = u0 - tile * HC;
            for (int u = u0; u < u1;) {
                // a stage: one or two half chunks of one tile (two when the tile and the share both go on)
                const int nh = min(2, min(HC - hc, u1 - u));
                const int row0 = tile * per_cta;
                const int row = gu ? row0 + (lane & 7) : row0 + lane;
                const uint8_t* base = (gu && ((lane >> 3) & 1)) ? d.w1 : d.w0;
                const uint8_t* src = (lane < ROWS && row < d.rows) ? base + (size_t)row * row_bytes : nullptr;
                const uint32_t nvalid = (uint32_t)__popc(__ballot_sync(0xffffffffu, src != nullptr));
                const uint32_t piece = (uint32_t)min(nh * 16, bpr - hc * 16) * 36u;
                if (!first_round && !mbar_wait(&empty[s], par ^ 1u)) {
                    cn_dev_fail(CN_DEV_WAIT_EMPTY);
                    return;
                }
                uint8_t* dst = smem + p.stage_off + (size_t)s * STAGE_BYTES;
                if (lane == 0) {
                    mbar_expect_tx(&full[s], nvalid * piece);
                    mbar_arrive(&full[s]);
                }
                __syncwarp();
                if (src) bulk_g2s_stream(dst + (size_t)lane * PSTRIDE, src + (size_t)hc * 16 * 36, piece, &full[s], pol);
                if (++s == S) {
                    s = 0;
                    par ^= 1u;
                    first_round = false;
                }
                u += nh, hc += nh;
                if (hc == HC) hc = 0, tile++;
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumer warps
    pdl_launch_dependents();
    if (p.pdl) pdl_wait();  // the activation row (and this plan's run counter) may come from the kernel just before this one
    const unsigned int run = *(volatile const unsigned int*)p.runs;  // completed runs before this one (stable until every CTA has left)
    const int g = lane >> 2, t = lane & 3;
    const int myq = ((g & 1) == (t >> 1)) ? (g >> 1) : -1;
    const int xb0 = 2 * warp + (g >> 2);
    const uint32_t xoff_lane = (uint32_t)XS_OFF + (uint32_t)(xb0 * XB + (((2 * (g & 3) + (t & 1)) ^ (xb0 & 7)) << 4));
    const uint32_t aoff = (uint32_t)(g * PSTRIDE + 4 * t + warp * 72);
    const int sdelta = -4 * t + (t >> 1) * 36 + 2 * (t & 1);
    const uint32_t stage_off = p.stage_off;
    int* fail_s = (int*)(smem + 216);  // set by the thread that gave up a wait between two barriers
    if (tid == 0) *fail_s = 0;
    if (tid < 4) ((uint32_t*)(smem + ZERO_OFF))[tid] = 0u;
    if (tid >= 4 && tid < 8) ((uint32_t*)(smem + ZERO2_OFF))[tid - 4] = 0u;
    asm volatile("bar.sync 2, %0;" ::"n"(NTHREADS) : "memory");  // the ring's barriers exist

    int s = 0, rslot = 0;
    uint32_t par = 0, rpar = 0;
    bool ok = true;
    for (int st = 0; st < p.nsteps && ok; st++) {
        const SeqStepDev d = p.steps[st];
        const bool gu = d.w1 != nullptr;
        const int bpr = d.k >> 6, HC = (bpr + 15) >> 4;
        const int per_cta = gu ? ROWS / 2 : ROWS;
        const int T = (d.rows + per_cta - 1) / per_cta, U = T * HC;
        const int u0 = share_start(cid, U, ncta), u1 = share_start(cid + 1, U, ncta);
        uint8_t* xs0 = smem + XS_OFF;
        float* xinv0 = (float*)(xs0 + (size_t)bpr * XB);
        // everybody has left the previous step's activations (and warp 0 has arrived on its counter)
        asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
        CN_STAMP(0);
        if (d.after >= 0) {
            if (tid == 0 && !wait_reached(p.done + d.after, (run + 1u) * (unsigned)ncta)) {
                cn_dev_fail(CN_DEV_WAIT_STEP);
                *fail_s = 1;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
        }
        if (*(volatile int*)fail_s) break;  // a wait ran out here or in warp 0's hand-over: the whole CTA leaves
        CN_STAMP(1);
        // ---- stage the activation row: bf16 -> f16 * 2^e per 64-value block, chunk i of block b at chunk i ^ (b & 7)
        {
            const float gs0 = __ldg(d.gs0), gs1 = gu ? __ldg(d.gs1) : gs0;
            const int ntask = bpr * 8;
            const char* xbase = (const char*)d.x;
            constexpr int PF = 4;
            auto load_x = [&](int task) -> uint4 { return task < ntask ? __ldcg((const uint4*)xbase + task) : make_uint4(0u, 0u, 0u, 0u); };
            uint4 pre[PF];
#pragma unroll
            for (int i = 0; i < PF; i++) pre[i] = load_x(tid + i * (NW * 32));
            for (int b = tid; b < 256; b += NW * 32) {
                const float u = ue4m3_f32((uint32_t)b, true);
                lut[b] = u * gs0;
                lut[256 + b] = u * gs1;
            }
            for (int task0 = tid; task0 < ntask; task0 += PF * NW * 32) {
#pragma unroll
                for (int pf = 0; pf < PF; pf++) {
                    const int task = task0 + pf * (NW * 32);
                    const uint4 raw = pre[pf];
                    pre[pf] = load_x(task + PF * NW * 32);
                    if (task >= ntask) break;
                    const int b = task >> 3, i = task & 7;
                    const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
                    float amax = 0.0f;
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        amax = fmaxf(amax, fabsf(__uint_as_float(u[q] << 16)));
                        amax = fmaxf(amax, fabsf(__uint_as_float(u[q] & 0xffff0000u)));
                    }
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
                    uint32_t e = (__float_as_uint(amax) >> 23) & 0xFF;
                    float mul = 1.0f, inv = 1.0f;
                    if (amax > 0.0f && e < 255) {
                        e = e < 15 ? 15 : e;
                        mul = __uint_as_float((268u - e) << 23);
                        inv = __uint_as_float((e - 14u) << 23);
                    }
                    uint32_t h[4];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const __half2 hh = __floats2half2_rn(__uint_as_float(u[q] << 16) * mul, __uint_as_float(u[q] & 0xffff0000u) * mul);
                        h[q] = *(const uint32_t*)&hh;
                    }
                    ((uint4*)(xs0 + (size_t)b * XB))[i ^ (b & 7)] = make_uint4(h[0], h[1], h[2], h[3]);
                    if (i == 0) xinv0[b] = inv;
                }
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
        CN_STAMP(2);

        // ---- this CTA's share of the step's units
        const float* xinv_lane = xinv0 + 2 * warp + (t >> 1);
        const float* lut_b = lut + (gu ? 256 : 0);
        int tile = u0 / HC, hc = u0 - tile * HC;
        float acc0 = 0.0f, acc1 = 0.0f;
        int c_first = hc;
        for (int u = u0; u < u1 && ok;) {
            const int nh = min(2, min(HC - hc, u1 - u));
            const int ng = min(nh * 16, bpr - hc * 16) >> 1;  // groups of two blocks in this stage
            if (!mbar_wait(&full[s], par)) {
                cn_dev_fail(CN_DEV_WAIT_FULL);
                ok = false;
                break;
            }
#ifdef CN_SEQ_TRACE
            if (u == u0) CN_STAMP(3);
#endif
            const uint8_t* pa0 = smem + stage_off + (size_t)s * STAGE_BYTES + aoff;
            const uint32_t xoff = xoff_lane + (uint32_t)(hc * 16 * XB);
            uint32_t bq[4];
#pragma unroll
            for (int q = 0; q < 4; q++) bq[q] = myq == q ? xoff : (uint32_t)ZERO_OFF;
            const float* xip = xinv_lane + hc * 16;
            auto group = [&](int j) {
                const uint8_t* pa = pa0 + j * (NW * 72);
                const uint8_t* pb = pa + 8 * PSTRIDE;
                float cc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int off = (q >> 1) * 36 + 4 + 16 * (q & 1);
                    uint32_t ha[4], hb[4];
                    e2m1x8_to_f16x2(*(const uint32_t*)(pa + off), ha);
                    e2m1x8_to_f16x2(*(const uint32_t*)(pb + off), hb);
                    const uint4 xv = *(const uint4*)(smem + bq[q] + j * 2048);
                    mma16816(cc, ha[0], hb[0], ha[1], hb[1], xv.x, xv.y);
                    mma16816(cc, ha[2], hb[2], ha[3], hb[3], xv.z, xv.w);
                }
                const uint8_t* sc = pa + sdelta;
                const float s0 = lut[sc[0]], s1 = lut[sc[1]], s2 = lut_b[sc[8 * PSTRIDE]], s3 = lut_b[sc[8 * PSTRIDE + 1]];
                const float xi = xip[16 * j];
                acc0 = fmaf(fmaf(cc[1], s1, cc[0] * s0), xi, acc0);
                acc1 = fmaf(fmaf(cc[3], s3, cc[2] * s2), xi, acc1);
            };
            if (ng == TX / 2) {
                group(0);
                group(1);
            } else {
                if (warp < ng) group(0);
                if (warp + NW < ng) group(1);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            if (++s == S) {
                s = 0;
                par ^= 1u;
            }
            u += nh, hc += nh;
            const bool tile_ends = hc == HC, share_ends = u == u1;
            if (tile_ends || share_ends) {
                // the quad's four lanes hold two columns each; then the eight warps' K ranges meet in shared memory
                float a = acc0, b = acc1;
                a += __shfl_xor_sync(0xffffffffu, a, 1);
                b += __shfl_xor_sync(0xffffffffu, b, 1);
                a += __shfl_xor_sync(0xffffffffu, a, 2);
                b += __shfl_xor_sync(0xffffffffu, b, 2);
                float* rb = red + rslot * (NW * 16);
                if (t == 0) {
                    rb[warp * 16 + g] = a;
                    rb[warp * 16 + g + 8] = b;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&tbar[rslot]);
                if (warp == 0) {
                    if (!mbar_wait(&tbar[rslot], rpar)) {
                        cn_dev_fail(CN_DEV_WAIT_FULL);
                        *fail_s = 1;
                    } else {
                        float v = 0.0f;
                        if (lane < 16) {
                            v = rb[lane];
                            for (int w = 1; w < NW; w++) v += rb[w * 16 + lane];
                        }
                        if (c_first != 0) {
                            // the tile's first chunks belong to an earlier CTA: hand the 16 sums over
                            float* dst = p.part + ((size_t)st * ncta + cid) * 16;
                            if (lane < 16) __stcg(dst + lane, v);
                            __syncwarp();
                            if (lane == 0) {
                                __threadfence();
                                st_release_gpu(p.pflag + (size_t)st * ncta + cid, run + 1u);
                            }
                        } else {
                            if (!tile_ends) {
                                // the tile goes on in the following CTAs, which took it first and have posted by now
                                const int tile_end_u = (tile + 1) * HC;
                                for (int cc2 = cid + 1; cc2 < ncta; cc2++) {
                                    const int a2 = share_start(cc2, U, ncta), b2 = share_start(cc2 + 1, U, ncta);
                                    if (a2 >= tile_end_u) break;
                                    if (b2 == a2) continue;
                                    // one lane polls, the warp follows its verdict together
                                    int got = lane == 0 ? (int)wait_reached(p.pflag + (size_t)st * ncta + cc2, run + 1u) : 1;
                                    got = __shfl_sync(0xffffffffu, got, 0);
                                    if (!got) {
                                        if (lane == 0) {
                                            cn_dev_fail(CN_DEV_WAIT_PART);
                                            *fail_s = 1;
                                        }
                                        break;
                                    }
                                    if (lane < 16) v += __ldcg(p.part + ((size_t)st * ncta + cc2) * 16 + lane);
                                }
                            }
                            const float up = __shfl_down_sync(0xffffffffu, v, 8);
                            const int row = tile * per_cta + lane;
                            if (lane < per_cta && row < d.rows) {
                                const float r = gu ? act_gu(v, up, d.limit) : v;
                                if (d.out_f32)
                                    ((float*)d.y)[row] = r;
                                else
                                    ((__nv_bfloat16*)d.y)[row] = __float2bfloat16_rn(r);
                            }
                        }
                    }
                }
                if (++rslot == RED_DEPTH) {
                    rslot = 0;
                    rpar ^= 1u;
                }
                acc0 = acc1 = 0.0f;
                c_first = 0;
            }
            if (hc == HC) hc = 0, tile++;
        }
        // this CTA's outputs of the step are written: arrive (warp 0 wrote them, lane 0 of it publishes)
        if (warp == 0) {
            __syncwarp();
            CN_STAMP(4);
            if (lane == 0) {
                __threadfence();
                red_release_gpu_add(p.done + st, 1u);
            }
            CN_STAMP(5);
        }
    }
    // the last CTA to leave closes the run: later launches see one more completed run
    if (tid == 0) {
        __threadfence();
        const unsigned int ticket = atomicAdd(p.runs + 1, 1u);
        if (ticket == (unsigned)ncta - 1u) {
            p.runs[1] = 0u;
            __threadfence();
            atomicAdd(p.runs, 1u);
        }
    }
}

struct SeqPlan {
    SeqStepDev* steps;
    unsigned int *done, *pflag, *runs;
    float* part;
    int nsteps, grid, stages, cps, pdl;
    uint32_t stage_off;
    size_t smem;
    int device;
};

}  // namespace

extern "C" int cn_nvfp4_seq_destroy(void* plan) {
    SeqPlan* p = (SeqPlan*)plan;
    if (!p) return CN_OK;
    cudaFree(p->steps), cudaFree(p->done), cudaFree(p->pflag), cudaFree(p->runs), cudaFree(p->part);
    delete p;
    return CN_OK;
}

extern "C" int cn_nvfp4_seq_create(void** plan_out, const cn_gemv_step* steps, int nsteps) {
    if (!plan_out || !steps || nsteps < 1 || nsteps > 4096) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_seq_create: %d steps (1..4096)", nsteps);
    std::vector<SeqStepDev> host((size_t)nsteps);
    int kmax = 0;
    for (int i = 0; i < nsteps; i++) {
        const cn_gemv_step& a = steps[i];
        if (a.rows <= 0 || a.k < 2048 || a.k % 256 != 0 || a.k > 32768)
            CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_seq_create: step %d: k = %d must be a multiple of 256 and at least 2048, rows %d positive", i, a.k, a.rows);
        if (!a.w || !a.gs || !a.x || !a.y) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_seq_create: step %d: null pointer", i);
        if (((uintptr_t)a.w & 15) || ((uintptr_t)a.w_up & 15) || ((uintptr_t)a.x & 15))
            CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_seq_create: step %d: weight and activation pointers must be 16-byte aligned", i);
        if (a.after >= i) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_seq_create: step %d waits for step %d, which does not come before it", i, a.after);
        SeqStepDev d = {};
        d.w0 = (const uint8_t*)a.w, d.w1 = (const uint8_t*)a.w_up, d.gs0 = a.gs, d.gs1 = a.gs_up ? a.gs_up : a.gs, d.x = a.x, d.y = a.y;
        d.rows = a.rows, d.k = a.k, d.limit = a.limit, d.after = a.after < 0 ? -1 : a.after, d.out_f32 = a.out_f32 ? 1 : 0;
        host[(size_t)i] = d;
        if (a.k > kmax) kmax = a.k;
    }
    SeqPlan* p = new SeqPlan();
    p->nsteps = nsteps;
    cudaError_t e = cudaGetDevice(&p->device);
    int sms = 0;
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, p->device);
    // three CTAs per SM when the longest activation row leaves each of them a ring of three stages, else two
    const int bprmax = kmax / 64;
    p->stage_off = (uint32_t)((XS_OFF + bprmax * XB + bprmax * 4 + 127) & ~127);
    int cps = 3;
    int stages = (int)(((227 * 1024) / cps - 1024 - (long long)p->stage_off) / STAGE_BYTES);
    if (stages < 3) {
        cps = 2;
        stages = (int)(((227 * 1024) / cps - 1024 - (long long)p->stage_off) / STAGE_BYTES);
    }
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) {
        delete p;
        CN_FAIL(CN_ERR_LIMIT, "cn_nvfp4_seq_create: k = %d leaves no room for a weight ring beside the activation row", kmax);
    }
    // one step that waits for nothing: a plain launch that may overlap its predecessor's tail (the CTAs still hand partial
    // sums to one another, which a grid no larger than the machine allows); chains need every CTA resident: cooperative
    p->cps = cps, p->pdl = (nsteps == 1 && host[0].after < 0) ? 1 : 0;
    p->stages = stages, p->grid = sms * cps, p->smem = p->stage_off + (size_t)stages * STAGE_BYTES;
    auto step = [&](cudaError_t r) { if (e == cudaSuccess) e = r; };
    const size_t n = (size_t)nsteps, g = (size_t)p->grid;
    step(cudaMalloc(&p->steps, n * sizeof(SeqStepDev)));
    step(cudaMalloc(&p->done, n * 4));
    step(cudaMalloc(&p->pflag, n * g * 4));
    step(cudaMalloc(&p->part, n * g * 64));
    step(cudaMalloc(&p->runs, 8));
    if (e == cudaSuccess) step(cudaMemcpy(p->steps, host.data(), n * sizeof(SeqStepDev), cudaMemcpyHostToDevice));
    if (e == cudaSuccess) step(cudaMemset(p->done, 0, n * 4));
    if (e == cudaSuccess) step(cudaMemset(p->pflag, 0, n * g * 4));
    if (e == cudaSuccess) step(cudaMemset(p->runs, 0, 8));
    if (e != cudaSuccess) {
        cn_nvfp4_seq_destroy(p);
        CN_FAIL(CN_ERR_CUDA, "cn_nvfp4_seq_create: %s", cudaGetErrorString(e));
    }
    *plan_out = p;
    return CN_OK;
}

#ifdef CN_SEQ_TRACE
static unsigned long long* g_seq_trace = nullptr;
extern "C" void cn_nvfp4_seq_trace(unsigned long long* buf) { g_seq_trace = buf; }
#endif

extern "C" int cn_nvfp4_seq_run(void* plan, cn_stream_t stream) {
    SeqPlan* p = (SeqPlan*)plan;
    if (!p) CN_FAIL(CN_ERR_SHAPE, "cn_nvfp4_seq_run: null plan");
    SeqParams a;
    a.steps = p->steps, a.nsteps = p->nsteps, a.stages = p->stages, a.stage_off = p->stage_off, a.done = p->done, a.pflag = p->pflag, a.part = p->part,
    a.runs = p->runs, a.pdl = p->pdl;
#ifdef CN_SEQ_TRACE
    a.trace = g_seq_trace;
#endif
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p->grid), cfg.blockDim = dim3(NTHREADS), cfg.dynamicSmemBytes = p->smem, cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute at[1];
    if (p->pdl) {
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
    } else {
        // cooperative: the CTAs wait on one another across steps, so all of them must be resident (the launch fails otherwise)
        at[0].id = cudaLaunchAttributeCooperative;
        at[0].val.cooperative = 1;
    }
    cfg.attrs = at, cfg.numAttrs = 1;
    if (p->cps == 3) {
        CN_ALLOW_SMEM(nvfp4_gemv_seq_kernel<3>, 75 * 1024);
        CN_CUDA(cudaLaunchKernelEx(&cfg, nvfp4_gemv_seq_kernel<3>, a));
    } else {
        CN_ALLOW_SMEM(nvfp4_gemv_seq_kernel<2>, 113 * 1024);
        CN_CUDA(cudaLaunchKernelEx(&cfg, nvfp4_gemv_seq_kernel<2>, a));
    }
    return CN_OK;
}
