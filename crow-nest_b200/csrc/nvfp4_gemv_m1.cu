// NVFP4 GEMV for 1..8 bf16 activation rows (decode, MTP verify, and every combo of the routed-expert
// step): persistent CTAs, tensor-core inner loop in "word" form. Supersedes gemv_nvfp4_w / _gu / _wm /
// _gum (engine/src/kernels_p2.rs:355-530) and the routed record kernels gemv_fp4(_b), gemv_fp4_ptrb
// (engine/src/kernels.rs:118-195) for bf16 activations.
//
// A CTA owns a list of 16-row tiles (tile = blockIdx.x + i * gridDim.x). The activation rows are staged
// once per CTA (f16 with a power-of-two scale per 64-value block: exact for bf16), the producer warp
// streams the tiles' weight bytes through one mbarrier ring without draining it between tiles, and
// eight consumer warps split the K range of every stage between them; their 16 sums per tile meet in a
// small shared-memory ring with one mbarrier per slot, so no CTA-wide barrier sits in the loop.
// With more than one activation row the C columns are packed (four activation rows x the two sub-blocks
// of a pair: 8 MMAs per group for up to four rows, 16 for eight); row i of an m-row call is summed in
// exactly the order of a one-row call.
// When the tiles do not fill the last wave and a CTA's share is long enough (the down projection), or the
// tiles are too few to fill the machine (a tensor-parallel rank's share of it), the launch is made of
// clusters of two or four CTAs that take a part of K each (see the helpers below).
// The LN variant (one activation row) also stores the output rows as 16-byte lines into the line buffers of
// the other GPUs of a tensor-parallel group: the exchange that follows the projection starts in its epilogue.
//
// Inner loop. mma.sync.m16n8k16 (f16 x f16 -> f32) takes the f16x2 registers that
// cvt.rn.f16x2.e2m1x2 makes: A = 16 weight rows x 16 codes, B = the matching activations. The order
// of k inside an MMA is free as long as A and B agree, so it is chosen to make the loads wide:
// a "group" is two 36-byte blocks (eight 16-code sub-blocks), a "pair" is two sub-blocks = 16 code
// bytes of a row, and thread t of a quad takes word t of the pair: ONE 32-bit shared-memory load per
// row feeds four cvt and two MMAs (bytes 0,1 -> first MMA, bytes 2,3 -> second). Column j of the C
// tile collects sub-block j of the group: in pair q only columns 2q and 2q+1 have non-zero B, and
// since B's column index is the lane's quad number, a lane has activations for exactly one pair and
// reads a 16-byte zero chunk for the other three (one select + one 128-bit load per pair). After the
// eight MMAs of a group the C tile holds eight sub-block sums per row, and the UE4M3 scale x tensor
// scale x inverse activation scale is applied once per sub-block and row.
// Products are exact, accumulation is the tensor core's f32 and f32 FMAs in a fixed order.
#include "common.cuh"
#include "nvfp4_gemv.cuh"

namespace {

constexpr int NW = 8;  // consumer warps
constexpr int NTHREADS = (NW + 1) * 32;
constexpr int MAX_STAGES = 8;
constexpr int RED_DEPTH = 10;  // tile sums in flight: a warp runs at most MAX_STAGES chunks ahead of warp 0
constexpr int XB = 128;        // one 64-value block of f16 activations, 16-byte chunks XOR-swizzled
// header: mbarriers (full, empty, tile), two 16-byte zero chunks 2048 B apart (the second group of a chunk
// reads everything 2048 B further on), scale table, tile sums
constexpr int TBAR_OFF = 128, ZERO_OFF = 224;
constexpr int ZERO2_OFF = ZERO_OFF + 2048;
constexpr int LUT_OFF = 2304;
constexpr int RED_OFF = LUT_OFF + 2048;  // [RED_DEPTH][NW][16] f32
static_assert(ZERO2_OFF + 16 <= LUT_OFF && TBAR_OFF + RED_DEPTH * 8 <= ZERO_OFF, "header regions overlap");
constexpr int ROWS = 16;

// ---- two-CTA cluster helpers (K range of a tile shared between the CTAs of a pair)
// f32 [8 slots][up to 3 senders][16] sums from the other CTAs of a cluster of two or four, then a barrier per slot
constexpr int XCH_OFF = 256, XCH_SLOTS = 8, XBAR_OFF = XCH_OFF + XCH_SLOTS * 3 * 64;
static_assert(XBAR_OFF + XCH_SLOTS * 8 <= ZERO2_OFF, "the cluster exchange overlaps the header");
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_addr(const void* local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_peer_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void arrive_peer(uint32_t bar_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_addr) : "memory");
}
// bounded wait with cluster-scope acquire: the peer CTA's stores before its arrive are visible afterwards
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
    const long long t0 = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
        if (clock64() - t0 > 2000000000LL) return false;
    }
}

// Diagnostic build (-DCN_M1_TRACE): every CTA stamps %globaltimer at entry (0), after the wait on the predecessor grid (1),
// after the activations are staged (2), when its first stage has landed (3), at the end of its consumers (4), and its
// producer warp at its first (5) and after its last (6) bulk copy. Off in the product build.
#ifdef CN_M1_TRACE
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define CN_STAMP(i) if (p.trace) p.trace[(size_t)blockIdx.x * 8 + (i)] = gtime()
#else
#define CN_STAMP(i)
#endif

// Tensor-parallel line output, called by all lanes of warp 0: lane l < 16 holds output row row0 + l as r. Four rows make one
// 16-byte line {rows 0-1, number, rows 2-3, number}; lane (d, j) = (lane >> 2, lane & 3) stores line j of the tile into
// rank d's line buffer. Plain stores: the receiver polls the numbers, nothing waits for an acknowledgement here.
__device__ __forceinline__ void push_lines(const GemvParams& p, int row0, int nrows, float r, int lane, unsigned int seq, unsigned int buf) {
    const uint32_t b = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(r));
    const uint32_t pair = b | (__shfl_down_sync(0xffffffffu, b, 1) << 16);  // even lanes: rows l, l + 1
    const uint32_t next = __shfl_down_sync(0xffffffffu, pair, 2);           // lanes 4 j: rows 4 j + 2, 4 j + 3
    const int j = lane & 3, d = lane >> 2;
    const uint32_t a0 = __shfl_sync(0xffffffffu, pair, 4 * j), a1 = __shfl_sync(0xffffffffu, next, 4 * j);
    if (d < p.yl_world && p.yl[d] != 0ull && 4 * j < nrows) {
        uint4* dst = (uint4*)(uintptr_t)(p.yl[d] + (unsigned long long)buf * p.yl_stride) + ((p.yl_row0 + row0) >> 2) + j;
        asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(a0), "r"(seq), "r"(a1), "r"(seq) : "memory");
    }
}

// TX: 36-byte blocks per row and stage (32 or 16); the last chunk of a row may be shorter
// CPS: CTAs per SM the register allocation must allow; MT: activation rows (1, 2, 4 or 8; p.m of them live)
// KS: 1, or 2 = launched as two-CTA clusters, the CTAs of a pair sharing every tile's K range (MT = 1 only)
// LN: tensor-parallel line output compiled in (one activation row only); without it the kernel carries none of that code
template <int TX, int CPS, int MT, int KS = 1, bool LN = false>
__global__ void __launch_bounds__(NTHREADS, CPS) nvfp4_gemv_m1_kernel(const GemvParams p) {
    static_assert(!LN || MT == 1, "line output takes one activation row");
    extern __shared__ __align__(128) uint8_t smem[];
    if (threadIdx.x == 0) { CN_STAMP(0); }
    const float gs0_early = __ldg(p.gs0), gs1_early = __ldg(p.gs1);  // tensor scales: asked for first, used late
    constexpr int pstride = TX * 36 + 16;  // padded: the eight rows of a quad column hit distinct banks
    constexpr int stage_bytes = ROWS * pstride;
    constexpr int GPW = TX / 2 / NW > 0 ? TX / 2 / NW : 1;  // groups per warp and full chunk
    // KS = 2 (one activation row only): the CTAs of a cluster pair walk the same tiles, each over half of K
    static_assert(KS == 1 || MT == 1, "the K range is shared between CTAs for one activation row only");
    const int crank = KS > 1 ? (int)(blockIdx.x % KS) : 0;
    const int cid = KS > 1 ? (int)(blockIdx.x / KS) : (int)blockIdx.x, ncl = KS > 1 ? (int)(gridDim.x / KS) : (int)gridDim.x;
    const int bpr_all = p.k >> 6;
    const int bpr = bpr_all / KS, b0 = crank * bpr;  // this CTA's blocks of every row: [b0, b0 + bpr)
    const size_t row_bytes = (size_t)bpr_all * 36;
    const int nch = (bpr + TX - 1) / TX;
    const int S = p.stages;
    const uint8_t* w0 = p.w0 + (size_t)b0 * 36;
    const uint8_t* w1 = p.w1 ? p.w1 + (size_t)b0 * 36 : nullptr;
    const char* xbase = (const char*)p.x + (size_t)b0 * 128;
    char* ybase = (char*)p.y;
    if (p.ids) {
        // Routed form: ids, order and the tables may come from the kernels just before this one, and a CTA whose
        // expert is not resident returns at once. Every thread therefore waits for the predecessor grid first, so that
        // a grid in which every CTA returns early still completes only after its predecessor has, and a later
        // kernel's wait on this grid keeps covering the whole chain.
        pdl_wait();
        const int c = p.order ? p.order[blockIdx.y] : (int)blockIdx.y;
        const int e = p.ids[c];
        if (e < 0 || (p.experts > 0 && e >= p.experts)) return;  // uniform over the CTA, before any barrier
        w0 = (const uint8_t*)p.tab0[e];
        if (!w0) return;
        w1 = p.tab1 ? (const uint8_t*)p.tab1[e] : (p.fused_up_rows > 0 ? w0 + (size_t)p.fused_up_rows * row_bytes : nullptr);
        xbase += (size_t)(c / p.x_div) * p.k * 2;
        ybase = p.yptrs ? (char*)p.yptrs[c] : ybase + (size_t)c * p.ldy * (p.out_f32 ? 4 : 2);
    }
    const bool gu = w1 != nullptr;

    uint64_t* full = (uint64_t*)smem;
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* tbar = (uint64_t*)(smem + TBAR_OFF);  // [RED_DEPTH] one per tile-sum buffer
    float* lut = (float*)(smem + LUT_OFF);  // [2][256] ue4m3 * gs
    float* red = (float*)(smem + RED_OFF);  // [red_depth][NW][MT][16] partial sums of a tile
    const int RD = p.red_depth;             // tile sums in flight (<= RED_DEPTH)
    const uint32_t xs_off = (uint32_t)(RED_OFF + RD * NW * MT * 64);
    uint8_t* xs0 = smem + xs_off;           // [MT][bpr][128] f16 activations
    const uint32_t XS = (uint32_t)bpr * XB;  // bytes of one activation row
    float* xinv0 = (float*)(xs0 + (size_t)MT * XS);  // [MT][bpr]
    uint8_t* stage0 = (uint8_t*)(xinv0 + ((MT * bpr + 3) & ~3));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int per_cta = gu ? ROWS / 2 : ROWS;  // gate/up: 8 indices, row slots 0-7 gate, 8-15 up
    const int ntiles = (p.rows + per_cta - 1) / per_cta;

    // The producer warp sets up the ring's barriers itself and starts streaming at once (the weights do not
    // depend on the previous kernel); the consumers meet it on named barrier 2 before their first wait.
    if (warp == NW) {
        // one barrier per lane and round: S full + S empty + RD tile-sum (+ the pair's exchange slots), side by side
        for (int i = lane; i < 2 * S + RD + (KS > 1 ? XCH_SLOTS : 0); i += 32) {
            if (i < S) mbar_init(&full[i], 1);
            else if (i < 2 * S) mbar_init(&empty[i - S], NW);
            else if (i < 2 * S + RD) mbar_init(&tbar[i - 2 * S], NW);
            else mbar_init((uint64_t*)(smem + XBAR_OFF) + (i - 2 * S - RD), KS - 1);  // one arrival per other CTA of the cluster
        }
#ifdef CN_M1_TRACE
        if (lane == 0) { CN_STAMP(7); }
#endif
        mbar_fence_init();
        __syncwarp();
        asm volatile("bar.arrive 2, %0;" ::"n"(NTHREADS) : "memory");
        pdl_launch_dependents();
    }
    if (KS > 1) cluster_sync_all();  // the first CTA's barriers exist before anything is sent to them

    if (warp == NW) {
        // ------------------------------------------------------------ weight producer warp
        const uint64_t pol = l2_policy_evict_first();
        int s = 0;
        uint32_t par = 0;  // parity of the current use of stage s
        bool first_round = true, pfail = false, waited_pred = p.ids != nullptr;  // the routed form has waited already
        for (int tile = cid; tile < ntiles && !pfail; tile += ncl) {
            const int row0 = tile * per_cta;
            const int row = gu ? row0 + (lane & 7) : row0 + lane;
            const uint8_t* base = (gu && ((lane >> 3) & 1)) ? w1 : w0;
            const uint8_t* src = (lane < ROWS && row < p.rows) ? base + (size_t)row * row_bytes : nullptr;
            const uint32_t nvalid = (uint32_t)__popc(__ballot_sync(0xffffffffu, src != nullptr));
            for (int c = 0; c < nch; c++) {
                const int nblk = min(TX, bpr - c * TX);
                const uint32_t piece = (uint32_t)nblk * 36u;
                if (LN && !first_round && !waited_pred) {
                    // The ring is full: a slot frees only once the consumers run, and they wait for the predecessor grid.
                    // The producer waits for it too (a dependency wait, not a spin) so that the bounded wait below
                    // times the consumers alone, however long a predecessor that waits for other GPUs takes.
                    pdl_wait();
                    waited_pred = true;
                }
                if (!first_round && !mbar_wait(&empty[s], par ^ 1u)) {
                    cn_dev_fail(CN_DEV_WAIT_EMPTY);
                    pfail = true;
                    break;
                }
                uint8_t* st = stage0 + (size_t)s * stage_bytes;
                if (lane == 0) {
                    mbar_expect_tx(&full[s], nvalid * piece);
                    mbar_arrive(&full[s]);
                }
                __syncwarp();
                if (src) bulk_g2s_stream(st + (size_t)lane * pstride, src + (size_t)c * TX * 36, piece, &full[s], pol);
                if (lane == 0 && first_round && s == 0) { CN_STAMP(5); }
                if (++s == S) {
                    s = 0;
                    par ^= 1u;
                    first_round = false;
                }
            }
        }
        if (lane == 0) { CN_STAMP(6); }
        if (KS > 1) cluster_sync_all();  // nobody leaves while a CTA of the cluster may still send or receive
        return;
    }

    // ---------------------------------------------------------------- consumer warps: the activation rows and the scale table.
    // The first activation loads are issued right after the wait on the previous kernel and the table is built while they
    // fly; each later load is issued before the previous chunk is converted.
    pdl_launch_dependents();
    pdl_wait();  // the activations may come from the previous kernel of the stream
    if (threadIdx.x == 0) { CN_STAMP(1); }
    // the number of this exchange (tensor-parallel line output) from the step counter, which was advanced at the step's start
    const unsigned int line_epoch = LN ? *(volatile const unsigned int*)p.yl_epoch : 0u;
    const unsigned int line_seq = line_epoch * 4096u + (unsigned int)p.yl_tag, line_buf = (unsigned int)p.yl_buf ^ ((unsigned int)p.yl_flip & line_epoch & 1u);
    const int ntask = MT * bpr * 8;
    auto load_x = [&](int task) -> uint4 {
        // task = (row * bpr + block) * 8 + chunk; rows beyond p.m read as zero
        return (task < ntask && (MT == 1 || (task >> 3) < p.m * bpr)) ? __ldcg((const uint4*)xbase + task) : make_uint4(0u, 0u, 0u, 0u);
    };
    // PF loads of every thread are in flight at any time: the staging loop costs about one trip to L2 per PF tasks
    constexpr int PF = CPS >= 4 ? 2 : 4;
    uint4 pre[PF];
#pragma unroll
    for (int i = 0; i < PF; i++) pre[i] = load_x(tid + i * (NW * 32));
    if (tid < 4) ((uint32_t*)(smem + ZERO_OFF))[tid] = 0u;
    if (tid >= 4 && tid < 8) ((uint32_t*)(smem + ZERO2_OFF))[tid - 4] = 0u;
    {
        const float g1 = gu ? gs1_early : gs0_early;
        for (int b = tid; b < 256; b += NW * 32) {
            const float u = ue4m3_f32((uint32_t)b, true);
            lut[b] = u * gs0_early;
            lut[256 + b] = u * g1;
        }
    }
    bool ok = true;
    // bf16 -> f16 * 2^e per 64-value block, chunk i of block b stored at chunk i ^ (b & 7). Eight lanes per block,
    // one 16-byte chunk each, straight from global memory (k % 256 == 0 makes every warp wholly in or out of range).
    for (int task0 = tid; task0 < ntask; task0 += PF * NW * 32) {
#pragma unroll
      for (int pf = 0; pf < PF; pf++) {
        const int task = task0 + pf * (NW * 32);
        const uint4 raw = pre[pf];
        pre[pf] = load_x(task + PF * NW * 32);
        if (task >= ntask) break;  // uniform over the warp
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
        const int blk = MT == 1 ? b : b % bpr;
        ((uint4*)(xs0 + (size_t)b * XB))[i ^ (blk & 7)] = make_uint4(h[0], h[1], h[2], h[3]);
        if (i == 0) xinv0[b] = inv;
      }
    }
    asm volatile("bar.sync 2, %0;" ::"n"(NTHREADS) : "memory");  // staging done, and the ring's barriers are initialised
    if (threadIdx.x == 0) { CN_STAMP(2); }

    // ---------------------------------------------------------------- main loop
    const int g = lane >> 2, t = lane & 3;
    // the one pair of a group whose B columns this lane fills (column g = sub-block g of the group, and the
    // k slots of thread t belong to sub-block 2q + (t >> 1) of pair q): -1 = none
    const int myq = ((g & 1) == (t >> 1)) ? (g >> 1) : -1;
    // byte offset (from smem) of this lane's 16 activations in the first group of a chunk: block 2 warp + (g >> 2),
    // chunk 2 (g & 3) + (t & 1), swizzled by the block index mod 8, which chunk and group number do not change
    const int xb0 = 2 * warp + (g >> 2);
    const uint32_t xoff_lane = xs_off + (uint32_t)(xb0 * XB + (((2 * (g & 3) + (t & 1)) ^ (xb0 & 7)) << 4));
    const uint32_t aoff = (uint32_t)(g * pstride + 4 * t + warp * 72);
    const int sdelta = -4 * t + (t >> 1) * 36 + 2 * (t & 1);  // from a row's code word to its two scale bytes
    const float* xinv_lane = xinv0 + 2 * warp + (t >> 1);  // row m: + m * bpr
    const float* lut_b = lut + (gu ? 256 : 0);  // gate/up: rows 8-15 are up rows
    // More than one activation row: "packed columns". Column g of the C tile = activation row (g >> 1) of a pass of
    // four rows, sub-block (g & 1) of the pair in hand, so the two MMAs of a pair serve four rows at once and a lane
    // (g, t) ends up with the sums of activation row t for weight rows g and g + 8. A lane fills column g where its
    // k slots belong to that column's sub-block (t >> 1 == g & 1) and reads the zero chunk otherwise. A pair's C tile
    // is scaled on its own (every lane looks up both rows' eight scales of a group), and the four pairs of a group keep
    // separate running sums that are added as (p0 + p1) + (p2 + p3) at the end of the tile: the order in which the
    // one-row form's quad shuffle adds them, which keeps row i of an m-row call bit-identical to a one-row call.
    constexpr int NP = MT > 4 ? 2 : 1;  // passes of four activation rows
    const bool live = MT > 1 && (t >> 1) == (g & 1) && (g >> 1) < MT;
    uint32_t xq_lane[4];
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const int blk = 2 * warp + (q >> 1);
        xq_lane[q] = live ? xs_off + (uint32_t)((g >> 1) * XS + blk * XB + (((4 * (q & 1) + t) ^ (blk & 7)) << 4)) : (uint32_t)ZERO_OFF;
    }
    const uint32_t cstep = live ? (uint32_t)(TX * XB) : 0u, pstep = live ? 4u * XS : 0u;
    const int mrow = t < MT ? t : MT - 1;  // this lane's activation row of a pass (lanes without one compute a copy)

    int s = 0, rslot = 0;
    uint32_t par = 0, rpar = 0;
    int titer = 0;
    for (int tile = cid; tile < ntiles && ok; tile += ncl, titer++) {
        float acc0[MT], acc1[MT];  // one row: rows g and g + 8 of the tile, this lane's two columns
        float pk0[NP][4], pk1[NP][4];  // packed columns: rows g and g + 8, activation row t of each pass, per pair
#pragma unroll
        for (int m = 0; m < MT; m++) acc0[m] = acc1[m] = 0.0f;
#pragma unroll
        for (int ps = 0; ps < NP; ps++)
#pragma unroll
            for (int q = 0; q < 4; q++) pk0[ps][q] = pk1[ps][q] = 0.0f;
        for (int c = 0; c < nch; c++) {
            const int ng = min(TX, bpr - c * TX) >> 1;  // groups of two blocks in this chunk
            if (!mbar_wait(&full[s], par)) {
                cn_dev_fail(CN_DEV_WAIT_FULL);
                ok = false;
                break;
            }
#ifdef CN_M1_TRACE
            if (threadIdx.x == 0 && titer == 0 && c == 0) { CN_STAMP(3); }
#endif
            const uint8_t* pa0 = stage0 + (size_t)s * stage_bytes + aoff;
            const uint32_t xoff = xoff_lane + (uint32_t)(c * TX * XB);
            if constexpr (MT == 1) {
                // where this lane's B registers of pair q come from: its activations or the zero chunk
                uint32_t bq[4];
#pragma unroll
                for (int q = 0; q < 4; q++) bq[q] = myq == q ? xoff : (uint32_t)ZERO_OFF;
                const float* xip = xinv_lane + c * TX;
                auto group = [&](int j) {
                    const uint8_t* pa = pa0 + j * (NW * 72);
                    const uint8_t* pb = pa + 8 * pstride;
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
                    // columns 2t, 2t + 1 of C = sub-blocks 2t, 2t + 1 of the group: block t >> 1, scale bytes 2 (t & 1), + 1
                    const uint8_t* sc = pa + sdelta;
                    const float s0 = lut[sc[0]], s1 = lut[sc[1]], s2 = lut_b[sc[8 * pstride]], s3 = lut_b[sc[8 * pstride + 1]];
                    const float xi = xip[16 * j];
                    acc0[0] = fmaf(fmaf(cc[1], s1, cc[0] * s0), xi, acc0[0]);
                    acc1[0] = fmaf(fmaf(cc[3], s3, cc[2] * s2), xi, acc1[0]);
                };
                if (ng == TX / 2) {  // a full chunk: every warp has all its groups, nothing to test between them
#pragma unroll
                    for (int j = 0; j < GPW; j++) group(j);
                } else {
#pragma unroll
                    for (int j = 0; j < GPW; j++)
                        if (warp + NW * j < ng) group(j);
                }
            } else {
                const float* xip = xinv0 + 2 * warp + c * TX;
                auto group = [&](int j) {
                    const uint8_t* pa = pa0 + j * (NW * 72);
                    const uint8_t* pb = pa + 8 * pstride;
                    // the scale bytes of rows g and g + 8: one word per 64-value block
                    const uint8_t* sr = pa - 4 * t;
                    const uint32_t sw0[2] = {*(const uint32_t*)sr, *(const uint32_t*)(sr + 36)};
                    const uint32_t sw1[2] = {*(const uint32_t*)(sr + 8 * pstride), *(const uint32_t*)(sr + 8 * pstride + 36)};
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int off = (q >> 1) * 36 + 4 + 16 * (q & 1);
                        uint32_t ha[4], hb[4];
                        e2m1x8_to_f16x2(*(const uint32_t*)(pa + off), ha);
                        e2m1x8_to_f16x2(*(const uint32_t*)(pb + off), hb);
                        // table look-ups by byte offset: one shift and one mask per scale byte
                        const uint32_t wa = sw0[q >> 1], wb = sw1[q >> 1];
                        const uint32_t o0 = (q & 1) ? (wa >> 14) & 0x3fcu : (wa << 2) & 0x3fcu, o1 = (q & 1) ? (wa >> 22) & 0x3fcu : (wa >> 6) & 0x3fcu;
                        const uint32_t o2 = (q & 1) ? (wb >> 14) & 0x3fcu : (wb << 2) & 0x3fcu, o3 = (q & 1) ? (wb >> 22) & 0x3fcu : (wb >> 6) & 0x3fcu;
                        const float s0 = *(const float*)((const char*)lut + o0), s1 = *(const float*)((const char*)lut + o1);
                        const float s2 = *(const float*)((const char*)lut_b + o2), s3 = *(const float*)((const char*)lut_b + o3);
#pragma unroll
                        for (int ps = 0; ps < NP; ps++) {
                            const uint4 xv = *(const uint4*)(smem + xq_lane[q] + c * cstep + ps * pstep + j * 2048);
                            float cc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                            mma16816(cc, ha[0], hb[0], ha[1], hb[1], xv.x, xv.y);
                            mma16816(cc, ha[2], hb[2], ha[3], hb[3], xv.z, xv.w);
                            const float xi = xip[(ps * 4 + mrow) * bpr + 16 * j + (q >> 1)];
                            pk0[ps][q] = fmaf(fmaf(cc[1], s1, cc[0] * s0), xi, pk0[ps][q]);
                            pk1[ps][q] = fmaf(fmaf(cc[3], s3, cc[2] * s2), xi, pk1[ps][q]);
                        }
                    }
                };
                if (ng == TX / 2) {
#pragma unroll
                    for (int j = 0; j < GPW; j++) group(j);
                } else {
#pragma unroll
                    for (int j = 0; j < GPW; j++)
                        if (warp + NW * j < ng) group(j);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            if (++s == S) {
                s = 0;
                par ^= 1u;
            }
        }
        if (!ok) break;
        // the four lanes of a quad hold two columns each; then the eight warps' K ranges meet in shared memory:
        // every warp posts its sums and arrives on the slot's barrier, warp 0 alone waits for all eight
        float* rb = red + rslot * (NW * MT * 16);
        if constexpr (MT == 1) {
            float a = acc0[0], b = acc1[0];
            a += __shfl_xor_sync(0xffffffffu, a, 1);
            b += __shfl_xor_sync(0xffffffffu, b, 1);
            a += __shfl_xor_sync(0xffffffffu, a, 2);
            b += __shfl_xor_sync(0xffffffffu, b, 2);
            if (t == 0) {
                rb[warp * 16 + g] = a;
                rb[warp * 16 + g + 8] = b;
            }
        } else {
#pragma unroll
            for (int ps = 0; ps < NP; ps++) {
                const int m = ps * 4 + t;
                if (m < MT) {
                    rb[(warp * MT + m) * 16 + g] = (pk0[ps][0] + pk0[ps][1]) + (pk0[ps][2] + pk0[ps][3]);
                    rb[(warp * MT + m) * 16 + g + 8] = (pk1[ps][0] + pk1[ps][1]) + (pk1[ps][2] + pk1[ps][3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&tbar[rslot]);
        if (warp == 0) {
            if (!mbar_wait(&tbar[rslot], rpar)) {
                cn_dev_fail(CN_DEV_WAIT_FULL);
                ok = false;
            } else if (MT == 1 && KS > 1) {
                // lane l < 16: row slot l of the tile over this CTA's part of K, the eight warps in order
                float v = 0.0f;
                if (lane < 16) {
                    v = rb[lane];
                    for (int w = 1; w < NW; w++) v += rb[w * 16 + lane];
                }
                float* xch = (float*)(smem + XCH_OFF) + titer * (KS - 1) * 16;
                uint64_t* xb = (uint64_t*)(smem + XBAR_OFF) + titer;
                if (crank != 0) {
                    // hand the sums to the cluster's first CTA: into this CTA's place of the slot, then one arrival on its barrier
                    if (lane < 16) st_peer_f32(peer_addr(xch + (crank - 1) * 16 + lane, 0), v);
                    __syncwarp();
                    if (lane == 0) arrive_peer(peer_addr(xb, 0));
                } else {
                    if (!mbar_wait_cluster(xb, 0)) {
                        cn_dev_fail(CN_DEV_WAIT_FULL);
                        ok = false;
                    } else {
                        if (lane < 16)
                            for (int c = 0; c < KS - 1; c++) v += xch[c * 16 + lane];  // the parts of K in order: a fixed sum
                        const float up = __shfl_down_sync(0xffffffffu, v, 8);
                        const int row = tile * per_cta + lane;
                        const float r = gu ? act_gu(v, up, p.limit) : v;
                        if (lane < per_cta && row < p.rows) {
                            if (p.out_f32)
                                ((float*)ybase)[row] = r;
                            else
                                ((__nv_bfloat16*)ybase)[row] = __float2bfloat16_rn(r);
                        }
                        if (LN) push_lines(p, tile * per_cta, min(per_cta, p.rows - tile * per_cta), r, lane, line_seq, line_buf);
                    }
                }
            } else if (LN) {
                // one activation row with line output: every lane of the warp takes part in the shuffles
                const int row = tile * per_cta + lane;
                float v0 = 0.0f, v1 = 0.0f;
                if (lane < per_cta) {
                    v0 = rb[lane], v1 = gu ? rb[lane + 8] : 0.0f;
                    for (int w = 1; w < NW; w++) {  // warps in order: deterministic
                        v0 += rb[w * 16 + lane];
                        if (gu) v1 += rb[w * 16 + lane + 8];
                    }
                }
                const float v = gu ? act_gu(v0, v1, p.limit) : v0;
                if (lane < per_cta && row < p.rows) ((__nv_bfloat16*)ybase)[row] = __float2bfloat16_rn(v);
                push_lines(p, tile * per_cta, min(per_cta, p.rows - tile * per_cta), v, lane, line_seq, line_buf);
            } else if (lane < per_cta) {
                const int row = tile * per_cta + lane;
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    float v0 = rb[m * 16 + lane], v1 = gu ? rb[m * 16 + lane + 8] : 0.0f;
                    for (int w = 1; w < NW; w++) {  // warps in order: deterministic
                        v0 += rb[(w * MT + m) * 16 + lane];
                        if (gu) v1 += rb[(w * MT + m) * 16 + lane + 8];
                    }
                    if (row < p.rows && m < p.m) {
                        const float v = gu ? act_gu(v0, v1, p.limit) : v0;
                        if (p.out_f32)
                            ((float*)ybase)[(size_t)m * p.ldy + row] = v;
                        else
                            ((__nv_bfloat16*)ybase)[(size_t)m * p.ldy + row] = __float2bfloat16_rn(v);
                    }
                }
            }
        }
        if (++rslot == RD) {
            rslot = 0;
            rpar ^= 1u;
        }
    }
    if (threadIdx.x == 0) { CN_STAMP(4); }
    if (KS > 1) cluster_sync_all();  // nobody leaves while a CTA of the cluster may still send or receive
}

template <int TX, int CPS, int MT, int KS = 1, bool LN = false>
int launch_m1(const cudaLaunchConfig_t& cfg, const GemvParams& p) {
    CN_ALLOW_SMEM((nvfp4_gemv_m1_kernel<TX, CPS, MT, KS, LN>), 226 * 1024);
    CN_CUDA(cudaLaunchKernelEx(&cfg, nvfp4_gemv_m1_kernel<TX, CPS, MT, KS, LN>, p));
    return CN_OK;
}

}  // namespace

#ifdef CN_M1_TRACE
// diagnostic build: launch i after the call (i = 0, 1, ...) stamps into buf + i * 512 * 8 words; `launches` of them
static unsigned long long* g_m1_trace = nullptr;
static int g_m1_trace_n = 0, g_m1_trace_i = 0;
extern "C" void cn_m1_trace(unsigned long long* buf, int launches) { g_m1_trace = buf, g_m1_trace_n = launches, g_m1_trace_i = 0; }
#endif

int cn_gemv_m1_launch(const GemvCall& a, cudaStream_t stream, const char* who) {
    const int rows = a.rows, k = a.k, m = a.m;
    const bool routed = a.ids != nullptr;
    const bool gu = a.w1 != nullptr || a.tab1 != nullptr || a.fused_up_rows > 0;
    const int bpr = k / 64;
    const int mt = m == 1 ? 1 : (m == 2 ? 2 : (m <= 4 ? 4 : 8));
    // blocks per row and stage: the same rule for every row count, so that row i of an m-row call is summed in the
    // order of a one-row call
    const int tx = bpr >= 32 ? 32 : 16;
    const int pstride = tx * 36 + 16;
    const size_t stage_bytes = (size_t)ROWS * pstride;
    const size_t xbytes = (size_t)mt * bpr * XB + (size_t)((mt * bpr + 3) & ~3) * 4;
    const int per_cta = gu ? ROWS / 2 : ROWS;
    const int ntiles = (rows + per_cta - 1) / per_cta;
    int nch = (bpr + tx - 1) / tx;
    // fixed part of a CTA's shared memory for a ring of `st` stages: header, tile-sum slots (a warp runs at most
    // `st` chunks ahead of warp 0, i.e. st / nch + 1 tiles), activations
    auto fixed = [&](int st) { return (long long)RED_OFF + (long long)((st + nch) / nch + 1) * NW * mt * 64 + (long long)xbytes; };
    // CTAs per SM: as many (up to 4 for one row, 2 for more) as leave every CTA a ring of at least three stages
    int cps = 1;
    for (int c = mt == 1 ? 4 : 2; c > 1; c--)
        if ((227 * 1024) / c - 1024 - fixed(3) >= 3 * (long long)stage_bytes) {
            cps = c;
            break;
        }
    if (mt == 1 && cps < 2) cps = 2;
    // persistent CTAs, each walking its share of the tiles (the routed form keeps one tile per CTA)
    int grid = ntiles;
    if (!routed && grid > 148 * cps) grid = 148 * cps;
    if (routed && (long long)ntiles * a.combos > 3LL * 148 * cps / 2) {
        // many combos: a few persistent CTAs per combo (the activation row is staged once per CTA), about one wave in all
        grid = 148 * cps / a.combos;
        if (grid <= 2) {
            // combos near or beyond the CTA slots: 1..6 CTAs per combo, whichever fills the last wave best (fewer on a near tie)
            const double slots = 148.0 * cps;
            double best = 0.0;
            for (int gx = 1; gx <= 6 && gx <= ntiles; gx++) {
                const double waves = gx * (double)a.combos / slots, eff = waves / (double)(long long)(waves + 0.999999);
                if (eff > best + 0.03) best = eff, grid = gx;
            }
            if (grid < 1) grid = 1;
        }
        grid = (ntiles + ((ntiles + grid - 1) / grid) - 1) / ((ntiles + grid - 1) / grid);  // the same tiles per CTA, fewer CTAs
    }
    // Clusters of two or four CTAs can share every tile, each CTA over its part of K, the others handing their 16 sums to
    // the first through distributed shared memory: the wave quantum drops from a tile to a half or a quarter, and a
    // matrix of few, long rows (a tensor-parallel rank's share of a down projection) gets CTAs enough to stream it.
    // Taken when it shortens the longest CTA by a tenth or more and either the machine is not filled otherwise or a CTA's
    // share stays long enough to hide the hand-over (measured on full machines: 235 KB yes, 69 KB no).
    int ksplit = 1;
    size_t xbytes_l = xbytes;
    if (!routed && mt == 1 && tx == 32) {
        double best = (double)((ntiles + 148 * cps - 1) / (148 * cps));  // tiles per CTA without a split
        int best_cps = cps;
        for (int ks = 2; ks <= 4; ks *= 2) {
            if (bpr % (4 * ks) != 0) continue;  // every part starts on a 16-byte boundary of the row
            const int bk = bpr / ks, nchk = (bk + tx - 1) / tx;
            const long long xk = (long long)bk * XB + (long long)((bk + 3) & ~3) * 4;
            int ck = 2;
            if ((227 * 1024) / 3 - 1024 - ((long long)RED_OFF + (long long)((3 + nchk) / nchk + 1) * NW * 64 + xk) >= 3 * (long long)stage_bytes) ck = 3;
            const int clusters = 148 * ck / ks;
            const int waves = (ntiles + clusters - 1) / clusters;
            const long long share = (long long)waves * ROWS * bk * 36;
            const bool underfilled = (long long)ntiles * ks <= 148LL * ck;
            if (waves > XCH_SLOTS || share < 32 * 1024 || !(underfilled || share >= 160 * 1024)) continue;
            const double t = (double)waves / ks;
            if (t <= 0.9 * best) best = t, ksplit = ks, best_cps = ck, xbytes_l = (size_t)xk;
        }
        if (ksplit > 1) {
            cps = best_cps;
            const int clusters = 148 * cps / ksplit;
            grid = ksplit * (ntiles < clusters ? ntiles : clusters);
            nch = (bpr / ksplit + tx - 1) / tx;
        }
    }
    auto fixed2 = [&](int st) { return (long long)RED_OFF + (long long)((st + nch) / nch + 1) * NW * mt * 64 + (long long)xbytes_l; };
    int fit = MAX_STAGES;  // ring depth that fits beside the fixed part
    while (fit > 1 && fixed2(fit) + (long long)fit * (long long)stage_bytes > (227 * 1024) / cps - 1024) fit--;
    int stages = fit;
    const int total_chunks = nch * ((ntiles + grid / ksplit - 1) / (grid / ksplit));
    if (stages > total_chunks) stages = total_chunks;
    if (stages < 1) stages = 1;
    int red_depth = (stages + nch) / nch + 1;
    if (red_depth > RED_DEPTH) red_depth = RED_DEPTH;
    const size_t smem = (size_t)RED_OFF + (size_t)red_depth * NW * mt * 64 + xbytes_l + stages * stage_bytes;
    if (smem > 226 * 1024 || fit < 2) {
        // the staged activations of all m rows do not fit beside a ring: two calls over half the rows each
        if (m == 1) CN_FAIL(CN_ERR_LIMIT, "%s: k = %d needs %zu B of shared memory per block", who, k, smem);
        GemvCall lo = a, hi = a;
        const int m0 = m / 2;
        lo.m = m0, hi.m = m - m0;
        hi.x = (const char*)a.x + (size_t)m0 * k * 2;
        hi.y = (char*)a.y + (size_t)m0 * a.ldy * (a.out_f32 ? 4 : 2);
        int rc = cn_gemv_m1_launch(lo, stream, who);
        return rc ? rc : cn_gemv_m1_launch(hi, stream, who);
    }
    GemvParams p;
    p.w0 = (const uint8_t*)a.w0, p.w1 = (const uint8_t*)a.w1, p.gs0 = a.gs0, p.gs1 = a.gs1 ? a.gs1 : a.gs0, p.x = a.x, p.y = a.y;
    p.rows = rows, p.k = k, p.m = m, p.ldy = a.ldy, p.limit = a.limit, p.tx = tx, p.stages = stages, p.out_f32 = a.out_f32;
    p.ids = a.ids, p.order = a.order, p.tab0 = a.tab0, p.tab1 = a.tab1, p.fused_up_rows = a.fused_up_rows, p.x_div = a.x_div;
    p.red_depth = red_depth;
    p.ksplit = ksplit;
    p.experts = a.experts, p.yptrs = a.yptrs;
    p.yl_world = 0, p.yl_row0 = 0, p.yl_stride = 0, p.yl_epoch = nullptr, p.yl_tag = 0, p.yl_buf = 0, p.yl_flip = 0;
    for (int d = 0; d < 8; d++) p.yl[d] = 0ull;
    if (a.line_bases) {
        if (routed || m != 1 || a.out_f32 || a.line_world < 2 || a.line_world > 8 || (rows & 3) || (a.line_row0 & 3) || !a.line_epoch ||
            a.line_tag < 1 || a.line_tag > 4095 || (a.line_buf & ~1))
            CN_FAIL(CN_ERR_SHAPE, "%s: line output needs one bf16 row, 2..8 ranks and row counts in multiples of 4 (rows %d, first row %d, ranks %d)", who,
                    rows, a.line_row0, a.line_world);
        p.yl_world = a.line_world, p.yl_row0 = a.line_row0, p.yl_stride = (unsigned long long)a.line_stride, p.yl_epoch = a.line_epoch;
        p.yl_tag = a.line_tag, p.yl_buf = a.line_buf, p.yl_flip = a.line_flip ? 1 : 0;
        for (int d = 0; d < a.line_world; d++) p.yl[d] = a.line_bases[d];
    }
#ifdef CN_M1_TRACE
    p.trace = (g_m1_trace && g_m1_trace_i < g_m1_trace_n && !routed) ? g_m1_trace + (size_t)(g_m1_trace_i++) * 512 * 8 : nullptr;
#endif
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, (unsigned)(routed ? a.combos : 1));
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (ksplit > 1) {
        at[1].id = cudaLaunchAttributeClusterDimension;
        at[1].val.clusterDim.x = (unsigned)ksplit, at[1].val.clusterDim.y = 1, at[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
        if (p.yl_world > 0) {
            if (ksplit == 2) return cps == 2 ? launch_m1<32, 2, 1, 2, true>(cfg, p) : launch_m1<32, 3, 1, 2, true>(cfg, p);
            return cps == 2 ? launch_m1<32, 2, 1, 4, true>(cfg, p) : launch_m1<32, 3, 1, 4, true>(cfg, p);
        }
        if (ksplit == 2) return cps == 2 ? launch_m1<32, 2, 1, 2>(cfg, p) : launch_m1<32, 3, 1, 2>(cfg, p);
        return cps == 2 ? launch_m1<32, 2, 1, 4>(cfg, p) : launch_m1<32, 3, 1, 4>(cfg, p);
    }
    if (p.yl_world > 0) {
        // line output: the shapes of a tensor-parallel rank (32 blocks per stage)
        if (tx == 32 && cps == 2) return launch_m1<32, 2, 1, 1, true>(cfg, p);
        if (tx == 32 && cps == 3) return launch_m1<32, 3, 1, 1, true>(cfg, p);
        if (tx == 32 && cps == 4) return launch_m1<32, 4, 1, 1, true>(cfg, p);
        CN_FAIL(CN_ERR_SHAPE, "%s: line output needs k >= 2048 (k = %d)", who, k);
    }
#define CN_M1_CASE(TXV, CPSV, MTV) \
    if (tx == TXV && cps == CPSV && mt == MTV) return launch_m1<TXV, CPSV, MTV>(cfg, p);
    CN_M1_CASE(32, 2, 1) CN_M1_CASE(32, 3, 1) CN_M1_CASE(32, 4, 1) CN_M1_CASE(16, 2, 1) CN_M1_CASE(16, 3, 1) CN_M1_CASE(16, 4, 1)
    CN_M1_CASE(32, 1, 2) CN_M1_CASE(32, 2, 2) CN_M1_CASE(16, 1, 2) CN_M1_CASE(16, 2, 2)
    CN_M1_CASE(32, 1, 4) CN_M1_CASE(32, 2, 4) CN_M1_CASE(16, 1, 4) CN_M1_CASE(16, 2, 4)
    CN_M1_CASE(32, 1, 8) CN_M1_CASE(32, 2, 8) CN_M1_CASE(16, 1, 8) CN_M1_CASE(16, 2, 8)
#undef CN_M1_CASE
    CN_FAIL(CN_ERR_SHAPE, "%s: no kernel for %d blocks per stage, %d CTAs per SM, %d rows", who, tx, cps, mt);
}
