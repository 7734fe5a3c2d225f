// Expert-parallel token exchange over NVLink peer memory: all-to-all DISPATCH of the routed activation rows to the
// ranks that hold their experts, and all-to-all RETURN of the expert outputs to the rank that holds the token.
//
// The reference is single-GPU; what this replaces there is the gather in front of the expert kernels and the combine
// behind them (glm5_moe_gather / glm5_moe_combine, engine/src/kernels_glm5_moe.cu:101-156; router_top10's pointer
// gather, engine/src/kernels.rs:3172-3173): with the experts spread over ranks (expert e on rank e / (experts / world))
// the gather becomes "send row c to the owner of ids[c]" and the combine runs where the token lives.
//
// Every rank holds one buffer of the same layout, mapped by all peers (cn_peer_export / cn_peer_open):
//   inbox_x    [world][cap][hidden] bf16   activation rows received from each source rank
//   inbox_meta [world][cap] {i32 expert, i32 source combo}
//   ret        [cap][hidden] f32           expert outputs of this rank's own combos, written by the owners
//   flags      u64 dispatch[world] (sequence << 32 | rows sent), u64 returned[world], u32 seq, u32 ticket
// cap = the most combos one rank can send (tokens per rank x top-k): whatever the routing, nothing overflows.
// A step: route the local tokens; cn_ep_dispatch pushes row (c / topk) and {expert, c} of every local combo c into its
// owner's inbox (plain peer stores, rows of one destination in expert order) and meets the other ranks on the dispatch
// flags; the owner runs its experts over the inbox rows, the down projection storing each result straight into the
// source rank's `ret` at row c (cn_ep_targets builds those addresses); cn_ep_return meets the ranks again; the source
// combines ret with its own routing weights in pick order - the same sum, in the same order, as on one GPU.
// Sequence numbers live on the device (a captured graph replays); waits are bounded and report through the device
// status word. Only plain loads and stores cross NVLink: no multicast, no bulk copies.
#include "common.cuh"

namespace {

constexpr int MAX_WORLD = 8;
#define CN_DEV_WAIT_EP 105

struct EpLayout {
    unsigned char* base[MAX_WORLD];
    size_t inbox_x, inbox_meta, ret, flags;  // byte offsets in every rank's buffer
    int rank, world, cap, hidden;
};

__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
// flags block of a buffer: [0..8) dispatch words, [8..16) return words, then {u32 seq, u32 ticket}
__device__ __forceinline__ unsigned long long* flag_words(unsigned char* base, size_t off) { return (unsigned long long*)(base + off); }

// The last CTA of a grid (by ticket) tells every peer "my part of exchange `seq` is in your memory" (with a count) and
// waits until every peer has said the same. which = 0 dispatch, 1 return.
__device__ void meet_peers(const EpLayout& L, int which, unsigned int seq, const int* counts) {
    unsigned long long* mine = flag_words(L.base[L.rank], L.flags) + which * MAX_WORLD;
    const int p = threadIdx.x;
    if (p < L.world) {
        if (p != L.rank) {
            const unsigned long long word = ((unsigned long long)seq << 32) | (unsigned int)(counts ? counts[p] : 0);
            st_release_sys_u64(flag_words(L.base[p], L.flags) + which * MAX_WORLD + L.rank, word);
            const long long t0 = clock64();
            while ((int)((unsigned int)(ld_acquire_sys_u64(mine + p) >> 32) - seq) < 0) {
                if (clock64() - t0 > 2000000000LL || *(volatile int*)&g_cn_status != 0) {
                    cn_dev_fail(CN_DEV_WAIT_EP);
                    break;
                }
            }
        } else {
            mine[p] = ((unsigned long long)seq << 32) | (unsigned int)(counts ? counts[p] : 0);
        }
    }
}

// combos of this rank sorted by expert (order[], from cn_moe_sort) fall into one contiguous run per destination rank
__global__ void __launch_bounds__(256) ep_dispatch_kernel(EpLayout L, const int32_t* __restrict__ ids, const int32_t* __restrict__ order,
                                                          const void* __restrict__ x, int combos, int topk, int experts) {
    __shared__ int start[MAX_WORLD + 1];
    __shared__ unsigned int seq_s;
    __shared__ int last_s;
    pdl_wait();
    const int epr = experts / L.world;
    unsigned int* ctl = (unsigned int*)(flag_words(L.base[L.rank], L.flags) + 2 * MAX_WORLD);
    if (threadIdx.x == 0) seq_s = ctl[0] + 1u;
    // start[r] = first position of the sorted list whose expert belongs to rank >= r (invalid ids sort last)
    if (threadIdx.x <= L.world) {
        const int r = threadIdx.x;
        int lo = 0, hi = combos;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            const int e = ids[order[mid]];
            const int dest = (e < 0 || e >= experts) ? L.world : e / epr;
            if (dest < r) lo = mid + 1; else hi = mid;
        }
        start[r] = lo;
    }
    __syncthreads();
    const unsigned int seq = seq_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpc = blockDim.x >> 5;
    const int n16 = L.hidden * 2 / 16;
    for (int i = blockIdx.x * wpc + warp; i < start[L.world]; i += gridDim.x * wpc) {
        const int c = order[i], e = ids[c];
        const int dest = e / epr, slot = i - start[dest];
        unsigned char* b = L.base[dest];
        const uint4* src = (const uint4*)((const char*)x + (size_t)(c / topk) * L.hidden * 2);
        uint4* dst = (uint4*)(b + L.inbox_x + ((size_t)L.rank * L.cap + slot) * L.hidden * 2);
        for (int j = lane; j < n16; j += 32) dst[j] = src[j];
        if (lane == 0) ((int2*)(b + L.inbox_meta))[(size_t)L.rank * L.cap + slot] = make_int2(e, c);
    }
    // every CTA's stores are out before its ticket; the last ticket holder speaks for the grid
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) last_s = atomicAdd(&ctl[1], 1u) == gridDim.x - 1;
    __syncthreads();
    if (!last_s) return;
    __threadfence_system();
    __shared__ int counts[MAX_WORLD];
    if (threadIdx.x < L.world) counts[threadIdx.x] = start[threadIdx.x + 1] - start[threadIdx.x];
    __syncthreads();
    meet_peers(L, 0, seq, counts);
    __syncthreads();
    if (threadIdx.x == 0) ctl[1] = 0u;  // the sequence number itself is advanced by the return, which closes the step
}

// After the dispatch: the id of every inbox slot (-1 = empty) for the routed kernels, and where each slot's result
// goes: row `source combo` of the source rank's `ret`.
__global__ void ep_targets_kernel(EpLayout L, int32_t* __restrict__ ids_in, unsigned long long* __restrict__ out_ptrs) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= L.world * L.cap) return;
    const int s = i / L.cap, slot = i - s * L.cap;
    const unsigned long long word = flag_words(L.base[L.rank], L.flags)[s];
    const int n = (int)(unsigned int)(word & 0xffffffffu);
    if (slot < n) {
        const int2 m = ((const int2*)(L.base[L.rank] + L.inbox_meta))[i];
        ids_in[i] = m.x;
        out_ptrs[i] = (unsigned long long)(uintptr_t)(L.base[s] + L.ret + (size_t)m.y * L.hidden * 4);
    } else {
        ids_in[i] = -1;
        out_ptrs[i] = 0ull;
    }
}

// Optional copy (results that were computed into a local buffer `eo` [world * cap][hidden] f32 go to their source
// rank's `ret`), then the return meeting.
__global__ void __launch_bounds__(256) ep_return_kernel(EpLayout L, const float* __restrict__ eo, const int32_t* __restrict__ ids_in,
                                                        const unsigned long long* __restrict__ out_ptrs) {
    __shared__ int last_s;
    pdl_wait();
    unsigned int* ctl = (unsigned int*)(flag_words(L.base[L.rank], L.flags) + 2 * MAX_WORLD);
    const unsigned int seq = ctl[0] + 1u;
    if (eo) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpc = blockDim.x >> 5;
        const int n16 = L.hidden * 4 / 16;
        for (int i = blockIdx.x * wpc + warp; i < L.world * L.cap; i += gridDim.x * wpc) {
            if (ids_in[i] < 0) continue;
            const uint4* src = (const uint4*)(eo + (size_t)i * L.hidden);
            uint4* dst = (uint4*)(uintptr_t)out_ptrs[i];
            for (int j = lane; j < n16; j += 32) dst[j] = src[j];
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) last_s = atomicAdd(&ctl[1], 1u) == gridDim.x - 1;
    __syncthreads();
    if (!last_s) return;
    __threadfence_system();
    meet_peers(L, 1, seq, nullptr);
    __syncthreads();
    if (threadIdx.x == 0) {
        ctl[1] = 0u;
        ctl[0] = seq;
    }
}

int make_layout(EpLayout* L, const void* const* peer_bases, int rank, int world, int cap, int hidden, size_t inbox_x, size_t inbox_meta,
                size_t ret, size_t flags, const char* who) {
    if (world < 2 || world > MAX_WORLD || rank < 0 || rank >= world) CN_FAIL(CN_ERR_SHAPE, "%s: rank %d of %d", who, rank, world);
    if (cap < 1 || hidden < 8 || hidden % 8) CN_FAIL(CN_ERR_SHAPE, "%s: cap %d, hidden %d (a multiple of 8)", who, cap, hidden);
    if ((inbox_x & 15) || (inbox_meta & 15) || (ret & 15) || (flags & 15)) CN_FAIL(CN_ERR_SHAPE, "%s: offsets must be multiples of 16 bytes", who);
    for (int p = 0; p < world; p++) {
        if (!peer_bases[p]) CN_FAIL(CN_ERR_SHAPE, "%s: no buffer for rank %d", who, p);
        L->base[p] = (unsigned char*)peer_bases[p];
    }
    L->rank = rank, L->world = world, L->cap = cap, L->hidden = hidden, L->inbox_x = inbox_x, L->inbox_meta = inbox_meta, L->ret = ret, L->flags = flags;
    return CN_OK;
}

}  // namespace

extern "C" size_t cn_ep_flag_bytes(void) { return (2 * MAX_WORLD) * 8 + 16; }

extern "C" int cn_ep_dispatch(const void* const* peer_bases, int rank, int world, int cap, int hidden, size_t inbox_x, size_t inbox_meta, size_t ret,
                              size_t flags, const int32_t* ids, const int32_t* order, const void* x, int combos, int topk, int experts,
                              int32_t* ids_in, unsigned long long* out_ptrs, cn_stream_t stream) {
    EpLayout L = {};
    if (int rc = make_layout(&L, peer_bases, rank, world, cap, hidden, inbox_x, inbox_meta, ret, flags, "cn_ep_dispatch")) return rc;
    if (combos < 1 || combos > cap || topk < 1 || experts < world || experts % world)
        CN_FAIL(CN_ERR_SHAPE, "cn_ep_dispatch: %d combos (cap %d), top-%d, %d experts over %d ranks", combos, cap, topk, experts, world);
    if (!ids || !order || !x || !ids_in || !out_ptrs) CN_FAIL(CN_ERR_SHAPE, "cn_ep_dispatch: null argument");
    int grid = (combos + 7) / 8;
    if (grid > 148) grid = 148;
    CN_CUDA(cn_launch_pdl(ep_dispatch_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, L, ids, order, x, combos, topk, experts));
    const int n = world * cap;
    ep_targets_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(L, ids_in, out_ptrs);
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}

extern "C" int cn_ep_return(const void* const* peer_bases, int rank, int world, int cap, int hidden, size_t inbox_x, size_t inbox_meta, size_t ret,
                            size_t flags, const float* eo, const int32_t* ids_in, const unsigned long long* out_ptrs, cn_stream_t stream) {
    EpLayout L = {};
    if (int rc = make_layout(&L, peer_bases, rank, world, cap, hidden, inbox_x, inbox_meta, ret, flags, "cn_ep_return")) return rc;
    if (eo && (!ids_in || !out_ptrs)) CN_FAIL(CN_ERR_SHAPE, "cn_ep_return: a copy needs the slot ids and targets of cn_ep_dispatch");
    const int grid = eo ? 148 : 1;
    CN_CUDA(cn_launch_pdl(ep_return_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, L, eo, ids_in, out_ptrs));
    return CN_OK;
}
