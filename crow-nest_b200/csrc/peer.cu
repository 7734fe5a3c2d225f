// Tensor-parallel exchange over NVLink peer memory: every rank pushes its slice of an activation vector
// straight into the same place of every peer's buffer and the ranks meet on per-source arrival counters.
// One small kernel per exchange in place of an NCCL all-gather, whose latency (about 12 us per call
// for these 10 - 34 KB messages) bounds a decode step that has 256 of them.
//
// The reference has no multi-GPU path; this belongs to the row-split projections of the dense stack.
//
// Buffer, identical on every rank (allocated by the caller, exported / opened with the calls below):
//   data ...                           activation vectors, rank r's slice at data_off + r * slice_bytes
//   flags at flag_off: u32 arrive[8]   arrive[s] = sequence number of the last exchange whose slice from
//                                      rank s has landed here
//                      u32 seq         this rank's own count of exchanges at this exchange point
// The sequence numbers live on the device, so a captured graph can be replayed: nothing about the
// exchange is baked into the launch. Every exchange is also a barrier between the ranks (nobody passes
// before all slices have landed), which is what allows one buffer per exchange point without double
// buffering: a rank can write a vector's next version only after every reader of the previous one has
// arrived at a later exchange.
// Peer stores are plain st.global to the peer's address (no multicast, no bulk copy); the wait is bounded
// (about a second) and reports through the device status word.
//
// Two further forms carry the sequence number inside the data instead of behind it: 16-byte lines {word, number,
// word, number} through two line buffers per vector, pushed by a kernel of this file (tp_allgather_ll_kernel) or by
// the epilogue of the GEMV that produces the slice (nvfp4_gemv_m1.cu), in which case only the receiving half runs
// here (tp_recv_lines_kernel). A line is valid when both halves carry the expected number, so nothing waits for
// a store to be acknowledged and an exchange costs one trip over NVLink.
#include <string.h>

#include "common.cuh"

namespace {

constexpr int MAX_WORLD = 8;

struct PeerPtrs {
    unsigned char* base[MAX_WORLD];
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// The block's 512 threads are dealt to the peers in equal groups of whole warps (world 2: 512 threads for the one peer,
// world 8: two warps for each of the seven): a group stores this rank's slice into its peer's buffer, makes it visible
// system-wide, meets on its own named barrier, and its first thread publishes the sequence number right behind the data and
// waits for that peer's slice of the same exchange. The peers are served side by side.
// Diagnostic build (-DCN_M1_TRACE): thread 0 (which serves the first peer) stamps %globaltimer at entry (0), after the wait on
// the predecessor grid (1), after its stores and the system-scope fence (2), after its flag store (3), when its peer's flag
// has arrived (4) and when every group has seen its peer's (5).
#ifdef CN_M1_TRACE
#define CN_TP_STAMP(i) if (threadIdx.x == 0 && trace) trace[i] = tp_gtime()
__device__ __forceinline__ unsigned long long tp_gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#else
#define CN_TP_STAMP(i)
#endif

__global__ void __launch_bounds__(512) tp_allgather_kernel(PeerPtrs peers, int rank, int world, size_t data_off, size_t slice_bytes,
                                                           size_t flag_off, unsigned long long* trace) {
    CN_TP_STAMP(0);
    pdl_wait();  // the slice comes from the kernel before this one
    CN_TP_STAMP(1);
    unsigned char* mine = peers.base[rank];
    unsigned int* my_flags = (unsigned int*)(mine + flag_off);
    const unsigned int seq = my_flags[MAX_WORLD] + 1u;  // read by everybody before anybody can advance it (barrier below)
    const int gsz = (512 / (world - 1)) & ~31;          // threads per peer
    const int gi = threadIdx.x / gsz, gt = threadIdx.x - gi * gsz;
    if (gi < world - 1) {
        const int p = gi < rank ? gi : gi + 1;  // the peers in rank order, this rank left out
        const uint4* src = (const uint4*)(mine + data_off + (size_t)rank * slice_bytes);
        uint4* dst = (uint4*)(peers.base[p] + data_off + (size_t)rank * slice_bytes);
        const size_t n16 = slice_bytes >> 4;
        for (size_t i = gt; i < n16; i += gsz) dst[i] = src[i];
        // Every thread makes its own stores visible system-wide before the barrier. Leaving that to the first thread's release
        // alone (barrier, then one st.release.sys) was measured 15 % faster per step, but rests on that release covering the
        // other threads' stores to another GPU's memory, which was not confirmed beyond a few passing runs.
        __threadfence_system();
        CN_TP_STAMP(2);
        asm volatile("bar.sync %0, %1;" ::"r"(gi + 1), "r"(gsz) : "memory");
        if (gt == 0) {
            st_release_sys((unsigned int*)(peers.base[p] + flag_off) + rank, seq);
            CN_TP_STAMP(3);
            const long long t0 = clock64();
            while ((int)(ld_acquire_sys(my_flags + p) - seq) < 0) {
                if (clock64() - t0 > 2000000000LL) {
                    cn_dev_fail(CN_DEV_WAIT_FULL);
                    break;
                }
            }
            CN_TP_STAMP(4);
        }
    }
    __syncthreads();
    CN_TP_STAMP(5);
    if (threadIdx.x == 0) my_flags[MAX_WORLD] = seq;
    pdl_launch_dependents();
}

// The same exchange without a flag behind the data: every two 32-bit words of the slice travel as a 16-byte line {word,
// sequence number, word, sequence number} into the peer's line buffer (each 8-byte half carries its own number, so the
// line may arrive in two pieces); the receiver reads its own line buffer until both halves of a line carry the current
// sequence number and writes the words into its copy of the vector. No release has to wait for the peer to
// acknowledge the data, so an exchange costs one trip over NVLink instead of two. Two line buffers are used in turn
// (sequence number odd / even): a peer can be one exchange ahead of this rank, never two, because its exchange after next
// needs this rank's lines of the next one.
__device__ __forceinline__ void st_line(uint4* p, unsigned int w0, unsigned int w1, unsigned int seq) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(w0), "r"(seq), "r"(w1), "r"(seq) : "memory");
}
__device__ __forceinline__ uint4 ld_line(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(512) tp_allgather_ll_kernel(PeerPtrs peers, int rank, int world, size_t data_off, size_t slice_bytes,
                                                              size_t ll_off, size_t flag_off, unsigned long long* trace) {
    CN_TP_STAMP(0);
    pdl_wait();  // the slice comes from the kernel before this one
    CN_TP_STAMP(1);
    unsigned char* mine = peers.base[rank];
    unsigned int* my_flags = (unsigned int*)(mine + flag_off);
    const unsigned int seq = my_flags[MAX_WORLD] + 1u;  // read by everybody before anybody can advance it (barrier below)
    const size_t nl = slice_bytes >> 3;                 // lines of a slice: two 32-bit words each
    const size_t line_slice = slice_bytes * 2;          // the same slice as lines
    const size_t par_off = ll_off + (size_t)(seq & 1u) * (size_t)world * line_slice;
    const int gsz = (512 / (world - 1)) & ~31;  // threads per peer
    const int gi = threadIdx.x / gsz, gt = threadIdx.x - gi * gsz;
    if (gi < world - 1) {
        const int p = gi < rank ? gi : gi + 1;  // the peers in rank order, this rank left out
        const uint2* src = (const uint2*)(mine + data_off + (size_t)rank * slice_bytes);
        uint4* dst = (uint4*)(peers.base[p] + par_off + (size_t)rank * line_slice);
        for (size_t i = gt; i < nl; i += gsz) {
            const uint2 w = src[i];
            st_line(dst + i, w.x, w.y, seq);
        }
        CN_TP_STAMP(2);
        const uint4* in = (const uint4*)(mine + par_off + (size_t)p * line_slice);
        uint2* out = (uint2*)(mine + data_off + (size_t)p * slice_bytes);
        const long long t0 = clock64();
        bool ok = true;
        for (size_t i = gt; i < nl && ok; i += gsz) {
            uint4 v = ld_line(in + i);
            while (v.y != seq || v.w != seq) {
                if (clock64() - t0 > 2000000000LL) {
                    cn_dev_fail(CN_DEV_WAIT_FULL);
                    ok = false;
                    break;
                }
                v = ld_line(in + i);
            }
            out[i] = make_uint2(v.x, v.z);
        }
        CN_TP_STAMP(4);
    }
    __syncthreads();
    CN_TP_STAMP(5);
    if (threadIdx.x == 0) my_flags[MAX_WORLD] = seq;
    pdl_launch_dependents();
}

// The receiving half of an exchange whose lines were stored by the producing GEMV itself (cn_nvfp4_gemv_lines): polls this
// rank's line buffer for the peers' slices and writes them into its copy of the vector. The exchange number comes from the
// rank's step counter (advanced once at the start of a step by cn_tp_epoch_advance, long before this kernel can start) and a
// tag fixed at launch, not from anything an earlier exchange writes: with every kernel letting its successor start early,
// kernels many exchanges ahead can be resident at once.
// Resident long before the producing kernels end (it lets its successor start at once and waits for its predecessor only
// before it leaves), so the vector is complete one NVLink trip after the slowest rank's last tile.
__global__ void __launch_bounds__(512) tp_recv_lines_kernel(unsigned char* mine, int rank, int world, size_t data_off, size_t slice_bytes,
                                                            size_t line_off, const unsigned int* epoch_ptr, int tag, int buf, int flip,
                                                            unsigned long long* trace) {
    CN_TP_STAMP(0);
    pdl_launch_dependents();
    const unsigned int epoch = *(volatile const unsigned int*)epoch_ptr;
    const unsigned int seq = epoch * 4096u + (unsigned int)tag;
    const size_t nl = slice_bytes >> 3, line_slice = slice_bytes * 2;
    const size_t par_off = line_off + (size_t)((unsigned int)buf ^ ((unsigned int)flip & epoch & 1u)) * (size_t)world * line_slice;
    const int gsz = (512 / (world - 1)) & ~31;  // threads per peer
    const int gi = threadIdx.x / gsz, gt = threadIdx.x - gi * gsz;
    if (gi < world - 1) {
        const int p = gi < rank ? gi : gi + 1;  // the peers in rank order, this rank left out
        const uint4* in = (const uint4*)(mine + par_off + (size_t)p * line_slice);
        uint2* out = (uint2*)(mine + data_off + (size_t)p * slice_bytes);
        const long long t0 = clock64();
        bool ok = true;
        for (size_t i = gt; i < nl && ok; i += gsz) {
            uint4 v = ld_line(in + i);
            while (v.y != seq || v.w != seq) {
                if (clock64() - t0 > 2000000000LL || *(volatile int*)&g_cn_status != 0) {
                    cn_dev_fail(CN_DEV_WAIT_FULL);
                    ok = false;
                    break;
                }
                v = ld_line(in + i);
            }
            out[i] = make_uint2(v.x, v.z);
        }
        CN_TP_STAMP(4);
    }
    __syncthreads();
    pdl_wait();  // this rank's own slice comes from the kernel before this one: the grid ends only after it has
    CN_TP_STAMP(5);
}

__global__ void tp_epoch_kernel(unsigned int* epoch) { *epoch = *epoch + 1u; }

}  // namespace

extern "C" int cn_peer_export(const void* ptr, void* handle64, size_t* offset) {
    if (!ptr || !handle64 || !offset) CN_FAIL(CN_ERR_SHAPE, "cn_peer_export: null argument");
    cudaIpcMemHandle_t h;
    CN_CUDA(cudaIpcGetMemHandle(&h, (void*)ptr));
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    // the handle names the whole allocation: find where `ptr` sits in it
    void* base = nullptr;
    size_t size = 0;
    {
        typedef int (*range_fn)(unsigned long long*, size_t*, unsigned long long);
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        CN_CUDA(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q));
        if (!fn) CN_FAIL(CN_ERR_CUDA, "cn_peer_export: cuMemGetAddressRange is not available");
        unsigned long long b = 0;
        if (((range_fn)fn)(&b, &size, (unsigned long long)(uintptr_t)ptr) != 0) CN_FAIL(CN_ERR_CUDA, "cn_peer_export: cuMemGetAddressRange failed");
        base = (void*)(uintptr_t)b;
    }
    *offset = (size_t)((const char*)ptr - (const char*)base);
    return CN_OK;
}

extern "C" int cn_peer_open(const void* handle64, size_t offset, void** ptr) {
    if (!handle64 || !ptr) CN_FAIL(CN_ERR_SHAPE, "cn_peer_open: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* base = nullptr;
    CN_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr = (char*)base + offset;
    return CN_OK;
}

extern "C" int cn_peer_close(void* ptr, size_t offset) {
    if (!ptr) return CN_OK;
    CN_CUDA(cudaIpcCloseMemHandle((char*)ptr - offset));
    return CN_OK;
}

#ifdef CN_M1_TRACE
// diagnostic build: exchange i after the call (i = 0, 1, ...) stamps into buf + 8 i words; `launches` of them
static unsigned long long* g_tp_trace = nullptr;
static int g_tp_trace_n = 0, g_tp_trace_i = 0;
extern "C" void cn_tp_trace(unsigned long long* buf, int launches) { g_tp_trace = buf, g_tp_trace_n = launches, g_tp_trace_i = 0; }
#endif

extern "C" int cn_tp_allgather(const void* const* peer_bases, int rank, int world, size_t data_off, size_t slice_bytes, size_t flag_off,
                               cn_stream_t stream) {
    if (world < 2 || world > MAX_WORLD || rank < 0 || rank >= world) CN_FAIL(CN_ERR_SHAPE, "cn_tp_allgather: rank %d of %d", rank, world);
    if (slice_bytes == 0 || (slice_bytes & 15) || (data_off & 15) || (flag_off & 15))
        CN_FAIL(CN_ERR_SHAPE, "cn_tp_allgather: offsets and the slice size must be multiples of 16 bytes");
    PeerPtrs pp = {};
    for (int p = 0; p < world; p++) {
        if (!peer_bases[p]) CN_FAIL(CN_ERR_SHAPE, "cn_tp_allgather: no buffer for rank %d", p);
        pp.base[p] = (unsigned char*)peer_bases[p];
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1), cfg.blockDim = dim3(512), cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at, cfg.numAttrs = 1;
    unsigned long long* trace = nullptr;
#ifdef CN_M1_TRACE
    if (g_tp_trace && g_tp_trace_i < g_tp_trace_n) trace = g_tp_trace + (size_t)(g_tp_trace_i++) * 8;
#endif
    CN_CUDA(cudaLaunchKernelEx(&cfg, tp_allgather_kernel, pp, rank, world, data_off, slice_bytes, flag_off, trace));
    return CN_OK;
}

extern "C" int cn_tp_allgather_ll(const void* const* peer_bases, int rank, int world, size_t data_off, size_t slice_bytes, size_t line_off,
                                  size_t flag_off, cn_stream_t stream) {
    if (world < 2 || world > MAX_WORLD || rank < 0 || rank >= world) CN_FAIL(CN_ERR_SHAPE, "cn_tp_allgather_ll: rank %d of %d", rank, world);
    if (!peer_bases || (data_off & 15) || (slice_bytes & 15) || (line_off & 15) || (flag_off & 15) || slice_bytes == 0)
        CN_FAIL(CN_ERR_SHAPE, "cn_tp_allgather_ll: offsets and the slice size must be multiples of 16 bytes");
    PeerPtrs pp;
    for (int r = 0; r < MAX_WORLD; r++) pp.base[r] = r < world ? (unsigned char*)peer_bases[r] : nullptr;
    for (int r = 0; r < world; r++)
        if (!pp.base[r]) CN_FAIL(CN_ERR_SHAPE, "cn_tp_allgather_ll: null base pointer for rank %d", r);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1), cfg.blockDim = dim3(512), cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at, cfg.numAttrs = 1;
    unsigned long long* trace = nullptr;
#ifdef CN_M1_TRACE
    if (g_tp_trace && g_tp_trace_i < g_tp_trace_n) trace = g_tp_trace + (size_t)(g_tp_trace_i++) * 8;
#endif
    CN_CUDA(cudaLaunchKernelEx(&cfg, tp_allgather_ll_kernel, pp, rank, world, data_off, slice_bytes, line_off, flag_off, trace));
    return CN_OK;
}

extern "C" int cn_tp_epoch_advance(void* epoch, cn_stream_t stream) {
    if (!epoch || ((uintptr_t)epoch & 3)) CN_FAIL(CN_ERR_SHAPE, "cn_tp_epoch_advance: null or unaligned counter");
    // a plain launch: it neither starts before its predecessor has ended nor lets its successor start before it has
    tp_epoch_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((unsigned int*)epoch);
    CN_CUDA(cudaGetLastError());
    return CN_OK;
}

extern "C" int cn_tp_recv_lines(void* base, int rank, int world, size_t data_off, size_t slice_bytes, size_t line_off, const void* epoch,
                                int tag, int buf, int flip, cn_stream_t stream) {
    if (world < 2 || world > MAX_WORLD || rank < 0 || rank >= world) CN_FAIL(CN_ERR_SHAPE, "cn_tp_recv_lines: rank %d of %d", rank, world);
    if (!base || !epoch || (data_off & 15) || (slice_bytes & 15) || (line_off & 15) || slice_bytes == 0 || tag < 1 || tag > 4095 || (buf & ~1))
        CN_FAIL(CN_ERR_SHAPE, "cn_tp_recv_lines: offsets and the slice size must be multiples of 16 bytes, the tag in 1..4095, the buffer 0 or 1");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1), cfg.blockDim = dim3(512), cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at, cfg.numAttrs = 1;
    unsigned long long* trace = nullptr;
#ifdef CN_M1_TRACE
    if (g_tp_trace && g_tp_trace_i < g_tp_trace_n) trace = g_tp_trace + (size_t)(g_tp_trace_i++) * 8;
#endif
    CN_CUDA(cudaLaunchKernelEx(&cfg, tp_recv_lines_kernel, (unsigned char*)base, rank, world, data_off, slice_bytes, line_off,
                               (const unsigned int*)epoch, tag, buf, flip ? 1 : 0, trace));
    return CN_OK;
}
