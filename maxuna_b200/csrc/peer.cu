// Exchanges of an expert-parallel decode step over peer memory (NVLink), without a communication library:
// each rank stores its rows straight into the receive buffers of the other ranks and raises a flag there; the
// receiver's next kernels are held back by a small kernel that waits (bounded) for the flags of all ranks.
// The reference has no counterpart (one GPU).  A multi-GPU host uses these between the per-rank entries
// (lmoe_route, lmoe_experts_forward_ep, lmoe_ep_combine) in place of an all-gather and an all-to-all.
//
//   lmoe_peer_alloc / lmoe_peer_open : a device buffer that other processes can map (CUDA IPC), and its mapping
//   lmoe_peer_put                    : chunk s of `src` (or the same chunk for everyone) -> slot `rank` of rank s's
//                                      buffer, then flag[rank] = epoch on rank s, released at system scope
//   lmoe_peer_wait                   : until flag[0 .. world) have all reached the epoch
// The epoch lives on the device (one word per direction, advanced by the put kernel), so a recorded sequence of
// launches (a CUDA graph) can be replayed.  Only plain stores and loads touch peer memory.
#include "common.cuh"
#include "fused.cuh"

namespace {

constexpr int PEER_MAX_WORLD = 16;
constexpr uint32_t PEER_SPIN_LIMIT = 1u << 22;

struct PeerPutParams {
    const uint8_t *src;
    uint8_t *dst[PEER_MAX_WORLD];    // receive buffers of the ranks (peer-mapped; dst[rank] is local)
    uint32_t *flags[PEER_MAX_WORLD]; // flag arrays of the ranks: flags[s][rank] is this rank's flag on rank s
    uint32_t *epoch;                 // local: epochs sent so far in this direction
    uint32_t *arrived;               // local: CTAs done per destination (returns to zero)
    int64_t chunk_bytes;             // multiple of 16
    int world, rank, per_rank_src;   // per_rank_src: chunk s of src goes to rank s; else chunk 0 goes to everyone
};

__global__ void __launch_bounds__(256) peer_put_kernel(const PeerPutParams P) {
    const int s = blockIdx.y; // destination rank
    const uint32_t e = *reinterpret_cast<volatile uint32_t *>(P.epoch) + 1u;
    const uint4 *src = reinterpret_cast<const uint4 *>(P.src + (P.per_rank_src ? (int64_t)s * P.chunk_bytes : 0));
    uint4 *dst = reinterpret_cast<uint4 *>(P.dst[s] + (int64_t)P.rank * P.chunk_bytes);
    const int64_t n = P.chunk_bytes / 16;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) dst[i] = src[i];
    __threadfence_system(); // this thread's stores are visible to the destination GPU before the flag can be
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t done = atomicAdd(&P.arrived[s], 1u) + 1u;
        if (done == gridDim.x) {
            // the last CTA of this destination: every CTA fenced its stores before it counted itself
            __threadfence_system();
            P.arrived[s] = 0u;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(P.flags[s] + P.rank), "r"(e) : "memory");
            // the epoch word advances once per launch: by the last CTA of the last destination to finish
            const uint32_t fin = atomicAdd(&P.arrived[PEER_MAX_WORLD], 1u) + 1u;
            if (fin == gridDim.y) {
                P.arrived[PEER_MAX_WORLD] = 0u;
                __threadfence();
                *reinterpret_cast<volatile uint32_t *>(P.epoch) = e;
            }
        }
    }
}

// One CTA: thread i waits for rank i's flag to reach the local epoch (wrap-safe comparison).
__global__ void peer_wait_kernel(const uint32_t *flags, const uint32_t *epoch, int world, uint32_t *status) {
    const int i = threadIdx.x;
    if (i >= world) return;
    const uint32_t e = *reinterpret_cast<const volatile uint32_t *>(epoch);
    for (uint32_t it = 0; it < PEER_SPIN_LIMIT; it++) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + i) : "memory");
        if ((int32_t)(v - e) >= 0) return;
        __nanosleep(64);
    }
    atomicOr(status, (uint32_t)LMOE_FLAG_WAIT_TIMEOUT | (0x100u << i));
}

} // namespace

extern "C" lmoe_status lmoe_peer_alloc(size_t bytes, void **ptr, void *handle64) {
    lmoe_clear_error();
    if (!ptr || !handle64 || bytes == 0) return lmoe_fail(LMOE_ERR_INVALID, "peer_alloc: ptr/handle is NULL or bytes is 0");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is exchanged as 64 bytes");
    void *p = nullptr;
    LMOE_CUDA(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return lmoe_fail(LMOE_ERR_CUDA, "peer_alloc: %s", cudaGetErrorString(e));
    }
    memcpy(handle64, &h, 64);
    *ptr = p;
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_peer_open(const void *handle64, void **ptr) {
    lmoe_clear_error();
    if (!ptr || !handle64) return lmoe_fail(LMOE_ERR_INVALID, "peer_open: ptr/handle is NULL");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void *p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return lmoe_fail(LMOE_ERR_CUDA, "peer_open: %s", cudaGetErrorString(e));
    }
    *ptr = p;
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_peer_close(void *ptr) {
    lmoe_clear_error();
    if (ptr) LMOE_CUDA(cudaIpcCloseMemHandle(ptr));
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_peer_free(void *ptr) {
    lmoe_clear_error();
    if (ptr) LMOE_CUDA(cudaFree(ptr));
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_peer_put(const void *src, int64_t chunk_bytes, int32_t world, int32_t rank, int32_t per_rank_src,
                                     void *const *peer_bufs, void *const *peer_flags, void *local_ctrl, int32_t direction,
                                     void *stream) {
    lmoe_clear_error();
    if (!src || !peer_bufs || !peer_flags || !local_ctrl) return lmoe_fail(LMOE_ERR_INVALID, "peer_put: NULL argument");
    if (world < 1 || world > PEER_MAX_WORLD || rank < 0 || rank >= world)
        return lmoe_fail(LMOE_ERR_INVALID, "peer_put: world (%d) must be 1..%d and rank (%d) inside it", world, PEER_MAX_WORLD, rank);
    if (direction < 0 || direction > 1) return lmoe_fail(LMOE_ERR_INVALID, "peer_put: direction must be 0 or 1");
    if (chunk_bytes <= 0 || chunk_bytes % 16 || (reinterpret_cast<uintptr_t>(src) & 15u))
        return lmoe_fail(LMOE_ERR_INVALID, "peer_put: chunks are multiples of 16 bytes from a 16-byte aligned source");
    PeerPutParams P;
    P.src = static_cast<const uint8_t *>(src);
    for (int s = 0; s < PEER_MAX_WORLD; s++) {
        P.dst[s] = s < world ? static_cast<uint8_t *>(peer_bufs[s]) : nullptr;
        // every rank's control block: [0..15] flags of direction 0, [16..31] flags of direction 1
        P.flags[s] = s < world ? static_cast<uint32_t *>(peer_flags[s]) + 16 * direction : nullptr;
        if (s < world && (!P.dst[s] || !P.flags[s] || (reinterpret_cast<uintptr_t>(P.dst[s]) & 15u)))
            return lmoe_fail(LMOE_ERR_INVALID, "peer_put: buffer of rank %d is NULL or not 16-byte aligned", s);
    }
    uint32_t *ctrl = static_cast<uint32_t *>(local_ctrl);
    P.epoch = ctrl + 32 + direction;           // [32], [33]: epochs sent
    P.arrived = ctrl + 64 + 32 * direction;    // [64..80] / [96..112]: CTA counters, zero between launches
    P.chunk_bytes = chunk_bytes;
    P.world = world; P.rank = rank; P.per_rank_src = per_rank_src ? 1 : 0;
    int64_t want = (chunk_bytes / 16 + 255) / 256;
    const unsigned gx = (unsigned)(want < 1 ? 1 : (want > 16 ? 16 : want));
    peer_put_kernel<<<dim3(gx, (unsigned)world), 256, 0, (cudaStream_t)stream>>>(P);
    LMOE_LAUNCH_CHECK("peer_put_kernel");
    return LMOE_OK;
}

extern "C" lmoe_status lmoe_peer_wait(void *local_ctrl, int32_t world, int32_t direction, void *stream) {
    lmoe_clear_error();
    if (!local_ctrl) return lmoe_fail(LMOE_ERR_INVALID, "peer_wait: control block is NULL");
    if (world < 1 || world > PEER_MAX_WORLD || direction < 0 || direction > 1)
        return lmoe_fail(LMOE_ERR_INVALID, "peer_wait: world (%d) must be 1..%d, direction 0 or 1", world, PEER_MAX_WORLD);
    uint32_t *ctrl = static_cast<uint32_t *>(local_ctrl);
    peer_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ctrl + 16 * direction, ctrl + 32 + direction, world, ctrl + 40);
    LMOE_LAUNCH_CHECK("peer_wait_kernel");
    return LMOE_OK;
}

// Words of a rank's control block (lmoe_peer_alloc'd, zero-initialised): 128.  Word 40 collects wait time-outs.
extern "C" size_t lmoe_peer_ctrl_bytes(void) { return 128 * 4; }
