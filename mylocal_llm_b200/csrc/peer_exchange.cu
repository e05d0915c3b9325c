// Exchange of activations and expert terms between the GPUs of one node through peer memory.
//
// Every rank (one process per GPU) owns one arena allocated with cudaMalloc and exported with a
// CUDA IPC handle; every rank maps every other rank's arena. The arena holds a small signal pad,
// the gathered activation rows and the term rows this rank is home of. Kernels then move data with
// plain stores into the mapped peer arenas (NVLink); nothing here uses TMA or multicast.
//
//   b200q_peer_push_rows : copy this rank's rows into slot `rank` of every rank's gather buffer
//   b200q_peer_barrier   : all ranks have finished everything they launched before the barrier
//   (the grouped down projection writes its term rows straight into the home rank's arena, see
//    b200q_moe_down_peer)
//
// The barrier kernels of the different ranks wait on one another. They run on different GPUs, one
// process each; they must never be launched as several ranks on one GPU. Every wait is bounded: a
// rank that does not see its peers within the time limit records STATUS_PEER_BARRIER in the device
// status word and returns, so the context stays usable and the host can report the failure.
#include "common.cuh"

namespace b200q {

constexpr int PEER_MAX_RANKS = 16;
constexpr int PEER_EPOCH_SLOT = PEER_MAX_RANKS;        // pad[16]: this rank's barrier count
constexpr int STATUS_PEER_BARRIER = 201;

__device__ __forceinline__ void store_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One warp. Lane p signals rank p (writes this rank's barrier count into slot `rank` of p's pad) and
// then waits until rank p's count has arrived in slot p of the local pad.
__global__ void __launch_bounds__(32) peer_barrier_kernel(const uint64_t *pads, int rank, int world,
                                                          unsigned long long timeout_ns, int *status) {
    uint32_t *mine = reinterpret_cast<uint32_t *>(pads[rank]);
    const int lane = threadIdx.x;
    uint32_t epoch = 0;
    if (lane == 0) {
        epoch = mine[PEER_EPOCH_SLOT] + 1u;
        mine[PEER_EPOCH_SLOT] = epoch;
    }
    epoch = __shfl_sync(0xffffffffu, epoch, 0);
    __threadfence_system();
    if (lane < world && lane != rank) {
        store_release_sys(reinterpret_cast<uint32_t *>(pads[lane]) + rank, epoch);
        const uint64_t t0 = global_timer_ns();
        while (true) {
            const uint32_t seen = load_acquire_sys(mine + lane);
            if (static_cast<int32_t>(seen - epoch) >= 0) break;
            if (global_timer_ns() - t0 > timeout_ns) {
                atomicExch(status, STATUS_PEER_BARRIER);
                break;
            }
            __nanosleep(64);
        }
    }
    __threadfence_system();
}

// grid (blocks, world): block column p copies the local rows into rank p's gather buffer.
__global__ void __launch_bounds__(256) peer_push_kernel(const uint4 *src, long long n16, const uint64_t *dst_bases,
                                                        long long dst_offset16) {
    uint4 *dst = reinterpret_cast<uint4 *>(dst_bases[blockIdx.y]) + dst_offset16;
    for (long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; i < n16;
         i += static_cast<long long>(gridDim.x) * 256)
        dst[i] = src[i];
}

// Up to three buffers in one launch: grid (blocks, world, 3); segment z of rank p goes to
// dst_bases[p] + offset[z].
struct PushSegments {
    const uint8_t *src[3];
    long long bytes[3];
    long long dst_offset[3];
    int wide[3];          // 1: everything is 16-byte aligned (uint4 copies), 0: 4-byte copies
};
__global__ void __launch_bounds__(256) peer_push3_kernel(const PushSegments seg, const uint64_t *dst_bases) {
    const int z = blockIdx.z;
    const uint8_t *src = seg.src[z];
    uint8_t *dst = reinterpret_cast<uint8_t *>(dst_bases[blockIdx.y]) + seg.dst_offset[z];
    const long long first = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    const long long step = static_cast<long long>(gridDim.x) * 256;
    if (seg.wide[z]) {
        for (long long i = first; i < seg.bytes[z] / 16; i += step)
            reinterpret_cast<uint4 *>(dst)[i] = reinterpret_cast<const uint4 *>(src)[i];
    } else {
        for (long long i = first; i < seg.bytes[z] / 4; i += step)
            reinterpret_cast<uint32_t *>(dst)[i] = reinterpret_cast<const uint32_t *>(src)[i];
    }
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_peer_alloc(size_t bytes, void **ptr, unsigned char *handle) {
    if (!ptr || !handle || bytes == 0) return fail(B200Q_EINVAL, "peer_alloc: bad argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void *p = nullptr;
    cudaError_t err = cudaMalloc(&p, bytes);
    if (err == cudaSuccess) err = cudaMemset(p, 0, bytes);
    if (err == cudaSuccess) err = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (err == cudaSuccess) err = cudaIpcGetMemHandle(&h, p);
    if (err != cudaSuccess) {
        cudaGetLastError();
        if (p) cudaFree(p);
        return fail(B200Q_ECUDA, "peer_alloc: %s", cudaGetErrorString(err));
    }
    memcpy(handle, &h, sizeof(h));
    *ptr = p;
    return B200Q_OK;
}

int b200q_peer_open(const unsigned char *handle, void **ptr) {
    if (!handle || !ptr) return fail(B200Q_EINVAL, "peer_open: NULL pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void *p = nullptr;
    cudaError_t err = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "peer_open: %s", cudaGetErrorString(err));
    }
    *ptr = p;
    return B200Q_OK;
}

int b200q_peer_close(void *ptr) {
    if (!ptr) return B200Q_OK;
    cudaError_t err = cudaIpcCloseMemHandle(ptr);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "peer_close: %s", cudaGetErrorString(err));
    }
    return B200Q_OK;
}

int b200q_peer_free(void *ptr) {
    if (!ptr) return B200Q_OK;
    cudaError_t err = cudaFree(ptr);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "peer_free: %s", cudaGetErrorString(err));
    }
    return B200Q_OK;
}

int b200q_peer_barrier(const uint64_t *pads, int rank, int world, int timeout_ms, void *stream) {
    if (!pads) return fail(B200Q_EINVAL, "peer_barrier: NULL pointer");
    if (world < 1 || world > PEER_MAX_RANKS || rank < 0 || rank >= world || timeout_ms < 1)
        return fail(B200Q_EINVAL, "peer_barrier: bad argument (world <= %d)", PEER_MAX_RANKS);
    int *status = device_status_word();
    if (!status) return fail(B200Q_ECUDA, "peer_barrier: no CUDA device");
    peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        pads, rank, world, static_cast<unsigned long long>(timeout_ms) * 1000000ull, status);
    return check_launch("peer_barrier");
}

int b200q_peer_push_rows(const void *src, size_t bytes, const uint64_t *dst_bases, size_t dst_offset_bytes,
                         int world, void *stream) {
    if (!src || !dst_bases) return fail(B200Q_EINVAL, "peer_push_rows: NULL pointer");
    if (world < 1 || world > PEER_MAX_RANKS) return fail(B200Q_EINVAL, "peer_push_rows: bad world size");
    if (bytes == 0) return B200Q_OK;
    if (bytes % 16 || dst_offset_bytes % 16 || reinterpret_cast<uintptr_t>(src) % 16)
        return fail(B200Q_EINVAL, "peer_push_rows: sizes and addresses must be multiples of 16 bytes");
    const long long n16 = static_cast<long long>(bytes / 16);
    const int blocks = static_cast<int>(std::min<long long>((n16 + 255) / 256, 64));
    peer_push_kernel<<<dim3(blocks, world), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4 *>(src), n16, dst_bases, static_cast<long long>(dst_offset_bytes / 16));
    return check_launch("peer_push_rows");
}

int b200q_peer_push3(const void *src0, size_t bytes0, size_t dst_offset0, const void *src1, size_t bytes1,
                     size_t dst_offset1, const void *src2, size_t bytes2, size_t dst_offset2,
                     const uint64_t *dst_bases, int world, void *stream) {
    if (!dst_bases) return fail(B200Q_EINVAL, "peer_push3: NULL pointer");
    if (world < 1 || world > PEER_MAX_RANKS) return fail(B200Q_EINVAL, "peer_push3: bad world size");
    const void *srcs[3] = {src0, src1, src2};
    const size_t bytes[3] = {bytes0, bytes1, bytes2}, offs[3] = {dst_offset0, dst_offset1, dst_offset2};
    PushSegments seg{};
    long long most = 0;
    for (int z = 0; z < 3; ++z) {
        if (bytes[z] && !srcs[z]) return fail(B200Q_EINVAL, "peer_push3: NULL source");
        if (bytes[z] % 4 || offs[z] % 4 || reinterpret_cast<uintptr_t>(srcs[z]) % 4)
            return fail(B200Q_EINVAL, "peer_push3: sizes and addresses must be multiples of 4 bytes");
        seg.src[z] = static_cast<const uint8_t *>(srcs[z]);
        seg.bytes[z] = static_cast<long long>(bytes[z]);
        seg.dst_offset[z] = static_cast<long long>(offs[z]);
        seg.wide[z] = !(bytes[z] % 16 || offs[z] % 16 || reinterpret_cast<uintptr_t>(srcs[z]) % 16);
        const long long units = static_cast<long long>(bytes[z]) / (seg.wide[z] ? 16 : 4);
        if (units > most) most = units;
    }
    if (most == 0) return B200Q_OK;
    const int blocks = static_cast<int>(std::min<long long>((most + 255) / 256, 64));
    peer_push3_kernel<<<dim3(blocks, world, 3), 256, 0, static_cast<cudaStream_t>(stream)>>>(seg, dst_bases);
    return check_launch("peer_push3");
}

}  // extern "C"
