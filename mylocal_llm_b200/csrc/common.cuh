// Shared device/host helpers for the b200q kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200q.h"

namespace b200q {

// ---------------------------------------------------------------------------------------------
// Formats (block layouts: mini_llm/ops/quantized_weight.py:24-37 of the reference)
// ---------------------------------------------------------------------------------------------
__host__ __device__ constexpr int fmt_elems(int fmt) { return (fmt == B200Q_Q8_0 || fmt == B200Q_Q4_0) ? 32 : 256; }
__host__ __device__ constexpr int fmt_bytes(int fmt) {
    return fmt == B200Q_Q8_0 ? 34 : fmt == B200Q_Q4_0 ? 18 : fmt == B200Q_Q3_K ? 110 : fmt == B200Q_Q4_K ? 144
         : fmt == B200Q_Q5_K ? 176 : fmt == B200Q_Q6_K ? 210 : 0;
}
inline bool fmt_valid(int fmt) {
    return fmt == B200Q_Q8_0 || fmt == B200Q_Q4_0 || fmt == B200Q_Q3_K || fmt == B200Q_Q4_K || fmt == B200Q_Q5_K ||
           fmt == B200Q_Q6_K;
}
// The two legacy formats run on the FP32-lane kernels only (no tensor-core fragment builder, no tile layout).
inline bool fmt_lanes_only(int fmt) { return fmt == B200Q_Q4_0 || fmt == B200Q_Q3_K; }
inline bool dtype_valid(int dt) { return dt == B200Q_F32 || dt == B200Q_F16 || dt == B200Q_BF16; }
inline size_t dtype_size(int dt) { return dt == B200Q_F32 ? 4 : 2; }

// Host-side error reporting (thread local; message of the last failing call).
void set_error(const char *fmt, ...);
int fail(int rc, const char *fmt, ...);
int check_launch(const char *what);

// Device status word: kernels that give up on a bounded wait store a code here.
int *device_status_word();
constexpr int STATUS_WAIT_FULL = 101;   // consumer gave up waiting for a staged tile
constexpr int STATUS_WAIT_EMPTY = 102;  // producer gave up waiting for a free stage
constexpr int STATUS_POSITION_RANGE = 301;  // a decode position lay outside the cache or the RoPE tables

constexpr int NUM_SMS_FALLBACK = 148;
int sm_count();

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch. The decode step is a chain of short kernels on one stream; a
// kernel launched through launch_chained() may become resident while its predecessor drains, and
// blocks in chain_wait() until the predecessor grid has completed and its writes are visible.
// Rules every such kernel follows:
//   * chain_wait() is executed by every thread before the first access to memory that a preceding
//     kernel writes (activations, plans, caches) and before its own first global write; only
//     read-only weights may be requested earlier;
//   * chain_trigger() lets the next kernel in the stream be scheduled; it carries no memory
//     guarantee (the next kernel's own chain_wait() does).
// Launched without the attribute (B200Q_CHAIN=0, or after a kernel that is launched normally)
// both calls are no-ops and the stream order is the usual full serialisation.
// ---------------------------------------------------------------------------------------------
bool chain_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = chain_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a kernel that runs as thread-block clusters of `cluster_x` CTAs along x.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                          cudaStream_t stream, int cluster_x, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = chain_enabled() ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster_x;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Q4_K / Q5_K in their tile layouts: the GGUF format a tile-layout id stands for, or -1 for any other id.
inline int direct_tiled_base(int fmt) {
    return fmt == B200Q_Q4_K_TILED ? B200Q_Q4_K : fmt == B200Q_Q5_K_TILED ? B200Q_Q5_K : -1;
}

// Routing-plan outputs the top-k kernel fills itself when it routes a single row (order == nullptr:
// none). For one row the plan is a sort of k distinct ids, so the separate plan launch of a
// one-token decode step is saved; the arrays are those of b200q_moe_plan.
struct RowPlanOut {
    int32_t *counts, *offsets, *order, *inv, *seg_expert, *seg_begin, *seg_count, *num_segments, *status;
    int e;                 // experts of the plan (counts has e entries, offsets e + 1)
    int max_segments;
};

// ---------------------------------------------------------------------------------------------
// Small device utilities
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Asks L2 for the lines of [base, base + bytes), all threads of the CTA taking part; nothing is
// requested when the range exceeds `cap` bytes. It returns nothing to the thread, so it may run
// before chain_wait(): a small dense GEMV that became resident early pulls its slice of the
// weights towards L2 while the preceding kernel finishes. (Large slices are left alone: a
// prefetch running ahead of the register loads of a long stream measured 7-30 % slower than the
// loads by themselves.)
__device__ __forceinline__ void prefetch_l2_range(const uint8_t *base, size_t bytes, size_t cap, int tid, int threads) {
    if (bytes > cap) return;
    for (size_t off = static_cast<size_t>(tid) * 128; off < bytes; off += static_cast<size_t>(threads) * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
}
constexpr size_t CHAIN_PREFETCH_BYTES = 256 * 1024;     // per CTA

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ float half_bits_to_float(uint32_t bits16) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
}

__device__ __forceinline__ float load_as_float(const void *p, int dtype, size_t i) {
    if (dtype == B200Q_F32) return static_cast<const float *>(p)[i];
    if (dtype == B200Q_F16) return __half2float(static_cast<const __half *>(p)[i]);
    return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
}

__device__ __forceinline__ void store_from_float(void *p, int dtype, size_t i, float v) {
    if (dtype == B200Q_F32) static_cast<float *>(p)[i] = v;
    else if (dtype == B200Q_F16) static_cast<__half *>(p)[i] = __float2half_rn(v);
    else static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// silu(g)*u with an overflow-safe logistic, as the reference's CPU kernel
// (mini_llm/ops/native_packed_cpu.cpp:236-238).
__device__ __forceinline__ float swiglu_f32(float g, float u) {
    float s = g >= 0.0f ? 1.0f / (1.0f + __expf(-g)) : __expf(g) / (1.0f + __expf(g));
    return (g * s) * u;
}

// Start of expert `e`'s packed matrix: entry of a device pointer table when one is given,
// otherwise base + e * stride inside a contiguous bank.
// Where a route-weighted term row goes. Without a table: row `row` of the local buffer. With a table
// (one base address per rank, possibly peer memory): rank row / rows_per_rank owns the row.
__device__ __forceinline__ float *term_row_pointer(float *local, const uint64_t *table, int rows_per_rank, int n,
                                                   int row) {
    if (!table) return local + static_cast<size_t>(row) * n;
    const int home = row / rows_per_rank;
    return reinterpret_cast<float *>(table[home]) + static_cast<size_t>(row - home * rows_per_rank) * n;
}

__device__ __forceinline__ const uint8_t *expert_matrix(const uint8_t *base, long long stride,
                                                        const unsigned long long *table, int e) {
    if (table) return reinterpret_cast<const uint8_t *>(static_cast<uintptr_t>(table[e]));
    return base + static_cast<long long>(e) * stride;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------------------------------------
// mbarrier + bulk-copy (TMA, untiled) wrappers. No cluster multicast anywhere.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wait with a wall-clock limit. Returns false (and records `code`) instead of spinning forever.
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;  // 2 s
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, int *status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > WAIT_LIMIT_NS) {
            atomicExch(status, code);
            return false;
        }
    }
}

// 1-D bulk copy global -> this CTA's shared memory; dst, src 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_copy_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes,
                                              uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

}  // namespace b200q
