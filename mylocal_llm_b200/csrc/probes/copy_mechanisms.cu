// Probe: how fast can the SMs pull bytes from HBM with (a) cp.async.bulk of various sizes,
// (b) plain 128-bit loads, (c) cp.async 16B. Standalone; prints GB/s.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include <cstdlib>

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__global__ void __launch_bounds__(288, 1) bulk_kernel(const uint8_t* src, size_t bytes_per_cta, int chunk, int copies_per_stage,
                                                   int stages, unsigned long long* sink) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = (uint64_t*)smem;
    uint64_t* empty = full + 16;
    uint8_t* ring = smem + 1024;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int stage_bytes = chunk * copies_per_stage;
    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&full[s])), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&empty[s])), "r"(8));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    const uint8_t* base = src + (size_t)blockIdx.x * bytes_per_cta;
    const int tiles = (int)(bytes_per_cta / stage_bytes);
    if (warp == 8) {
        for (int it = 0; it < tiles; ++it) {
            const int s = it % stages;
            if (it >= stages) {
                uint32_t ok = 0;
                const uint32_t par = ((it / stages) - 1) & 1;
                for (int spin = 0; !ok && spin < (1 << 24); ++spin) asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0,1,0,p; }" : "=r"(ok) : "r"(s32(&empty[s])), "r"(par) : "memory");
            }
            if (lane == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(&full[s])), "r"(stage_bytes) : "memory");
            __syncwarp();
            for (int c = lane; c < copies_per_stage; c += 32) {
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 s32(ring + (size_t)s * stage_bytes + (size_t)c * chunk)),
                             "l"(base + (size_t)it * stage_bytes + (size_t)c * chunk), "r"(chunk), "r"(s32(&full[s]))
                             : "memory");
            }
        }
        return;
    }
    unsigned long long acc = 0;
    for (int it = 0; it < tiles; ++it) {
        const int s = it % stages;
        uint32_t ok = 0;
        const uint32_t par = (it / stages) & 1;
        for (int spin = 0; !ok && spin < (1 << 24); ++spin) asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0,1,0,p; }" : "=r"(ok) : "r"(s32(&full[s])), "r"(par) : "memory");
        acc += ring[(size_t)s * stage_bytes + tid];
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(&empty[s])) : "memory");
    }
    if (acc == 0x1234567) sink[0] = acc;
}

__global__ void __launch_bounds__(512) ldg_kernel(const uint4* src, size_t vec_per_cta, unsigned long long* sink) {
    const uint4* p = src + (size_t)blockIdx.x * vec_per_cta;
    uint4 acc = make_uint4(0, 0, 0, 0);
    for (size_t i = threadIdx.x; i + 7 * 512 < vec_per_cta; i += 8 * 512) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w) : "l"(p + i + u * 512));
#pragma unroll
        for (int u = 0; u < 8; ++u) { acc.x ^= v[u].x; acc.y ^= v[u].y; acc.z ^= v[u].z; acc.w ^= v[u].w; }
    }
    if ((acc.x ^ acc.y ^ acc.z ^ acc.w) == 0x12345) sink[0] = acc.x;
}

// cp.async 16B ring: stage = 512 threads * 16 B * per = chunk
__global__ void __launch_bounds__(512, 1) ldgsts_kernel(const uint8_t* src, size_t bytes_per_cta, int per, int stages, unsigned long long* sink) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x;
    const int stage_bytes = 512 * 16 * per;
    const uint8_t* base = src + (size_t)blockIdx.x * bytes_per_cta;
    const int tiles = (int)(bytes_per_cta / stage_bytes);
    unsigned acc = 0;
    auto issue = [&](int it) {
        const int s = it % stages;
        if (it < tiles) {
            for (int j = 0; j < per; ++j) {
                const size_t off = ((size_t)j * 512 + tid) * 16;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s32(smem + (size_t)s * stage_bytes + off)), "l"(base + (size_t)it * stage_bytes + off) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int it = 0; it < stages - 1; ++it) issue(it);
    for (int it = 0; it < tiles; ++it) {
        asm volatile("cp.async.wait_group %0;" ::"n"(6) : "memory");   // stages-2 == 6 when stages == 8
        __syncthreads();
        issue(it + stages - 1);
        acc += smem[(size_t)(it % stages) * stage_bytes + tid * 16];
    }
    if (acc == 0x1234567) sink[0] = acc;
}

int main(int argc, char** argv) {
    const size_t total = (size_t)2 << 30;  // 2 GiB
    uint8_t* buf; unsigned long long* sink;
    cudaMalloc(&buf, total); cudaMalloc(&sink, 8);
    cudaMemset(buf, 1, total);
    int sms = 148;
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    auto report = [&](const char* name, float ms, size_t bytes) { printf("%-40s %8.1f GB/s  (%.3f ms)\n", name, bytes / ms / 1e6, ms); };
    // (a) bulk
    cudaFuncSetAttribute(bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    struct Cfg { int chunk, copies, stages; } cfgs[] = {
        {1152, 16, 8}, {1152, 16, 4}, {1152, 32, 4}, {2304, 8, 8}, {4608, 4, 8}, {18432, 1, 8}, {18432, 1, 4}, {36864, 1, 4}, {36864, 1, 5}, {65536, 1, 3}, {9216, 2, 8}, {1152, 64, 2}, {576, 32, 8}};
    for (auto c : cfgs) {
        const int stage_bytes = c.chunk * c.copies;
        size_t per_cta = (total / sms) / stage_bytes * stage_bytes;
        per_cta = per_cta / 4;  // 0.5 GiB total
        const int smem = 1024 + stage_bytes * c.stages;
        for (int rep = 0; rep < 2; ++rep) {
            cudaEventRecord(e0);
            bulk_kernel<<<sms, 288, smem>>>(buf, per_cta, c.chunk, c.copies, c.stages, sink);
            cudaEventRecord(e1); cudaEventSynchronize(e1);
        }
        float ms; cudaEventElapsedTime(&ms, e0, e1);
        char name[128]; snprintf(name, 128, "bulk chunk=%d x%d stages=%d (%d KB ring)", c.chunk, c.copies, c.stages, stage_bytes * c.stages / 1024);
        report(name, ms, per_cta * sms);
        cudaError_t err = cudaGetLastError(); if (err) printf("  err %s\n", cudaGetErrorString(err));
    }
    // (b) ldg
    for (int ctas_per_sm = 1; ctas_per_sm <= 4; ctas_per_sm *= 2) {
        const int grid = sms * ctas_per_sm;
        size_t vec_per_cta = (total / 4 / 16) / grid / 4096 * 4096;
        for (int rep = 0; rep < 2; ++rep) { cudaEventRecord(e0); ldg_kernel<<<grid, 512>>>((const uint4*)buf, vec_per_cta, sink); cudaEventRecord(e1); cudaEventSynchronize(e1); }
        float ms; cudaEventElapsedTime(&ms, e0, e1);
        char name[128]; snprintf(name, 128, "ldg.128 x8 unroll, %d CTA/SM of 512", ctas_per_sm);
        report(name, ms, vec_per_cta * 16 * grid);
    }
    // (c) cp.async 16B ring
    cudaFuncSetAttribute(ldgsts_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    for (int per = 1; per <= 3; ++per) {
        const int stages = 8;
        const int stage_bytes = 512 * 16 * per;
        size_t per_cta = (total / 4 / sms) / stage_bytes * stage_bytes;
        for (int rep = 0; rep < 2; ++rep) { cudaEventRecord(e0); ldgsts_kernel<<<sms, 512, stage_bytes * stages>>>(buf, per_cta, per, stages, sink); cudaEventRecord(e1); cudaEventSynchronize(e1); }
        float ms; cudaEventElapsedTime(&ms, e0, e1);
        char name[128]; snprintf(name, 128, "cp.async16 stage=%d KB x8 stages", stage_bytes / 1024);
        report(name, ms, per_cta * sms);
        cudaError_t err = cudaGetLastError(); if (err) printf("  err %s\n", cudaGetErrorString(err));
    }
    return 0;
}
