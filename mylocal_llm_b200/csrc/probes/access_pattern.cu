// Probe: HBM read rate of the direct kernel's per-lane access pattern (no arithmetic) as a function
// of how many items each warp keeps in flight, versus contiguous patterns. Standalone.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include <cstdlib>

__device__ __forceinline__ uint4 ldg128(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ldg128_l1(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// PATTERN 0: Q4_K rows (rb bytes per row): item = 16 rows x one 144-byte block; lane (g,tig) loads
//            hd(16) + qa(16 at 16+16tig) + qb(16 at 80+16tig) for rows g and g+8  (6 loads, 3 KB useful... 2304 B unique)
// PATTERN 1: same bytes but without the redundant hd loads by tig != 0 (predicated)
// PATTERN 2: contiguous: item = 6 x 512 contiguous bytes per warp (tile layout)
// PATTERN 3: pattern 0 with L1-allocating loads
template <int PATTERN, int DEPTH>
__global__ void __launch_bounds__(512, 1) pat_kernel(const uint8_t *w, int n_rows, int nsb, unsigned *sink) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int rb = nsb * 144;
    const int groups = n_rows / 16;
    const long long items = (long long)groups * nsb;
    const long long per_warp = items / ((long long)gridDim.x * 16);
    const long long first = ((long long)blockIdx.x * 16 + warp) * per_warp;
    uint4 buf[DEPTH][6];
    unsigned acc = 0;
    auto issue = [&](long long it, uint4 (&b)[6]) {
        const long long grp = it / nsb;
        const int sb = (int)(it - grp * nsb);
        if (PATTERN == 2) {
            const uint8_t *tile = w + (size_t)it * 2304;   // same unique bytes per item, contiguous
#pragma unroll
            for (int p = 0; p < 6; ++p) b[p] = (p < 5 || lane < 16) ? ldg128(tile + (p * 512 + lane * 16) % 2304) : make_uint4(0,0,0,0);
        } else {
            const uint8_t *lo = w + ((size_t)grp * 16 + g) * rb + (size_t)sb * 144;
            const uint8_t *hi = lo + (size_t)8 * rb;
            if (PATTERN == 3) {
                b[0] = ldg128_l1(lo); b[1] = ldg128_l1(lo + 16 + 16 * tig); b[2] = ldg128_l1(lo + 80 + 16 * tig);
                b[3] = ldg128_l1(hi); b[4] = ldg128_l1(hi + 16 + 16 * tig); b[5] = ldg128_l1(hi + 80 + 16 * tig);
            } else {
                b[0] = (PATTERN == 1 && tig) ? make_uint4(0,0,0,0) : ldg128(lo);
                b[1] = ldg128(lo + 16 + 16 * tig); b[2] = ldg128(lo + 80 + 16 * tig);
                b[3] = (PATTERN == 1 && tig) ? make_uint4(0,0,0,0) : ldg128(hi);
                b[4] = ldg128(hi + 16 + 16 * tig); b[5] = ldg128(hi + 80 + 16 * tig);
            }
        }
    };
#pragma unroll
    for (int d = 0; d < DEPTH - 1; ++d) issue(first + d, buf[d]);
    for (long long i = 0; i < per_warp; i += DEPTH) {
#pragma unroll
        for (int d = 0; d < DEPTH; ++d) {
            const long long nxt = i + d + DEPTH - 1;
            if (nxt < per_warp) issue(first + nxt, buf[(d + DEPTH - 1) % DEPTH]);
            if (i + d < per_warp) {
#pragma unroll
                for (int p = 0; p < 6; ++p) acc ^= buf[d][p].x ^ buf[d][p].y ^ buf[d][p].z ^ buf[d][p].w;
            }
        }
    }
    if (acc == 0x12345u) sink[0] = acc;
}

template <int P, int D>
static void run(const char *name, const uint8_t *w, int n_rows, int nsb, unsigned *sink) {
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    float best = 1e9f;
    for (int rep = 0; rep < 3; ++rep) {
        cudaEventRecord(e0);
        pat_kernel<P, D><<<148, 512>>>(w, n_rows, nsb, sink);
        cudaEventRecord(e1); cudaEventSynchronize(e1);
        float ms; cudaEventElapsedTime(&ms, e0, e1);
        if (ms < best) best = ms;
    }
    const double bytes = (double)n_rows * nsb * 144;
    printf("%-44s depth %d  nsb %2d : %7.1f GB/s (%.3f ms)  %s\n", name, D, nsb, bytes / best / 1e6, best, cudaGetErrorString(cudaGetLastError()));
}

int main() {
    const size_t total = (size_t)1 << 30;
    uint8_t *buf; unsigned *sink;
    cudaMalloc(&buf, total + 4096); cudaMalloc(&sink, 8);
    cudaMemset(buf, 1, total + 4096);
    for (int nsb : {8, 32}) {
        const int n_rows = (int)(total / ((size_t)nsb * 144)) / 16 * 16;
        run<0, 1>("rows: hd+qa+qb per lane", buf, n_rows, nsb, sink);
        run<0, 2>("rows: hd+qa+qb per lane", buf, n_rows, nsb, sink);
        run<0, 3>("rows: hd+qa+qb per lane", buf, n_rows, nsb, sink);
        run<0, 4>("rows: hd+qa+qb per lane", buf, n_rows, nsb, sink);
        run<1, 1>("rows: hd by tig 0 only", buf, n_rows, nsb, sink);
        run<1, 2>("rows: hd by tig 0 only", buf, n_rows, nsb, sink);
        run<1, 4>("rows: hd by tig 0 only", buf, n_rows, nsb, sink);
        run<3, 1>("rows: L1-allocating loads", buf, n_rows, nsb, sink);
        run<3, 2>("rows: L1-allocating loads", buf, n_rows, nsb, sink);
        run<3, 4>("rows: L1-allocating loads", buf, n_rows, nsb, sink);
        run<2, 1>("contiguous 2304 B per warp item", buf, n_rows, nsb, sink);
        run<2, 2>("contiguous 2304 B per warp item", buf, n_rows, nsb, sink);
        run<2, 4>("contiguous 2304 B per warp item", buf, n_rows, nsb, sink);
    }
    return 0;
}
