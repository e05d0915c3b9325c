// Row-wise RMSNorm and the ordered combine fused with it, as device functions: the kernels of
// aux_kernels.cu run them for one row per CTA, the persistent one-token MoE step for its single row.
#pragma once

#include "common.cuh"

namespace b200q {

// ---------------------------------------------------------------------------------- RMSNorm
// One 256-thread CTA per row. FP32 math with the reference's operation order
// (mini_llm/ops/rmsnorm_inference.py:80-119): mean = sum/d, inv = 1/sqrt(mean+eps) by correctly
// rounded division and square root, y = (x*inv)*gamma.
// rmsnorm_row is the work of the 256 threads that handle row `row` (res_out may be null: the sum is then not stored)
// rmsnorm_row is the work of the 256 threads that handle row `row` (tid = 0..255; they meet at named barrier
// ROW_BARRIER, so a CTA with more threads can run it on its first eight warps).
constexpr int ROW_BARRIER = 12;
constexpr int ROW_THREADS = 256;
__device__ __forceinline__ void row_sync() { named_barrier_sync(ROW_BARRIER, ROW_THREADS); }

template <bool RESIDUAL>
__device__ __forceinline__ void rmsnorm_row(const int row, const int tid, const void *x, int x_dtype, const float *residual,
                                            float alpha, const void *gamma, int gamma_dtype, int d, float eps,
                                            float *res_out, void *y, int y_dtype) {
    __shared__ float warp_sums[8];
    __shared__ float inv_shared;
    const size_t base = static_cast<size_t>(row) * d;
    const int lane = tid & 31, warp = tid >> 5;
    // Rows of up to 256 * KEEP columns stay in registers between the two passes (with their gamma
    // values, requested together with the row), so nothing is loaded after the reduction.
    constexpr int KEEP = 16;
    const bool in_regs = d <= 256 * KEEP;
    float kept[KEEP], gam[KEEP];
    float ss = 0.f;
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < KEEP; ++i) {
            const int c = tid + 256 * i;
            kept[i] = 0.f;
            gam[i] = 0.f;
            if (c < d) {
                float v = load_as_float(x, x_dtype, base + c);
                if (RESIDUAL) v = residual[base + c] + alpha * v;
                kept[i] = v;
                gam[i] = load_as_float(gamma, gamma_dtype, c);
            }
        }
#pragma unroll
        for (int i = 0; i < KEEP; ++i)
            if (tid + 256 * i < d) ss += kept[i] * kept[i];
    } else {
        for (int c = tid; c < d; c += 256) {
            float v = load_as_float(x, x_dtype, base + c);
            if (RESIDUAL) v = residual[base + c] + alpha * v;
            ss += v * v;
        }
    }
    ss = warp_sum(ss);
    if (lane == 0) warp_sums[warp] = ss;
    row_sync();
    if (warp == 0) {
        float t = lane < 8 ? warp_sums[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) inv_shared = __fdiv_rn(1.0f, __fsqrt_rn(__fdiv_rn(t, static_cast<float>(d)) + eps));
    }
    row_sync();
    const float inv = inv_shared;
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < KEEP; ++i) {
            const int c = tid + 256 * i;
            if (c < d) {
                if (RESIDUAL && res_out) res_out[base + c] = kept[i];
                store_from_float(y, y_dtype, base + c, (kept[i] * inv) * gam[i]);
            }
        }
        return;
    }
    for (int c = tid; c < d; c += 256) {
        float v = load_as_float(x, x_dtype, base + c);
        if (RESIDUAL) {
            v = residual[base + c] + alpha * v;
            if (res_out) res_out[base + c] = v;
        }
        store_from_float(y, y_dtype, base + c, (v * inv) * load_as_float(gamma, gamma_dtype, c));
    }
}

// A value after a round trip through the storage type `dtype` (what a kernel that stored it and a
// kernel that loaded it again would see).
__device__ __forceinline__ float round_through(int dtype, float v) {
    if (dtype == B200Q_F16) return __half2float(__float2half_rn(v));
    if (dtype == B200Q_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    return v;
}

// Ordered combine of a row's k expert terms fused with the residual add and RMSNorm that follow it
// in a decoder layer: branch = the ordered sum rounded to `branch_dtype`, res = residual +
// alpha*branch, y = rmsnorm(res)*gamma. The arithmetic is that of moe_combine_cols_kernel followed
// by rmsnorm_kernel<true> (same order of adds, same rounding of the branch to its storage type,
// same column-to-thread mapping and reduction tree), so the fused step returns the same bits as the
// two kernels, one launch and one round trip through HBM earlier.
template <int KMAX, int CU = 4>
__device__ __forceinline__ void combine_norm_row(const int row, const int tid, const float *terms, const int32_t *inv, int k,
                                                 int d, const float *extra, const float *extra_scale, int branch_dtype,
                                                 const float *residual, float alpha, const void *gamma, int gamma_dtype,
                                                 float eps, float *res_out, void *y, int y_dtype) {
    __shared__ int pos_sorted[KMAX];
    __shared__ int pos_raw[KMAX];
    __shared__ float warp_sums[8];
    __shared__ float inv_shared;
    const int lane = tid & 31, warp = tid >> 5;
    if (tid < k) pos_raw[tid] = inv[static_cast<size_t>(row) * k + tid];
    row_sync();
    if (tid < k) {
        const int p = pos_raw[tid];
        int r = 0;
        for (int j = 0; j < k; ++j) r += pos_raw[j] < p;
        pos_sorted[r] = p;
    }
    row_sync();
    const size_t base = static_cast<size_t>(row) * d;
    const float scale = (extra && extra_scale) ? extra_scale[row] : 1.0f;
    // A thread owns columns tid, tid+256, ... (the mapping of rmsnorm_kernel, so the sum of squares
    // is accumulated in the same order). CU columns are in flight together: all their term loads are
    // issued before the first add. The first KEEP results stay in registers for the second pass.
    constexpr int KEEP = 16;        // (CU: a caller with fewer registers per thread keeps fewer columns in flight)
    float ss = 0.f;
    auto chunk = [&](int c0, float (&out)[CU]) {
        float t[CU][KMAX], res_in[CU], ex[CU];
#pragma unroll
        for (int u = 0; u < CU; ++u) {
            const int c = c0 + 256 * u;
            if (c < d) {
#pragma unroll
                for (int r = 0; r < KMAX; ++r)
                    if (r < k) t[u][r] = terms[static_cast<size_t>(pos_sorted[r]) * d + c];
                res_in[u] = residual[base + c];
                ex[u] = extra ? extra[base + c] : 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < CU; ++u) {
            const int c = c0 + 256 * u;
            out[u] = 0.f;
            if (c < d) {
                float acc = 0.f;
#pragma unroll
                for (int r = 0; r < KMAX; ++r)
                    if (r < k) acc = __fadd_rn(acc, t[u][r]);
                if (extra) acc = __fadd_rn(acc, __fmul_rn(ex[u], scale));
                float v = round_through(branch_dtype, acc);
                v = res_in[u] + alpha * v;
                res_out[base + c] = v;
                out[u] = v;
                ss += v * v;
            }
        }
    };
    float kept[KEEP / CU][CU];
#pragma unroll
    for (int it = 0; it < KEEP / CU; ++it)
        if (tid + 256 * CU * it < d) chunk(tid + 256 * CU * it, kept[it]);
    for (int c0 = tid + 256 * KEEP; c0 < d; c0 += 256 * CU) {
        float unused[CU];
        chunk(c0, unused);
    }
    ss = warp_sum(ss);
    if (lane == 0) warp_sums[warp] = ss;
    row_sync();
    if (warp == 0) {
        float t = lane < 8 ? warp_sums[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) inv_shared = __fdiv_rn(1.0f, __fsqrt_rn(__fdiv_rn(t, static_cast<float>(d)) + eps));
    }
    row_sync();
    const float inv_rms = inv_shared;
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
        const int c = tid + 256 * i;
        if (c < d)
            store_from_float(y, y_dtype, base + c, (kept[i / CU][i % CU] * inv_rms) * load_as_float(gamma, gamma_dtype, c));
    }
    for (int c = tid + 256 * KEEP; c < d; c += 256) {
        const float v = res_out[base + c];          // written by this thread above
        store_from_float(y, y_dtype, base + c, (v * inv_rms) * load_as_float(gamma, gamma_dtype, c));
    }
}

}  // namespace b200q
