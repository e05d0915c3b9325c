// Decode-oriented router kernels: logits from an [E, D] weight (one warp per expert row), and
// softmax + top-k with one four-warp CTA per token row. Semantics as in aux_kernels.cu / the reference
// (mini_llm/ops/router_decode.py:16-96): descending logit, ties -> lower id, NaN last,
// p = exp(v - max) / sum, optional division by max(selected mass, floor).
#include "common.cuh"
#include "router_device.cuh"

namespace b200q {

constexpr int RT_CHUNK = 2048;  // D positions held in registers at a time

// logits[t, e] = x[t, :] . wt[e, :] + bias[e];  wt is [E, D] row-major FP32.
// CTA = 8 warps; warp w handles expert rows (blockIdx.x*8 + w) * rpw .. +rpw-1; the TOK tokens of
// tile blockIdx.y are staged in shared memory as FP32 (vector loads: d is a multiple of 4).
template <int TOK>
__global__ void __launch_bounds__(256) router_logits_t_kernel(const void *x, int x_dtype, int t, int d, const float *wt,
                                                              const float *bias, int e, int rpw, float *logits) {
    chain_trigger();      // the next kernel of the stream may be scheduled; it waits for this grid itself
    chain_wait();         // inputs come from preceding kernels
    extern __shared__ float xs[];   // [TOK][d]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t0 = blockIdx.y * TOK;
    const int nt = min(TOK, t - t0);
    {
        const size_t esize = x_dtype == B200Q_F32 ? 4 : 2;
        const bool vec_ok = (reinterpret_cast<uintptr_t>(x) % (4 * esize)) == 0;
        const size_t base = static_cast<size_t>(t0) * d;
        for (int i = tid * 4; i < nt * d; i += 256 * 4) {
            float v[4];
            if (vec_ok) {
                if (x_dtype == B200Q_F32) {
                    const float4 q = *reinterpret_cast<const float4 *>(static_cast<const float *>(x) + base + i);
                    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
                } else {
                    const uint2 raw = *reinterpret_cast<const uint2 *>(static_cast<const uint16_t *>(x) + base + i);
                    if (x_dtype == B200Q_F16) {
                        v[0] = half_bits_to_float(raw.x & 0xffffu); v[1] = half_bits_to_float(raw.x >> 16);
                        v[2] = half_bits_to_float(raw.y & 0xffffu); v[3] = half_bits_to_float(raw.y >> 16);
                    } else {
                        v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xffff0000u);
                        v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xffff0000u);
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = load_as_float(x, x_dtype, base + i + j);
            }
            *reinterpret_cast<float4 *>(xs + i) = make_float4(v[0], v[1], v[2], v[3]);
        }
    }
    __syncthreads();
    for (int r = 0; r < rpw; ++r) {
        const int row = (blockIdx.x * 8 + warp) * rpw + r;
        if (row >= e) break;
        float acc[TOK];
#pragma unroll
        for (int i = 0; i < TOK; ++i) acc[i] = 0.f;
        for (int c0 = 0; c0 < d; c0 += RT_CHUNK) {
            float4 w[RT_CHUNK / 128];
#pragma unroll
            for (int i = 0; i < RT_CHUNK / 128; ++i) {
                const int col = c0 + i * 128 + lane * 4;
                w[i] = col < d ? *reinterpret_cast<const float4 *>(wt + static_cast<size_t>(row) * d + col)
                               : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int tt = 0; tt < TOK; ++tt) {
                if (tt < nt) {
                    float s = 0.f;
#pragma unroll
                    for (int i = 0; i < RT_CHUNK / 128; ++i) {
                        const int col = c0 + i * 128 + lane * 4;
                        if (col < d) {
                            const float4 xv = *reinterpret_cast<const float4 *>(xs + tt * d + col);
                            s = fmaf(w[i].x, xv.x, s);
                            s = fmaf(w[i].y, xv.y, s);
                            s = fmaf(w[i].z, xv.z, s);
                            s = fmaf(w[i].w, xv.w, s);
                        }
                    }
                    acc[tt] += s;
                }
            }
        }
#pragma unroll
        for (int tt = 0; tt < TOK; ++tt) {
            if (tt < nt) {
                const float s = warp_sum(acc[tt]);
                if (lane == 0) logits[static_cast<size_t>(t0 + tt) * e + row] = s + (bias ? bias[row] : 0.f);
            }
        }
    }
}

// Ordered combine, one thread per output column: the k terms are loaded first (independent
// loads), then added one by one in ascending position order with plain FP32 adds.
template <int KMAX>
__global__ void __launch_bounds__(256) moe_combine_cols_kernel(const float *terms, const int32_t *inv, int k, int d,
                                                               const float *extra, const float *extra_scale,
                                                               void *out, int out_dtype) {
    chain_trigger();      // the next kernel of the stream may be scheduled; it waits for this grid itself
    chain_wait();         // inputs come from preceding kernels
    __shared__ int pos_sorted[KMAX];
    __shared__ int pos_raw[KMAX];
    const int row = blockIdx.x, tid = threadIdx.x;
    if (tid < k) pos_raw[tid] = inv[static_cast<size_t>(row) * k + tid];
    __syncthreads();
    if (tid < k) {
        const int p = pos_raw[tid];
        int r = 0;
        for (int j = 0; j < k; ++j) r += pos_raw[j] < p;
        pos_sorted[r] = p;
    }
    __syncthreads();
    const int c = blockIdx.y * 256 + tid;
    if (c >= d) return;
    float v[KMAX];
#pragma unroll
    for (int r = 0; r < KMAX; ++r)
        if (r < k) v[r] = terms[static_cast<size_t>(pos_sorted[r]) * d + c];
    float acc = 0.f;
#pragma unroll
    for (int r = 0; r < KMAX; ++r)
        if (r < k) acc = __fadd_rn(acc, v[r]);
    if (extra) acc = __fadd_rn(acc, __fmul_rn(extra[static_cast<size_t>(row) * d + c], extra_scale ? extra_scale[row] : 1.0f));
    store_from_float(out, out_dtype, static_cast<size_t>(row) * d + c, acc);
}

// Same ordered sum for terms stored at the flat assignment index (row*k + slot): the slots of a row
// are ordered by (expert id, slot) - the order the stable sort by expert id gives them.
template <int KMAX>
__global__ void __launch_bounds__(256) moe_combine_ids_kernel(const float *terms, const void *ids, int ids_is_i64,
                                                              int k, int d, const float *extra,
                                                              const float *extra_scale, void *out, int out_dtype) {
    chain_trigger();      // the next kernel of the stream may be scheduled; it waits for this grid itself
    chain_wait();         // inputs come from preceding kernels
    __shared__ int slot_sorted[KMAX];
    __shared__ long long id_raw[KMAX];
    const int row = blockIdx.x, tid = threadIdx.x;
    if (tid < k)
        id_raw[tid] = ids_is_i64 ? static_cast<const long long *>(ids)[static_cast<size_t>(row) * k + tid]
                                 : static_cast<long long>(static_cast<const int *>(ids)[static_cast<size_t>(row) * k + tid]);
    __syncthreads();
    if (tid < k) {
        const long long mine = id_raw[tid];
        int r = 0;
        for (int j = 0; j < k; ++j) r += (id_raw[j] < mine) || (id_raw[j] == mine && j < tid);
        slot_sorted[r] = tid;
    }
    __syncthreads();
    const int c = blockIdx.y * 256 + tid;
    if (c >= d) return;
    float v[KMAX];
#pragma unroll
    for (int r = 0; r < KMAX; ++r)
        if (r < k) v[r] = terms[(static_cast<size_t>(row) * k + slot_sorted[r]) * d + c];
    float acc = 0.f;
#pragma unroll
    for (int r = 0; r < KMAX; ++r)
        if (r < k) acc = __fadd_rn(acc, v[r]);
    if (extra) acc = __fadd_rn(acc, __fmul_rn(extra[static_cast<size_t>(row) * d + c], extra_scale ? extra_scale[row] : 1.0f));
    store_from_float(out, out_dtype, static_cast<size_t>(row) * d + c, acc);
}

int launch_combine_cols(const float *terms, const int32_t *inv, int rows, int k, int d, const float *extra,
                        const float *extra_scale, void *out, int out_dtype, cudaStream_t stream) {
    dim3 grid(rows, (d + 255) / 256);
    if (k <= 16)
        launch_chained(moe_combine_cols_kernel<16>, grid, dim3(256), 0, stream, terms, inv, k, d, extra, extra_scale, out,
                       out_dtype);
    else
        launch_chained(moe_combine_cols_kernel<64>, grid, dim3(256), 0, stream, terms, inv, k, d, extra, extra_scale, out,
                       out_dtype);
    return check_launch("moe_combine");
}

// One CTA of four warps per row, n <= 1024; the arithmetic is topk_row (router_device.cuh).
__global__ void __launch_bounds__(128) router_topk_block_kernel(const float *logits, int n, int k, int renorm,
                                                                float floor_value, int extra_id,
                                                                const float *extra_weight, float *weights,
                                                                int64_t *ids, const RowPlanOut plan) {
    chain_trigger();      // the next kernel of the stream may be scheduled; it waits for this grid itself
    chain_wait();         // inputs come from preceding kernels
    topk_row(blockIdx.x, threadIdx.x, logits, n, k, renorm, floor_value, extra_id, extra_weight, weights, ids, plan);
}

int launch_topk_warp(const float *logits, int rows, int n, int k, int renorm, float floor_value, int extra_id,
                     const float *extra_weight, float *weights, int64_t *ids, const RowPlanOut &plan,
                     cudaStream_t stream) {
    launch_chained(router_topk_block_kernel, dim3(rows), dim3(128), 0, stream, logits, n, k, renorm, floor_value,
                   extra_id, extra_weight, weights, ids, plan);
    return check_launch("router_topk");
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_moe_combine_ids(const float *terms, const void *ids, int ids_is_i64, int rows, int k, int d,
                                     const float *extra, const float *extra_scale, void *out, int out_dtype,
                                     void *stream) {
    if (!terms || !ids || !out) return fail(B200Q_EINVAL, "moe_combine_ids: NULL pointer");
    if (rows <= 0 || k < 1 || k > 64 || d <= 0 || !dtype_valid(out_dtype))
        return fail(B200Q_EINVAL, "moe_combine_ids: bad argument (k <= 64)");
    dim3 grid(rows, (d + 255) / 256);
    if (k <= 16)
        launch_chained(moe_combine_ids_kernel<16>, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), terms, ids,
                       ids_is_i64, k, d, extra, extra_scale, out, out_dtype);
    else
        launch_chained(moe_combine_ids_kernel<64>, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), terms, ids,
                       ids_is_i64, k, d, extra, extra_scale, out, out_dtype);
    return check_launch("moe_combine_ids");
}

extern "C" int b200q_router_logits_t(const void *x, int x_dtype, int t, int d, const float *wt, const float *bias,
                                     int e, float *logits, void *stream) {
    if (!x || !wt || !logits) return fail(B200Q_EINVAL, "router_logits_t: NULL pointer");
    if (!dtype_valid(x_dtype)) return fail(B200Q_EINVAL, "router_logits_t: bad dtype");
    if (t <= 0 || d <= 0 || e <= 0 || d % 4) return fail(B200Q_EINVAL, "router_logits_t: bad shape (d %% 4 == 0)");
    if (reinterpret_cast<uintptr_t>(wt) & 15) return fail(B200Q_EINVAL, "router_logits_t: weight must be 16-byte aligned");
    // 8 tokens per CTA (three CTAs per SM at d = 2048) up to 128 rows, 16 beyond
    const int tok = t <= 128 ? 8 : 16;
    const size_t smem = static_cast<size_t>(tok) * d * sizeof(float);
    if (smem > 200 * 1024) return fail(B200Q_EUNSUPPORTED, "router_logits_t: d=%d too large", d);
    auto kernel = tok == 8 ? router_logits_t_kernel<8> : router_logits_t_kernel<16>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "router_logits_t: %s", cudaGetErrorString(err));
    }
    const int tiles = (t + tok - 1) / tok;
    int rpw = 4;   // fewer rows per warp when the grid would leave SMs idle
    while (rpw > 1 && static_cast<long long>((e + 8 * rpw - 1) / (8 * rpw)) * tiles < 2LL * sm_count()) rpw >>= 1;
    dim3 grid((e + 8 * rpw - 1) / (8 * rpw), tiles);
    launch_chained(kernel, grid, dim3(256), smem, static_cast<cudaStream_t>(stream), x, x_dtype, t, d, wt, bias, e, rpw,
                   logits);
    return check_launch("router_logits_t");
}
