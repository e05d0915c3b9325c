// Decode-oriented router kernels: logits from an [E, D] weight (one warp per expert row), and
// softmax + top-k with one four-warp CTA per token row. Semantics as in aux_kernels.cu / the reference
// (mini_llm/ops/router_decode.py:16-96): descending logit, ties -> lower id, NaN last,
// p = exp(v - max) / sum, optional division by max(selected mass, floor).
#include "common.cuh"

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

// One CTA of four warps per row, n <= 1024 (eight values per thread, value idx = i*128 + tid).
// Every value becomes a 64-bit key that orders like the selection rule: high word = the float's
// bits made monotonic (NaN -> 0, below -inf; -0 counted as +0), low word = ~index, so the largest
// key is the largest logit and, among equals, the lowest index. A round is then two warp-wide
// integer maximum reductions plus one exchange between the four warps.
__device__ __forceinline__ uint32_t orderable_bits(float v) {
    if (isnan(v)) return 0u;
    const uint32_t b = __float_as_uint(v + 0.0f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float from_orderable_bits(uint32_t h) {
    if (h == 0u) return __int_as_float(0x7fc00000);
    return __uint_as_float((h & 0x80000000u) ? (h & 0x7fffffffu) : ~h);
}

__global__ void __launch_bounds__(128) router_topk_block_kernel(const float *logits, int n, int k, int renorm,
                                                                float floor_value, int extra_id,
                                                                const float *extra_weight, float *weights,
                                                                int64_t *ids, const RowPlanOut plan) {
    chain_trigger();      // the next kernel of the stream may be scheduled; it waits for this grid itself
    chain_wait();         // inputs come from preceding kernels
    __shared__ unsigned long long warp_best[2][4];
    __shared__ float red[4];
    __shared__ float sel_p[32];
    __shared__ int sel_i[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.x;
    const float neg_inf = __int_as_float(0xff800000), qnan = __int_as_float(0x7fc00000);
    const float *src = logits + static_cast<size_t>(row) * n;
    float v[8];
    uint32_t hi[8];
    float mx = neg_inf;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int idx = i * 128 + tid;
        v[i] = idx < n ? src[idx] : neg_inf;
        hi[i] = idx < n ? orderable_bits(v[i]) : 0u;
        if (idx < n) mx = (isnan(v[i]) || isnan(mx)) ? qnan : fmaxf(mx, v[i]);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, mx, o);
        mx = (isnan(mx) || isnan(other)) ? qnan : fmaxf(mx, other);
    }
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < 4; ++w) mx = (isnan(mx) || isnan(red[w])) ? qnan : fmaxf(mx, red[w]);
    __syncthreads();
    float den = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (i * 128 + tid < n) den += expf(v[i] - mx);
    den = warp_sum(den);
    if (lane == 0) red[warp] = den;
    __syncthreads();
    den = ((red[0] + red[1]) + red[2]) + red[3];

    for (int slot = 0; slot < k; ++slot) {
        // best key of this thread among its values that are inside the row and not yet taken
        uint32_t bh = 0u, bl = 0u;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t lo = ~static_cast<uint32_t>(i * 128 + tid);
            const bool take = (i * 128 + tid < n) && (hi[i] > bh || (hi[i] == bh && lo > bl)) && hi[i] != 0xffffffffu;
            if (take) { bh = hi[i]; bl = lo; }
        }
        const uint32_t wh = __reduce_max_sync(0xffffffffu, bh);
        const uint32_t wl = __reduce_max_sync(0xffffffffu, bh == wh ? bl : 0u);
        if (lane == 0) warp_best[slot & 1][warp] = (static_cast<unsigned long long>(wh) << 32) | wl;
        __syncthreads();
        unsigned long long best = warp_best[slot & 1][0];
#pragma unroll
        for (int w = 1; w < 4; ++w) best = max(best, warp_best[slot & 1][w]);
        const int bi = static_cast<int>(~static_cast<uint32_t>(best));
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i * 128 + tid == bi) hi[i] = 0xffffffffu;          // marks "taken" (never a real key)
        if (tid == 0) {
            sel_p[slot] = __fdiv_rn(expf(from_orderable_bits(static_cast<uint32_t>(best >> 32)) - mx), den);
            sel_i[slot] = bi;
        }
    }
    __syncthreads();
    const int k_out = k + (extra_id >= 0 ? 1 : 0);
    float norm = 1.0f;
    if (renorm) {
        float mass = 0.f;
        for (int s = 0; s < k; ++s) mass = __fadd_rn(mass, sel_p[s]);      // slot order, same on every thread
        norm = isnan(mass) ? mass : fmaxf(mass, floor_value);
    }
    if (tid < k) {
        weights[static_cast<size_t>(row) * k_out + tid] = renorm ? __fdiv_rn(sel_p[tid], norm) : sel_p[tid];
        ids[static_cast<size_t>(row) * k_out + tid] = sel_i[tid];
    }
    if (extra_id >= 0 && tid == 0) {
        ids[static_cast<size_t>(row) * k_out + k] = extra_id;
        weights[static_cast<size_t>(row) * k_out + k] = extra_weight ? extra_weight[row] : 1.0f;
    }
    if (plan.order != nullptr) {
        // Single row (grid of one CTA): the routing plan of its k_out distinct ids. Position of an
        // assignment = number of smaller ids; one segment of one row per selected expert, ascending.
        auto id_of = [&](int j) { return j < k ? sel_i[j] : extra_id; };
        if (tid < k_out) {
            const int mine = id_of(tid);
            int pos = 0;
            for (int j = 0; j < k_out; ++j) pos += id_of(j) < mine;
            plan.order[pos] = tid;
            plan.inv[tid] = pos;
            if (pos < plan.max_segments) {
                plan.seg_expert[pos] = mine;
                plan.seg_begin[pos] = pos;
                plan.seg_count[pos] = 1;
            }
        }
        for (int ex = tid; ex <= plan.e; ex += 128) {
            int below = 0, hit = 0;
            for (int j = 0; j < k_out; ++j) {
                below += id_of(j) < ex;
                hit += id_of(j) == ex;
            }
            plan.offsets[ex] = below;
            if (ex < plan.e) plan.counts[ex] = hit;
        }
        if (tid == 0) {
            plan.num_segments[0] = min(k_out, plan.max_segments);
            plan.status[0] = k_out > plan.max_segments ? 2 : 0;
        }
    }
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
