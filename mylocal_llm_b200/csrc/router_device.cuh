// Softmax + top-k of one router row (and the routing plan of a single row) as a device function: the kernel
// of router_kernels.cu runs it for one row per CTA, the persistent one-token MoE step inside its stages.
#pragma once

#include "common.cuh"

namespace b200q {

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

// topk_row is the work of the 128 threads (tid = 0..127) that route row `row`; they meet at named barrier
// TOPK_BARRIER, so a CTA with more threads can run it on its first four warps.
constexpr int TOPK_BARRIER = 11;
constexpr int TOPK_THREADS = 128;
__device__ __forceinline__ void topk_sync() { named_barrier_sync(TOPK_BARRIER, TOPK_THREADS); }

__device__ __forceinline__ void topk_row(const int row, const int tid, const float *logits, int n, int k, int renorm,
                                         float floor_value, int extra_id, const float *extra_weight, float *weights,
                                         int64_t *ids, const RowPlanOut &plan) {
    __shared__ unsigned long long warp_best[2][4];
    __shared__ float red[4];
    __shared__ float sel_p[32];
    __shared__ int sel_i[32];
    const int lane = tid & 31, warp = tid >> 5;
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
    topk_sync();
    mx = red[0];
#pragma unroll
    for (int w = 1; w < 4; ++w) mx = (isnan(mx) || isnan(red[w])) ? qnan : fmaxf(mx, red[w]);
    topk_sync();
    float den = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (i * 128 + tid < n) den += expf(v[i] - mx);
    den = warp_sum(den);
    if (lane == 0) red[warp] = den;
    topk_sync();
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
        topk_sync();
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
    topk_sync();
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

// topk_row for one warp: the same results bit for bit, without a barrier - for a caller whose step is a chain
// of dependent latencies (the persistent one-token MoE step). Lane L plays threads L, L + 32, L + 64, L + 96
// of topk_row ("virtual warps" w = 0..3): every partial sum is formed over the same values in the same order
// and reduced by the same butterfly; maxima and the selection are order-independent (keys are unique). A lane
// keeps its NE = n / 32 (rounded up to 16 or 32) keys in registers; a selection round is a tree of 32-bit maxima
// over them (carrying the entry's position), a warp-wide maximum, a warp-wide minimum of the index among the equal
// keys and one cleared bit, and the k probabilities are computed together after the last round. Writes weights / ids (k + 1 entries with the appended id) and the one-row plan's order,
// inv, segment arrays and num_segments; counts / offsets only when given. n <= 32 NE, k <= 31, extra_id >= 0.
template <int NE>
__device__ __forceinline__ void topk_plan_warp(const int lane, const float *logits, int n, int k, int renorm,
                                               float floor_value, int extra_id, float extra_weight, float *weights,
                                               int64_t *ids, const RowPlanOut &plan) {
    static_assert(NE == 16 || NE == 32, "16 or 32 keys per lane");
    const float neg_inf = __int_as_float(0xff800000), qnan = __int_as_float(0x7fc00000);
    uint32_t hi[NE];           // entry t of the lane: index lane + 32 t = i * 128 + 32 w + lane with t = 4 i + w
    uint32_t alive = 0u;       // bit t: inside the row and not yet selected
    {
        float v[NE];
#pragma unroll
        for (int t = 0; t < NE; ++t) v[t] = (lane + 32 * t < n) ? logits[lane + 32 * t] : neg_inf;
#pragma unroll
        for (int t = 0; t < NE; ++t) {
            const bool in = lane + 32 * t < n;
            hi[t] = in ? orderable_bits(v[t]) : 0u;
            alive |= in ? (1u << t) : 0u;
        }
    }
    // (orderable_bits folds -0 into +0 and all NaNs into one: neither changes max or exp(v - max))
    float mx = neg_inf;
#pragma unroll
    for (int t = 0; t < NE; ++t)
        if (lane + 32 * t < n) {
            const float v = from_orderable_bits(hi[t]);
            mx = (isnan(v) || isnan(mx)) ? qnan : fmaxf(mx, v);
        }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, mx, o);
        mx = (isnan(mx) || isnan(other)) ? qnan : fmaxf(mx, other);
    }
    // the four virtual warps' partial sums, each over its values in ascending order, reduced by four butterflies
    // that advance together
    float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < NE / 4; ++i)
#pragma unroll
        for (int w = 0; w < 4; ++w)
            if (i * 128 + 32 * w + lane < n) part[w] += expf(from_orderable_bits(hi[4 * i + w]) - mx);
#pragma unroll
    for (int o = 16; o; o >>= 1)
#pragma unroll
        for (int w = 0; w < 4; ++w) part[w] += __shfl_xor_sync(0xffffffffu, part[w], o);
    const float den = ((part[0] + part[1]) + part[2]) + part[3];

    // Selection keys: monotonic float bits + 1, so that 0 can stand for "taken / outside the row" (a NaN's key is
    // 1, the largest key is +inf's 0xFF800001: no wrap). Within a lane a lower entry is a lower index, so a
    // strict "greater" keeps the lower index on ties; across lanes the smallest index among the equal keys wins.
    uint32_t h1[NE];
#pragma unroll
    for (int t = 0; t < NE; ++t) h1[t] = hi[t] + 1u;
    uint32_t my_h = 0u;        // lane s keeps slot s
    int my_i = 0;
#pragma unroll 1
    for (int slot = 0; slot < k; ++slot) {
        uint32_t val[NE], pos[NE];
#pragma unroll
        for (int t = 0; t < NE; ++t) {
            val[t] = ((alive >> t) & 1u) ? h1[t] : 0u;
            pos[t] = t;
        }
#pragma unroll
        for (int span = NE / 2; span >= 1; span >>= 1)
#pragma unroll
            for (int t = 0; t < span; ++t) {
                const bool take = val[t + span] > val[t];
                pos[t] = take ? pos[t + span] : pos[t];
                val[t] = max(val[t], val[t + span]);
            }
        const uint32_t wv = __reduce_max_sync(0xffffffffu, val[0]);
        const uint32_t idx = static_cast<uint32_t>(lane) + 32u * pos[0];
        const uint32_t bi_u = __reduce_min_sync(0xffffffffu, (val[0] == wv && wv != 0u) ? idx : 0xffffffffu);
        const int bi = static_cast<int>(bi_u);                    // -1 when nothing is left, as in topk_row
        if (bi >= 0 && (bi & 31) == lane) alive &= ~(1u << ((bi >> 5) & 31));
        if (lane == slot) { my_h = wv - 1u; my_i = bi; }
    }
    const float my_p = __fdiv_rn(expf(from_orderable_bits(my_h) - mx), den);
    const int k_out = k + 1;
    float norm = 1.0f;
    if (renorm) {
        float mass = 0.f;
        for (int s = 0; s < k; ++s) mass = __fadd_rn(mass, __shfl_sync(0xffffffffu, my_p, s));
        norm = isnan(mass) ? mass : fmaxf(mass, floor_value);
    }
    if (lane == k) my_i = extra_id;
    const float my_w = lane < k ? (renorm ? __fdiv_rn(my_p, norm) : my_p) : extra_weight;
    // position of an assignment = number of smaller ids; one segment of one row per selected expert, ascending
    int pos = 0;
    for (int j = 0; j < k_out; ++j) pos += (__shfl_sync(0xffffffffu, my_i, j) < my_i) ? 1 : 0;
    if (lane < k_out) {
        weights[lane] = my_w;
        ids[lane] = my_i;
        plan.order[pos] = lane;
        plan.inv[lane] = pos;
        if (pos < plan.max_segments) {
            plan.seg_expert[pos] = my_i;
            plan.seg_begin[pos] = pos;
            plan.seg_count[pos] = 1;
        }
    }
    if (plan.counts != nullptr && plan.offsets != nullptr) {
        for (int ex = lane; ex <= plan.e; ex += 32) {
            int below = 0, hit = 0;
            for (int j = 0; j < k_out; ++j) {
                const int id = __shfl_sync(0xffffffffu, my_i, j);
                below += id < ex;
                hit += id == ex;
            }
            plan.offsets[ex] = below;
            if (ex < plan.e) plan.counts[ex] = hit;
        }
    }
    if (lane == 0) {
        plan.num_segments[0] = min(k_out, plan.max_segments);
        plan.status[0] = k_out > plan.max_segments ? 2 : 0;
    }
}

}  // namespace b200q
