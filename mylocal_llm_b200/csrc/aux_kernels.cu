// Small kernels around the streaming GEMV: dequantise, RMSNorm, router, routing plan, combine.
#include "common.cuh"
#include "norm_device.cuh"

namespace b200q {

// ------------------------------------------------------------------------------- dequantize
// One thread per weight; evaluates the reference's formula with the same roundings
// (mini_llm/ops/quantized_weight.py:208-250): every product below is exact in FP32, the single
// rounding is the final subtraction of Q4_K/Q5_K.
__device__ __forceinline__ float decode_one(const uint8_t *blk, int fmt, int e) {
    if (fmt == B200Q_Q8_0) {
        const float d = half_bits_to_float(blk[0] | (blk[1] << 8));
        return __fmul_rn(d, static_cast<float>(static_cast<int>(static_cast<int8_t>(blk[2 + e]))));
    }
    if (fmt == B200Q_Q4_0) {        // 16 code bytes: low nibbles = values 0..15, high nibbles = 16..31; q - 8
        const float d = half_bits_to_float(blk[0] | (blk[1] << 8));
        const int q = ((blk[2 + (e & 15)] >> (4 * (e >> 4))) & 15) - 8;
        return __fmul_rn(d, static_cast<float>(q));
    }
    if (fmt == B200Q_Q3_K) {
        // hmask[32] | qs[64] | 12 scale bytes | d: two low bits from qs, minus 4 unless the mask bit is set,
        // sixteen 6-bit scales minus 32 (mini_llm/ops/quantized_weight.py:251-265)
        const float d = half_bits_to_float(blk[108] | (blk[109] << 8));
        const int j = e & 31, low = (blk[32 + 32 * (e >> 7) + j] >> (2 * ((e >> 5) & 3))) & 3;
        const int high = (blk[j] >> (e >> 5)) & 1;
        const int s = e >> 4;
        const int sc = (((blk[96 + (s & 7)] >> (4 * (s >> 3))) & 15) | (((blk[104 + (s & 3)] >> (2 * (s >> 2))) & 3) << 4)) - 32;
        const float scale = __fmul_rn(d, static_cast<float>(sc));
        return __fmul_rn(scale, static_cast<float>(low - ((high ^ 1) << 2)));
    }
    if (fmt == B200Q_Q4_K || fmt == B200Q_Q5_K) {
        const float d = half_bits_to_float(blk[0] | (blk[1] << 8));
        const float dmin = half_bits_to_float(blk[2] | (blk[3] << 8));
        const uint8_t *m = blk + 4;
        const int g = e >> 5, j = e & 31;
        int sc, mn;
        if (g < 4) {
            sc = m[g] & 63;
            mn = m[4 + g] & 63;
        } else {
            sc = (m[4 + g] & 15) | ((m[g - 4] >> 2) & 48);
            mn = (m[4 + g] >> 4) | ((m[g] >> 2) & 48);
        }
        const uint8_t *qs = blk + (fmt == B200Q_Q5_K ? 48 : 16);
        int q = (qs[32 * (g >> 1) + j] >> (4 * (g & 1))) & 15;
        if (fmt == B200Q_Q5_K) q |= ((blk[16 + j] >> g) & 1) << 4;
        const float scale = __fmul_rn(d, static_cast<float>(sc));
        const float minimum = __fmul_rn(dmin, static_cast<float>(mn));
        return __fsub_rn(__fmul_rn(scale, static_cast<float>(q)), minimum);
    }
    // Q6_K
    const float d = half_bits_to_float(blk[208] | (blk[209] << 8));
    const int half = e >> 7, r = e & 127;
    const int lo = (blk[64 * half + (r & 63)] >> (4 * (r >> 6))) & 15;
    const int hi = (blk[128 + 32 * half + (r & 31)] >> (2 * (r >> 5))) & 3;
    const int q = (lo | (hi << 4)) - 32;
    const float scale = __fmul_rn(d, static_cast<float>(static_cast<int>(static_cast<int8_t>(blk[192 + (e >> 4)]))));
    return __fmul_rn(scale, static_cast<float>(q));
}

__global__ void dequantize_kernel(const uint8_t *w, int fmt, long long total, float *out) {
    const int qk = fmt_elems(fmt), qb = fmt_bytes(fmt);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long b = i / qk;
        out[i] = decode_one(w + b * qb, fmt, static_cast<int>(i - b * qk));
    }
}

// ---------------------------------------------------------------------------------- RMSNorm
// One 256-thread CTA per row; the arithmetic is rmsnorm_row / combine_norm_row (norm_device.cuh).
template <bool RESIDUAL>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const void *x, int x_dtype, const float *residual,
                                                      float alpha, const void *gamma, int gamma_dtype, int d,
                                                      float eps, float *res_out, void *y, int y_dtype) {
    chain_trigger();      // the next kernel of the stream may be scheduled; it waits for this grid itself
    chain_wait();         // inputs come from preceding kernels
    rmsnorm_row<RESIDUAL>(blockIdx.x, threadIdx.x, x, x_dtype, residual, alpha, gamma, gamma_dtype, d, eps, res_out, y,
                          y_dtype);
}

template <int KMAX>
__global__ void __launch_bounds__(256) moe_combine_norm_kernel(const float *terms, const int32_t *inv, int k, int d,
                                                               const float *extra, const float *extra_scale,
                                                               int branch_dtype, const float *residual, float alpha,
                                                               const void *gamma, int gamma_dtype, float eps,
                                                               float *res_out, void *y, int y_dtype) {
    chain_trigger();      // the next kernel of the stream may be scheduled; it waits for this grid itself
    chain_wait();         // inputs come from preceding kernels
    combine_norm_row<KMAX>(blockIdx.x, threadIdx.x, terms, inv, k, d, extra, extra_scale, branch_dtype, residual, alpha,
                           gamma, gamma_dtype, eps, res_out, y, y_dtype);
}

// ---------------------------------------------------------------------------- router logits
// logits[t,e] = sum_d x[t,d]*W[d,e] + bias[e]. CTA = 8 warps x 32 columns x up to 8 tokens; the
// warps split d, partial sums are combined in ascending warp order (deterministic).
constexpr int RL_TOK = 8;
__global__ void __launch_bounds__(256) router_logits_kernel(const void *x, int x_dtype, int t, int d,
                                                            const float *w, const float *bias, int e,
                                                            float *logits) {
    extern __shared__ float rl_smem[];  // x tile [tok][d] then partial [8][RL_TOK][32]
    float *xs = rl_smem;
    float *part = rl_smem + RL_TOK * d;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int col = blockIdx.x * 32 + lane;
    const int t0 = blockIdx.y * RL_TOK;
    const int nt = min(RL_TOK, t - t0);
    for (int i = tid; i < nt * d; i += 256) xs[i] = load_as_float(x, x_dtype, static_cast<size_t>(t0) * d + i);
    __syncthreads();
    float acc[RL_TOK];
#pragma unroll
    for (int i = 0; i < RL_TOK; ++i) acc[i] = 0.f;
    const int chunk = (d + 7) / 8;
    const int d0 = warp * chunk, d1 = min(d, d0 + chunk);
    if (col < e) {
        for (int dd = d0; dd < d1; ++dd) {
            const float wv = w[static_cast<size_t>(dd) * e + col];
#pragma unroll
            for (int i = 0; i < RL_TOK; ++i)
                if (i < nt) acc[i] = fmaf(xs[i * d + dd], wv, acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < RL_TOK; ++i) part[(warp * RL_TOK + i) * 32 + lane] = acc[i];
    __syncthreads();
    for (int o = tid; o < nt * 32; o += 256) {
        const int i = o >> 5, l = o & 31;
        const int c = blockIdx.x * 32 + l;
        if (c >= e) continue;
        float s = 0.f;
        for (int wv = 0; wv < 8; ++wv) s += part[(wv * RL_TOK + i) * 32 + l];
        if (bias) s += bias[c];
        logits[static_cast<size_t>(t0 + i) * e + c] = s;
    }
}

// --------------------------------------------------------------------------- shared gate
// scale[t] = sigmoid(x[t] . g): one warp per token (mini_llm/external/qwen3next_moe.py:145-146).
__global__ void __launch_bounds__(256) shared_gate_kernel(const void *x, int x_dtype, int t, int d,
                                                          const float *g, float *scale) {
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= t) return;
    float s = 0.f;
    for (int c = lane; c < d; c += 32) s = fmaf(load_as_float(x, x_dtype, static_cast<size_t>(row) * d + c), g[c], s);
    s = warp_sum(s);
    if (lane == 0) scale[row] = s >= 0.f ? 1.0f / (1.0f + expf(-s)) : expf(s) / (1.0f + expf(s));
}

// ------------------------------------------------------------------------------ router top-k
// One 128-thread CTA per row. Ordering: larger logit first, NaN last, equal -> lower id
// (mini_llm/ops/router_decode.py:18-25). No FMA contraction is possible in this kernel's
// arithmetic (only subtract, exp, add, divide).
__device__ __forceinline__ bool route_better(float a, int ia, float b, int ib, int n) {
    if (ia == n) return false;
    if (ib == n) return true;
    if (isnan(a)) return isnan(b) && ia < ib;
    if (isnan(b)) return true;
    return a > b || (a == b && ia < ib);
}

__global__ void __launch_bounds__(128) router_topk_kernel(const float *logits, int n, int k, int renorm,
                                                          float floor_value, float *weights, int64_t *ids) {
    __shared__ float values[4096];
    __shared__ unsigned char used[4096];
    __shared__ float red_v[4];
    __shared__ int red_i[4];
    __shared__ float selected[32];
    __shared__ float stat[2];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *row = logits + static_cast<size_t>(blockIdx.x) * n;
    const float neg_inf = __int_as_float(0xff800000);
    const float qnan = __int_as_float(0x7fc00000);

    float mx = neg_inf;
    for (int i = tid; i < n; i += 128) {
        const float v = row[i];
        values[i] = v;
        used[i] = 0;
        mx = (isnan(v) || isnan(mx)) ? qnan : fmaxf(mx, v);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, mx, o);
        mx = (isnan(mx) || isnan(other)) ? qnan : fmaxf(mx, other);
    }
    if (lane == 0) red_v[warp] = mx;
    __syncthreads();
    if (tid == 0) {
        float m = red_v[0];
        for (int w = 1; w < 4; ++w) m = (isnan(m) || isnan(red_v[w])) ? qnan : fmaxf(m, red_v[w]);
        stat[0] = m;
    }
    __syncthreads();
    mx = stat[0];
    float den = 0.f;
    for (int i = tid; i < n; i += 128) den += expf(values[i] - mx);
    den = warp_sum(den);
    __syncthreads();
    if (lane == 0) red_v[warp] = den;
    __syncthreads();
    if (tid == 0) stat[1] = (red_v[0] + red_v[1]) + (red_v[2] + red_v[3]);
    __syncthreads();
    den = stat[1];

    for (int slot = 0; slot < k; ++slot) {
        float best = neg_inf;
        int idx = n;
        for (int i = tid; i < n; i += 128)
            if (!used[i] && route_better(values[i], i, best, idx, n)) { best = values[i]; idx = i; }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (route_better(ov, oi, best, idx, n)) { best = ov; idx = oi; }
        }
        if (lane == 0) { red_v[warp] = best; red_i[warp] = idx; }
        __syncthreads();
        if (tid == 0) {
            float bv = red_v[0];
            int bi = red_i[0];
            for (int w = 1; w < 4; ++w)
                if (route_better(red_v[w], red_i[w], bv, bi, n)) { bv = red_v[w]; bi = red_i[w]; }
            ids[static_cast<size_t>(blockIdx.x) * k + slot] = bi;
            used[bi] = 1;
            selected[slot] = __fdiv_rn(expf(values[bi] - mx), den);
        }
        __syncthreads();
    }
    if (tid == 0) {
        float norm = 1.0f;
        if (renorm) {
            float mass = 0.f;
            for (int s = 0; s < k; ++s) mass = __fadd_rn(mass, selected[s]);
            norm = isnan(mass) ? mass : fmaxf(mass, floor_value);
        }
        for (int s = 0; s < k; ++s)
            weights[static_cast<size_t>(blockIdx.x) * k + s] = renorm ? __fdiv_rn(selected[s], norm) : selected[s];
    }
}

// ------------------------------------------------------------------------------ routing plan
// Single CTA, 1024 threads: stable counting sort of the assignments by expert id, then the
// compacted list of active experts split into runs of at most seg_cap assignments.
constexpr int PLAN_THREADS = 1024;
constexpr int PLAN_MAX_EXPERTS = 4096;

// Optional id translation for an expert-parallel rank: global ids first..first+n_local-1 become
// 0..n_local-1; the shared-expert id becomes n_local for the rows this rank is home of; every other
// assignment becomes n_local+1, which the caller passes as skip_expert.
struct PlanIdMap {
    int enabled, k, first, n_local, shared_id, home_lo, home_hi, e_global;
};

// Exclusive scan of one value per thread over the CTA (PLAN_THREADS threads); *total gets the sum.
__device__ __forceinline__ int plan_block_scan(int v, int *warp_tot, int *total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = warp_tot[lane];
        int winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        warp_tot[lane] = winc - w;              // exclusive prefix of the warp totals
        if (lane == 31) *total = winc;
    }
    __syncthreads();
    const int out = warp_tot[warp] + inc - v;
    __syncthreads();                            // warp_tot may be reused right away
    return out;
}

// words > 0: `bits` (dynamic shared memory) holds one bit per (expert, row); an assignment's rank
// inside its expert is then a population count over the rows before it - no serial pass. This needs
// every row to name an expert at most once (top-k output does); a row that repeats an expert sets
// `dup` and the kernel falls back to the ordered pass. Assignments of skip_expert are never run
// and only need distinct positions.
__global__ void __launch_bounds__(PLAN_THREADS) moe_plan_kernel(const void *ids, int ids_is_i64, int total, int k,
                                                                int e, int skip_expert, const PlanIdMap map,
                                                                int words, int seg_cap, int32_t *counts,
                                                                int32_t *offsets, int32_t *order, int32_t *inv,
                                                                int32_t *seg_expert, int32_t *seg_begin,
                                                                int32_t *seg_count, int32_t *num_segments,
                                                                int max_segments, int32_t *status) {
    chain_trigger();      // the next kernel of the stream may be scheduled; it waits for this grid itself
    chain_wait();         // inputs come from preceding kernels
    extern __shared__ unsigned int bits[];    // [e][words]
    __shared__ int cnt[PLAN_MAX_EXPERTS];     // counts, then running cursor
    __shared__ int off[PLAN_MAX_EXPERTS + 1];
    __shared__ int warp_tot[32];
    __shared__ int carry, scan_total, skip_cursor;
    __shared__ int bad, dup;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    for (int i = tid; i < e; i += PLAN_THREADS) cnt[i] = 0;
    for (int i = tid; i < e * words; i += PLAN_THREADS) bits[i] = 0u;
    if (tid == 0) { bad = 0; dup = 0; carry = 0; skip_cursor = 0; }
    __syncthreads();

    auto load_id = [&](int i) -> int {
        long long v = ids_is_i64 ? static_cast<const long long *>(ids)[i]
                                 : static_cast<long long>(static_cast<const int *>(ids)[i]);
        if (map.enabled) {
            // v == e_global: a padding entry (a rank that brought fewer rows than its slot) - nobody runs it
            if (v < 0 || v > map.e_global) { bad = 1; v = map.first; }
            const int row = i / map.k;
            if (v == map.e_global) v = map.n_local + 1;
            else if (v >= map.first && v < map.first + map.n_local) v -= map.first;
            else if (v == map.shared_id && row >= map.home_lo && row < map.home_hi) v = map.n_local;
            else v = map.n_local + 1;
        } else if (v < 0 || v >= e) { bad = 1; v = 0; }
        return static_cast<int>(v);
    };

    for (int i = tid; i < total; i += PLAN_THREADS) {
        const int ex = load_id(i);
        atomicAdd(&cnt[ex], 1);
        if (words && ex != skip_expert) {
            const int row = i / k;
            const unsigned int bit = 1u << (row & 31);
            if (atomicOr(&bits[ex * words + (row >> 5)], bit) & bit) dup = 1;
        }
    }
    __syncthreads();

    // exclusive scan of counts over experts, 1024 at a time
    for (int base = 0; base < e; base += PLAN_THREADS) {
        const int i = base + tid;
        const int c = i < e ? cnt[i] : 0;
        const int ex_prefix = plan_block_scan(c, warp_tot, &scan_total);
        if (i < e) off[i] = carry + ex_prefix;
        __syncthreads();
        if (tid == 0) carry += scan_total;
        __syncthreads();
    }
    if (tid == 0) off[e] = carry;
    __syncthreads();
    for (int i = tid; i < e; i += PLAN_THREADS) {
        counts[i] = cnt[i];
        offsets[i] = off[i];
    }
    if (tid == 0) offsets[e] = off[e];
    __syncthreads();

    if (words && !dup) {
        for (int i = tid; i < total; i += PLAN_THREADS) {
            const int ex = load_id(i);
            int pos;
            if (ex == skip_expert) {
                pos = off[ex] + atomicAdd(&skip_cursor, 1);
            } else {
                const int row = i / k;
                const unsigned int *w = bits + ex * words;
                int rank = __popc(w[row >> 5] & ((1u << (row & 31)) - 1u));
                for (int q = 0; q < (row >> 5); ++q) rank += __popc(w[q]);
                pos = off[ex] + rank;
            }
            order[pos] = i;
            inv[i] = pos;
        }
    } else {
        for (int i = tid; i < e; i += PLAN_THREADS) cnt[i] = off[i];  // running cursor
        __syncthreads();
        // stable placement: chunks of 1024 assignments in order, warps of a chunk in order
        for (int base = 0; base < total; base += PLAN_THREADS) {
            const int i = base + tid;
            const bool valid = i < total;
            const int ex = valid ? load_id(i) : -1;
            const unsigned same = __match_any_sync(0xffffffffu, ex);
            const int rank = __popc(same & ((1u << lane) - 1u));
            const int leader = __ffs(same) - 1;
            const int nwarps = (min(total - base, PLAN_THREADS) + 31) >> 5;
            int pos = 0;
            for (int w = 0; w < nwarps; ++w) {
                if (warp == w && valid) {
                    int start = 0;
                    if (lane == leader) {
                        start = cnt[ex];
                        cnt[ex] = start + __popc(same);
                    }
                    start = __shfl_sync(same, start, leader);
                    pos = start + rank;
                }
                __syncthreads();
            }
            if (valid) {
                order[pos] = i;
                inv[i] = pos;
            }
        }
    }
    __syncthreads();

    // active-expert segments, ascending id, runs of at most seg_cap
    if (tid == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < e; base += PLAN_THREADS) {
        const int i = base + tid;
        const int c = (i < e && i != skip_expert) ? (off[i + 1] - off[i]) : 0;   // skipped expert: no segments
        const int nsegs = (c + seg_cap - 1) / seg_cap;
        const int s0 = carry + plan_block_scan(nsegs, warp_tot, &scan_total);
        for (int r = 0; r < nsegs; ++r) {
            if (s0 + r < max_segments) {
                seg_expert[s0 + r] = i;
                seg_begin[s0 + r] = off[i] + r * seg_cap;
                seg_count[s0 + r] = min(seg_cap, c - r * seg_cap);
            }
        }
        __syncthreads();
        if (tid == 0) carry += scan_total;
        __syncthreads();
    }
    if (tid == 0) {
        num_segments[0] = min(carry, max_segments);
        status[0] = bad ? 1 : (carry > max_segments ? 2 : 0);
    }
}

// ----------------------------------------------------------------------------------- combine
// One CTA per token row: sort the row's k sorted-positions ascending (= ascending expert id) and
// add the per-assignment terms one by one with plain FP32 adds
// (mini_llm/ops/grouped_quantized_experts.py:70-79).
__global__ void __launch_bounds__(256) moe_combine_kernel(const float *terms, const int32_t *inv, int k, int d,
                                                          const float *extra, const float *extra_scale, void *out,
                                                          int out_dtype) {
    __shared__ int pos_sorted[64];
    __shared__ int pos_raw[64];
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
    const float sc = extra_scale ? extra_scale[row] : 1.0f;
    for (int c = tid; c < d; c += 256) {
        float acc = 0.f;
        for (int r = 0; r < k; ++r) acc = __fadd_rn(acc, terms[static_cast<size_t>(pos_sorted[r]) * d + c]);
        if (extra) acc = __fadd_rn(acc, __fmul_rn(extra[static_cast<size_t>(row) * d + c], sc));
        store_from_float(out, out_dtype, static_cast<size_t>(row) * d + c, acc);
    }
}

int launch_combine_cols(const float *terms, const int32_t *inv, int rows, int k, int d, const float *extra,
                        const float *extra_scale, void *out, int out_dtype, cudaStream_t stream);
int launch_topk_warp(const float *logits, int rows, int n, int k, int renorm, float floor_value, int extra_id,
                     const float *extra_weight, float *weights, int64_t *ids, const RowPlanOut &plan,
                     cudaStream_t stream);

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_dequantize(const void *w, int fmt, int64_t n, int k, float *out, void *stream) {
    if (!w || !out) return fail(B200Q_EINVAL, "dequantize: NULL pointer");
    if (!fmt_valid(fmt)) return fail(B200Q_EINVAL, "dequantize: unknown format %d", fmt);
    if (n <= 0 || k <= 0 || k % fmt_elems(fmt)) return fail(B200Q_EINVAL, "dequantize: bad shape");
    const long long total = static_cast<long long>(n) * k;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    dequantize_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t *>(w), fmt, total, out);
    return check_launch("dequantize");
}

int b200q_rmsnorm(const void *x, int x_dtype, const void *gamma, int gamma_dtype, int rows, int d, float eps,
                  void *y, int y_dtype, void *stream) {
    if (!x || !gamma || !y) return fail(B200Q_EINVAL, "rmsnorm: NULL pointer");
    if (!dtype_valid(x_dtype) || !dtype_valid(gamma_dtype) || !dtype_valid(y_dtype))
        return fail(B200Q_EINVAL, "rmsnorm: bad dtype");
    if (rows <= 0 || d <= 0) return fail(B200Q_EINVAL, "rmsnorm: bad shape");
    launch_chained(rmsnorm_kernel<false>, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), x, x_dtype,
                   nullptr, 0.f, gamma, gamma_dtype, d, eps, nullptr, y, y_dtype);
    return check_launch("rmsnorm");
}

int b200q_residual_rmsnorm(const float *residual, const void *branch, int branch_dtype, float alpha,
                           const void *gamma, int gamma_dtype, int rows, int d, float eps, float *res_out,
                           void *y, int y_dtype, void *stream) {
    if (!residual || !branch || !gamma || !res_out || !y) return fail(B200Q_EINVAL, "residual_rmsnorm: NULL pointer");
    if (!dtype_valid(branch_dtype) || !dtype_valid(gamma_dtype) || !dtype_valid(y_dtype))
        return fail(B200Q_EINVAL, "residual_rmsnorm: bad dtype");
    if (rows <= 0 || d <= 0) return fail(B200Q_EINVAL, "residual_rmsnorm: bad shape");
    launch_chained(rmsnorm_kernel<true>, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), branch,
                   branch_dtype, residual, alpha, gamma, gamma_dtype, d, eps, res_out, y, y_dtype);
    return check_launch("residual_rmsnorm");
}

int b200q_router_logits(const void *x, int x_dtype, int t, int d, const float *wr, const float *bias, int e,
                        float *logits, void *stream) {
    if (!x || !wr || !logits) return fail(B200Q_EINVAL, "router_logits: NULL pointer");
    if (!dtype_valid(x_dtype)) return fail(B200Q_EINVAL, "router_logits: bad dtype");
    if (t <= 0 || d <= 0 || e <= 0) return fail(B200Q_EINVAL, "router_logits: bad shape");
    const size_t smem = (static_cast<size_t>(RL_TOK) * d + 8 * RL_TOK * 32) * sizeof(float);
    if (smem > 200 * 1024) return fail(B200Q_EUNSUPPORTED, "router_logits: d=%d too large", d);
    cudaError_t err = cudaFuncSetAttribute(router_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           200 * 1024);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "router_logits: %s", cudaGetErrorString(err));
    }
    dim3 grid((e + 31) / 32, (t + RL_TOK - 1) / RL_TOK);
    router_logits_kernel<<<grid, 256, smem, static_cast<cudaStream_t>(stream)>>>(x, x_dtype, t, d, wr, bias, e,
                                                                                 logits);
    return check_launch("router_logits");
}

int b200q_shared_gate(const void *x, int x_dtype, int t, int d, const float *gate, float *scale, void *stream) {
    if (!x || !gate || !scale) return fail(B200Q_EINVAL, "shared_gate: NULL pointer");
    if (!dtype_valid(x_dtype) || t <= 0 || d <= 0) return fail(B200Q_EINVAL, "shared_gate: bad argument");
    shared_gate_kernel<<<(t + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, x_dtype, t, d, gate, scale);
    return check_launch("shared_gate");
}

int b200q_router_topk_ex(const float *logits, int rows, int n, int k, int renormalize, float floor_value,
                         int extra_id, const float *extra_weight, float *weights, int64_t *ids, void *stream) {
    if (!logits || !weights || !ids) return fail(B200Q_EINVAL, "router_topk: NULL pointer");
    if (rows <= 0 || n < 1 || n > 4096 || k < 1 || k > 32 || k > n)
        return fail(B200Q_EINVAL, "router_topk: need 1<=n<=4096, 1<=k<=min(32,n)");
    if (renormalize && !(floor_value > 0.0f)) return fail(B200Q_EINVAL, "router_topk: floor must be positive");
    if (n <= 1024)
        return launch_topk_warp(logits, rows, n, k, renormalize, floor_value, extra_id, extra_weight, weights, ids,
                                RowPlanOut{}, static_cast<cudaStream_t>(stream));
    if (extra_id >= 0) return fail(B200Q_EUNSUPPORTED, "router_topk: an appended expert needs n <= 1024");
    router_topk_kernel<<<rows, 128, 0, static_cast<cudaStream_t>(stream)>>>(logits, n, k, renormalize, floor_value,
                                                                            weights, ids);
    return check_launch("router_topk");
}

int b200q_router_topk_plan_row(const float *logits, int n, int k, int renormalize, float floor_value, int extra_id,
                               const float *extra_weight, float *weights, int64_t *ids, int e, int32_t *counts,
                               int32_t *offsets, int32_t *order, int32_t *inv, int32_t *seg_expert, int32_t *seg_begin,
                               int32_t *seg_count, int32_t *num_segments, int max_segments, int32_t *status,
                               void *stream) {
    if (!logits || !weights || !ids || !counts || !offsets || !order || !inv || !seg_expert || !seg_begin ||
        !seg_count || !num_segments || !status)
        return fail(B200Q_EINVAL, "router_topk_plan_row: NULL pointer");
    if (n < 1 || n > 1024 || k < 1 || k > 31 || k > n)
        return fail(B200Q_EINVAL, "router_topk_plan_row: need 1<=n<=1024, 1<=k<=min(31,n)");
    if (renormalize && !(floor_value > 0.0f)) return fail(B200Q_EINVAL, "router_topk_plan_row: floor must be positive");
    const int top = extra_id >= 0 ? (extra_id >= n ? extra_id + 1 : n) : n;      // ids run up to max(n - 1, extra_id)
    if (e < top || e > PLAN_MAX_EXPERTS || max_segments < 1 || (extra_id >= 0 && extra_id < n))
        return fail(B200Q_EINVAL, "router_topk_plan_row: the plan must cover every id; an appended id lies above n");
    RowPlanOut plan{counts, offsets, order, inv, seg_expert, seg_begin, seg_count, num_segments, status, e, max_segments};
    return launch_topk_warp(logits, 1, n, k, renormalize, floor_value, extra_id, extra_weight, weights, ids, plan,
                            static_cast<cudaStream_t>(stream));
}

int b200q_router_topk(const float *logits, int rows, int n, int k, int renormalize, float floor_value,
                      float *weights, int64_t *ids, void *stream) {
    return b200q_router_topk_ex(logits, rows, n, k, renormalize, floor_value, -1, nullptr, weights, ids, stream);
}

// Chooses the rank-by-bitmask path when its table fits in shared memory.
static int launch_plan(const void *ids, int ids_is_i64, int rows, int k, int e, int skip_expert, const PlanIdMap &map,
                       int seg_cap, int32_t *counts, int32_t *offsets, int32_t *order, int32_t *inv,
                       int32_t *seg_expert, int32_t *seg_begin, int32_t *seg_count, int32_t *num_segments,
                       int max_segments, int32_t *status, void *stream, const char *what) {
    constexpr size_t PLAN_BITS_LIMIT = 160 * 1024;
    int words = (rows + 31) / 32;
    size_t bits_bytes = static_cast<size_t>(e) * words * sizeof(unsigned int);
    if (bits_bytes > PLAN_BITS_LIMIT) { words = 0; bits_bytes = 0; }
    if (bits_bytes > 8 * 1024) {      // beyond what fits next to the static arrays without opting in
        cudaError_t err = cudaFuncSetAttribute(reinterpret_cast<const void *>(moe_plan_kernel),
                                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(PLAN_BITS_LIMIT));
        if (err != cudaSuccess) {
            cudaGetLastError();
            return fail(B200Q_ECUDA, "%s: shared memory opt-in failed: %s", what, cudaGetErrorString(err));
        }
    }
    launch_chained(moe_plan_kernel, dim3(1), dim3(PLAN_THREADS), bits_bytes, static_cast<cudaStream_t>(stream), ids,
                   ids_is_i64, rows * k, k, e, skip_expert, map, words, seg_cap, counts, offsets, order, inv,
                   seg_expert, seg_begin, seg_count, num_segments, max_segments, status);
    return check_launch(what);
}

int b200q_moe_plan_ex(const void *ids, int ids_is_i64, int rows, int k, int e, int skip_expert, int seg_cap,
                      int32_t *counts,
                   int32_t *offsets, int32_t *order, int32_t *inv, int32_t *seg_expert, int32_t *seg_begin,
                   int32_t *seg_count, int32_t *num_segments, int max_segments, int32_t *status, void *stream) {
    if (!ids || !counts || !offsets || !order || !inv || !seg_expert || !seg_begin || !seg_count || !num_segments ||
        !status)
        return fail(B200Q_EINVAL, "moe_plan: NULL pointer");
    if (rows <= 0 || k <= 0 || e <= 0 || e > PLAN_MAX_EXPERTS || seg_cap < 1 || seg_cap > 8 || max_segments < 1)
        return fail(B200Q_EINVAL, "moe_plan: bad argument (experts <= %d, 1 <= seg_cap <= 8)", PLAN_MAX_EXPERTS);
    const long long total = static_cast<long long>(rows) * k;
    if (total > (1 << 24)) return fail(B200Q_EUNSUPPORTED, "moe_plan: too many assignments");
    return launch_plan(ids, ids_is_i64, rows, k, e, skip_expert, PlanIdMap{}, seg_cap, counts, offsets, order, inv,
                       seg_expert, seg_begin, seg_count, num_segments, max_segments, status, stream, "moe_plan");
}

int b200q_moe_plan_ep(const void *ids, int ids_is_i64, int rows, int k, int e_global, int first_expert, int n_local,
                      int shared_id, int home_lo, int home_hi, int seg_cap, int32_t *counts, int32_t *offsets,
                      int32_t *order, int32_t *inv, int32_t *seg_expert, int32_t *seg_begin, int32_t *seg_count,
                      int32_t *num_segments, int max_segments, int32_t *status, void *stream) {
    if (!ids || !counts || !offsets || !order || !inv || !seg_expert || !seg_begin || !seg_count || !num_segments ||
        !status)
        return fail(B200Q_EINVAL, "moe_plan_ep: NULL pointer");
    if (rows <= 0 || k <= 0 || n_local <= 0 || n_local + 2 > PLAN_MAX_EXPERTS || first_expert < 0 ||
        e_global < first_expert + n_local || seg_cap < 1 || seg_cap > 8 || max_segments < 1 || home_lo < 0 ||
        home_hi < home_lo || home_hi > rows)
        return fail(B200Q_EINVAL, "moe_plan_ep: bad argument");
    const long long total = static_cast<long long>(rows) * k;
    if (total > (1 << 24)) return fail(B200Q_EUNSUPPORTED, "moe_plan_ep: too many assignments");
    PlanIdMap map{1, k, first_expert, n_local, shared_id, home_lo, home_hi, e_global};
    return launch_plan(ids, ids_is_i64, rows, k, n_local + 2, n_local + 1, map, seg_cap, counts, offsets, order, inv,
                       seg_expert, seg_begin, seg_count, num_segments, max_segments, status, stream, "moe_plan_ep");
}

int b200q_moe_plan(const void *ids, int ids_is_i64, int rows, int k, int e, int seg_cap, int32_t *counts,
                   int32_t *offsets, int32_t *order, int32_t *inv, int32_t *seg_expert, int32_t *seg_begin,
                   int32_t *seg_count, int32_t *num_segments, int max_segments, int32_t *status, void *stream) {
    return b200q_moe_plan_ex(ids, ids_is_i64, rows, k, e, -1, seg_cap, counts, offsets, order, inv, seg_expert,
                             seg_begin, seg_count, num_segments, max_segments, status, stream);
}

int b200q_moe_combine(const float *terms, const int32_t *inv, int rows, int k, int d, const float *extra,
                      const float *extra_scale, void *out, int out_dtype, void *stream) {
    if (!terms || !inv || !out) return fail(B200Q_EINVAL, "moe_combine: NULL pointer");
    if (rows <= 0 || k < 1 || k > 64 || d <= 0 || !dtype_valid(out_dtype))
        return fail(B200Q_EINVAL, "moe_combine: bad argument (k <= 64)");
    return launch_combine_cols(terms, inv, rows, k, d, extra, extra_scale, out, out_dtype,
                               static_cast<cudaStream_t>(stream));
}

int b200q_moe_combine_norm(const float *terms, const int32_t *inv, int rows, int k, int d, const float *extra,
                           const float *extra_scale, int branch_dtype, const float *residual, float alpha,
                           const void *gamma, int gamma_dtype, float eps, float *res_out, void *y, int y_dtype,
                           void *stream) {
    if (!terms || !inv || !residual || !gamma || !res_out || !y)
        return fail(B200Q_EINVAL, "moe_combine_norm: NULL pointer");
    if (rows <= 0 || k < 1 || d <= 0 || !dtype_valid(branch_dtype) || !dtype_valid(gamma_dtype) ||
        !dtype_valid(y_dtype))
        return fail(B200Q_EINVAL, "moe_combine_norm: bad argument");
    if (k > 16) return fail(B200Q_EUNSUPPORTED, "moe_combine_norm: k=%d (at most 16 terms per row)", k);
    if (res_out == residual) return fail(B200Q_EINVAL, "moe_combine_norm: res_out must not alias residual");
    launch_chained(moe_combine_norm_kernel<16>, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), terms, inv,
                   k, d, extra, extra_scale, branch_dtype, residual, alpha, gamma, gamma_dtype, eps, res_out, y, y_dtype);
    return check_launch("moe_combine_norm");
}

}  // extern "C"
