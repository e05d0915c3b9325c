// Decode-step bookkeeping kernels of the Llama path: rotate-half RoPE fused with the KV-cache
// store, and single-query attention over the cache. They replace a few dozen small framework
// kernels per layer in the one-token step; the packed linears around them are the hot path.
// Semantics follow the reference's inference attention (mini_llm/ops/attention_inference.py:255-277
// for the rotation, 1/sqrt(d_head) scaled softmax over positions 0..pos, grouped KV heads).
#include <cooperative_groups.h>
#include <cstdlib>

#include "common.cuh"
#include "norm_device.cuh"

namespace b200q {

// Rotate-half pair (x0 = dimension i, x1 = dimension i + Dh/2) by the angle with cosine c and sine s. One
// definition with explicit roundings for the stand-alone kernel and for the attention kernel that rotates by
// itself: both give the same bits.
__device__ __forceinline__ float rope_lo(float x0, float x1, float c, float s) {
    return __fmaf_rn(x0, c, -__fmul_rn(x1, s));
}
__device__ __forceinline__ float rope_hi(float x0, float x1, float c, float s) {
    return __fmaf_rn(x0, s, __fmul_rn(x1, c));
}

// q [B, T, H, Dh], k / v [B, T, Hkv, Dh] FP32, each with its own element stride between (b, t)
// rows (so they may be column slices of one fused projection output); positions [T] (device);
// cos / sin [table_rows, Dh/2]. q is rotated in place; rotated k and plain v go to
// cache[b, hkv, positions[t], :]. A position outside [0, min(horizon, table_rows)) touches nothing
// (no table read, q left as it is, no cache store) and records STATUS_POSITION_RANGE: a captured
// step replayed past the end of the cache must not read past the end of the tables.
__global__ void __launch_bounds__(256) rope_kv_store_kernel(float *q, const float *k, const float *v, long long q_row,
                                                            long long k_row, long long v_row,
                                                            const long long *positions, const float *cos_t,
                                                            const float *sin_t, int table_rows, int b, int t, int h,
                                                            int hkv, int dh, int horizon, void *k_cache,
                                                            void *v_cache, int cache_dtype, int *status) {
    chain_trigger();      // the next kernel of the stream may be scheduled; it waits for this grid itself
    chain_wait();         // inputs come from preceding kernels
    const int half = dh >> 1;
    const long long total = static_cast<long long>(b) * t * (h + 2 * hkv) * half;
    for (long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * 256) {
        const int i = static_cast<int>(idx % half);
        long long rest = idx / half;
        const int head = static_cast<int>(rest % (h + 2 * hkv));
        rest /= (h + 2 * hkv);
        const int tt = static_cast<int>(rest % t);
        const int bb = static_cast<int>(rest / t);
        const long long pos = positions[tt];
        if (pos < 0 || pos >= horizon || pos >= table_rows) {
            if (i == 0 && head == 0) atomicExch(status, STATUS_POSITION_RANGE);
            continue;
        }
        if (head < h) {
            float *p = q + (static_cast<size_t>(bb) * t + tt) * q_row + static_cast<size_t>(head) * dh;
            const float c = cos_t[pos * half + i], s = sin_t[pos * half + i];
            const float x0 = p[i], x1 = p[half + i];
            p[i] = rope_lo(x0, x1, c, s);
            p[half + i] = rope_hi(x0, x1, c, s);
        } else if (head < h + hkv) {
            const int kh = head - h;
            const float *p = k + (static_cast<size_t>(bb) * t + tt) * k_row + static_cast<size_t>(kh) * dh;
            const float c = cos_t[pos * half + i], s = sin_t[pos * half + i];
            const float x0 = p[i], x1 = p[half + i];
            const size_t dst = ((static_cast<size_t>(bb) * hkv + kh) * horizon + pos) * dh;
            store_from_float(k_cache, cache_dtype, dst + i, rope_lo(x0, x1, c, s));
            store_from_float(k_cache, cache_dtype, dst + half + i, rope_hi(x0, x1, c, s));
        } else {
            const int vh = head - h - hkv;
            const float *p = v + (static_cast<size_t>(bb) * t + tt) * v_row + static_cast<size_t>(vh) * dh;
            const size_t dst = ((static_cast<size_t>(bb) * hkv + vh) * horizon + pos) * dh;
            store_from_float(v_cache, cache_dtype, dst + i, p[i]);
            store_from_float(v_cache, cache_dtype, dst + half + i, p[half + i]);
        }
    }
}

// EPL consecutive cache elements starting at element index `idx` (a multiple of EPL) as floats.
template <int EPL>
__device__ __forceinline__ void load_row_piece(const void *cache, int dtype, size_t idx, float (&out)[EPL]) {
    if (dtype == B200Q_F32) {
        if (EPL == 2) {
            const float2 v = *reinterpret_cast<const float2 *>(static_cast<const float *>(cache) + idx);
            out[0] = v.x; out[1] = v.y;
        } else {
            const float4 v = *reinterpret_cast<const float4 *>(static_cast<const float *>(cache) + idx);
            out[0] = v.x; out[1] = v.y; out[2 % EPL] = v.z; out[3 % EPL] = v.w;
        }
    } else {
        uint32_t raw[EPL / 2];
        if (EPL == 2) raw[0] = *reinterpret_cast<const uint32_t *>(static_cast<const uint16_t *>(cache) + idx);
        else {
            const uint2 v = *reinterpret_cast<const uint2 *>(static_cast<const uint16_t *>(cache) + idx);
            raw[0] = v.x; raw[(EPL / 2) - 1] = v.y;
        }
#pragma unroll
        for (int e = 0; e < EPL / 2; ++e) {
            if (dtype == B200Q_F16) {
                out[2 * e] = half_bits_to_float(raw[e] & 0xffffu);
                out[2 * e + 1] = half_bits_to_float(raw[e] >> 16);
            } else {
                out[2 * e] = __uint_as_float(raw[e] << 16);
                out[2 * e + 1] = __uint_as_float(raw[e] & 0xffff0000u);
            }
        }
    }
}

// One CTA of 32 warps per (batch, head): warp w takes groups of ATT_U consecutive cache positions
// (all their key and value loads are issued before any arithmetic, so the loop is not bound by one
// load latency per position); each lane holds EPL = Dh/32 dimensions; scores by warp reduction,
// running (max, sum, weighted values) per warp, merged across the warps at the end. A one-token
// step has only batch x heads CTAs, so the positions of a head are spread over as many warps as a
// CTA can hold: with 8 warps a 512-token context took nine dependent iterations (44 us per launch,
// 40 % of a 1.7B Llama step), with 32 warps it takes three. When batch x heads already fills the
// GPU several times over, 8 warps per CTA are the faster shape (less merging, no idle warps).
// SPLIT > 1: a thread-block cluster of SPLIT CTAs shares one (batch, head); CTA r of the cluster
// takes every SPLIT-th group of positions, the partial (max, sum, weighted values) of the CTAs are
// merged by CTA 0 through distributed shared memory between two cluster barriers (hardware
// barriers; nothing spins). The kernel must then be launched with cluster dimension SPLIT.
// FUSE: the kernel also does the work of rope_kv_store_kernel for a one-token step (same results, one launch
// less per layer): q, k, v are the raw projection outputs; every CTA rotates its own query head and the new key
// of its KV head, keeps the new key / value (rounded through the cache type) in shared memory for the position
// it stands for, and the first CTA of each KV head writes them to the caches. A position outside
// [0, min(horizon, table_rows)) leaves q unrotated and the caches untouched and records STATUS_POSITION_RANGE,
// as the stand-alone kernel does.
struct RopeFuse {
    const float *k, *v;
    long long k_row, v_row;
    const float *cos_t, *sin_t;
    int table_rows;
    void *k_cache, *v_cache;       // writable views of the caches
    int *status;
};

template <int EPL, int ATT_U, int ATT_WARPS, int SPLIT, bool FUSE>
__global__ void __launch_bounds__(ATT_WARPS * 32) decode_attention_kernel(const float *q, const void *k_cache,
                                                                          const void *v_cache, int cache_dtype,
                                                                          const long long *position, long long q_row,
                                                                          int h, int hkv, int horizon, float scale,
                                                                          void *out, int out_dtype, const RopeFuse rf) {
    chain_trigger();      // the next kernel of the stream may be scheduled; it waits for this grid itself
    constexpr int DH = EPL * 32;
    __shared__ float sm_m[ATT_WARPS], sm_l[ATT_WARPS], sm_acc[ATT_WARPS][DH];
    __shared__ float fin_ml[2], fin_acc[DH];            // this CTA's merged partial (SPLIT > 1)
    __shared__ float new_k[FUSE ? DH : 1], new_v[FUSE ? DH : 1];
    const int part = SPLIT > 1 ? static_cast<int>(blockIdx.x % SPLIT) : 0;      // rank inside the cluster
    const int bh = blockIdx.x / SPLIT, bb = bh / h, head = bh - bb * h;
    const int kvh = head / (h / hkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    {
        // Before the dependency wait: the cache rows of this warp's first (up to sixteen) groups of positions are asked into L2
        // while the projection that precedes this kernel still runs (the rows were written by earlier steps and left
        // L2 since: a step streams the whole model through it). The position read here may be one step old - it only
        // steers the hint; the real one is read after the wait.
        long long hint = position[0];
        if (hint >= horizon) hint = horizon - 1;
        const int esize = cache_dtype == B200Q_F32 ? 4 : 2;
        const size_t row0 = (static_cast<size_t>(bb) * hkv + kvh) * horizon;
        for (int gi = 0; gi < 16; ++gi) {
            const long long j0 = (static_cast<long long>(gi) * SPLIT * ATT_WARPS + part * ATT_WARPS + warp) * ATT_U;
            if (j0 > hint) break;
#pragma unroll
            for (int u = 0; u < ATT_U; ++u) {
                if (j0 + u > hint) break;
                const size_t off = ((row0 + j0 + u) * DH + lane * EPL) * esize;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const uint8_t *>(k_cache) + off));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const uint8_t *>(v_cache) + off));
            }
        }
    }
    chain_wait();         // inputs come from preceding kernels
    const long long pos = position[0];
    long long last = pos;                               // newest valid cache position
    if (last >= horizon) last = horizon - 1;
    const float *qp = q + static_cast<size_t>(bb) * q_row + static_cast<size_t>(head) * DH;
    float qv[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) qv[e] = qp[lane * EPL + e];
    const bool fuse_valid = FUSE && pos >= 0 && pos < horizon && pos < rf.table_rows;
    if constexpr (FUSE) {
        // lane l holds dimensions l*EPL..; the partner of dimension i < Dh/2 is i + Dh/2 = the same slot of lane l ^ 16
        constexpr int HALF = DH / 2;
        if (!fuse_valid && blockIdx.x == 0 && threadIdx.x == 0) atomicExch(rf.status, STATUS_POSITION_RANGE);
        const bool low = lane < 16;
        float cs[EPL], sn[EPL];
        if (fuse_valid) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                const int i = (lane & 15) * EPL + e;
                cs[e] = rf.cos_t[pos * HALF + i];
                sn[e] = rf.sin_t[pos * HALF + i];
            }
        }
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, qv[e], 16);
            if (fuse_valid) qv[e] = low ? rope_lo(qv[e], other, cs[e], sn[e]) : rope_hi(other, qv[e], cs[e], sn[e]);
        }
        if (warp == 0) {
            const float *kp = rf.k + static_cast<size_t>(bb) * rf.k_row + static_cast<size_t>(kvh) * DH;
            const float *vp = rf.v + static_cast<size_t>(bb) * rf.v_row + static_cast<size_t>(kvh) * DH;
            const bool writer = fuse_valid && part == 0 && head == kvh * (h / hkv);
            const size_t dst = ((static_cast<size_t>(bb) * hkv + kvh) * horizon + (fuse_valid ? pos : 0)) * DH + lane * EPL;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                const float kraw = kp[lane * EPL + e], vraw = vp[lane * EPL + e];
                const float other = __shfl_xor_sync(0xffffffffu, kraw, 16);
                if (fuse_valid) {
                    const float kr = low ? rope_lo(kraw, other, cs[e], sn[e]) : rope_hi(other, kraw, cs[e], sn[e]);
                    new_k[lane * EPL + e] = round_through(cache_dtype, kr);
                    new_v[lane * EPL + e] = round_through(cache_dtype, vraw);
                    if (writer) {
                        store_from_float(rf.k_cache, cache_dtype, dst + e, kr);
                        store_from_float(rf.v_cache, cache_dtype, dst + e, vraw);
                    }
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) qv[e] *= scale;
    const size_t base = (static_cast<size_t>(bb) * hkv + kvh) * horizon * DH + lane * EPL;
    float m = __int_as_float(0xff800000), l = 0.f, acc[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = 0.f;
    for (long long j0 = static_cast<long long>(part * ATT_WARPS + warp) * ATT_U; j0 <= last;
         j0 += SPLIT * ATT_WARPS * ATT_U) {
        float kk[ATT_U][EPL], vv[ATT_U][EPL], dot[ATT_U];
#pragma unroll
        for (int u = 0; u < ATT_U; ++u) {
            const long long j = (j0 + u <= last) ? j0 + u : last;        // clamped rows are masked below
            load_row_piece<EPL>(k_cache, cache_dtype, base + j * DH, kk[u]);
            load_row_piece<EPL>(v_cache, cache_dtype, base + j * DH, vv[u]);
        }
        if (fuse_valid && j0 + ATT_U > pos) {        // the group holds the new position: its row is not in the cache yet
#pragma unroll
            for (int u = 0; u < ATT_U; ++u)
                if (j0 + u >= pos) {                     // the position itself and the masked rows clamped to it
#pragma unroll
                    for (int e = 0; e < EPL; ++e) {
                        kk[u][e] = new_k[lane * EPL + e];
                        vv[u][e] = new_v[lane * EPL + e];
                    }
                }
        }
#pragma unroll
        for (int u = 0; u < ATT_U; ++u) {
            float d = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) d = fmaf(qv[e], kk[u][e], d);
            dot[u] = d;
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
#pragma unroll
            for (int u = 0; u < ATT_U; ++u) dot[u] += __shfl_xor_sync(0xffffffffu, dot[u], o);
        }
        float m_new = m;
#pragma unroll
        for (int u = 0; u < ATT_U; ++u)
            if (j0 + u <= last) m_new = fmaxf(m_new, dot[u]);
        const float corr = __expf(m - m_new);
        l *= corr;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[e] *= corr;
#pragma unroll
        for (int u = 0; u < ATT_U; ++u) {
            const float p = (j0 + u <= last) ? __expf(dot[u] - m_new) : 0.f;
            l += p;
#pragma unroll
            for (int e = 0; e < EPL; ++e) acc[e] = fmaf(p, vv[u][e], acc[e]);
        }
        m = m_new;
    }
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int e = 0; e < EPL; ++e) sm_acc[warp][lane * EPL + e] = acc[e];
    __syncthreads();
    if (warp == 0) {
        float mm = sm_m[0];
#pragma unroll
        for (int w = 1; w < ATT_WARPS; ++w) mm = fmaxf(mm, sm_m[w]);
        float ll = 0.f, r[EPL];
#pragma unroll
        for (int e = 0; e < EPL; ++e) r[e] = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) {
            const float f = sm_l[w] > 0.f ? __expf(sm_m[w] - mm) : 0.f;
            ll += sm_l[w] * f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) r[e] += sm_acc[w][lane * EPL + e] * f;
        }
        if (SPLIT == 1) {
            const float inv = ll > 0.f ? 1.0f / ll : 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e)
                store_from_float(out, out_dtype, (static_cast<size_t>(bb) * h + head) * DH + lane * EPL + e, r[e] * inv);
        } else {
            if (lane == 0) { fin_ml[0] = mm; fin_ml[1] = ll; }
#pragma unroll
            for (int e = 0; e < EPL; ++e) fin_acc[lane * EPL + e] = r[e];
        }
    }
    if constexpr (SPLIT > 1) {
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();                                   // every CTA's partial is in its shared memory
        if (part == 0 && warp == 0) {
            float pm[SPLIT], pl[SPLIT], mm = __int_as_float(0xff800000);
#pragma unroll
            for (int p = 0; p < SPLIT; ++p) {
                const float *ml = cluster.map_shared_rank(fin_ml, p);
                pm[p] = ml[0];
                pl[p] = ml[1];
                mm = fmaxf(mm, pm[p]);
            }
            float ll = 0.f, r[EPL];
#pragma unroll
            for (int e = 0; e < EPL; ++e) r[e] = 0.f;
#pragma unroll
            for (int p = 0; p < SPLIT; ++p) {
                const float f = pl[p] > 0.f ? __expf(pm[p] - mm) : 0.f;
                const float *pa = cluster.map_shared_rank(fin_acc, p);
                ll += pl[p] * f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) r[e] += pa[lane * EPL + e] * f;
            }
            const float inv = ll > 0.f ? 1.0f / ll : 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e)
                store_from_float(out, out_dtype, (static_cast<size_t>(bb) * h + head) * DH + lane * EPL + e, r[e] * inv);
        }
        cluster.sync();                                   // partials stay alive until CTA 0 has read them
    }
}

// act[m, f] = silu(gu[m, f]) * gu[m, F + f] for a stacked gate|up projection output gu [M, 2F] (FP32).
__global__ void __launch_bounds__(256) silu_mul_kernel(const float *gu, int m, int f, void *out, int out_dtype) {
    chain_trigger();      // the next kernel of the stream may be scheduled; it waits for this grid itself
    chain_wait();         // inputs come from preceding kernels
    const long long total = static_cast<long long>(m) * f;
    for (long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * 256) {
        const long long row = idx / f, col = idx - row * f;
        const float g = gu[row * 2 * f + col], u = gu[row * 2 * f + f + col];
        store_from_float(out, out_dtype, static_cast<size_t>(idx), swiglu_f32(g, u));
    }
}

constexpr int ATT_SPLIT = 4;

// B200Q_ATTENTION_SPLIT=0 keeps one CTA per (batch, head) (A/B measurements).
static bool attention_split_enabled() {
    const char *v = std::getenv("B200Q_ATTENTION_SPLIT");
    return !(v && v[0] == '0' && v[1] == 0);
}

// few (batch, head) pairs: 32 warps per CTA, and four CTAs (a cluster) per pair while those still fit the GPU
template <bool FUSE>
static void launch_attention(const float *q, int64_t q_row_stride, const void *k_cache, const void *v_cache, int cache_dtype,
                             const int64_t *position, int batch, int heads, int kv_heads, int head_dim, int horizon,
                             float scale, void *out, int out_dtype, const RopeFuse rf, void *stream) {
    const long long *pos = reinterpret_cast<const long long *>(position);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long pairs = static_cast<long long>(batch) * heads;
    const bool wide = pairs < 2LL * sm_count();
    const bool split = wide && pairs * ATT_SPLIT <= 2LL * sm_count() && attention_split_enabled();
    const long long q_row = q_row_stride;
    if (head_dim == 64 && split)
        launch_chained_cluster(decode_attention_kernel<2, 8, 32, ATT_SPLIT, FUSE>, dim3(pairs * ATT_SPLIT), dim3(1024), 0, s,
                               ATT_SPLIT, q, k_cache, v_cache, cache_dtype, pos, q_row, heads, kv_heads, horizon, scale,
                               out, out_dtype, rf);
    else if (head_dim == 64 && wide)
        launch_chained(decode_attention_kernel<2, 8, 32, 1, FUSE>, dim3(pairs), dim3(1024), 0, s, q, k_cache, v_cache,
                       cache_dtype, pos, q_row, heads, kv_heads, horizon, scale, out, out_dtype, rf);
    else if (head_dim == 64)
        launch_chained(decode_attention_kernel<2, 8, 8, 1, FUSE>, dim3(pairs), dim3(256), 0, s, q, k_cache, v_cache,
                       cache_dtype, pos, q_row, heads, kv_heads, horizon, scale, out, out_dtype, rf);
    else if (split)
        launch_chained_cluster(decode_attention_kernel<4, 4, 32, ATT_SPLIT, FUSE>, dim3(pairs * ATT_SPLIT), dim3(1024), 0, s,
                               ATT_SPLIT, q, k_cache, v_cache, cache_dtype, pos, q_row, heads, kv_heads, horizon, scale,
                               out, out_dtype, rf);
    else if (wide)
        launch_chained(decode_attention_kernel<4, 4, 32, 1, FUSE>, dim3(pairs), dim3(1024), 0, s, q, k_cache, v_cache,
                       cache_dtype, pos, q_row, heads, kv_heads, horizon, scale, out, out_dtype, rf);
    else
        launch_chained(decode_attention_kernel<4, 8, 8, 1, FUSE>, dim3(pairs), dim3(256), 0, s, q, k_cache, v_cache,
                       cache_dtype, pos, q_row, heads, kv_heads, horizon, scale, out, out_dtype, rf);
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_rope_kv_store(float *q, const float *k, const float *v, int64_t q_row_stride, int64_t k_row_stride,
                        int64_t v_row_stride, const int64_t *positions, const float *cos_table,
                        const float *sin_table, int table_rows, int batch, int t, int heads, int kv_heads,
                        int head_dim, int horizon, void *k_cache, void *v_cache, int cache_dtype, void *stream) {
    if (!q || !k || !v || !positions || !cos_table || !sin_table || !k_cache || !v_cache)
        return fail(B200Q_EINVAL, "rope_kv_store: NULL pointer");
    if (batch <= 0 || t <= 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || head_dim % 2 || horizon <= 0 ||
        table_rows <= 0 || !dtype_valid(cache_dtype) || q_row_stride < static_cast<int64_t>(heads) * head_dim ||
        k_row_stride < static_cast<int64_t>(kv_heads) * head_dim ||
        v_row_stride < static_cast<int64_t>(kv_heads) * head_dim)
        return fail(B200Q_EINVAL, "rope_kv_store: bad argument");
    const long long total = static_cast<long long>(batch) * t * (heads + 2 * kv_heads) * (head_dim / 2);
    const int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 4096));
    launch_chained(rope_kv_store_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), q, k, v,
                   q_row_stride, k_row_stride, v_row_stride, reinterpret_cast<const long long *>(positions), cos_table,
                   sin_table, table_rows, batch, t, heads, kv_heads, head_dim, horizon, k_cache, v_cache, cache_dtype,
                   device_status_word());
    return check_launch("rope_kv_store");
}

int b200q_silu_mul(const float *gate_up, int m, int f, void *out, int out_dtype, void *stream) {
    if (!gate_up || !out) return fail(B200Q_EINVAL, "silu_mul: NULL pointer");
    if (m <= 0 || f <= 0 || !dtype_valid(out_dtype)) return fail(B200Q_EINVAL, "silu_mul: bad argument");
    const long long total = static_cast<long long>(m) * f;
    const int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 4096));
    launch_chained(silu_mul_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), gate_up, m, f, out,
                   out_dtype);
    return check_launch("silu_mul");
}

int b200q_decode_attention(const float *q, int64_t q_row_stride, const void *k_cache, const void *v_cache,
                           int cache_dtype, const int64_t *position, int batch, int heads, int kv_heads, int head_dim,
                           int horizon, float scale, void *out, int out_dtype, void *stream) {
    if (!q || !k_cache || !v_cache || !position || !out) return fail(B200Q_EINVAL, "decode_attention: NULL pointer");
    if (batch <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || horizon <= 0 || !dtype_valid(cache_dtype) ||
        !dtype_valid(out_dtype) || q_row_stride < static_cast<int64_t>(heads) * head_dim)
        return fail(B200Q_EINVAL, "decode_attention: bad argument");
    if (head_dim != 64 && head_dim != 128) return fail(B200Q_EUNSUPPORTED, "decode_attention: head_dim must be 64 or 128");
    launch_attention<false>(q, q_row_stride, k_cache, v_cache, cache_dtype, position, batch, heads, kv_heads, head_dim,
                            horizon, scale, out, out_dtype, RopeFuse{}, stream);
    return check_launch("decode_attention");
}

int b200q_rope_attention(const float *q, const float *k, const float *v, int64_t q_row_stride, int64_t k_row_stride,
                         int64_t v_row_stride, const int64_t *position, const float *cos_table, const float *sin_table,
                         int table_rows, int batch, int heads, int kv_heads, int head_dim, int horizon, void *k_cache,
                         void *v_cache, int cache_dtype, float scale, void *out, int out_dtype, void *stream) {
    if (!q || !k || !v || !position || !cos_table || !sin_table || !k_cache || !v_cache || !out)
        return fail(B200Q_EINVAL, "rope_attention: NULL pointer");
    if (batch <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || horizon <= 0 || table_rows <= 0 ||
        !dtype_valid(cache_dtype) || !dtype_valid(out_dtype) || q_row_stride < static_cast<int64_t>(heads) * head_dim ||
        k_row_stride < static_cast<int64_t>(kv_heads) * head_dim || v_row_stride < static_cast<int64_t>(kv_heads) * head_dim)
        return fail(B200Q_EINVAL, "rope_attention: bad argument");
    if (head_dim != 64 && head_dim != 128) return fail(B200Q_EUNSUPPORTED, "rope_attention: head_dim must be 64 or 128");
    int *status = device_status_word();
    if (!status) return fail(B200Q_ECUDA, "rope_attention: no CUDA device");
    const RopeFuse rf{k, v, k_row_stride, v_row_stride, cos_table, sin_table, table_rows, k_cache, v_cache, status};
    launch_attention<true>(q, q_row_stride, k_cache, v_cache, cache_dtype, position, batch, heads, kv_heads, head_dim,
                           horizon, scale, out, out_dtype, rf, stream);
    return check_launch("rope_attention");
}

}  // extern "C"
