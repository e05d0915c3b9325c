// Integer-dot mode: Q8_1 activations against Q4_K weights (decode GEMV, 1..4 tokens per pass).
//
// The FP32-lane and FP16-fragment kernels turn every 4-bit code into a floating-point value before
// it meets the activation; at HBM speed that decode, not the memory system, bounds the Q4_K GEMV.
// With activations quantised to int8 (Q8_1: blocks of 32 values with an FP16 scale d and the FP16
// sum of the block, mini_llm/ops/q8_1_gpu.py:30-58 of the reference) a masked nibble word is
// already the operand of a 4-way integer dot (dp4a), so a weight costs about one instruction.
// Arithmetic per 256-value super-block and token, as in the reference's mixed Q8 kernels
// (mini_llm/ops/mixed_q8_gpu.py:86-139): per sub-block s
//     sd += dx_s * float(dot_s * sc_s),   sm += dx_s * float(sum_s * mn_s)
// with dot_s = integer dot of codes and activation codes, sum_s = integer sum of the activation
// codes, and the super-block contributes dw * sd - dmin * sm. Every integer quantity is exact; the
// FP32 partial sums are added in this kernel's own order (lane, K part), so results agree with the
// reference formula to FP32 rounding, not bit for bit. The mode changes numerics with respect to
// FP32 activations (int8 rounding of x: relative 1/254 of a block's largest value) and is therefore
// opt-in.
//
// Layout of the work: as the direct-load kernel (mma_direct.cuh). A CTA of 16 warps = rg row groups
// of 16 rows x kp parts of K; a warp streams the packed bytes of its rows' super-blocks with 128-bit
// loads (GGUF layout or the Q4_K tile layout), one item ahead in registers; lane (g, tig) handles
// rows g and g+8 and, of every super-block, the 16-value halves tig&1 of sub-blocks 2*(tig>>1),
// +1, +4, +5. The int8 activations of the whole K range sit in shared memory (32-byte blocks, so a
// half block is one aligned 16-byte load), with dx and dx * (sum of a half block's codes) beside them.
#include "common.cuh"

namespace b200q {

constexpr int Q8G_WARPS = 16;
constexpr int Q8G_THREADS = Q8G_WARPS * 32;
constexpr int Q8G_TILE_BYTES = 2304;      // Q4_K tile: 16 rows x one super-block (b200q_q4k_retile)

struct Q8GemvArgs {
    const uint8_t *w;
    int tiled;
    int n, k, m;
    long long row_bytes;
    const uint8_t *xq;        // Q8_1 blocks [m, k/32] of 36 bytes
    void *y;
    int y_dtype;
    int kp, rg;               // K parts and row groups per CTA (kp * rg == 16)
};

__device__ __forceinline__ uint4 q8g_ldg128(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

struct Q4Item {
    uint4 hd_a, hd_b;         // d, dmin, 12 scale bytes of rows g and g+8
    uint4 qa_a, qb_a, qa_b, qb_b;
    uint4 qh_a, qh_b;         // Q5_K: the fifth bits of the lane's 16 elements (all eight sub-blocks), rows g and g+8
};

// ---------------------------------------------------------------------------------------------
// Q8_1 quantiser: one warp per block of 32 values, IEEE arithmetic (the reference's "ieee" control:
// no fast-math). d32 = bounded(max|x| / 127); code = 0 for an all-zero block, else round-half-away
// (x / d32) clamped to +-127; stores half(d32), half(bounded(sum x)) with the sum taken by the
// xor butterfly 16, 8, 4, 2, 1 (lane 0's value), then the 32 codes.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float q8_bounded(float x) { return fabsf(x) > 65504.f ? copysignf(65504.f, x) : x; }

__global__ void q8_1_quantize_kernel(const void *x, int x_dtype, long long total, uint8_t *out) {
    chain_trigger();
    chain_wait();
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;                       // total is a multiple of 32: whole warps leave together
    const float v = load_as_float(x, x_dtype, static_cast<size_t>(i));
    float a = fabsf(v), s = v;
#pragma unroll
    for (int off = 16; off; off >>= 1) {
        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, off));
        s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, off));
    }
    const float d = q8_bounded(__fdiv_rn(a, 127.f));
    float q = a == 0.f ? 0.f : roundf(__fdiv_rn(v, d));
    q = q > 127.f ? 127.f : q < -127.f ? -127.f : q;
    uint8_t *blk = out + (i >> 5) * 36;
    blk[4 + (i & 31)] = static_cast<uint8_t>(static_cast<int8_t>(q));
    if ((i & 31) == 0) {
        *reinterpret_cast<__half *>(blk) = __float2half_rn(q8_bounded(d));
        *reinterpret_cast<__half *>(blk + 2) = __float2half_rn(q8_bounded(s));
    }
}

// ---------------------------------------------------------------------------------------------
// GEMV kernel
// ---------------------------------------------------------------------------------------------
template <int MT, bool Q5>
__global__ void __launch_bounds__(Q8G_THREADS, 1) q4k_q8_gemv_kernel(const Q8GemvArgs a) {
    constexpr int QB = Q5 ? 176 : 144;                        // bytes of a native super-block
    constexpr int TILE = Q5 ? 2816 : Q8G_TILE_BYTES;           // bytes of a 16-row tile (b200q_q4k_retile / b200q_q5k_retile)
    chain_trigger();
    extern __shared__ __align__(16) uint8_t smem[];
    const int nblk = a.k >> 5, nsb = a.k >> 8;
    // shared memory: codes [MT][k] | dx [MT][nblk] | dxs [MT][nblk][2] | partial [2][16 warps][16 rows][MT]
    int8_t *qs_s = reinterpret_cast<int8_t *>(smem);
    float *dx_s = reinterpret_cast<float *>(smem + static_cast<size_t>(MT) * a.k);
    float *dxs_s = dx_s + MT * nblk;
    float *partial = dxs_s + 2 * MT * nblk;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tig = lane & 3;
    const int rgi = warp / a.kp, kpi = warp - rgi * a.kp;
    const int rows_per_block = 16 * a.rg;
    const int total_blocks = (a.n + rows_per_block - 1) / rows_per_block;
    const int blk_begin = static_cast<int>(static_cast<long long>(total_blocks) * blockIdx.x / gridDim.x);
    const int blk_end = static_cast<int>(static_cast<long long>(total_blocks) * (blockIdx.x + 1) / gridDim.x);

    auto issue = [&](int row0, int sb, Q4Item &it) {
        if (a.tiled) {
            const int group = min((row0 >> 4) + rgi, (a.n >> 4) - 1);
            const uint8_t *tile = a.w + (static_cast<size_t>(group) * nsb + sb) * TILE;
            constexpr int P = Q5 ? 768 : 256;                  // first quant plane (Q5_K: behind the fifth bits)
            it.hd_a = q8g_ldg128(tile + 16 * g);
            it.hd_b = q8g_ldg128(tile + 16 * (g + 8));
            if (Q5) {
                it.qh_a = q8g_ldg128(tile + 256 + 32 * g + 16 * (tig & 1));
                it.qh_b = q8g_ldg128(tile + 256 + 32 * (g + 8) + 16 * (tig & 1));
            }
            it.qa_a = q8g_ldg128(tile + P + lane * 16);
            it.qb_a = q8g_ldg128(tile + P + 512 + lane * 16);
            it.qa_b = q8g_ldg128(tile + P + 1024 + lane * 16);
            it.qb_b = q8g_ldg128(tile + P + 1536 + lane * 16);
        } else {
            const uint8_t *ra = a.w + static_cast<size_t>(min(row0 + 16 * rgi + g, a.n - 1)) * a.row_bytes + sb * QB;
            const uint8_t *rb = a.w + static_cast<size_t>(min(row0 + 16 * rgi + g + 8, a.n - 1)) * a.row_bytes + sb * QB;
            constexpr int Q = Q5 ? 48 : 16;                    // first quant byte of a native block
            it.hd_a = q8g_ldg128(ra);
            it.hd_b = q8g_ldg128(rb);
            if (Q5) {
                it.qh_a = q8g_ldg128(ra + 16 + 16 * (tig & 1));
                it.qh_b = q8g_ldg128(rb + 16 + 16 * (tig & 1));
            }
            it.qa_a = q8g_ldg128(ra + Q + 16 * tig);
            it.qb_a = q8g_ldg128(ra + Q + 64 + 16 * tig);
            it.qa_b = q8g_ldg128(rb + Q + 16 * tig);
            it.qb_b = q8g_ldg128(rb + Q + 64 + 16 * tig);
        }
    };
    const int sb_count = kpi < nsb ? (nsb - kpi + a.kp - 1) / a.kp : 0;     // this warp's super-blocks: kpi, kpi+kp, ..
    Q4Item cur, nxt;
    if (blk_begin < blk_end && sb_count > 0) issue(blk_begin * rows_per_block, kpi, nxt);   // weights: before the wait

    chain_wait();                 // the activation blocks come from the preceding kernel (the quantiser)
    // stage the activations: 36-byte blocks -> 32-byte code blocks + scales
    for (int i = tid; i < MT * nblk; i += Q8G_THREADS) {
        const int t = i / nblk, b = i - t * nblk;
        const bool live = t < a.m;
        const uint8_t *src = a.xq + (static_cast<size_t>(t) * nblk + b) * 36;
        uint32_t wds[8];
        int s0 = 0, s1 = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            wds[j] = live ? *reinterpret_cast<const uint32_t *>(src + 4 + 4 * j) : 0u;
            if (j < 4) s0 = __dp4a(0x01010101, static_cast<int>(wds[j]), s0);
            else s1 = __dp4a(0x01010101, static_cast<int>(wds[j]), s1);
        }
        uint4 *dst = reinterpret_cast<uint4 *>(qs_s + static_cast<size_t>(t) * a.k + 32 * b);
        dst[0] = make_uint4(wds[0], wds[1], wds[2], wds[3]);
        dst[1] = make_uint4(wds[4], wds[5], wds[6], wds[7]);
        const float dx = live ? __half2float(*reinterpret_cast<const __half *>(src)) : 0.f;
        dx_s[i] = dx;
        dxs_s[2 * i] = dx * static_cast<float>(s0);
        dxs_s[2 * i + 1] = dx * static_cast<float>(s1);
    }
    __syncthreads();
    if (blk_begin >= blk_end) return;

    const int pair = tig >> 1, half = tig & 1;
    int pbuf = 0;
    for (int blk = blk_begin; blk < blk_end; ++blk) {
        const int row0 = blk * rows_per_block;
        float tot_a[MT], tot_b[MT];
#pragma unroll
        for (int t = 0; t < MT; ++t) tot_a[t] = tot_b[t] = 0.f;
        for (int it = 0; it < sb_count; ++it) {
            cur = nxt;
            if (it + 1 < sb_count) issue(row0, kpi + (it + 1) * a.kp, nxt);
            else if (blk + 1 < blk_end) issue(row0 + rows_per_block, kpi, nxt);
            const int sb = kpi + it * a.kp;
            // scales and minima of the lane's four sub-blocks 2*pair, +1, +4, +5 for both rows
            auto scales = [&](const uint4 &hd, int (&sc)[4], float (&mn)[4], float &d, float &dmin) {
                d = half_bits_to_float(hd.x & 0xffffu);
                dmin = half_bits_to_float(hd.x >> 16);
                const uint32_t lo = hd.y >> (16 * pair), lm = hd.z >> (16 * pair), hi = hd.w >> (16 * pair);
                sc[0] = lo & 63;
                sc[1] = (lo >> 8) & 63;
                sc[2] = (hi & 15) | ((lo >> 2) & 48);
                sc[3] = ((hi >> 8) & 15) | ((lo >> 10) & 48);
                mn[0] = static_cast<float>(lm & 63);
                mn[1] = static_cast<float>((lm >> 8) & 63);
                mn[2] = static_cast<float>(((hi >> 4) & 15) | ((lm >> 2) & 48));
                mn[3] = static_cast<float>(((hi >> 12) & 15) | ((lm >> 10) & 48));
            };
            int sc_a[4], sc_b[4];
            float mn_a[4], mn_b[4], d_a, dm_a, d_b, dm_b;
            scales(cur.hd_a, sc_a, mn_a, d_a, dm_a);
            scales(cur.hd_b, sc_b, mn_b, d_b, dm_b);
            const uint32_t wa[2][4] = {{cur.qa_a.x, cur.qa_a.y, cur.qa_a.z, cur.qa_a.w}, {cur.qb_a.x, cur.qb_a.y, cur.qb_a.z, cur.qb_a.w}};
            const uint32_t wb[2][4] = {{cur.qa_b.x, cur.qa_b.y, cur.qa_b.z, cur.qa_b.w}, {cur.qb_b.x, cur.qb_b.y, cur.qb_b.z, cur.qb_b.w}};
            const uint32_t ha[4] = {cur.qh_a.x, cur.qh_a.y, cur.qh_a.z, cur.qh_a.w}, hb[4] = {cur.qh_b.x, cur.qh_b.y, cur.qh_b.z, cur.qh_b.w};
#pragma unroll
            for (int t = 0; t < MT; ++t) {
                float sd_a = 0.f, sm_a = 0.f, sd_b = 0.f, sm_b = 0.f;
#pragma unroll
                for (int X = 0; X < 2; ++X) {
#pragma unroll
                    for (int nib = 0; nib < 2; ++nib) {
                        const int si = 2 * X + nib;                       // index into sc / mn
                        const int ablk = sb * 8 + 4 * X + 2 * pair + nib;  // activation block = sub-block
                        const uint4 u = *reinterpret_cast<const uint4 *>(qs_s + static_cast<size_t>(t) * a.k + 32 * ablk + 16 * half);
                        const int uw[4] = {static_cast<int>(u.x), static_cast<int>(u.y), static_cast<int>(u.z), static_cast<int>(u.w)};
                        int dot_a = 0, dot_b = 0;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t ua = (wa[X][j] >> (4 * nib)) & 0x0f0f0f0fu, ub = (wb[X][j] >> (4 * nib)) & 0x0f0f0f0fu;
                            if (Q5) {                          // bit (sub-block) of the fifth-bit byte -> bit 4 of the code
                                const int sub = 4 * X + 2 * pair + nib;
                                ua |= ((ha[j] >> sub) << 4) & 0x10101010u;
                                ub |= ((hb[j] >> sub) << 4) & 0x10101010u;
                            }
                            const int ca = static_cast<int>(ua), cb = static_cast<int>(ub);
                            dot_a = __dp4a(ca, uw[j], dot_a);
                            dot_b = __dp4a(cb, uw[j], dot_b);
                        }
                        const float dx = dx_s[t * nblk + ablk], dxs = dxs_s[2 * (t * nblk + ablk) + half];
                        sd_a = fmaf(dx, static_cast<float>(dot_a * sc_a[si]), sd_a);
                        sd_b = fmaf(dx, static_cast<float>(dot_b * sc_b[si]), sd_b);
                        sm_a = fmaf(dxs, mn_a[si], sm_a);
                        sm_b = fmaf(dxs, mn_b[si], sm_b);
                    }
                }
                tot_a[t] += d_a * sd_a - dm_a * sm_a;
                tot_b[t] += d_b * sd_b - dm_b * sm_b;
            }
        }
        // the four lanes of a quad hold the four quarters of each sub-block pair: add them, then the K parts
#pragma unroll
        for (int t = 0; t < MT; ++t) {
            tot_a[t] += __shfl_xor_sync(0xffffffffu, tot_a[t], 1);
            tot_a[t] += __shfl_xor_sync(0xffffffffu, tot_a[t], 2);
            tot_b[t] += __shfl_xor_sync(0xffffffffu, tot_b[t], 1);
            tot_b[t] += __shfl_xor_sync(0xffffffffu, tot_b[t], 2);
        }
        // The K parts of a row group are added by that group's own warps behind a barrier of just those warps, with
        // the partial sums double-buffered: no CTA-wide stop per row block (a warp writes buffer b again only after
        // its group's next barrier, which every reader of b has reached by then).
        float *pb = partial + pbuf * (Q8G_WARPS * 16 * MT);
        if (tig == 0) {
#pragma unroll
            for (int t = 0; t < MT; ++t) {
                pb[(warp * 16 + g) * MT + t] = tot_a[t];
                pb[(warp * 16 + g + 8) * MT + t] = tot_b[t];
            }
        }
        const int group_threads = a.kp * 32;
        if (a.kp == 1) __syncwarp();
        else named_barrier_sync(2 + rgi, group_threads);          // kp >= 2: at most 8 row groups, ids 2..9
        for (int o = kpi * 32 + lane; o < 16 * MT; o += group_threads) {
            const int t = o % MT, r = o / MT;
            const int orow = row0 + 16 * rgi + r;
            if (orow >= a.n || t >= a.m) continue;
            float sum = 0.f;
            for (int kq = 0; kq < a.kp; ++kq) sum += pb[((rgi * a.kp + kq) * 16 + r) * MT + t];
            store_from_float(a.y, a.y_dtype, static_cast<size_t>(t) * a.n + orow, sum);
        }
        pbuf ^= 1;
    }
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_quantize_q8_1(const void *x, int x_dtype, int rows, int k, void *out, void *stream) {
    if (!x || !out) return fail(B200Q_EINVAL, "quantize_q8_1: NULL pointer");
    if (!dtype_valid(x_dtype) || rows <= 0 || k <= 0 || k % 32) return fail(B200Q_EINVAL, "quantize_q8_1: bad argument (K %% 32)");
    const long long total = static_cast<long long>(rows) * k;
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    launch_chained(q8_1_quantize_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), x, x_dtype, total,
                   static_cast<uint8_t *>(out));
    return check_launch("quantize_q8_1");
}

extern "C" int b200q_gemv_q8_1(const void *w, int fmt, int n, int k, const void *xq, int m, void *y, int y_dtype,
                               void *stream) {
    if (!w || !xq || !y) return fail(B200Q_EINVAL, "gemv_q8_1: NULL pointer");
    const bool tiled = fmt == B200Q_Q4_K_TILED || fmt == B200Q_Q5_K_TILED;
    const bool q5 = fmt == B200Q_Q5_K || fmt == B200Q_Q5_K_TILED;
    if (fmt != B200Q_Q4_K && fmt != B200Q_Q5_K && !tiled)
        return fail(B200Q_EUNSUPPORTED, "gemv_q8_1: the integer-dot mode reads Q4_K / Q5_K (GGUF or tile layout)");
    if (!dtype_valid(y_dtype) || n <= 0 || m <= 0 || k <= 0 || k % 256) return fail(B200Q_EINVAL, "gemv_q8_1: bad shape n=%d k=%d m=%d", n, k, m);
    if (tiled && n % 16) return fail(B200Q_EINVAL, "gemv_q8_1: the tile layout needs rows in multiples of 16");
    if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(xq) & 3))
        return fail(B200Q_EUNSUPPORTED, "gemv_q8_1: weights must be 16-byte and activation blocks 4-byte aligned");
    const int nsb = k / 256;
    for (int t0 = 0; t0 < m;) {
        const int mt = m - t0 >= 4 ? 4 : m - t0 >= 2 ? 2 : 1;        // tokens of this pass (1, 2 or 4)
        Q8GemvArgs a{};
        a.w = static_cast<const uint8_t *>(w); a.tiled = tiled ? 1 : 0; a.n = n; a.k = k;
        a.m = mt;
        a.row_bytes = static_cast<long long>(nsb) * (q5 ? 176 : 144);
        a.xq = static_cast<const uint8_t *>(xq) + static_cast<size_t>(t0) * (k / 32) * 36;
        a.y = static_cast<uint8_t *>(y) + static_cast<size_t>(t0) * n * dtype_size(y_dtype);
        a.y_dtype = y_dtype;
        // K parts: as few as still give every SM about six row blocks (see the direct-load kernel)
        int kp = 1;
        auto blocks_for = [&](int parts) { return (static_cast<long long>(n) + 16 * (Q8G_WARPS / parts) - 1) / (16 * (Q8G_WARPS / parts)); };
        while (kp * 2 <= Q8G_WARPS && kp * 2 <= nsb && blocks_for(kp) < 6LL * sm_count()) kp *= 2;
        a.kp = kp; a.rg = Q8G_WARPS / kp;
        const size_t smem = static_cast<size_t>(mt) * k + static_cast<size_t>(mt) * (k / 32) * 12 + 2 * Q8G_WARPS * 16 * mt * 4;
        if (smem > 200 * 1024) return fail(B200Q_EUNSUPPORTED, "gemv_q8_1: K=%d too large for the activation tile", k);
        auto fn = q5 ? (mt == 4 ? q4k_q8_gemv_kernel<4, true> : mt == 2 ? q4k_q8_gemv_kernel<2, true> : q4k_q8_gemv_kernel<1, true>)
                     : (mt == 4 ? q4k_q8_gemv_kernel<4, false> : mt == 2 ? q4k_q8_gemv_kernel<2, false> : q4k_q8_gemv_kernel<1, false>);
        cudaError_t err = cudaFuncSetAttribute(reinterpret_cast<const void *>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (err != cudaSuccess) {
            cudaGetLastError();
            return fail(B200Q_ECUDA, "gemv_q8_1: shared memory opt-in failed: %s", cudaGetErrorString(err));
        }
        int grid = sm_count();
        const long long blocks = blocks_for(kp);
        if (blocks < grid) grid = static_cast<int>(blocks);
        launch_chained(fn, dim3(grid), dim3(Q8G_THREADS), smem, static_cast<cudaStream_t>(stream), a);
        int rc = check_launch("gemv_q8_1");
        if (rc) return rc;
        t0 += mt;
    }
    return B200Q_OK;
}
