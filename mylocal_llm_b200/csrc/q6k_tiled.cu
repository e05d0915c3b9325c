// Q6_K tile layout: re-ordering kernels, the GEMV launcher and the C ABI entry points.
#include "q6k_tiled.cuh"
#include "mma_host.h"

namespace b200q {

// One thread per (tile, lane): writes the lane's 24 code words; lanes 0-15 also copy one row's
// scales (biased by 128) and d.
__global__ void __launch_bounds__(256) q6k_retile_kernel(const uint8_t *src, uint8_t *dst, long long tiles, int nsb) {
    const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    const long long tile = idx >> 5;
    if (tile >= tiles) return;
    const int lane = static_cast<int>(idx & 31), g = lane >> 2, tig = lane & 3;
    const long long group = tile / nsb;
    const int sb = static_cast<int>(tile - group * nsb);
    const size_t row_bytes = static_cast<size_t>(nsb) * 210;
    uint8_t *out = dst + static_cast<size_t>(tile) * Q6T_TILE_BYTES;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const uint8_t *blk = src + (static_cast<size_t>(group) * 16 + g + 8 * half) * row_bytes + static_cast<size_t>(sb) * 210;
        uint32_t words[12];
        for (int c = 0; c < 4; ++c) {
            uint32_t w[3];
            q6k_pack_chunk(blk, c, tig, w);
            words[3 * c] = w[0]; words[3 * c + 1] = w[1]; words[3 * c + 2] = w[2];
        }
        for (int p = 0; p < 3; ++p)
            *reinterpret_cast<uint4 *>(out + (3 * half + p) * 512 + lane * 16) =
                make_uint4(words[4 * p], words[4 * p + 1], words[4 * p + 2], words[4 * p + 3]);
    }
    if (lane < 16) {
        const uint8_t *blk = src + (static_cast<size_t>(group) * 16 + lane) * row_bytes + static_cast<size_t>(sb) * 210;
        for (int i = 0; i < 16; ++i) out[Q6T_SCALES_OFF + 16 * lane + i] = blk[192 + i] ^ 0x80u;
        out[Q6T_D_OFF + 2 * lane] = blk[208];
        out[Q6T_D_OFF + 2 * lane + 1] = blk[209];
    }
}

// Inverse: one thread per (tile, row): rebuilds the row's native 210-byte block.
__global__ void __launch_bounds__(256) q6k_untile_kernel(const uint8_t *src, uint8_t *dst, long long tiles, int nsb) {
    const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    const long long tile = idx >> 4;
    if (tile >= tiles) return;
    const int row = static_cast<int>(idx & 15), g = row & 7, half = row >> 3;
    const long long group = tile / nsb;
    const int sb = static_cast<int>(tile - group * nsb);
    const uint8_t *in = src + static_cast<size_t>(tile) * Q6T_TILE_BYTES;
    uint8_t *blk = dst + (static_cast<size_t>(group) * 16 + row) * (static_cast<size_t>(nsb) * 210) + static_cast<size_t>(sb) * 210;
    for (int i = 0; i < 192; ++i) blk[i] = 0;
    for (int tig = 0; tig < 4; ++tig) {
        const int lane = 4 * g + tig;
        uint32_t words[12];
        for (int p = 0; p < 3; ++p) {
            const uint4 v = *reinterpret_cast<const uint4 *>(in + (3 * half + p) * 512 + lane * 16);
            words[4 * p] = v.x; words[4 * p + 1] = v.y; words[4 * p + 2] = v.z; words[4 * p + 3] = v.w;
        }
        for (int c = 0; c < 4; ++c) {
            const uint32_t w[3] = {words[3 * c], words[3 * c + 1], words[3 * c + 2]};
            for (int j = 0; j < 4; ++j)
                for (int i = 0; i < 4; ++i) {
                    const uint32_t code = q6k_tiled_code(w, j, i);
                    const int h = c >> 1, l = 16 * (c & 1) + 4 * tig + i;
                    const int qi = 64 * h + 32 * (j & 1) + l;
                    blk[qi] |= static_cast<uint8_t>((j >> 1) ? (code & 15u) << 4 : (code & 15u));
                    blk[128 + 32 * h + l] |= static_cast<uint8_t>((code >> 4) << (2 * j));
                }
        }
    }
    for (int i = 0; i < 16; ++i) blk[192 + i] = in[Q6T_SCALES_OFF + 16 * row + i] ^ 0x80u;
    blk[208] = in[Q6T_D_OFF + 2 * row];
    blk[209] = in[Q6T_D_OFF + 2 * row + 1];
}

// Q4_K <-> tile layout: a permutation of 16-byte pieces. One thread per (tile, lane): four pieces of
// its two rows; lanes 0-15 also move one row's first 16 bytes. FORWARD: native -> tiled.
template <bool FORWARD>
__global__ void __launch_bounds__(256) q4k_retile_kernel(const uint8_t *src, uint8_t *dst, long long tiles, int nsb) {
    const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    const long long tile = idx >> 5;
    if (tile >= tiles) return;
    const int lane = static_cast<int>(idx & 31), g = lane >> 2, tig = lane & 3;
    const long long group = tile / nsb;
    const int sb = static_cast<int>(tile - group * nsb);
    const size_t row_bytes = static_cast<size_t>(nsb) * 144;
    const size_t tile_off = static_cast<size_t>(tile) * Q4T_TILE_BYTES;
    auto native_at = [&](int row, int byte) { return (static_cast<size_t>(group) * 16 + row) * row_bytes + static_cast<size_t>(sb) * 144 + byte; };
    auto move = [&](size_t native_off, size_t tiled_off) {
        if (FORWARD) *reinterpret_cast<uint4 *>(dst + tiled_off) = *reinterpret_cast<const uint4 *>(src + native_off);
        else *reinterpret_cast<uint4 *>(dst + native_off) = *reinterpret_cast<const uint4 *>(src + tiled_off);
    };
    move(native_at(g, 16 + 16 * tig), tile_off + 256 + lane * 16);
    move(native_at(g, 80 + 16 * tig), tile_off + 768 + lane * 16);
    move(native_at(g + 8, 16 + 16 * tig), tile_off + 1280 + lane * 16);
    move(native_at(g + 8, 80 + 16 * tig), tile_off + 1792 + lane * 16);
    if (lane < 16) move(native_at(lane, 0), tile_off + 16 * lane);
}

// Q5_K <-> tile layout: as Q4_K, plus the rows' 32 bytes of fifth bits (lanes 0-15 move a row's two halves).
template <bool FORWARD>
__global__ void __launch_bounds__(256) q5k_retile_kernel(const uint8_t *src, uint8_t *dst, long long tiles, int nsb) {
    const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    const long long tile = idx >> 5;
    if (tile >= tiles) return;
    const int lane = static_cast<int>(idx & 31), g = lane >> 2, tig = lane & 3;
    const long long group = tile / nsb;
    const int sb = static_cast<int>(tile - group * nsb);
    const size_t row_bytes = static_cast<size_t>(nsb) * 176;
    const size_t tile_off = static_cast<size_t>(tile) * Q5T_TILE_BYTES;
    auto native_at = [&](int row, int byte) { return (static_cast<size_t>(group) * 16 + row) * row_bytes + static_cast<size_t>(sb) * 176 + byte; };
    auto move = [&](size_t native_off, size_t tiled_off) {
        if (FORWARD) *reinterpret_cast<uint4 *>(dst + tiled_off) = *reinterpret_cast<const uint4 *>(src + native_off);
        else *reinterpret_cast<uint4 *>(dst + native_off) = *reinterpret_cast<const uint4 *>(src + tiled_off);
    };
    move(native_at(g, 48 + 16 * tig), tile_off + 768 + lane * 16);
    move(native_at(g, 112 + 16 * tig), tile_off + 1280 + lane * 16);
    move(native_at(g + 8, 48 + 16 * tig), tile_off + 1792 + lane * 16);
    move(native_at(g + 8, 112 + 16 * tig), tile_off + 2304 + lane * 16);
    if (lane < 16) {
        move(native_at(lane, 0), tile_off + 16 * lane);
        move(native_at(lane, 16), tile_off + 256 + 32 * lane);
        move(native_at(lane, 32), tile_off + 256 + 32 * lane + 16);
    }
}

using Q6Fn = void (*)(const Q6TiledArgs);

// Q8_0 <-> tile layout. One thread per (tile, lane): the 16 code words of its two rows (codes +128);
// lanes 0-15 also move one row's eight block scales. FORWARD: native -> tiled.
template <bool FORWARD>
__global__ void __launch_bounds__(256) q8_retile_kernel(const uint8_t *src, uint8_t *dst, long long tiles, int nsb) {
    const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    const long long tile = idx >> 5;
    if (tile >= tiles) return;
    const int lane = static_cast<int>(idx & 31), g = lane >> 2, tig = lane & 3;
    const long long group = tile / nsb;
    const int sb = static_cast<int>(tile - group * nsb);
    const size_t row_bytes = static_cast<size_t>(nsb) * 272;
    const uint8_t *in = FORWARD ? src : src + static_cast<size_t>(tile) * Q8T_TILE_BYTES;
    uint8_t *out = FORWARD ? dst + static_cast<size_t>(tile) * Q8T_TILE_BYTES : dst;
    for (int half = 0; half < 2; ++half) {
        const size_t row_off = (static_cast<size_t>(group) * 16 + g + 8 * half) * row_bytes + static_cast<size_t>(sb) * 272;
        for (int s = 0; s < 16; ++s) {
            // step s = values 16s..16s+15 of the 256: block s>>1, byte 2 + 16*(s&1) + 4*tig + i inside it
            const size_t native = row_off + static_cast<size_t>(s >> 1) * 34 + 2 + 16 * (s & 1) + 4 * tig;
            const size_t tiled = static_cast<size_t>(4 * half + (s >> 2)) * 512 + lane * 16 + (s & 3) * 4;
            for (int i = 0; i < 4; ++i) {
                if (FORWARD) out[tiled + i] = in[native + i] ^ 0x80u;
                else out[native + i] = in[tiled + i] ^ 0x80u;
            }
        }
    }
    if (lane < 16) {
        const size_t row_off = (static_cast<size_t>(group) * 16 + lane) * row_bytes + static_cast<size_t>(sb) * 272;
        for (int b = 0; b < 8; ++b)
            for (int i = 0; i < 2; ++i) {
                const size_t native = row_off + static_cast<size_t>(b) * 34 + i;
                const size_t tiled = Q8T_SCALES_OFF + 16 * lane + 2 * b + i;
                if (FORWARD) out[tiled] = in[native];
                else out[native] = in[tiled];
            }
    }
}

// Tokens one launch of the tiled kernel can take: 16 (two 8-token tiles share one pass over the
// weights) when both tiles' activation fragments fit in shared memory, else 8.
int tiled_tokens_per_pass(int mode, int k, int x_dtype) {
    if (mode != 0) return 8;
    const long long nterms = (x_dtype == B200Q_F32) ? 2 : 1;
    const long long smem2 = Q6T_CTRL_BYTES + 2LL * Q6T_PART_BYTES + 2LL * nterms * (k / 16) * 256;
    return smem2 <= MM_SMEM_LIMIT ? 16 : 8;
}

// Runs the tiled kernel for a mode 0 or mode 3 request whose weights are in a tile layout
// (q.fmt_a: B200Q_Q6_K_TILED or B200Q_Q8_0_TILED).
int tiled_plan_args(const MmaRequest &q, Q6TiledArgs *out, long long *smem_out) {
    const bool grouped = q.mode == 3;
    if (q.mode != 0 && q.mode != 3) return fail(B200Q_EUNSUPPORTED, "tiled Q6_K: only linear and grouped down");
    const int nt = q.m > 8 ? 2 : 1;                    // 8-token tiles served by one pass over the weights
    if (q.k % 256 != 0 || q.n % 16 != 0 || q.m < 1 || q.m > tiled_tokens_per_pass(q.mode, q.k, q.x_dtype))
        return fail(B200Q_EUNSUPPORTED, "tiled Q6_K: needs K %% 256 == 0, N %% 16 == 0, 1..%d tokens per pass",
                    tiled_tokens_per_pass(q.mode, q.k, q.x_dtype));
    if ((reinterpret_cast<uintptr_t>(q.wa) & 15) || (grouped && !q.table_a && (q.stride_a & 15)) ||
        (grouped && q.table_a && !q.tables_aligned16))
        return fail(B200Q_EINVAL, "tiled Q6_K: weights must be 16-byte aligned");
    Q6TiledArgs a{};
    a.w = q.wa; a.stride = q.stride_a; a.table = q.table_a;
    a.n = q.n; a.k = q.k; a.m = q.m;
    a.nterms = (q.x_dtype == B200Q_F32) ? 2 : 1;
    const int nsb = q.k / 256;
    const long long row_groups = static_cast<long long>(q.n / 16) * (grouped ? q.max_segments : 1);
    const long long wanted = 3LL * sm_count() * Q6T_WARPS;
    int kp = 1;
    while (kp * 2 <= Q6T_WARPS && kp * 2 <= nsb && row_groups * kp < wanted) kp *= 2;
    // enough row blocks that the CTAs finish together (six per SM; half the segment bound when grouped)
    auto blocks_for = [&](int parts) {
        const int groups = Q6T_WARPS / parts;
        const long long per_unit = (q.n / 16 + groups - 1) / groups;
        return per_unit * (grouped ? (q.max_segments > 1 ? q.max_segments / 2 : 1) : 1);
    };
    while (kp * 2 <= Q6T_WARPS && kp * 2 <= nsb && blocks_for(kp) < 6LL * sm_count()) kp *= 2;
    // a plan of a few segments: at most one block per CTA rather than one for most and two for some (each block
    // is one chain of dependent loads; see the direct kernel's launcher)
    if (grouped) {
        auto most = [&](int parts) {
            const int groups = Q6T_WARPS / parts;
            return static_cast<long long>((q.n / 16 + groups - 1) / groups) * q.max_segments;
        };
        if (most(kp) > sm_count() && most(kp) <= 2LL * sm_count())
            while (kp > 1 && most(kp) > sm_count()) kp /= 2;
    }
    a.kp = kp;
    a.rg = Q6T_WARPS / kp;
    a.off_bfrag = Q6T_CTRL_BYTES + nt * Q6T_PART_BYTES;
    const long long smem = a.off_bfrag + static_cast<long long>(nt) * a.nterms * (q.k / 16) * 256;
    if (smem > MM_SMEM_LIMIT) return fail(B200Q_EUNSUPPORTED, "tiled Q6_K: K=%d too large", q.k);
    a.x = q.x; a.x_dtype = q.x_dtype; a.y = q.y; a.y_dtype = q.y_dtype;
    a.order = q.order; a.seg_expert = q.seg_expert; a.seg_begin = q.seg_begin; a.seg_count = q.seg_count;
    a.num_segments = q.num_segments; a.max_segments = q.max_segments; a.route = q.route;
    a.flat_rows = q.flat_rows; a.y_table = q.y_table; a.rows_per_rank = q.rows_per_rank;
    *out = a;
    *smem_out = smem;
    return B200Q_OK;
}

int q6k_tiled_launch(const MmaRequest &q, cudaStream_t stream) {
    const bool grouped = q.mode == 3;
    const int nt = q.m > 8 ? 2 : 1;
    Q6TiledArgs a{};
    long long smem = 0;
    const int rc = tiled_plan_args(q, &a, &smem);
    if (rc) return rc;
    Q6Fn fn;
    if (q.fmt_a == B200Q_Q8_0_TILED) {
        if (grouped) fn = a.nterms == 2 ? tiled_kernel<Q8Tile, 3, 2, 1> : tiled_kernel<Q8Tile, 3, 1, 1>;
        else if (nt == 2) fn = a.nterms == 2 ? tiled_kernel<Q8Tile, 0, 2, 2> : tiled_kernel<Q8Tile, 0, 1, 2>;
        else fn = a.nterms == 2 ? tiled_kernel<Q8Tile, 0, 2, 1> : tiled_kernel<Q8Tile, 0, 1, 1>;
    } else {
        if (grouped) fn = a.nterms == 2 ? tiled_kernel<Q6Tile, 3, 2, 1> : tiled_kernel<Q6Tile, 3, 1, 1>;
        else if (nt == 2) fn = a.nterms == 2 ? tiled_kernel<Q6Tile, 0, 2, 2> : tiled_kernel<Q6Tile, 0, 1, 2>;
        else fn = a.nterms == 2 ? tiled_kernel<Q6Tile, 0, 2, 1> : tiled_kernel<Q6Tile, 0, 1, 1>;
    }
    cudaError_t err = cudaFuncSetAttribute(reinterpret_cast<const void *>(fn),
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, MM_SMEM_LIMIT);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "tiled Q6_K: shared memory opt-in failed: %s", cudaGetErrorString(err));
    }
    int grid = sm_count();
    if (!grouped) {
        const int blocks = (q.n / 16 + a.rg - 1) / a.rg;
        if (blocks < grid) grid = blocks;
    }
    launch_chained(fn, dim3(grid), dim3(Q6T_THREADS), static_cast<size_t>(smem), stream, a);
    return check_launch("tiled Q6_K gemv");
}

static int retile_common(const void *src, void *dst, long long rows, int k, bool forward, void *stream) {
    if (!src || !dst) return fail(B200Q_EINVAL, "q6k_retile: NULL pointer");
    if (rows <= 0 || rows % 16 != 0 || k <= 0 || k % 256 != 0)
        return fail(B200Q_EINVAL, "q6k_retile: rows must be a multiple of 16 and K a multiple of 256");
    if (src == dst) return fail(B200Q_EINVAL, "q6k_retile: in-place conversion is not supported");
    if (reinterpret_cast<uintptr_t>(forward ? dst : src) & 15)
        return fail(B200Q_EINVAL, "q6k_retile: the tiled buffer must be 16-byte aligned");
    const int nsb = k / 256;
    const long long tiles = rows / 16 * nsb;
    const long long threads = tiles * (forward ? 32 : 16);
    const unsigned blocks = static_cast<unsigned>((threads + 255) / 256);
    if (forward)
        q6k_retile_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst), tiles, nsb);
    else
        q6k_untile_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst), tiles, nsb);
    return check_launch("q6k_retile");
}

}  // namespace b200q

using namespace b200q;

// b200q_gemv_norm: y[m, n] = rmsnorm(residual + alpha * branch) W^T with the new residual stream stored as well;
// tile-layout Q6_K / Q8_0 weights, at most NORM_GEMV_MAX_ROWS rows (every CTA normalises the rows itself).
constexpr int NORM_GEMV_MAX_ROWS = 4;

extern "C" int b200q_gemv_norm_supported(int fmt, int n, int k, int act_dtype, int m) {
    if (fmt != B200Q_Q6_K_TILED && fmt != B200Q_Q8_0_TILED) return 0;
    if (act_dtype != B200Q_BF16 && act_dtype != B200Q_F16) return 0;
    if (m < 1 || m > NORM_GEMV_MAX_ROWS || n < 16 || n % 16 != 0 || k < 256 || k % 256 != 0) return 0;
    const long long body = Q6T_CTRL_BYTES + Q6T_PART_BYTES + static_cast<long long>(k / 16) * 256;
    return body + 128 + static_cast<long long>(m) * k * 2 + 10LL * k <= MM_SMEM_LIMIT - 4096 ? 1 : 0;      // + one row's staging
}

extern "C" int b200q_gemv_norm(const void *w, int fmt, int n, int k, const float *residual, const void *branch,
                               int branch_dtype, float alpha, const void *gamma, int act_dtype, float eps, int m,
                               float *res_out, void *y, int y_dtype, void *stream) {
    if (!w || !residual || !branch || !gamma || !res_out || !y) return fail(B200Q_EINVAL, "gemv_norm: NULL pointer");
    if (!dtype_valid(branch_dtype) || !dtype_valid(y_dtype)) return fail(B200Q_EINVAL, "gemv_norm: bad dtype");
    if (!b200q_gemv_norm_supported(fmt, n, k, act_dtype, m))
        return fail(B200Q_EUNSUPPORTED, "gemv_norm: needs tile-layout Q6_K / Q8_0 weights, 16-bit activations, at most %d rows",
                    NORM_GEMV_MAX_ROWS);
    MmaRequest q{};
    q.mode = 0; q.wa = static_cast<const uint8_t *>(w); q.fmt_a = q.fmt_b = fmt; q.n = n; q.k = k; q.m = m;
    q.x = residual;            // placeholder: the kernel reads the normalised rows from its shared memory
    q.x_dtype = act_dtype; q.y = y; q.y_dtype = y_dtype;
    Q6TiledArgs a{};
    long long smem = 0;
    int rc = tiled_plan_args(q, &a, &smem);
    if (rc) return rc;
    NormPrologue pro{};
    pro.residual = residual; pro.branch = branch; pro.branch_dtype = branch_dtype; pro.alpha = alpha;
    pro.gamma = gamma; pro.gamma_dtype = act_dtype; pro.eps = eps; pro.res_out = res_out;
    pro.x_off = static_cast<int>((smem + 127) / 128 * 128);
    smem = pro.x_off + static_cast<long long>(m) * k * 2 + 10LL * k;
    using NormFn = void (*)(const Q6TiledArgs, const NormPrologue);
    NormFn fn = fmt == B200Q_Q8_0_TILED ? tiled_norm_kernel<Q8Tile, 1> : tiled_norm_kernel<Q6Tile, 1>;
    cudaError_t err = cudaFuncSetAttribute(reinterpret_cast<const void *>(fn),
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, MM_SMEM_LIMIT - 4096);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "gemv_norm: shared memory opt-in failed: %s", cudaGetErrorString(err));
    }
    int grid = sm_count();
    const int blocks = (n / 16 + a.rg - 1) / a.rg;
    if (blocks < grid) grid = blocks;
    launch_chained(fn, dim3(grid), dim3(Q6T_THREADS), static_cast<size_t>(smem), static_cast<cudaStream_t>(stream), a, pro);
    return check_launch("gemv_norm");
}

// b200q_gemv_silu: y[m, n] = (silu(gate) * up) W^T for a stacked FP32 gate|up row [m, 2k]; same shapes as b200q_gemv_norm.
extern "C" int b200q_gemv_silu_supported(int fmt, int n, int k, int act_dtype, int m) {
    if (fmt != B200Q_Q6_K_TILED && fmt != B200Q_Q8_0_TILED) return 0;
    if (act_dtype != B200Q_BF16 && act_dtype != B200Q_F16) return 0;
    if (m < 1 || m > NORM_GEMV_MAX_ROWS || n < 16 || n % 16 != 0 || k < 256 || k % 256 != 0) return 0;
    const long long body = Q6T_CTRL_BYTES + Q6T_PART_BYTES + static_cast<long long>(k / 16) * 256;
    return body + 128 + static_cast<long long>(m) * k * 2 <= MM_SMEM_LIMIT - 4096 ? 1 : 0;
}

extern "C" int b200q_gemv_silu(const void *w, int fmt, int n, int k, const float *gate_up, int act_dtype, int m, void *y,
                               int y_dtype, void *stream) {
    if (!w || !gate_up || !y) return fail(B200Q_EINVAL, "gemv_silu: NULL pointer");
    if (!dtype_valid(y_dtype)) return fail(B200Q_EINVAL, "gemv_silu: bad dtype");
    if (reinterpret_cast<uintptr_t>(gate_up) & 15) return fail(B200Q_EUNSUPPORTED, "gemv_silu: gate|up must be 16-byte aligned");
    if (!b200q_gemv_silu_supported(fmt, n, k, act_dtype, m))
        return fail(B200Q_EUNSUPPORTED, "gemv_silu: needs tile-layout Q6_K / Q8_0 weights, 16-bit activations, at most %d rows",
                    NORM_GEMV_MAX_ROWS);
    MmaRequest q{};
    q.mode = 0; q.wa = static_cast<const uint8_t *>(w); q.fmt_a = q.fmt_b = fmt; q.n = n; q.k = k; q.m = m;
    q.x = gate_up;             // placeholder: the kernel reads the activation rows from its shared memory
    q.x_dtype = act_dtype; q.y = y; q.y_dtype = y_dtype;
    Q6TiledArgs a{};
    long long smem = 0;
    int rc = tiled_plan_args(q, &a, &smem);
    if (rc) return rc;
    const int x_off = static_cast<int>((smem + 127) / 128 * 128);
    smem = x_off + static_cast<long long>(m) * k * 2;
    using SiluFn = void (*)(const Q6TiledArgs, const float *, int);
    SiluFn fn = fmt == B200Q_Q8_0_TILED ? tiled_silu_kernel<Q8Tile, 1> : tiled_silu_kernel<Q6Tile, 1>;
    cudaError_t err = cudaFuncSetAttribute(reinterpret_cast<const void *>(fn),
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, MM_SMEM_LIMIT - 4096);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "gemv_silu: shared memory opt-in failed: %s", cudaGetErrorString(err));
    }
    int grid = sm_count();
    const int blocks = (n / 16 + a.rg - 1) / a.rg;
    if (blocks < grid) grid = blocks;
    launch_chained(fn, dim3(grid), dim3(Q6T_THREADS), static_cast<size_t>(smem), static_cast<cudaStream_t>(stream), a, gate_up,
                   x_off);
    return check_launch("gemv_silu");
}

static int q4k_retile_common(const void *src, void *dst, long long rows, int k, bool forward, void *stream) {
    if (!src || !dst) return fail(B200Q_EINVAL, "q4k_retile: NULL pointer");
    if (rows <= 0 || rows % 16 != 0 || k <= 0 || k % 256 != 0)
        return fail(B200Q_EINVAL, "q4k_retile: rows must be a multiple of 16 and K a multiple of 256");
    if (src == dst) return fail(B200Q_EINVAL, "q4k_retile: in-place conversion is not supported");
    if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15)
        return fail(B200Q_EINVAL, "q4k_retile: both buffers must be 16-byte aligned");
    const int nsb = k / 256;
    const long long tiles = rows / 16 * nsb;
    const unsigned blocks = static_cast<unsigned>((tiles * 32 + 255) / 256);
    if (forward)
        q4k_retile_kernel<true><<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst), tiles, nsb);
    else
        q4k_retile_kernel<false><<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst), tiles, nsb);
    return check_launch("q4k_retile");
}

static int q5k_retile_common(const void *src, void *dst, long long rows, int k, bool forward, void *stream) {
    if (!src || !dst) return fail(B200Q_EINVAL, "q5k_retile: NULL pointer");
    if (rows <= 0 || rows % 16 != 0 || k <= 0 || k % 256 != 0)
        return fail(B200Q_EINVAL, "q5k_retile: rows must be a multiple of 16 and K a multiple of 256");
    if (src == dst) return fail(B200Q_EINVAL, "q5k_retile: in-place conversion is not supported");
    if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15)
        return fail(B200Q_EINVAL, "q5k_retile: both buffers must be 16-byte aligned");
    const int nsb = k / 256;
    const long long tiles = rows / 16 * nsb;
    const unsigned blocks = static_cast<unsigned>((tiles * 32 + 255) / 256);
    if (forward)
        q5k_retile_kernel<true><<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst), tiles, nsb);
    else
        q5k_retile_kernel<false><<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst), tiles, nsb);
    return check_launch("q5k_retile");
}

static int q8_retile_common(const void *src, void *dst, long long rows, int k, bool forward, void *stream) {
    if (!src || !dst) return fail(B200Q_EINVAL, "q8_0_retile: NULL pointer");
    if (rows <= 0 || rows % 16 != 0 || k <= 0 || k % 256 != 0)
        return fail(B200Q_EINVAL, "q8_0_retile: rows must be a multiple of 16 and K a multiple of 256");
    if (src == dst) return fail(B200Q_EINVAL, "q8_0_retile: in-place conversion is not supported");
    const int nsb = k / 256;
    const long long tiles = rows / 16 * nsb;
    const unsigned blocks = static_cast<unsigned>((tiles * 32 + 255) / 256);
    if (forward)
        q8_retile_kernel<true><<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst), tiles, nsb);
    else
        q8_retile_kernel<false><<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst), tiles, nsb);
    return check_launch("q8_0_retile");
}

extern "C" int b200q_q8_0_retile(const void *native, void *tiled, int64_t rows, int k, void *stream) {
    return q8_retile_common(native, tiled, rows, k, true, stream);
}

extern "C" int b200q_q8_0_untile(const void *tiled, void *native, int64_t rows, int k, void *stream) {
    return q8_retile_common(tiled, native, rows, k, false, stream);
}

extern "C" int b200q_q5k_retile(const void *native, void *tiled, int64_t rows, int k, void *stream) {
    return q5k_retile_common(native, tiled, rows, k, true, stream);
}

extern "C" int b200q_q5k_untile(const void *tiled, void *native, int64_t rows, int k, void *stream) {
    return q5k_retile_common(tiled, native, rows, k, false, stream);
}

extern "C" int b200q_q4k_retile(const void *native, void *tiled, int64_t rows, int k, void *stream) {
    return q4k_retile_common(native, tiled, rows, k, true, stream);
}

extern "C" int b200q_q4k_untile(const void *tiled, void *native, int64_t rows, int k, void *stream) {
    return q4k_retile_common(tiled, native, rows, k, false, stream);
}

extern "C" int b200q_q6k_retile(const void *native, void *tiled, int64_t rows, int k, void *stream) {
    return retile_common(native, tiled, rows, k, true, stream);
}

extern "C" int b200q_q6k_untile(const void *tiled, void *native, int64_t rows, int k, void *stream) {
    return retile_common(tiled, native, rows, k, false, stream);
}
