// Instantiations and launcher of the direct-load tensor-core GEMV (Q4_K / Q5_K).
#include "mma_direct.cuh"
#include "mma_host.h"

namespace b200q {

using DirectFn = void (*)(const DirectArgs);

template <bool Q5, int NTERMS>
static DirectFn pick_mode(int mode, int token_tiles) {
    switch (mode) {
        case 0: return token_tiles == 2 ? mma_direct_kernel<Q5, 0, NTERMS, 2> : mma_direct_kernel<Q5, 0, NTERMS, 1>;
        case 1: return token_tiles == 2 ? mma_direct_kernel<Q5, 1, NTERMS, 2> : mma_direct_kernel<Q5, 1, NTERMS, 1>;
        case 2: return mma_direct_kernel<Q5, 2, NTERMS, 1>;
        case 3: return mma_direct_kernel<Q5, 3, NTERMS, 1>;
    }
    return nullptr;
}

static long long direct_smem_bytes(int k, int x_dtype, int token_tiles) {
    const long long nterms = (x_dtype == B200Q_F32) ? 2 : 1;
    const long long nsb = k / 256;
    return MD_CTRL_BYTES + static_cast<long long>(token_tiles) * (MD_PART_BYTES + nterms * nsb * 16 * 256 + nsb * 2 * 128);
}

// Tokens one launch of the direct kernel can take: 16 in the dense modes (two 8-token tiles share
// one pass over the weights) when both tiles' activation fragments fit in shared memory, else 8.
int direct_tokens_per_pass(int fmt, int mode, int k, int x_dtype) {
    if ((fmt != B200Q_Q4_K && fmt != B200Q_Q5_K) || mode > 1 || k <= 0 || k % 256 != 0) return 8;
    return direct_smem_bytes(k, x_dtype, 2) <= MM_SMEM_LIMIT ? 16 : 8;
}

bool direct_plan_args(const MmaRequest &q, DirectArgs *out, long long *smem_out) {
    const bool dual = (q.mode == 1 || q.mode == 2);
    const bool grouped = q.mode >= 2;
    if (q.fmt_a != B200Q_Q4_K && q.fmt_a != B200Q_Q5_K) return false;
    if (dual && q.fmt_a != q.fmt_b) return false;
    if (q.k % 256 != 0 || q.m > direct_tokens_per_pass(q.fmt_a, q.mode, q.k, q.x_dtype)) return false;
    const int token_tiles = q.m > 8 ? 2 : 1;
    if (q.tiled && q.n % 16 != 0) return false;
    if (reinterpret_cast<uintptr_t>(q.wa) & 15) return false;
    if (dual && (reinterpret_cast<uintptr_t>(q.wb) & 15)) return false;
    if (grouped && !q.table_a && ((q.stride_a & 15) || (dual && (q.stride_b & 15)))) return false;
    if (grouped && q.table_a && !q.tables_aligned16) return false;

    DirectArgs a{};
    a.wa = q.wa; a.wb = q.wb; a.stride_a = q.stride_a; a.stride_b = q.stride_b;
    a.table_a = q.table_a; a.table_b = q.table_b;
    a.rb = q.k / 256 * fmt_bytes(q.fmt_a);
    a.tiled = q.tiled;
    a.n = q.n; a.k = q.k; a.m = q.m;
    a.nterms = (q.x_dtype == B200Q_F32) ? 2 : 1;
    const int nsb = q.k / 256;
    // Warps along K: as few as still give every warp of every SM a few tasks (fewer partial sums
    // to combine, longer runs per warp), never more than there are super-blocks in a row.
    const long long row_groups = (static_cast<long long>(q.n) + 15) / 16 * (grouped ? q.max_segments : 1);
    const long long wanted = 3LL * sm_count() * MD_WARPS;
    int kp = 1;
    while (kp * 2 <= MD_WARPS && kp * 2 <= nsb && row_groups * kp < wanted) kp *= 2;
    // ... and enough row blocks that the CTAs finish together: at least six per SM (a grouped launch
    // counts half of the segment bound, the usual number of active segments).
    auto blocks_for = [&](int parts) {
        const int rows = 16 * (MD_WARPS / parts);
        const long long per_unit = (q.n + rows - 1) / rows;
        return per_unit * (grouped ? (q.max_segments > 1 ? q.max_segments / 2 : 1) : 1);
    };
    while (kp * 2 <= MD_WARPS && kp * 2 <= nsb && blocks_for(kp) < 6LL * sm_count()) kp *= 2;
    // A plan of a few segments (one decoded token) cannot fill the SMs six times over whatever the split; what
    // counts then is that no CTA runs two blocks - each block is one chain of dependent loads - while most run one:
    // with between one and two blocks per SM at most, widen the blocks until every CTA has at most one.
    if (grouped) {
        auto most = [&](int parts) {
            const int rows = 16 * (MD_WARPS / parts);
            return static_cast<long long>((q.n + rows - 1) / rows) * q.max_segments;
        };
        if (most(kp) > sm_count() && most(kp) <= 2LL * sm_count())
            while (kp > 1 && most(kp) > sm_count()) kp /= 2;
    }
    a.kp = kp;
    a.rg = MD_WARPS / kp;
    a.off_bfrag = MD_CTRL_BYTES + token_tiles * MD_PART_BYTES;
    const long long bfrag_bytes = static_cast<long long>(token_tiles) * a.nterms * nsb * 16 * 256;
    const long long smem = direct_smem_bytes(q.k, q.x_dtype, token_tiles);
    if (smem > MM_SMEM_LIMIT) return false;
    a.off_xsfrag = static_cast<int>(a.off_bfrag + bfrag_bytes);
    a.x = q.x; a.x_dtype = q.x_dtype; a.y = q.y; a.y_dtype = q.y_dtype;
    a.topk = q.topk; a.order = q.order; a.seg_expert = q.seg_expert; a.seg_begin = q.seg_begin;
    a.seg_count = q.seg_count; a.num_segments = q.num_segments; a.max_segments = q.max_segments;
    a.route = q.route; a.flat_rows = q.flat_rows; a.y_table = q.y_table; a.rows_per_rank = q.rows_per_rank;
    a.images = q.mode == 2 ? static_cast<const uint8_t *>(q.images) : nullptr;
    a.image_stride = direct_token_image_bytes(q.k, q.x_dtype);
    if (a.images && (a.image_stride == 0 || (reinterpret_cast<uintptr_t>(a.images) & 15))) a.images = nullptr;
    *out = a;
    *smem_out = smem;
    return true;
}

int direct_try_launch(const MmaRequest &q, cudaStream_t stream, bool *launched) {
    *launched = false;
    const bool grouped = q.mode >= 2;
    const int token_tiles = q.m > 8 ? 2 : 1;
    DirectArgs a{};
    long long smem = 0;
    if (!direct_plan_args(q, &a, &smem)) return B200Q_OK;
    const bool q5 = q.fmt_a == B200Q_Q5_K;
    DirectFn fn = q5 ? (a.nterms == 2 ? pick_mode<true, 2>(q.mode, token_tiles) : pick_mode<true, 1>(q.mode, token_tiles))
                     : (a.nterms == 2 ? pick_mode<false, 2>(q.mode, token_tiles)
                                      : pick_mode<false, 1>(q.mode, token_tiles));
    if (!fn) return B200Q_OK;
    cudaError_t err = cudaFuncSetAttribute(reinterpret_cast<const void *>(fn),
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, MM_SMEM_LIMIT);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "direct gemv: shared memory opt-in failed: %s", cudaGetErrorString(err));
    }
    int grid = sm_count();
    if (!grouped) {
        const int blocks = (q.n + 16 * a.rg - 1) / (16 * a.rg);
        if (blocks < grid) grid = blocks;
    }
    launch_chained(fn, dim3(grid), dim3(MD_THREADS), static_cast<size_t>(smem), stream, a);
    *launched = true;
    return check_launch("direct gemv");
}

static long long token_image_smem(int k, int x_dtype) {
    const long long nterms = (x_dtype == B200Q_F32) ? 2 : 1;
    const long long nsb = k / 256;
    return MD_CTRL_BYTES + nterms * nsb * 16 * 256 + nsb * 2 * 128;
}

int direct_token_image_bytes(int k, int x_dtype) {
    if (k <= 0 || k % 256 != 0 || token_image_smem(k, x_dtype) > MM_SMEM_LIMIT) return 0;
    return token_image_units(x_dtype == B200Q_F32 ? 2 : 1, k / 256) * 16;
}

int direct_token_images(const void *x, int x_dtype, int rows, int k, void *images, cudaStream_t stream) {
    if (direct_token_image_bytes(k, x_dtype) == 0)
        return fail(B200Q_EUNSUPPORTED, "token images: K=%d is not a multiple of 256 or too large", k);
    if (reinterpret_cast<uintptr_t>(images) & 15) return fail(B200Q_EINVAL, "token images: the buffer must be 16-byte aligned");
    using ImageFn = void (*)(const void *, int, int, uint8_t *);
    ImageFn fn = x_dtype == B200Q_F32 ? token_image_kernel<2> : token_image_kernel<1>;
    cudaError_t err = cudaFuncSetAttribute(reinterpret_cast<const void *>(fn),
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, MM_SMEM_LIMIT);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "token images: shared memory opt-in failed: %s", cudaGetErrorString(err));
    }
    launch_chained(fn, dim3(rows), dim3(MD_THREADS), static_cast<size_t>(token_image_smem(k, x_dtype)), stream, x,
                   x_dtype, k, static_cast<uint8_t *>(images));
    return check_launch("token images");
}

}  // namespace b200q
