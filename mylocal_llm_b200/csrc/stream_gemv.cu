// Host launchers + C ABI for the streaming GEMV family (linear, SwiGLU, grouped experts).
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "mma_host.h"
#include "stream_gemv.cuh"

namespace b200q {

using KernelFn = void (*)(const StreamArgs);

template <int MODE, int FA>
static KernelFn pick_b(int fb) {
    switch (fb) {
        case B200Q_Q8_0: return stream_gemv_kernel<FA, B200Q_Q8_0, MODE>;
        case B200Q_Q4_K: return stream_gemv_kernel<FA, B200Q_Q4_K, MODE>;
        case B200Q_Q5_K: return stream_gemv_kernel<FA, B200Q_Q5_K, MODE>;
        case B200Q_Q6_K: return stream_gemv_kernel<FA, B200Q_Q6_K, MODE>;
    }
    return nullptr;
}

template <int MODE>
static KernelFn pick_dual(int fa, int fb) {
    // the two legacy formats pair only with themselves (keeps the number of kernel variants down)
    if (fa == B200Q_Q4_0 && fb == B200Q_Q4_0) return stream_gemv_kernel<B200Q_Q4_0, B200Q_Q4_0, MODE>;
    if (fa == B200Q_Q3_K && fb == B200Q_Q3_K) return stream_gemv_kernel<B200Q_Q3_K, B200Q_Q3_K, MODE>;
    switch (fa) {
        case B200Q_Q8_0: return pick_b<MODE, B200Q_Q8_0>(fb);
        case B200Q_Q4_K: return pick_b<MODE, B200Q_Q4_K>(fb);
        case B200Q_Q5_K: return pick_b<MODE, B200Q_Q5_K>(fb);
        case B200Q_Q6_K: return pick_b<MODE, B200Q_Q6_K>(fb);
    }
    return nullptr;
}

template <int MODE>
static KernelFn pick_single(int fa) {
    switch (fa) {
        case B200Q_Q8_0: return stream_gemv_kernel<B200Q_Q8_0, B200Q_Q8_0, MODE>;
        case B200Q_Q4_K: return stream_gemv_kernel<B200Q_Q4_K, B200Q_Q4_K, MODE>;
        case B200Q_Q5_K: return stream_gemv_kernel<B200Q_Q5_K, B200Q_Q5_K, MODE>;
        case B200Q_Q6_K: return stream_gemv_kernel<B200Q_Q6_K, B200Q_Q6_K, MODE>;
        case B200Q_Q4_0: return stream_gemv_kernel<B200Q_Q4_0, B200Q_Q4_0, MODE>;
        case B200Q_Q3_K: return stream_gemv_kernel<B200Q_Q3_K, B200Q_Q3_K, MODE>;
    }
    return nullptr;
}

static int align16(int v) { return (v + 15) & ~15; }

// Tile geometry for a (row bytes, K, token count) combination. Returns 0 or an error code.
static int plan_tiles(StreamArgs &a, bool dual, int xbuf_tokens) {
    const int NW = NUM_CONSUMER_WARPS;
    a.kslices = (a.k + SLICE_K - 1) / SLICE_K;
    if (a.kslices > NW) return fail(B200Q_EUNSUPPORTED, "K=%d exceeds %d", a.k, NW * SLICE_K);
    const int unit = (NW % a.kslices == 0) ? NW / a.kslices : 1;
    const long long rbt = static_cast<long long>(a.rb_a) + (dual ? a.rb_b : 0);
    long long r = STAGE_TARGET / rbt;
    r -= r % unit;
    if (r < unit) r = unit;
    if (a.kslices > 1 && r * a.kslices > MAX_PART_ITEMS) r = MAX_PART_ITEMS / a.kslices;
    if (r > a.n) r = a.n;
    if (r < 1) r = 1;
    a.rows_per_tile = static_cast<int>(r);
    a.region_a = align16(a.rows_per_tile * a.rb_a + 32);
    a.region_b = dual ? align16(a.rows_per_tile * a.rb_b + 32) : 0;
    const long long xbytes = static_cast<long long>(xbuf_tokens) * a.k * 4;
    if (xbytes > XBUF_LIMIT) return fail(B200Q_EUNSUPPORTED, "activation tile of %lld bytes too large", xbytes);
    a.xbuf_bytes = align16(static_cast<int>(xbytes));
    const int fixed = SMEM_CTRL_BYTES + SMEM_PART_BYTES + a.xbuf_bytes;
    const int stage = a.region_a + a.region_b;
    int stages = (SMEM_LIMIT - fixed) / stage;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) return fail(B200Q_EUNSUPPORTED, "row of %lld bytes does not fit the staging ring", rbt);
    a.stages = stages;
    return B200Q_OK;
}

static int launch(KernelFn fn, const StreamArgs &a, bool dual, int grid, cudaStream_t stream, const char *what) {
    const int smem = SMEM_CTRL_BYTES + SMEM_PART_BYTES + a.xbuf_bytes + a.stages * (a.region_a + (dual ? a.region_b : 0));
    cudaError_t err = cudaFuncSetAttribute(reinterpret_cast<const void *>(fn),
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "%s: shared memory opt-in failed: %s", what, cudaGetErrorString(err));
    }
    fn<<<grid, STREAM_THREADS, smem, stream>>>(a);
    return check_launch(what);
}

static int tokens_per_launch(int m, int k) {
    int mt = XBUF_LIMIT / (4 * k);
    if (mt > MAX_TOKENS) mt = MAX_TOKENS;
    if (mt > m) mt = m;
    return mt;
}

static bool k_ok(int fmt, int k) { return k > 0 && k % fmt_elems(fmt) == 0; }

// B200Q_KERNEL=lanes forces the FP32-lane kernels (used by the parity tests to cover both
// families); anything else lets every call pick the tensor-core kernel when it applies.
static bool mma_allowed() {
    const char *v = std::getenv("B200Q_KERNEL");
    return !(v && std::strcmp(v, "lanes") == 0);
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_gemv(const void *w, int fmt, int n, int k, const void *x, int x_dtype, int m, void *y, int y_dtype,
               void *stream) {
    if (!w || !x || !y) return fail(B200Q_EINVAL, "gemv: NULL pointer");
    if (fmt == B200Q_Q6_K_TILED || fmt == B200Q_Q8_0_TILED) {
        if (!dtype_valid(x_dtype) || !dtype_valid(y_dtype)) return fail(B200Q_EINVAL, "gemv: bad dtype");
        if (n <= 0 || m <= 0 || k <= 0) return fail(B200Q_EINVAL, "gemv: bad shape n=%d k=%d m=%d", n, k, m);
        const int per_pass = tiled_tokens_per_pass(0, k, x_dtype);
        for (int t0 = 0; t0 < m; t0 += per_pass) {
            MmaRequest q{};
            q.mode = 0; q.wa = static_cast<const uint8_t *>(w); q.fmt_a = q.fmt_b = fmt; q.n = n; q.k = k;
            q.m = (m - t0 < per_pass) ? m - t0 : per_pass;
            q.x = static_cast<const uint8_t *>(x) + static_cast<size_t>(t0) * k * dtype_size(x_dtype);
            q.x_dtype = x_dtype;
            q.y = static_cast<uint8_t *>(y) + static_cast<size_t>(t0) * n * dtype_size(y_dtype);
            q.y_dtype = y_dtype;
            int rc = q6k_tiled_launch(q, static_cast<cudaStream_t>(stream));
            if (rc) return rc;
        }
        return B200Q_OK;
    }
    const bool tiled = direct_tiled_base(fmt) >= 0;
    if (tiled) fmt = direct_tiled_base(fmt);
    if (!fmt_valid(fmt)) return fail(B200Q_EINVAL, "gemv: unknown format %d", fmt);
    if (!dtype_valid(x_dtype) || !dtype_valid(y_dtype)) return fail(B200Q_EINVAL, "gemv: bad dtype");
    if (n <= 0 || m <= 0 || !k_ok(fmt, k)) return fail(B200Q_EINVAL, "gemv: bad shape n=%d k=%d m=%d", n, k, m);
    int *status = device_status_word();
    if (!status) return fail(B200Q_ECUDA, "gemv: no CUDA device");
    StreamArgs a{};
    a.wa = static_cast<const uint8_t *>(w);
    a.wb = nullptr;
    a.rb_a = k / fmt_elems(fmt) * fmt_bytes(fmt);
    a.n = n;
    a.k = k;
    a.x_dtype = x_dtype;
    a.y_dtype = y_dtype;
    a.status = status;
    if (mma_allowed() || tiled) {
        // 8 (or, for the direct kernel with two token tiles, 16) tokens per pass on the tensor cores
        const int per_pass = mma_tokens_per_pass(fmt, 0, k, x_dtype, tiled);
        bool all = true;
        for (int t0 = 0; t0 < m && all; t0 += per_pass) {
            MmaRequest q{};
            q.mode = 0; q.wa = a.wa; q.fmt_a = q.fmt_b = fmt; q.n = n; q.k = k;
            q.m = (m - t0 < per_pass) ? m - t0 : per_pass;
            q.x = static_cast<const uint8_t *>(x) + static_cast<size_t>(t0) * k * dtype_size(x_dtype);
            q.x_dtype = x_dtype;
            q.y = static_cast<uint8_t *>(y) + static_cast<size_t>(t0) * n * dtype_size(y_dtype);
            q.y_dtype = y_dtype; q.status = status; q.tiled = tiled;
            bool launched = false;
            int rc = mma_try_launch(q, static_cast<cudaStream_t>(stream), &launched);
            if (rc) return rc;
            if (!launched) {
                if (t0) return fail(B200Q_ECUDA, "gemv: kernel selection changed between token groups");
                all = false;
            }
        }
        if (all) return B200Q_OK;
    }
    if (tiled) return fail(B200Q_EUNSUPPORTED, "gemv: no kernel reads this shape in the Q4_K / Q5_K tile layout");
    const int mt = tokens_per_launch(m, k);
    if (mt < 1) return fail(B200Q_EUNSUPPORTED, "gemv: K=%d too large", k);
    int rc = plan_tiles(a, false, mt);
    if (rc) return rc;
    KernelFn fn = pick_single<0>(fmt);
    int grid = sm_count();
    const int min_rows = a.rows_per_tile < 4 ? a.rows_per_tile : 4;
    if (static_cast<long long>(grid) * min_rows > n) grid = (n + min_rows - 1) / min_rows;
    for (int t0 = 0; t0 < m; t0 += mt) {
        a.m = (m - t0 < mt) ? m - t0 : mt;
        a.x = static_cast<const uint8_t *>(x) + static_cast<size_t>(t0) * k * dtype_size(x_dtype);
        a.y = static_cast<uint8_t *>(y) + static_cast<size_t>(t0) * n * dtype_size(y_dtype);
        rc = launch(fn, a, false, grid, static_cast<cudaStream_t>(stream), "gemv");
        if (rc) return rc;
    }
    return B200Q_OK;
}

int b200q_swiglu(const void *gate, int gate_fmt, const void *up, int up_fmt, int f, int k, const void *x,
                 int x_dtype, int m, void *h, int h_dtype, void *stream) {
    if (!gate || !up || !x || !h) return fail(B200Q_EINVAL, "swiglu: NULL pointer");
    const bool tiled = direct_tiled_base(gate_fmt) >= 0;
    if (tiled != (direct_tiled_base(up_fmt) >= 0)) return fail(B200Q_EINVAL, "swiglu: gate and up must share the layout");
    if (tiled) { gate_fmt = direct_tiled_base(gate_fmt); up_fmt = direct_tiled_base(up_fmt); }
    if (!fmt_valid(gate_fmt) || !fmt_valid(up_fmt)) return fail(B200Q_EINVAL, "swiglu: unknown format");
    if (!dtype_valid(x_dtype) || !dtype_valid(h_dtype)) return fail(B200Q_EINVAL, "swiglu: bad dtype");
    if (f <= 0 || m <= 0 || !k_ok(gate_fmt, k) || !k_ok(up_fmt, k))
        return fail(B200Q_EINVAL, "swiglu: bad shape f=%d k=%d m=%d", f, k, m);
    int *status = device_status_word();
    if (!status) return fail(B200Q_ECUDA, "swiglu: no CUDA device");
    StreamArgs a{};
    a.wa = static_cast<const uint8_t *>(gate);
    a.wb = static_cast<const uint8_t *>(up);
    a.rb_a = k / fmt_elems(gate_fmt) * fmt_bytes(gate_fmt);
    a.rb_b = k / fmt_elems(up_fmt) * fmt_bytes(up_fmt);
    a.n = f;
    a.k = k;
    a.x_dtype = x_dtype;
    a.y_dtype = h_dtype;
    a.status = status;
    if (mma_allowed() || tiled) {
        const int per_pass = gate_fmt == up_fmt ? mma_tokens_per_pass(gate_fmt, 1, k, x_dtype, tiled) : 8;
        bool all = true;
        for (int t0 = 0; t0 < m && all; t0 += per_pass) {
            MmaRequest q{};
            q.tiled = tiled;
            q.mode = 1; q.wa = a.wa; q.wb = a.wb; q.fmt_a = gate_fmt; q.fmt_b = up_fmt; q.n = f; q.k = k;
            q.m = (m - t0 < per_pass) ? m - t0 : per_pass;
            q.x = static_cast<const uint8_t *>(x) + static_cast<size_t>(t0) * k * dtype_size(x_dtype);
            q.x_dtype = x_dtype;
            q.y = static_cast<uint8_t *>(h) + static_cast<size_t>(t0) * f * dtype_size(h_dtype);
            q.y_dtype = h_dtype; q.status = status;
            bool launched = false;
            int rc = mma_try_launch(q, static_cast<cudaStream_t>(stream), &launched);
            if (rc) return rc;
            if (!launched) {
                if (t0) return fail(B200Q_ECUDA, "swiglu: kernel selection changed between token groups");
                all = false;
            }
        }
        if (all) return B200Q_OK;
    }
    if (tiled) return fail(B200Q_EUNSUPPORTED, "swiglu: no kernel reads this shape in the Q4_K / Q5_K tile layout");
    const int mt = tokens_per_launch(m, k);
    if (mt < 1) return fail(B200Q_EUNSUPPORTED, "swiglu: K=%d too large", k);
    int rc = plan_tiles(a, true, mt);
    if (rc) return rc;
    KernelFn fn = pick_dual<1>(gate_fmt, up_fmt);
    if (!fn) return fail(B200Q_EUNSUPPORTED, "swiglu: Q4_0 / Q3_K pair only with the same format");
    int grid = sm_count();
    const int min_rows = a.rows_per_tile < 4 ? a.rows_per_tile : 4;
    if (static_cast<long long>(grid) * min_rows > f) grid = (f + min_rows - 1) / min_rows;
    for (int t0 = 0; t0 < m; t0 += mt) {
        a.m = (m - t0 < mt) ? m - t0 : mt;
        a.x = static_cast<const uint8_t *>(x) + static_cast<size_t>(t0) * k * dtype_size(x_dtype);
        a.y = static_cast<uint8_t *>(h) + static_cast<size_t>(t0) * f * dtype_size(h_dtype);
        rc = launch(fn, a, true, grid, static_cast<cudaStream_t>(stream), "swiglu");
        if (rc) return rc;
    }
    return B200Q_OK;
}

static int moe_gate_up_impl(const void *gate_base, int64_t gate_stride, int gate_fmt, const void *up_base,
                            int64_t up_stride, int up_fmt, const uint64_t *gate_table, const uint64_t *up_table,
                            int tables_aligned16, int f, int d, const void *x, int x_dtype, int k,
                            const int32_t *order, const int32_t *seg_expert, const int32_t *seg_begin,
                            const int32_t *seg_count, const int32_t *num_segments, int max_segments, float *hbuf,
                            const void *images, void *stream) {
    if ((!gate_table != !up_table) || (!gate_table && (!gate_base || !up_base)) || !x || !order || !seg_expert || !seg_begin || !seg_count || !num_segments || !hbuf)
        return fail(B200Q_EINVAL, "moe_gate_up: NULL pointer");
    const bool tiled = direct_tiled_base(gate_fmt) >= 0;
    if (tiled != (direct_tiled_base(up_fmt) >= 0))
        return fail(B200Q_EINVAL, "moe_gate_up: gate and up must share the layout");
    if (tiled) { gate_fmt = direct_tiled_base(gate_fmt); up_fmt = direct_tiled_base(up_fmt); }
    if (!fmt_valid(gate_fmt) || !fmt_valid(up_fmt) || !dtype_valid(x_dtype))
        return fail(B200Q_EINVAL, "moe_gate_up: bad format/dtype");
    if (f <= 0 || k <= 0 || max_segments <= 0 || !k_ok(gate_fmt, d) || !k_ok(up_fmt, d))
        return fail(B200Q_EINVAL, "moe_gate_up: bad shape f=%d d=%d", f, d);
    int *status = device_status_word();
    if (!status) return fail(B200Q_ECUDA, "moe_gate_up: no CUDA device");
    StreamArgs a{};
    a.wa = static_cast<const uint8_t *>(gate_base);
    a.wb = static_cast<const uint8_t *>(up_base);
    a.stride_a = gate_stride;
    a.stride_b = up_stride;
    a.table_a = reinterpret_cast<const unsigned long long *>(gate_table);
    a.table_b = reinterpret_cast<const unsigned long long *>(up_table);
    a.rb_a = d / fmt_elems(gate_fmt) * fmt_bytes(gate_fmt);
    a.rb_b = d / fmt_elems(up_fmt) * fmt_bytes(up_fmt);
    a.n = f;
    a.k = d;
    a.m = MAX_TOKENS;
    a.x = x;
    a.x_dtype = x_dtype;
    a.y = hbuf;
    a.y_dtype = B200Q_F32;
    a.topk = k;
    a.order = order;
    a.seg_expert = seg_expert;
    a.seg_begin = seg_begin;
    a.seg_count = seg_count;
    a.num_segments = num_segments;
    a.max_segments = max_segments;
    a.status = status;
    if (mma_allowed() || tiled) {
        MmaRequest q{};
        q.tiled = tiled;
        q.mode = 2; q.wa = a.wa; q.wb = a.wb; q.fmt_a = gate_fmt; q.fmt_b = up_fmt; q.stride_a = gate_stride;
        q.stride_b = up_stride; q.table_a = a.table_a; q.table_b = a.table_b; q.tables_aligned16 = tables_aligned16;
        q.n = f; q.k = d; q.m = MAX_TOKENS; q.x = x; q.x_dtype = x_dtype; q.y = hbuf;
        q.y_dtype = B200Q_F32; q.topk = k; q.order = order; q.seg_expert = seg_expert; q.seg_begin = seg_begin;
        q.seg_count = seg_count; q.num_segments = num_segments; q.max_segments = max_segments; q.status = status;
        q.images = images;
        bool launched = false;
        int rc = mma_try_launch(q, static_cast<cudaStream_t>(stream), &launched);
        if (rc || launched) return rc;
    }
    if (tiled) return fail(B200Q_EUNSUPPORTED, "moe_gate_up: no kernel reads this shape in the Q4_K / Q5_K tile layout");
    if (static_cast<long long>(MAX_TOKENS) * d * 4 > XBUF_LIMIT)
        return fail(B200Q_EUNSUPPORTED, "moe_gate_up: d=%d too large for %d tokens per segment", d, MAX_TOKENS);
    int rc = plan_tiles(a, true, MAX_TOKENS);
    if (rc) return rc;
    if (!pick_dual<2>(gate_fmt, up_fmt)) return fail(B200Q_EUNSUPPORTED, "moe_gate_up: Q4_0 / Q3_K pair only with the same format");
    return launch(pick_dual<2>(gate_fmt, up_fmt), a, true, sm_count(), static_cast<cudaStream_t>(stream),
                  "moe_gate_up");
}

int b200q_moe_gate_up(const void *gate_base, int64_t gate_stride, int gate_fmt, const void *up_base,
                      int64_t up_stride, int up_fmt, const uint64_t *gate_table, const uint64_t *up_table,
                      int tables_aligned16, int f, int d, const void *x, int x_dtype, int k,
                      const int32_t *order, const int32_t *seg_expert, const int32_t *seg_begin,
                      const int32_t *seg_count, const int32_t *num_segments, int max_segments, float *hbuf,
                      void *stream) {
    return moe_gate_up_impl(gate_base, gate_stride, gate_fmt, up_base, up_stride, up_fmt, gate_table, up_table,
                            tables_aligned16, f, d, x, x_dtype, k, order, seg_expert, seg_begin, seg_count, num_segments,
                            max_segments, hbuf, nullptr, stream);
}

int b200q_moe_token_image_bytes(int d, int x_dtype) {
    return dtype_valid(x_dtype) ? direct_token_image_bytes(d, x_dtype) : 0;
}

int b200q_moe_token_images(const void *x, int x_dtype, int rows, int d, void *images, void *stream) {
    if (!x || !images) return fail(B200Q_EINVAL, "moe_token_images: NULL pointer");
    if (!dtype_valid(x_dtype) || rows <= 0 || d <= 0) return fail(B200Q_EINVAL, "moe_token_images: bad shape rows=%d d=%d", rows, d);
    return direct_token_images(x, x_dtype, rows, d, images, static_cast<cudaStream_t>(stream));
}

int b200q_moe_gate_up_images(const void *gate_base, int64_t gate_stride, int gate_fmt, const void *up_base,
                             int64_t up_stride, int up_fmt, const uint64_t *gate_table, const uint64_t *up_table,
                             int tables_aligned16, int f, int d, const void *x, int x_dtype, const void *images, int k,
                             const int32_t *order, const int32_t *seg_expert, const int32_t *seg_begin,
                             const int32_t *seg_count, const int32_t *num_segments, int max_segments, float *hbuf,
                             void *stream) {
    if (!images) return fail(B200Q_EINVAL, "moe_gate_up_images: NULL image buffer");
    return moe_gate_up_impl(gate_base, gate_stride, gate_fmt, up_base, up_stride, up_fmt, gate_table, up_table,
                            tables_aligned16, f, d, x, x_dtype, k, order, seg_expert, seg_begin, seg_count, num_segments,
                            max_segments, hbuf, images, stream);
}

static int moe_down_impl(const void *down_base, int64_t down_stride, int down_fmt, const uint64_t *down_table,
                         int tables_aligned16, int flat_rows, int d, int f, const float *hbuf, const float *route,
                         const int32_t *order, const int32_t *seg_expert, const int32_t *seg_begin,
                         const int32_t *seg_count, const int32_t *num_segments, int max_segments, float *terms,
                         const uint64_t *y_table, int rows_per_rank, void *stream) {
    if ((!down_base && !down_table) || !hbuf || !route || !order || !seg_expert || !seg_begin || !seg_count ||
        !num_segments || (!terms && !y_table))
        return fail(B200Q_EINVAL, "moe_down: NULL pointer");
    if (y_table && rows_per_rank < 1) return fail(B200Q_EINVAL, "moe_down: rows_per_rank must be positive");
    if (down_fmt == B200Q_Q6_K_TILED || down_fmt == B200Q_Q8_0_TILED) {
        if (d <= 0 || f <= 0 || max_segments <= 0) return fail(B200Q_EINVAL, "moe_down: bad shape d=%d f=%d", d, f);
        MmaRequest q{};
        q.mode = 3; q.wa = static_cast<const uint8_t *>(down_base); q.fmt_a = q.fmt_b = down_fmt;
        q.stride_a = down_stride; q.table_a = reinterpret_cast<const unsigned long long *>(down_table);
        q.tables_aligned16 = tables_aligned16; q.n = d; q.k = f; q.m = MAX_TOKENS; q.x = hbuf; q.x_dtype = B200Q_F32;
        q.y = terms; q.y_dtype = B200Q_F32; q.topk = 1; q.order = order; q.seg_expert = seg_expert;
        q.seg_begin = seg_begin; q.seg_count = seg_count; q.num_segments = num_segments; q.max_segments = max_segments;
        q.route = route; q.flat_rows = (flat_rows || y_table) ? 1 : 0; q.y_table = y_table;
        q.rows_per_rank = rows_per_rank;
        return q6k_tiled_launch(q, static_cast<cudaStream_t>(stream));
    }
    const bool tiled = direct_tiled_base(down_fmt) >= 0;
    if (tiled) down_fmt = direct_tiled_base(down_fmt);
    if (!fmt_valid(down_fmt)) return fail(B200Q_EINVAL, "moe_down: bad format");
    if (d <= 0 || max_segments <= 0 || !k_ok(down_fmt, f)) return fail(B200Q_EINVAL, "moe_down: bad shape d=%d f=%d", d, f);
    int *status = device_status_word();
    if (!status) return fail(B200Q_ECUDA, "moe_down: no CUDA device");
    StreamArgs a{};
    a.wa = static_cast<const uint8_t *>(down_base);
    a.stride_a = down_stride;
    a.table_a = reinterpret_cast<const unsigned long long *>(down_table);
    a.rb_a = f / fmt_elems(down_fmt) * fmt_bytes(down_fmt);
    a.n = d;
    a.k = f;
    a.m = MAX_TOKENS;
    a.x = hbuf;
    a.x_dtype = B200Q_F32;
    a.y = terms;
    a.y_dtype = B200Q_F32;
    a.topk = 1;
    a.order = order;
    a.seg_expert = seg_expert;
    a.seg_begin = seg_begin;
    a.seg_count = seg_count;
    a.num_segments = num_segments;
    a.max_segments = max_segments;
    a.route = route;
    a.flat_rows = (flat_rows || y_table) ? 1 : 0;
    a.y_table = y_table;
    a.rows_per_rank = rows_per_rank;
    a.status = status;
    if (mma_allowed() || tiled) {
        MmaRequest q{};
        q.tiled = tiled;
        q.mode = 3; q.wa = a.wa; q.fmt_a = q.fmt_b = down_fmt; q.stride_a = down_stride; q.table_a = a.table_a;
        q.tables_aligned16 = tables_aligned16; q.n = d; q.k = f;
        q.m = MAX_TOKENS; q.x = hbuf; q.x_dtype = B200Q_F32; q.y = terms; q.y_dtype = B200Q_F32; q.topk = 1;
        q.order = order; q.seg_expert = seg_expert; q.seg_begin = seg_begin; q.seg_count = seg_count;
        q.num_segments = num_segments; q.max_segments = max_segments; q.route = route; q.flat_rows = a.flat_rows;
        q.y_table = y_table; q.rows_per_rank = rows_per_rank;
        q.status = status;
        bool launched = false;
        int rc = mma_try_launch(q, static_cast<cudaStream_t>(stream), &launched);
        if (rc || launched) return rc;
    }
    if (tiled) return fail(B200Q_EUNSUPPORTED, "moe_down: no kernel reads this shape in the Q4_K / Q5_K tile layout");
    if (static_cast<long long>(MAX_TOKENS) * f * 4 > XBUF_LIMIT)
        return fail(B200Q_EUNSUPPORTED, "moe_down: f=%d too large for %d tokens per segment", f, MAX_TOKENS);
    int rc = plan_tiles(a, false, MAX_TOKENS);
    if (rc) return rc;
    return launch(pick_single<3>(down_fmt), a, false, sm_count(), static_cast<cudaStream_t>(stream), "moe_down");
}

int b200q_moe_down(const void *down_base, int64_t down_stride, int down_fmt, const uint64_t *down_table,
                   int tables_aligned16, int flat_rows, int d, int f, const float *hbuf,
                   const float *route, const int32_t *order, const int32_t *seg_expert, const int32_t *seg_begin,
                   const int32_t *seg_count, const int32_t *num_segments, int max_segments, float *terms,
                   void *stream) {
    return moe_down_impl(down_base, down_stride, down_fmt, down_table, tables_aligned16, flat_rows, d, f, hbuf, route,
                         order, seg_expert, seg_begin, seg_count, num_segments, max_segments, terms, nullptr, 0,
                         stream);
}

int b200q_moe_down_peer(const void *down_base, int64_t down_stride, int down_fmt, const uint64_t *down_table,
                        int tables_aligned16, int d, int f, const float *hbuf, const float *route,
                        const int32_t *order, const int32_t *seg_expert, const int32_t *seg_begin,
                        const int32_t *seg_count, const int32_t *num_segments, int max_segments,
                        const uint64_t *term_tables, int rows_per_rank, void *stream) {
    if (!term_tables) return fail(B200Q_EINVAL, "moe_down_peer: NULL term table");
    return moe_down_impl(down_base, down_stride, down_fmt, down_table, tables_aligned16, 1, d, f, hbuf, route, order,
                         seg_expert, seg_begin, seg_count, num_segments, max_segments, nullptr, term_tables,
                         rows_per_rank, stream);
}

}  // extern "C"
