// Streaming packed-weight GEMV for sm_100a: persistent CTAs, one per SM.
//
//   producer warp : walks this CTA's contiguous range of weight rows in tiles and moves each
//                   tile's bytes HBM -> shared memory with one (or two) 1-D bulk copies
//                   (cp.async.bulk, completion on an mbarrier), several tiles ahead;
//   consumer warps: wait for a tile, compute (row, 2048-wide K slice) dot products with the
//                   activations held in registers (decode.cuh), reduce over the warp, write
//                   the outputs, and hand the stage back through a second mbarrier.
//
// HBM traffic is the packed bytes once plus activations/outputs: the weights of a tile are
// used for every token of the launch (up to 8) before the stage is released.
//
// The same kernel runs four "modes":
//   0  y = x W^T                         (quantized_linear)
//   1  h = silu(x G^T) * (x U^T)         (quantized_swiglu; two weight streams per tile)
//   2  mode 1 over expert segments       (grouped experts, gate/up)
//   3  mode 0 over expert segments with the route weight applied (grouped experts, down)
// In modes 2/3 the rows of all active segments form one virtual row space that is split evenly
// over the CTAs; the tokens of a segment are gathered through the routing plan.
//
// Every wait on an mbarrier has a wall-clock limit; a wait that gives up records a code in the
// device status word and the CTA drains and returns.
#pragma once

#include "decode.cuh"

namespace b200q {

constexpr int NUM_CONSUMER_WARPS = 12;
constexpr int STREAM_THREADS = (NUM_CONSUMER_WARPS + 1) * 32;
constexpr int MAX_TOKENS = 8;
constexpr int MAX_PART_ITEMS = 32;
constexpr int MAX_STAGES = 8;
constexpr int SMEM_CTRL_BYTES = 1024;
constexpr int SMEM_PART_BYTES = 2 * MAX_TOKENS * MAX_PART_ITEMS * 2 * 4;
constexpr int SMEM_LIMIT = 232448;  // 227 KB opt-in maximum per CTA
constexpr int STAGE_TARGET = 36864;
constexpr int XBUF_LIMIT = 65536;

struct StreamArgs {
    // weights: stream A (and B in dual modes); grouped modes add expert * stride
    const uint8_t *wa;
    const uint8_t *wb;
    long long stride_a, stride_b;
    const unsigned long long *table_a, *table_b;   // optional per-expert pointer tables
    int rb_a, rb_b;        // packed bytes per row
    int n;                 // rows per matrix
    int k;                 // reduction length
    int m;                 // tokens (modes 0/1); grouped: upper bound on tokens per segment
    int kslices;           // ceil(k / 2048)
    int rows_per_tile;
    int stages;
    int region_a, region_b;  // bytes reserved per stage for each stream (16-byte multiples)
    int xbuf_bytes;
    // activations / outputs
    const void *x;
    int x_dtype;
    void *y;
    int y_dtype;
    // grouped plan
    int topk;              // assignments per token (mode 2: token = order[pos] / topk)
    const int32_t *order;
    const int32_t *seg_expert;
    const int32_t *seg_begin;
    const int32_t *seg_count;
    const int32_t *num_segments;
    int max_segments;
    const float *route;    // mode 3: flat [rows*topk] route weights
    int flat_rows;         // mode 3: store term rows at the flat assignment index instead of the sorted position
    const uint64_t *y_table;   // mode 3, optional: per-rank base addresses of the term buffers (peer memory)
    int rows_per_rank;     // flat rows owned by each rank when y_table is set
    int *status;
};

struct TileDesc {
    int unit;   // segment index (grouped) or 0
    int row0;   // first row inside the matrix
    int rows;   // rows in this tile (0 = no more tiles)
};

// Walk of one CTA's virtual-row range; identical on the producer and consumer side.
struct TileWalker {
    long long v, v_end;
    int n_rows, tile_rows;
    __device__ __forceinline__ TileDesc next() {
        TileDesc t;
        if (v >= v_end) { t.unit = 0; t.row0 = 0; t.rows = 0; return t; }
        t.unit = static_cast<int>(v / n_rows);
        t.row0 = static_cast<int>(v - static_cast<long long>(t.unit) * n_rows);
        long long r = tile_rows;
        if (r > n_rows - t.row0) r = n_rows - t.row0;
        if (r > v_end - v) r = v_end - v;
        t.rows = static_cast<int>(r);
        v += r;
        return t;
    }
};

// Issue the copy of `rows` packed rows starting at `src` into `dst_region`; returns the byte
// offset of the first row inside the region. Runs on the whole producer warp.
// `limit` is the end of the weight buffer: the 16-byte window of a bulk copy never reads past it.
__device__ __forceinline__ int issue_rows(uint8_t *dst_region, const uint8_t *src, const uint8_t *buffer_base,
                                          const uint8_t *limit, uint32_t bytes, uint64_t *bar, int lane,
                                          uint32_t &tx_bytes) {
    const uintptr_t g = reinterpret_cast<uintptr_t>(src);
    if ((reinterpret_cast<uintptr_t>(buffer_base) & 15) != 0) {
        // Unaligned weight buffer: plain byte copy by the producer warp (slow, always correct).
        for (uint32_t i = lane; i < bytes; i += 32) dst_region[i] = src[i];
        return 0;
    }
    const uintptr_t a0 = g & ~uintptr_t(15);
    const int head = static_cast<int>(g - a0);
    uintptr_t a1 = (g + bytes + 15) & ~uintptr_t(15);
    const uintptr_t lim = reinterpret_cast<uintptr_t>(limit);
    uint32_t tail = 0;
    if (a1 > lim) {
        a1 = lim & ~uintptr_t(15);
        tail = static_cast<uint32_t>((g + bytes) - a1);  // < 16 bytes, copied by hand
    }
    const uint32_t bulk = a1 > a0 ? static_cast<uint32_t>(a1 - a0) : 0u;
    if (tail) {
        const uint8_t *ts = reinterpret_cast<const uint8_t *>(a1);
        uint8_t *td = dst_region + (a1 - a0);
        if (lane < static_cast<int>(tail)) td[lane] = ts[lane];
    }
    if (bulk && lane == 0) bulk_copy_g2s(dst_region, reinterpret_cast<const void *>(a0), bulk, bar);
    tx_bytes += bulk;
    return head;
}

// Head offset of a tile's first row inside its stage region (must match issue_rows).
__device__ __forceinline__ int region_head(const uint8_t *src, const uint8_t *buffer_base) {
    if ((reinterpret_cast<uintptr_t>(buffer_base) & 15) != 0) return 0;
    return static_cast<int>(reinterpret_cast<uintptr_t>(src) & 15);
}

template <int FMT_A, int FMT_B, int MODE>
__global__ void __launch_bounds__(STREAM_THREADS, 1) stream_gemv_kernel(const StreamArgs a) {
    constexpr bool DUAL = (MODE == 1 || MODE == 2);
    constexpr bool GROUPED = (MODE >= 2);
    using DecA = LaneDecoder<FMT_A>;
    using DecB = LaneDecoder<FMT_B>;

    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty_bar = full_bar + MAX_STAGES;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 256);
    float *route_w = reinterpret_cast<float *>(smem + 512);            // [MAX_TOKENS]
    int *seg_tokens = reinterpret_cast<int *>(smem + 512 + 64);        // [MAX_TOKENS]
    float **out_ptr = reinterpret_cast<float **>(smem + 512 + 128);    // [MAX_TOKENS] mode 3 output row pointers
    float *partial = reinterpret_cast<float *>(smem + SMEM_CTRL_BYTES);
    float *xbuf = reinterpret_cast<float *>(smem + SMEM_CTRL_BYTES + SMEM_PART_BYTES);
    uint8_t *stage_base = smem + SMEM_CTRL_BYTES + SMEM_PART_BYTES + a.xbuf_bytes;
    const int stage_bytes = a.region_a + (DUAL ? a.region_b : 0);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = a.stages;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], NUM_CONSUMER_WARPS);
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();

    // This CTA's share of the (virtual) row space.
    long long total_rows = a.n;
    if (GROUPED) {
        int nseg = *a.num_segments;
        if (nseg > a.max_segments) nseg = a.max_segments;
        total_rows = static_cast<long long>(nseg) * a.n;
    }
    TileWalker walk;
    walk.v = total_rows * blockIdx.x / gridDim.x;
    walk.v_end = total_rows * (blockIdx.x + 1) / gridDim.x;
    walk.n_rows = a.n;
    walk.tile_rows = a.rows_per_tile;
    if (walk.v >= walk.v_end) return;

    const size_t matrix_bytes_a = static_cast<size_t>(a.n) * a.rb_a;
    const size_t matrix_bytes_b = static_cast<size_t>(a.n) * a.rb_b;

    if (warp == NUM_CONSUMER_WARPS) {
        // ------------------------------------------------------------------ producer warp
        for (int it = 0;; ++it) {
            const TileDesc t = walk.next();
            if (t.rows == 0 || *abort_flag) break;
            const int s = it % S;
            if (it >= S) {
                if (!mbar_wait_bounded(&empty_bar[s], ((it / S) - 1) & 1, a.status, STATUS_WAIT_EMPTY)) {
                    *abort_flag = 1;
                    break;
                }
            }
            const int expert = GROUPED ? a.seg_expert[t.unit] : 0;
            const uint8_t *base_a = expert_matrix(a.wa, a.stride_a, a.table_a, expert);
            uint8_t *region = stage_base + static_cast<size_t>(s) * stage_bytes;
            uint32_t tx = 0;
            // Reads of this stage by the consumers (generic proxy) are ordered before the
            // asynchronous writes that refill it.
            fence_proxy_async();
            issue_rows(region, base_a + static_cast<size_t>(t.row0) * a.rb_a, base_a, base_a + matrix_bytes_a,
                       static_cast<uint32_t>(t.rows) * a.rb_a, &full_bar[s], lane, tx);
            if (DUAL) {
                const uint8_t *base_b = expert_matrix(a.wb, a.stride_b, a.table_b, expert);
                issue_rows(region + a.region_a, base_b + static_cast<size_t>(t.row0) * a.rb_b, base_b,
                           base_b + matrix_bytes_b, static_cast<uint32_t>(t.rows) * a.rb_b, &full_bar[s], lane, tx);
            }
            __syncwarp();
            if (lane == 0) {
                if (tx) mbar_arrive_expect_tx(&full_bar[s], tx);
                else mbar_arrive(&full_bar[s]);
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumer warps
    const int ctid = tid;  // 0 .. NUM_CONSUMER_WARPS*32-1
    constexpr int CTHREADS = NUM_CONSUMER_WARPS * 32;
    const int K = a.k, KS = a.kslices;
    int m_tokens = a.m;

    if (!GROUPED) {
        // Stage the activations once, converted to FP32.
        const int total = a.m * K;
        for (int i = ctid; i < total; i += CTHREADS) xbuf[i] = load_as_float(a.x, a.x_dtype, i);
        named_barrier_sync(1, CTHREADS);
    }

    float xr[XREGS];
    float xs[8];
    int cur_m = -1, cur_slice = -1;
    int cur_unit = -1, last_single_token = -1;
    int pbuf = 0;
    int seg_begin = 0;

    for (int it = 0;; ++it) {
        const TileDesc t = walk.next();
        if (t.rows == 0 || *abort_flag) break;
        const int s = it % S;

        const uint8_t *base_a = a.wa, *base_b = a.wb;
        if (GROUPED) {
            const int expert = a.seg_expert[t.unit];
            base_a = expert_matrix(a.wa, a.stride_a, a.table_a, expert);
            if (DUAL) base_b = expert_matrix(a.wb, a.stride_b, a.table_b, expert);
            if (t.unit != cur_unit) {
                // New segment: gather its tokens' activations into shared memory.
                cur_unit = t.unit;
                seg_begin = a.seg_begin[t.unit];
                m_tokens = a.seg_count[t.unit];
                if (m_tokens > MAX_TOKENS) m_tokens = MAX_TOKENS;
                int single = -1;
                if (MODE == 2 && m_tokens == 1) single = a.order[seg_begin] / a.topk;
                const bool reuse = (MODE == 2 && single >= 0 && single == last_single_token);
                last_single_token = single;
                if (!reuse) {
                    named_barrier_sync(1, CTHREADS);  // everyone is done with the previous x
                    if (ctid < m_tokens) {
                        const int flat = a.order[seg_begin + ctid];
                        seg_tokens[ctid] = (MODE == 2) ? flat / a.topk : seg_begin + ctid;
                        if (MODE == 3) {
                            route_w[ctid] = a.route[flat];
                            out_ptr[ctid] = term_row_pointer(static_cast<float *>(a.y), a.y_table, a.rows_per_rank, a.n, a.flat_rows ? flat : seg_begin + ctid);
                        }
                    }
                    named_barrier_sync(1, CTHREADS);
                    const int total = m_tokens * K;
                    for (int i = ctid; i < total; i += CTHREADS) {
                        const int mm = i / K, kk = i - mm * K;
                        xbuf[i] = load_as_float(a.x, a.x_dtype, static_cast<size_t>(seg_tokens[mm]) * K + kk);
                    }
                    named_barrier_sync(1, CTHREADS);
                    cur_m = -1;
                } else if (MODE == 3) {
                    // unreachable: reuse is only taken in mode 2
                }
            }
        }

        if (!mbar_wait_bounded(&full_bar[s], (it / S) & 1, a.status, STATUS_WAIT_FULL)) {
            *abort_flag = 1;
            break;
        }

        const uint8_t *region = stage_base + static_cast<size_t>(s) * stage_bytes;
        const uint8_t *rows_a = region + region_head(base_a + static_cast<size_t>(t.row0) * a.rb_a, base_a);
        const uint8_t *rows_b = nullptr;
        if (DUAL)
            rows_b = region + a.region_a + region_head(base_b + static_cast<size_t>(t.row0) * a.rb_b, base_b);

        const int items = t.rows * KS;
        for (int m = 0; m < m_tokens; ++m) {
            for (int item = warp; item < items; item += NUM_CONSUMER_WARPS) {
                const int row = item / KS, slice = item - row * KS;
                if (slice != cur_slice || m != cur_m) {
                    DecA::load_x(xbuf + static_cast<size_t>(m) * K, K, slice, lane, xr, xs);
                    cur_slice = slice;
                    cur_m = m;
                }
                float pa = DecA::dot(rows_a + static_cast<size_t>(row) * a.rb_a, K, slice, lane, xr, xs);
                float pb = 0.f;
                if (DUAL) {
                    if (FMT_B != FMT_A && (FMT_A == B200Q_Q6_K || FMT_A == B200Q_Q8_0 || FMT_B == B200Q_Q6_K ||
                                           FMT_B == B200Q_Q8_0)) {
                        // the two formats map lanes to different K positions: reload for B
                        float xr2[XREGS];
                        float xs2[8];
                        DecB::load_x(xbuf + static_cast<size_t>(m) * K, K, slice, lane, xr2, xs2);
                        pb = DecB::dot(rows_b + static_cast<size_t>(row) * a.rb_b, K, slice, lane, xr2, xs2);
                    } else {
                        pb = DecB::dot(rows_b + static_cast<size_t>(row) * a.rb_b, K, slice, lane, xr, xs);
                    }
                }
                pa = warp_sum(pa);
                if (DUAL) pb = warp_sum(pb);
                if (KS == 1) {
                    if (lane == 0) {
                        const int orow = t.row0 + row;
                        if (MODE == 0) store_from_float(a.y, a.y_dtype, static_cast<size_t>(m) * a.n + orow, pa);
                        else if (MODE == 1)
                            store_from_float(a.y, a.y_dtype, static_cast<size_t>(m) * a.n + orow, swiglu_f32(pa, pb));
                        else if (MODE == 2)
                            static_cast<float *>(a.y)[static_cast<size_t>(seg_begin + m) * a.n + orow] =
                                swiglu_f32(pa, pb);
                        else
                            out_ptr[m][orow] =
                                pa * route_w[m];
                    }
                } else if (lane == 0) {
                    float *dst = partial + ((pbuf * MAX_TOKENS + m) * MAX_PART_ITEMS + item) * 2;
                    dst[0] = pa;
                    dst[1] = pb;
                }
            }
        }

        // The stage's bytes are no longer needed: hand it back to the producer.
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[s]);

        if (KS > 1) {
            named_barrier_sync(2, CTHREADS);
            const int outs = m_tokens * t.rows;
            for (int o = ctid; o < outs; o += CTHREADS) {
                const int m = o / t.rows, row = o - m * t.rows;
                const float *src = partial + ((pbuf * MAX_TOKENS + m) * MAX_PART_ITEMS + row * KS) * 2;
                float pa = 0.f, pb = 0.f;
                for (int sl = 0; sl < KS; ++sl) { pa += src[2 * sl]; pb += src[2 * sl + 1]; }
                const int orow = t.row0 + row;
                if (MODE == 0) store_from_float(a.y, a.y_dtype, static_cast<size_t>(m) * a.n + orow, pa);
                else if (MODE == 1)
                    store_from_float(a.y, a.y_dtype, static_cast<size_t>(m) * a.n + orow, swiglu_f32(pa, pb));
                else if (MODE == 2)
                    static_cast<float *>(a.y)[static_cast<size_t>(seg_begin + m) * a.n + orow] = swiglu_f32(pa, pb);
                else
                    out_ptr[m][orow] = pa * route_w[m];
            }
            pbuf ^= 1;
        }
    }
}

}  // namespace b200q
