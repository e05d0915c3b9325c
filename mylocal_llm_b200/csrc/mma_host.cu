// Host-side planning and launch of the tensor-core GEMV (mma_gemv.cuh).
#include <cstdlib>
#include <cstring>

#include "mma_gemv.cuh"
#include "mma_host.h"

namespace b200q {

using MmaKernelFn = void (*)(const MmaArgs);
MmaKernelFn mma_pick_single(int mode, int fmt, int nterms);
MmaKernelFn mma_pick_dual(int mode, int fmt, int nterms);

static int round_up(int v, int a) { return (v + a - 1) / a * a; }

// Row-slot pitch: room for the 16-byte aligned window of a segment, and an odd number of 16-byte
// units so that the eight rows a warp reads at once fall into different shared-memory banks.
static int slot_pitch(int seg_bytes) {
    int p = round_up(seg_bytes + 30, 16);
    if ((p / 16) % 2 == 0) p += 16;
    return p;
}

// Worst number of lanes of one 32-bit shared-memory load that fall on the same bank when eight
// rows `row_bytes` apart are read at the same column (four consecutive words per row).
static int bank_conflict_degree(int row_bytes) {
    int hits[32] = {0};
    for (int g = 0; g < 8; ++g)
        for (int t = 0; t < 4; ++t) ++hits[((static_cast<long long>(g) * row_bytes) / 4 + t) & 31];
    int worst = 0;
    for (int b = 0; b < 32; ++b) worst = hits[b] > worst ? hits[b] : worst;
    return worst;
}

static bool plan(MmaArgs &a, int fmt_a, int fmt_b, bool dual, int cw) {
    int kp = 1;
    while (kp * 2 <= cw && kp * 2 * 256 <= a.k) kp *= 2;
    a.cw = cw;
    a.kp = kp;
    a.rg = cw / kp;
    a.seg_a = kp * 256 / fmt_elems(fmt_a) * fmt_bytes(fmt_a);
    a.seg_b = dual ? kp * 256 / fmt_elems(fmt_b) * fmt_bytes(fmt_b) : 0;
    // One copy per tile when the tile spans whole rows and the natural row stride spreads the
    // rows over the banks; otherwise one copy per row into padded slots.
    a.contig = (kp * 256 >= a.k && bank_conflict_degree(a.rb_a) <= 2 &&
                (!dual || bank_conflict_degree(a.rb_b) <= 2)) ? 1 : 0;
    int region_b = 0;
    if (a.contig) {
        a.pitch_a = a.rb_a;
        a.region_a = (16 * a.rg * a.rb_a + 32 + 15) / 16 * 16;
        a.pitch_b = dual ? a.rb_b : 0;
        if (dual) region_b = (16 * a.rg * a.rb_b + 32 + 15) / 16 * 16;
    } else {
        a.pitch_a = slot_pitch(a.seg_a);
        a.region_a = 16 * a.rg * a.pitch_a;
        a.pitch_b = 0;
        if (dual) {
            a.pitch_b = slot_pitch(a.seg_b);
            region_b = 16 * a.rg * a.pitch_b;
        }
    }
    a.stage_bytes = a.region_a + region_b;
    a.off_bfrag = MM_CTRL_BYTES + MM_STAB_BYTES + MM_PART_BYTES;
    const long long bfrag_bytes = static_cast<long long>(a.nterms) * (a.k / 16) * 256;
    const long long xsum_bytes = a.k;  // (k/32) chunks x 8 tokens x 4 bytes
    const long long off_stage = round_up(static_cast<int>(a.off_bfrag + bfrag_bytes + xsum_bytes), 128);
    if (off_stage + 2LL * a.stage_bytes > MM_SMEM_LIMIT) return false;
    a.off_xsum = static_cast<int>(a.off_bfrag + bfrag_bytes);
    a.off_stage = static_cast<int>(off_stage);
    int stages = static_cast<int>((MM_SMEM_LIMIT - off_stage) / a.stage_bytes);
    a.stages = stages > MM_MAX_STAGES ? MM_MAX_STAGES : stages;
    return true;
}

static bool direct_allowed() {
    const char *v = std::getenv("B200Q_KERNEL");
    return !(v && std::strcmp(v, "staged") == 0);
}

int mma_tokens_per_pass(int fmt, int mode, int k, int x_dtype, bool tiled) {
    return (direct_allowed() || tiled) ? direct_tokens_per_pass(fmt, mode, k, x_dtype) : 8;
}

int mma_try_launch(const MmaRequest &q, cudaStream_t stream, bool *launched) {
    *launched = false;
    if (fmt_lanes_only(q.fmt_a) || fmt_lanes_only(q.fmt_b)) return B200Q_OK;    // FP32-lane kernels only
    if (direct_allowed() || q.tiled) {
        int rc = direct_try_launch(q, stream, launched);
        if (rc || *launched) return rc;
    }
    if (q.tiled) return B200Q_OK;       // only the direct kernel reads the tile layout
    const bool dual = (q.mode == 1 || q.mode == 2);
    const bool grouped = q.mode >= 2;
    if (q.k % 256 != 0 || q.k > 65536) return B200Q_OK;
    if (dual && q.fmt_a != q.fmt_b) return B200Q_OK;
    if (reinterpret_cast<uintptr_t>(q.wa) & 15) return B200Q_OK;
    if (dual && (reinterpret_cast<uintptr_t>(q.wb) & 15)) return B200Q_OK;
    if (grouped && !q.table_a && ((q.stride_a & 15) || (dual && (q.stride_b & 15)))) return B200Q_OK;
    if (grouped && q.table_a && !q.tables_aligned16) return B200Q_OK;
    if (q.m > 8) return B200Q_OK;

    MmaArgs a{};
    a.wa = q.wa; a.wb = q.wb;
    a.stride_a = q.stride_a; a.stride_b = q.stride_b;
    a.table_a = q.table_a; a.table_b = q.table_b;
    a.rb_a = q.k / fmt_elems(q.fmt_a) * fmt_bytes(q.fmt_a);
    a.rb_b = dual ? q.k / fmt_elems(q.fmt_b) * fmt_bytes(q.fmt_b) : 0;
    a.n = q.n; a.k = q.k; a.m = q.m;
    a.nterms = (q.x_dtype == B200Q_F32) ? 2 : 1;
    a.x = q.x; a.x_dtype = q.x_dtype; a.y = q.y; a.y_dtype = q.y_dtype;
    a.topk = q.topk; a.order = q.order; a.seg_expert = q.seg_expert; a.seg_begin = q.seg_begin;
    a.seg_count = q.seg_count; a.num_segments = q.num_segments; a.max_segments = q.max_segments;
    a.route = q.route; a.flat_rows = q.flat_rows; a.y_table = q.y_table; a.rows_per_rank = q.rows_per_rank; a.status = q.status;
    if (!plan(a, q.fmt_a, q.fmt_b, dual, MM_WARPS) && !plan(a, q.fmt_a, q.fmt_b, dual, MM_WARPS / 2)) return B200Q_OK;

    MmaKernelFn fn = dual ? mma_pick_dual(q.mode, q.fmt_a, a.nterms) : mma_pick_single(q.mode, q.fmt_a, a.nterms);
    if (!fn) return B200Q_OK;
    const int smem = a.off_stage + a.stages * a.stage_bytes;
    cudaError_t err = cudaFuncSetAttribute(reinterpret_cast<const void *>(fn),
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, MM_SMEM_LIMIT);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "mma gemv: shared memory opt-in failed: %s", cudaGetErrorString(err));
    }
    int grid = sm_count();
    if (!grouped) {
        const int blocks = (q.n + 16 * a.rg - 1) / (16 * a.rg);
        if (blocks < grid) grid = blocks;
    }
    fn<<<grid, MM_THREADS, smem, stream>>>(a);
    *launched = true;
    return check_launch("mma gemv");
}

}  // namespace b200q
