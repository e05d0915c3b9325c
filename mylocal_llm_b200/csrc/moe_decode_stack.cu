// One-token decode step of a stack of packed MoE layers as ONE persistent kernel (sm_100a).
//
// The step of a layer is a chain of short stages - router logits, top-k + routing plan, grouped gate/up,
// grouped down, ordered combine + residual add + RMSNorm (mini_llm/external/cuda_graph_decode.py:379-449 runs
// the same chain as separate launches; so do the entry points b200q_router_logits_t,
// b200q_router_topk_plan_row, b200q_moe_gate_up, b200q_moe_down, b200q_moe_combine_norm). With one token
// every stage is a few microseconds of dependent loads, and a launch boundary costs as much as the stage.
// Here one cooperative grid (one CTA per SM, all co-resident) walks all stages of all layers:
//
//   per layer   A  every warp of the grid takes router rows: logits[e] = x . W[e]        -> grid barrier
//               B  every CTA runs the top-k and builds the one-row routing plan in its own shared memory
//                  (identical in every CTA: no exchange needed)
//               C  grouped gate/up + SwiGLU  (mma_direct_body, the kernel's own split of the work) -> grid barrier
//               D  grouped down, route-weighted (tiled_body)                              -> grid barrier
//               E  every CTA combines the k+1 terms in order, adds the residual and normalises for the next
//                  layer, keeping the residual stream and the activations in its shared memory
//
// The stages are the device functions the separate kernels are made of, called with the same arguments and
// the same grid size, so the step returns the same bits as the chain of launches. The grid barrier is an
// arrival counter and a generation word in global memory; every wait is bounded (GRID_WAIT_NS): a CTA that
// gives up sets the abort word and the status code, and all CTAs leave the kernel.
#include "q6k_tiled.cuh"
#include "router_device.cuh"
#include "norm_device.cuh"
#include "mma_host.h"

#include <cstdlib>
#include <mutex>

namespace b200q {

constexpr int STATUS_GRID_WAIT = 401;          // a CTA gave up waiting at the grid barrier of the persistent step
constexpr uint64_t GRID_WAIT_NS = 1000000000ull;
constexpr int DS_THREADS = 512;
static_assert(DS_THREADS == MD_THREADS && DS_THREADS == Q6T_THREADS, "the stage bodies expect 512 threads");
constexpr int DS_MAX_TERMS = 16;               // k + 1 <= 16: combine_norm_row<16>
constexpr int DS_PLAN_SLOTS = 64;              // entries reserved per per-row plan array

struct DecodeStackLayer {                      // one per layer, in device memory (five 8-byte pointers)
    const float *router_wt;                    // [E, D] FP32, expert-major
    const unsigned long long *gate_table, *up_table, *down_table;      // E + 1 addresses each
    const void *gamma_next;                    // weight of the norm that follows the layer
};

struct DecodeStackArgs {
    const DecodeStackLayer *layers;
    int n_layers;
    int d, f, e, k;
    int renorm;
    float floor_value;
    const void *gamma0;
    int act_dtype;
    float eps;
    const float *residual_in;
    float *residual_out;
    void *hidden_out;
    float *logits, *hbuf, *terms;              // [e], [(k+1) f], [(k+1) d]
    unsigned int *sync;                        // [0] arrivals, [1] generation, [2] abort
    unsigned long long *stamps;                // optional: nine %globaltimer readings of the last layer (CTA 1)
    int *status;
    int max_segments;
    int off_state;                             // byte offset of the per-CTA state in dynamic shared memory
    DirectArgs gu;
    Q6TiledArgs dn;
};

__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// All CTAs of the (co-resident) grid meet here; writes made before it are visible after it. Returns false
// when the step is being abandoned (this CTA's wait ran out, or another CTA's did).
__device__ __forceinline__ bool grid_barrier(unsigned int *words, unsigned int &generation, int nblocks, int *status,
                                             volatile int *abort_smem) {
    __syncthreads();
    if (threadIdx.x == 0) {
        bool ok = true;
        __threadfence();
        const unsigned int arrived = atomicAdd(&words[0], 1u);
        if (arrived == static_cast<unsigned int>(nblocks) - 1u) {
            atomicExch(&words[0], 0u);
            __threadfence();
            atomicAdd(&words[1], 1u);
        } else {
            const uint64_t t0 = global_timer_ns();
            while (ld_acquire_u32(&words[1]) == generation) {
                if (ld_acquire_u32(&words[2]) != 0u) { ok = false; break; }
                if (global_timer_ns() - t0 > GRID_WAIT_NS) {
                    atomicExch(status, STATUS_GRID_WAIT);
                    atomicExch(&words[2], 1u);
                    ok = false;
                    break;
                }
            }
        }
        if (!ok) *abort_smem = 1;
    }
    ++generation;
    __syncthreads();
    return *abort_smem == 0;
}

// The small stages are separate functions (not inlined): each gets its own register allocation, so the two
// grouped stages keep the allocation they have as kernels of their own.
__device__ __noinline__ void stage_first_norm(int tid, const float *resid, const void *gamma, int act_dtype, int d, float eps,
                                              void *x_act) {
    rmsnorm_row<false>(0, tid, resid, B200Q_F32, nullptr, 0.f, gamma, act_dtype, d, eps, nullptr, x_act, act_dtype);
}

__device__ __noinline__ void stage_topk(int lane, const float *logits, int e, int k, int renorm, float floor_value,
                                        float *weights, int64_t *ids, const RowPlanOut *plan) {
    if (e <= 512) topk_plan_warp<16>(lane, logits, e, k, renorm, floor_value, e, 1.0f, weights, ids, *plan);
    else topk_plan_warp<32>(lane, logits, e, k, renorm, floor_value, e, 1.0f, weights, ids, *plan);
}

// Ordered combine + residual add + RMSNorm of the single row, all DS_THREADS threads: the arithmetic of
// combine_norm_row (terms added in ascending plan position with plain FP32 adds, the branch rounded to the
// activation type, the sum of squares of thread t over columns t, t + 256, ... in ascending order, the same
// reduction tree). Every load of a thread is requested before its first add (one asm block per four terms): left
// to the compiler the loads were issued one by one next to their adds, and one L2 round trip (~0.3 us) per term
// made this stage 13 us; the single warp of the top-k gets its logits through shared memory for the same reason.
__device__ __noinline__ void stage_combine_norm(int tid, const float *terms, const int32_t *inv, int k_out, int d,
                                                int act_dtype, float *resid, const void *gamma, float eps, void *x_act) {
    __shared__ int pos_sorted[DS_MAX_TERMS];
    __shared__ float warp_sums[8];
    __shared__ float inv_shared;
    const int lane = tid & 31, warp = tid >> 5;
    if (tid < k_out) {
        const int p = inv[tid];
        int r = 0;
        for (int j = 0; j < k_out; ++j) r += inv[j] < p;
        pos_sorted[r] = p;
    }
    __syncthreads();
    // four consecutive columns per thread: k_out 16-byte loads in flight, then the ordered adds (which thread
    // forms a column's sum does not matter; the sum of squares below keeps combine_norm_row's ownership)
#pragma unroll 1
    for (int c0 = 4 * tid; c0 < d; c0 += 4 * DS_THREADS) {
        float4 t[DS_MAX_TERMS];
        // (all requests leave before the first add; rows past k_out repeat the last term and are not added)
#pragma unroll
        for (int r = 0; r < DS_MAX_TERMS; r += 4) {
            const float *p0 = terms + static_cast<size_t>(pos_sorted[min(r, k_out - 1)]) * d + c0;
            const float *p1 = terms + static_cast<size_t>(pos_sorted[min(r + 1, k_out - 1)]) * d + c0;
            const float *p2 = terms + static_cast<size_t>(pos_sorted[min(r + 2, k_out - 1)]) * d + c0;
            const float *p3 = terms + static_cast<size_t>(pos_sorted[min(r + 3, k_out - 1)]) * d + c0;
            asm volatile(
                "ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%16];\n\t"
                "ld.global.cg.v4.f32 {%4,%5,%6,%7}, [%17];\n\t"
                "ld.global.cg.v4.f32 {%8,%9,%10,%11}, [%18];\n\t"
                "ld.global.cg.v4.f32 {%12,%13,%14,%15}, [%19];"
                : "=f"(t[r].x), "=f"(t[r].y), "=f"(t[r].z), "=f"(t[r].w), "=f"(t[r + 1].x), "=f"(t[r + 1].y),
                  "=f"(t[r + 1].z), "=f"(t[r + 1].w), "=f"(t[r + 2].x), "=f"(t[r + 2].y), "=f"(t[r + 2].z),
                  "=f"(t[r + 2].w), "=f"(t[r + 3].x), "=f"(t[r + 3].y), "=f"(t[r + 3].z), "=f"(t[r + 3].w)
                : "l"(p0), "l"(p1), "l"(p2), "l"(p3)
                : "memory");
        }
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < DS_MAX_TERMS; ++r)
            if (r < k_out) {
                acc[0] = __fadd_rn(acc[0], t[r].x);
                acc[1] = __fadd_rn(acc[1], t[r].y);
                acc[2] = __fadd_rn(acc[2], t[r].z);
                acc[3] = __fadd_rn(acc[3], t[r].w);
            }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v = round_through(act_dtype, acc[j]);
            v = resid[c0 + j] + 1.0f * v;
            resid[c0 + j] = v;
        }
    }
    __syncthreads();
    if (tid < ROW_THREADS) {
        float ss = 0.f;
#pragma unroll 1
        for (int c = tid; c < d; c += ROW_THREADS) {
            const float v = resid[c];
            ss += v * v;
        }
        ss = warp_sum(ss);
        if (lane == 0) warp_sums[warp] = ss;
    }
    __syncthreads();
    if (warp == 0) {
        float t = lane < 8 ? warp_sums[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) inv_shared = __fdiv_rn(1.0f, __fsqrt_rn(__fdiv_rn(t, static_cast<float>(d)) + eps));
    }
    __syncthreads();
    const float inv_rms = inv_shared;
#pragma unroll 1
    for (int c0 = 4 * tid; c0 < d; c0 += 4 * DS_THREADS) {          // 16-bit norm weights: four per 8-byte load
        const uint2 g = *reinterpret_cast<const uint2 *>(static_cast<const uint16_t *>(gamma) + c0);
        const uint32_t bits[4] = {g.x & 0xffffu, g.x >> 16, g.y & 0xffffu, g.y >> 16};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float gv = act_dtype == B200Q_BF16 ? __uint_as_float(bits[j] << 16) : half_bits_to_float(bits[j]);
            store_from_float(x_act, act_dtype, c0 + j, (resid[c0 + j] * inv_rms) * gv);
        }
    }
}

// Router logits of one token: a warp per expert row, the arithmetic of router_logits_t_kernel.
__device__ __noinline__ void stage_router(int first_row, int row_step, int lane, int e, int d, const float *wt,
                                          const float *xs, float *logits) {
    for (int row = first_row; row < e; row += row_step) {
        float acc = 0.f;
        for (int c0 = 0; c0 < d; c0 += 2048) {
            float4 w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int col = c0 + i * 128 + lane * 4;
                w[i] = col < d ? *reinterpret_cast<const float4 *>(wt + static_cast<size_t>(row) * d + col)
                               : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int col = c0 + i * 128 + lane * 4;
                if (col < d) {
                    const float4 xv = *reinterpret_cast<const float4 *>(xs + col);
                    s = fmaf(w[i].x, xv.x, s);
                    s = fmaf(w[i].y, xv.y, s);
                    s = fmaf(w[i].z, xv.z, s);
                    s = fmaf(w[i].w, xv.w, s);
                }
            }
            acc += s;
        }
        const float s = warp_sum(acc);
        if (lane == 0) logits[row] = s + 0.f;
    }
}

__global__ void __launch_bounds__(DS_THREADS, 1) moe_decode_stack_kernel(const DecodeStackArgs p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int abort_flag;
    __shared__ StagePointers gu_ptrs, dn_ptrs;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int block = blockIdx.x, nblocks = gridDim.x;
    const int d = p.d, e = p.e, k_out = p.k + 1;

    // per-CTA state behind the stage bodies' shared memory
    uint8_t *st = smem + p.off_state;
    float *xs = reinterpret_cast<float *>(st);                          // normalised activations as FP32 [d]
    uint8_t *x_act = st + static_cast<size_t>(d) * 4;                   // the same in the activation type [d]
    float *resid = reinterpret_cast<float *>(st + static_cast<size_t>(d) * 8);      // residual stream [d]
    int64_t *ids = reinterpret_cast<int64_t *>(st + static_cast<size_t>(d) * 12);      // [k + 1]; d * 12 is a multiple of 8
    float *weights = reinterpret_cast<float *>(ids + DS_PLAN_SLOTS);    // [k + 1]
    int32_t *order = reinterpret_cast<int32_t *>(weights + DS_PLAN_SLOTS);
    int32_t *inv = order + DS_PLAN_SLOTS;
    int32_t *seg_expert = inv + DS_PLAN_SLOTS;
    int32_t *seg_begin = seg_expert + DS_PLAN_SLOTS;
    int32_t *seg_count = seg_begin + DS_PLAN_SLOTS;
    int32_t *num_segments = seg_count + DS_PLAN_SLOTS;                  // [1] (+ the plan's status word)
    float *logit_s = reinterpret_cast<float *>(num_segments + 2);       // [e] the row's logits
    // The selected experts' matrix addresses, per segment: fetched once per layer right after the top-k, so the
    // stage bodies (given the identity as their segment -> expert map and these as their pointer tables) do not
    // start with a dependent look-up in global memory.
    __shared__ unsigned long long gate_ptrs[DS_PLAN_SLOTS], up_ptrs[DS_PLAN_SLOTS], down_ptrs[DS_PLAN_SLOTS];
    __shared__ int32_t seg_ident[DS_PLAN_SLOTS];

    if (tid == 0) abort_flag = 0;
    unsigned int generation = 0;                                         // the host zeroes the words before the launch
    for (int c = tid; c < d; c += DS_THREADS) resid[c] = p.residual_in[c];
    __syncthreads();
    if (tid < ROW_THREADS)
        stage_first_norm(tid, resid, p.gamma0, p.act_dtype, d, p.eps, x_act);
    __syncthreads();

    if (tid == 0) {
        gu_ptrs = StagePointers{x_act, p.hbuf, gate_ptrs, up_ptrs, order, seg_ident, seg_begin, seg_count, num_segments, nullptr, 0};
        dn_ptrs = StagePointers{p.hbuf, p.terms, down_ptrs, nullptr, order, seg_ident, seg_begin, seg_count, num_segments, weights, -1};
    }
    if (tid < DS_PLAN_SLOTS) seg_ident[tid] = tid;
    __syncthreads();
    const RowPlanOut plan{nullptr, nullptr, order, inv, seg_expert, seg_begin, seg_count, num_segments, num_segments + 1,
                          e + 1, p.max_segments};
    bool ok = true;
    for (int layer = 0; layer < p.n_layers && ok; ++layer) {
        const DecodeStackLayer lay = p.layers[layer];
        // diagnostic (B200Q_STAGE_TIMES=1): when the stages of the last layer ended on CTA 1 (which has a block in
        // both grouped stages of a one-row plan), in nanoseconds
        unsigned long long *stamp = (p.stamps && block == min(1, nblocks - 1) && tid == 0 && layer == p.n_layers - 1) ? p.stamps : nullptr;
        if (stamp) stamp[0] = global_timer_ns();
        // A: router logits; a warp per expert row, the arithmetic of router_logits_t_kernel for one token
        for (int c = tid; c < d; c += DS_THREADS) xs[c] = load_as_float(x_act, p.act_dtype, c);
        __syncthreads();
        stage_router(block * (DS_THREADS / 32) + warp, nblocks * (DS_THREADS / 32), lane, e, d, lay.router_wt, xs, p.logits);
        if (stamp) stamp[1] = global_timer_ns();
        if (!(ok = grid_barrier(p.sync, generation, nblocks, p.status, &abort_flag))) break;
        if (stamp) stamp[2] = global_timer_ns();

        // B: top-k and the one-row plan, in every CTA
        // (every thread fetches a logit or two into shared memory: one round trip instead of the lane's sixteen)
        for (int i = tid; i < e; i += DS_THREADS) logit_s[i] = __ldcg(p.logits + i);
        __syncthreads();
        if (warp == 0) {
            stage_topk(lane, logit_s, e, p.k, p.renorm, p.floor_value, weights, ids, &plan);
            __syncwarp();
            const int nseg = min(num_segments[0], p.max_segments);
            for (int u = lane; u < nseg; u += 32) {
                const int ex = seg_expert[u];
                gate_ptrs[u] = lay.gate_table[ex];
                up_ptrs[u] = lay.up_table[ex];
                down_ptrs[u] = lay.down_table[ex];
            }
        } else {
            // meanwhile the other fifteen warps turn the row into the gate/up stage's activation fragments (the
            // stage's own preparation, run by 480 threads; the stage finds its single row prepared and skips it)
            prepare_direct<1, 2, DS_THREADS - 32, 13>([](int) { return 0; }, 1, d, x_act, p.act_dtype,
                                                      reinterpret_cast<uint2 *>(smem + p.gu.off_bfrag),
                                                      reinterpret_cast<uint32_t *>(smem + p.gu.off_xsfrag),
                                                      reinterpret_cast<float *>(smem), tid - 32);
        }
        __syncthreads();
        // (L2 prefetches issued here - the next layer's router rows, this CTA's down tiles - cost this stage more
        // than they saved the later ones: 1.1 us against 0.4 us, measured with the stage stamps)
        if (stamp) stamp[3] = global_timer_ns();
        // C: grouped gate/up + SwiGLU -> hbuf
        mma_direct_body<false, 2, 1, 1>(p.gu, gu_ptrs, smem, block, nblocks);
        if (stamp) stamp[4] = global_timer_ns();
        if (!(ok = grid_barrier(p.sync, generation, nblocks, p.status, &abort_flag))) break;
        if (stamp) stamp[5] = global_timer_ns();

        // D: grouped down, route-weighted -> terms
        tiled_body<Q6Tile, 3, 2, 1>(p.dn, dn_ptrs, smem, block, nblocks);
        if (stamp) stamp[6] = global_timer_ns();
        if (!(ok = grid_barrier(p.sync, generation, nblocks, p.status, &abort_flag))) break;
        if (stamp) stamp[7] = global_timer_ns();

        // E: ordered combine + residual add + norm of the next layer, in every CTA
        stage_combine_norm(tid, p.terms, inv, k_out, d, p.act_dtype, resid, lay.gamma_next, p.eps, x_act);
        __syncthreads();
        if (stamp) stamp[8] = global_timer_ns();
    }
    if (ok && block == 0) {
        const int esize = p.act_dtype == B200Q_F32 ? 4 : 2;
        for (int c = tid; c < d; c += DS_THREADS) p.residual_out[c] = resid[c];
        for (int c = tid; c < d * esize; c += DS_THREADS) static_cast<uint8_t *>(p.hidden_out)[c] = x_act[c];
    }
}

// Bytes of per-CTA state behind the stage bodies' shared memory (layout in the kernel).
static long long decode_state_bytes(int d, int e) {
    return static_cast<long long>(d) * 12 + DS_PLAN_SLOTS * 8 + DS_PLAN_SLOTS * 4 * 6 + 8 + (2LL * e + 3) * 4 + 64;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace b200q

using namespace b200q;

extern "C" long long b200q_moe_decode_stack_workspace(int d, int f, int e, int k) {
    if (d <= 0 || f <= 0 || e <= 0 || k <= 0) return 0;
    return static_cast<long long>(align_up(static_cast<size_t>(e) * 4, 256) + align_up(static_cast<size_t>(k + 1) * f * 4, 256) +
                                  align_up(static_cast<size_t>(k + 1) * d * 4, 256) + 256);
}

extern "C" int b200q_moe_decode_stack(const void *layers, int n_layers, int d, int f, int e, int k, int renormalize,
                                      float floor_value, int gate_up_fmt, int down_fmt, const void *gamma0,
                                      int act_dtype, float eps, const float *residual_in, float *residual_out,
                                      void *hidden_out, void *workspace, long long workspace_bytes, void *stream) {
    if (!layers || !gamma0 || !residual_in || !residual_out || !hidden_out || !workspace)
        return fail(B200Q_EINVAL, "moe_decode_stack: NULL pointer");
    if (n_layers < 1 || d <= 0 || f <= 0 || e <= 0 || k <= 0 || k > e)
        return fail(B200Q_EINVAL, "moe_decode_stack: bad shape layers=%d d=%d f=%d e=%d k=%d", n_layers, d, f, e, k);
    if (renormalize && !(floor_value > 0.0f)) return fail(B200Q_EINVAL, "moe_decode_stack: floor must be positive");
    if ((gate_up_fmt != B200Q_Q4_K && gate_up_fmt != B200Q_Q4_K_TILED) || down_fmt != B200Q_Q6_K_TILED ||
        (act_dtype != B200Q_BF16 && act_dtype != B200Q_F16))
        return fail(B200Q_EUNSUPPORTED, "moe_decode_stack: Q4_K gate/up, tiled Q6_K down, 16-bit activations only");
    if (e > 1024 || k > 31 || k + 1 > DS_MAX_TERMS || d % 256 != 0 || f % 256 != 0)
        return fail(B200Q_EUNSUPPORTED, "moe_decode_stack: needs e <= 1024, k <= 15, d and f multiples of 256");
    if (workspace_bytes < b200q_moe_decode_stack_workspace(d, f, e, k) || (reinterpret_cast<uintptr_t>(workspace) & 255))
        return fail(B200Q_EINVAL, "moe_decode_stack: workspace too small or not 256-byte aligned");
    int *status = device_status_word();
    if (!status) return fail(B200Q_ECUDA, "moe_decode_stack: no CUDA device");
    const int k_out = k + 1;
    const int max_segments = (e + 1 < k_out ? e + 1 : k_out) + k_out / 8;       // the bound of a one-row plan

    // the arguments the two grouped launches would get for this step (same split of the work)
    static const unsigned long long dummy_table[1] = {0};
    MmaRequest q{};
    q.mode = 2; q.fmt_a = q.fmt_b = B200Q_Q4_K; q.tiled = gate_up_fmt == B200Q_Q4_K_TILED;
    q.table_a = q.table_b = dummy_table; q.tables_aligned16 = 1;
    q.n = f; q.k = d; q.m = 8; q.x_dtype = act_dtype; q.y_dtype = B200Q_F32; q.topk = k_out; q.max_segments = max_segments;
    DecodeStackArgs a{};
    long long gu_smem = 0, dn_smem = 0;
    if (!direct_plan_args(q, &a.gu, &gu_smem))
        return fail(B200Q_EUNSUPPORTED, "moe_decode_stack: the gate/up stage does not fit this shape");
    MmaRequest r{};
    r.mode = 3; r.fmt_a = r.fmt_b = B200Q_Q6_K_TILED; r.table_a = dummy_table; r.tables_aligned16 = 1;
    r.n = d; r.k = f; r.m = 8; r.x_dtype = B200Q_F32; r.y_dtype = B200Q_F32; r.topk = 1; r.max_segments = max_segments;
    int rc = tiled_plan_args(r, &a.dn, &dn_smem);
    if (rc) return rc;
    const long long off_state = static_cast<long long>(align_up(static_cast<size_t>(gu_smem > dn_smem ? gu_smem : dn_smem), 128));
    const long long smem = off_state + decode_state_bytes(d, e);
    if (smem > MM_SMEM_LIMIT - 4096) return fail(B200Q_EUNSUPPORTED, "moe_decode_stack: d=%d e=%d need too much shared memory", d, e);

    uint8_t *ws = static_cast<uint8_t *>(workspace);
    a.layers = static_cast<const DecodeStackLayer *>(layers);
    a.n_layers = n_layers;
    a.d = d; a.f = f; a.e = e; a.k = k;
    a.renorm = renormalize ? 1 : 0;
    a.floor_value = floor_value;
    a.gamma0 = gamma0; a.act_dtype = act_dtype; a.eps = eps;
    a.residual_in = residual_in; a.residual_out = residual_out; a.hidden_out = hidden_out;
    a.logits = reinterpret_cast<float *>(ws);
    ws += align_up(static_cast<size_t>(e) * 4, 256);
    a.hbuf = reinterpret_cast<float *>(ws);
    ws += align_up(static_cast<size_t>(k_out) * f * 4, 256);
    a.terms = reinterpret_cast<float *>(ws);
    ws += align_up(static_cast<size_t>(k_out) * d * 4, 256);
    a.sync = reinterpret_cast<unsigned int *>(ws);
    {
        const char *v = std::getenv("B200Q_STAGE_TIMES");
        a.stamps = (v && v[0] == '1') ? reinterpret_cast<unsigned long long *>(ws + 64) : nullptr;      // behind the barrier words
    }
    a.status = status;
    a.max_segments = max_segments;
    a.off_state = static_cast<int>(off_state);

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    {
        // opt in to the dynamic shared memory this step needs (kept per device; raised when a larger step comes)
        static std::mutex mu;
        static long long opted[64] = {0};
        int dev = 0;
        cudaGetDevice(&dev);
        std::lock_guard<std::mutex> lock(mu);
        if (dev >= 0 && dev < 64 && opted[dev] < smem) {
            cudaError_t err = cudaFuncSetAttribute(reinterpret_cast<const void *>(moe_decode_stack_kernel),
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (err != cudaSuccess) {
                cudaGetLastError();
                return fail(B200Q_ECUDA, "moe_decode_stack: shared memory opt-in failed: %s", cudaGetErrorString(err));
            }
            opted[dev] = smem;
        }
    }
    {
        // the whole grid has to be resident at once: one CTA per SM must fit
        int per_sm = 0;
        cudaError_t err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_decode_stack_kernel, DS_THREADS,
                                                                        static_cast<size_t>(smem));
        if (err != cudaSuccess || per_sm < 1) {
            cudaGetLastError();
            return fail(B200Q_EUNSUPPORTED, "moe_decode_stack: a CTA of this step does not fit an SM of this device");
        }
    }
    cudaError_t err = cudaMemsetAsync(a.sync, 0, 16, st);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "moe_decode_stack: %s", cudaGetErrorString(err));
    }
    // cooperative launch: the grid (one CTA per SM, as the separate launches use) is resident as a whole or the
    // launch fails - a CTA at the grid barrier never waits for one that has not started
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(sm_count());
    cfg.blockDim = dim3(DS_THREADS);
    cfg.dynamicSmemBytes = static_cast<size_t>(smem);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    err = cudaLaunchKernelEx(&cfg, moe_decode_stack_kernel, a);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "moe_decode_stack: launch failed: %s", cudaGetErrorString(err));
    }
    return check_launch("moe_decode_stack");
}
