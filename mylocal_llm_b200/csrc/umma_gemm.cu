// Batched / prefill GEMM on packed GGUF weights: y[m, n] = x[m, k] @ W[n, k]^T for m > 16 tokens.
//
// A GEMV pass re-reads the packed matrix once per 8 or 16 tokens; from a few dozen tokens on the
// product is a real contraction and belongs on the 5th-generation tensor cores. The roles are
// swapped with respect to the textbook GEMM: the weight rows are the M dimension of the MMA. One CTA
// owns 128 weight rows x NTOK tokens (NTOK = the batch rounded up to 16, at most 256; one or two
// such token tiles per CTA) and walks K in slabs of 64:
//   * the activation slab [NTOK tokens x 64 k] (BF16) arrives by TMA (cp.async.bulk.tensor.2d,
//     128-byte swizzle, rows beyond m zero-filled by the tensor map);
//   * sixteen decoder warps turn the packed weights of the slab [128 rows x 64 k] into BF16 - the
//     reference's dequantisation (mini_llm/ops/quantized_weight.py:208-250) in FP32, rounded once -
//     and store them in the same 128-byte-swizzled K-major layout; the packed bytes of a 256-wide
//     group are requested a group ahead and wait in registers;
//   * both arrive on the stage's `full` mbarrier (transaction bytes + one arrival per decoder warp);
//     one lane of another warp waits for it and issues tcgen05.mma (kind::f16, M = 128, N = NTOK,
//     K = 16, four per slab and token tile) with both operands described by shared-memory
//     descriptors; the FP32 accumulator [128 x NTOK] lives in tensor memory; tcgen05.commit arrives
//     on the stage's `free` mbarrier when the tensor core has consumed the slab, which lets the
//     decoders and the TMA lane (one more warp) refill it;
//   * after the last slab the decoder warps read the accumulator back with tcgen05.ld (each
//     warp its 32-lane quarter = 32 weight rows), convert and store y (a warp stores 32 consecutive
//     outputs of one token per instruction).
// The MMA-issuing lane never waits for its own commits, so the tensor core always has queued work.
// With a few dozen tokens the kernel is bound by the decoders' instruction issue (~170 warp
// instructions per warp and slab, sixteen warps on four schedulers: ~0.35 us per slab); with 256-token
// tiles the tensor core's time per slab is of the same size and the two overlap.
//
// Paired variant (PAIR, from about a thousand tokens on): CTAs 2p and 2p + 1 are a cluster of two on
// neighbouring SMs and one tensor-core unit (cta_group::2, D = [256 weight rows x NTOK tokens]). Each
// decodes its own 128 rows into its own shared memory and loads half of the token rows; the first CTA's
// `full` barrier collects the decoder arrivals of both CTAs (the second CTA's come as remote arrivals)
// and the bytes of both TMA halves (the second CTA's loads name the first CTA's barrier); the first CTA
// issues the MMAs for both and commits to the `free` and `done` barriers of both; each CTA reads its own
// 128 accumulator rows back. Tensor memory is allocated and freed by warp 0 of both CTAs, with a cluster
// barrier after the allocation and before the release.
// Weights are rounded to BF16, so results carry BF16-weight precision (relative 2^-9 per weight,
// like the BF16 activations this path requires); the GEMV kernels keep their exact-product
// arithmetic for m <= 16 and for FP32 activations.
//
// Every mbarrier wait is bounded (2 s): on expiry the waiting thread records a status code and
// raises the CTA's abort flag; every role then leaves its loop, the copies in flight are waited for
// (bounded), the tensor memory is freed and the CTA returns.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <utility>
#include <vector>

#include "common.cuh"

namespace b200q {

constexpr int UG_BM = 128;          // weight rows per CTA (UMMA M)
constexpr int UG_BK = 64;           // K per slab: 64 BF16 = one 128-byte swizzle row
constexpr int UG_W_BYTES = UG_BM * UG_BK * 2;      // one decoded weight slab
constexpr int STATUS_UMMA_WAIT_TMA = 111;   // gave up waiting for an activation slab
constexpr int STATUS_UMMA_WAIT_MMA = 112;   // gave up waiting for the tensor core to release a stage

struct UmmaGemmArgs {
    const uint8_t *w;
    int n, k, m;
    long long row_bytes;      // packed bytes per weight row (native layouts)
    void *y;
    int y_dtype;
    int ntok;                 // tokens per accumulator (UMMA N): a multiple of 16, 16..256
    int mt;                   // token tiles (accumulators) per CTA: 1 or 2
    int stages;               // shared-memory stages (2..4)
    int *status;
    int groups_per_split;     // 256-position groups of K per CTA along grid.z (split-K); k / 256 without a split
    float *partial;           // split-K: FP32 partial results [grid.z][m][n], summed by splitk_reduce_kernel
};

// ---------------------------------------------------------------------------------------------
// tcgen05 / TMA wrappers (sm_100a)
// ---------------------------------------------------------------------------------------------
// PAIR: the two CTAs of a cluster work as one tensor-core unit (cta_group::2). Tensor memory is then allocated
// and freed by the same warp of both CTAs, with the same shared-memory slot for the address.
template <bool PAIR>
__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t cols) {
    if (PAIR)
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                     "r"(cols)
                     : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                     "r"(cols)
                     : "memory");
}
template <bool PAIR>
__device__ __forceinline__ void tmem_relinquish() {
    if (PAIR) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    else asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <bool PAIR>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// True in exactly one lane of a converged warp. The warps that issue MMAs and TMA loads run their loops with all 32
// lanes and elect the issuer per instruction group: a loop kept inside an `if (lane == 0)` branch is divergent code
// to the compiler, which then feeds every tensor-core / TMA instruction (they take their operands from the warp-wide
// uniform registers) through per-thread registers - the issuing lane spent ~0.55 us per slab that way, whatever
// the tile size.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// Cluster helpers for the paired kernel.
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Every thread of both CTAs; orders shared-memory and barrier initialisation across the pair.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The shared::cluster address of this CTA's shared-memory address `addr` as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Waits of the MMA-issuing lane of a pair: the arrivals come from both CTAs.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint64_t *bar, uint32_t parity, int *status, int code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait_cluster(bar, parity)) return true;
        if (global_timer_ns() - t0 > WAIT_LIMIT_NS) {
            atomicExch(status, code);
            return false;
        }
    }
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]; `accumulate` = 0 overwrites D.
// In a pair (issued by the first CTA only) D is [256 x N]: each CTA's tensor memory holds the 128 rows of its own A
// operand; the N rows of B come half from each CTA's shared memory, at the same offsets.
template <bool PAIR>
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    if (PAIR)
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
}
// The mbarrier (a shared::cluster address: this CTA's or, in a pair, the partner's) receives one arrival when every
// tcgen05.mma issued so far by this thread has completed.
template <bool PAIR>
__device__ __forceinline__ void umma_commit(uint32_t bar_addr) {
    if (PAIR)
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr)
                     : "memory");
    else
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr)
                     : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 2-D tiled TMA load into this CTA's shared memory (no cluster, no multicast); coordinates in
// elements: x = innermost (k), y = row. x * 2 bytes is a multiple of 128 here.
__device__ __forceinline__ void tma_load_2d(void *dst_smem, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// The same load issued by a CTA of a pair: the completion bytes go to the mbarrier at `bar_addr`, a shared::cluster
// address that may lie in the partner CTA (the one that issues the MMAs); the data lands in this CTA.
__device__ __forceinline__ void tma_load_2d_pair(void *dst_smem, const CUtensorMap *map, int x, int y, uint32_t bar_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_addr), "r"(x), "r"(y)
        : "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes (64 BF16)
// with the 128-byte swizzle, groups of eight rows 1024 bytes apart: start address >> 4 in bits
// [0,14), leading byte offset (unused for swizzled K-major, 1) in [16,30), stride byte offset
// 1024 >> 4 in [32,46), descriptor version 1 in [46,48), layout type 2 (128-byte swizzle) in [61,64).
__device__ __forceinline__ uint64_t smem_desc_sw128(const void *tile) {
    const uint64_t addr = (smem_u32(tile) & 0x3ffffu) >> 4;
    return addr | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor of kind::f16: FP32 accumulator (bits [4,6) = 1), A and B BF16 (bits [7,10)
// and [10,13) = 1), both K-major (bits 15, 16 = 0), N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------
// Decoding. A decoder thread owns one weight row of the tile and one 16-position quarter of every
// 64-position slab. It fetches what it needs of a whole 256-position group (a K-quant super-block,
// eight Q8_0 blocks) at once - four 16-byte code pieces, one per slab, plus the group's scales - and
// keeps the next group in a second register set, so global-memory latency never sits on the path of
// a slab. decode_slab<SL> turns the piece of slab SL of the group into 16 FP32 weights with the
// reference's arithmetic: (d*sc)*q - (dmin*mn) for Q4_K / Q5_K, (d*sc)*q for Q6_K, d*q for Q8_0.
// ---------------------------------------------------------------------------------------------
// 16 bytes from an address that is a multiple of 2.
__device__ __forceinline__ uint4 load16(const uint8_t *p) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    uint4 v;
    if ((a & 15) == 0) {
        v = *reinterpret_cast<const uint4 *>(p);
    } else if ((a & 3) == 0) {
        const uint32_t *w = reinterpret_cast<const uint32_t *>(p);
        v = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
        // two bytes past a word boundary: five aligned words, each output word straddles two of them
        const uint32_t *w = reinterpret_cast<const uint32_t *>(p - 2);
        const uint32_t w0 = w[0], w1 = w[1], w2 = w[2], w3 = w[3], w4 = w[4];
        v.x = __funnelshift_r(w0, w1, 16);
        v.y = __funnelshift_r(w1, w2, 16);
        v.z = __funnelshift_r(w2, w3, 16);
        v.w = __funnelshift_r(w3, w4, 16);
    }
    return v;
}

__host__ __device__ constexpr int fmt_group_bytes(int fmt) {        // packed bytes of 256 positions of a row
    return fmt == B200Q_Q8_0 ? 8 * 34 : fmt == B200Q_Q4_K ? 144 : fmt == B200Q_Q5_K ? 176 : 210;
}

struct RawGroup {
    uint4 q[4];   // slab SL's 16 code bytes (Q4_K / Q5_K: nibble bytes; Q6_K: low-nibble bytes; Q8_0: codes)
    uint4 h[2];   // Q5_K: h[0] = high-bit bytes; Q6_K: h[half] = bytes holding the upper two bits
    uint4 hdr;    // Q4_K / Q5_K: d, dmin, 12 scale bytes; Q6_K: .x = 4 scale bytes (one per slab), .y = d;
                  // Q8_0: .x, .y = the four slabs' block scales as FP16 pairs
};

// quart = the thread's quarter (0..3) of a slab; blk = the row's bytes of the group.
template <int FMT>
__device__ __forceinline__ void fetch_group(const uint8_t *blk, int quart, RawGroup &r) {
    if constexpr (FMT == B200Q_Q8_0) {
        // slab SL, quarter quart -> block 2*SL + (quart >> 1), half quart & 1 of its 32 codes
        // The codes start 2 bytes (even blocks) or 0 bytes (odd blocks) past a word boundary: every lane reads five
        // aligned words from the boundary at or below its piece and shifts by its own amount, so the lanes of a
        // warp (which hold blocks of both kinds) stay on one path. The fifth word is needed only by the shifted
        // lanes; the others do not read it (it may lie past the end of the tensor).
        const uint8_t *b = blk + (quart >> 1) * 34;
        uint32_t d[4];
#pragma unroll
        for (int sl = 0; sl < 4; ++sl) {
            d[sl] = *reinterpret_cast<const uint16_t *>(b + 68 * sl);
            const uint8_t *p = b + 68 * sl + 2 + 16 * (quart & 1);
            const uint32_t shift = (static_cast<uint32_t>(reinterpret_cast<uintptr_t>(p)) & 2u) * 8u;   // 0 or 16 bits
            const uint32_t *w = reinterpret_cast<const uint32_t *>(p - (shift >> 3));
            const uint32_t w0 = w[0], w1 = w[1], w2 = w[2], w3 = w[3], w4 = shift ? w[4] : 0u;
            r.q[sl] = make_uint4(__funnelshift_r(w0, w1, shift), __funnelshift_r(w1, w2, shift),
                                 __funnelshift_r(w2, w3, shift), __funnelshift_r(w3, w4, shift));
        }
        r.hdr.x = d[0] | (d[1] << 16);
        r.hdr.y = d[2] | (d[3] << 16);
        return;
    }
    if constexpr (FMT == B200Q_Q4_K || FMT == B200Q_Q5_K) {
        // slab SL, quarter quart -> sub-block 2*SL + (quart >> 1), nibble bytes [32*SL + 16*(quart & 1), +16)
        r.hdr = load16(blk);
        const uint8_t *qs = blk + (FMT == B200Q_Q5_K ? 48 : 16) + 16 * (quart & 1);
#pragma unroll
        for (int sl = 0; sl < 4; ++sl) r.q[sl] = load16(qs + 32 * sl);
        if (FMT == B200Q_Q5_K) r.h[0] = load16(blk + 16 + 16 * (quart & 1));
        return;
    } else {
    // Q6_K: slab SL, quarter quart -> position 64*SL + 16*quart: half = SL >> 1, low-nibble bytes
    // [64*half + 16*quart, +16) shifted by 4*(SL & 1), upper bits in bytes [128 + 32*half + 16*(quart & 1), +16)
    // shifted by 2*(2*(SL & 1) + (quart >> 1)), scale 4*SL + quart
#pragma unroll
    for (int sl = 0; sl < 4; sl += 2) r.q[sl] = r.q[sl + 1] = load16(blk + 64 * (sl >> 1) + 16 * quart);
    r.h[0] = load16(blk + 128 + 16 * (quart & 1));
    r.h[1] = load16(blk + 160 + 16 * (quart & 1));
    const uint8_t *sc = blk + 192 + quart;
    r.hdr.x = sc[0] | (static_cast<uint32_t>(sc[4]) << 8) | (static_cast<uint32_t>(sc[8]) << 16) |
              (static_cast<uint32_t>(sc[12]) << 24);
    r.hdr.y = *reinterpret_cast<const uint16_t *>(blk + 208);
    }
}

// Packed FP32 pairs (sm_100: one instruction for two IEEE operations, each rounded as the scalar one): the
// decoders are bound by the number of instructions they issue, and these halve their floating-point part.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// Bytes j and j + 1 of `codes` as floats minus `bias` (each byte becomes the low mantissa byte of 2^23: exact).
__device__ __forceinline__ uint64_t bytes_to_float2(uint32_t codes, int j, uint64_t neg_bias2) {
    const float lo = __uint_as_float(__byte_perm(codes, 0x4B000000u, 0x7650u | static_cast<uint32_t>(j)));
    const float hi = __uint_as_float(__byte_perm(codes, 0x4B000000u, 0x7650u | static_cast<uint32_t>(j + 1)));
    return add2(pack2(lo, hi), neg_bias2);
}

// out[p] = weights 2p, 2p + 1 of the piece as a packed FP32 pair.
template <int FMT, int SL>
__device__ __forceinline__ void decode_slab(const RawGroup &r, int quart, uint64_t (&out)[8]) {
    const uint32_t qw[4] = {r.q[SL].x, r.q[SL].y, r.q[SL].z, r.q[SL].w};
    if constexpr (FMT == B200Q_Q8_0) {
        const float d = half_bits_to_float(((SL < 2 ? r.hdr.x : r.hdr.y) >> (16 * (SL & 1))) & 0xffffu);
        const uint64_t d2 = pack2(d, d), nb = pack2(-8388736.0f, -8388736.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t u = qw[i] ^ 0x80808080u;              // code + 128 in every byte
            out[2 * i] = mul2(d2, bytes_to_float2(u, 0, nb));
            out[2 * i + 1] = mul2(d2, bytes_to_float2(u, 2, nb));
        }
        return;
    }
    if constexpr (FMT == B200Q_Q4_K || FMT == B200Q_Q5_K) {
        const int hi_sub = quart >> 1;                           // sub-block g = 2*SL + hi_sub
        const float d = half_bits_to_float(r.hdr.x & 0xffffu), dmin = half_bits_to_float(r.hdr.x >> 16);
        uint32_t sc, mn;
        if (SL < 2) {                                            // g < 4: low six bits of bytes g and 4 + g
            const int sh = 16 * SL + 8 * hi_sub;
            sc = (r.hdr.y >> sh) & 63u;
            mn = (r.hdr.z >> sh) & 63u;
        } else {                                                 // g >= 4: nibbles of byte 4 + g, top bits of bytes g - 4, g
            const int sh = 16 * (SL - 2) + 8 * hi_sub;
            const uint32_t hi = (r.hdr.w >> sh) & 0xffu;
            sc = (hi & 15u) | (((r.hdr.y >> sh) >> 2) & 48u);
            mn = (hi >> 4) | (((r.hdr.z >> sh) >> 2) & 48u);
        }
        const float scale = d * static_cast<float>(sc), neg_min = -(dmin * static_cast<float>(mn));
        const uint32_t hw[4] = {r.h[0].x, r.h[0].y, r.h[0].z, r.h[0].w};
        const int shift = 4 * hi_sub, g = 2 * SL + hi_sub;
        const uint64_t scale2 = pack2(scale, scale), min2 = pack2(neg_min, neg_min), nb = pack2(-8388608.0f, -8388608.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t code = (qw[i] >> shift) & 0x0f0f0f0fu;
            if (FMT == B200Q_Q5_K) code |= ((hw[i] >> g) & 0x01010101u) << 4;
            out[2 * i] = fma2(scale2, bytes_to_float2(code, 0, nb), min2);
            out[2 * i + 1] = fma2(scale2, bytes_to_float2(code, 2, nb), min2);
        }
        return;
    }
    // Q6_K
    const float scale = half_bits_to_float(r.hdr.y) *
                        static_cast<float>(static_cast<int>(static_cast<int8_t>((r.hdr.x >> (8 * SL)) & 0xffu)));
    const uint4 hv = r.h[SL >> 1];
    const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
    const int lo_shift = 4 * (SL & 1), hi_shift = 2 * (2 * (SL & 1) + (quart >> 1));
    const uint64_t scale2 = pack2(scale, scale), nb = pack2(-8388640.0f, -8388640.0f);          // code - 32
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t code = ((qw[i] >> lo_shift) & 0x0f0f0f0fu) | (((hw[i] >> hi_shift) & 0x03030303u) << 4);
        out[2 * i] = mul2(scale2, bytes_to_float2(code, 0, nb));
        out[2 * i + 1] = mul2(scale2, bytes_to_float2(code, 2, nb));
    }
}

__device__ __forceinline__ uint32_t pack_bf16(uint64_t pair) {
    float lo, hi;
    unpack2(pair, lo, hi);
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// One output y[t, col] from FP32 register bits.
__device__ __forceinline__ void store_out(void *yv, int y_dtype, size_t idx, uint32_t bits) {
    const float v = __uint_as_float(bits);
    if (y_dtype == B200Q_F32) static_cast<float *>(yv)[idx] = v;
    else if (y_dtype == B200Q_BF16) static_cast<__nv_bfloat16 *>(yv)[idx] = __float2bfloat16_rn(v);
    else static_cast<__half *>(yv)[idx] = __float2half_rn(v);
}

// The weight ring as a decoder thread sees it.
struct DecoderRing {
    uint8_t *base;            // stage 0 of the ring (a stage's decoded weight slab comes first)
    uint64_t *free_bar, *full_bar;
    volatile int *abort_flag;
    int *status;
    int stage_bytes, stages;
    int stage, wraps;         // stage of the next slab, and how many times the ring has wrapped
    uint32_t remote_full;     // second CTA of a pair: shared::cluster address of the first CTA's full_bar[0]; else 0
};

// Waits until the tensor core has released stage `stage` for its `wraps`-th reuse. The CTA's abort flag is read
// only when the stage is not free at once; false = this thread or another one gave up.
__device__ __forceinline__ bool ring_wait_free(const DecoderRing &ring, int stage, int wraps) {
    if (wraps == 0 || mbar_try_wait(&ring.free_bar[stage], (wraps - 1) & 1)) return true;
    if (*ring.abort_flag) return false;
    if (mbar_wait_bounded(&ring.free_bar[stage], (wraps - 1) & 1, ring.status, STATUS_UMMA_WAIT_MMA)) return true;
    *ring.abort_flag = 1;
    return false;
}

// The pieces of slab SL of the groups in `grp`, decoded and stored into `stage` (a 16 KB weight slab of the ring).
template <int FMT, int SL, int PIECES>
__device__ __forceinline__ void decode_into(const RawGroup (&grp)[PIECES], const int (&prow)[PIECES],
                                            const int (&pquart)[PIECES], uint8_t *stage) {
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
        uint64_t wv[8];
        decode_slab<FMT, SL>(grp[j], pquart[j], wv);
        uint8_t *dst_row = stage + (prow[j] >> 3) * 1024 + (prow[j] & 7) * 128;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            uint4 v;
            v.x = pack_bf16(wv[4 * c + 0]);
            v.y = pack_bf16(wv[4 * c + 1]);
            v.z = pack_bf16(wv[4 * c + 2]);
            v.w = pack_bf16(wv[4 * c + 3]);
            const int chunk = (pquart[j] * 2 + c) ^ (prow[j] & 7);         // 128-byte swizzle
            *reinterpret_cast<uint4 *>(dst_row + chunk * 16) = v;
        }
    }
}

// Decode slabs SL and SL + 1 of the groups in `grp` into the ring's next two stages and publish both; false =
// gave up. Two slabs per round: the per-round chain of a warp (wait, scale decode, proxy fence, warp barrier,
// arrival) is paid once for 32 weights per thread, and the two slabs' arithmetic interleaves.
template <int FMT, int SL, int PIECES>
__device__ __forceinline__ bool decode_store_two(const RawGroup (&grp)[PIECES], const int (&prow)[PIECES],
                                                 const int (&pquart)[PIECES], DecoderRing &ring, int lane) {
    const int s0 = ring.stage, w0 = ring.wraps;
    int s1 = s0 + 1, w1 = w0;
    if (s1 == ring.stages) {
        s1 = 0;
        ++w1;
    }
    if (!ring_wait_free(ring, s0, w0) || !ring_wait_free(ring, s1, w1)) return false;
    decode_into<FMT, SL, PIECES>(grp, prow, pquart, ring.base + static_cast<size_t>(s0) * ring.stage_bytes);
    decode_into<FMT, SL + 1, PIECES>(grp, prow, pquart, ring.base + static_cast<size_t>(s1) * ring.stage_bytes);
    fence_proxy_async();          // the decoded pieces must be visible to the tensor core's reads
    __syncwarp();
    if (lane == 0) {
        if (ring.remote_full) {
            mbar_arrive_cluster(ring.remote_full + 8u * s0);
            mbar_arrive_cluster(ring.remote_full + 8u * s1);
        } else {
            mbar_arrive(&ring.full_bar[s0]);
            mbar_arrive(&ring.full_bar[s1]);
        }
    }
    ring.stage = s1 + 1;
    ring.wraps = w1;
    if (ring.stage == ring.stages) {
        ring.stage = 0;
        ++ring.wraps;
    }
    return true;
}

// The four slabs of group g from `cur`; after the first two of them (when cur's bytes have arrived and no other
// load of this thread is in flight) the packed bytes of group g + 1 are requested into `nxt`, and L2 is asked
// for group g + 3. The request sits after a slab and not at the end of the previous group on purpose: the
// hardware waits for "all loads issued so far under this dependency counter", and with the loads of both
// register sets in flight at the first use of one of them a decoder waited out the full memory latency of
// the set it had just requested (2.6 stalled warps per issue at [8192 x 2048] x 512).
template <int FMT, int PIECES>
__device__ __forceinline__ bool decode_group(const RawGroup (&cur)[PIECES], RawGroup (&nxt)[PIECES],
                                             const uint8_t *const (&row_ptr)[PIECES], const int (&prow)[PIECES],
                                             const int (&pquart)[PIECES], int g, int ngroups, DecoderRing &ring, int lane) {
    constexpr int GB = fmt_group_bytes(FMT);
    if (!decode_store_two<FMT, 0, PIECES>(cur, prow, pquart, ring, lane)) return false;
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
        fetch_group<FMT>(row_ptr[j] + static_cast<size_t>(min(g + 1, ngroups - 1)) * GB, pquart[j], nxt[j]);
        if (g + 3 < ngroups) asm volatile("prefetch.global.L2 [%0];" ::"l"(row_ptr[j] + static_cast<size_t>(g + 3) * GB));
    }
    return decode_store_two<FMT, 2, PIECES>(cur, prow, pquart, ring, lane);
}

// ---------------------------------------------------------------------------------------------
// Kernel. FMT: native GGUF format. Eighteen warps: 0-15 decode (and run the epilogue), one lane of warp
// 16 issues the MMAs, one lane of warp 17 the TMA loads. A stage holds one decoded weight slab (16 KB) followed by
// `mt` activation slabs of ntok rows x 128 bytes.
// ---------------------------------------------------------------------------------------------
constexpr int UG_MAX_STAGES = 6;
constexpr int UG_DECODE_THREADS = 512;
constexpr int UG_THREADS = UG_DECODE_THREADS + 64;
constexpr int UG_PIECES = UG_BM * 4 / UG_DECODE_THREADS;      // 16-weight pieces per decoder thread and slab

template <int FMT, bool SPLIT, bool PAIR>
__global__ void __launch_bounds__(UG_THREADS, 1) umma_gemm_kernel(const __grid_constant__ CUtensorMap xmap,
                                                                  const UmmaGemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[UG_MAX_STAGES], free_bar[UG_MAX_STAGES], acc_done;
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    chain_trigger();
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * UG_BM;
    const int ntok = a.ntok, mt_count = a.mt;
    const int m0 = blockIdx.y * (mt_count * ntok);
    // PAIR: CTAs 2p and 2p + 1 form a cluster and one [256 weight rows x ntok tokens] tensor-core tile. Each decodes
    // its own 128 rows and stages half of the tokens; rank 0 issues the MMAs for both and owns the `full` barriers.
    const uint32_t rank = PAIR ? cluster_cta_rank() : 0;
    const int ntok_cta = PAIR ? ntok >> 1 : ntok;               // token rows this CTA stages per accumulator
    // split-K: this CTA walks the groups [group0, group0 + ngroups) of K
    // (SPLIT is a template argument: the one-CTA-per-tile kernel keeps the code it had before the split existed;
    // the same source with a run-time test measured 9 % slower at [8192 x 2048] x 512)
    const int group0 = SPLIT ? blockIdx.z * a.groups_per_split : 0;
    const int ngroups = SPLIT ? min(a.groups_per_split, a.k / 256 - group0) : a.k / 256;
    const int nslab = ngroups * (256 / UG_BK);
    const int S = a.stages;
    const int x_bytes = ntok_cta * UG_BK * 2;                   // this CTA's activation slab of one token tile
    const int stage_bytes = UG_W_BYTES + mt_count * x_bytes;
    const int acc_stride = (ntok + 31) & ~31;                   // TMEM columns between the accumulators
    uint32_t tmem_cols = 32;
    while (tmem_cols < static_cast<uint32_t>(mt_count * acc_stride)) tmem_cols <<= 1;

    if (tid == 0) {
        for (int s = 0; s < UG_MAX_STAGES; ++s) {
            // one arrival per decoder warp (of both CTAs in a pair) + the TMA lane's
            mbar_init(&full_bar[s], (PAIR ? 2 : 1) * (UG_DECODE_THREADS / 32) + 1);
            mbar_init(&free_bar[s], 1);
        }
        mbar_init(&acc_done, 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 0) {
        tmem_alloc<PAIR>(&tmem_base_slot, tmem_cols);
        tmem_relinquish<PAIR>();
    }
    tc_fence_before();
    if (PAIR) cluster_sync_all();        // the partner's barriers are initialised before anything arrives on them
    else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = tmem_base_slot;

    if (warp < UG_DECODE_THREADS / 32) {
        // ---------------------------------------------------------------- decoders
        // piece j of this thread: weight row prow[j] of the tile, 16-value quarter pquart[j] of a slab's
        // 64 positions; four consecutive lanes hold the four quarters of a row (their loads cover 64 contiguous
        // bytes of it, a warp eight rows; the 16-byte swizzled stores of a warp still take the minimum of four
        // wavefronts: for each quarter the eight rows land in the eight different chunks)
        const uint8_t *row_ptr[UG_PIECES];
        int prow[UG_PIECES], pquart[UG_PIECES];
#pragma unroll
        for (int j = 0; j < UG_PIECES; ++j) {
            const int id = tid + UG_DECODE_THREADS * j;
            prow[j] = (id >> 2) % UG_BM;
            pquart[j] = id & 3;
            const int wrow = min(n0 + prow[j], a.n - 1);      // rows past the end decode the last row; never stored
            row_ptr[j] = a.w + static_cast<size_t>(wrow) * a.row_bytes + static_cast<size_t>(group0) * fmt_group_bytes(FMT);
        }
        // Two register sets take turns: one holds the group being decoded, the other receives the next group's
        // packed bytes (requested two slabs before their first use; two groups further ahead the lines are
        // only asked into L2). Weights are read-only: no dependency wait. The loop is unrolled by two so the
        // sets are named statically and nothing is copied.
        constexpr int GB = fmt_group_bytes(FMT);
        DecoderRing ring{smem, free_bar, full_bar, &abort_flag, a.status, stage_bytes, S, 0, 0,
                         (PAIR && rank == 1) ? cluster_map(smem_u32(&full_bar[0]), 0) : 0u};
        RawGroup set0[UG_PIECES], set1[UG_PIECES];
#pragma unroll
        for (int j = 0; j < UG_PIECES; ++j) {
            fetch_group<FMT>(row_ptr[j], pquart[j], set0[j]);
            for (int ahead = 1; ahead <= 2; ++ahead)
                if (ahead < ngroups) asm volatile("prefetch.global.L2 [%0];" ::"l"(row_ptr[j] + static_cast<size_t>(ahead) * GB));
        }
        for (int g = 0; g < ngroups; g += 2) {
            if (!decode_group<FMT, UG_PIECES>(set0, set1, row_ptr, prow, pquart, g, ngroups, ring, lane)) break;
            if (g + 1 < ngroups && !decode_group<FMT, UG_PIECES>(set1, set0, row_ptr, prow, pquart, g + 1, ngroups, ring, lane))
                break;
        }
    } else if (warp == UG_DECODE_THREADS / 32 + 1) {
        // ---------------------------------------------------------------- TMA loads of the activation slabs
        // (the whole warp walks the loop, one elected lane issues)
        {
        chain_wait();                 // the activations come from the preceding kernel on the stream
        // (stage index and barrier phase are kept as running counters: this lane's loop is a chain of
        // dependent instructions, and a runtime division per slab would cost more than the copies' issue)
        int issued = 0, s = 0, wraps = 0, xcol = group0 * 256;
        uint8_t *dst = smem + UG_W_BYTES;
        const uint32_t full0 = PAIR ? cluster_map(smem_u32(&full_bar[0]), 0) : 0u;
        const int row0 = m0 + static_cast<int>(rank) * ntok_cta;
        for (int i = 0; i < nslab; ++i) {
            // (votes keep the 32 lanes on one path: the elections below name all of them)
            if (__any_sync(0xffffffffu, abort_flag != 0)) break;
            if (wraps > 0 && !__all_sync(0xffffffffu, mbar_wait_bounded(&free_bar[s], (wraps - 1) & 1, a.status,
                                                                        STATUS_UMMA_WAIT_MMA))) {
                abort_flag = 1;
                break;
            }
            if (elect_one()) {
                if (PAIR) {
                    // the first CTA announces the bytes of both halves; either half may land first
                    if (rank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * mt_count * x_bytes);
                    for (int mt = 0; mt < mt_count; ++mt)
                        tma_load_2d_pair(dst + mt * x_bytes, &xmap, xcol, row0 + mt * ntok, full0 + 8u * s);
                } else {
                    mbar_arrive_expect_tx(&full_bar[s], mt_count * x_bytes);
                    for (int mt = 0; mt < mt_count; ++mt)
                        tma_load_2d(dst + mt * x_bytes, &xmap, xcol, m0 + mt * ntok, &full_bar[s]);
                }
            }
            __syncwarp();
            issued = i + 1;
            xcol += UG_BK;
            dst += stage_bytes;
            if (++s == S) {
                s = 0;
                ++wraps;
                dst = smem + UG_W_BYTES;
            }
        }
        if (abort_flag) {
            // gave up somewhere: the copies already requested still write shared memory; they complete on
            // their own within microseconds - give them that time before the CTA can exit
            const uint64_t t0 = global_timer_ns();
            while (issued > 0 && global_timer_ns() - t0 < 100000) {
            }
        }
        }
        __syncwarp();
    } else if (warp == UG_DECODE_THREADS / 32) {
        // ---------------------------------------------------------------- MMA issue (whole warp, elected lane)
        if (rank == 0) {
        const uint32_t idesc = umma_idesc_bf16(PAIR ? 2 * UG_BM : UG_BM, ntok);
        const uint32_t free0 = smem_u32(&free_bar[0]), free0_peer = PAIR ? cluster_map(free0, 1) : 0u;
        // descriptors advance by running additions (address field = bytes >> 4); see the note in the TMA lane
        const uint64_t w_desc0 = smem_desc_sw128(smem);
        const uint32_t stage_step = static_cast<uint32_t>(stage_bytes) >> 4, x_off = UG_W_BYTES >> 4,
                       x_step = static_cast<uint32_t>(x_bytes) >> 4;
        uint64_t w_desc = w_desc0;
        uint32_t accumulate = 0;
        int done_slabs = 0, s = 0, phase = 0;
        for (int i = 0; i < nslab; ++i) {
            if (__any_sync(0xffffffffu, abort_flag != 0)) break;
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(&full_bar[s], phase, a.status, STATUS_UMMA_WAIT_TMA))) {
                abort_flag = 1;
                break;
            }
            tc_fence_after();
            if (elect_one()) {
                for (int mt = 0; mt < mt_count; ++mt) {
                    const uint64_t x_desc = w_desc + x_off + mt * x_step;
                    const uint32_t d = tmem_d + mt * acc_stride;
                    umma_bf16<PAIR>(d, w_desc, x_desc, idesc, accumulate);        // 16 BF16 = 32 bytes per step:
                    umma_bf16<PAIR>(d, w_desc + 2, x_desc + 2, idesc, 1u);        // +2 in the address field
                    umma_bf16<PAIR>(d, w_desc + 4, x_desc + 4, idesc, 1u);
                    umma_bf16<PAIR>(d, w_desc + 6, x_desc + 6, idesc, 1u);
                }
                umma_commit<PAIR>(free0 + 8u * s);                       // the stage is free again in this CTA ...
                if (PAIR) umma_commit<PAIR>(free0_peer + 8u * s);        // ... and in the partner
            }
            __syncwarp();
            accumulate = 1u;
            done_slabs = i + 1;
            w_desc += stage_step;
            if (++s == S) {
                s = 0;
                phase ^= 1;
                w_desc = w_desc0;
            }
        }
        if (done_slabs == nslab && elect_one()) {
            umma_commit<PAIR>(smem_u32(&acc_done));
            if (PAIR) umma_commit<PAIR>(cluster_map(smem_u32(&acc_done), 1));
        }
        }
        __syncwarp();
    }

    // ---------------------------------------------------------------- epilogue (warps 0-7)
    bool ok = !abort_flag;
    if (ok && !mbar_wait_bounded(&acc_done, 0, a.status, STATUS_UMMA_WAIT_MMA)) {
        abort_flag = 1;
        ok = false;
    }
    ok = __syncthreads_and(ok) != 0;      // one answer for the CTA: the groups below meet at named barriers
    if (ok && warp < UG_DECODE_THREADS / 32) {
        tc_fence_after();
        chain_wait();        // y may still be read by what precedes this kernel on the stream
        // warp w reads TMEM lanes 32*(w%4)..+31 = 32 weight rows; the 32-token chunks of every accumulator
        // are dealt round-robin to the four groups of four warps. A group turns its chunk [128 rows x 32 tokens]
        // into the output's layout in shared memory (the ring is idle by now: every MMA has completed) and stores
        // it in 16-byte pieces, a warp instruction covering whole 128-byte lines of two (BF16) tokens; outputs
        // whose rows are not 16-byte aligned take the direct path, 32 two- or four-byte stores per thread.
        const int quarter = warp & 3, group = warp >> 2;
        const int row_local = 32 * quarter + lane;
        const int row = n0 + row_local;
        const int nchunks = (ntok + 31) >> 5;
        uint8_t *out = SPLIT ? reinterpret_cast<uint8_t *>(a.partial + static_cast<size_t>(blockIdx.z) * a.m * a.n)
                             : static_cast<uint8_t *>(a.y);
        const int out_dtype = SPLIT ? B200Q_F32 : a.y_dtype;
        const int esize = out_dtype == B200Q_F32 ? 4 : 2;
        const bool staged = a.n % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
        uint8_t *tile = smem + group * (32 * UG_BM * 4);          // 16 KB per group
        for (int mt = 0; mt < mt_count; ++mt) {
            const int tile_t0 = m0 + mt * ntok;
            if (tile_t0 >= a.m) break;                           // whole token tile beyond m (uniform in the CTA)
            for (int c = group; c < nchunks; c += UG_DECODE_THREADS / 128) {
                uint32_t r[32];
                tmem_ld32(tmem_d + (static_cast<uint32_t>(32 * quarter) << 16) + mt * acc_stride + 32 * c, r);
                tmem_ld_wait();
                if (staged) {
                    if (esize == 4) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) reinterpret_cast<uint32_t *>(tile)[j * UG_BM + row_local] = r[j];
                    } else if (out_dtype == B200Q_BF16) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            reinterpret_cast<uint16_t *>(tile)[j * UG_BM + row_local] =
                                __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(r[j])));
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            reinterpret_cast<uint16_t *>(tile)[j * UG_BM + row_local] =
                                __half_as_ushort(__float2half_rn(__uint_as_float(r[j])));
                    }
                    named_barrier_sync(1 + group, 128);
                    const int pieces_per_token = 8 * esize;                  // 16-byte pieces of a 128-row line
                    const int piece_shift = esize == 4 ? 5 : 4;
                    for (int p = row_local; p < 32 * pieces_per_token; p += 128) {
                        const int j = p >> piece_shift, piece = p & (pieces_per_token - 1);
                        const int t = tile_t0 + 32 * c + j;
                        const int col = n0 + piece * (16 / esize);
                        if (32 * c + j < ntok && t < a.m && col < a.n) {
                            const uint4 v = *reinterpret_cast<const uint4 *>(tile + static_cast<size_t>(j) * UG_BM * esize +
                                                                             piece * 16);
                            *reinterpret_cast<uint4 *>(out + (static_cast<size_t>(t) * a.n + col) * esize) = v;
                        }
                    }
                    named_barrier_sync(1 + group, 128);                      // the tile is rewritten by the next chunk
                } else if (row < a.n) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int t = tile_t0 + 32 * c + j;
                        if (32 * c + j < ntok && t < a.m) store_out(out, out_dtype, static_cast<size_t>(t) * a.n + row, r[j]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    // a pair frees its tensor memory together, and neither CTA leaves while the other may still signal its barriers
    // or read its activation half
    if (PAIR) cluster_sync_all();
    else __syncthreads();
    if (warp == 0) tmem_dealloc<PAIR>(tmem_d, tmem_cols);
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    });
    return fn;
}

using GemmFn = void (*)(const CUtensorMap, const UmmaGemmArgs);

template <bool SPLIT, bool PAIR>
static GemmFn gemm_kernel_for(int fmt) {
    return fmt == B200Q_Q8_0 ? umma_gemm_kernel<B200Q_Q8_0, SPLIT, PAIR>
         : fmt == B200Q_Q4_K ? umma_gemm_kernel<B200Q_Q4_K, SPLIT, PAIR>
         : fmt == B200Q_Q5_K ? umma_gemm_kernel<B200Q_Q5_K, SPLIT, PAIR>
                             : umma_gemm_kernel<B200Q_Q6_K, SPLIT, PAIR>;
}

static int gemm_pair_mode() {          // read at every call, so a test can compare the kernels in one process
    const char *v = std::getenv("B200Q_GEMM_PAIR");
    return (v && v[0] == '0') ? 0 : (v && v[0] == '2') ? 2 : 1;
}

// y[t, col] = partial[0][t, col] + partial[1][t, col] + ... in ascending split order (deterministic), rounded once.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *partial, int splits, long long count, void *y,
                                                            int y_dtype) {
    chain_trigger();
    chain_wait();
    const long long i = (static_cast<long long>(blockIdx.x) * 256 + threadIdx.x) * 4;
    if (i >= count) return;                           // count is a multiple of 4 (n is)
    float4 acc = *reinterpret_cast<const float4 *>(partial + i);
    for (int z = 1; z < splits; ++z) {
        const float4 v = *reinterpret_cast<const float4 *>(partial + static_cast<size_t>(z) * count + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    store_out(y, y_dtype, i, __float_as_uint(acc.x));
    store_out(y, y_dtype, i + 1, __float_as_uint(acc.y));
    store_out(y, y_dtype, i + 2, __float_as_uint(acc.z));
    store_out(y, y_dtype, i + 3, __float_as_uint(acc.w));
}

// Split of K over grid.z for shapes with too few (weight-row tile x token tile) CTAs to fill the SMs: a power
// of two, at least 4 groups (16 slabs) of K per CTA, no more CTAs than SMs; 1 = no split.
static int gemm_splits(int n, int k, int m) {
    if (n % 4 != 0) return 1;
    const int ntok = m >= 256 ? 256 : (m + 15) / 16 * 16;
    const int token_tiles = (m + ntok - 1) / ntok;
    const int n_tiles = (n + UG_BM - 1) / UG_BM;
    const int mt = (token_tiles >= 2 && static_cast<long long>(n_tiles) * ((token_tiles + 1) / 2) >= sm_count()) ? 2 : 1;
    const long long ctas = static_cast<long long>(n_tiles) * ((token_tiles + mt - 1) / mt);
    int splits = 1;
    while (splits < 8 && ctas * splits * 2 <= sm_count() && (k / 256) / (splits * 2) >= 4) splits *= 2;
    return splits;
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_gemm_supported(int fmt, int n, int k, int x_dtype, int m) {
    if (fmt != B200Q_Q8_0 && fmt != B200Q_Q4_K && fmt != B200Q_Q5_K && fmt != B200Q_Q6_K) return 0;
    if (x_dtype != B200Q_BF16 || n < 1 || m < 1 || k < 256 || k % 256 != 0) return 0;
    return 1;
}

extern "C" long long b200q_gemm_workspace_bytes(int fmt, int n, int k, int x_dtype, int m) {
    if (!b200q_gemm_supported(fmt, n, k, x_dtype, m)) return 0;
    const int splits = gemm_splits(n, k, m);
    return splits > 1 ? static_cast<long long>(splits) * m * n * 4 : 0;
}

static int gemm_impl(const void *w, int fmt, int n, int k, const void *x, int x_dtype, int m, void *y, int y_dtype,
                     void *workspace, long long workspace_bytes, void *stream) {
    if (!w || !x || !y) return fail(B200Q_EINVAL, "gemm: NULL pointer");
    if (!fmt_valid(fmt)) return fail(B200Q_EINVAL, "gemm: unknown or device-only format %d", fmt);
    if (!dtype_valid(x_dtype) || !dtype_valid(y_dtype)) return fail(B200Q_EINVAL, "gemm: bad dtype");
    if (n <= 0 || m <= 0 || k <= 0 || k % fmt_elems(fmt) != 0)
        return fail(B200Q_EINVAL, "gemm: bad shape n=%d k=%d m=%d", n, k, m);
    if (!b200q_gemm_supported(fmt, n, k, x_dtype, m))
        return fail(B200Q_EUNSUPPORTED, "gemm: needs BF16 activations and K a multiple of 256 (use b200q_gemv)");
    if (reinterpret_cast<uintptr_t>(x) & 15) return fail(B200Q_EUNSUPPORTED, "gemm: activations must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(w) & 1) return fail(B200Q_EUNSUPPORTED, "gemm: weights must be 2-byte aligned");
    // the Q8_0 decoder reads whole aligned words around its 16-byte pieces; a base on a word boundary keeps the
    // last word of the tensor inside it
    if (fmt == B200Q_Q8_0 && (reinterpret_cast<uintptr_t>(w) & 3))
        return fail(B200Q_EUNSUPPORTED, "gemm: Q8_0 weights must be 4-byte aligned");
    int *status = device_status_word();
    if (!status) return fail(B200Q_ECUDA, "gemm: no CUDA device");
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return fail(B200Q_ECUDA, "gemm: the driver does not provide cuTensorMapEncodeTiled");

    // Token tile: the whole batch rounded up to 16 when it fits one accumulator, else 256. Two tiles per
    // CTA (every decoded weight slab then feeds 512 tokens) only when that still leaves a CTA for every SM.
    const int ntok = m >= 256 ? 256 : (m + 15) / 16 * 16;
    const int token_tiles = (m + ntok - 1) / ntok;
    const int n_tiles = (n + UG_BM - 1) / UG_BM;
    const int mt = (token_tiles >= 2 && static_cast<long long>(n_tiles) * ((token_tiles + 1) / 2) >= sm_count()) ? 2 : 1;
    const int m_tiles = (token_tiles + mt - 1) / mt;
    // From about a thousand tokens on, two CTAs on neighbouring SMs share a token tile (cta_group::2): each stages
    // half of the activation rows, so the tensor core's operand reads and the TMA writes take less of each SM's
    // shared-memory bandwidth ([8192 x 2048] x 2048: 70.9 -> 66.1 us; below that the one-CTA kernel is 1-4 %
    // faster, its barriers being local). B200Q_GEMM_PAIR=0 keeps the one-CTA kernel, =2 pairs at every size.
    const int pair_mode = gemm_pair_mode();
    const bool pair = pair_mode == 2 || (pair_mode == 1 && token_tiles >= 4);
    const int stage_bytes = UG_W_BYTES + mt * (pair ? ntok / 2 : ntok) * UG_BK * 2;
    int stages = (224 * 1024) / stage_bytes;
    if (stages > UG_MAX_STAGES) stages = UG_MAX_STAGES;

    CUtensorMap xmap;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
    const cuuint32_t box[2] = {UG_BK, static_cast<cuuint32_t>(pair ? ntok / 2 : ntok)};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult res = encode(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(x), dims, strides, box,
                                elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) return fail(B200Q_ECUDA, "gemm: cuTensorMapEncodeTiled failed (%d)", static_cast<int>(res));

    UmmaGemmArgs a{};
    a.w = static_cast<const uint8_t *>(w);
    a.n = n; a.k = k; a.m = m;
    a.row_bytes = static_cast<long long>(k / fmt_elems(fmt)) * fmt_bytes(fmt);
    a.y = y; a.y_dtype = y_dtype; a.ntok = ntok; a.mt = mt; a.stages = stages; a.status = status;
    int splits = gemm_splits(n, k, m);
    if (!workspace || workspace_bytes < static_cast<long long>(splits) * m * n * 4 ||
        (reinterpret_cast<uintptr_t>(workspace) & 15))
        splits = 1;                                    // no room for partial results: one CTA walks all of K
    a.groups_per_split = (k / 256 + splits - 1) / splits;
    a.partial = splits > 1 ? static_cast<float *>(workspace) : nullptr;
    const GemmFn fn = pair ? (splits > 1 ? gemm_kernel_for<true, true>(fmt) : gemm_kernel_for<false, true>(fmt))
                           : (splits > 1 ? gemm_kernel_for<true, false>(fmt) : gemm_kernel_for<false, false>(fmt));
    const size_t smem = static_cast<size_t>(stages) * stage_bytes + 1024;
    // the opt-in to large dynamic shared memory is per function and device: done once each
    {
        static std::mutex mu;
        static std::vector<std::pair<const void *, int>> opted;
        int dev = 0;
        cudaGetDevice(&dev);
        std::lock_guard<std::mutex> lock(mu);
        const std::pair<const void *, int> key(reinterpret_cast<const void *>(fn), dev);
        if (std::find(opted.begin(), opted.end(), key) == opted.end()) {
            cudaError_t err = cudaFuncSetAttribute(reinterpret_cast<const void *>(fn),
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
            if (err != cudaSuccess) {
                cudaGetLastError();
                return fail(B200Q_ECUDA, "gemm: shared memory opt-in failed: %s", cudaGetErrorString(err));
            }
            opted.push_back(key);
        }
    }
    if (pair)      // an odd last weight-row tile gets a partner that decodes clamped rows and stores nothing
        launch_chained_cluster(fn, dim3((n_tiles + 1) & ~1, m_tiles, splits), dim3(UG_THREADS), smem,
                               static_cast<cudaStream_t>(stream), 2, xmap, a);
    else
        launch_chained(fn, dim3(n_tiles, m_tiles, splits), dim3(UG_THREADS), smem, static_cast<cudaStream_t>(stream), xmap,
                       a);
    int rc = check_launch("gemm");
    if (rc || splits == 1) return rc;
    const long long count = static_cast<long long>(m) * n;
    launch_chained(splitk_reduce_kernel, dim3(static_cast<unsigned>((count / 4 + 255) / 256)), dim3(256), 0,
                   static_cast<cudaStream_t>(stream), static_cast<const float *>(workspace), splits, count, y, y_dtype);
    return check_launch("gemm (split-K sum)");
}

extern "C" int b200q_gemm(const void *w, int fmt, int n, int k, const void *x, int x_dtype, int m, void *y,
                          int y_dtype, void *stream) {
    return gemm_impl(w, fmt, n, k, x, x_dtype, m, y, y_dtype, nullptr, 0, stream);
}

extern "C" int b200q_gemm_ws(const void *w, int fmt, int n, int k, const void *x, int x_dtype, int m, void *y,
                             int y_dtype, void *workspace, long long workspace_bytes, void *stream) {
    return gemm_impl(w, fmt, n, k, x, x_dtype, m, y, y_dtype, workspace, workspace_bytes, stream);
}
