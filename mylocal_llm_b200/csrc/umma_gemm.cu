// Batched / prefill GEMM on packed GGUF weights: y[m, n] = x[m, k] @ W[n, k]^T for m > 16 tokens.
//
// A GEMV pass re-reads the packed matrix once per 8 or 16 tokens; from a few dozen tokens on the
// product is a real contraction and belongs on the 5th-generation tensor cores. One CTA owns a tile
// of 128 (or 256) tokens x NT weight rows and walks K in slabs of 64:
//   * the activation slab [128 tokens x 64 k] (BF16) arrives by TMA (cp.async.bulk.tensor.2d, 128-byte
//     swizzle, rows beyond m zero-filled by the tensor map) and signals an mbarrier;
//   * all threads decode the packed weights of the slab [NT rows x 64 k] - the reference's
//     dequantisation (mini_llm/ops/quantized_weight.py:208-250), FP32 arithmetic, rounded once to
//     BF16 - and store them in the same 128-byte-swizzled K-major layout;
//   * one thread issues tcgen05.mma (kind::f16, M = 128, N = NT, K = 16, four per slab) with both
//     operands described by shared-memory descriptors; the FP32 accumulator [128 x NT] lives in
//     tensor memory; tcgen05.commit arrives on the stage's mbarrier when the tensor core has
//     consumed the slab, which frees the stage for the decode two slabs later;
//   * after the last slab the eight warps read the accumulator back with tcgen05.ld (each warp its
//     32-lane quarter), convert and store y.
// The tensor core works on slab i while the threads decode slab i+1 (four stages). Weights are
// rounded to BF16, so results carry BF16-weight precision (relative 2^-9 per weight, like the BF16
// activations this path requires); the GEMV kernels keep their exact-product arithmetic for m <= 16
// and for FP32 activations.
//
// Every mbarrier wait is bounded (2 s): on expiry the CTA records a status code, skips the rest of
// its work, waits (bounded) for what it has in flight, frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace b200q {

constexpr int UG_THREADS = 256;
constexpr int UG_BM = 128;          // tokens per accumulator (UMMA M)
constexpr int UG_BK = 64;           // K per slab: 64 BF16 = one 128-byte swizzle row
constexpr int UG_STAGES = 4;
constexpr int UG_A_BYTES = UG_BM * UG_BK * 2;
constexpr int STATUS_UMMA_WAIT_TMA = 111;   // gave up waiting for an activation slab
constexpr int STATUS_UMMA_WAIT_MMA = 112;   // gave up waiting for the tensor core to release a stage

struct UmmaGemmArgs {
    const uint8_t *w;
    int n, k, m;
    long long row_bytes;      // packed bytes per weight row (native layouts)
    void *y;
    int y_dtype;
    int *status;
};

// ---------------------------------------------------------------------------------------------
// tcgen05 / TMA wrappers (sm_100a)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]; `accumulate` = 0 overwrites D.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier receives one arrival when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
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
// Decoding 32 consecutive weights of one packed row (positions 32*u .. 32*u+31) to FP32, with the
// reference's arithmetic: (d*sc)*q - (dmin*mn) for Q4_K / Q5_K, (d*sc)*q for Q6_K, d*q for Q8_0.
// ---------------------------------------------------------------------------------------------
// 32 bytes from an address with any alignment that is a multiple of 2.
__device__ __forceinline__ void load32(const uint8_t *p, uint32_t (&w)[8]) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    if ((a & 15) == 0) {
        const uint4 lo = *reinterpret_cast<const uint4 *>(p), hi = *reinterpret_cast<const uint4 *>(p + 16);
        w[0] = lo.x; w[1] = lo.y; w[2] = lo.z; w[3] = lo.w; w[4] = hi.x; w[5] = hi.y; w[6] = hi.z; w[7] = hi.w;
    } else if ((a & 3) == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = reinterpret_cast<const uint32_t *>(p)[i];
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint16_t *h = reinterpret_cast<const uint16_t *>(p) + 2 * i;
            w[i] = static_cast<uint32_t>(h[0]) | (static_cast<uint32_t>(h[1]) << 16);
        }
    }
}
__device__ __forceinline__ float half_at(const uint8_t *p) {
    return half_bits_to_float(*reinterpret_cast<const uint16_t *>(p));
}

template <int FMT>
__device__ __forceinline__ void decode32(const uint8_t *row, int u, float (&out)[32]) {
    uint32_t q[8];
    if (FMT == B200Q_Q8_0) {
        const uint8_t *b = row + static_cast<size_t>(u) * 34;
        const float d = half_at(b);
        // the 32 codes start 2 bytes into a 34-byte block
        const uint16_t *h = reinterpret_cast<const uint16_t *>(b + 2);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t v = h[i];
            out[2 * i] = d * static_cast<float>(static_cast<int>(static_cast<int8_t>(v & 0xffu)));
            out[2 * i + 1] = d * static_cast<float>(static_cast<int>(static_cast<int8_t>(v >> 8)));
        }
        return;
    }
    const int sb = u >> 3, g = u & 7;
    if (FMT == B200Q_Q4_K || FMT == B200Q_Q5_K) {
        constexpr int QB = FMT == B200Q_Q5_K ? 176 : 144;
        const uint8_t *b = row + static_cast<size_t>(sb) * QB;
        const float d = half_at(b), dmin = half_at(b + 2);
        const uint8_t *m = b + 4;
        int sc, mn;
        if (g < 4) {
            sc = m[g] & 63;
            mn = m[4 + g] & 63;
        } else {
            sc = (m[4 + g] & 15) | ((m[g - 4] >> 2) & 48);
            mn = (m[4 + g] >> 4) | ((m[g] >> 2) & 48);
        }
        const float scale = d * static_cast<float>(sc), minimum = dmin * static_cast<float>(mn);
        load32(b + (FMT == B200Q_Q5_K ? 48 : 16) + 32 * (g >> 1), q);
        uint32_t hb[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (FMT == B200Q_Q5_K) load32(b + 16, hb);
        const int shift = 4 * (g & 1);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t nib = (q[i] >> shift) & 0x0f0f0f0fu;
            const uint32_t top = FMT == B200Q_Q5_K ? ((hb[i] >> g) & 0x01010101u) << 4 : 0u;
            const uint32_t code = nib | top;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                out[4 * i + j] = __fmaf_rn(scale, static_cast<float>((code >> (8 * j)) & 0xffu), -minimum);
        }
        return;
    }
    // Q6_K: position p = 32*g inside the super-block; half = p / 128, quarter = (p % 128) / 32
    const uint8_t *b = row + static_cast<size_t>(sb) * 210;
    const float d = half_at(b + 208);
    const int half = g >> 2, quarter = g & 3;
    uint32_t hi[8];
    load32(b + 64 * half + 32 * (quarter & 1), q);
    load32(b + 128 + 32 * half, hi);
    const int8_t *scales = reinterpret_cast<const int8_t *>(b + 192 + 2 * g);
    const float s0 = d * static_cast<float>(scales[0]), s1 = d * static_cast<float>(scales[1]);
    const int lo_shift = 4 * (quarter >> 1), hi_shift = 2 * quarter;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t lo4 = (q[i] >> lo_shift) & 0x0f0f0f0fu;
        const uint32_t hi2 = ((hi[i] >> hi_shift) & 0x03030303u) << 4;
        const uint32_t code = lo4 | hi2;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int v = static_cast<int>((code >> (8 * j)) & 0xffu) - 32;
            out[4 * i + j] = (i < 4 ? s0 : s1) * static_cast<float>(v);
        }
    }
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// ---------------------------------------------------------------------------------------------
// Kernel. FMT: native GGUF format; NT: weight rows per CTA (UMMA N, 64 or 128); MT: token tiles of
// 128 per CTA (1 or 2; both use every decoded weight slab).
// ---------------------------------------------------------------------------------------------
template <int FMT, int NT, int MT>
__global__ void __launch_bounds__(UG_THREADS, 1) umma_gemm_kernel(const __grid_constant__ CUtensorMap xmap,
                                                                  const UmmaGemmArgs a) {
    constexpr int B_BYTES = NT * UG_BK * 2;
    constexpr int STAGE_BYTES = MT * UG_A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = MT * NT;                   // 64, 128 or 256: a power of two >= 32
    constexpr uint32_t IDESC = umma_idesc_bf16(UG_BM, NT);
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_a[UG_STAGES], mma_done[UG_STAGES];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    chain_trigger();
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * NT;
    const int m0 = blockIdx.y * (MT * UG_BM);
    const int nslab = a.k / UG_BK;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < UG_STAGES; ++s) {
            mbar_init(&full_a[s], 1);
            mbar_init(&mma_done[s], 1);
        }
        abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 0) {
        tmem_alloc(&tmem_base_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = tmem_base_slot;
    chain_wait();            // the activations come from the preceding kernel on the stream

    // decode unit of this thread inside a slab: weight row `urow` of the tile, 32-value half `uhalf`
    const int unit = tid;
    const bool has_unit = unit < 2 * NT;
    const int urow = unit % NT, uhalf = unit / NT;
    const int wrow = min(n0 + urow, a.n - 1);                 // rows past the end decode the last row; never stored
    const uint8_t *row_ptr = a.w + static_cast<size_t>(wrow) * a.row_bytes;

    int issued = 0;          // slabs whose loads / MMAs have been issued (thread 0)
    bool failed = false;
    for (int i = 0; i < nslab; ++i) {
        const int s = i % UG_STAGES;
        uint8_t *stage = smem + static_cast<size_t>(s) * STAGE_BYTES;
        if (i >= UG_STAGES &&
            !mbar_wait_bounded(&mma_done[s], ((i / UG_STAGES) - 1) & 1, a.status, STATUS_UMMA_WAIT_MMA)) {
            abort_flag = 1;
        }
        if (tid == 0 && !abort_flag) {
            mbar_arrive_expect_tx(&full_a[s], MT * UG_A_BYTES);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
                tma_load_2d(stage + mt * UG_A_BYTES, &xmap, i * UG_BK, m0 + mt * UG_BM, &full_a[s]);
            issued = i + 1;
        }
        if (has_unit) {
            float wv[32];
            decode32<FMT>(row_ptr, i * 2 + uhalf, wv);
            uint8_t *dst_row = stage + MT * UG_A_BYTES + (urow >> 3) * 1024 + (urow & 7) * 128;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint4 v;
                v.x = pack_bf16(wv[8 * c + 0], wv[8 * c + 1]);
                v.y = pack_bf16(wv[8 * c + 2], wv[8 * c + 3]);
                v.z = pack_bf16(wv[8 * c + 4], wv[8 * c + 5]);
                v.w = pack_bf16(wv[8 * c + 6], wv[8 * c + 7]);
                const int chunk = (uhalf * 4 + c) ^ (urow & 7);            // 128-byte swizzle
                *reinterpret_cast<uint4 *>(dst_row + chunk * 16) = v;
            }
        }
        fence_proxy_async();          // the decoded slab must be visible to the tensor core's reads
        __syncthreads();
        if (abort_flag) {
            failed = true;
            break;
        }
        if (tid == 0) {
            if (!mbar_wait_bounded(&full_a[s], (i / UG_STAGES) & 1, a.status, STATUS_UMMA_WAIT_TMA)) {
                abort_flag = 1;       // seen by everyone after the next barrier
            } else {
                tc_fence_after();
                const uint64_t b_desc = smem_desc_sw128(stage + MT * UG_A_BYTES);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint64_t a_desc = smem_desc_sw128(stage + mt * UG_A_BYTES);
#pragma unroll
                    for (int kk = 0; kk < UG_BK / 16; ++kk)      // 16 BF16 = 32 bytes per step: +2 in the address field
                        umma_bf16(tmem_d + mt * NT, a_desc + 2 * kk, b_desc + 2 * kk, IDESC, (i | kk) ? 1u : 0u);
                }
                umma_commit(&mma_done[s]);
            }
        }
    }

    if (!failed) {
        // the last commit covers every MMA of the tile
        const int last = nslab - 1;
        if (!mbar_wait_bounded(&mma_done[last % UG_STAGES], (last / UG_STAGES) & 1, a.status, STATUS_UMMA_WAIT_MMA))
            abort_flag = 1;
        __syncthreads();
        failed = abort_flag != 0;
    }
    if (!failed) {
        tc_fence_after();
        // warp w reads TMEM lanes 32*(w%4)..+31 (token rows) and the columns of its half of the tile
        const int quarter = warp & 3, col_half = warp >> 2;
        constexpr int COLS_PER_WARP = NT / 2;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int t = m0 + mt * UG_BM + 32 * quarter + lane;
#pragma unroll
            for (int c0 = 0; c0 < COLS_PER_WARP; c0 += 32) {
                const int col = col_half * COLS_PER_WARP + c0;
                uint32_t r[32];
                tmem_ld32(tmem_d + (static_cast<uint32_t>(32 * quarter) << 16) + mt * NT + col, r);
                tmem_ld_wait();
                if (t < a.m) {
                    const int nbase = n0 + col;
                    const size_t off = static_cast<size_t>(t) * a.n + nbase;
                    const bool full = nbase + 32 <= a.n;
                    if (a.y_dtype == B200Q_F32) {
                        float *y = static_cast<float *>(a.y) + off;
                        if (full && (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                reinterpret_cast<uint4 *>(y)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (nbase + j < a.n) y[j] = __uint_as_float(r[j]);
                        }
                    } else {
                        uint16_t *y = static_cast<uint16_t *>(a.y) + off;
                        uint32_t packed[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float lo = __uint_as_float(r[2 * j]), hi = __uint_as_float(r[2 * j + 1]);
                            if (a.y_dtype == B200Q_BF16) packed[j] = pack_bf16(lo, hi);
                            else {
                                const __half2 h = __floats2half2_rn(lo, hi);
                                packed[j] = *reinterpret_cast<const uint32_t *>(&h);
                            }
                        }
                        if (full && (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                reinterpret_cast<uint4 *>(y)[j] =
                                    make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (nbase + j < a.n)
                                    y[j] = static_cast<uint16_t>((packed[j >> 1] >> (16 * (j & 1))) & 0xffffu);
                        }
                    }
                }
            }
        }
    } else if (tid == 0) {
        // gave up: let what is in flight land (bounded) before the tensor memory is released
        for (int i = max(0, issued - UG_STAGES); i < issued; ++i)
            mbar_wait_bounded(&full_a[i % UG_STAGES], (i / UG_STAGES) & 1, a.status, STATUS_UMMA_WAIT_TMA);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_d, TMEM_COLS);
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

template <int FMT>
static GemmFn pick_tile(int nt, int mt) {
    if (nt == 128) return mt == 2 ? umma_gemm_kernel<FMT, 128, 2> : umma_gemm_kernel<FMT, 128, 1>;
    return mt == 2 ? umma_gemm_kernel<FMT, 64, 2> : umma_gemm_kernel<FMT, 64, 1>;
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_gemm_supported(int fmt, int n, int k, int x_dtype, int m) {
    if (fmt != B200Q_Q8_0 && fmt != B200Q_Q4_K && fmt != B200Q_Q5_K && fmt != B200Q_Q6_K) return 0;
    if (x_dtype != B200Q_BF16 || n < 1 || m < 1 || k < UG_BK || k % UG_BK != 0 || k % fmt_elems(fmt) != 0) return 0;
    return 1;
}

extern "C" int b200q_gemm(const void *w, int fmt, int n, int k, const void *x, int x_dtype, int m, void *y,
                          int y_dtype, void *stream) {
    if (!w || !x || !y) return fail(B200Q_EINVAL, "gemm: NULL pointer");
    if (!fmt_valid(fmt)) return fail(B200Q_EINVAL, "gemm: unknown or device-only format %d", fmt);
    if (!dtype_valid(x_dtype) || !dtype_valid(y_dtype)) return fail(B200Q_EINVAL, "gemm: bad dtype");
    if (n <= 0 || m <= 0 || k <= 0 || k % fmt_elems(fmt) != 0)
        return fail(B200Q_EINVAL, "gemm: bad shape n=%d k=%d m=%d", n, k, m);
    if (!b200q_gemm_supported(fmt, n, k, x_dtype, m))
        return fail(B200Q_EUNSUPPORTED, "gemm: needs BF16 activations and K a multiple of %d (use b200q_gemv)", UG_BK);
    if (reinterpret_cast<uintptr_t>(x) & 15) return fail(B200Q_EUNSUPPORTED, "gemm: activations must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(w) & 1) return fail(B200Q_EUNSUPPORTED, "gemm: weights must be 2-byte aligned");
    int *status = device_status_word();
    if (!status) return fail(B200Q_ECUDA, "gemm: no CUDA device");
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return fail(B200Q_ECUDA, "gemm: the driver does not provide cuTensorMapEncodeTiled");

    CUtensorMap xmap;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
    const cuuint32_t box[2] = {UG_BK, UG_BM};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult res = encode(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(x), dims, strides, box,
                                elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) return fail(B200Q_ECUDA, "gemm: cuTensorMapEncodeTiled failed (%d)", static_cast<int>(res));

    // Tile choice: two token tiles per CTA once there are more than 128 tokens (every decoded weight slab
    // then feeds 256 tokens); 64 weight rows per CTA while 128 would leave most SMs without a tile.
    const int mt = m > UG_BM ? 2 : 1;
    const int m_tiles = (m + mt * UG_BM - 1) / (mt * UG_BM);
    const int nt = (static_cast<long long>((n + 127) / 128) * m_tiles >= sm_count()) ? 128 : 64;
    const int n_tiles = (n + nt - 1) / nt;

    UmmaGemmArgs a{};
    a.w = static_cast<const uint8_t *>(w);
    a.n = n; a.k = k; a.m = m;
    a.row_bytes = static_cast<long long>(k / fmt_elems(fmt)) * fmt_bytes(fmt);
    a.y = y; a.y_dtype = y_dtype; a.status = status;
    GemmFn fn = fmt == B200Q_Q8_0 ? pick_tile<B200Q_Q8_0>(nt, mt)
              : fmt == B200Q_Q4_K ? pick_tile<B200Q_Q4_K>(nt, mt)
              : fmt == B200Q_Q5_K ? pick_tile<B200Q_Q5_K>(nt, mt)
                                  : pick_tile<B200Q_Q6_K>(nt, mt);
    const size_t smem = static_cast<size_t>(UG_STAGES) * (mt * UG_A_BYTES + nt * UG_BK * 2) + 1024;
    cudaError_t err = cudaFuncSetAttribute(reinterpret_cast<const void *>(fn),
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "gemm: shared memory opt-in failed: %s", cudaGetErrorString(err));
    }
    launch_chained(fn, dim3(n_tiles, m_tiles), dim3(UG_THREADS), smem, static_cast<cudaStream_t>(stream), xmap, a);
    return check_launch("gemm");
}
