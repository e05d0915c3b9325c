// Streaming packed-weight GEMV on the tensor cores (sm_100a), up to 8 tokens per pass.
//
// Why tensor cores for a bandwidth-bound op: at HBM speed a Q4_K stream delivers ~11.5e12 weights
// per second, which leaves about three issue slots per weight per lane. Converting every code to
// FP32 and multiplying it on the CUDA cores costs more than that. Here the integer codes are
// turned into FP16 *pairs* with one or two bit operations per pair (the code is placed into the
// mantissa of a fixed power of two), those pairs ARE the A fragments of mma.m16n8k16, and the
// multiply-accumulate of 16 rows x 16 k x 8 tokens is one instruction. Codes are small integers,
// so every product is exact and accumulation is FP32; scales and minima are applied in FP32 per
// scale group, as in the reference's decoder (mini_llm/ops/quantized_linear.py:91-172).
//
// Activations: each token row is scaled by a power of two so that its largest magnitude sits near
// 2^13, then stored as FP16 (16-bit inputs) or as an FP16 high part plus an FP16 remainder (FP32
// inputs, ~22 significant bits), already arranged as B fragments in shared memory. The scale is
// undone exactly at the output.
//
// Structure: persistent CTAs; a producer warp copies (16 * rg) rows x (256 * kp) K positions per
// tile with one 1-D bulk copy per row segment into padded shared-memory slots; 8 consumer warps =
// rg row groups x kp K parts. A row block's partial sums are combined across the kp warps through
// shared memory in a fixed order (deterministic). Modes as in stream_gemv.cuh (0 linear, 1 SwiGLU,
// 2 grouped gate/up, 3 grouped down with route weight).
#pragma once

#include "common.cuh"

namespace b200q {

#ifndef B200Q_MM_WARPS
#define B200Q_MM_WARPS 8
#endif
constexpr int MM_WARPS = B200Q_MM_WARPS;
constexpr int MM_CTHREADS = MM_WARPS * 32;
constexpr int MM_THREADS = MM_CTHREADS + 32;
constexpr int MM_MAX_STAGES = 8;
constexpr int MM_SMEM_LIMIT = 232448;
constexpr int MM_CTRL_BYTES = 1024;
constexpr int MM_STAB_BYTES = MM_WARPS * 2 * 1024;   // per warp: 16 rows x 16 floats, two streams
constexpr int MM_PART_FLOATS = MM_WARPS * 128 * 2;   // [warp][16 rows][8 tokens][2 streams]
constexpr int MM_PART_BYTES = 2 * MM_PART_FLOATS * 4; // double buffered

struct MmaArgs {
    const uint8_t *wa;
    const uint8_t *wb;
    long long stride_a, stride_b;
    const unsigned long long *table_a, *table_b;   // optional per-expert pointer tables
    int rb_a, rb_b;      // packed bytes per full weight row
    int n, k, m;
    int kp, rg;          // warps along K, row groups per tile (kp * rg == cw)
    int cw;              // consumer warps that compute (8, or 4 when shared memory is tight)
    int contig;          // 1: a tile spans whole rows and is fetched with one copy per stream
                         //    (pitch == row bytes); 0: one copy per row segment into padded slots
    int seg_a, seg_b;    // packed bytes of one row segment of a full tile (kp * 256 positions)
    int pitch_a, pitch_b;  // shared-memory bytes per row slot (== 16 mod 128)
    int region_a;        // bytes of stream A inside a stage
    int stage_bytes;
    int stages;
    int nterms;          // 1: 16-bit activations, 2: FP32 activations (high + remainder)
    int off_bfrag, off_xsum, off_stage;   // shared-memory offsets
    const void *x;
    int x_dtype;
    void *y;
    int y_dtype;
    int topk;
    const int32_t *order;
    const int32_t *seg_expert;
    const int32_t *seg_begin;
    const int32_t *seg_count;
    const int32_t *num_segments;
    int max_segments;
    const float *route;
    int flat_rows;       // mode 3: term rows stored at the flat assignment index
    const uint64_t *y_table;   // mode 3, optional: per-rank base addresses of the term buffers (peer memory)
    int rows_per_rank;   // flat rows owned by each rank when y_table is set
    int *status;
};

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Bytes 0 and 2 (or 1 and 3) of `w` as the FP16 pair (1024+b_lo, 1024+b_hi), then minus `bias`
// (1024 + code offset) so the pair holds the exact signed codes.
__device__ __forceinline__ uint32_t pair02(uint32_t w, uint32_t bias) {
    return hsub2_u32(__byte_perm(w, 0x64646464u, 0x4240), bias);
}
__device__ __forceinline__ uint32_t pair13(uint32_t w, uint32_t bias) {
    return hsub2_u32(__byte_perm(w, 0x64646464u, 0x4341), bias);
}

__device__ __forceinline__ uint32_t lds_u32_a2(const uint8_t *p) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t *base = reinterpret_cast<const uint32_t *>(a & ~uintptr_t(3));
    return __byte_perm(base[0], base[1], (a & 2u) ? 0x5432 : 0x3210);
}
__device__ __forceinline__ uint32_t lds_u16_a2(const uint8_t *p) {
    return *reinterpret_cast<const uint16_t *>(p);
}

// One B fragment (and its optional remainder) for k16 block `f`.
struct BFrag {
    uint32_t h0, h1, l0, l1;
};
template <int NTERMS>
__device__ __forceinline__ BFrag load_bfrag(const uint2 *bfrag, int nfrag, int f, int lane) {
    BFrag b;
    const uint2 v = bfrag[f * 32 + lane];
    b.h0 = v.x; b.h1 = v.y; b.l0 = 0; b.l1 = 0;
    if (NTERMS == 2) {
        const uint2 u = bfrag[(nfrag + f) * 32 + lane];
        b.l0 = u.x; b.l1 = u.y;
    }
    return b;
}
template <int NTERMS>
__device__ __forceinline__ void mma_terms(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          const BFrag &b) {
    mma_f16(c, a0, a1, a2, a3, b.h0, b.h1);
    if (NTERMS == 2) mma_f16(c, a0, a1, a2, a3, b.l0, b.l1);
}

// ---------------------------------------------------------------------------------------------
// Per-format processing of one warp task: 16 rows x 256 K positions.
//   ra / rb : shared-memory address of the task's first packed byte in row g / row g+8
//   stab    : warp-private table filled by `header` (per row: scales / min terms)
//   f0      : index of the task's first k16 activation fragment
// `tot` accumulates rows (g, g+8) x tokens (2*tig, 2*tig+1).
// ---------------------------------------------------------------------------------------------
template <int FMT, int NTERMS>
struct MmaFormat;

// Q4_K: codes 0..15 placed at mantissa bits 6..9 of 16.0 -> pair value 16 + q with one shift and
// one logic op per pair; the constant 16 is folded into the per-sub-block min term.
template <int NTERMS>
struct MmaFormat<B200Q_Q4_K, NTERMS> {
    static constexpr int TASK_BYTES = 144;
    // lanes 0..31: row = lane & 15, sub-blocks 4*(lane>>4) .. +3 -> stab[row][sub] = (scale, minterm)
    __device__ static __forceinline__ void header(const uint8_t *row_task, int lane, float *stab) {
        const int part = lane >> 4;
        const uint4 hd = *reinterpret_cast<const uint4 *>(row_task);
        const float d = half_bits_to_float(hd.x & 0xffffu), dmin = half_bits_to_float(hd.x >> 16);
        uint32_t sc4, mn4;
        if (part == 0) {
            sc4 = hd.y & 0x3f3f3f3fu;
            mn4 = hd.z & 0x3f3f3f3fu;
        } else {
            sc4 = (hd.w & 0x0f0f0f0fu) | ((hd.y >> 2) & 0x30303030u);
            mn4 = ((hd.w >> 4) & 0x0f0f0f0fu) | ((hd.z >> 2) & 0x30303030u);
        }
        float2 *dst = reinterpret_cast<float2 *>(stab) + (lane & 15) * 8 + part * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float s = d * static_cast<float>((sc4 >> (8 * i)) & 0xffu);
            const float mn = dmin * static_cast<float>((mn4 >> (8 * i)) & 0xffu);
            dst[i] = make_float2(s, fmaf(16.0f, s, mn));
        }
    }
    __device__ static __forceinline__ uint32_t pk(uint32_t shifted) {
        return (shifted & 0x03c003c0u) | 0x4c004c00u;
    }
    __device__ static __forceinline__ void task(const uint8_t *ra, const uint8_t *rb, const float *stab,
                                                const uint2 *bfrag, int nfrag, const float *xsum, int f0, int lane,
                                                float (&tot)[4]) {
        const int g = lane >> 2, tig = lane & 3;
        const float2 *sa = reinterpret_cast<const float2 *>(stab) + g * 8;
        const float2 *sb = sa + 64;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint32_t qa0 = *reinterpret_cast<const uint32_t *>(ra + 16 + 32 * p + 4 * tig);
            const uint32_t qa1 = *reinterpret_cast<const uint32_t *>(ra + 32 + 32 * p + 4 * tig);
            const uint32_t qb0 = *reinterpret_cast<const uint32_t *>(rb + 16 + 32 * p + 4 * tig);
            const uint32_t qb1 = *reinterpret_cast<const uint32_t *>(rb + 32 + 32 * p + 4 * tig);
#pragma unroll
            for (int nib = 0; nib < 2; ++nib) {
                const int s = 2 * p + nib;
                const int f = f0 + 2 * s;
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                {
                    const BFrag b = load_bfrag<NTERMS>(bfrag, nfrag, f, lane);
                    const uint32_t a0 = nib ? pk(qa0 << 2) : pk(qa0 << 6);
                    const uint32_t a2 = nib ? pk(qa0 >> 6) : pk(qa0 >> 2);
                    const uint32_t a1 = nib ? pk(qb0 << 2) : pk(qb0 << 6);
                    const uint32_t a3 = nib ? pk(qb0 >> 6) : pk(qb0 >> 2);
                    mma_terms<NTERMS>(c, a0, a1, a2, a3, b);
                }
                {
                    const BFrag b = load_bfrag<NTERMS>(bfrag, nfrag, f + 1, lane);
                    const uint32_t a0 = nib ? pk(qa1 << 2) : pk(qa1 << 6);
                    const uint32_t a2 = nib ? pk(qa1 >> 6) : pk(qa1 >> 2);
                    const uint32_t a1 = nib ? pk(qb1 << 2) : pk(qb1 << 6);
                    const uint32_t a3 = nib ? pk(qb1 >> 6) : pk(qb1 >> 2);
                    mma_terms<NTERMS>(c, a0, a1, a2, a3, b);
                }
                const float2 xs = *reinterpret_cast<const float2 *>(xsum + (f >> 1) * 8 + 2 * tig);
                const float2 va = sa[s], vb = sb[s];
                tot[0] = fmaf(va.x, c[0], fmaf(-va.y, xs.x, tot[0]));
                tot[1] = fmaf(va.x, c[1], fmaf(-va.y, xs.y, tot[1]));
                tot[2] = fmaf(vb.x, c[2], fmaf(-vb.y, xs.x, tot[2]));
                tot[3] = fmaf(vb.x, c[3], fmaf(-vb.y, xs.y, tot[3]));
            }
        }
    }
};

// Q5_K: 5-bit codes assembled per byte, paired by byte permute, made exact by one packed subtract.
template <int NTERMS>
struct MmaFormat<B200Q_Q5_K, NTERMS> {
    static constexpr int TASK_BYTES = 176;
    __device__ static __forceinline__ void header(const uint8_t *row_task, int lane, float *stab) {
        const int part = lane >> 4;
        const uint4 hd = *reinterpret_cast<const uint4 *>(row_task);
        const float d = half_bits_to_float(hd.x & 0xffffu), dmin = half_bits_to_float(hd.x >> 16);
        uint32_t sc4, mn4;
        if (part == 0) {
            sc4 = hd.y & 0x3f3f3f3fu;
            mn4 = hd.z & 0x3f3f3f3fu;
        } else {
            sc4 = (hd.w & 0x0f0f0f0fu) | ((hd.y >> 2) & 0x30303030u);
            mn4 = ((hd.w >> 4) & 0x0f0f0f0fu) | ((hd.z >> 2) & 0x30303030u);
        }
        float2 *dst = reinterpret_cast<float2 *>(stab) + (lane & 15) * 8 + part * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            dst[i] = make_float2(d * static_cast<float>((sc4 >> (8 * i)) & 0xffu),
                                 dmin * static_cast<float>((mn4 >> (8 * i)) & 0xffu));
    }
    __device__ static __forceinline__ void task(const uint8_t *ra, const uint8_t *rb, const float *stab,
                                                const uint2 *bfrag, int nfrag, const float *xsum, int f0, int lane,
                                                float (&tot)[4]) {
        const int g = lane >> 2, tig = lane & 3;
        const float2 *sa = reinterpret_cast<const float2 *>(stab) + g * 8;
        const float2 *sb = sa + 64;
        const uint32_t bias = 0x64006400u;
        // high bits: byte e of qh holds bit s of element e for every sub-block s
        const uint32_t ha0 = *reinterpret_cast<const uint32_t *>(ra + 16 + 4 * tig);
        const uint32_t ha1 = *reinterpret_cast<const uint32_t *>(ra + 32 + 4 * tig);
        const uint32_t hb0 = *reinterpret_cast<const uint32_t *>(rb + 16 + 4 * tig);
        const uint32_t hb1 = *reinterpret_cast<const uint32_t *>(rb + 32 + 4 * tig);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint32_t qa0 = *reinterpret_cast<const uint32_t *>(ra + 48 + 32 * p + 4 * tig);
            const uint32_t qa1 = *reinterpret_cast<const uint32_t *>(ra + 64 + 32 * p + 4 * tig);
            const uint32_t qb0 = *reinterpret_cast<const uint32_t *>(rb + 48 + 32 * p + 4 * tig);
            const uint32_t qb1 = *reinterpret_cast<const uint32_t *>(rb + 64 + 32 * p + 4 * tig);
#pragma unroll
            for (int nib = 0; nib < 2; ++nib) {
                const int s = 2 * p + nib;
                const int f = f0 + 2 * s;
                // code = nibble | (bit s of the high-bit byte) << 4
                auto code = [&](uint32_t q, uint32_t h) -> uint32_t {
                    const uint32_t nibble = nib ? (q >> 4) & 0x0f0f0f0fu : q & 0x0f0f0f0fu;
                    const uint32_t hb = s <= 4 ? (h << (4 - s)) : (h >> (s - 4));
                    return nibble | (hb & 0x10101010u);
                };
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                {
                    const BFrag b = load_bfrag<NTERMS>(bfrag, nfrag, f, lane);
                    const uint32_t wa = code(qa0, ha0), wb = code(qb0, hb0);
                    mma_terms<NTERMS>(c, pair02(wa, bias), pair02(wb, bias), pair13(wa, bias), pair13(wb, bias), b);
                }
                {
                    const BFrag b = load_bfrag<NTERMS>(bfrag, nfrag, f + 1, lane);
                    const uint32_t wa = code(qa1, ha1), wb = code(qb1, hb1);
                    mma_terms<NTERMS>(c, pair02(wa, bias), pair02(wb, bias), pair13(wa, bias), pair13(wb, bias), b);
                }
                const float2 xs = *reinterpret_cast<const float2 *>(xsum + (f >> 1) * 8 + 2 * tig);
                const float2 va = sa[s], vb = sb[s];
                tot[0] = fmaf(va.x, c[0], fmaf(-va.y, xs.x, tot[0]));
                tot[1] = fmaf(va.x, c[1], fmaf(-va.y, xs.y, tot[1]));
                tot[2] = fmaf(vb.x, c[2], fmaf(-vb.y, xs.x, tot[2]));
                tot[3] = fmaf(vb.x, c[3], fmaf(-vb.y, xs.y, tot[3]));
            }
        }
    }
};

// Q6_K: 6-bit codes (stored +32) per 16-value scale group; one k16 step per scale group.
template <int NTERMS>
struct MmaFormat<B200Q_Q6_K, NTERMS> {
    static constexpr int TASK_BYTES = 210;
    // stab[row][16] floats: d * int8 scale
    __device__ static __forceinline__ void header(const uint8_t *row_task, int lane, float *stab) {
        const int part = lane >> 4;
        const float d = half_bits_to_float(lds_u16_a2(row_task + 208));
        const uint8_t *sc = row_task + 192 + 8 * part;
        float *dst = stab + (lane & 15) * 16 + part * 8;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t two = lds_u16_a2(sc + 2 * i);
            dst[2 * i] = d * static_cast<float>(static_cast<int>(static_cast<int8_t>(two & 0xffu)));
            dst[2 * i + 1] = d * static_cast<float>(static_cast<int>(static_cast<int8_t>(two >> 8)));
        }
    }
    __device__ static __forceinline__ void task(const uint8_t *ra, const uint8_t *rb, const float *stab,
                                                const uint2 *bfrag, int nfrag, const float *xsum, int f0, int lane,
                                                float (&tot)[4]) {
        (void)xsum;
        const int g = lane >> 2, tig = lane & 3;
        const float *sa = stab + g * 16;
        const float *sb = sa + 128;
        const uint32_t bias = 0x64206420u;  // 1024 + 32: removes the magic constant and the stored offset
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int ls = 0; ls < 2; ++ls) {  // elements 4*tig.. (first scale group) or 16+4*tig.. (second)
                const int l = 16 * ls + 4 * tig;
                const uint32_t Aa = lds_u32_a2(ra + 64 * half + l), Ba = lds_u32_a2(ra + 64 * half + 32 + l);
                const uint32_t Ha = lds_u32_a2(ra + 128 + 32 * half + l);
                const uint32_t Ab = lds_u32_a2(rb + 64 * half + l), Bb = lds_u32_a2(rb + 64 * half + 32 + l);
                const uint32_t Hb = lds_u32_a2(rb + 128 + 32 * half + l);
#pragma unroll
                for (int qd = 0; qd < 4; ++qd) {
                    auto code = [&](uint32_t A, uint32_t B, uint32_t H) -> uint32_t {
                        const uint32_t src = (qd & 1) ? B : A;
                        const uint32_t nibble = (qd >> 1) ? (src >> 4) & 0x0f0f0f0fu : src & 0x0f0f0f0fu;
                        const uint32_t hi = qd == 0 ? (H << 4) : qd == 1 ? (H << 2) : qd == 2 ? H : (H >> 2);
                        return nibble | (hi & 0x30303030u);
                    };
                    const int grp = 8 * half + 2 * qd + ls;          // 16-value scale group
                    const int f = f0 + grp;
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
                    const BFrag b = load_bfrag<NTERMS>(bfrag, nfrag, f, lane);
                    const uint32_t wa = code(Aa, Ba, Ha), wb = code(Ab, Bb, Hb);
                    mma_terms<NTERMS>(c, pair02(wa, bias), pair02(wb, bias), pair13(wa, bias), pair13(wb, bias), b);
                    const float va = sa[grp], vb = sb[grp];
                    tot[0] = fmaf(va, c[0], tot[0]);
                    tot[1] = fmaf(va, c[1], tot[1]);
                    tot[2] = fmaf(vb, c[2], tot[2]);
                    tot[3] = fmaf(vb, c[3], tot[3]);
                }
            }
        }
    }
};

// Q8_0: eight 34-byte blocks per task; signed bytes biased by 128, paired, made exact.
template <int NTERMS>
struct MmaFormat<B200Q_Q8_0, NTERMS> {
    static constexpr int TASK_BYTES = 272;
    // stab[row][8] floats: block scale d
    __device__ static __forceinline__ void header(const uint8_t *row_task, int lane, float *stab) {
        const int part = lane >> 4;
        float *dst = stab + (lane & 15) * 16 + part * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = half_bits_to_float(lds_u16_a2(row_task + 34 * (4 * part + i)));
    }
    __device__ static __forceinline__ void task(const uint8_t *ra, const uint8_t *rb, const float *stab,
                                                const uint2 *bfrag, int nfrag, const float *xsum, int f0, int lane,
                                                float (&tot)[4]) {
        (void)xsum;
        const int g = lane >> 2, tig = lane & 3;
        const float *sa = stab + g * 16;
        const float *sb = sa + 128;
        const uint32_t bias = 0x64806480u;  // 1024 + 128
#pragma unroll
        for (int blk = 0; blk < 8; ++blk) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t wa = lds_u32_a2(ra + 34 * blk + 2 + 16 * h + 4 * tig) ^ 0x80808080u;
                const uint32_t wb = lds_u32_a2(rb + 34 * blk + 2 + 16 * h + 4 * tig) ^ 0x80808080u;
                const BFrag b = load_bfrag<NTERMS>(bfrag, nfrag, f0 + 2 * blk + h, lane);
                mma_terms<NTERMS>(c, pair02(wa, bias), pair02(wb, bias), pair13(wa, bias), pair13(wb, bias), b);
            }
            const float va = sa[blk], vb = sb[blk];
            tot[0] = fmaf(va, c[0], tot[0]);
            tot[1] = fmaf(va, c[1], tot[1]);
            tot[2] = fmaf(vb, c[2], tot[2]);
            tot[3] = fmaf(vb, c[3], tot[3]);
        }
    }
};

// 16-byte aligned copy window of a row segment [g, g+len). The window never extends past `limit`
// (end of the weight matrix); bytes cut off there (fewer than 16) are returned as `tail`.
struct CopyWindow {
    uintptr_t start;
    uint32_t bytes;
    uint32_t tail;
};
__device__ __forceinline__ CopyWindow copy_window(uintptr_t g, uint32_t len, uintptr_t limit) {
    CopyWindow w;
    w.start = g & ~uintptr_t(15);
    uintptr_t end = (g + len + 15) & ~uintptr_t(15);
    w.tail = 0;
    if (end > limit) {
        end = limit & ~uintptr_t(15);
        w.tail = static_cast<uint32_t>((g + len) - end);
    }
    w.bytes = end > w.start ? static_cast<uint32_t>(end - w.start) : 0u;
    return w;
}

// ---------------------------------------------------------------------------------------------
// Activation preparation (consumer threads): scale each token by a power of two, split into FP16
// terms, store as B fragments; per 32 positions also the FP32 sum of the stored values (needed by
// the min terms of Q4_K / Q5_K).
//   fragment f, lane (g = lane>>2, tig = lane&3): positions 16 f + 4 tig + {0,2} -> b0, {1,3} -> b1
// ---------------------------------------------------------------------------------------------
template <int NTERMS, typename RowFn>
__device__ __forceinline__ void prepare_activations(RowFn row_of, int m_tokens, int k, const void *x, int x_dtype,
                                                    uint2 *bfrag, float *xsum, float *tok_scale, int ctid) {
    const int warp = ctid >> 5, lane = ctid & 31;
    const int nfrag = k >> 4;
    // 1. per-token power-of-two scale (warp w handles token w)
    {
        float amax = 0.f;
        if (warp < m_tokens) {
            const size_t base = static_cast<size_t>(row_of(warp)) * k;
            for (int i = lane; i < k; i += 32) amax = fmaxf(amax, fabsf(load_as_float(x, x_dtype, base + i)));
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (lane == 0 && warp < 8) {
            float s = 1.0f;
            if (amax > 0.f && amax < __int_as_float(0x7f800000)) {
                int e;
                frexpf(amax, &e);            // amax = f * 2^e, f in [0.5, 1)
                s = ldexpf(1.0f, min(14 - e, 100));   // scaled max in [2^13, 2^14)
            }
            tok_scale[warp] = s;
            tok_scale[8 + warp] = 1.0f / s;
        }
    }
    named_barrier_sync(1, MM_CTHREADS);
    // 2. fragments: warp handles 32-position chunks c = warp, warp+8, ...
    const int g = lane >> 2, tig = lane & 3;
    const bool live = g < m_tokens;
    const float s = tok_scale[g];
    const size_t base = live ? static_cast<size_t>(row_of(g)) * k : 0;
    for (int c = warp; c < (k >> 5); c += MM_WARPS) {
        float sum = 0.f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int f = 2 * c + h;
            const int k0 = 16 * f + 4 * tig;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (live) {
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = load_as_float(x, x_dtype, base + k0 + i) * s;
            }
            __half hi[4], lo[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                hi[i] = __float2half_rn(v[i]);
                const float r = v[i] - __half2float(hi[i]);
                lo[i] = __float2half_rn(r);
                sum += __half2float(hi[i]);
                if (NTERMS == 2) sum += __half2float(lo[i]);
            }
            uint2 out;
            out.x = static_cast<uint32_t>(__half_as_ushort(hi[0])) | (static_cast<uint32_t>(__half_as_ushort(hi[2])) << 16);
            out.y = static_cast<uint32_t>(__half_as_ushort(hi[1])) | (static_cast<uint32_t>(__half_as_ushort(hi[3])) << 16);
            bfrag[f * 32 + lane] = out;
            if (NTERMS == 2) {
                out.x = static_cast<uint32_t>(__half_as_ushort(lo[0])) | (static_cast<uint32_t>(__half_as_ushort(lo[2])) << 16);
                out.y = static_cast<uint32_t>(__half_as_ushort(lo[1])) | (static_cast<uint32_t>(__half_as_ushort(lo[3])) << 16);
                bfrag[(nfrag + f) * 32 + lane] = out;
            }
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (tig == 0) xsum[c * 8 + g] = sum;
    }
    named_barrier_sync(1, MM_CTHREADS);
}

template <int FMT_A, int FMT_B, int MODE, int NTERMS>
__global__ void __launch_bounds__(MM_THREADS, 1) mma_gemv_kernel(const MmaArgs a) {
    constexpr bool DUAL = (MODE == 1 || MODE == 2);
    constexpr bool GROUPED = (MODE >= 2);
    using FA = MmaFormat<FMT_A, NTERMS>;
    using FB = MmaFormat<FMT_B, NTERMS>;
    constexpr int QK_A = fmt_elems(FMT_A), QB_A = fmt_bytes(FMT_A);
    constexpr int QK_B = fmt_elems(FMT_B), QB_B = fmt_bytes(FMT_B);

    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty_bar = full_bar + MM_MAX_STAGES;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 256);
    float *tok_scale = reinterpret_cast<float *>(smem + 512);   // [8] scale, [8] inverse
    float *route_w = reinterpret_cast<float *>(smem + 640);     // [8]
    int *seg_tokens = reinterpret_cast<int *>(smem + 704);      // [8]
    float **out_ptr = reinterpret_cast<float **>(smem + 768);   // [8] mode 3 output row pointers
    float *stab_all = reinterpret_cast<float *>(smem + MM_CTRL_BYTES);
    float *partial = reinterpret_cast<float *>(smem + MM_CTRL_BYTES + MM_STAB_BYTES);
    uint2 *bfrag = reinterpret_cast<uint2 *>(smem + a.off_bfrag);
    float *xsum = reinterpret_cast<float *>(smem + a.off_xsum);
    uint8_t *stage_base = smem + a.off_stage;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = a.stages;
    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], MM_WARPS);
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();

    // Work: row blocks of 16*rg rows of every unit (matrix or expert segment), split evenly.
    const int rows_per_block = 16 * a.rg;
    const int blocks_per_unit = (a.n + rows_per_block - 1) / rows_per_block;
    long long units = 1;
    if (GROUPED) {
        int nseg = *a.num_segments;
        if (nseg > a.max_segments) nseg = a.max_segments;
        units = nseg;
    }
    const long long total_blocks = units * blocks_per_unit;
    const long long blk_begin = total_blocks * blockIdx.x / gridDim.x;
    const long long blk_end = total_blocks * (blockIdx.x + 1) / gridDim.x;
    if (blk_begin >= blk_end) return;
    const int kc = a.kp * 256;
    const int ktiles = (a.k + kc - 1) / kc;

    if (warp == MM_WARPS) {
        // ------------------------------------------------------------------ producer warp
        int it = 0;
        for (long long blk = blk_begin; blk < blk_end; ++blk) {
            const int unit = static_cast<int>(blk / blocks_per_unit);
            const int row0 = static_cast<int>(blk - static_cast<long long>(unit) * blocks_per_unit) * rows_per_block;
            const int rows = min(rows_per_block, a.n - row0);
            const int expert = GROUPED ? a.seg_expert[unit] : 0;
            const uint8_t *base_a = expert_matrix(a.wa, a.stride_a, a.table_a, expert);
            const uint8_t *base_b = DUAL ? expert_matrix(a.wb, a.stride_b, a.table_b, expert) : nullptr;
            for (int kt = 0; kt < ktiles; ++kt, ++it) {
                if (*abort_flag) return;
                const int s = it % S;
                if (it >= S && !mbar_wait_bounded(&empty_bar[s], ((it / S) - 1) & 1, a.status, STATUS_WAIT_EMPTY)) {
                    *abort_flag = 1;
                    return;
                }
                uint8_t *stage = stage_base + static_cast<size_t>(s) * a.stage_bytes;
                const int kvalid = min(kc, a.k - kt * kc);
                // contiguous mode: the whole tile is one "row" of rows * row_bytes
                const int copies = a.contig ? 1 : rows;
                const uint32_t len_a = a.contig ? static_cast<uint32_t>(rows) * a.rb_a
                                                : static_cast<uint32_t>(kvalid / QK_A * QB_A);
                const uint32_t len_b = !DUAL ? 0u
                                       : a.contig ? static_cast<uint32_t>(rows) * a.rb_b
                                                  : static_cast<uint32_t>(kvalid / QK_B * QB_B);
                // pass 1: total bytes of all aligned windows; the few bytes a window may not cover
                // at the very end of a matrix are copied by hand before the barrier is armed
                const uintptr_t lim_a = reinterpret_cast<uintptr_t>(base_a) + static_cast<size_t>(a.n) * a.rb_a;
                const uintptr_t lim_b = DUAL ? reinterpret_cast<uintptr_t>(base_b) + static_cast<size_t>(a.n) * a.rb_b : 0;
                uint32_t tx = 0;
                for (int r = lane; r < copies; r += 32) {
                    const uintptr_t ga = reinterpret_cast<uintptr_t>(base_a + static_cast<size_t>(row0 + r) * a.rb_a +
                                                                     static_cast<size_t>(kt) * a.seg_a);
                    const CopyWindow wa = copy_window(ga, len_a, lim_a);
                    tx += wa.bytes;
                    for (uint32_t i = 0; i < wa.tail; ++i)
                        stage[static_cast<size_t>(r) * a.pitch_a + wa.bytes + i] =
                            reinterpret_cast<const uint8_t *>(wa.start + wa.bytes)[i];
                    if (DUAL) {
                        const uintptr_t gb = reinterpret_cast<uintptr_t>(base_b + static_cast<size_t>(row0 + r) * a.rb_b +
                                                                         static_cast<size_t>(kt) * a.seg_b);
                        const CopyWindow wb = copy_window(gb, len_b, lim_b);
                        tx += wb.bytes;
                        for (uint32_t i = 0; i < wb.tail; ++i)
                            stage[a.region_a + static_cast<size_t>(r) * a.pitch_b + wb.bytes + i] =
                                reinterpret_cast<const uint8_t *>(wb.start + wb.bytes)[i];
                    }
                }
#pragma unroll
                for (int o = 16; o; o >>= 1) tx += __shfl_xor_sync(0xffffffffu, tx, o);
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    if (tx) mbar_arrive_expect_tx(&full_bar[s], tx);
                    else mbar_arrive(&full_bar[s]);
                }
                __syncwarp();
                // pass 2: one bulk copy per row segment (or per tile)
                for (int r = lane; r < copies; r += 32) {
                    const uintptr_t ga = reinterpret_cast<uintptr_t>(base_a + static_cast<size_t>(row0 + r) * a.rb_a +
                                                                     static_cast<size_t>(kt) * a.seg_a);
                    const CopyWindow wa = copy_window(ga, len_a, lim_a);
                    if (wa.bytes)
                        bulk_copy_g2s(stage + static_cast<size_t>(r) * a.pitch_a, reinterpret_cast<const void *>(wa.start),
                                      wa.bytes, &full_bar[s]);
                    if (DUAL) {
                        const uintptr_t gb = reinterpret_cast<uintptr_t>(base_b + static_cast<size_t>(row0 + r) * a.rb_b +
                                                                         static_cast<size_t>(kt) * a.seg_b);
                        const CopyWindow wb = copy_window(gb, len_b, lim_b);
                        if (wb.bytes)
                            bulk_copy_g2s(stage + a.region_a + static_cast<size_t>(r) * a.pitch_b,
                                          reinterpret_cast<const void *>(wb.start), wb.bytes, &full_bar[s]);
                    }
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumer warps
    const int ctid = tid;
    const int rgi = warp / a.kp, kpi = warp - rgi * a.kp;
    const int g = lane >> 2, tig = lane & 3;
    float *stab = stab_all + warp * 512;       // 2 KB per warp: stream A, stream B
    const int nfrag = a.k >> 4;
    int m_tokens = a.m;
    int seg_begin = 0;
    int cur_unit = -1, last_single = -1;

    if (!GROUPED) {
        prepare_activations<NTERMS>([](int t) { return t; }, a.m, a.k, a.x, a.x_dtype, bfrag, xsum, tok_scale, ctid);
    }

    int it = 0, pbuf = 0;
    for (long long blk = blk_begin; blk < blk_end; ++blk) {
        const int unit = static_cast<int>(blk / blocks_per_unit);
        const int row0 = static_cast<int>(blk - static_cast<long long>(unit) * blocks_per_unit) * rows_per_block;
        const uint8_t *base_a = a.wa, *base_b = a.wb;
        if (GROUPED) {
            const int expert = a.seg_expert[unit];
            base_a = expert_matrix(a.wa, a.stride_a, a.table_a, expert);
            if (DUAL) base_b = expert_matrix(a.wb, a.stride_b, a.table_b, expert);
            if (unit != cur_unit) {
                cur_unit = unit;
                seg_begin = a.seg_begin[unit];
                m_tokens = min(a.seg_count[unit], 8);
                int single = -1;
                if (MODE == 2 && m_tokens == 1) single = a.order[seg_begin] / a.topk;
                const bool reuse = (single >= 0 && single == last_single);
                last_single = single;
                if (!reuse) {
                    named_barrier_sync(1, MM_CTHREADS);      // previous activations no longer in use
                    if (ctid < m_tokens) {
                        const int flat = a.order[seg_begin + ctid];
                        seg_tokens[ctid] = (MODE == 2) ? flat / a.topk : seg_begin + ctid;
                        if (MODE == 3) {
                            route_w[ctid] = a.route[flat];
                            out_ptr[ctid] = term_row_pointer(static_cast<float *>(a.y), a.y_table, a.rows_per_rank, a.n, a.flat_rows ? flat : seg_begin + ctid);
                        }
                    }
                    named_barrier_sync(1, MM_CTHREADS);
                    prepare_activations<NTERMS>([&](int t) { return seg_tokens[t]; }, m_tokens, a.k, a.x, a.x_dtype,
                                                bfrag, xsum, tok_scale, ctid);
                }
            }
        }
        const int my_row = row0 + 16 * rgi;            // first row of this warp's row group
        const bool rows_live = my_row < a.n && warp < a.cw;
        float tot_a[4] = {0.f, 0.f, 0.f, 0.f}, tot_b[4] = {0.f, 0.f, 0.f, 0.f};

        for (int kt = 0; kt < ktiles; ++kt, ++it) {
            const int s = it % S;
            if (!mbar_wait_bounded(&full_bar[s], (it / S) & 1, a.status, STATUS_WAIT_FULL)) {
                *abort_flag = 1;
                return;
            }
            const int k0 = kt * kc + kpi * 256;
            if (rows_live && k0 < a.k) {
                const uint8_t *stage = stage_base + static_cast<size_t>(s) * a.stage_bytes;
                const int f0 = k0 >> 4;
                {
                    // rows beyond n read stale slot bytes; their results are never stored
                    const size_t seg_off = static_cast<size_t>(kt) * a.seg_a;
                    const int task_off = kpi * (256 / QK_A * QB_A);
                    auto slot = [&](int r) -> const uint8_t * {
                        const int head_row = a.contig ? row0 : my_row + r;
                        const int head = static_cast<int>(
                            reinterpret_cast<uintptr_t>(base_a + static_cast<size_t>(head_row) * a.rb_a + seg_off) & 15);
                        return stage + static_cast<size_t>(16 * rgi + r) * a.pitch_a + head + task_off;
                    };
                    FA::header(slot(lane & 15), lane, stab);
                    __syncwarp();
                    FA::task(slot(g), slot(g + 8), stab, bfrag, nfrag, xsum, f0, lane, tot_a);
                }
                if (DUAL) {
                    const size_t seg_off = static_cast<size_t>(kt) * a.seg_b;
                    const int task_off = kpi * (256 / QK_B * QB_B);
                    auto slot = [&](int r) -> const uint8_t * {
                        const int head_row = a.contig ? row0 : my_row + r;
                        const int head = static_cast<int>(
                            reinterpret_cast<uintptr_t>(base_b + static_cast<size_t>(head_row) * a.rb_b + seg_off) & 15);
                        return stage + a.region_a + static_cast<size_t>(16 * rgi + r) * a.pitch_b + head + task_off;
                    };
                    FB::header(slot(lane & 15), lane, stab + 256);
                    __syncwarp();
                    FB::task(slot(g), slot(g + 8), stab + 256, bfrag, nfrag, xsum, f0, lane, tot_b);
                }
                __syncwarp();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
        }

        // Combine the kp partial sums of every row group in fixed order and store.
        float *pb = partial + pbuf * MM_PART_FLOATS + warp * 256;
        if (warp < a.cw) {
            // [row 0..15][token 0..7][stream]
            pb[((g)*8 + 2 * tig) * 2 + 0] = tot_a[0];
            pb[((g)*8 + 2 * tig + 1) * 2 + 0] = tot_a[1];
            pb[((g + 8) * 8 + 2 * tig) * 2 + 0] = tot_a[2];
            pb[((g + 8) * 8 + 2 * tig + 1) * 2 + 0] = tot_a[3];
            if (DUAL) {
                pb[((g)*8 + 2 * tig) * 2 + 1] = tot_b[0];
                pb[((g)*8 + 2 * tig + 1) * 2 + 1] = tot_b[1];
                pb[((g + 8) * 8 + 2 * tig) * 2 + 1] = tot_b[2];
                pb[((g + 8) * 8 + 2 * tig + 1) * 2 + 1] = tot_b[3];
            }
        }
        named_barrier_sync(2, MM_CTHREADS);
        const int outs = a.rg * 128;
        for (int o = ctid; o < outs; o += MM_CTHREADS) {
            const int rgo = o >> 7, r = (o >> 3) & 15, t = o & 7;
            const int orow = row0 + 16 * rgo + r;
            if (orow >= a.n || t >= m_tokens) continue;
            const float *src = partial + pbuf * MM_PART_FLOATS + (rgo * a.kp) * 256 + (r * 8 + t) * 2;
            float pa = 0.f, pbv = 0.f;
            for (int kq = 0; kq < a.kp; ++kq) {
                pa += src[kq * 256];
                if (DUAL) pbv += src[kq * 256 + 1];
            }
            const float inv = tok_scale[8 + t];
            pa *= inv;
            pbv *= inv;
            if (MODE == 0) store_from_float(a.y, a.y_dtype, static_cast<size_t>(t) * a.n + orow, pa);
            else if (MODE == 1)
                store_from_float(a.y, a.y_dtype, static_cast<size_t>(t) * a.n + orow, swiglu_f32(pa, pbv));
            else if (MODE == 2)
                static_cast<float *>(a.y)[static_cast<size_t>(seg_begin + t) * a.n + orow] = swiglu_f32(pa, pbv);
            else
                out_ptr[t][orow] = pa * route_w[t];
        }
        pbuf ^= 1;
    }
}

}  // namespace b200q
