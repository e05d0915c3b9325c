// Per-format lane decoders for the streaming GEMV kernels.
//
// A "slice" is 2048 consecutive K positions of one packed weight row. One warp computes the dot
// product of one row-slice with the matching 2048 activations, which it keeps in registers
// (64 floats per lane), so the activations are read once per (token, slice) and the packed row
// bytes are read once from shared memory. Which K positions a lane owns is a property of the
// format, chosen so that every lane owns whole scale groups:
//
//   Q4_K / Q5_K  lane = (super-block 0..7 of the slice) x (64-value chunk 0..3): two whole
//                sub-blocks (low nibbles, high nibbles) = 32 packed bytes, 64 contiguous x.
//   Q6_K         two steps of four super-blocks; lane = (super-block, 128-value half, 8-byte run):
//                4 quarters x 8 values, each quarter inside one 16-value scale group.
//   Q8_0         two steps; lane = one 34-byte block.
//
// Arithmetic: integer codes are converted exactly to FP32 and multiplied with FP32 activations
// (packed two-wide FMA), scales and minima are applied once per scale group. All products
// d*scale*q are exact in FP32, so the only difference from the reference's per-weight
// (d*sc)*q - dmin*mn evaluation (mini_llm/ops/quantized_linear.py:91-172) is summation order.
#pragma once

#include "common.cuh"

namespace b200q {

constexpr int SLICE_K = 2048;
constexpr int XREGS = 64;

// Four unsigned bytes of `w` -> four floats (exact).
__device__ __forceinline__ void cvt_u8x4(uint32_t w, float &f0, float &f1, float &f2, float &f3) {
    f0 = static_cast<float>(w & 0xffu);
    f1 = static_cast<float>((w >> 8) & 0xffu);
    f2 = static_cast<float>((w >> 16) & 0xffu);
    f3 = static_cast<float>(w >> 24);
}

// Four signed bytes of `w` -> four floats (exact).
__device__ __forceinline__ void cvt_s8x4(uint32_t w, float &f0, float &f1, float &f2, float &f3) {
    f0 = static_cast<float>(static_cast<int>(static_cast<int8_t>(w & 0xffu)));
    f1 = static_cast<float>(static_cast<int>(static_cast<int8_t>((w >> 8) & 0xffu)));
    f2 = static_cast<float>(static_cast<int>(static_cast<int8_t>((w >> 16) & 0xffu)));
    f3 = static_cast<float>(static_cast<int>(static_cast<int8_t>(w >> 24)));
}

// acc += (four codes of w as floats) . x[0..3], as two packed FMAs.
__device__ __forceinline__ void fma_u8x4(uint32_t w, const float *x, float2 &acc0, float2 &acc1) {
    float f0, f1, f2, f3;
    cvt_u8x4(w, f0, f1, f2, f3);
    acc0 = __ffma2_rn(make_float2(f0, f1), make_float2(x[0], x[1]), acc0);
    acc1 = __ffma2_rn(make_float2(f2, f3), make_float2(x[2], x[3]), acc1);
}
__device__ __forceinline__ void fma_s8x4(uint32_t w, const float *x, float2 &acc0, float2 &acc1) {
    float f0, f1, f2, f3;
    cvt_s8x4(w, f0, f1, f2, f3);
    acc0 = __ffma2_rn(make_float2(f0, f1), make_float2(x[0], x[1]), acc0);
    acc1 = __ffma2_rn(make_float2(f2, f3), make_float2(x[2], x[3]), acc1);
}

// 32-bit load from shared memory at an address that is only 2-byte aligned.
__device__ __forceinline__ uint32_t lds_u32_align2(const uint8_t *p) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t *base = reinterpret_cast<const uint32_t *>(a & ~uintptr_t(3));
    const uint32_t lo = base[0], hi = base[1];
    return __byte_perm(lo, hi, (a & 2) ? 0x5432 : 0x3210);
}

// 6-bit scale/min pairs of sub-blocks 2j and 2j+1 of a Q4_K/Q5_K super-block.
// m0,m1,m2 are the three little-endian words of the 12 metadata bytes
// (mini_llm/ops/quantized_weight.py:221-225 of the reference).
__device__ __forceinline__ void kquant_scale_min(uint32_t m0, uint32_t m1, uint32_t m2, int j, float &sc_a,
                                                 float &sc_b, float &mn_a, float &mn_b) {
    const int sh = (j & 1) * 16;
    const uint32_t a = (m0 >> sh) & 0xffffu, b = (m1 >> sh) & 0xffffu, c = (m2 >> sh) & 0xffffu;
    uint32_t sc2, mn2;
    if (j < 2) {
        sc2 = a & 0x3f3fu;
        mn2 = b & 0x3f3fu;
    } else {
        sc2 = (c & 0x0f0fu) | ((a >> 2) & 0x3030u);
        mn2 = ((c >> 4) & 0x0f0fu) | ((b >> 2) & 0x3030u);
    }
    sc_a = static_cast<float>(sc2 & 0xffu);
    sc_b = static_cast<float>(sc2 >> 8);
    mn_a = static_cast<float>(mn2 & 0xffu);
    mn_b = static_cast<float>(mn2 >> 8);
}

template <int FMT>
struct LaneDecoder;

// ------------------------------------------------------------------------------------------ Q4_K
template <>
struct LaneDecoder<B200Q_Q4_K> {
    static constexpr int NSUM = 2;
    // x registers of `lane` for slice `slice`: 64 contiguous activations.
    __device__ static __forceinline__ int x_offset(int slice, int lane, int step, int part) {
        (void)step; (void)part;
        return slice * SLICE_K + (lane >> 2) * 256 + (lane & 3) * 64;
    }
    __device__ static __forceinline__ void load_x(const float *x, int k, int slice, int lane, float (&xr)[XREGS],
                                                  float (&xs)[4 * 2]) {
        const int k0 = slice * SLICE_K + (lane >> 2) * 256 + (lane & 3) * 64;
        const bool ok = k0 < k;
        const float4 *src = reinterpret_cast<const float4 *>(x + (ok ? k0 : 0));
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float4 v = ok ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            xr[4 * i] = v.x; xr[4 * i + 1] = v.y; xr[4 * i + 2] = v.z; xr[4 * i + 3] = v.w;
        }
        float a = 0.f, b = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) { a += xr[i]; b += xr[32 + i]; }
        xs[0] = a; xs[1] = b;
    }
    // Partial dot of one packed row (shared memory, 16-byte aligned super-blocks) with the slice.
    __device__ static __forceinline__ float dot(const uint8_t *row, int k, int slice, int lane,
                                                const float (&xr)[XREGS], const float (&xs)[4 * 2]) {
        const int sb = slice * 8 + (lane >> 2);
        if (sb * 256 >= k) return 0.f;
        const int j = lane & 3;
        const uint8_t *blk = row + sb * 144;
        const uint4 hd = *reinterpret_cast<const uint4 *>(blk);
        const uint4 qa = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * j);
        const uint4 qb = *reinterpret_cast<const uint4 *>(blk + 32 + 32 * j);
        float sc_a, sc_b, mn_a, mn_b;
        kquant_scale_min(hd.y, hd.z, hd.w, j, sc_a, sc_b, mn_a, mn_b);
        const float d = half_bits_to_float(hd.x & 0xffffu), dmin = half_bits_to_float(hd.x >> 16);
        const uint32_t q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        float2 lo0 = make_float2(0.f, 0.f), lo1 = lo0, hi0 = lo0, hi1 = lo0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            fma_u8x4(q[i] & 0x0f0f0f0fu, &xr[4 * i], lo0, lo1);
            fma_u8x4((q[i] >> 4) & 0x0f0f0f0fu, &xr[32 + 4 * i], hi0, hi1);
        }
        const float dot_a = (lo0.x + lo0.y) + (lo1.x + lo1.y);
        const float dot_b = (hi0.x + hi0.y) + (hi1.x + hi1.y);
        return (d * sc_a) * dot_a + (d * sc_b) * dot_b - (dmin * mn_a) * xs[0] - (dmin * mn_b) * xs[1];
    }
};

// ------------------------------------------------------------------------------------------ Q5_K
template <>
struct LaneDecoder<B200Q_Q5_K> {
    __device__ static __forceinline__ void load_x(const float *x, int k, int slice, int lane, float (&xr)[XREGS],
                                                  float (&xs)[4 * 2]) {
        LaneDecoder<B200Q_Q4_K>::load_x(x, k, slice, lane, xr, xs);
    }
    __device__ static __forceinline__ float dot(const uint8_t *row, int k, int slice, int lane,
                                                const float (&xr)[XREGS], const float (&xs)[4 * 2]) {
        const int sb = slice * 8 + (lane >> 2);
        if (sb * 256 >= k) return 0.f;
        const int j = lane & 3;
        const uint8_t *blk = row + sb * 176;
        const uint4 hd = *reinterpret_cast<const uint4 *>(blk);
        const uint4 ha = *reinterpret_cast<const uint4 *>(blk + 16);
        const uint4 hb = *reinterpret_cast<const uint4 *>(blk + 32);
        const uint4 qa = *reinterpret_cast<const uint4 *>(blk + 48 + 32 * j);
        const uint4 qb = *reinterpret_cast<const uint4 *>(blk + 64 + 32 * j);
        float sc_a, sc_b, mn_a, mn_b;
        kquant_scale_min(hd.y, hd.z, hd.w, j, sc_a, sc_b, mn_a, mn_b);
        const float d = half_bits_to_float(hd.x & 0xffffu), dmin = half_bits_to_float(hd.x >> 16);
        const uint32_t q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        const uint32_t h[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
        float2 lo0 = make_float2(0.f, 0.f), lo1 = lo0, hi0 = lo0, hi1 = lo0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t hw = h[i] >> (2 * j);  // bit 0: sub-block 2j, bit 1: sub-block 2j+1
            const uint32_t lo = (q[i] & 0x0f0f0f0fu) | ((hw << 4) & 0x10101010u);
            const uint32_t hi = ((q[i] >> 4) & 0x0f0f0f0fu) | ((hw << 3) & 0x10101010u);
            fma_u8x4(lo, &xr[4 * i], lo0, lo1);
            fma_u8x4(hi, &xr[32 + 4 * i], hi0, hi1);
        }
        const float dot_a = (lo0.x + lo0.y) + (lo1.x + lo1.y);
        const float dot_b = (hi0.x + hi0.y) + (hi1.x + hi1.y);
        return (d * sc_a) * dot_a + (d * sc_b) * dot_b - (dmin * mn_a) * xs[0] - (dmin * mn_b) * xs[1];
    }
};

// ------------------------------------------------------------------------------------------ Q6_K
template <>
struct LaneDecoder<B200Q_Q6_K> {
    __device__ static __forceinline__ void load_x(const float *x, int k, int slice, int lane, float (&xr)[XREGS],
                                                  float (&xs)[4 * 2]) {
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const int sb = slice * 8 + t * 4 + (lane >> 3);
            const int kbase = sb * 256 + ((lane >> 2) & 1) * 128 + (lane & 3) * 8;
            const bool ok = sb * 256 < k;
#pragma unroll
            for (int qd = 0; qd < 4; ++qd) {
                const float4 *src = reinterpret_cast<const float4 *>(x + (ok ? kbase + 32 * qd : 0));
                float4 v0 = ok ? src[0] : make_float4(0.f, 0.f, 0.f, 0.f);
                float4 v1 = ok ? src[1] : make_float4(0.f, 0.f, 0.f, 0.f);
                float *dst = &xr[32 * t + 8 * qd];
                dst[0] = v0.x; dst[1] = v0.y; dst[2] = v0.z; dst[3] = v0.w;
                dst[4] = v1.x; dst[5] = v1.y; dst[6] = v1.z; dst[7] = v1.w;
                xs[4 * t + qd] = ((v0.x + v0.y) + (v0.z + v0.w)) + ((v1.x + v1.y) + (v1.z + v1.w));
            }
        }
    }
    __device__ static __forceinline__ float dot(const uint8_t *row, int k, int slice, int lane,
                                                const float (&xr)[XREGS], const float (&xs)[4 * 2]) {
        float total = 0.f;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const int sb = slice * 8 + t * 4 + (lane >> 3);
            if (sb * 256 >= k) continue;
            const int half = (lane >> 2) & 1, l0 = (lane & 3) * 8;
            const uint8_t *blk = row + sb * 210;  // 2-byte aligned
            const uint8_t *ql = blk + 64 * half + l0;
            const uint8_t *qh = blk + 128 + 32 * half + l0;
            const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(blk + 208));
            const int8_t *scales = reinterpret_cast<const int8_t *>(blk + 192 + 8 * half + (l0 >> 4));
            float part = 0.f;
#pragma unroll
            for (int w = 0; w < 2; ++w) {
                const uint32_t A = lds_u32_align2(ql + 4 * w);
                const uint32_t B = lds_u32_align2(ql + 32 + 4 * w);
                const uint32_t H = lds_u32_align2(qh + 4 * w);
                const uint32_t q0 = (A & 0x0f0f0f0fu) | ((H << 4) & 0x30303030u);
                const uint32_t q1 = (B & 0x0f0f0f0fu) | ((H << 2) & 0x30303030u);
                const uint32_t q2 = ((A >> 4) & 0x0f0f0f0fu) | (H & 0x30303030u);
                const uint32_t q3 = ((B >> 4) & 0x0f0f0f0fu) | ((H >> 2) & 0x30303030u);
                const uint32_t qq[4] = {q0, q1, q2, q3};
#pragma unroll
                for (int qd = 0; qd < 4; ++qd) {
                    float2 a0 = make_float2(0.f, 0.f), a1 = a0;
                    fma_u8x4(qq[qd], &xr[32 * t + 8 * qd + 4 * w], a0, a1);
                    const float sc = d * static_cast<float>(static_cast<int>(scales[2 * qd]));
                    part += sc * ((a0.x + a0.y) + (a1.x + a1.y));
                }
            }
            // the stored code is q+32: remove 32 * sum(x) once per scale group
#pragma unroll
            for (int qd = 0; qd < 4; ++qd) {
                const float sc = d * static_cast<float>(static_cast<int>(scales[2 * qd]));
                part -= (32.0f * sc) * xs[4 * t + qd];
            }
            total += part;
        }
        return total;
    }
};

// ------------------------------------------------------------------------------------------ Q8_0
template <>
struct LaneDecoder<B200Q_Q8_0> {
    __device__ static __forceinline__ void load_x(const float *x, int k, int slice, int lane, float (&xr)[XREGS],
                                                  float (&xs)[4 * 2]) {
        (void)xs;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const int k0 = slice * SLICE_K + t * 1024 + lane * 32;
            const bool ok = k0 < k;
            const float4 *src = reinterpret_cast<const float4 *>(x + (ok ? k0 : 0));
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float4 v = ok ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                float *dst = &xr[32 * t + 4 * i];
                dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
            }
        }
    }
    __device__ static __forceinline__ float dot(const uint8_t *row, int k, int slice, int lane,
                                                const float (&xr)[XREGS], const float (&xs)[4 * 2]) {
        (void)xs;
        float total = 0.f;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const int b = slice * 64 + t * 32 + lane;
            if (b * 32 >= k) continue;
            const uint8_t *blk = row + b * 34;  // 2-byte aligned
            const uintptr_t a = reinterpret_cast<uintptr_t>(blk);
            const uint32_t *base = reinterpret_cast<const uint32_t *>(a & ~uintptr_t(3));
            const bool odd = (a & 2) != 0;  // block starts in the upper half of base[0]
            uint32_t wv[9];
#pragma unroll
            for (int i = 0; i < 9; ++i) wv[i] = base[i];
            const float d = half_bits_to_float(odd ? (wv[0] >> 16) : (wv[0] & 0xffffu));
            const uint32_t sel = odd ? 0x7654u : 0x5432u;
            float2 a0 = make_float2(0.f, 0.f), a1 = a0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t q = __byte_perm(wv[i], wv[i + 1], sel);
                fma_s8x4(q, &xr[32 * t + 4 * i], a0, a1);
            }
            total += d * ((a0.x + a0.y) + (a1.x + a1.y));
        }
        return total;
    }
};

// ------------------------------------------------------------------------------------------ Q4_0
// 18-byte blocks of 32 values: fp16 d, 16 code bytes (low nibbles = values 0..15, high nibbles =
// values 16..31), weight = d * (code - 8) (mini_llm/ops/quantized_weight.py:212-216).
template <>
struct LaneDecoder<B200Q_Q4_0> {
    __device__ static __forceinline__ void load_x(const float *x, int k, int slice, int lane, float (&xr)[XREGS],
                                                  float (&xs)[4 * 2]) {
        LaneDecoder<B200Q_Q8_0>::load_x(x, k, slice, lane, xr, xs);       // 32 consecutive activations per block
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) s += xr[32 * t + i];
            xs[4 * t] = s;
        }
    }
    __device__ static __forceinline__ float dot(const uint8_t *row, int k, int slice, int lane,
                                                const float (&xr)[XREGS], const float (&xs)[4 * 2]) {
        float total = 0.f;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const int b = slice * 64 + t * 32 + lane;
            if (b * 32 >= k) continue;
            const uint8_t *blk = row + b * 18;  // 2-byte aligned
            const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(blk));
            float2 a0 = make_float2(0.f, 0.f), a1 = a0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t q = lds_u32_align2(blk + 2 + 4 * i);
                fma_u8x4(q & 0x0f0f0f0fu, &xr[32 * t + 4 * i], a0, a1);
                fma_u8x4((q >> 4) & 0x0f0f0f0fu, &xr[32 * t + 16 + 4 * i], a0, a1);
            }
            total += d * (((a0.x + a0.y) + (a1.x + a1.y)) - 8.0f * xs[4 * t]);
        }
        return total;
    }
};

// ------------------------------------------------------------------------------------------ Q3_K
// 110-byte super-blocks of 256 values: hmask[32] | qs[64] | 12 scale bytes | fp16 d. Value p takes its two
// low bits from qs[32*(p/128) + p%32] >> 2*((p/32)%4) and is lowered by 4 unless bit p/32 of hmask[p%32]
// is set; sixteen 6-bit scales (minus 32) apply per 16 values (mini_llm/ops/quantized_weight.py:251-265).
// A lane covers 64 consecutive positions: one 32-byte half of qs at two shifts, two mask bits, four scales.
template <>
struct LaneDecoder<B200Q_Q3_K> {
    __device__ static __forceinline__ void load_x(const float *x, int k, int slice, int lane, float (&xr)[XREGS],
                                                  float (&xs)[4 * 2]) {
        LaneDecoder<B200Q_Q4_K>::load_x(x, k, slice, lane, xr, xs);       // 64 consecutive activations
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) s += xr[16 * g + i];
            xs[g] = s;
        }
    }
    __device__ static __forceinline__ float dot(const uint8_t *row, int k, int slice, int lane,
                                                const float (&xr)[XREGS], const float (&xs)[4 * 2]) {
        const int sb = slice * 8 + (lane >> 2);
        if (sb * 256 >= k) return 0.f;
        const int j = lane & 3;                                  // positions 64j .. 64j+63 of the super-block
        const uint8_t *blk = row + sb * 110;                     // 2-byte aligned
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(blk + 108));
        const uint8_t *qs = blk + 32 + 32 * (j >> 1);
        const int sh = 4 * (j & 1);                              // shifts 2*(2*(j&1)) and +2
        float total = 0.f;
#pragma unroll
        for (int part = 0; part < 2; ++part) {                   // 32 positions each: mask bit 2j + part
            float2 a0 = make_float2(0.f, 0.f), a1 = a0, b0 = a0, b1 = a0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t q = lds_u32_align2(qs + 4 * i), h = lds_u32_align2(blk + 4 * i);
                const uint32_t code = ((q >> (sh + 2 * part)) & 0x03030303u) | (((h >> (2 * j + part)) & 0x01010101u) << 2);
                if (i < 4) fma_u8x4(code, &xr[32 * part + 4 * i], a0, a1);
                else fma_u8x4(code, &xr[32 * part + 4 * i], b0, b1);
            }
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int s = 4 * j + 2 * part + half;           // scale index = position / 16
                const int sc = (((blk[96 + (s & 7)] >> (4 * (s >> 3))) & 15) | (((blk[104 + (s & 3)] >> (2 * (s >> 2))) & 3) << 4)) - 32;
                const float sum = half ? (b0.x + b0.y) + (b1.x + b1.y) : (a0.x + a0.y) + (a1.x + a1.y);
                total += (d * static_cast<float>(sc)) * (sum - 4.0f * xs[2 * part + half]);
            }
        }
        return total;
    }
};

}  // namespace b200q
