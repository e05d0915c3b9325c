// Q6_K and Q8_0 in device-side tile layouts, and the tensor-core GEMV that reads them (sm_100a).
//
// A GGUF Q6_K super-block is 210 bytes (ql[128] | qh[64] | int8 scales[16] | fp16 d), so rows and
// blocks start on 2-byte boundaries only: no 128-bit load, no aligned bulk copy, and every 32-bit
// fetch of a code word straddles two words half of the time. The kernels that read the native
// layout therefore stage rows through shared memory and pay two loads plus a byte permute per
// word. Weights are written once and read on every decode step, so the bytes are re-ordered once,
// at upload, into tiles that a warp can consume straight from global memory:
//
//   tile = 16 rows x 1 super-block = 3360 bytes (the size of the 16 native blocks, 16-byte aligned)
//     [   0, 3072)  six planes of 512 bytes; plane p holds one uint4 per lane (lane*16):
//                   planes 0-2 = the 12 code words of row g = lane>>2, planes 3-5 = row g+8
//     [3072, 3328)  16 rows x 16 scale bytes, stored as scale+128 (unsigned)
//     [3328, 3360)  16 x fp16 d
//   tiles are ordered (row group, super-block), so a row group's K range is contiguous.
//
// Code words: lane tig = lane&3 owns, in each 16-value scale group s of the block, the values
// 4*tig .. 4*tig+3. For chunk c = 0..3 (scale groups c, c+2, c+4, c+6 of one half: s = 8*(c>>1) +
// 2*j + (c&1), j = 0..3) three words W0..W2 hold its 16 six-bit codes as FP16-pair fields:
//   Wj (j<3): bits [0,6) value0, [16,22) value2 of group j  -> pair P0
//             bits [6,12) value1, [22,28) value3 of group j -> pair P1
//   group j = 3: low nibbles of (value0, value2) in W0[12,16) / W0[28,32), of (value1, value3) in
//             W1[12,16) / W1[28,32); high two bits in W2[12,14) / W2[28,30) and W2[14,16) / W2[30,32)
// so one AND-OR (after at most one shift) turns a field into the FP16 pair (1024+code, 1024+code),
// and one packed add of -1056 gives the exact signed codes (code - 32) as an mma A operand. The
// pairing (values 0,2 | 1,3) matches the activation fragments of prepare_fragments().
//
// The re-ordering is lossless: b200q_q6k_untile restores the GGUF bytes bit for bit.
#pragma once

#include "mma_direct.cuh"

namespace b200q {

constexpr int Q6T_TILE_BYTES = 3360;
constexpr int Q6T_SCALES_OFF = 3072;
constexpr int Q6T_D_OFF = 3328;
constexpr int Q6T_WARPS = 16;
constexpr int Q6T_THREADS = Q6T_WARPS * 32;
constexpr int Q6T_CTRL_BYTES = 1024;
constexpr int Q6T_PART_FLOATS = Q6T_WARPS * 128;           // [warp][16 rows][8 tokens]
constexpr int Q6T_PART_BYTES = 2 * Q6T_PART_FLOATS * 4;    // double buffered

struct Q6TiledArgs {
    const uint8_t *w;
    long long stride;
    const unsigned long long *table;
    int n, k, m;
    int kp, rg;
    int nterms;
    int off_bfrag;
    const void *x;
    int x_dtype;
    void *y;
    int y_dtype;
    const int32_t *order;
    const int32_t *seg_expert;
    const int32_t *seg_begin;
    const int32_t *seg_count;
    const int32_t *num_segments;
    int max_segments;
    const float *route;
    int flat_rows;
    const uint64_t *y_table;
    int rows_per_rank;
};

// Code of value `i` (0..3) of lane `tig` in scale group s of a native block.
__host__ __device__ inline uint32_t q6k_native_code(const uint8_t *blk, int s, int tig, int i) {
    const int h = s >> 3, j = (s >> 1) & 3, l = 16 * (s & 1) + 4 * tig + i;
    const uint32_t qlb = blk[64 * h + 32 * (j & 1) + l];
    const uint32_t nib = (j >> 1) ? (qlb >> 4) : (qlb & 15u);
    const uint32_t hi = (blk[128 + 32 * h + l] >> (2 * j)) & 3u;
    return nib | (hi << 4);
}

// The three words of chunk c for lane tig of one native block.
__host__ __device__ inline void q6k_pack_chunk(const uint8_t *blk, int c, int tig, uint32_t (&w)[3]) {
    uint32_t code[4][4];
    for (int j = 0; j < 4; ++j)
        for (int i = 0; i < 4; ++i) code[j][i] = q6k_native_code(blk, 8 * (c >> 1) + 2 * j + (c & 1), tig, i);
    for (int j = 0; j < 3; ++j)
        w[j] = code[j][0] | (code[j][2] << 16) | (code[j][1] << 6) | (code[j][3] << 22);
    w[0] |= ((code[3][0] & 15u) << 12) | ((code[3][2] & 15u) << 28);
    w[1] |= ((code[3][1] & 15u) << 12) | ((code[3][3] & 15u) << 28);
    w[2] |= ((code[3][0] >> 4) << 12) | ((code[3][2] >> 4) << 28) | ((code[3][1] >> 4) << 14) | ((code[3][3] >> 4) << 30);
}

// Inverse of q6k_pack_chunk: code of (group j of the chunk, value i).
__host__ __device__ inline uint32_t q6k_tiled_code(const uint32_t (&w)[3], int j, int i) {
    const int half = (i >> 1) * 16;            // values 0,1 in the low half-word, 2,3 in the high one
    const int odd = i & 1;
    if (j < 3) return (w[j] >> (half + 6 * odd)) & 63u;
    const uint32_t nib = (w[odd] >> (half + 12)) & 15u;
    const uint32_t hi = (w[2] >> (half + 12 + 2 * odd)) & 3u;
    return nib | (hi << 4);
}

struct Q6TileRegs {
    uint4 c[6];      // planes 0-2: row g, planes 3-5: row g+8
    uint4 sa, sb;    // biased scales of row g / row g+8
    uint32_t dd;     // fp16 d of row g (low half) and row g+8 (high half)
};

__device__ __forceinline__ uint32_t ldg_u16(const uint8_t *p) {
    unsigned short v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ void load_q6_tile(Q6TileRegs &r, const uint8_t *tile, int lane) {
    const int g = lane >> 2;
#pragma unroll
    for (int p = 0; p < 6; ++p) r.c[p] = ldg128(tile + p * 512 + lane * 16);
    r.sa = ldg128(tile + Q6T_SCALES_OFF + 16 * g);
    r.sb = ldg128(tile + Q6T_SCALES_OFF + 16 * (g + 8));
    r.dd = ldg_u16(tile + Q6T_D_OFF + 2 * g) | (ldg_u16(tile + Q6T_D_OFF + 2 * (g + 8)) << 16);
}

__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t c) { return (a & mask) | c; }

__device__ __forceinline__ uint32_t hadd2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("add.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Scale byte b of `word` (stored +128) as an exact float.
__device__ __forceinline__ float biased_byte_to_float(uint32_t word, int b) {
    const uint32_t bits = __byte_perm(word, 0x4b000000u, 0x7650 + b);     // 8388608 + byte
    return __uint_as_float(bits) - 8388736.0f;
}

// One tile: 16 scale groups = 16 mma steps; tot += d * sum_s scale_s * (codes_s . x_s). With NT
// token tiles (8 tokens each, their fragments `tile_stride` entries apart) every decoded A operand
// is multiplied into each of them, so the decode cost is paid once per 8*NT tokens.
template <int NTERMS, int NT>
__device__ __forceinline__ void q6_tile_mma(const Q6TileRegs &r, const uint2 *bfrag, int tile_stride, int nfrag, int sb,
                                            int lane, float (&tot)[NT][4]) {
    const uint32_t magic = 0x64006400u, neg = 0xe420e420u;       // 1024 | code ; -(1024 + 32)
    const uint32_t wa[12] = {r.c[0].x, r.c[0].y, r.c[0].z, r.c[0].w, r.c[1].x, r.c[1].y,
                             r.c[1].z, r.c[1].w, r.c[2].x, r.c[2].y, r.c[2].z, r.c[2].w};
    const uint32_t wb[12] = {r.c[3].x, r.c[3].y, r.c[3].z, r.c[3].w, r.c[4].x, r.c[4].y,
                             r.c[4].z, r.c[4].w, r.c[5].x, r.c[5].y, r.c[5].z, r.c[5].w};
    const uint32_t sa[4] = {r.sa.x, r.sa.y, r.sa.z, r.sa.w}, sb4[4] = {r.sb.x, r.sb.y, r.sb.z, r.sb.w};
    float blk[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) blk[nt][i] = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t a0w = wa[3 * c], a1w = wa[3 * c + 1], a2w = wa[3 * c + 2];
        const uint32_t b0w = wb[3 * c], b1w = wb[3 * c + 1], b2w = wb[3 * c + 2];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t p0a, p1a, p0b, p1b;
            if (j < 3) {
                const uint32_t va = j == 0 ? a0w : (j == 1 ? a1w : a2w);
                const uint32_t vb = j == 0 ? b0w : (j == 1 ? b1w : b2w);
                p0a = and_or(va, 0x003f003fu, magic);
                p1a = and_or(va >> 6, 0x003f003fu, magic);
                p0b = and_or(vb, 0x003f003fu, magic);
                p1b = and_or(vb >> 6, 0x003f003fu, magic);
            } else {
                p0a = and_or(a2w >> 8, 0x00300030u, and_or(a0w >> 12, 0x000f000fu, magic));
                p1a = and_or(a2w >> 10, 0x00300030u, and_or(a1w >> 12, 0x000f000fu, magic));
                p0b = and_or(b2w >> 8, 0x00300030u, and_or(b0w >> 12, 0x000f000fu, magic));
                p1b = and_or(b2w >> 10, 0x00300030u, and_or(b1w >> 12, 0x000f000fu, magic));
            }
            const int s = 8 * (c >> 1) + 2 * j + (c & 1);
            const uint32_t a0 = hadd2_u32(p0a, neg), a1 = hadd2_u32(p0b, neg), a2 = hadd2_u32(p1a, neg),
                           a3 = hadd2_u32(p1b, neg);
            const float fa = biased_byte_to_float(sa[s >> 2], s & 3), fb = biased_byte_to_float(sb4[s >> 2], s & 3);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                const BFrag b = load_bfrag<NTERMS>(bfrag + nt * tile_stride, nfrag, sb * 16 + s, lane);
                mma_terms<NTERMS>(acc, a0, a1, a2, a3, b);
                blk[nt][0] = fmaf(fa, acc[0], blk[nt][0]);
                blk[nt][1] = fmaf(fa, acc[1], blk[nt][1]);
                blk[nt][2] = fmaf(fb, acc[2], blk[nt][2]);
                blk[nt][3] = fmaf(fb, acc[3], blk[nt][3]);
            }
        }
    }
    const float da = half_bits_to_float(r.dd & 0xffffu), db = half_bits_to_float(r.dd >> 16);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        tot[nt][0] = fmaf(da, blk[nt][0], tot[nt][0]);
        tot[nt][1] = fmaf(da, blk[nt][1], tot[nt][1]);
        tot[nt][2] = fmaf(db, blk[nt][2], tot[nt][2]);
        tot[nt][3] = fmaf(db, blk[nt][3], tot[nt][3]);
    }
}

// Tile policies of the kernel below: bytes per 16-row x 256-value tile, the registers of one tile,
// how a lane loads them and how it multiplies them into its four accumulators.
struct Q6Tile {
    static constexpr int BYTES = Q6T_TILE_BYTES;
    using Regs = Q6TileRegs;
    static __device__ __forceinline__ void load(Regs &r, const uint8_t *tile, int lane) { load_q6_tile(r, tile, lane); }
    template <int NTERMS, int NT>
    static __device__ __forceinline__ void mma(const Regs &r, const uint2 *bfrag, int tile_stride, int nfrag, int sb,
                                               int lane, float (&tot)[NT][4]) {
        q6_tile_mma<NTERMS, NT>(r, bfrag, tile_stride, nfrag, sb, lane, tot);
    }
};

// Q8_0 tile (16 rows x 8 blocks of 32 values = 4352 bytes, the size of the 128 native 34-byte blocks):
//   [   0, 4096)  eight planes of 512 bytes, one uint4 per lane: planes 0-3 = the 16 code words of
//                 row g (word s = values 4*tig..4*tig+3 of the 16-value step s), planes 4-7 = row g+8;
//                 codes are stored +128 (unsigned), so a byte permute gives the FP16 pair 1024+code+128
//   [4096, 4352)  16 rows x 8 fp16 block scales
constexpr int Q8T_TILE_BYTES = 4352;
constexpr int Q8T_SCALES_OFF = 4096;
struct Q8TileRegs {
    uint4 c[8];
    uint4 da, db;      // eight fp16 scales of row g / row g+8
};
struct Q8Tile {
    static constexpr int BYTES = Q8T_TILE_BYTES;
    using Regs = Q8TileRegs;
    static __device__ __forceinline__ void load(Regs &r, const uint8_t *tile, int lane) {
        const int g = lane >> 2;
#pragma unroll
        for (int p = 0; p < 8; ++p) r.c[p] = ldg128(tile + p * 512 + lane * 16);
        r.da = ldg128(tile + Q8T_SCALES_OFF + 16 * g);
        r.db = ldg128(tile + Q8T_SCALES_OFF + 16 * (g + 8));
    }
    template <int NTERMS, int NT>
    static __device__ __forceinline__ void mma(const Regs &r, const uint2 *bfrag, int tile_stride, int nfrag, int sb,
                                               int lane, float (&tot)[NT][4]) {
        const uint32_t neg = 0xe480e480u;                       // -(1024 + 128)
        const uint32_t wa[16] = {r.c[0].x, r.c[0].y, r.c[0].z, r.c[0].w, r.c[1].x, r.c[1].y, r.c[1].z, r.c[1].w,
                                 r.c[2].x, r.c[2].y, r.c[2].z, r.c[2].w, r.c[3].x, r.c[3].y, r.c[3].z, r.c[3].w};
        const uint32_t wb[16] = {r.c[4].x, r.c[4].y, r.c[4].z, r.c[4].w, r.c[5].x, r.c[5].y, r.c[5].z, r.c[5].w,
                                 r.c[6].x, r.c[6].y, r.c[6].z, r.c[6].w, r.c[7].x, r.c[7].y, r.c[7].z, r.c[7].w};
        const uint32_t da[4] = {r.da.x, r.da.y, r.da.z, r.da.w}, db[4] = {r.db.x, r.db.y, r.db.z, r.db.w};
#pragma unroll
        for (int blk = 0; blk < 8; ++blk) {
            float acc[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int s = 2 * blk + h;
                const uint32_t va = wa[s], vb = wb[s];
                const uint32_t a0 = hadd2_u32(__byte_perm(va, 0x64646464u, 0x4240), neg),
                               a1 = hadd2_u32(__byte_perm(vb, 0x64646464u, 0x4240), neg),
                               a2 = hadd2_u32(__byte_perm(va, 0x64646464u, 0x4341), neg),
                               a3 = hadd2_u32(__byte_perm(vb, 0x64646464u, 0x4341), neg);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const BFrag b = load_bfrag<NTERMS>(bfrag + nt * tile_stride, nfrag, sb * 16 + s, lane);
                    mma_terms<NTERMS>(acc[nt], a0, a1, a2, a3, b);
                }
            }
            const float fa = half_bits_to_float((da[blk >> 1] >> (16 * (blk & 1))) & 0xffffu);
            const float fb = half_bits_to_float((db[blk >> 1] >> (16 * (blk & 1))) & 0xffffu);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                tot[nt][0] = fmaf(fa, acc[nt][0], tot[nt][0]);
                tot[nt][1] = fmaf(fa, acc[nt][1], tot[nt][1]);
                tot[nt][2] = fmaf(fb, acc[nt][2], tot[nt][2]);
                tot[nt][3] = fmaf(fb, acc[nt][3], tot[nt][3]);
            }
        }
    }
};

// Activation fragments in natural order: fragment f (16 positions 16f..16f+15), lane (g, tig):
// token g, positions 16f + 4tig + {0,2} -> b0, {1,3} -> b1; FP16 high part (+ remainder plane for
// FP32 inputs) after a per-token power-of-two scaling. All Q6T_THREADS threads take part.
template <int NTERMS, int KEEP, typename RowFn>
__device__ __forceinline__ void prepare_fragments(RowFn row_of, int m_tokens, int k, const void *x, int x_dtype,
                                                  uint2 *bfrag, float *tok_scale, int tid) {
    const int lane = tid & 31;
    const int nfrag = k >> 4;
    const size_t esize = x_dtype == B200Q_F32 ? 4 : 2;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(x) % (4 * esize)) == 0;
    unsigned int *amax_bits = reinterpret_cast<unsigned int *>(tok_scale + 16);
    if (tid < 8) amax_bits[tid] = 0u;
    named_barrier_sync(1, Q6T_THREADS);
    // Every thread owns whole chunks of four consecutive activations (= one fragment entry): the first
    // pass loads them and finds the per-token maximum, the second converts from registers (chunks
    // beyond KEEP per thread are loaded again). Entries of tokens >= m_tokens stay as they are: a
    // column of B only feeds the same column of the product, and those columns are never stored.
    const int chunks_per_token = k >> 2;              // a multiple of 64: a warp's 32 chunks share one token
    const int total = m_tokens * chunks_per_token;
    const int first = tid & ~31;
    float kept[KEEP][4];
    auto load_chunk = [&](int c0, float (&v)[4]) {
        const int t = c0 / chunks_per_token;
        load4(x, x_dtype, static_cast<size_t>(row_of(t)) * k + static_cast<size_t>(c0 + lane - t * chunks_per_token) * 4,
              vec_ok, v);
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
        for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (lane == 0) atomicMax(&amax_bits[t], __float_as_uint(amax));
    };
#pragma unroll
    for (int sl = 0; sl < KEEP; ++sl)
        if (first + sl * Q6T_THREADS < total) load_chunk(first + sl * Q6T_THREADS, kept[sl]);
    for (int c0 = first + KEEP * Q6T_THREADS; c0 < total; c0 += Q6T_THREADS) {
        float v[4];
        load_chunk(c0, v);
    }
    named_barrier_sync(1, Q6T_THREADS);
    if (tid < 8) {
        const float amax = __uint_as_float(amax_bits[tid]);
        float s = 1.0f;
        if (amax > 0.f && amax < __int_as_float(0x7f800000)) {
            int e;
            frexpf(amax, &e);
            s = ldexpf(1.0f, min(14 - e, 100));
        }
        tok_scale[tid] = s;
        tok_scale[8 + tid] = 1.0f / s;
    }
    named_barrier_sync(1, Q6T_THREADS);
    auto store_chunk = [&](int c0, const float (&v)[4]) {
        const int t = c0 / chunks_per_token;
        const int p = (c0 + lane - t * chunks_per_token) * 4;      // position of the chunk in the row
        const float s = tok_scale[t];
        unsigned short hi[4], lo[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float sv = v[i] * s;
            const __half h = __float2half_rn(sv);
            hi[i] = __half_as_ushort(h);
            lo[i] = __half_as_ushort(__float2half_rn(sv - __half2float(h)));
        }
        const int f = p >> 4, dst = 4 * t + ((p >> 2) & 3);
        bfrag[f * 32 + dst] = make_uint2(hi[0] | (static_cast<uint32_t>(hi[2]) << 16),
                                         hi[1] | (static_cast<uint32_t>(hi[3]) << 16));
        if (NTERMS == 2)
            bfrag[(nfrag + f) * 32 + dst] = make_uint2(lo[0] | (static_cast<uint32_t>(lo[2]) << 16),
                                                       lo[1] | (static_cast<uint32_t>(lo[3]) << 16));
    };
#pragma unroll
    for (int sl = 0; sl < KEEP; ++sl)
        if (first + sl * Q6T_THREADS < total) store_chunk(first + sl * Q6T_THREADS, kept[sl]);
    for (int c0 = first + KEEP * Q6T_THREADS; c0 < total; c0 += Q6T_THREADS) {
        const int t = c0 / chunks_per_token;
        float v[4];
        load4(x, x_dtype, static_cast<size_t>(row_of(t)) * k + static_cast<size_t>(c0 + lane - t * chunks_per_token) * 4,
              vec_ok, v);
        store_chunk(c0, v);
    }
    named_barrier_sync(1, Q6T_THREADS);
}

// MODE 0: y[m, n] = x W^T.  MODE 3: grouped down projection over the plan's segments, rows scaled
// by the route weight. Warp (rgi, kpi) owns row group rgi of the CTA's row block and the
// super-blocks kpi, kpi+kp, ...; the next tile is requested before the current one is computed.
// NT (mode 0 only) is the number of 8-token tiles served by one pass over the weights: tile nt
// holds tokens 8nt..8nt+7, with its own scales (Q6T_TOK_STRIDE floats further on) and fragments.
constexpr int Q6T_TOK_STRIDE = 128;     // floats between the token tiles' scale blocks (inside the control bytes)
// tiled_body is the work of CTA `block` of `nblocks` (Q6T_THREADS threads, all of them call; `smem` 128-byte
// aligned): the kernel runs it for its own index in the grid, a persistent multi-stage kernel likewise.
template <typename TILE, int MODE, int NTERMS, int NT>
__device__ __forceinline__ void tiled_body(const Q6TiledArgs &a, const StagePointers &gp, uint8_t *smem, const int block,
                                           const int nblocks) {
    constexpr bool GROUPED = (MODE == 3);
    static_assert(NT == 1 || MODE == 0, "several token tiles only in the linear mode");
    float *tok_scale = reinterpret_cast<float *>(smem);           // per token tile: [8] scale, [8] inverse, [8] amax bits
    float *route_w = reinterpret_cast<float *>(smem + 128);       // [8]
    int *seg_tokens = reinterpret_cast<int *>(smem + 192);        // [8]
    float **out_ptr = reinterpret_cast<float **>(smem + 256);     // [8]
    float *partial = reinterpret_cast<float *>(smem + Q6T_CTRL_BYTES);
    uint2 *bfrag = reinterpret_cast<uint2 *>(smem + a.off_bfrag);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tig = lane & 3;
    const int rgi = warp / a.kp, kpi = warp - rgi * a.kp;
    const int nsb = a.k >> 8;
    const int nfrag = a.k >> 4;
    const int tile_stride = NTERMS * nfrag * 32;           // fragment entries of one token tile
    const int groups_total = a.n >> 4;                     // n is a multiple of 16

    const int blocks_per_unit = (groups_total + a.rg - 1) / a.rg;
    long long units = 1;
    if (GROUPED) {
        int nseg = *gp.num_segments;
        if (nseg > a.max_segments) nseg = a.max_segments;
        units = nseg;
    }
    const long long total_blocks = units * blocks_per_unit;
    const long long blk_begin = total_blocks * block / nblocks;
    const long long blk_end = total_blocks * (block + 1) / nblocks;
    if (!GROUPED) {
        // the CTA's row blocks are one contiguous run of tiles
        if (blk_begin < blk_end) {
            const size_t first = static_cast<size_t>(blk_begin) * a.rg * nsb * TILE::BYTES;
            const size_t last = static_cast<size_t>(min(static_cast<long long>(groups_total), blk_end * a.rg)) * nsb * TILE::BYTES;
            prefetch_l2_range(a.w + first, last - first, CHAIN_PREFETCH_BYTES, tid, Q6T_THREADS);
        }
        chain_wait();     // activations come from the preceding kernel
    }
    if (blk_begin >= blk_end) return;

    const int items_per_block = kpi < nsb ? (nsb - kpi + a.kp - 1) / a.kp : 0;
    auto block_base = [&](int unit, int bi) -> const uint8_t * {
        const int expert = GROUPED ? gp.seg_expert[unit] : 0;
        const int group = min(bi * a.rg + rgi, groups_total - 1);      // clamped groups are loaded, never stored
        return expert_matrix(a.w, a.stride, gp.table_a, expert) +
               (static_cast<size_t>(group) * nsb + kpi) * TILE::BYTES;
    };
    const size_t item_step = static_cast<size_t>(a.kp) * TILE::BYTES;

    int unit_i = static_cast<int>(blk_begin / blocks_per_unit);
    int bi = static_cast<int>(blk_begin - static_cast<long long>(unit_i) * blocks_per_unit);
    const uint8_t *cur_p = block_base(unit_i, bi), *nxt_p = cur_p;
    typename TILE::Regs cur, nxt;
    if (items_per_block > 0) TILE::load(nxt, cur_p, lane);

    int m_tokens = a.m;
    int seg_begin = 0, cur_unit = -1;
    if (!GROUPED) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            prepare_fragments<NTERMS, (NT == 1 ? 4 : 2)>([nt](int t) { return 8 * nt + t; }, max(min(a.m - 8 * nt, 8), 0),
                                                         a.k, gp.x, a.x_dtype, bfrag + nt * tile_stride,
                                                         tok_scale + nt * Q6T_TOK_STRIDE, tid);
    }

    int pbuf = 0;
    for (long long blk = blk_begin; blk < blk_end; ++blk) {
        const int unit = unit_i;
        const int group0 = bi * a.rg;
        if (++bi == blocks_per_unit) { bi = 0; ++unit_i; }
        const bool has_next = blk + 1 < blk_end;
        if (has_next) nxt_p = block_base(unit_i, bi);
        if (GROUPED && unit != cur_unit) {
            cur_unit = unit;
            seg_begin = gp.seg_begin[unit];
            m_tokens = min(gp.seg_count[unit], 8);
            named_barrier_sync(1, Q6T_THREADS);
            if (tid < m_tokens) {
                const int flat = gp.order[seg_begin + tid];
                seg_tokens[tid] = seg_begin + tid;
                route_w[tid] = gp.route[flat];
                out_ptr[tid] = term_row_pointer(static_cast<float *>(gp.y), a.y_table, a.rows_per_rank, a.n,
                                                a.flat_rows ? flat : seg_begin + tid);
            }
            named_barrier_sync(1, Q6T_THREADS);
            prepare_fragments<NTERMS, 2>([&](int t) { return seg_tokens[t]; }, m_tokens, a.k, gp.x, a.x_dtype, bfrag,
                                      tok_scale, tid);
        }

        float tot[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) tot[nt][i] = 0.f;
        for (int item = 0; item < items_per_block; ++item) {
            cur = nxt;
            if (item + 1 < items_per_block) TILE::load(nxt, cur_p + (item + 1) * item_step, lane);
            else if (has_next) TILE::load(nxt, nxt_p, lane);
            TILE::template mma<NTERMS, NT>(cur, bfrag, tile_stride, nfrag, kpi + item * a.kp, lane, tot);
        }

        const int group = group0 + rgi;
        if (a.kp == 1) {
            // the warp owns its rows' whole K range: store straight from the accumulators
            if (group < groups_total) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int orow = group * 16 + g + 8 * (i >> 1), tl = 2 * tig + (i & 1), t = 8 * nt + tl;
                        if (t < m_tokens) {
                            const float v = tot[nt][i] * tok_scale[nt * Q6T_TOK_STRIDE + 8 + tl];
                            if (MODE == 0) store_from_float(gp.y, a.y_dtype, static_cast<size_t>(t) * a.n + orow, v);
                            else out_ptr[t][orow] = v * route_w[t];
                        }
                    }
            }
        } else {
            // partial sums [warp][token tile][16 rows][8 tokens], combined over the kp warps in fixed order
            float *pb = partial + pbuf * (NT * Q6T_PART_FLOATS) + warp * (NT * 128);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                pb[nt * 128 + g * 8 + 2 * tig] = tot[nt][0];
                pb[nt * 128 + g * 8 + 2 * tig + 1] = tot[nt][1];
                pb[nt * 128 + (g + 8) * 8 + 2 * tig] = tot[nt][2];
                pb[nt * 128 + (g + 8) * 8 + 2 * tig + 1] = tot[nt][3];
            }
            const int group_threads = a.kp * 32;
            named_barrier_sync(2 + rgi, group_threads);            // kp >= 2: at most 8 row groups, ids 2..9
            for (int o = kpi * 32 + lane; o < NT * 128; o += group_threads) {
                const int nt = o >> 7, r = (o >> 3) & 15, tl = o & 7, t = 8 * nt + tl;
                if (group >= groups_total || t >= m_tokens) continue;
                const float *src = partial + pbuf * (NT * Q6T_PART_FLOATS) + (rgi * a.kp) * (NT * 128) + o;
                float v = 0.f;
                for (int kq = 0; kq < a.kp; ++kq) v += src[kq * (NT * 128)];
                v *= tok_scale[nt * Q6T_TOK_STRIDE + 8 + tl];
                const int orow = group * 16 + r;
                if (MODE == 0) store_from_float(gp.y, a.y_dtype, static_cast<size_t>(t) * a.n + orow, v);
                else out_ptr[t][orow] = v * route_w[t];
            }
            pbuf ^= 1;
        }
        cur_p = nxt_p;
    }
}

template <typename TILE, int MODE, int NTERMS, int NT>
__global__ void __launch_bounds__(Q6T_THREADS, 1) tiled_kernel(const Q6TiledArgs a) {
    chain_trigger();      // the next kernel of the stream may be scheduled; it waits for this grid itself
    if (MODE == 3) chain_wait();      // the segment list comes from the plan kernel
    extern __shared__ __align__(128) uint8_t smem[];
    const StagePointers gp{a.x, a.y, a.table, nullptr, a.order, a.seg_expert, a.seg_begin, a.seg_count, a.num_segments, a.route, -1};
    tiled_body<TILE, MODE, NTERMS, NT>(a, gp, smem, blockIdx.x, gridDim.x);
}

// Residual add + RMSNorm fused into the GEMV that consumes it (one-token decoder steps: the norm is a 4-5 us launch
// of its own for a row of a few KB). Every CTA normalises the rows itself - the arithmetic of rmsnorm_kernel<true>,
// run by its first 256 threads, the normalised row kept in shared memory behind the GEMV's buffers in the
// activation type - and then runs the GEMV body on it; CTA 0 also stores the new residual stream. Same bits as
// the two launches.
struct NormPrologue {
    const float *residual;     // [m, k] FP32
    const void *branch;        // [m, k], added to the residual (alpha * branch)
    int branch_dtype;
    float alpha;
    const void *gamma;         // [k]; its type is the type of the normalised activations
    int gamma_dtype;
    float eps;
    float *res_out;            // [m, k] FP32: residual + alpha * branch
    int x_off;                 // byte offset of the normalised rows in dynamic shared memory
};

}  // namespace b200q

#include "norm_device.cuh"

namespace b200q {

// One row of residual add + RMSNorm by the whole CTA with the arithmetic of rmsnorm_row<true>: thread t < 256 owns
// columns t, t + 256, ... (sum of squares in ascending order, the same reduction tree, the same roundings). The
// inputs are first copied to shared memory with one vector load per thread - inside this large kernel the compiler
// issued rmsnorm_row's 24 loads per thread one by one, 6 us per launch.
__device__ __forceinline__ void norm_row_staged(int row, int tid, const NormPrologue &n, int k, float *res_s,
                                                uint8_t *br_s, uint8_t *gam_s, uint8_t *x_row, bool store_residual) {
    __shared__ float warp_sums[8];
    __shared__ float inv_shared;
    const int lane = tid & 31, warp = tid >> 5;
    const size_t base = static_cast<size_t>(row) * k;
    const int bsize = n.branch_dtype == B200Q_F32 ? 4 : 2;
    for (int i = tid; i < k / 4; i += Q6T_THREADS)
        reinterpret_cast<float4 *>(res_s)[i] = reinterpret_cast<const float4 *>(n.residual + base)[i];
    for (int i = tid; i < k * bsize / 16; i += Q6T_THREADS)
        reinterpret_cast<uint4 *>(br_s)[i] = reinterpret_cast<const uint4 *>(static_cast<const uint8_t *>(n.branch) + base * bsize)[i];
    for (int i = tid; i < k * 2 / 16; i += Q6T_THREADS)
        reinterpret_cast<uint4 *>(gam_s)[i] = reinterpret_cast<const uint4 *>(n.gamma)[i];
    __syncthreads();
    if (tid < ROW_THREADS) {
        float ss = 0.f;
        for (int c = tid; c < k; c += ROW_THREADS) {
            float v = load_as_float(br_s, n.branch_dtype, c);
            v = res_s[c] + n.alpha * v;
            res_s[c] = v;
            ss += v * v;
        }
        ss = warp_sum(ss);
        if (lane == 0) warp_sums[warp] = ss;
    }
    __syncthreads();
    if (warp == 0) {
        float t = lane < 8 ? warp_sums[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) inv_shared = __fdiv_rn(1.0f, __fsqrt_rn(__fdiv_rn(t, static_cast<float>(k)) + n.eps));
    }
    __syncthreads();
    const float inv = inv_shared;
    for (int c = tid; c < k; c += Q6T_THREADS)
        store_from_float(x_row, n.gamma_dtype, c, (res_s[c] * inv) * load_as_float(gam_s, n.gamma_dtype, c));
    if (store_residual)
        for (int i = tid; i < k / 4; i += Q6T_THREADS)
            reinterpret_cast<float4 *>(n.res_out + base)[i] = reinterpret_cast<const float4 *>(res_s)[i];
    __syncthreads();
}

template <typename TILE, int NTERMS>
__global__ void __launch_bounds__(Q6T_THREADS, 1) tiled_norm_kernel(const Q6TiledArgs a, const NormPrologue n) {
    chain_trigger();
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x;
    {
        // the CTA's slice of the weights is asked into L2 before the wait (as the GEMV body does): the norm
        // below then runs while the bytes arrive
        const int groups_total = a.n >> 4, nsb = a.k >> 8;
        const long long total_blocks = (groups_total + a.rg - 1) / a.rg;
        const long long blk_begin = total_blocks * blockIdx.x / gridDim.x, blk_end = total_blocks * (blockIdx.x + 1) / gridDim.x;
        if (blk_begin < blk_end) {
            const size_t first = static_cast<size_t>(blk_begin) * a.rg * nsb * TILE::BYTES;
            const size_t last = static_cast<size_t>(min(static_cast<long long>(groups_total), blk_end * a.rg)) * nsb * TILE::BYTES;
            prefetch_l2_range(a.w + first, last - first, CHAIN_PREFETCH_BYTES, tid, Q6T_THREADS);
        }
    }
    chain_wait();              // residual and branch come from preceding kernels
    uint8_t *x_rows = smem + n.x_off;                          // [m][k] activations, then the staging of one row
    uint8_t *stage = x_rows + static_cast<size_t>(a.m) * a.k * 2;
    float *res_s = reinterpret_cast<float *>(stage);
    uint8_t *br_s = stage + static_cast<size_t>(a.k) * 4;
    uint8_t *gam_s = br_s + static_cast<size_t>(a.k) * 4;
    for (int row = 0; row < a.m; ++row)
        norm_row_staged(row, tid, n, a.k, res_s, br_s, gam_s, x_rows + static_cast<size_t>(row) * a.k * 2, blockIdx.x == 0);
    const StagePointers gp{x_rows, a.y, a.table, nullptr, a.order, a.seg_expert, a.seg_begin, a.seg_count, a.num_segments, a.route, -1};
    tiled_body<TILE, 0, NTERMS, 1>(a, gp, smem, blockIdx.x, gridDim.x);
}

// SiLU(gate) * up fused into the GEMV that consumes it (the down projection of a one-token decoder step): every CTA
// computes the activation rows itself from the stacked FP32 gate|up projection output [m, 2k] - the arithmetic and
// the rounding to the activation type of the stand-alone element-wise kernel - keeps them in shared memory behind
// the GEMV's buffers and runs the GEMV body on them. Same bits as the two launches.
template <typename TILE, int NTERMS>
__global__ void __launch_bounds__(Q6T_THREADS, 1) tiled_silu_kernel(const Q6TiledArgs a, const float *gate_up, int x_off) {
    chain_trigger();
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x;
    {
        const int groups_total = a.n >> 4, nsb = a.k >> 8;
        const long long total_blocks = (groups_total + a.rg - 1) / a.rg;
        const long long blk_begin = total_blocks * blockIdx.x / gridDim.x, blk_end = total_blocks * (blockIdx.x + 1) / gridDim.x;
        if (blk_begin < blk_end) {
            const size_t first = static_cast<size_t>(blk_begin) * a.rg * nsb * TILE::BYTES;
            const size_t last = static_cast<size_t>(min(static_cast<long long>(groups_total), blk_end * a.rg)) * nsb * TILE::BYTES;
            prefetch_l2_range(a.w + first, last - first, CHAIN_PREFETCH_BYTES, tid, Q6T_THREADS);
        }
    }
    chain_wait();              // the gate|up projection comes from the preceding kernel
    uint8_t *x_rows = smem + x_off;                            // [m][k] activations (16-bit)
    const int quads = a.k >> 2;
    for (int i = tid; i < a.m * quads; i += Q6T_THREADS) {
        const int row = i / quads, c4 = i - row * quads;
        const float4 g = reinterpret_cast<const float4 *>(gate_up + static_cast<size_t>(row) * 2 * a.k)[c4];
        const float4 u = reinterpret_cast<const float4 *>(gate_up + static_cast<size_t>(row) * 2 * a.k + a.k)[c4];
        const size_t o = static_cast<size_t>(row) * a.k + 4 * c4;
        store_from_float(x_rows, a.x_dtype, o, swiglu_f32(g.x, u.x));
        store_from_float(x_rows, a.x_dtype, o + 1, swiglu_f32(g.y, u.y));
        store_from_float(x_rows, a.x_dtype, o + 2, swiglu_f32(g.z, u.z));
        store_from_float(x_rows, a.x_dtype, o + 3, swiglu_f32(g.w, u.w));
    }
    __syncthreads();
    const StagePointers gp{x_rows, a.y, a.table, nullptr, a.order, a.seg_expert, a.seg_begin, a.seg_count, a.num_segments, a.route, -1};
    tiled_body<TILE, 0, NTERMS, 1>(a, gp, smem, blockIdx.x, gridDim.x);
}

}  // namespace b200q
