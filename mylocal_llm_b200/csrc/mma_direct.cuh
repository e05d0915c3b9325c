// Direct-load tensor-core GEMV for Q4_K / Q5_K (sm_100a), 8 tokens per token tile, one or two
// token tiles per pass over the weights.
//
// Q4_K / Q5_K super-blocks are 16-byte multiples, so every lane can fetch exactly the packed
// bytes it needs with 128-bit global loads (four lanes cover 64 contiguous bytes of a row, eight
// rows per instruction) - no shared-memory staging of weights, no producer warp, no barrier on
// the weight path. 16 warps per SM, each with the next super-block already in flight, keep about
// 48 KB of loads outstanding per SM.
//
// Arithmetic per super-block (256 weights of one row):
//   * 4- or 5-bit codes -> FP16 pairs by byte permute; one packed FMA turns (1024+q) into sc*q
//     exactly (sc*q <= 63*31 < 2048 is an integer FP16 holds exactly), so the 6-bit sub-block
//     scales ride inside the A fragments and one accumulator serves the whole super-block;
//   * 16 mma.m16n8k16 steps accumulate sum(sc*q*x) in FP32 for 16 rows x 8 tokens;
//   * the minima go through one more mma: A = the eight 6-bit mins, B = per-sub-block activation
//     sums (FP16 high + remainder), giving sum(mn * sum_x);
//   * y += d * acc - dmin * acc_min in FP32.
// Every product is exact; roundings are the FP32 accumulations, as in the FP32-lane kernels.
//
// Activations are prepared once per CTA (or per expert segment) exactly as in mma_gemv.cuh:
// power-of-two scaling per token, FP16 high (+ remainder for FP32 inputs), stored as B fragments.
#pragma once

#include "mma_gemv.cuh"

namespace b200q {

constexpr int MD_WARPS = 16;
constexpr int MD_THREADS = MD_WARPS * 32;
constexpr int MD_CTRL_BYTES = 1024;
constexpr int MD_PART_FLOATS = MD_WARPS * 256;          // [warp][16 rows][8 tokens][2 streams]
constexpr int MD_PART_BYTES = 2 * MD_PART_FLOATS * 4;   // double buffered
constexpr float MD_XS_SCALE = 0.015625f;                // activation sums are stored divided by 64

struct DirectArgs {
    const uint8_t *wa;
    const uint8_t *wb;
    long long stride_a, stride_b;
    const unsigned long long *table_a, *table_b;   // optional per-expert pointer tables
    int rb;              // packed bytes per weight row (both streams share the format)
    int tiled;           // weights in the 16-row tile layout of their format (see load_superblock_tiled)
    int n, k, m;
    int kp, rg;          // warps along K and row groups per CTA pass (kp * rg == 16)
    int nterms;
    int off_bfrag, off_xsfrag;
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
    const uint8_t *images;   // mode 2, optional: token images (token_image_kernel), image_stride bytes per row of x
    int image_stride;
};

// The pointers of a launch that a persistent multi-stage kernel changes between calls of a stage body (the
// kernels fill it from their arguments; the shapes and the split of the work stay in the argument block).
struct StagePointers {
    const void *x;
    void *y;
    const unsigned long long *table_a, *table_b;
    const int32_t *order, *seg_expert, *seg_begin, *seg_count, *num_segments;
    const float *route;
    int prepared_row;      // grouped gate/up: the row of x whose fragments the caller has already prepared in the
                           // CTA's buffers (-1: none); a first segment of just that row then needs no preparation
};

__device__ __forceinline__ uint4 ldg128(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Packed bytes of one row's super-block as seen by one lane.
template <bool Q5>
struct SuperBlockRegs {
    uint4 hd;   // d, dmin, 12 scale/min bytes
    uint4 qa;   // quants bytes [16*tig, +16)        -> sub-blocks 2*(tig>>1), +1
    uint4 qb;   // quants bytes [64 + 16*tig, +16)   -> sub-blocks 4 + 2*(tig>>1), +1
    uint4 qh;   // Q5_K: high-bit bytes of elements [16*(tig&1), +16)
};

template <bool Q5>
__device__ __forceinline__ void load_superblock(SuperBlockRegs<Q5> &r, const uint8_t *blk, int tig) {
    r.hd = ldg128(blk);
    if (Q5) {
        r.qh = ldg128(blk + 16 + 16 * (tig & 1));
        r.qa = ldg128(blk + 48 + 16 * tig);
        r.qb = ldg128(blk + 112 + 16 * tig);
    } else {
        r.qh = make_uint4(0u, 0u, 0u, 0u);
        r.qa = ldg128(blk + 16 + 16 * tig);
        r.qb = ldg128(blk + 80 + 16 * tig);
    }
}

// Q4_K tile layout (device-side re-ordering of the GGUF bytes, same size): a tile holds the 16
// super-blocks of 16 consecutive rows at one K position (2304 bytes):
//   [0, 256)     the 16 rows' first 16 bytes (d, dmin, scales/mins), row r at 16*r
//   [256, 2304)  four planes of 512 bytes with one 16-byte piece per lane (lane*16): planes 0/1 =
//                bytes [16+16tig, +16) and [80+16tig, +16) of row g's block, planes 2/3 the same of
//                row g+8 - exactly the pieces load_superblock() fetches, so the arithmetic is shared.
// Tiles are ordered (row group, super-block): a warp instruction reads 512 contiguous bytes.
constexpr int Q4T_TILE_BYTES = 2304;
// Q5_K the same way (2816 bytes, the size of 16 native blocks): the 16 headers, then the rows' 32 bytes of
// fifth bits (row r at 256 + 32 r; a lane reads the half its elements need, lanes tig and tig + 2 the same
// one), then the four quant planes:
//   [0, 256) headers | [256, 768) fifth bits | [768, 2816) planes 0/1 (row g), 2/3 (row g + 8), lane * 16 each
constexpr int Q5T_TILE_BYTES = 2816;
template <bool Q5>
__host__ __device__ constexpr int direct_tile_bytes() { return Q5 ? Q5T_TILE_BYTES : Q4T_TILE_BYTES; }

template <bool Q5>
__device__ __forceinline__ void load_superblock_tiled(SuperBlockRegs<Q5> &ra, SuperBlockRegs<Q5> &rb,
                                                      const uint8_t *tile, int lane) {
    const int g = lane >> 2, tig = lane & 3;
    ra.hd = ldg128(tile + 16 * g);
    rb.hd = ldg128(tile + 16 * (g + 8));
    if (Q5) {
        ra.qh = ldg128(tile + 256 + 32 * g + 16 * (tig & 1));
        rb.qh = ldg128(tile + 256 + 32 * (g + 8) + 16 * (tig & 1));
        ra.qa = ldg128(tile + 768 + lane * 16);
        ra.qb = ldg128(tile + 1280 + lane * 16);
        rb.qa = ldg128(tile + 1792 + lane * 16);
        rb.qb = ldg128(tile + 2304 + lane * 16);
    } else {
        ra.qa = ldg128(tile + 256 + lane * 16);
        ra.qb = ldg128(tile + 768 + lane * 16);
        rb.qa = ldg128(tile + 1280 + lane * 16);
        rb.qb = ldg128(tile + 1792 + lane * 16);
        ra.qh = rb.qh = make_uint4(0u, 0u, 0u, 0u);
    }
}

// Scales of one row for this lane: the four sub-blocks its quant bytes belong to, as FP16 pairs
// (sc, sc) and (-1024*sc, -1024*sc); plus the A operand of the min product and d, dmin.
struct RowScales {
    uint32_t sc[4];     // [span A low, span A high, span B low, span B high]
    uint32_t nsc[4];
    uint32_t mins;      // (mn[2*tig], mn[2*tig+1]) as exact FP16 pair
    float d, dmin;
};

__device__ __forceinline__ RowScales decode_scales(const uint4 &hd, int tig) {
    RowScales s;
    s.d = half_bits_to_float(hd.x & 0xffffu);
    s.dmin = half_bits_to_float(hd.x >> 16);
    const uint32_t sc_lo = hd.y & 0x3f3f3f3fu;                                       // sub-blocks 0..3
    const uint32_t sc_hi = (hd.w & 0x0f0f0f0fu) | ((hd.y >> 2) & 0x30303030u);        // sub-blocks 4..7
    const uint32_t mn_lo = hd.z & 0x3f3f3f3fu;
    const uint32_t mn_hi = ((hd.w >> 4) & 0x0f0f0f0fu) | ((hd.z >> 2) & 0x30303030u);
    const int sh = (tig >> 1) * 16;   // sub-block pair 2*(tig>>1) inside each word
    const uint32_t a2 = sc_lo >> sh, b2 = sc_hi >> sh;   // low two bytes: the lane's two sub-blocks
    const uint32_t bias = 0x64006400u, k1024 = 0xe400e400u;   // 1024, -1024 as FP16 pairs
    s.sc[0] = hsub2_u32(__byte_perm(a2, 0x64646464u, 0x4040), bias);
    s.sc[1] = hsub2_u32(__byte_perm(a2, 0x64646464u, 0x4141), bias);
    s.sc[2] = hsub2_u32(__byte_perm(b2, 0x64646464u, 0x4040), bias);
    s.sc[3] = hsub2_u32(__byte_perm(b2, 0x64646464u, 0x4141), bias);
#pragma unroll
    for (int i = 0; i < 4; ++i) s.nsc[i] = hmul2_u32(s.sc[i], k1024);
    const uint32_t mw = ((tig & 2) ? mn_hi : mn_lo) >> ((tig & 1) * 16);
    s.mins = hsub2_u32(__byte_perm(mw, 0x64646464u, 0x4140), bias);
    return s;
}


// ---------------------------------------------------------------------------------------------
// Activation fragments for the direct kernel. Fragment (sb, fi) with fi = (X*2 + nib)*4 + j holds,
// for lane (g = lane>>2, tig = lane&3), token g at positions
//   256*sb + 32*(4*X + 2*(tig>>1) + nib) + 16*(tig&1) + 4*j + {0,2 -> b0 ; 1,3 -> b1}
// which are exactly the positions of the codes that lane extracts from word j of its quant bytes.
// xsfrag (sb, term) holds (sum_x[sub 2*tig], sum_x[sub 2*tig+1]) / 64 for token g.
// ---------------------------------------------------------------------------------------------
// Four consecutive activations starting at element index e (a multiple of 4) as floats.
// `vec_ok` tells whether the tensor allows aligned vector loads.
__device__ __forceinline__ void load4(const void *x, int x_dtype, size_t e, bool vec_ok, float (&v)[4]) {
    if (x_dtype == B200Q_F32) {
        if (vec_ok) {
            const float4 t = *reinterpret_cast<const float4 *>(static_cast<const float *>(x) + e);
            v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = static_cast<const float *>(x)[e + i];
        }
    } else {
        uint2 raw;
        if (vec_ok) raw = *reinterpret_cast<const uint2 *>(static_cast<const uint16_t *>(x) + e);
        else {
            const uint16_t *p = static_cast<const uint16_t *>(x) + e;
            raw.x = p[0] | (static_cast<uint32_t>(p[1]) << 16);
            raw.y = p[2] | (static_cast<uint32_t>(p[3]) << 16);
        }
        if (x_dtype == B200Q_F16) {
            v[0] = __half2float(__ushort_as_half(static_cast<unsigned short>(raw.x & 0xffffu)));
            v[1] = __half2float(__ushort_as_half(static_cast<unsigned short>(raw.x >> 16)));
            v[2] = __half2float(__ushort_as_half(static_cast<unsigned short>(raw.y & 0xffffu)));
            v[3] = __half2float(__ushort_as_half(static_cast<unsigned short>(raw.y >> 16)));
        } else {  // bf16: the upper 16 bits of an FP32
            v[0] = __uint_as_float(raw.x << 16);
            v[1] = __uint_as_float(raw.x & 0xffff0000u);
            v[2] = __uint_as_float(raw.y << 16);
            v[3] = __uint_as_float(raw.y & 0xffff0000u);
        }
    }
}

// Every thread owns whole chunks of four consecutive activations (chunk c of token t covers
// positions 4c..4c+3, which is exactly one fragment entry): one pass loads them and finds the
// per-token maximum, the second converts from registers (chunks beyond KEEP per thread are
// loaded again). Entries of tokens >= m_tokens are left as they are: a column of B only feeds the
// same column of the product, and those columns are never stored.

// (THREADS consecutive threads tid = 0..THREADS-1 take part and meet at named barrier BARRIER; the result does
// not depend on THREADS, which must be a multiple of 32.)
template <int NTERMS, int KEEP, int THREADS = MD_THREADS, int BARRIER = 1, typename RowFn>
__device__ __forceinline__ void prepare_direct(RowFn row_of, int m_tokens, int k, const void *x, int x_dtype,
                                               uint2 *bfrag, uint32_t *xsfrag, float *tok_scale, int tid) {
    const int lane = tid & 31;
    const int nsb = k >> 8;
    const int nfrag = nsb * 16;
    const size_t esize = x_dtype == B200Q_F32 ? 4 : 2;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(x) % (4 * esize)) == 0;   // rows are multiples of 256 elements
    unsigned int *amax_bits = reinterpret_cast<unsigned int *>(tok_scale + 16);   // [8], non-negative floats as ints
    if (tid < 8) amax_bits[tid] = 0u;
    named_barrier_sync(BARRIER, THREADS);
    const int chunks_per_token = k >> 2;            // a multiple of 64: a warp's 32 chunks share one token
    const int total = m_tokens * chunks_per_token;
    float kept[KEEP][4];
    const int first = tid & ~31;
    // 1. load, per-token maximum magnitude
    auto load_chunk = [&](int c0, float (&v)[4]) {
        const int t = c0 / chunks_per_token;
        load4(x, x_dtype, static_cast<size_t>(row_of(t)) * k + static_cast<size_t>(c0 + lane - t * chunks_per_token) * 4,
              vec_ok, v);
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
        for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        // NaN/Inf inputs: keep the scale at 1 (the bit pattern compares above every finite value)
        if (lane == 0) atomicMax(&amax_bits[t], __float_as_uint(amax));
    };
#pragma unroll
    for (int sl = 0; sl < KEEP; ++sl)
        if (first + sl * THREADS < total) load_chunk(first + sl * THREADS, kept[sl]);
    for (int c0 = first + KEEP * THREADS; c0 < total; c0 += THREADS) {
        float v[4];
        load_chunk(c0, v);
    }
    named_barrier_sync(BARRIER, THREADS);
    if (tid < 8) {
        const float amax = __uint_as_float(amax_bits[tid]);
        float s = 1.0f;
        if (amax > 0.f && amax < __int_as_float(0x7f800000)) {
            int e;
            frexpf(amax, &e);
            s = ldexpf(1.0f, min(14 - e, 100));   // scaled maximum in [2^13, 2^14)
        }
        tok_scale[tid] = s;
        tok_scale[8 + tid] = 1.0f / s;
    }
    named_barrier_sync(BARRIER, THREADS);
    // 2. scale, split, store: the chunk at position p of token t is fragment entry (f, lane 4t+tig) with
    //    sb = p>>8, sub = (p>>5)&7, X = sub>>2, nib = sub&1, tig = 2*((sub>>1)&1) + ((p>>4)&1), j = (p>>2)&3
    auto store_chunk = [&](int c0, const float (&v)[4]) {
        const int t = c0 / chunks_per_token;
        const int p = (c0 + lane - t * chunks_per_token) * 4;
        const float s = tok_scale[t];
        __half hi[4], lo[4];
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float sv = v[i] * s;
            hi[i] = __float2half_rn(sv);
            sum += __half2float(hi[i]);
            if (NTERMS == 2) {
                lo[i] = __float2half_rn(sv - __half2float(hi[i]));
                sum += __half2float(lo[i]);
            }
        }
        const int sb = p >> 8, sub = (p >> 5) & 7;
        const int X = sub >> 2, nib = sub & 1, tig = 2 * ((sub >> 1) & 1) + ((p >> 4) & 1), j = (p >> 2) & 3;
        const int f = sb * 16 + (X * 2 + nib) * 4 + j;
        const int dst = 4 * t + tig;
        uint2 out;
        out.x = static_cast<uint32_t>(__half_as_ushort(hi[0])) | (static_cast<uint32_t>(__half_as_ushort(hi[2])) << 16);
        out.y = static_cast<uint32_t>(__half_as_ushort(hi[1])) | (static_cast<uint32_t>(__half_as_ushort(hi[3])) << 16);
        bfrag[f * 32 + dst] = out;
        if (NTERMS == 2) {
            out.x = static_cast<uint32_t>(__half_as_ushort(lo[0])) | (static_cast<uint32_t>(__half_as_ushort(lo[2])) << 16);
            out.y = static_cast<uint32_t>(__half_as_ushort(lo[1])) | (static_cast<uint32_t>(__half_as_ushort(lo[3])) << 16);
            bfrag[(nfrag + f) * 32 + dst] = out;
        }
        // sub-block sum: its eight chunks sit in eight consecutive lanes
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if ((lane & 7) == 0) {
            const float scaled = sum * MD_XS_SCALE;
            const __half h = __float2half_rn(scaled);
            const __half l = __float2half_rn(scaled - __half2float(h));
            // operand of the min product: lane 4*t + (sub>>1) holds sub-blocks (sub & ~1, sub | 1)
            const int lane_t = 4 * t + (sub >> 1);
            reinterpret_cast<unsigned short *>(xsfrag + (sb * 2 + 0) * 32 + lane_t)[nib] = __half_as_ushort(h);
            reinterpret_cast<unsigned short *>(xsfrag + (sb * 2 + 1) * 32 + lane_t)[nib] = __half_as_ushort(l);
        }
    };
#pragma unroll
    for (int sl = 0; sl < KEEP; ++sl)
        if (first + sl * THREADS < total) store_chunk(first + sl * THREADS, kept[sl]);
    for (int c0 = first + KEEP * THREADS; c0 < total; c0 += THREADS) {
        const int t = c0 / chunks_per_token;
        float v[4];
        load4(x, x_dtype, static_cast<size_t>(row_of(t)) * k + static_cast<size_t>(c0 + lane - t * chunks_per_token) * 4,
              vec_ok, v);
        store_chunk(c0, v);
    }
    named_barrier_sync(BARRIER, THREADS);
}

// ---------------------------------------------------------------------------------------------
// Token images. In the grouped gate/up launch every expert segment needs the fragments of its tokens, and
// a token routed to k experts would be converted k times (at 64 tokens: 704 conversions of 64 distinct
// rows, each a chain of dependent loads, a reduction and three barriers). token_image_kernel runs
// prepare_direct once per token - same code, so the same bits - and stores what it wrote for token slot 0:
//   [NTERMS * nfrag * 32 bytes]  the slot's four fragment lanes (tig 0..3, 8 bytes each) of every fragment
//   [nsb * 2 * 16 bytes]         the slot's four words of every activation-sum row
//   [16 bytes]                   scale, inverse scale
// gather_token_images copies the images of a segment's tokens into the slots of the CTA's buffers with
// independent 16-byte loads.
// ---------------------------------------------------------------------------------------------
__host__ __device__ constexpr int token_image_units(int nterms, int nsb) {      // 16-byte units per token
    return nterms * nsb * 16 * 2 + nsb * 2 + 1;
}

template <int NTERMS>
__global__ void __launch_bounds__(MD_THREADS, 1) token_image_kernel(const void *x, int x_dtype, int k, uint8_t *images) {
    extern __shared__ __align__(128) uint8_t smem[];
    chain_trigger();
    chain_wait();                 // x comes from the preceding kernel
    const int nsb = k >> 8, nfrag = nsb * 16;
    float *tok_scale = reinterpret_cast<float *>(smem);
    uint2 *bfrag = reinterpret_cast<uint2 *>(smem + MD_CTRL_BYTES);
    uint32_t *xsfrag = reinterpret_cast<uint32_t *>(smem + MD_CTRL_BYTES + NTERMS * nfrag * 256);
    const int row = blockIdx.x, tid = threadIdx.x;
    prepare_direct<NTERMS, 4>([row](int) { return row; }, 1, k, x, x_dtype, bfrag, xsfrag, tok_scale, tid);
    const int nb = NTERMS * nfrag * 2, units = token_image_units(NTERMS, nsb);
    uint4 *dst = reinterpret_cast<uint4 *>(images + static_cast<size_t>(row) * units * 16);
    for (int u = tid; u < units; u += MD_THREADS) {
        uint4 v;
        if (u < nb) v = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint8_t *>(bfrag) + (u >> 1) * 256 + (u & 1) * 16);
        else if (u < units - 1) v = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint8_t *>(xsfrag) + (u - nb) * 128);
        else v = make_uint4(__float_as_uint(tok_scale[0]), __float_as_uint(tok_scale[8]), 0u, 0u);
        dst[u] = v;
    }
}

// Slots 0..m_tokens-1 of the CTA's buffers <- the images of rows order[seg_begin + t] / topk. The caller
// brackets the call with CTA barriers.
__device__ __forceinline__ void gather_token_images(const uint8_t *images, int image_stride, const int32_t *order,
                                                    int seg_begin, int topk, int m_tokens, int nterms, int nsb,
                                                    uint2 *bfrag, uint32_t *xsfrag, float *tok_scale, int tid) {
    const int nb = nterms * nsb * 32, units = token_image_units(nterms, nsb);
    const int t = (tid >> 5) & 7;                 // two warps per token slot, all their loads independent
    if (t < m_tokens) {
        const int row = order[seg_begin + t] / topk;
        const uint4 *src = reinterpret_cast<const uint4 *>(images + static_cast<size_t>(row) * image_stride);
#pragma unroll 5
        for (int u = (tid >> 8) * 32 + (tid & 31); u < units; u += 64) {
            const uint4 v = src[u];
            if (u < nb) *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(bfrag) + (u >> 1) * 256 + t * 32 + (u & 1) * 16) = v;
            else if (u < units - 1) *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(xsfrag) + (u - nb) * 128 + t * 16) = v;
            else {
                tok_scale[t] = __uint_as_float(v.x);
                tok_scale[8 + t] = __uint_as_float(v.y);
            }
        }
    }
}

// 16 mma steps of one super-block for rows (g, g+8): acc += sum(sc*q*x); accm += sum(mn * sum_x/64).
// With NT token tiles (8 tokens each; their fragments `btile` / `xtile` entries apart) every decoded
// A operand is multiplied into each tile, so the decode cost is paid once per 8*NT tokens; the
// arithmetic of one token does not depend on NT.
template <bool Q5, int NTERMS, int NT>
__device__ __forceinline__ void superblock_mma(const SuperBlockRegs<Q5> &ra, const SuperBlockRegs<Q5> &rb,
                                               const uint2 *bfrag, int btile, int nfrag, const uint32_t *xsfrag,
                                               int xtile, int sb, int lane, float (&tot)[NT][4]) {
    const int tig = lane & 3;
    const RowScales sa = decode_scales(ra.hd, tig), sbk = decode_scales(rb.hd, tig);
    float acc[NT][4], acc2[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = acc2[nt][i] = 0.f;
    const uint32_t qa_a[4] = {ra.qa.x, ra.qa.y, ra.qa.z, ra.qa.w}, qb_a[4] = {ra.qb.x, ra.qb.y, ra.qb.z, ra.qb.w};
    const uint32_t qa_b[4] = {rb.qa.x, rb.qa.y, rb.qa.z, rb.qa.w}, qb_b[4] = {rb.qb.x, rb.qb.y, rb.qb.z, rb.qb.w};
    const uint32_t qh_a[4] = {ra.qh.x, ra.qh.y, ra.qh.z, ra.qh.w}, qh_b[4] = {rb.qh.x, rb.qh.y, rb.qh.z, rb.qh.w};
    const int pair = tig >> 1;
#pragma unroll
    for (int X = 0; X < 2; ++X) {
#pragma unroll
        for (int nib = 0; nib < 2; ++nib) {
            const int si = X * 2 + nib;
            // Q5_K: bit (sub-block index) of the high-bit byte, moved to bit 4 of the code
            const int sub = 4 * X + 2 * pair + nib;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t wa = X ? qb_a[j] : qa_a[j], wb = X ? qb_b[j] : qa_b[j];
                uint32_t va = nib ? (wa >> 4) & 0x0f0f0f0fu : wa & 0x0f0f0f0fu;
                uint32_t vb = nib ? (wb >> 4) & 0x0f0f0f0fu : wb & 0x0f0f0f0fu;
                if (Q5) {
                    va |= ((qh_a[j] >> sub) << 4) & 0x10101010u;
                    vb |= ((qh_b[j] >> sub) << 4) & 0x10101010u;
                }
                const uint32_t a0 = hfma2_u32(__byte_perm(va, 0x64646464u, 0x4240), sa.sc[si], sa.nsc[si]);
                const uint32_t a2 = hfma2_u32(__byte_perm(va, 0x64646464u, 0x4341), sa.sc[si], sa.nsc[si]);
                const uint32_t a1 = hfma2_u32(__byte_perm(vb, 0x64646464u, 0x4240), sbk.sc[si], sbk.nsc[si]);
                const uint32_t a3 = hfma2_u32(__byte_perm(vb, 0x64646464u, 0x4341), sbk.sc[si], sbk.nsc[si]);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const BFrag b = load_bfrag<NTERMS>(bfrag + nt * btile, nfrag, sb * 16 + si * 4 + j, lane);
                    if (X) mma_terms<NTERMS>(acc2[nt], a0, a1, a2, a3, b);
                    else mma_terms<NTERMS>(acc[nt], a0, a1, a2, a3, b);
                }
            }
        }
    }
    const float ma = sa.dmin * 64.0f, mb = sbk.dmin * 64.0f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] += acc2[nt][i];
        float accm[4] = {0.f, 0.f, 0.f, 0.f};
        mma_f16(accm, sa.mins, sbk.mins, 0u, 0u, xsfrag[nt * xtile + (sb * 2 + 0) * 32 + lane], 0u);
        mma_f16(accm, sa.mins, sbk.mins, 0u, 0u, xsfrag[nt * xtile + (sb * 2 + 1) * 32 + lane], 0u);
        tot[nt][0] = fmaf(sa.d, acc[nt][0], fmaf(-ma, accm[0], tot[nt][0]));
        tot[nt][1] = fmaf(sa.d, acc[nt][1], fmaf(-ma, accm[1], tot[nt][1]));
        tot[nt][2] = fmaf(sbk.d, acc[nt][2], fmaf(-mb, accm[2], tot[nt][2]));
        tot[nt][3] = fmaf(sbk.d, acc[nt][3], fmaf(-mb, accm[3], tot[nt][3]));
    }
}


// ---------------------------------------------------------------------------------------------
// Kernel. MODE as in stream_gemv.cuh: 0 linear, 1 SwiGLU, 2 grouped gate/up, 3 grouped down.
// Work item of a warp = (row block, super-block of its K part, stream); the packed bytes of the
// next item are requested before the current one is computed.
// ---------------------------------------------------------------------------------------------
// NT (modes 0 and 1 only) is the number of 8-token tiles served by one pass over the weights: tile
// nt holds tokens 8nt..8nt+7 with its own scales (MD_TOK_STRIDE floats further on), fragments and
// activation sums.
constexpr int MD_TOK_STRIDE = 128;     // floats between the token tiles' scale blocks (inside the control bytes)
// The work of CTA `block` of `nblocks` (MD_THREADS threads, all of them call): the kernel below is this body
// for (blockIdx.x, gridDim.x); a persistent kernel that walks several stages calls it with its own.
// `smem`: 128-byte aligned, direct-kernel layout (control bytes, partial sums, fragments at a.off_bfrag).
template <bool Q5, int MODE, int NTERMS, int NT = 1>
__device__ __forceinline__ void mma_direct_body(const DirectArgs &a, const StagePointers &gp, uint8_t *smem, const int block,
                                                const int nblocks) {
    constexpr bool DUAL = (MODE == 1 || MODE == 2);
    constexpr bool GROUPED = (MODE >= 2);
    constexpr int QB = Q5 ? 176 : 144;
    static_assert(NT == 1 || !GROUPED, "several token tiles only in the dense modes");
    float *tok_scale = reinterpret_cast<float *>(smem);           // [8] scale, [8] inverse
    float *route_w = reinterpret_cast<float *>(smem + 128);       // [8]
    int *seg_tokens = reinterpret_cast<int *>(smem + 192);        // [8]
    float **out_ptr = reinterpret_cast<float **>(smem + 256);     // [8] mode 3 output row pointers
    float *partial = reinterpret_cast<float *>(smem + MD_CTRL_BYTES);
    uint2 *bfrag = reinterpret_cast<uint2 *>(smem + a.off_bfrag);
    uint32_t *xsfrag = reinterpret_cast<uint32_t *>(smem + a.off_xsfrag);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tig = lane & 3;
    const int rgi = warp / a.kp, kpi = warp - rgi * a.kp;
    const int nsb = a.k >> 8;
    const int nfrag = nsb * 16;
    const int btile = NTERMS * nfrag * 32, xtile = nsb * 64;     // fragment / sum entries of one token tile

    const int rows_per_block = 16 * a.rg;
    const int blocks_per_unit = (a.n + rows_per_block - 1) / rows_per_block;
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
        // the CTA's row blocks are one contiguous byte range of the matrix (rows, or 16-row tiles)
        if (blk_begin < blk_end) {
            size_t first, last;
            if (a.tiled) {
                first = static_cast<size_t>(blk_begin) * a.rg * nsb * direct_tile_bytes<Q5>();
                last = static_cast<size_t>(min(static_cast<long long>(a.n >> 4), blk_end * a.rg)) * nsb * direct_tile_bytes<Q5>();
            } else {
                first = static_cast<size_t>(blk_begin) * rows_per_block * a.rb;
                last = static_cast<size_t>(min(static_cast<long long>(a.n), blk_end * rows_per_block)) * a.rb;
            }
            const size_t cap = DUAL ? CHAIN_PREFETCH_BYTES / 2 : CHAIN_PREFETCH_BYTES;
            prefetch_l2_range(a.wa + first, last - first, cap, tid, MD_THREADS);
            if (DUAL) prefetch_l2_range(a.wb + first, last - first, cap, tid, MD_THREADS);
        }
        chain_wait();     // activations come from the preceding kernel
    }
    if (blk_begin >= blk_end) return;

    // items of this warp inside one row block: its super-blocks x streams
    const int sb_count = kpi < nsb ? (nsb - kpi + a.kp - 1) / a.kp : 0;
    const int items_per_block = sb_count * (DUAL ? 2 : 1);

    // Row pointers of a row block for this lane (rows g and g+8 of its row group, both streams);
    // rows past the end are clamped to the last row (loaded, never stored).
    struct BlockPtrs {
        const uint8_t *a_lo, *a_hi, *b_lo, *b_hi;
    };
    auto block_ptrs = [&](int unit, int row0) {
        BlockPtrs p;
        const int expert = GROUPED ? gp.seg_expert[unit] : 0;
        size_t off_lo, off_hi;
        if (a.tiled) {   // tile of (row group, super-block kpi); n is a multiple of 16 here
            const int group = min((row0 >> 4) + rgi, (a.n >> 4) - 1);
            off_lo = off_hi = (static_cast<size_t>(group) * nsb + kpi) * direct_tile_bytes<Q5>();
        } else {
            off_lo = static_cast<size_t>(min(row0 + 16 * rgi + g, a.n - 1)) * a.rb + static_cast<size_t>(kpi) * QB;
            off_hi = static_cast<size_t>(min(row0 + 16 * rgi + g + 8, a.n - 1)) * a.rb + static_cast<size_t>(kpi) * QB;
        }
        const uint8_t *base_a = expert_matrix(a.wa, a.stride_a, gp.table_a, expert);
        p.a_lo = base_a + off_lo;
        p.a_hi = base_a + off_hi;
        p.b_lo = p.b_hi = nullptr;
        if (DUAL) {
            const uint8_t *base_b = expert_matrix(a.wb, a.stride_b, gp.table_b, expert);
            p.b_lo = base_b + off_lo;
            p.b_hi = base_b + off_hi;
        }
        return p;
    };
    // item -> byte offset from the block pointers, and stream
    const int sb_step_bytes = a.kp * (a.tiled ? direct_tile_bytes<Q5>() : QB);
    auto issue_item = [&](const BlockPtrs &p, int item, SuperBlockRegs<Q5> &ra, SuperBlockRegs<Q5> &rb) {
        const int stream = DUAL ? (item & 1) : 0;
        const size_t off = static_cast<size_t>(DUAL ? (item >> 1) : item) * sb_step_bytes;
        if (a.tiled) {
            load_superblock_tiled<Q5>(ra, rb, (stream ? p.b_lo : p.a_lo) + off, lane);
            return;
        }
        load_superblock<Q5>(ra, (stream ? p.b_lo : p.a_lo) + off, tig);
        load_superblock<Q5>(rb, (stream ? p.b_hi : p.a_hi) + off, tig);
    };

    int unit_i = static_cast<int>(blk_begin / blocks_per_unit);
    int bi = static_cast<int>(blk_begin - static_cast<long long>(unit_i) * blocks_per_unit);
    BlockPtrs cur_p = block_ptrs(unit_i, bi * rows_per_block), nxt_p = cur_p;

    SuperBlockRegs<Q5> cur_a, cur_b, nxt_a, nxt_b;
    if (items_per_block > 0) issue_item(cur_p, 0, nxt_a, nxt_b);

    int m_tokens = a.m;
    int seg_begin = 0, cur_unit = -1, last_single = (MODE == 2) ? gp.prepared_row : -1;
    if (!GROUPED) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            prepare_direct<NTERMS, (NT == 1 ? 4 : 2)>([nt](int t) { return 8 * nt + t; }, max(min(a.m - 8 * nt, 8), 0),
                                                      a.k, gp.x, a.x_dtype, bfrag + nt * btile, xsfrag + nt * xtile,
                                                      tok_scale + nt * MD_TOK_STRIDE, tid);
    }

    int pbuf = 0;
    for (long long blk = blk_begin; blk < blk_end; ++blk) {
        const int unit = unit_i;
        const int row0 = bi * rows_per_block;
        // advance the (unit, block-in-unit) counters and look up the next block's pointers
        if (++bi == blocks_per_unit) { bi = 0; ++unit_i; }
        const bool has_next = blk + 1 < blk_end;
        if (has_next) nxt_p = block_ptrs(unit_i, bi * rows_per_block);
        if (GROUPED && unit != cur_unit) {
            cur_unit = unit;
            seg_begin = gp.seg_begin[unit];
            m_tokens = min(gp.seg_count[unit], 8);
            int single = -1;
            if (MODE == 2 && m_tokens == 1) single = gp.order[seg_begin] / a.topk;
            const bool reuse = (single >= 0 && single == last_single);
            last_single = single;
            if (!reuse && MODE == 2 && a.images) {
                named_barrier_sync(1, MD_THREADS);       // every warp is done with the previous segment's fragments
                gather_token_images(a.images, a.image_stride, gp.order, seg_begin, a.topk, m_tokens, NTERMS, nsb, bfrag,
                                    xsfrag, tok_scale, tid);
                named_barrier_sync(1, MD_THREADS);
            } else if (!reuse) {
                named_barrier_sync(1, MD_THREADS);
                if (tid < m_tokens) {
                    const int flat = gp.order[seg_begin + tid];
                    seg_tokens[tid] = (MODE == 2) ? flat / a.topk : seg_begin + tid;
                    if (MODE == 3) {
                        route_w[tid] = gp.route[flat];
                        out_ptr[tid] = term_row_pointer(static_cast<float *>(gp.y), a.y_table, a.rows_per_rank, a.n, a.flat_rows ? flat : seg_begin + tid);
                    }
                }
                named_barrier_sync(1, MD_THREADS);
                prepare_direct<NTERMS, 2>([&](int t) { return seg_tokens[t]; }, m_tokens, a.k, gp.x, a.x_dtype, bfrag,
                                       xsfrag, tok_scale, tid);
            }
        }

        float tot_a[NT][4], tot_b[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) tot_a[nt][i] = tot_b[nt][i] = 0.f;
        for (int item = 0; item < items_per_block; ++item) {
            // (copying the prefetched registers measured faster than alternating two register sets)
            cur_a = nxt_a;
            cur_b = nxt_b;
            // request the next item (same block, or the first item of the next block)
            if (item + 1 < items_per_block) issue_item(cur_p, item + 1, nxt_a, nxt_b);
            else if (has_next) issue_item(nxt_p, 0, nxt_a, nxt_b);
            const int stream = DUAL ? (item & 1) : 0;
            const int sb = kpi + (DUAL ? (item >> 1) : item) * a.kp;
            if (stream == 0)
                superblock_mma<Q5, NTERMS, NT>(cur_a, cur_b, bfrag, btile, nfrag, xsfrag, xtile, sb, lane, tot_a);
            else
                superblock_mma<Q5, NTERMS, NT>(cur_a, cur_b, bfrag, btile, nfrag, xsfrag, xtile, sb, lane, tot_b);
        }

        // combine the kp partial sums of each row group in fixed order:
        // partial[warp][token tile][16 rows][8 tokens][2 streams]
        float *pb = partial + pbuf * (NT * MD_PART_FLOATS) + warp * (NT * 256);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float *pt = pb + nt * 256;
            pt[(g * 8 + 2 * tig) * 2 + 0] = tot_a[nt][0];
            pt[(g * 8 + 2 * tig + 1) * 2 + 0] = tot_a[nt][1];
            pt[((g + 8) * 8 + 2 * tig) * 2 + 0] = tot_a[nt][2];
            pt[((g + 8) * 8 + 2 * tig + 1) * 2 + 0] = tot_a[nt][3];
            if (DUAL) {
                pt[(g * 8 + 2 * tig) * 2 + 1] = tot_b[nt][0];
                pt[(g * 8 + 2 * tig + 1) * 2 + 1] = tot_b[nt][1];
                pt[((g + 8) * 8 + 2 * tig) * 2 + 1] = tot_b[nt][2];
                pt[((g + 8) * 8 + 2 * tig + 1) * 2 + 1] = tot_b[nt][3];
            }
        }
        const int group_threads = a.kp * 32;
        if (a.kp == 1) __syncwarp();
        else named_barrier_sync(2 + rgi, group_threads);   // rg <= 8 here: barrier ids 2..9
        for (int o = kpi * 32 + lane; o < NT * 128; o += group_threads) {
            const int nt = o >> 7, r = (o >> 3) & 15, tl = o & 7, t = 8 * nt + tl;
            const int orow = row0 + 16 * rgi + r;
            if (orow >= a.n || t >= m_tokens) continue;
            const float *src = partial + pbuf * (NT * MD_PART_FLOATS) + (rgi * a.kp) * (NT * 256) + o * 2;
            float pa = 0.f, pbv = 0.f;
            for (int kq = 0; kq < a.kp; ++kq) {
                pa += src[kq * (NT * 256)];
                if (DUAL) pbv += src[kq * (NT * 256) + 1];
            }
            const float inv = tok_scale[nt * MD_TOK_STRIDE + 8 + tl];
            pa *= inv;
            pbv *= inv;
            if (MODE == 0) store_from_float(gp.y, a.y_dtype, static_cast<size_t>(t) * a.n + orow, pa);
            else if (MODE == 1)
                store_from_float(gp.y, a.y_dtype, static_cast<size_t>(t) * a.n + orow, swiglu_f32(pa, pbv));
            else if (MODE == 2)
                static_cast<float *>(gp.y)[static_cast<size_t>(seg_begin + t) * a.n + orow] = swiglu_f32(pa, pbv);
            else
                out_ptr[t][orow] = pa * route_w[t];
        }
        pbuf ^= 1;
        cur_p = nxt_p;
    }
}

template <bool Q5, int MODE, int NTERMS, int NT = 1>
__global__ void __launch_bounds__(MD_THREADS, 1) mma_direct_kernel(const DirectArgs a) {
    chain_trigger();      // the next kernel of the stream may be scheduled; it waits for this grid itself
    if (MODE >= 2) chain_wait();      // the segment list comes from the plan kernel
    extern __shared__ __align__(128) uint8_t smem[];
    const StagePointers gp{a.x, a.y, a.table_a, a.table_b, a.order, a.seg_expert, a.seg_begin, a.seg_count, a.num_segments, a.route, -1};
    mma_direct_body<Q5, MODE, NTERMS, NT>(a, gp, smem, blockIdx.x, gridDim.x);
}

}  // namespace b200q
