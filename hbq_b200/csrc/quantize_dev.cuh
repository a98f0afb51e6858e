// Device helpers shared by the quantize kernels: the packed E2Mx element quantizer, kernel
// arguments, chunk load / store and warp-group reductions.
#pragma once
#include "common.cuh"

namespace hbq {

// ------------------------------------------------------------------------------------------
// Packed element quantizer for E2Mx (x = MB mantissa bits), two values per call.
//
// For |b| >= 1 the reference's mantissa rounding floor(fp16(m + 0.50048828125)) is exactly
// round-half-up to MB mantissa bits with carry into the exponent, saturating at the format
// maximum: an integer add + mask on the fp16 bit pattern.  Below 1 the reference computes
// k = floor(fp16(|b| * 2^MB + 0.50048828125)) and returns k / 2^MB; one HFMA2 reproduces that
// rounding literally (the product is exact), including the thresholds that sit 3 and 1 ulp
// below the midpoints and the value 1.0 for [1 - 2^-(MB+1), 1).  E2M1 only: |b| = 0x39FF
// gives k = 2 in the subnormal branch, which the reference turns into 0.
// ZERO_SIGN: give b = -0 the reference's +0 result (the other callers only square it).
// ------------------------------------------------------------------------------------------
// floor of two fp16 values in [0, 1024) without a conversion instruction: adding 1024 rounds to the
// nearest integer (ties to even) in the fp16 adder; subtract one where that rounded up.
__device__ __forceinline__ __half2 floor_small_h2(__half2 v)
{
    const __half2 k1024 = bits_h2(0x64006400u);
    const __half2 n = __hsub2(__hadd2(v, k1024), k1024);
    return __hsub2(n, __hgt2(n, v));
}

template <int MB, bool ZERO_SIGN>
__device__ __forceinline__ __half2 q2_e2(__half2 b)
{
    constexpr uint32_t kHalf = (0x0200u >> MB) * 0x00010001u;
    constexpr uint32_t kMask = ~(((0x0400u >> MB) - 1u) * 0x00010001u);
    constexpr uint32_t kMax = (0x4400u | (((1u << MB) - 1u) << (10 - MB))) * 0x00010001u;
    const uint32_t u = h2_bits(b);
    const uint32_t a = u & 0x7FFF7FFFu;
    uint32_t sgn = u & 0x80008000u;
    const __half2 ab = bits_h2(a);
    // normal range
    const __half2 n = __hmin2(bits_h2((a + kHalf) & kMask), bits_h2(kMax));
    // below 1
    const __half2 v = __hfma2(ab, bits_h2(((uint32_t)(0x3C00u + (MB << 10))) * 0x00010001u),
                              bits_h2(0x38013801u));
    __half2 s = __hmul2(floor_small_h2(v), bits_h2(((uint32_t)(0x3C00u - (MB << 10))) * 0x00010001u));
    uint32_t sb = h2_bits(s);
    if (MB == 1) sb &= ~__heq2_mask(ab, bits_h2(0x39FF39FFu));
    const uint32_t m = __hge2_mask(ab, bits_h2(0x3C003C00u));
    uint32_t r = (h2_bits(n) & m) | (sb & ~m);
    if (ZERO_SIGN) sgn &= __hne2_mask(ab, bits_h2(0u));
    return bits_h2(r | sgn);
}

// Code magnitudes {exp field, mantissa} of two quantised E2Mx values, one per 16-bit half.
template <int MB>
__device__ __forceinline__ uint32_t code2_e2(__half2 c)
{
    const uint32_t a = h2_bits(c) & 0x7FFF7FFFu;
    // clamp below at 0.5 (0x3800) first so the packed subtraction cannot borrow across halves
    const uint32_t an = h2_bits(__hmax2(bits_h2(a), bits_h2(0x38003800u)));
    const uint32_t nrm = ((an - 0x38003800u) >> (10 - MB)) & (((1u << (MB + 2)) - 1u) * 0x00010001u);
    // below 1: k = c * 2^MB, read from the low mantissa bits of k + 1024
    const __half2 k = __hfma2(bits_h2(a), bits_h2(((uint32_t)(0x3C00u + (MB << 10))) * 0x00010001u),
                              bits_h2(0x64006400u));
    const uint32_t sub = h2_bits(k) & 0x00FF00FFu;
    const uint32_t m = __hge2_mask(bits_h2(a), bits_h2(0x3C003C00u));
    return (nrm & m) | (sub & ~m);
}

// ------------------------------------------------------------------------------------------
// Kernel arguments
// ------------------------------------------------------------------------------------------
struct QArgs {
    const void* x;
    void* deq;
    hbq_packed_out out;
    const float* tensor_amax;
    int64_t rows, K, Kp;
    int64_t cpr;            // 8-element chunks per (padded) row
    int64_t total_chunks;
    int64_t step_rows, step_chunks;   // one grid stride of chunks = step_rows rows + step_chunks chunks
    int in_bf16, out_bf16;
    int aligned;            // 128-bit loads/stores are legal
    int G;                  // lanes per block = block_size / 8
    int log2G;              // block index of a chunk = chunk-in-row >> log2G
    int nblk;
    hbq_format f;
    // HBQ
    int nscheme, nc;
    float tab[2][16];
    float inv_tab[2][16];
    float ele_max[2];
    // scale
    int scale_fast_e5m3;    // closed-form E5M3 round-half-up
    int exact_div;          // use IEEE division for x / scale (scale mantissa wider than 4 bits)
    float sc_lo, sc_hi;     // clip range of the FP scale
    float elem_max;         // MXFP FP-scale divisor / MXINT FP-scale divisor
    double pts_den;         // per-tensor scale: element max * scale max (src/quantizer.py:517-523)
    int pot_emin, pot_emax, pot_sub;
    uint16_t pot_thr[32];   // per fp16 exponent field of absmax: smallest mantissa whose floor|round(log2) is one higher
    uint16_t rm[8];         // fp16(1 / m) for the E5M3 mantissas m = 1 + i/8
    float inv_elem_max;     // 1 / elem_max (fp32), for the E5M3 scale
    uint32_t int_lim_pos, int_lim_neg;   // MXINT clip limits 2^(n-1)-1 and 2^(n-1) as packed fp16 pairs
    // fused K/Q-cache write: rows are (b, t, h) of a projection output, RoPE is applied on load and
    // the fake-quantised row is stored at (b, h, t)
    const uint16_t* rope_cos;   // fp16 [rope_rows, K] or NULL (no RoPE)
    const uint16_t* rope_sin;
    int64_t rope_rows;          // B*T (per-batch tables) or T (one table for every batch)
    int64_t perm_T, perm_H;     // > 0: permute output rows (b,t,h) -> (b,h,t)
    const uint16_t* k_center;   // fp16 [B, H, K] or NULL: subtracted after RoPE (K-cache centring, src/module.py:221-244)
    const void* glu_gate;   // fp16, same shape as x, or NULL: the quantised tensor is silu(glu_gate) * x
    int code_bits;          // bits per stored element code (4, 5 or 8)
    int sign_bit;           // position of the sign in a byte code: ebit + mbit
};

struct Chunk {
    __half2 h[4];
};

__device__ __forceinline__ Chunk load_chunk(const QArgs& a, int64_t row, int64_t k0)
{
    Chunk c;
    if (k0 >= a.K) {
        #pragma unroll
        for (int p = 0; p < 4; ++p) c.h[p] = bits_h2(0u);
        return c;
    }
    const int64_t off = row * a.K + k0;
    if (a.aligned && k0 + 8 <= a.K) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(
            reinterpret_cast<const uint16_t*>(a.x) + off));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        if (!a.in_bf16) {
            #pragma unroll
            for (int p = 0; p < 4; ++p) c.h[p] = bits_h2(w[p]);
        } else {
            #pragma unroll
            for (int p = 0; p < 4; ++p)
                c.h[p] = __floats2half2_rn(__uint_as_float(w[p] << 16),
                                           __uint_as_float(w[p] & 0xFFFF0000u));
        }
        return c;
    }
    const uint16_t* xp = reinterpret_cast<const uint16_t*>(a.x) + off;
    float v[8];
    #pragma unroll
    for (int j = 0; j < 8; ++j) {
        uint16_t b = (k0 + j < a.K) ? xp[j] : (uint16_t)0;
        v[j] = a.in_bf16 ? __uint_as_float((uint32_t)b << 16) : __half2float(bits_h(b));
    }
    #pragma unroll
    for (int p = 0; p < 4; ++p) c.h[p] = __floats2half2_rn(v[2 * p], v[2 * p + 1]);
    return c;
}

__device__ __forceinline__ void store_deq(const QArgs& a, int64_t row, int64_t k0, const __half2* d)
{
    if (!a.deq || k0 >= a.K) return;
    uint32_t w[4];
    if (!a.out_bf16) {
        #pragma unroll
        for (int p = 0; p < 4; ++p) w[p] = h2_bits(d[p]);
    } else {
        #pragma unroll
        for (int p = 0; p < 4; ++p) {
            const float2 f = __half22float2(d[p]);
            __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
            w[p] = *reinterpret_cast<uint32_t*>(&b);
        }
    }
    uint16_t* dp = reinterpret_cast<uint16_t*>(a.deq) + row * a.K + k0;
    if (a.aligned && k0 + 8 <= a.K) {
        *reinterpret_cast<uint4*>(dp) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
        #pragma unroll
        for (int j = 0; j < 8; ++j)
            if (k0 + j < a.K) dp[j] = (uint16_t)(w[j >> 1] >> ((j & 1) * 16));
    }
}

// codes: mag[p] holds two code magnitudes (one per 16-bit half), sgn[p] the fp16 sign bits.
// TWOS: integer elements, stored as two's complement of (sign, magnitude).
template <bool TWOS>
__device__ __forceinline__ void store_codes(const QArgs& a, int64_t row, int64_t k0,
                                            const uint32_t* mag_in, const uint32_t* sgn)
{
    if (!a.out.codes) return;
    uint32_t mag[4];
    #pragma unroll
    for (int p = 0; p < 4; ++p) {
        mag[p] = mag_in[p];
        if (TWOS) {
            const uint32_t cm = (1u << a.code_bits) - 1u;
            uint32_t lo = mag[p] & 0xFFFFu, hi = mag[p] >> 16;
            if ((sgn[p] >> 15) & 1u) lo = (0u - lo) & cm;
            if (sgn[p] >> 31) hi = (0u - hi) & cm;
            mag[p] = lo | (hi << 16);
        }
    }
    const int64_t e0 = row * a.Kp + k0;
    const int bits = a.code_bits;
    if (bits <= 5) {
        uint32_t w = 0, sb = 0;
        #pragma unroll
        for (int p = 0; p < 4; ++p) {
            uint32_t lo = mag[p] & 0xFFFFu, hi = mag[p] >> 16;
            const uint32_t slo = (sgn[p] >> 15) & 1u, shi = sgn[p] >> 31;
            if (bits == 4 && !TWOS) { lo |= slo << 3; hi |= shi << 3; }
            w |= ((lo & 0xFu) | ((hi & 0xFu) << 4)) << (8 * p);
            sb |= (slo | (shi << 1)) << (2 * p);
        }
        *reinterpret_cast<uint32_t*>(a.out.codes + (e0 >> 1)) = w;
        if (bits == 5 && a.out.sign) a.out.sign[e0 >> 3] = (uint8_t)sb;
    } else {
        uint32_t w[2] = {0, 0};
        #pragma unroll
        for (int p = 0; p < 4; ++p) {
            uint32_t lo = mag[p] & 0xFFFFu, hi = mag[p] >> 16;
            if (!TWOS) {
                lo |= ((sgn[p] >> 15) & 1u) << a.sign_bit;
                hi |= (sgn[p] >> 31) << a.sign_bit;
            }
            w[p >> 1] |= ((lo & 0xFFu) | ((hi & 0xFFu) << 8)) << (16 * (p & 1));
        }
        *reinterpret_cast<uint2*>(a.out.codes + e0) = make_uint2(w[0], w[1]);
    }
}

// (row, chunk-in-row) of a flat chunk index; 32-bit division when the tensor allows it.
__device__ __forceinline__ void split_chunk(const QArgs& a, int64_t ci, int64_t& row, int64_t& c)
{
    if (a.total_chunks <= 0x7FFFFFFFll) {
        const uint32_t r = (uint32_t)ci / (uint32_t)a.cpr;
        row = r; c = (uint32_t)ci - r * (uint32_t)a.cpr;
    } else { row = ci / a.cpr; c = ci % a.cpr; }
}

__device__ __forceinline__ float group_max(float v, int G)
{
    for (int off = G >> 1; off >= 1; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
    return v;
}
__device__ __forceinline__ float group_sum(float v, int lanes)
{
    for (int off = lanes >> 1; off >= 1; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    return v;
}
__device__ __forceinline__ uint32_t group_or(uint32_t v, int G)
{
    for (int off = G >> 1; off >= 1; off >>= 1) v |= __shfl_xor_sync(0xFFFFFFFFu, v, off);
    return v;
}

__device__ __forceinline__ float chunk_absmax(const Chunk& c)
{
    __half2 m = __hmax2(bits_h2(h2_bits(c.h[0]) & 0x7FFF7FFFu), bits_h2(h2_bits(c.h[1]) & 0x7FFF7FFFu));
    m = __hmax2(m, bits_h2(h2_bits(c.h[2]) & 0x7FFF7FFFu));
    m = __hmax2(m, bits_h2(h2_bits(c.h[3]) & 0x7FFF7FFFu));
    const float2 f = __half22float2(m);
    return fmaxf(f.x, f.y);
}

// FP shared scale: clip to [sc_lo, sc_hi] then fp_quant (HBQQuantizer.quant_scale,
// src/quantizer.py:735-739; MXFPQuantizer.get_shared_scale, src/quantizer.py:504-509).
// For E5M3 without subnormals and without ceil the chain reduces to round-half-up of the
// 3-bit mantissa on the fp16 pattern (checked over all fp16 inputs by the tests).
__device__ __forceinline__ void store_scale(const QArgs& a, int64_t row, int64_t kb, float s)
{
    const uint16_t b = h_bits(__float2half_rn(s));
    const int64_t i = row * a.nblk + kb;
    if (a.out.scale_h) a.out.scale_h[i] = b;
    if (a.out.scale_u8) a.out.scale_u8[i] = (uint8_t)(b >> 7);
}

// x / s rounded to fp16, for two values.  rs = 1/s correctly rounded.  The reciprocal form is
// exact because s has at most 4 significant bits: the quotient of an 11-bit by a <=4-bit
// integer never lies within 2^-16 (relative) of an fp16 rounding boundary unless it is
// exactly representable, while the two fp32 roundings err by at most 2^-23.
__device__ __forceinline__ __half2 div2_h(float x0, float x1, float s, float rs, bool exact)
{
    return exact ? __floats2half2_rn(__fdiv_rn(x0, s), __fdiv_rn(x1, s))
                 : __floats2half2_rn(x0 * rs, x1 * rs);
}



// Output row of input row r = (b*T + t)*H + h when the K/Q-cache permutation is on: (b*H + h)*T + t.
__device__ __forceinline__ int64_t out_row(const QArgs& a, int64_t r)
{
    if (a.perm_T <= 0) return r;
    const int64_t bt = r / a.perm_H, h = r - bt * a.perm_H;
    const int64_t b = bt / a.perm_T, t = bt - b * a.perm_T;
    return (b * a.perm_H + h) * a.perm_T + t;
}

// RoPE on a chunk (apply_rotary_pos_emb of transformers' Llama: x*cos + rotate_half(x)*sin with
// rotate_half(x) = cat(-x[D/2:], x[:D/2]); every product and the sum are rounded to fp16 as the
// reference's fp16 tensor ops round them).  A row is one head (K = D, a power of two <= 256), so its D/8
// chunks sit in consecutive lanes of one warp and the partner elements d +- D/2 live D/16 lanes away.
__device__ __forceinline__ void rope_chunk(const QArgs& a, Chunk& x, int64_t row, int64_t k0)
{
    const int64_t bt = a.perm_H > 0 ? row / a.perm_H : row;
    const int64_t crow = bt % a.rope_rows;
    const uint4 cv = __ldg(reinterpret_cast<const uint4*>(a.rope_cos + crow * a.K + k0));
    const uint4 sv = __ldg(reinterpret_cast<const uint4*>(a.rope_sin + crow * a.K + k0));
    const uint32_t c[4] = {cv.x, cv.y, cv.z, cv.w}, s[4] = {sv.x, sv.y, sv.z, sv.w};
    const uint32_t neg = (2 * k0 < a.K) ? 0x80008000u : 0u;         // first half of D takes -x[d + D/2]
    #pragma unroll
    for (int p = 0; p < 4; ++p) {
        const uint32_t partner = __shfl_xor_sync(0xFFFFFFFFu, h2_bits(x.h[p]), (int)(a.cpr >> 1));
        // the _rn forms keep ptxas from contracting the products into the sum
        const __half2 t1 = __hmul2_rn(x.h[p], bits_h2(c[p]));
        const __half2 t2 = __hmul2_rn(bits_h2(partner ^ neg), bits_h2(s[p]));
        x.h[p] = __hadd2_rn(t1, t2);
    }
}
// K-cache centring (src/module.py:229-244): key_states - center with center [B, H, 1, D], one fp16
// subtraction after the rotation.  Rows are (b, t, h) of the projection output.
__device__ __forceinline__ void center_chunk(const QArgs& a, Chunk& x, int64_t row, int64_t k0)
{
    const int64_t bt = row / a.perm_H, h = row - bt * a.perm_H, b = bt / a.perm_T;
    const uint4 cv = __ldg(reinterpret_cast<const uint4*>(a.k_center + ((b * a.perm_H + h) * a.K + k0)));
    const uint32_t c[4] = {cv.x, cv.y, cv.z, cv.w};
    #pragma unroll
    for (int p = 0; p < 4; ++p) x.h[p] = __hsub2_rn(x.h[p], bits_h2(c[p]));
}
}  // namespace hbq
