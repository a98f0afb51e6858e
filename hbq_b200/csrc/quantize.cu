// Block quantize-dequantize kernels: MXFP / NVFP / MXINT / HBQ (two-level scale).
//
// Reference semantics (src/quantizer.py): eager torch ops on fp16 tensors, i.e. every
// elementwise op rounds its result to fp16 and reductions accumulate in fp32.  The kernels
// reproduce that op by op with fp16 hardware arithmetic (one rounding per instruction) so the
// fake-quantised tensor, the shared scales, the micro-scale indices and the scheme bits are
// bit-identical to the reference's.
//
// Work decomposition: one thread owns 8 consecutive elements of a row (one 128-bit load);
// the G = block_size/8 lanes that own one quantisation block reduce with warp shuffles, so a
// tensor is read once from HBM and every output is written once.
#include "quantize_dev.cuh"
#include <stdlib.h>
#include "vcache_dev.cuh"
#include "quantize_tab.cuh"
#include <math.h>
#include <mutex>

namespace hbq {

// ------------------------------------------------------------------------------------------
// Scalar building blocks (literal restatement of the reference's op chain; used for the shared
// scale -- once per block -- and for element formats without a packed fast path).
// ------------------------------------------------------------------------------------------

__device__ __forceinline__ float sgnf(float x) { return x > 0.f ? 1.f : (x < 0.f ? -1.f : 0.f); }

// floor(log2(t)) as evaluated on an fp16 tensor: log2 in fp32, rounded to fp16, then floor.
__device__ __forceinline__ float log2_h(float t) { return rh(log2f(t)); }

struct FpFmt {
    int ebit, mbit, emax, emin;
    float min_norm, thr, mant_shift, mant_max;
};

__host__ __device__ inline FpFmt make_fpfmt(int ebit, int mbit)
{
    FpFmt f;
    f.ebit = ebit; f.mbit = mbit;
    f.emax = (ebit == 5) ? 15 : (1 << (ebit - 1));
    f.emin = 2 - (1 << (ebit - 1));
    f.min_norm = (ebit == 1) ? 1.f : ldexpf(1.f, f.emin);
    f.thr = f.min_norm - ldexpf(1.f, -(mbit + 1) + f.emin);
    f.mant_shift = ldexpf(1.f, mbit);
    f.mant_max = f.mant_shift - 1.f;
    return f;
}

// make_fp_quant closure (src/quantizer.py:202-255; elem_variant = 1: the "+0.5004" rounding,
// which the fp16 add sees as 0.50048828125) and the free function fp_quant
// (src/quantizer.py:259-328; elem_variant = 0: "+0.5").  x holds an fp16 value.
// *code receives {exp field, mantissa} as the detailed output defines them.
__device__ float fpq_chain(float x, const FpFmt& f, bool allow_sub, bool use_ceil,
                           bool elem_variant, int* code)
{
    const float ax = fabsf(x);
    const bool is_zero = (x == 0.f);
    const bool promote = (ax < f.min_norm) && (ax >= f.thr);
    const bool below = (ax < f.thr) && !is_zero;
    const bool sub = allow_sub && below;
    const bool under = !allow_sub && below;

    float e = floorf(log2_h(rh(ax + (is_zero ? 1.f : 0.f))));
    e = fminf(fmaxf(e, (float)f.emin), (float)f.emax);
    const float p2 = rh(exp2f(e));
    const float sg = sgnf(x);
    const float xs = rh(__fdiv_rn(x, p2));
    const float mant = sub ? rh(xs * f.mant_shift) : rh(rh(xs - sg) * f.mant_shift);
    const float am = fabsf(mant);
    float mr;
    if (use_ceil) mr = ceilf(am);
    else mr = floorf(rh(am + (elem_variant ? 0.50048828125f : 0.5f)));
    const bool overflow = (mr > f.mant_max) && (e != (float)f.emax);
    mr = fminf(mr, f.mant_max);
    if (is_zero || under || overflow || promote) mr = 0.f;
    if (overflow) e += 1.f;
    const float sm = sg * mr;
    const float p2b = rh(exp2f(e));
    float xq = sub ? rh(rh(__fdiv_rn(sm, f.mant_shift)) * p2b)
                   : rh(rh(rh(__fdiv_rn(sm, f.mant_shift)) + sg) * p2b);
    if (is_zero || under) xq = 0.f;
    if (f.ebit == 4 && f.mbit == 3) xq = fminf(fmaxf(xq, -448.f), 448.f);
    if (code) {
        int ef = (int)e + ((1 << (f.ebit - 1)) - 1);
        if (is_zero || under || sub) ef = 0;
        *code = (ef << f.mbit) | (int)mr;
    }
    return xq;
}

__device__ __forceinline__ float quant_scale_fp(const QArgs& a, float s)
{
    s = fminf(fmaxf(s, a.sc_lo), a.sc_hi);
    if (a.scale_fast_e5m3) {
        const uint32_t b = (uint32_t)h_bits(__float2half_rn(s));
        return __half2float(bits_h((uint16_t)((b + 0x40u) & 0xFF80u)));
    }
    const FpFmt sf = make_fpfmt(a.f.sc_ebit, a.f.sc_mbit);
    return fpq_chain(s, sf, a.f.scale_allow_subnormal != 0, a.f.use_ceil != 0, false, nullptr);
}

// Power-of-two shared exponent (src/quantizer.py:395-407, 491-503): log2 evaluated in fp16.
__device__ __forceinline__ float pot_scale(const QArgs& a, float amax, bool use_round)
{
    const float t = rh(amax + (amax == 0.f ? 6.103515625e-05f : 0.f));
    const float l = log2_h(t);
    float e = use_round ? rintf(l) : floorf(l);
    e = rh(e - (float)a.pot_sub);
    e = fminf(fmaxf(e, (float)a.pot_emin), (float)a.pot_emax);
    return rh(exp2f(e));
}

// ------------------------------------------------------------------------------------------
// MXFP / NVFP / MXINT kernel.  MB >= 0: E2M<MB> packed fast path; MB = -1: generic element
// format through the literal chain; KIND = MXINT ignores MB.
// ------------------------------------------------------------------------------------------
template <int KIND, int MB>
__global__ void __launch_bounds__(256) mx_quantize_kernel(const QArgs a)
{
    const int64_t ci = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool valid = ci < a.total_chunks;
    int64_t row = 0, c = 0;
    if (valid) split_chunk(a, ci, row, c);
    const int64_t k0 = c * 8;
    Chunk x;
    if (valid) x = load_chunk(a, row, k0);
    else { for (int p = 0; p < 4; ++p) x.h[p] = bits_h2(0u); }
    if (a.rope_cos) rope_chunk(a, x, row, k0);
    if (a.k_center) center_chunk(a, x, row, k0);

    // per-tensor scale (src/quantizer.py:516-524): the reference divides the fp16 tensor by a
    // Python double, which torch evaluates as an fp32 division by float(scale) rounded to fp16
    float tsf = 1.f;
    if (KIND == HBQ_KIND_MXFP && a.f.per_tensor_scale) {
        const float tmax = *a.tensor_amax;
        if (tmax != 0.f) tsf = (float)((double)tmax / a.pts_den);
        #pragma unroll
        for (int p = 0; p < 4; ++p) {
            const float2 f = __half22float2(x.h[p]);
            x.h[p] = __floats2half2_rn(__fdiv_rn(f.x, tsf), __fdiv_rn(f.y, tsf));
        }
    }
    const float amax = group_max(chunk_absmax(x), a.G);
    float s;
    if (KIND == HBQ_KIND_MXINT) {
        if (a.f.sc_mbit == 0) s = pot_scale(a, amax, false);
        else {
            // quantise first, then clip from below only (src/quantizer.py:409-412)
            const FpFmt sf = make_fpfmt(a.f.sc_ebit, a.f.sc_mbit);
            s = fpq_chain(rh(__fdiv_rn(amax, a.elem_max)), sf, a.f.scale_allow_subnormal != 0,
                          a.f.use_ceil != 0, false, nullptr);
            s = fmaxf(s, a.sc_lo);
        }
    } else {
        if (a.f.sc_mbit == 0) s = pot_scale(a, amax, a.f.use_round != 0);
        else s = quant_scale_fp(a, rh(__fdiv_rn(amax, a.elem_max)));
    }
    const float rs = __frcp_rn(s);
    const bool exact = a.exact_div != 0 || (KIND != HBQ_KIND_MXINT && MB < 0);
    const __half2 s2 = __float2half2_rn(s);

    __half2 d[4];
    uint32_t mag[4], sg[4];
    #pragma unroll
    for (int p = 0; p < 4; ++p) {
        const float2 xf = __half22float2(x.h[p]);
        const __half2 y = div2_h(xf.x, xf.y, s, rs, exact);
        __half2 q;
        if (KIND == HBQ_KIND_MXINT) {
            // sign(y) * floor(|y| + 0.5), clipped to [-2^(n-1), 2^(n-1)-1] (src/quantizer.py:421-422)
            const uint32_t u = h2_bits(y);
            const uint32_t ab = u & 0x7FFF7FFFu;
            uint32_t sgn = u & 0x80008000u;
            const __half2 k = h2floor(__hadd2(bits_h2(ab), bits_h2(0x38003800u)));
            const float qmax = (float)((1 << (a.f.mbit - 1)) - 1);
            const uint32_t lp = h2_bits(__float2half2_rn(qmax)), ln = h2_bits(__float2half2_rn(qmax + 1.f));
            const uint32_t nm = (sgn >> 15) * 0xFFFFu;
            const __half2 kc = __hmin2(k, bits_h2((lp & ~nm) | (ln & nm)));
            sgn &= __hne2_mask(bits_h2(ab), bits_h2(0u));
            q = bits_h2(h2_bits(kc) | sgn);
            // integer code magnitude: k + 1024 keeps k in the low mantissa bits
            mag[p] = h2_bits(__hadd2(kc, bits_h2(0x64006400u))) & 0x01FF01FFu;
            sg[p] = sgn;
        } else if (MB >= 0) {
            q = q2_e2<(MB >= 0 ? MB : 1), true>(y);
            mag[p] = code2_e2<(MB >= 0 ? MB : 1)>(q);
            sg[p] = h2_bits(q) & 0x80008000u;
        } else {
            const FpFmt ef = make_fpfmt(a.f.ebit, a.f.mbit);
            const float2 yf = __half22float2(y);
            int c0, c1;
            const float q0 = fpq_chain(yf.x, ef, true, false, true, &c0);
            const float q1 = fpq_chain(yf.y, ef, true, false, true, &c1);
            q = __floats2half2_rn(q0, q1);
            mag[p] = (uint32_t)c0 | ((uint32_t)c1 << 16);
            sg[p] = ((yf.x < 0.f) ? 0x8000u : 0u) | ((yf.y < 0.f) ? 0x80000000u : 0u);
        }
        d[p] = __hmul2(q, s2);
        if (KIND == HBQ_KIND_MXFP && a.f.per_tensor_scale) {
            const float2 f = __half22float2(d[p]);
            d[p] = __floats2half2_rn(f.x * tsf, f.y * tsf);
        }
    }
    if (!valid) return;
    const int64_t orow = out_row(a, row);
    store_deq(a, orow, k0, d);
    store_codes<KIND == HBQ_KIND_MXINT>(a, orow, k0, mag, sg);
    if ((threadIdx.x & (a.G - 1)) == 0) store_scale(a, orow, c >> a.log2G, s);
}

// ------------------------------------------------------------------------------------------
// Fast path of the same computation for the shipped MX / NV configurations: E2Mx or integer
// elements with (a) a power-of-two scale whose exponent stays inside fp16's normal range or
// (b) an E5M3 scale without subnormals / ceil.  Everything stays in packed fp16:
//   (a) floor|round(log2(absmax)) evaluated on an fp16 tensor equals the exponent field of
//       absmax, plus one when the mantissa reaches a per-exponent threshold (the 94 values just
//       below a power of two for floor; the sqrt(2) point for round) -- a 32-entry table built by
//       the host with the same log2f; x / 2^e is one exact HMUL2;
//   (b) absmax / elem_max is a multiplication by the rounded reciprocal, the E5M3 rounding an
//       add + mask on the pattern, and x / scale a pre-scaled two-step fp16 division (exact for
//       every quotient >= 2^-14; smaller ones quantise to zero anyway).
// CODES: also emit element codes (needs the extra extraction arithmetic).
// ------------------------------------------------------------------------------------------
// The arithmetic of one 8-element chunk on the fast path: block maximum (G lanes), shared scale `sb`
// (fp16 pattern), fake-quantised values d and, with CODES, code magnitudes and signs.
template <int KIND, int MB, bool CODES>
__device__ __forceinline__ void mx_fast_chunk(const QArgs& a, const Chunk& x, __half2* d, uint32_t* mag, uint32_t* sg,
                                              uint32_t& sb)
{
    uint32_t ax[4];
    #pragma unroll
    for (int p = 0; p < 4; ++p) ax[p] = h2_bits(x.h[p]) & 0x7FFF7FFFu;
    uint32_t mx = h2_bits(__hmax2(__hmax2(bits_h2(ax[0]), bits_h2(ax[1])), __hmax2(bits_h2(ax[2]), bits_h2(ax[3]))));
    for (int off = a.G >> 1; off >= 1; off >>= 1)
        mx = h2_bits(__hmax2(bits_h2(mx), bits_h2(__shfl_xor_sync(0xFFFFFFFFu, mx, off))));
    const uint32_t am16 = max(mx & 0xFFFFu, mx >> 16);

    __half2 y[4];
    if (a.f.sc_mbit == 0) {
        int g;                         // floor|round(log2(absmax)) as the reference's fp16 tensor op gives it
        const int E = (int)(am16 >> 10);
        if (am16 == 0) g = -14;        // log2(0 + 2^-14)
        else if (E == 0) {             // subnormal maximum: rare, evaluate literally
            const float l = log2_h(__half2float(bits_h((uint16_t)am16)));
            g = (int)((KIND == HBQ_KIND_MXFP && a.f.use_round) ? rintf(l) : floorf(l));
        } else g = E - 15 + ((am16 & 0x3FFu) >= a.pot_thr[E] ? 1 : 0);
        const int e = min(max(g - a.pot_sub, a.pot_emin), a.pot_emax);       // within [-14, 15] on this path
        sb = (uint32_t)(e + 15) << 10;
        const uint32_t rs2 = (e == 15 ? 0x0200u : (uint32_t)(15 - e) << 10) * 0x00010001u;   // 2^-e
        #pragma unroll
        for (int p = 0; p < 4; ++p) y[p] = __hmul2(x.h[p], bits_h2(rs2));
    } else {
        const float sf = __half2float(bits_h((uint16_t)am16)) * a.inv_elem_max;
        uint32_t t = (uint32_t)h_bits(__float2half_rn(sf));
        t = min(max(t, 0x0400u), 0x7B80u);
        sb = (t + 0x40u) & 0xFF80u;
        const int e5 = (int)(sb >> 10) - 15;
        const int s1 = min(15, 8 - e5);
        const uint32_t pre2 = ((uint32_t)(s1 + 15) << 10) * 0x00010001u;
        const uint32_t post2 = ((uint32_t)(15 - (s1 + e5)) << 10) * 0x00010001u;
        const uint32_t nm2 = (0xBC00u | (sb & 0x03FFu)) * 0x00010001u;
        const uint32_t rm2 = (uint32_t)a.rm[(sb >> 7) & 7u] * 0x00010001u;
        #pragma unroll
        for (int p = 0; p < 4; ++p) {
            const __half2 xs = __hmul2(x.h[p], bits_h2(pre2));
            const __half2 q0 = __hmul2(xs, bits_h2(rm2));
            const __half2 r = __hfma2(q0, bits_h2(nm2), xs);
            y[p] = __hmul2(__hfma2(r, bits_h2(rm2), q0), bits_h2(post2));
        }
        // quotients below 2^-14 may be off by an ulp, which can only matter for the sign of a zero
        // result (the reference returns +0 when the quotient is exactly 0): redo those exactly
        const float sfl = __half2float(bits_h((uint16_t)sb));
        #pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint32_t tiny = __hle2_mask(bits_h2(h2_bits(y[p]) & 0x7FFF7FFFu), bits_h2(0x00200020u));
            if (tiny) {
                const float2 xf = __half22float2(x.h[p]);
                const __half2 ex = __floats2half2_rn(__fdiv_rn(xf.x, sfl), __fdiv_rn(xf.y, sfl));
                y[p] = bits_h2((h2_bits(y[p]) & ~tiny) | (h2_bits(ex) & tiny));
            }
        }
    }
    const __half2 s2 = bits_h2(sb * 0x00010001u);

    #pragma unroll
    for (int p = 0; p < 4; ++p) {
        __half2 q;
        if (KIND == HBQ_KIND_MXINT) {
            // sign(y) * floor(|y| + 0.5), clipped to [-2^(n-1), 2^(n-1)-1] (src/quantizer.py:421-422)
            const uint32_t u = h2_bits(y[p]);
            const uint32_t ab = u & 0x7FFF7FFFu;
            uint32_t sgn = u & 0x80008000u;
            // |y| + 0.5 capped at 1023 first (everything above the clip range behaves the same)
            const __half2 k = floor_small_h2(__hmin2(__hadd2(bits_h2(ab), bits_h2(0x38003800u)), bits_h2(0x63FE63FEu)));
            const uint32_t nm = (sgn >> 15) * 0xFFFFu;
            const __half2 kc = __hmin2(k, bits_h2((a.int_lim_pos & ~nm) | (a.int_lim_neg & nm)));
            sgn &= __hne2_mask(bits_h2(ab), bits_h2(0u));
            q = bits_h2(h2_bits(kc) | sgn);
            if (CODES) { mag[p] = h2_bits(__hadd2(kc, bits_h2(0x64006400u))) & 0x01FF01FFu; sg[p] = sgn; }
        } else {
            q = q2_e2<MB, true>(y[p]);
            if (CODES) { mag[p] = code2_e2<MB>(q); sg[p] = h2_bits(q) & 0x80008000u; }
        }
        d[p] = __hmul2(q, s2);
    }
}

// LEAN: the tensor is contiguous, 16-byte aligned, K a multiple of the block, and only the
//        fake-quantised output is wanted: chunk ci is elements [8 ci, 8 ci + 8) of both tensors, so
//        the row / column bookkeeping, RoPE / permutation and side outputs drop out.
__device__ __forceinline__ Chunk lean_load(const QArgs& a, int64_t ci)
{
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(a.x) + ci);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    Chunk c;
    if (!a.in_bf16) {
        #pragma unroll
        for (int p = 0; p < 4; ++p) c.h[p] = bits_h2(w[p]);
    } else {
        #pragma unroll
        for (int p = 0; p < 4; ++p)
            c.h[p] = __floats2half2_rn(__uint_as_float(w[p] << 16), __uint_as_float(w[p] & 0xFFFF0000u));
    }
    return c;
}

// The lean form is held to 32 registers so that 8 CTAs (all 64 warp slots) fit an SM: it needs 34
// without the cap and loses nothing to it (no spills), and the issue-bound loop gains 4-7 % from the
// extra warps.  The general form spills under that cap and is left alone.
template <int KIND, int MB, bool CODES, bool LEAN>
__global__ void __launch_bounds__(256, LEAN ? 8 : 1) mx_fast_kernel(const QArgs a)
{
    // Grid-stride loop with the next chunk's load issued before the current one is processed, so
    // every thread keeps a 16-byte load in flight while it computes.
    const int lane = threadIdx.x & 31;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t ci = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t row = 0, c = 0;
    if (!LEAN) split_chunk(a, ci < a.total_chunks ? ci : 0, row, c);
    Chunk x;
    if (ci < a.total_chunks) x = LEAN ? lean_load(a, ci) : load_chunk(a, row, c * 8);
    else { for (int p = 0; p < 4; ++p) x.h[p] = bits_h2(0u); }
    for (; ci - lane < a.total_chunks; ci += stride) {
    const bool valid = ci < a.total_chunks;
    const int64_t k0 = c * 8;
    const int64_t row_cur = row, c_cur = c;
    // advance (row, chunk-in-row) by one grid stride and prefetch
    if (!LEAN) {
        row += a.step_rows; c += a.step_chunks;
        if (c >= a.cpr) { c -= a.cpr; ++row; }
    }
    Chunk xn;
    if (ci + stride < a.total_chunks) xn = LEAN ? lean_load(a, ci + stride) : load_chunk(a, row, c * 8);
    else { for (int p = 0; p < 4; ++p) xn.h[p] = bits_h2(0u); }

    if (!LEAN && a.rope_cos) rope_chunk(a, x, valid ? row_cur : 0, k0);
    if (!LEAN && a.k_center) center_chunk(a, x, valid ? row_cur : 0, k0);
    __half2 d[4];
    uint32_t mag[4], sg[4], sb;
    mx_fast_chunk<KIND, MB, CODES>(a, x, d, mag, sg, sb);
    if (LEAN) {
        if (valid) {
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
            reinterpret_cast<uint4*>(a.deq)[ci] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else if (valid) {
        const int64_t orow = out_row(a, row_cur);
        store_deq(a, orow, k0, d);
        if (CODES) store_codes<KIND == HBQ_KIND_MXINT>(a, orow, k0, mag, sg);
        if ((threadIdx.x & (a.G - 1)) == 0) {
            const int64_t i = orow * a.nblk + (c_cur >> a.log2G);
            if (a.out.scale_h) a.out.scale_h[i] = (uint16_t)sb;
            if (a.out.scale_u8) a.out.scale_u8[i] = (uint8_t)(sb >> 7);
        }
    }
    x = xn;
    }   // grid-stride loop
}

// V-cache write for the MX / NV fast-path formats: blocks of block_size consecutive tokens per channel,
// through the shared-memory tile of vcache_dev.cuh.
template <int KIND, int MB>
struct MxChunkFn {
    const QArgs& a;
    __device__ __forceinline__ void operator()(const uint32_t* xb, uint32_t* dq) const
    {
        Chunk x;
        #pragma unroll
        for (int p = 0; p < 4; ++p) x.h[p] = bits_h2(xb[p]);
        __half2 d[4];
        uint32_t mag[4], sg[4], sb;
        mx_fast_chunk<KIND, MB, false>(a, x, d, mag, sg, sb);
        #pragma unroll
        for (int p = 0; p < 4; ++p) dq[p] = h2_bits(d[p]);
    }
};

template <int KIND, int MB>
__global__ void __launch_bounds__(V_THREADS, 2) mx_v_kernel(const QArgs a, const VArgs v)
{
    extern __shared__ __align__(16) uint32_t v_tile[];
    const MxChunkFn<KIND, MB> fn = {a};
    v_cache_tiles(v, v_tile, fn);
}

template <int KIND, int MB>
static int launch_mx_v(const QArgs& a, const KvWriteOpts* kv, cudaStream_t stream)
{
    VArgs v;
    if (!v_args_fill(&v, a.x, a.deq, a.in_bf16, a.out_bf16, kv->B, kv->T, kv->H, kv->D, a.f.block_size, kv->v_out_token_major)) return HBQ_ERR_UNSUPPORTED;
    if (v.tiles == 0) return HBQ_OK;
    int sms = 0;
    { const int rc = device_sms(&sms); if (rc) return rc; }
    const int grid = (int)(v.tiles < 2 * sms ? v.tiles : 2 * sms);
    { const int rc = ensure_dynamic_smem(mx_v_kernel<KIND, MB>, V_TILE_BYTES); if (rc) return rc; }
    mx_v_kernel<KIND, MB><<<grid, V_THREADS, V_TILE_BYTES, stream>>>(a, v);
    HBQ_LAUNCH_CHECK("mx_v_kernel");
    return HBQ_OK;
}

// ------------------------------------------------------------------------------------------
// HBQ kernel (HBQQuantizer.q, src/quantizer.py:741-859).
//   per scheme s (1, or 2 for "Mix"):  l1_s = E5M3(clip(absmax / (elem_max * max T_s)))
//   per micro-block: the candidate T_s[i] minimising fp16(sum fp16((x - deq_i)^2)), first wins
//   "Mix": the scheme minimising fp16(sum over the block of the selected errors), first wins.
// Pass 1 evaluates every candidate's error, pass 2 recomputes the winner (values + codes);
// nothing but the winner is kept in registers, so the candidate count is a run-time value.
// LPM = lanes per micro-block (l2_block_size / 8), 0 when l2_block_size = 4 (two per lane).
// ------------------------------------------------------------------------------------------
template <int MB>
struct HbqEval {
    // dequantised candidate for two elements: fp16(fp16(Q(fp16(a / t)) * t) * l1)
    template <bool ZS>
    static __device__ __forceinline__ __half2 deq2(float a0, float a1, float it, __half2 t2,
                                                   __half2 l1_2, __half2* c_out)
    {
        const __half2 b = __floats2half2_rn(a0 * it, a1 * it);
        const __half2 c = q2_e2<MB, ZS>(b);
        if (c_out) *c_out = c;
        return __hmul2(__hmul2(c, t2), l1_2);
    }
};

template <int MB>
__global__ void __launch_bounds__(256) hbq_quantize_kernel(const QArgs a)
{
    const int64_t ci = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool valid = ci < a.total_chunks;
    int64_t row = 0, c = 0;
    if (valid) split_chunk(a, ci, row, c);
    const int64_t k0 = c * 8;
    Chunk x;
    if (valid) x = load_chunk(a, row, k0);
    else { for (int p = 0; p < 4; ++p) x.h[p] = bits_h2(0u); }
    if (a.rope_cos) rope_chunk(a, x, row, k0);
    if (a.k_center) center_chunk(a, x, row, k0);

    const int L = a.f.l2_block_size;
    const int lpm = L >> 3;                  // lanes per micro-block (0 => two micro-blocks per lane)
    const int lpm_shift = lpm > 0 ? 31 - __clz(lpm) : 0;
    const float amax = group_max(chunk_absmax(x), a.G);

    float xf[8];
    #pragma unroll
    for (int p = 0; p < 4; ++p) { const float2 f = __half22float2(x.h[p]); xf[2 * p] = f.x; xf[2 * p + 1] = f.y; }

    __half2 best_d[4];
    uint32_t best_mag[4], best_sg[4];
    float best_l1 = 0.f, best_err = 0.f;
    int best_s = 0, best_i0 = 0, best_i1 = 0;

    for (int s = 0; s < a.nscheme; ++s) {
        const float l1 = quant_scale_fp(a, rh(__fdiv_rn(amax, a.ele_max[s])));
        const float rl1 = __frcp_rn(l1);
        const __half2 l1_2 = __float2half2_rn(l1);
        float af[8];
        #pragma unroll
        for (int p = 0; p < 4; ++p) {
            const float2 f = __half22float2(div2_h(xf[2 * p], xf[2 * p + 1], l1, rl1, a.exact_div != 0));
            af[2 * p] = f.x; af[2 * p + 1] = f.y;
        }
        // ---- pass 1: error of every candidate --------------------------------------------
        float bE0 = 0.f, bE1 = 0.f;
        int i0 = 0, i1 = 0;
        for (int i = 0; i < a.nc; ++i) {
            const float it = a.inv_tab[s][i];
            const __half2 t2 = __float2half2_rn(a.tab[s][i]);
            float acc0 = 0.f, acc1 = 0.f;
            #pragma unroll
            for (int p = 0; p < 4; ++p) {
                const __half2 d = HbqEval<MB>::template deq2<false>(af[2 * p], af[2 * p + 1], it, t2, l1_2, nullptr);
                const __half2 r = __hsub2(x.h[p], d);
                const float2 e = __half22float2(__hmul2(r, r));
                if (p < 2 || lpm != 0) { acc0 += e.x; acc0 += e.y; } else { acc1 += e.x; acc1 += e.y; }
            }
            float E0, E1;
            if (lpm == 0) { E0 = rh(acc0); E1 = rh(acc1); }
            else { E0 = rh(group_sum(acc0, lpm)); E1 = E0; }
            if (i == 0 || E0 < bE0) { bE0 = E0; i0 = i; }
            if (i == 0 || E1 < bE1) { bE1 = E1; i1 = i; }
        }
        // ---- pass 2: recompute the winners -------------------------------------------------
        __half2 d[4];
        uint32_t mag[4], sg[4];
        float esum = 0.f;
        #pragma unroll
        for (int p = 0; p < 4; ++p) {
            const int i = (p < 2) ? i0 : i1;
            const float it = a.inv_tab[s][i];
            const __half2 t2 = __float2half2_rn(a.tab[s][i]);
            __half2 cq;
            d[p] = HbqEval<MB>::template deq2<true>(af[2 * p], af[2 * p + 1], it, t2, l1_2, &cq);
            mag[p] = code2_e2<MB>(cq);
            sg[p] = h2_bits(cq) & 0x80008000u;
            if (a.nscheme > 1) {
                const __half2 r = __hsub2(x.h[p], d[p]);
                const float2 e = __half22float2(__hmul2(r, r));
                esum += e.x; esum += e.y;
            }
        }
        float Es = 0.f;
        if (a.nscheme > 1) Es = rh(group_sum(esum, a.G));
        if (s == 0 || Es < best_err) {
            best_err = Es; best_s = s; best_l1 = l1; best_i0 = i0; best_i1 = i1;
            #pragma unroll
            for (int p = 0; p < 4; ++p) { best_d[p] = d[p]; best_mag[p] = mag[p]; best_sg[p] = sg[p]; }
        }
    }

    // ---- micro-scale indices ------------------------------------------------------------------
    const int lig = threadIdx.x & (a.G - 1);       // lane in group
    const int nl2 = a.f.block_size / L;
    uint32_t l2word = 0;
    if (lpm == 0) l2word = ((uint32_t)best_i0 | ((uint32_t)best_i1 << a.f.l2_sc_bit)) << (2 * lig * a.f.l2_sc_bit);
    else if ((lig & (lpm - 1)) == 0) l2word = (uint32_t)best_i0 << (((lig >> lpm_shift)) * a.f.l2_sc_bit);
    if (a.out.l2_packed) l2word = group_or(l2word, a.G);

    if (!valid) return;
    const int64_t kb = c >> a.log2G;
    row = out_row(a, row);
    store_deq(a, row, k0, best_d);
    store_codes<false>(a, row, k0, best_mag, best_sg);
    if (a.out.l2_idx) {
        uint8_t* lp = a.out.l2_idx + (row * a.nblk + kb) * nl2;
        if (lpm == 0) { lp[2 * lig] = (uint8_t)best_i0; lp[2 * lig + 1] = (uint8_t)best_i1; }
        else if ((lig & (lpm - 1)) == 0) lp[(lig >> lpm_shift)] = (uint8_t)best_i0;
    }
    if (lig == 0) {
        store_scale(a, row, kb, best_l1);
        if (a.out.scheme) a.out.scheme[row * a.nblk + kb] = (uint8_t)best_s;
        if (a.out.l2_packed) {
            const int nbytes = (nl2 * a.f.l2_sc_bit) >> 3;
            uint8_t* lp = a.out.l2_packed + (row * a.nblk + kb) * nbytes;
            if (nbytes == 4) *reinterpret_cast<uint32_t*>(lp) = l2word;
            else if (nbytes == 2) *reinterpret_cast<uint16_t*>(lp) = (uint16_t)l2word;
            else *lp = (uint8_t)l2word;
        }
    }
}

// ------------------------------------------------------------------------------------------
// Element quantizer alone (test / utility entry point).
// ------------------------------------------------------------------------------------------
__global__ void fp_quant_kernel(const uint16_t* x, int64_t n, int ebit, int mbit, int allow_sub,
                                int use_ceil, int elem_variant, uint16_t* out)
{
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i >= n) return;
    const bool two = i + 1 < n;
    const __half h0 = bits_h(x[i]), h1 = two ? bits_h(x[i + 1]) : __float2half(0.f);
    __half2 r;
    const bool fast = ebit == 2 && allow_sub && !use_ceil && elem_variant;
    const __half2 b = __halves2half2(h0, h1);
    if (fast && mbit == 1) r = q2_e2<1, true>(b);
    else if (fast && mbit == 2) r = q2_e2<2, true>(b);
    else if (fast && mbit == 3) r = q2_e2<3, true>(b);
    else if (fast && mbit == 5) r = q2_e2<5, true>(b);
    else {
        const FpFmt f = make_fpfmt(ebit, mbit);
        r = __floats2half2_rn(
            fpq_chain(__half2float(h0), f, allow_sub != 0, use_ceil != 0, elem_variant != 0, nullptr),
            fpq_chain(__half2float(h1), f, allow_sub != 0, use_ceil != 0, elem_variant != 0, nullptr));
    }
    out[i] = h_bits(__low2half(r));
    if (two) out[i + 1] = h_bits(__high2half(r));
}

// ------------------------------------------------------------------------------------------
// absmax (per-tensor scale support): two stages, partial maxima in caller-provided scratch.
// ------------------------------------------------------------------------------------------
constexpr int kAbsmaxBlocks = 1184;   // 8 x 148 SMs
constexpr int kAbsmaxThreads = 256;

__global__ void __launch_bounds__(kAbsmaxThreads)
absmax_partial_kernel(const uint16_t* x, int64_t n, int in_bf16, float* partial)
{
    float m = 0.f;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t nvec = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) ? n / 8 : 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(x) + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        #pragma unroll
        for (int p = 0; p < 4; ++p) {
            float f0, f1;
            if (in_bf16) { f0 = __uint_as_float(w[p] << 16); f1 = __uint_as_float(w[p] & 0xFFFF0000u); }
            else { const float2 f = __half22float2(bits_h2(w[p])); f0 = f.x; f1 = f.y; }
            m = fmaxf(m, fmaxf(fabsf(f0), fabsf(f1)));
        }
    }
    for (int64_t i = nvec * 8 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float f = in_bf16 ? __uint_as_float((uint32_t)x[i] << 16) : __half2float(bits_h(x[i]));
        m = fmaxf(m, fabsf(f));
    }
    m = group_max(m, 32);
    __shared__ float sm[kAbsmaxThreads / 32];
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = threadIdx.x < kAbsmaxThreads / 32 ? sm[threadIdx.x] : 0.f;
        m = group_max(m, 32);
        if (threadIdx.x == 0) partial[blockIdx.x] = m;
    }
}

__global__ void __launch_bounds__(kAbsmaxThreads)
absmax_final_kernel(const float* partial, int nparts, int in_bf16, float* amax)
{
    float m = 0.f;
    for (int i = threadIdx.x; i < nparts; i += blockDim.x) m = fmaxf(m, partial[i]);
    m = group_max(m, 32);
    __shared__ float sm[kAbsmaxThreads / 32];
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = threadIdx.x < kAbsmaxThreads / 32 ? sm[threadIdx.x] : 0.f;
        m = group_max(m, 32);
        // bf16 input is quantised in fp16: the maximum is that of the converted tensor
        if (threadIdx.x == 0) *amax = in_bf16 ? rh(m) : m;
    }
}

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
int hbq_lut_try_launch(const QArgs& qa, int mb, cudaStream_t stream, bool* launched);   // quantize_lut.cu

int quantize_extra_launch(const QArgs& qa, cudaStream_t stream);                                       // quantize_extra.cu
int hbq_lut_v_launch(const QArgs& qa, int mb, const void* in, void* out, int in_bf16, int out_bf16,
                     int64_t B, int64_t T, int64_t H, int64_t D, int out_token_major, cudaStream_t stream);                  // quantize_lut.cu

static float h_rh(float f) { return __half2float(__float2half_rn(f)); }

static double h_max_norm(int ebit, int mbit)
{
    if (ebit == 0) return ldexp(1.0, mbit - 1) - 1;
    if (ebit == 4 && mbit == 3) return 448.0;
    const int emax = (ebit == 5) ? 15 : (1 << (ebit - 1));
    return ldexp(1.0, emax) * (ldexp(1.0, mbit + 1) - 1) / ldexp(1.0, mbit);
}
static double h_min_norm(int ebit) { return ebit == 0 ? 0.0 : (ebit == 1 ? 1.0 : ldexp(1.0, 2 - (1 << (ebit - 1)))); }
static double h_min_subnorm(int ebit, int mbit) { return ldexp(1.0, 2 - (1 << (ebit - 1)) - mbit); }

// Micro-scale tables (src/quantizer.py:745-770), values as fp16 arithmetic produces them.
static int l2_tables(int scheme, int bits, float tab[2][16])
{
    const int n = 1 << bits;
    int ns = 1;
    for (int i = 0; i < n; ++i) {
        const float r = (float)i;
        const float fp = h_rh(1.f + h_rh(r / (float)(1 << bits)));
        const float fp10 = h_rh(1.f + h_rh(r / (float)(1 << (bits + 1))));
        switch (scheme) {
            case HBQ_L2_POT: tab[0][i] = h_rh(exp2f(r)); break;
            case HBQ_L2_INT: tab[0][i] = h_rh(r + 1.f); break;
            case HBQ_L2_SIG1: tab[0][i] = h_rh(1.f + h_rh(r / 2.f)); break;
            case HBQ_L2_FPM1: tab[0][i] = fp; break;
            case HBQ_L2_FP1: tab[0][i] = h_rh(1.f + h_rh(h_rh(r + 1.f) / (float)(1 << bits))); break;
            case HBQ_L2_FPM10: tab[0][i] = fp10; break;
            case HBQ_L2_FPM100: tab[0][i] = h_rh(1.f + h_rh(r / (float)(1 << (bits + 2)))); break;
            case HBQ_L2_MIX: tab[0][i] = fp; tab[1][i] = fp10; ns = 2; break;
            default: return -1;
        }
    }
    return ns;
}

static bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

// pot_thr[E] for the fast path: the smallest mantissa of an fp16 value with exponent field E whose
// floor (or round) of the fp16-rounded log2 is E - 14 instead of E - 15; 1024 if there is none.
static void build_pot_table(bool use_round, uint16_t thr[32])
{
    // computed once per process and rounding rule (30 x 1024 log2f evaluations)
    static uint16_t cache[2][32];
    static bool ready[2] = {false, false};
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const int w = use_round ? 1 : 0;
    if (!ready[w]) {
        for (int E = 0; E < 32; ++E) cache[w][E] = 1024;
        for (int E = 1; E <= 30; ++E) {
            for (int m = 0; m < 1024; ++m) {
                const float v = __half2float(__ushort_as_half((unsigned short)((E << 10) | m)));
                const float l = h_rh(log2f(v));
                const int g = (int)(use_round ? nearbyintf(l) : floorf(l));
                if (g > E - 15) { cache[w][E] = (uint16_t)m; break; }
            }
        }
        ready[w] = true;
    }
    memcpy(thr, cache[w], sizeof(cache[w]));
}

template <int KIND, int MB, bool CODES, bool LEAN>
static int launch_mx_fast_as(QArgs& a, dim3 grid, dim3 block, cudaStream_t stream)
{
    // a multiple of the CTAs that are resident at once (asked of the occupancy calculator: registers
    // decide, 8 for the lean form, fewer for the general one), each looping over chunks: no thinly
    // occupied last wave
    int sms = 0, per_sm = 0;
    { const int rc = device_sms(&sms); if (rc) return rc; }
    { const int rc = resident_ctas(mx_fast_kernel<KIND, MB, CODES, LEAN>, (int)block.x, 0, &per_sm); if (rc) return rc; }
    // ... times 4: the warps of an SM do not finish together, and with four generations of CTAs the
    // hardware scheduler refills the gaps (measured at 6 CTAs per SM: 1 wave 3949, 2: 4026, 4 or 8: 4125, 16: 3996 GB/s)
    constexpr int kWaves = 4;
    if ((int64_t)grid.x > (int64_t)sms * per_sm * kWaves) grid.x = (unsigned)(sms * per_sm * kWaves);
    const int64_t stride = (int64_t)grid.x * block.x;
    a.step_rows = stride / a.cpr;
    a.step_chunks = stride % a.cpr;
    mx_fast_kernel<KIND, MB, CODES, LEAN><<<grid, block, 0, stream>>>(a);
    return HBQ_OK;
}

template <int KIND, int MB>
static int launch_mx_fast(QArgs& a, dim3 grid, dim3 block, cudaStream_t stream)
{
    const bool side_out = a.out.codes || a.out.sign || a.out.scale_u8 || a.out.scale_h || a.out.l2_packed ||
                          a.out.l2_idx || a.out.scheme;
    if (a.deq && !side_out && a.aligned && a.K == a.Kp && !a.rope_cos && a.perm_T <= 0 && !a.k_center)
        return launch_mx_fast_as<KIND, MB, false, true>(a, grid, block, stream);
    if (a.out.codes) return launch_mx_fast_as<KIND, MB, true, false>(a, grid, block, stream);
    return launch_mx_fast_as<KIND, MB, false, false>(a, grid, block, stream);
}

// The packed form stores a block's scale as one byte (bits 14..7 of its fp16 pattern) and nothing per tensor.
// Formats whose scale does not fit that byte would dequantise to other values than their fake-quantised
// tensor, so they have no packed form: a per-tensor scale (the tensor maximum is not stored), a scale
// mantissa wider than 3 bits (truncated by the byte), a power-of-two scale outside fp16's exponent range.
int packed_form_supported(const hbq_format* f)
{
    if (f->kind == HBQ_KIND_MXFP && f->per_tensor_scale) return HBQ_ERR_UNSUPPORTED;
    if (f->kind == HBQ_KIND_MXFP || f->kind == HBQ_KIND_MXINT || f->kind == HBQ_KIND_HBQ) {
        if (f->sc_mbit > 3) return HBQ_ERR_UNSUPPORTED;
        if (f->sc_mbit > 0 && f->sc_ebit > 5) return HBQ_ERR_UNSUPPORTED;
        if (f->kind == HBQ_KIND_MXFP && f->sc_mbit == 0 && f->sc_ebit > 5) return HBQ_ERR_UNSUPPORTED;
    }
    return HBQ_OK;
}

// The format part of QArgs for an HBQ format (candidate tables, element maxima, scale rule), as
// quantize_launch fills it; *mb = mantissa bits of the E2Mx element.  HBQ_ERR_UNSUPPORTED for anything else.
int hbq_format_qargs(const hbq_format* f, QArgs* a, int* mb)
{
    if (!f || f->kind != HBQ_KIND_HBQ) return HBQ_ERR_UNSUPPORTED;
    const int B = f->block_size, L = f->l2_block_size;
    if (!is_pow2(B) || B < 8 || B > 256) return HBQ_ERR_UNSUPPORTED;
    if (f->ebit != 2 || f->mbit < 1 || f->mbit > 3 || f->sc_mbit == 0) return HBQ_ERR_UNSUPPORTED;
    if (!is_pow2(L) || L < 4 || L > B || f->l2_sc_bit < 0 || f->l2_sc_bit > 4) return HBQ_ERR_UNSUPPORTED;
    memset(a, 0, sizeof(*a));
    a->f = *f;
    a->f.per_tensor_scale = 0;
    a->G = B / 8;
    a->scale_fast_e5m3 = (f->sc_ebit == 5 && f->sc_mbit == 3 && !f->use_ceil && !f->scale_allow_subnormal);
    a->elem_max = (float)h_max_norm(f->ebit, f->mbit);
    a->nc = 1 << f->l2_sc_bit;
    a->nscheme = l2_tables(f->l2_scheme, f->l2_sc_bit, a->tab);
    if (a->nscheme < 0) return HBQ_ERR_ARG;
    for (int s = 0; s < a->nscheme; ++s) {
        float tmax = a->tab[s][0];
        for (int i = 0; i < a->nc; ++i) tmax = fmaxf(tmax, a->tab[s][i]);
        a->ele_max[s] = h_rh(h_rh(a->elem_max) * tmax);
    }
    *mb = f->mbit;
    return HBQ_OK;
}

int quantize_launch(const void* x, int dtype, int64_t rows, int64_t K, const hbq_format* f,
                    void* deq, int deq_dtype, const hbq_packed_out* out, const float* tensor_amax,
                    cudaStream_t stream, const KvWriteOpts* kv)
{
    if (!f || rows < 0 || K < 0) return HBQ_ERR_ARG;
    if (dtype != HBQ_DTYPE_F16 && dtype != HBQ_DTYPE_BF16) return HBQ_ERR_UNSUPPORTED;
    if (deq && deq_dtype != HBQ_DTYPE_F16 && deq_dtype != HBQ_DTYPE_BF16) return HBQ_ERR_UNSUPPORTED;
    if (rows == 0 || K == 0) return HBQ_OK;                 // empty tensors may come with null pointers
    if (!x) return HBQ_ERR_ARG;
    const int B = f->block_size;
    if (!is_pow2(B) || B < 8 || B > 256) return HBQ_ERR_UNSUPPORTED;
    const bool pts = f->kind == HBQ_KIND_MXFP && f->per_tensor_scale;    // the other kinds ignore it
    if (pts && !tensor_amax) return HBQ_ERR_ARG;
    if (out && (out->codes || out->scale_u8)) {
        const int rc = packed_form_supported(f);
        if (rc) return rc;
    }

    QArgs a;
    memset(&a, 0, sizeof(a));
    a.x = x; a.deq = deq;
    if (out) a.out = *out;
    a.tensor_amax = tensor_amax;
    a.rows = rows; a.K = K;
    a.nblk = (int)((K + B - 1) / B);
    a.Kp = (int64_t)a.nblk * B;
    a.cpr = a.Kp / 8;
    a.total_chunks = rows * a.cpr;
    a.in_bf16 = dtype == HBQ_DTYPE_BF16;
    a.out_bf16 = deq_dtype == HBQ_DTYPE_BF16;
    a.aligned = (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                (!deq || (reinterpret_cast<uintptr_t>(deq) & 15) == 0);
    a.G = B / 8;
    a.log2G = 0;
    while ((1 << a.log2G) < a.G) ++a.log2G;
    a.f = *f;
    a.f.per_tensor_scale = pts;
    if (kv && kv->glu_gate) {
        // fused silu(gate) * x: only the contiguous fp16 -> fp16 table path of the HBQ formats has it
        const bool side = out && (out->codes || out->sign || out->scale_u8 || out->scale_h || out->l2_packed ||
                                  out->l2_idx || out->scheme);
        if (!deq) return HBQ_ERR_ARG;
        if (f->kind != HBQ_KIND_HBQ || dtype != HBQ_DTYPE_F16 || deq_dtype != HBQ_DTYPE_F16 || side || pts || K % B != 0)
            return HBQ_ERR_UNSUPPORTED;
        if (!a.aligned || (reinterpret_cast<uintptr_t>(kv->glu_gate) & 15)) return HBQ_ERR_ALIGN;
        a.glu_gate = kv->glu_gate;
        kv = nullptr;
    }
    if (kv) {
        if (K % B != 0 || !is_pow2((int)K) || K < 16 || K > 256 || pts) return HBQ_ERR_UNSUPPORTED;
        if (kv->cos && (dtype != HBQ_DTYPE_F16 || !kv->sin || kv->rope_rows <= 0)) return HBQ_ERR_UNSUPPORTED;
        if (!deq) return HBQ_ERR_ARG;
        a.rope_cos = (const uint16_t*)kv->cos; a.rope_sin = (const uint16_t*)kv->sin; a.rope_rows = kv->rope_rows;
        a.perm_T = kv->T; a.perm_H = kv->H;
        a.k_center = (const uint16_t*)kv->center;
        if (kv->center && ((reinterpret_cast<uintptr_t>(kv->center) & 15) || dtype != HBQ_DTYPE_F16 || kv->v_axis)) return HBQ_ERR_UNSUPPORTED;
        if ((kv->cos && ((reinterpret_cast<uintptr_t>(kv->cos) | reinterpret_cast<uintptr_t>(kv->sin)) & 15)) || !a.aligned)
            return HBQ_ERR_ALIGN;
    }
    if (f->kind == HBQ_KIND_MXEX || f->kind == HBQ_KIND_VSQ) {
        if (kv) return HBQ_ERR_UNSUPPORTED;
        return quantize_extra_launch(a, stream);
    }
    a.scale_fast_e5m3 = (f->sc_ebit == 5 && f->sc_mbit == 3 && !f->use_ceil && !f->scale_allow_subnormal);
    a.exact_div = f->sc_mbit > 4;
    if (f->sc_mbit > 0) {
        a.sc_lo = (float)(f->scale_allow_subnormal ? h_min_subnorm(f->sc_ebit, f->sc_mbit) : h_min_norm(f->sc_ebit));
        a.sc_hi = (float)h_max_norm(f->sc_ebit, f->sc_mbit);
    }
    const dim3 block(256), grid((unsigned)((a.total_chunks + 255) / 256));

    if (f->kind == HBQ_KIND_MXINT) {
        if (f->mbit < 2 || f->mbit > 8) return HBQ_ERR_UNSUPPORTED;
        a.code_bits = f->mbit <= 4 ? 4 : 8;
        if (a.out.codes && f->mbit != 4 && f->mbit != 8) return HBQ_ERR_UNSUPPORTED;
        a.elem_max = (float)h_max_norm(0, f->mbit);
        a.pot_sub = f->mbit - 2; a.pot_emin = -14; a.pot_emax = 15;       // quantizer.py:403-405
        if (f->sc_mbit == 0) {
            build_pot_table(false, a.pot_thr);
            const float qmax = (float)((1 << (f->mbit - 1)) - 1);
            a.int_lim_pos = (uint32_t)__half_as_ushort(__float2half_rn(qmax)) * 0x00010001u;
            a.int_lim_neg = (uint32_t)__half_as_ushort(__float2half_rn(qmax + 1.f)) * 0x00010001u;
            if (kv && kv->v_axis) return launch_mx_v<HBQ_KIND_MXINT, 0>(a, kv, stream);
            { const int rc = launch_mx_fast<HBQ_KIND_MXINT, 0>(a, grid, block, stream); if (rc) return rc; }
            HBQ_LAUNCH_CHECK("mx_fast_kernel<mxint>");
            return HBQ_OK;
        }
        if (kv && kv->v_axis) return HBQ_ERR_UNSUPPORTED;      // token-axis write: fast-path formats only
        mx_quantize_kernel<HBQ_KIND_MXINT, 0><<<grid, block, 0, stream>>>(a);
        HBQ_LAUNCH_CHECK("mx_quantize_kernel<mxint>");
        return HBQ_OK;
    }
    if (f->ebit < 1 || f->ebit > 5 || f->mbit < 0 || f->mbit > 7 || f->ebit + f->mbit > 7) return HBQ_ERR_UNSUPPORTED;
    a.code_bits = 1 + f->ebit + f->mbit;
    if (a.code_bits < 4) a.code_bits = 4;
    if (a.code_bits > 5 && a.code_bits < 8) a.code_bits = 8;
    a.sign_bit = f->ebit + f->mbit;
    a.elem_max = (float)h_max_norm(f->ebit, f->mbit);
    const int fast_mb = (f->ebit == 2 && (f->mbit == 1 || f->mbit == 2 || f->mbit == 3 || f->mbit == 5)) ? f->mbit : -1;

    if (f->kind == HBQ_KIND_MXFP) {
        if (pts) {
            a.pts_den = (double)a.elem_max * h_max_norm(f->sc_ebit, f->sc_mbit);
        }
        a.pot_sub = 1 << (f->ebit - 1);
        a.pot_emin = 2 - (1 << (f->sc_ebit - 1)); a.pot_emax = (1 << (f->sc_ebit - 1)) - 1;   // quantizer.py:500-502
        if (f->sc_mbit == 0 && (f->sc_ebit < 2 || f->sc_ebit > 8)) return HBQ_ERR_UNSUPPORTED;
        const bool fast_scale = (f->sc_mbit == 0 && a.pot_emin >= -14 && a.pot_emax <= 15) ||
                                (a.scale_fast_e5m3 != 0);
        if (fast_mb >= 0 && !pts && fast_scale) {
            if (f->sc_mbit == 0) build_pot_table(f->use_round != 0, a.pot_thr);
            for (int i = 0; i < 8; ++i) a.rm[i] = __half_as_ushort(__float2half_rn(1.f / (1.f + i / 8.f)));
            a.inv_elem_max = 1.f / a.elem_max;
            if (kv && kv->v_axis) {
                switch (fast_mb) {
                    case 1: return launch_mx_v<HBQ_KIND_MXFP, 1>(a, kv, stream);
                    case 2: return launch_mx_v<HBQ_KIND_MXFP, 2>(a, kv, stream);
                    case 3: return launch_mx_v<HBQ_KIND_MXFP, 3>(a, kv, stream);
                    default: return launch_mx_v<HBQ_KIND_MXFP, 5>(a, kv, stream);
                }
            }
            int rc = HBQ_OK;
            switch (fast_mb) {
                case 1: rc = launch_mx_fast<HBQ_KIND_MXFP, 1>(a, grid, block, stream); break;
                case 2: rc = launch_mx_fast<HBQ_KIND_MXFP, 2>(a, grid, block, stream); break;
                case 3: rc = launch_mx_fast<HBQ_KIND_MXFP, 3>(a, grid, block, stream); break;
                default: rc = launch_mx_fast<HBQ_KIND_MXFP, 5>(a, grid, block, stream); break;
            }
            if (rc) return rc;
            HBQ_LAUNCH_CHECK("mx_fast_kernel<mxfp>");
            return HBQ_OK;
        }
        if (kv && kv->v_axis) return HBQ_ERR_UNSUPPORTED;
        switch (fast_mb) {
            case 1: mx_quantize_kernel<HBQ_KIND_MXFP, 1><<<grid, block, 0, stream>>>(a); break;
            case 2: mx_quantize_kernel<HBQ_KIND_MXFP, 2><<<grid, block, 0, stream>>>(a); break;
            case 3: mx_quantize_kernel<HBQ_KIND_MXFP, 3><<<grid, block, 0, stream>>>(a); break;
            case 5: mx_quantize_kernel<HBQ_KIND_MXFP, 5><<<grid, block, 0, stream>>>(a); break;
            default: mx_quantize_kernel<HBQ_KIND_MXFP, -1><<<grid, block, 0, stream>>>(a); break;
        }
        HBQ_LAUNCH_CHECK("mx_quantize_kernel<mxfp>");
        return HBQ_OK;
    }
    if (f->kind != HBQ_KIND_HBQ) return HBQ_ERR_ARG;
    // HBQ
    const int L = f->l2_block_size;
    if (fast_mb < 0 || fast_mb == 5) return HBQ_ERR_UNSUPPORTED;          // element must be E2M1/2/3
    if (f->sc_mbit == 0) return HBQ_ERR_UNSUPPORTED;
    if (!is_pow2(L) || L < 4 || L > B || f->l2_sc_bit < 0 || f->l2_sc_bit > 4) return HBQ_ERR_UNSUPPORTED;
    a.nc = 1 << f->l2_sc_bit;
    a.nscheme = l2_tables(f->l2_scheme, f->l2_sc_bit, a.tab);
    if (a.nscheme < 0) return HBQ_ERR_ARG;
    for (int s = 0; s < a.nscheme; ++s) {
        float tmax = a.tab[s][0];
        for (int i = 0; i < a.nc; ++i) {
            a.inv_tab[s][i] = 1.f / a.tab[s][i];
            tmax = fmaxf(tmax, a.tab[s][i]);
        }
        a.ele_max[s] = h_rh(h_rh(a.elem_max) * tmax);                   // quantizer.py:775-777
    }
    if (a.out.l2_packed) {
        const int tb = (B / L) * f->l2_sc_bit;
        if (tb != 8 && tb != 16 && tb != 32) return HBQ_ERR_UNSUPPORTED;
    }
    if (kv && kv->v_axis)
        return hbq_lut_v_launch(a, fast_mb, x, deq, a.in_bf16, a.out_bf16, kv->B, kv->T, kv->H, kv->D, kv->v_out_token_major, stream);
    {
        bool launched = false;
        int rc = hbq_tab_try_launch(a, fast_mb, stream, &launched);          // byte-table kernels (quantize_tab.cu)
        if (rc != HBQ_OK || launched) return rc;
        rc = hbq_lut_try_launch(a, fast_mb, stream, &launched);
        if (rc != HBQ_OK || launched) return rc;
    }
    if (a.glu_gate) return HBQ_ERR_UNSUPPORTED;
    switch (fast_mb) {
        case 1: hbq_quantize_kernel<1><<<grid, block, 0, stream>>>(a); break;
        case 2: hbq_quantize_kernel<2><<<grid, block, 0, stream>>>(a); break;
        default: hbq_quantize_kernel<3><<<grid, block, 0, stream>>>(a); break;
    }
    HBQ_LAUNCH_CHECK("hbq_quantize_kernel");
    return HBQ_OK;
}

int fp_quant_launch(const void* x, int64_t n, int ebit, int mbit, int allow_sub, int use_ceil,
                    int elem_variant, void* out, cudaStream_t stream)
{
    if (!x || !out || n < 0 || ebit < 1 || ebit > 5 || mbit < 0 || mbit > 9) return HBQ_ERR_ARG;
    if (n == 0) return HBQ_OK;
    const int64_t pairs = (n + 1) / 2;
    fp_quant_kernel<<<(unsigned)((pairs + 255) / 256), 256, 0, stream>>>(
        (const uint16_t*)x, n, ebit, mbit, allow_sub, use_ceil, elem_variant, (uint16_t*)out);
    HBQ_LAUNCH_CHECK("fp_quant_kernel");
    return HBQ_OK;
}

int64_t absmax_scratch_bytes() { return (int64_t)kAbsmaxBlocks * sizeof(float); }

int absmax_launch(const void* x, int dtype, int64_t n, float* amax, void* scratch, cudaStream_t stream)
{
    if (!x || !amax || !scratch || n < 0) return HBQ_ERR_ARG;
    if (dtype != HBQ_DTYPE_F16 && dtype != HBQ_DTYPE_BF16) return HBQ_ERR_UNSUPPORTED;
    absmax_partial_kernel<<<kAbsmaxBlocks, kAbsmaxThreads, 0, stream>>>(
        (const uint16_t*)x, n, dtype == HBQ_DTYPE_BF16, (float*)scratch);
    HBQ_LAUNCH_CHECK("absmax_partial_kernel");
    absmax_final_kernel<<<1, kAbsmaxThreads, 0, stream>>>((const float*)scratch, kAbsmaxBlocks,
                                                          dtype == HBQ_DTYPE_BF16, amax);
    HBQ_LAUNCH_CHECK("absmax_final_kernel");
    return HBQ_OK;
}

}  // namespace hbq
