// MXExQuantizer and VSQQuantizer (src/quantizer.py:541-702): the two quantizer classes of the
// reference that no shipped configuration selects.  Plain kernels (one thread per 8 consecutive
// elements, fp32 arithmetic with the reference's fp16 rounding after every tensor op); they exist for
// interface completeness, not for speed.
#include "quantize_dev.cuh"
#include <math.h>
#include <string.h>

namespace hbq {

// sign(v) * floor(|v| + 0.5) on an fp16 tensor, then clip (src/quantizer.py:603-604, 613-614, 691-692)
__device__ __forceinline__ float round_away_clip(float v, float lo, float hi)
{
    const float s = v > 0.f ? 1.f : (v < 0.f ? -1.f : 0.f);
    return fminf(fmaxf(rh(s * floorf(rh(fabsf(v) + 0.5f))), lo), hi);
}

struct ExArgs {
    QArgs q;
    int mbit, sc_bit, l2_sc_bit, L;      // MXEx
    int sc_mbit;                         // VSQ
};

// ---- MXEx ------------------------------------------------------------------------------------------
// Power-of-two shared scale 2^clip(floor(log2 max) - (mbit-2) - l2_sc_bit); per micro-block of L
// elements the better of an integer grid with step 1 and one with step 2 (smaller fp16 squared
// error, ties keep step 1).
__global__ void __launch_bounds__(256) mxex_kernel(const ExArgs a)
{
    const QArgs& q = a.q;
    const int64_t ci = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool valid = ci < q.total_chunks;
    int64_t row = 0, c = 0;
    if (valid) split_chunk(q, ci, row, c);
    const int64_t k0 = c * 8;
    Chunk x;
    if (valid) x = load_chunk(q, row, k0);
    else { for (int p = 0; p < 4; ++p) x.h[p] = bits_h2(0u); }
    float v[8];
    #pragma unroll
    for (int p = 0; p < 4; ++p) { const float2 f = __half22float2(x.h[p]); v[2 * p] = f.x; v[2 * p + 1] = f.y; }

    const float amax = group_max(chunk_absmax(x), q.G);
    const float t = rh(amax + rh(6.103515625e-05f * (amax == 0.f ? 1.f : 0.f)));     // :586-590
    const float emax = ldexpf(1.f, a.sc_bit - 1) - 1.f;
    float e = rh(rh(floorf(rh(log2f(t))) - (float)(a.mbit - 2)) - (float)a.l2_sc_bit);
    e = fminf(fmaxf(e, -emax), emax);                                                  // :593
    const float s = rh(exp2f(e));                                                      // :594
    const float qmin = -ldexpf(1.f, a.mbit - 1), qmax = ldexpf(1.f, a.mbit - 1) - 1.f;

    float y[8], q1[8], q2[8], e1[8], e2[8];
    #pragma unroll
    for (int j = 0; j < 8; ++j) {
        y[j] = rh(__fdiv_rn(v[j], s));                                                 // :601
        q2[j] = rh(round_away_clip(rh(y[j] * 0.5f), qmin, qmax) * 2.f);                // :605-608
        const float d2 = rh(q2[j] - y[j]);
        e2[j] = rh(d2 * d2);
        q1[j] = round_away_clip(y[j], qmin, qmax);                                     // :612-614
        const float d1 = rh(q1[j] - y[j]);
        e1[j] = rh(d1 * d1);
    }
    float out[8];
    for (int u = 0; u < 8; u += a.L) {
        float s1 = 0.f, s2 = 0.f;                                                      // fp32 accumulate, one rounding
        for (int j = 0; j < a.L; ++j) { s1 += e1[u + j]; s2 += e2[u + j]; }
        const bool shift = rh(s2) < rh(s1);                                            // :617
        for (int j = 0; j < a.L; ++j) out[u + j] = shift ? q2[u + j] : q1[u + j];
    }
    if (!valid) return;
    __half2 d[4];
    #pragma unroll
    for (int p = 0; p < 4; ++p) d[p] = __floats2half2_rn(out[2 * p] * s, out[2 * p + 1] * s);   // :621
    store_deq(q, row, k0, d);
}

// ---- VSQ -------------------------------------------------------------------------------------------
// One CTA per row.  Pass 1: per-vector scale max/qmax of every block, row maximum -> first-level scale
// l1 = max / (2^sc_mbit - 1).  Pass 2: l2 = clip(round(scale / l1)), elements quantised with the
// unquantised vector scale and dequantised with l1 * l2.
__global__ void __launch_bounds__(256) vsq_kernel(const ExArgs a)
{
    const QArgs& q = a.q;
    __shared__ float s_red[8];
    const int64_t row = blockIdx.x;
    const float qmaxe = ldexpf(1.f, a.mbit - 1) - 1.f, qmine = -ldexpf(1.f, a.mbit - 1);
    const float smax_u = ldexpf(1.f, a.sc_mbit) - 1.f;
    const int64_t cpr_round = (q.cpr + 255) / 256 * 256;        // whole-CTA trips keep the shuffles converged

    float mymax = 0.f;
    for (int64_t c = threadIdx.x; c < cpr_round; c += 256) {
        Chunk x;
        if (c < q.cpr) x = load_chunk(q, row, c * 8);
        else { for (int p = 0; p < 4; ++p) x.h[p] = bits_h2(0u); }
        const float amax = group_max(chunk_absmax(x), q.G);
        mymax = fmaxf(mymax, rh(__fdiv_rn(amax, qmaxe)));                              // :673
    }
    mymax = group_max(mymax, 32);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = mymax;
    __syncthreads();
    float max_scale = s_red[0];
    #pragma unroll
    for (int i = 1; i < 8; ++i) max_scale = fmaxf(max_scale, s_red[i]);               // :674
    const float l1 = rh(__fdiv_rn(max_scale, smax_u));                                 // :675
    const float safe_l1 = l1 == 0.f ? 1.f : l1;

    for (int64_t c = threadIdx.x; c < cpr_round; c += 256) {
        const bool valid = c < q.cpr;
        Chunk x;
        if (valid) x = load_chunk(q, row, c * 8);
        else { for (int p = 0; p < 4; ++p) x.h[p] = bits_h2(0u); }
        const float amax = group_max(chunk_absmax(x), q.G);
        const float sh = rh(__fdiv_rn(amax, qmaxe));
        const float l2 = round_away_clip(rh(__fdiv_rn(sh, safe_l1)), 0.f, smax_u);     // :677-679
        const float safe_sh = sh == 0.f ? 1.f : sh;
        __half2 d[4];
        #pragma unroll
        for (int p = 0; p < 4; ++p) {
            const float2 f = __half22float2(x.h[p]);
            const float q0 = round_away_clip(rh(__fdiv_rn(f.x, safe_sh)), qmine, qmaxe);   // :682-685
            const float q1 = round_away_clip(rh(__fdiv_rn(f.y, safe_sh)), qmine, qmaxe);
            d[p] = __floats2half2_rn(rh(q0 * l1) * l2, rh(q1 * l1) * l2);                  // :688
        }
        if (valid) store_deq(q, row, c * 8, d);
    }
}

// ---- host side -------------------------------------------------------------------------------------
// hbq_format mapping: MXEx: mbit = element bits, sc_ebit = sc_bit, l2_sc_bit, l2_block_size;
// VSQ: mbit = nbit, sc_mbit.  `a` carries the tensor geometry as quantize_launch fills it.
int quantize_extra_launch(const QArgs& qa, cudaStream_t stream)
{
    const hbq_format& f = qa.f;
    ExArgs a;
    memset(&a, 0, sizeof(a));
    a.q = qa;
    if (!qa.deq) return HBQ_ERR_ARG;
    const bool side_out = qa.out.codes || qa.out.sign || qa.out.scale_u8 || qa.out.scale_h || qa.out.l2_packed ||
                          qa.out.l2_idx || qa.out.scheme;
    if (side_out || qa.rope_cos || qa.perm_T > 0 || qa.k_center) return HBQ_ERR_UNSUPPORTED;
    if (f.kind == HBQ_KIND_MXEX) {
        const int L = f.l2_block_size;
        if (f.mbit < 2 || f.mbit > 8 || f.sc_ebit < 2 || f.sc_ebit > 8 || f.l2_sc_bit < 0 || f.l2_sc_bit > 4) return HBQ_ERR_UNSUPPORTED;
        if (L < 1 || (L & (L - 1)) || L > 8) return HBQ_ERR_UNSUPPORTED;     // a micro-block stays inside one thread's 8 elements
        a.mbit = f.mbit; a.sc_bit = f.sc_ebit; a.l2_sc_bit = f.l2_sc_bit; a.L = L;
        mxex_kernel<<<(unsigned)((qa.total_chunks + 255) / 256), 256, 0, stream>>>(a);
        HBQ_LAUNCH_CHECK("mxex_kernel");
        return HBQ_OK;
    }
    if (f.kind == HBQ_KIND_VSQ) {
        if (f.mbit < 2 || f.mbit > 8 || f.sc_mbit < 1 || f.sc_mbit > 8) return HBQ_ERR_UNSUPPORTED;
        if (qa.rows > 0x7FFFFFFFll) return HBQ_ERR_UNSUPPORTED;
        a.mbit = f.mbit; a.sc_mbit = f.sc_mbit;
        vsq_kernel<<<(unsigned)qa.rows, 256, 0, stream>>>(a);
        HBQ_LAUNCH_CHECK("vsq_kernel");
        return HBQ_OK;
    }
    return HBQ_ERR_ARG;
}

}  // namespace hbq
