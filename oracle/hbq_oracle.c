/*
 * CPU oracle for the HBQ hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * See hbq_oracle.h for the rules on who may use it and how its parity is pinned.
 *
 * The reference runs its quantizers as eager torch ops on fp16 tensors: every
 * elementwise op computes in fp32 and rounds its result to fp16, reductions
 * accumulate in fp32 and round once.  rh() below is that per-op rounding; each
 * statement that ends in rh() corresponds to one torch op of the reference.
 */
#include "hbq_oracle.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 f16;

static inline float h2f(uint16_t b) { f16 h; memcpy(&h, &b, 2); return (float)h; }
static inline uint16_t f2h(float f) { f16 h = (f16)f; uint16_t b; memcpy(&b, &h, 2); return b; }
static inline float rh(float f) { return (float)(f16)f; }
static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }
static inline float sgnf(float x) { return x > 0.f ? 1.f : (x < 0.f ? -1.f : 0.f); }

/* The literal 0.5004 of quantizer.py:229 as the fp16 add sees it: torch casts the
 * Python scalar to the tensor dtype first, i.e. to 0.50048828125. */
#define MANT_ROUND_CONST 0.50048828125f

/* get_max_norm / get_min_norm / get_min_subnorm, quantizer.py:148-185 */
static double max_norm(int ebit, int mbit, int uns) {
    if (ebit == 0) return uns ? ldexp(1.0, mbit) - 1 : ldexp(1.0, mbit - 1) - 1;
    if (ebit == 4 && mbit == 3) return 448.0;
    int emax = (ebit == 5) ? 15 : (1 << (ebit - 1));
    return ldexp(1.0, emax) * (ldexp(1.0, mbit + 1) - 1) / ldexp(1.0, mbit);
}
static double min_norm(int ebit, int mbit) {
    (void)mbit;
    if (ebit == 0) return 0.0;
    if (ebit == 1) return 1.0;
    return ldexp(1.0, 2 - (1 << (ebit - 1)));
}
static double min_subnorm(int ebit, int mbit) { return ldexp(1.0, 2 - (1 << (ebit - 1)) - mbit); }

/* floor(log2(t)) on an fp16 tensor: log2 computed in fp32, rounded to fp16, then floored. */
static inline float floor_log2_h(float t) { return floorf(rh(log2f(t))); }

/* make_fp_quant closure (quantizer.py:202-255, elem_variant=1) and the free
 * function fp_quant (quantizer.py:259-328, elem_variant=0).  x is an fp16 value. */
static float fpq_chain(float x, int ebit, int mbit, int allow_sub, int use_ceil,
                       int elem_variant, int* exp_field, int* mant_field)
{
    const int emax = (ebit == 5) ? 15 : (1 << (ebit - 1));
    const int emin = 2 - (1 << (ebit - 1));
    const float mn = (float)min_norm(ebit, mbit);
    const float thr = mn - ldexpf(1.f, -(mbit + 1) + emin);
    const float mant_shift = ldexpf(1.f, mbit);
    const float mant_max = mant_shift - 1.f;

    const float ax = fabsf(x);
    const int is_zero = (x == 0.f);
    const int promote = (ax < mn) && (ax >= thr);
    const int below = (ax < thr) && !is_zero;
    const int sub = allow_sub ? below : 0;
    const int under = allow_sub ? 0 : below;

    float e = clampf(floor_log2_h(rh(ax + (is_zero ? 1.f : 0.f))), (float)emin, (float)emax);
    const float p2 = rh(exp2f(e));
    const float sg = sgnf(x);
    float mant = sub ? rh(rh(x / p2) * mant_shift) : rh(rh(rh(x / p2) - sg) * mant_shift);
    float am = fabsf(mant), mr;
    if (use_ceil) mr = ceilf(am);
    else if (elem_variant) mr = floorf(rh(am + MANT_ROUND_CONST));
    else mr = floorf(rh(am + 0.5f));
    const int overflow = (mr > mant_max) && (e != (float)emax);
    if (mr > mant_max) mr = mant_max;
    if (is_zero || under || overflow || promote) mr = 0.f;
    if (overflow) e += 1.f;
    const float sm = sg * mr;
    const float p2b = rh(exp2f(e));
    float xq = sub ? rh(rh(sm / mant_shift) * p2b) : rh(rh(rh(sm / mant_shift) + sg) * p2b);
    if (is_zero || under) xq = 0.f;
    if (ebit == 4 && mbit == 3) xq = clampf(xq, -448.f, 448.f);
    if (exp_field) {
        int ef = (int)e + ((1 << (ebit - 1)) - 1);
        if (is_zero || under || sub) ef = 0;
        *exp_field = ef;
        *mant_field = (int)mr;
    }
    return xq;
}

void orc_fp_quant(const uint16_t* x, int64_t n, int ebit, int mbit, int allow_subnormal,
                  int use_ceil, int elem_variant, uint16_t* out)
{
    for (int64_t i = 0; i < n; ++i)
        out[i] = f2h(fpq_chain(h2f(x[i]), ebit, mbit, allow_subnormal, use_ceil, elem_variant, 0, 0));
}

void orc_floor_log2_h(const uint16_t* x, int64_t n, float* out)
{
    for (int64_t i = 0; i < n; ++i) out[i] = floor_log2_h(h2f(x[i]));
}

/* FP shared scale: clip then fp_quant (HBQQuantizer.quant_scale quantizer.py:735-739;
 * MXFPQuantizer.get_shared_scale quantizer.py:504-509). */
static float quant_scale_clip_first(float s, const orc_format* f)
{
    float lo = (float)(f->scale_allow_subnormal ? min_subnorm(f->sc_ebit, f->sc_mbit)
                                                : min_norm(f->sc_ebit, f->sc_mbit));
    float hi = (float)max_norm(f->sc_ebit, f->sc_mbit, 0);
    s = clampf(s, lo, hi);
    return fpq_chain(s, f->sc_ebit, f->sc_mbit, f->scale_allow_subnormal, f->use_ceil, 0, 0, 0);
}

/* Power-of-two shared exponent: floor|round(log2(max + min_normal*[max==0])) in fp16
 * (quantizer.py:395-407, 491-503).  torch.round is round-half-to-even. */
static float pot_exp(float amax, int use_round)
{
    float t = rh(amax + rh(6.103515625e-05f * (amax == 0.f ? 1.f : 0.f)));
    float l = rh(log2f(t));
    return use_round ? nearbyintf(l) : floorf(l);
}

static inline uint8_t fp_code(float x, int ef, int mf, int ebit, int mbit)
{
    return (uint8_t)(((x < 0.f ? 1 : 0) << (ebit + mbit)) | (ef << mbit) | mf);
}

static void l2_table(int scheme, int bits, float* t /* [2][16] */, int* nscheme)
{
    int n = 1 << bits;
    *nscheme = 1;
    for (int i = 0; i < n; ++i) {
        float r = (float)i;
        float pot = rh(exp2f(r)), in = rh(r + 1.f), sig1 = rh(1.f + rh(r / 2.f));
        float fp = rh(1.f + rh(r / (float)(1 << bits)));
        float fp1 = rh(1.f + rh(rh(r + 1.f) / (float)(1 << bits)));
        float fp10 = rh(1.f + rh(r / (float)(1 << (bits + 1))));
        float fp100 = rh(1.f + rh(r / (float)(1 << (bits + 2))));
        switch (scheme) {
            case ORC_L2_POT: t[i] = pot; break;
            case ORC_L2_INT: t[i] = in; break;
            case ORC_L2_SIG1: t[i] = sig1; break;
            case ORC_L2_FPM1: t[i] = fp; break;
            case ORC_L2_FP1: t[i] = fp1; break;
            case ORC_L2_FPM10: t[i] = fp10; break;
            case ORC_L2_FPM100: t[i] = fp100; break;
            case ORC_L2_MIX: t[i] = fp; t[16 + i] = fp10; *nscheme = 2; break;
        }
    }
}

/* One block of MXFPQuantizer.q (quantizer.py:513-539) without the per-tensor scale. */
static void mxfp_block(const float* x, int B, const orc_format* f, float* deq, float* scale_out,
                       uint8_t* codes)
{
    float amax = 0.f;
    for (int j = 0; j < B; ++j) amax = fmaxf(amax, fabsf(x[j]));
    float s;
    if (f->sc_mbit == 0) {
        float e = pot_exp(amax, f->use_round) - (float)(1 << (f->ebit - 1));
        e = clampf(e, (float)(2 - (1 << (f->sc_ebit - 1))), (float)((1 << (f->sc_ebit - 1)) - 1));
        s = rh(exp2f(e));
    } else {
        s = rh(amax / (float)max_norm(f->ebit, f->mbit, 0));
        s = quant_scale_clip_first(s, f);
    }
    for (int j = 0; j < B; ++j) {
        int ef, mf;
        float y = rh(x[j] / s);
        float q = fpq_chain(y, f->ebit, f->mbit, 1, 0, 1, &ef, &mf);
        deq[j] = rh(q * s);
        if (codes) codes[j] = fp_code(y, ef, mf, f->ebit, f->mbit);
    }
    *scale_out = s;
}

/* One block of MXINTQuantizer.q (quantizer.py:385-428). */
static void mxint_block(const float* x, int B, const orc_format* f, float* deq, float* scale_out,
                        uint8_t* codes)
{
    const int nbit = f->mbit;
    float amax = 0.f;
    for (int j = 0; j < B; ++j) amax = fmaxf(amax, fabsf(x[j]));
    float s;
    if (f->sc_mbit == 0) {
        float e = clampf(rh(pot_exp(amax, 0) - (float)(nbit - 2)), -14.f, 15.f);
        s = rh(exp2f(e));
    } else {
        s = rh(amax / (float)max_norm(0, nbit, 0));
        s = fpq_chain(s, f->sc_ebit, f->sc_mbit, f->scale_allow_subnormal, f->use_ceil, 0, 0, 0);
        float lo = (float)(f->scale_allow_subnormal ? min_subnorm(f->sc_ebit, f->sc_mbit)
                                                    : min_norm(f->sc_ebit, f->sc_mbit));
        if (s < lo) s = lo;
    }
    const float qmin = -ldexpf(1.f, nbit - 1), qmax = ldexpf(1.f, nbit - 1) - 1.f;
    for (int j = 0; j < B; ++j) {
        float y = rh(x[j] / s);
        float q = rh(sgnf(y) * floorf(rh(fabsf(y) + 0.5f)));
        q = clampf(q, qmin, qmax);
        deq[j] = rh(q * s);
        if (codes) codes[j] = (uint8_t)(int8_t)q;
    }
    *scale_out = s;
}

/* One block of HBQQuantizer.q (quantizer.py:741-859). */
static void hbq_block(const float* x, int B, const orc_format* f, const float* tab, int nscheme,
                      float* deq, float* scale_out, uint8_t* l2idx, uint8_t* scheme_out,
                      uint8_t* codes)
{
    const int L = f->l2_block_size, nl2 = B / L, nc = 1 << f->l2_sc_bit;
    float amax = 0.f;
    for (int j = 0; j < B; ++j) amax = fmaxf(amax, fabsf(x[j]));
    const float em = (float)max_norm(f->ebit, f->mbit, 0);

    float best_err = 0.f; int best_s = -1;
    float l1s[2]; uint8_t idxs[2][128];
    for (int s = 0; s < nscheme; ++s) {
        const float* t = tab + 16 * s;
        float tmax = t[0];
        for (int i = 1; i < nc; ++i) tmax = fmaxf(tmax, t[i]);
        const float ele_max = rh(rh(em) * tmax);                 /* quantizer.py:775-777 */
        float l1 = quant_scale_clip_first(rh(amax / ele_max), f); /* :778-779 */
        l1s[s] = l1;
        float tot = 0.f;                                           /* fp32 accumulate, :814 */
        for (int u = 0; u < nl2; ++u) {
            float bestE = 0.f; int bi = -1;
            float e[16][128];
            for (int i = 0; i < nc; ++i) {
                float acc = 0.f;                                   /* fp32 accumulate, :802 */
                for (int j = 0; j < L; ++j) {
                    float xv = x[u * L + j];
                    float a = rh(xv / l1);                         /* :781 */
                    float b = rh(a / t[i]);                        /* :789 */
                    float c = fpq_chain(b, f->ebit, f->mbit, 1, 0, 1, 0, 0); /* :790 */
                    float d = rh(rh(c * t[i]) * l1);               /* :791, :796 */
                    float r = fabsf(rh(xv - d));
                    e[i][j] = rh(r * r);
                    acc += e[i][j];
                }
                float E = rh(acc);
                if (bi < 0 || E < bestE) { bestE = E; bi = i; }   /* first index wins ties, :803 */
            }
            idxs[s][u] = (uint8_t)bi;
            /* :814 sums the selected candidates' per-element errors over the whole block. */
            for (int j = 0; j < L; ++j) tot += e[bi][j];
        }
        float Es = rh(tot);
        if (best_s < 0 || Es < best_err) { best_err = Es; best_s = s; }
    }
    const float* t = tab + 16 * best_s;
    const float l1 = l1s[best_s];
    for (int u = 0; u < nl2; ++u) {
        int bi = idxs[best_s][u];
        if (l2idx) l2idx[u] = (uint8_t)bi;
        for (int j = 0; j < L; ++j) {
            float xv = x[u * L + j];
            int ef, mf;
            float a = rh(xv / l1), b = rh(a / t[bi]);
            float c = fpq_chain(b, f->ebit, f->mbit, 1, 0, 1, &ef, &mf);
            deq[u * L + j] = rh(rh(c * t[bi]) * l1);
            if (codes) codes[u * L + j] = fp_code(b, ef, mf, f->ebit, f->mbit);
        }
    }
    *scale_out = l1;
    if (scheme_out) *scheme_out = (uint8_t)best_s;
}

/* sign(v) * floor(|v| + 0.5) on an fp16 tensor, then clip (quantizer.py:421-422, 603-604, 691-692). */
static inline float round_half_away_clip(float v, float lo, float hi)
{
    return clampf(rh(sgnf(v) * floorf(rh(fabsf(v) + 0.5f))), lo, hi);
}

/* One block of MXExQuantizer.q (quantizer.py:576-628): power-of-two shared scale, and per
 * micro-block of l2_block_size elements the better (smaller squared error, ties: unshifted) of an
 * integer grid with step 1 and one with step 2.  Format fields: mbit = element bits, sc_ebit =
 * sc_bit (scale exponent width), l2_sc_bit, l2_block_size.  l2idx: 1 where the step-2 grid won. */
static void mxex_block(const float* x, int B, const orc_format* f, float* deq, float* scale_out, uint8_t* l2idx)
{
    float amax = 0.f;
    for (int j = 0; j < B; ++j) amax = fmaxf(amax, fabsf(x[j]));
    const float emax = ldexpf(1.f, f->sc_ebit - 1) - 1.f;
    float e = rh(rh(pot_exp(amax, 0) - (float)(f->mbit - 2)) - (float)f->l2_sc_bit);       /* :588-593 */
    e = clampf(e, -emax, emax);
    const float s = rh(exp2f(e));                                                            /* :594 */
    const float qmin = -ldexpf(1.f, f->mbit - 1), qmax = ldexpf(1.f, f->mbit - 1) - 1.f;
    const int L = f->l2_block_size;
    for (int u = 0; u < B / L; ++u) {
        float y[64], q2[64], q1[64], e2 = 0.f, e1 = 0.f;
        for (int j = 0; j < L; ++j) {
            y[j] = rh(x[u * L + j] / s);                                                     /* :601 */
            q2[j] = rh(round_half_away_clip(rh(y[j] / 2.f), qmin, qmax) * 2.f);              /* :605-608 */
            const float d2 = fabsf(rh(q2[j] - y[j]));
            e2 += rh(d2 * d2);                                                               /* :609 */
            q1[j] = round_half_away_clip(y[j], qmin, qmax);                                  /* :612-614 */
            const float d1 = fabsf(rh(q1[j] - y[j]));
            e1 += rh(d1 * d1);                                                               /* :615 */
        }
        const int shift = rh(e2) < rh(e1);                                                   /* :617 */
        for (int j = 0; j < L; ++j) deq[u * L + j] = rh((shift ? q2[j] : q1[j]) * s);        /* :618-621 */
        if (l2idx) l2idx[u] = (uint8_t)shift;
    }
    *scale_out = s;
}

/* One row of VSQQuantizer.q (quantizer.py:668-701): per-vector scale max/qmax, quantised to
 * sc_mbit unsigned bits against a per-row first-level scale; the elements are quantised with the
 * unquantised vector scale and dequantised with l1 * l2.  Format fields: mbit = nbit, sc_mbit.
 * xr: the row zero padded to nblk * B values. */
static void vsq_row(const float* xr, int64_t nblk, int B, const orc_format* f, float* dr, float* l1_out,
                    uint8_t* l2_out)
{
    const float qmaxe = ldexpf(1.f, f->mbit - 1) - 1.f, qmine = -ldexpf(1.f, f->mbit - 1);
    const float smax_u = ldexpf(1.f, f->sc_mbit) - 1.f;
    float max_scale = 0.f;
    for (int64_t kb = 0; kb < nblk; ++kb) {
        float amax = 0.f;
        for (int j = 0; j < B; ++j) amax = fmaxf(amax, fabsf(xr[kb * B + j]));
        max_scale = fmaxf(max_scale, rh(amax / qmaxe));                                      /* :673-674 */
    }
    const float l1 = rh(max_scale / smax_u);                                                 /* :675 */
    const float safe_l1 = l1 == 0.f ? 1.f : l1;
    for (int64_t kb = 0; kb < nblk; ++kb) {
        float amax = 0.f;
        for (int j = 0; j < B; ++j) amax = fmaxf(amax, fabsf(xr[kb * B + j]));
        const float sh = rh(amax / qmaxe);
        const float l2 = round_half_away_clip(rh(sh / safe_l1), 0.f, smax_u);                /* :677-679 */
        const float safe_sh = sh == 0.f ? 1.f : sh;
        for (int j = 0; j < B; ++j) {
            const float q = round_half_away_clip(rh(xr[kb * B + j] / safe_sh), qmine, qmaxe); /* :682-685 */
            dr[kb * B + j] = rh(rh(q * l1) * l2);                                            /* :688 */
        }
        if (l2_out) l2_out[kb] = (uint8_t)l2;
    }
    *l1_out = l1;
}

int orc_quantize(const uint16_t* x, int64_t rows, int64_t K, const orc_format* f,
                 uint16_t* deq, uint16_t* scale, uint8_t* l2idx, uint8_t* scheme, uint8_t* codes)
{
    if (f->kind == ORC_KIND_VSQ) {
        /* scale: the per-row first-level scale in every block slot; l2idx: one l2 value per block */
        const int Bv = f->block_size;
        if (Bv <= 0 || Bv > 1024 || f->mbit < 2 || f->mbit > 8 || f->sc_mbit < 1 || f->sc_mbit > 8) return -1;
        const int64_t nb = (K + Bv - 1) / Bv;
        #pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            float* xr = (float*)malloc(sizeof(float) * (size_t)(nb * Bv) * 2);
            float* dr = xr + nb * Bv;
            uint8_t* l2r = (uint8_t*)malloc((size_t)nb);
            for (int64_t k = 0; k < nb * Bv; ++k) xr[k] = k < K ? h2f(x[r * K + k]) : 0.f;
            float l1;
            vsq_row(xr, nb, Bv, f, dr, &l1, l2r);
            for (int64_t k = 0; k < K; ++k) deq[r * K + k] = f2h(dr[k]);
            for (int64_t kb = 0; kb < nb; ++kb) {
                if (scale) scale[r * nb + kb] = f2h(l1);
                if (l2idx) l2idx[r * nb + kb] = l2r[kb];
            }
            free(xr); free(l2r);
        }
        return 0;
    }
    if (f->kind == ORC_KIND_MXEX && (f->l2_block_size <= 0 || f->l2_block_size > 64 || f->block_size / f->l2_block_size > 128 || f->block_size % f->l2_block_size != 0 ||
                                     f->mbit < 2 || f->mbit > 8)) return -1;
    const int B = f->block_size;
    if (B <= 0 || B > 1024) return -1;
    if (f->kind == ORC_KIND_HBQ && (B % f->l2_block_size != 0 || B / f->l2_block_size > 128 ||
                                    f->l2_sc_bit > 4 || f->l2_sc_bit < 0)) return -1;
    /* per-tensor scale, MXFPQuantizer.q quantizer.py:516-524 and :534-535: the fp16 tensor is
     * divided / multiplied by a Python double, which torch evaluates in fp32 with float(scale). */
    float tsf = 1.f;
    const int pts = (f->kind == ORC_KIND_MXFP && f->per_tensor_scale);
    if (pts) {
        float tmax = 0.f;
        for (int64_t i = 0; i < rows * K; ++i) tmax = fmaxf(tmax, fabsf(h2f(x[i])));
        if (tmax != 0.f)
            tsf = (float)((double)tmax / (max_norm(f->ebit, f->mbit, 0) * max_norm(f->sc_ebit, f->sc_mbit, 0)));
    }
    const int64_t nblk = (K + B - 1) / B;
    float tab[32]; int nscheme = 1;
    int nl2 = 0;
    if (f->kind == ORC_KIND_HBQ) { l2_table(f->l2_scheme, f->l2_sc_bit, tab, &nscheme); nl2 = B / f->l2_block_size; }
    if (f->kind == ORC_KIND_MXEX) nl2 = B / f->l2_block_size;

    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float xb[1024], db[1024]; uint8_t cb[1024]; uint8_t ib[128];
        for (int64_t kb = 0; kb < nblk; ++kb) {
            const int64_t k0 = kb * B;
            const int valid = (int)((K - k0) < B ? (K - k0) : B);
            for (int j = 0; j < B; ++j) xb[j] = j < valid ? h2f(x[r * K + k0 + j]) : 0.f;
            if (pts) for (int j = 0; j < B; ++j) xb[j] = rh(xb[j] / tsf);
            float s; uint8_t sch = 0;
            if (f->kind == ORC_KIND_MXFP) mxfp_block(xb, B, f, db, &s, cb);
            else if (f->kind == ORC_KIND_MXINT) mxint_block(xb, B, f, db, &s, cb);
            else if (f->kind == ORC_KIND_MXEX) mxex_block(xb, B, f, db, &s, ib);
            else hbq_block(xb, B, f, tab, nscheme, db, &s, ib, &sch, cb);
            if (pts) for (int j = 0; j < B; ++j) db[j] = rh(db[j] * tsf);
            for (int j = 0; j < valid; ++j) deq[r * K + k0 + j] = f2h(db[j]);
            if (scale) scale[r * nblk + kb] = f2h(s);
            if (codes && f->kind != ORC_KIND_MXEX) memcpy(codes + (r * nblk + kb) * B, cb, (size_t)B);
            if (f->kind == ORC_KIND_MXEX && l2idx) memcpy(l2idx + (r * nblk + kb) * nl2, ib, (size_t)nl2);
            if (f->kind == ORC_KIND_HBQ) {
                if (l2idx) memcpy(l2idx + (r * nblk + kb) * nl2, ib, (size_t)nl2);
                if (scheme) scheme[r * nblk + kb] = sch;
            }
        }
    }
    return 0;
}

/* ---------------------------------------------------------------------------------
 * GEMM accumulation models (gemm.cu).  Products of two fp16 values are exact in fp32.
 * --------------------------------------------------------------------------------- */

/* compute_scale_pow2_int8, gemm.cu:1145-1152 */
static inline float scale_pow2(float max_abs, int shift)
{
    if (!(max_abs > 0.f)) return 1.f;
    return ldexpf(1.f, ilogbf(max_abs) - shift);
}

/* e3m4_quantize_dequant, gemm.cu:677-737 (exact arithmetic; the reference build's
 * fast-math approximations are not modelled). */
static float e3m4_qdq(float x, float scale)
{
    float sg = copysignf(1.f, x), a = fabsf(x);
    if (a == 0.f) return copysignf(0.f, x);
    float y = a / scale;
    if (!isfinite(y)) return isnan(y) ? copysignf(NAN, x) : sg * 15.5f * scale;
    if (y < 0.5f * 0.015625f) return 0.f;
    if (y >= 0.25f) {
        int e = (int)floorf(log2f(y));
        if (e < -2) e = -2;
        if (e > 3) e = 3;
        float p = ldexpf(1.f, e);
        float m = nearbyintf((y / p - 1.f) * 16.f);
        if (m >= 16.f) { m = 0.f; ++e; if (e > 3) { e = 3; m = 15.f; } p = ldexpf(1.f, e); }
        float yq = (1.f + m * (1.f / 16.f)) * p;
        if (yq > 15.5f) yq = 15.5f;
        return sg * yq * scale;
    }
    float m = nearbyintf(y * 64.f);
    if (m <= 0.f) return 0.f;
    if (m >= 16.f) return sg * 0.25f * scale;
    return sg * (m * (1.f / 16.f)) * 0.25f * scale;
}

int orc_gemm_rows(const uint16_t* A, const uint16_t* B, uint16_t* C, int64_t M, int64_t N,
                  int64_t K, int mode, int group_k, int group_n, int64_t m0, int64_t m1)
{
    if (mode < 0 || mode > 4) return -1;
    if (mode >= ORC_ACC_GROUPED && group_k <= 0) return -1;
    if (mode >= ORC_ACC_PSUM_INT8 && group_n <= 0) return -1;
    if (m0 < 0) m0 = 0;
    if (m1 > M) m1 = M;
    /* fp32 copy of B once: the inner loops stream rows of B. */
    float* Bf = (float*)malloc(sizeof(float) * (size_t)K * (size_t)N);
    if (!Bf) return -3;
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < K * N; ++i) Bf[i] = h2f(B[i]);

    #pragma omp parallel
    {
        float* g = (float*)malloc(sizeof(float) * (size_t)N);     /* in-group fp32 sums */
        f16* acc = (f16*)malloc(sizeof(f16) * (size_t)N);         /* fp16 running sums */
        double* accd = (double*)malloc(sizeof(double) * (size_t)N);
        #pragma omp for schedule(dynamic, 4)
        for (int64_t m = m0; m < m1; ++m) {
            for (int64_t n = 0; n < N; ++n) { g[n] = 0.f; acc[n] = (f16)0.f; }
            int cnt = 0;
            for (int64_t k = 0; k < K; ++k) {
                const float a = h2f(A[m * K + k]);
                const float* b = Bf + k * N;
                if (mode == ORC_ACC_FP16) {
                    /* __hfma2 chain, gemm.cu:208-217: one rounding per k */
                    for (int64_t n = 0; n < N; ++n) {
                        accd[n] = (double)a * (double)b[n] + (double)(float)acc[n];
                        acc[n] = (f16)accd[n];
                    }
                    continue;
                }
                for (int64_t n = 0; n < N; ++n) g[n] = fmaf(a, b[n], g[n]);
                if (mode == ORC_ACC_FP32) continue;
                if (++cnt == group_k || k + 1 == K) {
                    cnt = 0;
                    if (mode == ORC_ACC_PSUM_INT8 || mode == ORC_ACC_PSUM_E3M4) {
                        for (int64_t n0 = 0; n0 < N; n0 += group_n) {
                            int64_t n1 = n0 + group_n < N ? n0 + group_n : N;
                            float mx = 0.f;
                            for (int64_t n = n0; n < n1; ++n) { float av = fabsf(g[n]); if (av > mx) mx = av; }
                            if (mode == ORC_ACC_PSUM_INT8) {
                                float sc = scale_pow2(mx, 6), inv = 1.f / sc;
                                for (int64_t n = n0; n < n1; ++n) {
                                    float v = g[n] * inv;
                                    if (!isfinite(v)) { if (isnan(v)) { g[n] = NAN; continue; } v = copysignf(127.f, v); }
                                    float q = nearbyintf(v);
                                    if (q > 127.f) q = 127.f;
                                    if (q < -127.f) q = -127.f;
                                    g[n] = q * sc;
                                }
                            } else {
                                float sc = scale_pow2(mx, 3);
                                for (int64_t n = n0; n < n1; ++n) g[n] = e3m4_qdq(g[n], sc);
                            }
                        }
                    }
                    for (int64_t n = 0; n < N; ++n) {
                        f16 p = (f16)g[n];
                        acc[n] = (f16)((double)acc[n] + (double)p); /* __hadd */
                        g[n] = 0.f;
                    }
                }
            }
            for (int64_t n = 0; n < N; ++n)
                C[m * N + n] = (mode == ORC_ACC_FP32) ? f2h(g[n]) : f2h((float)acc[n]);
        }
        free(g); free(acc); free(accd);
    }
    free(Bf);
    return 0;
}

int orc_gemm(const uint16_t* A, const uint16_t* B, uint16_t* C, int64_t M, int64_t N,
             int64_t K, int mode, int group_k, int group_n)
{
    return orc_gemm_rows(A, B, C, M, N, K, mode, group_k, group_n, 0, M);
}

void orc_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
