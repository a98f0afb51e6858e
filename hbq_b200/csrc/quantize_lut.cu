// HBQ activation quantize, table-driven variant (one scale scheme, up to 4 micro-scale candidates).
//
// The arithmetic variant in quantize.cu evaluates Q(fp16(a / t_i)) for every candidate t_i with
// ~20 instructions per element pair and is instruction-issue bound at ~10 % of HBM bandwidth.
// Here the observation is that, for a fixed format, fp16(Q(fp16(a / t_i)) * t_i) is a function of
// the fp16 pattern of |a| = |x / l1| alone, monotone (bar one E2M1 exception), and saturated
// above ~18.  Each CTA therefore builds, once, a shared-memory table indexed by that pattern
// holding the four candidates' values as fp16; the per-element work becomes one 8-byte shared
// load plus packed fp16 arithmetic in which the two halves of a half2 are two CANDIDATES:
//   r = fma(-value, l1, |x|)  (= fp16(|x| - fp16(value * l1)), the product is exact)
//   e = r * r                 (fp16, as the reference rounds it)
//   acc += e                  (fp32, add.rn.f32.f16)
// The table is filled from 60 thresholds that the host finds by bisection with an exact scalar
// restatement of the element quantizer, so the kernel's results stay bit-identical to the
// reference's (src/quantizer.py:741-859).
#include "quantize_dev.cuh"
#include "vcache_dev.cuh"
#include "quantize_tab.cuh"
#include <math.h>
#include <stdlib.h>
#include <string.h>

namespace hbq {

constexpr int LUT_MAX_CAND = 4;
constexpr int LUT_MAX_LEVELS = 32;
constexpr int LUT_MAX_SEG = 192;

struct LutPlan {
    int nlev;                                   // 2^(mbit+2) magnitudes of E2M<mbit>
    int base, hi;                               // table covers |a| patterns [base, hi]; entry 0 = all zero
    uint16_t thr[LUT_MAX_CAND][LUT_MAX_LEVELS]; // thr[i][k]: smallest |a| pattern whose level is >= k
    uint16_t val[LUT_MAX_CAND][LUT_MAX_LEVELS]; // fp16 pattern of level_k * t_i
    uint16_t zmax[LUT_MAX_CAND];                // largest |a| pattern with fp16(a / t_i) == 0
    uint16_t hole[LUT_MAX_CAND][4];             // E2M1: |a| patterns with fp16(a / t_i) == 0x39FF (value 0)
    int nhole[LUT_MAX_CAND];
    // the table is piecewise constant: sorted first patterns of its runs (every threshold of every
    // candidate, and both edges of every hole), so a CTA fills it run by run
    int nseg;
    uint16_t seg_start[LUT_MAX_SEG];
};

// ---- exact host-side scalar arithmetic on fp16 patterns ------------------------------------------
static double h2d(uint16_t b)
{
    const int e = (b >> 10) & 31, m = b & 1023;
    const double v = e == 0 ? ldexp((double)m, -24) : ldexp((double)(1024 + m), e - 25);
    return (b & 0x8000) ? -v : v;
}
// round a non-negative double to the nearest fp16 pattern (ties to even); saturates to infinity
static uint16_t d2h(double v)
{
    if (!(v > 0.0)) return 0;
    int ex;
    frexp(v, &ex);                              // v = f * 2^ex, f in [0.5, 1)
    int e = ex - 1;                             // floor(log2 v)
    if (e < -14) e = -14;                       // subnormal range: fixed quantum 2^-24
    const double q = ldexp(v, 10 - e);          // in units of the quantum
    double r = nearbyint(q);                    // FE_TONEAREST: ties to even
    if (e == -14 && r < 1024.0) return (uint16_t)r;
    if (r >= 2048.0) { r = 1024.0; ++e; }
    if (e > 15) return 0x7C00;
    return (uint16_t)(((e + 15) << 10) | ((int)r - 1024));
}

// Level index (= code magnitude {exp, mant}) of the E2M<mb> element quantizer for |b| given as an
// fp16 pattern: the closed form of make_fp_quant (src/quantizer.py:202-255) used by the kernels.
// hole_as: what the E2M1 exception |b| = 0x39FF returns (the reference gives 0).
static int e2_level(int mb, uint16_t b, int hole_as)
{
    const uint16_t a = b & 0x7FFF;
    if (a >= 0x3C00) {
        const uint16_t half = 0x0200 >> mb, mask = ~((0x0400 >> mb) - 1);
        uint16_t n = (uint16_t)((a + half) & mask);
        const uint16_t mx = 0x4400 | (((1u << mb) - 1u) << (10 - mb));
        if (n > mx) n = mx;
        return (n - 0x3800) >> (10 - mb);
    }
    if (mb == 1 && a == 0x39FF) return hole_as;
    const uint16_t w = d2h(h2d(a) * (double)(1 << mb) + 0.50048828125);
    return (int)floor(h2d(w));
}
static double e2_value(int mb, int level)
{
    const int ef = level >> mb, mf = level & ((1 << mb) - 1);
    return ef == 0 ? (double)mf / (1 << mb) : (1.0 + (double)mf / (1 << mb)) * ldexp(1.0, ef - 1);
}

// Build the plan for element E2M<mb> and candidate micro-scales tab[0..nc).  Returns false when
// the format does not fit the table kernel.
bool lut_plan_build(int mb, const float* tab, int nc, LutPlan* p)
{
    if (mb < 1 || mb > 3 || nc < 1 || nc > LUT_MAX_CAND) return false;
    memset(p, 0, sizeof(*p));
    p->nlev = 1 << (mb + 2);
    int lo = 0x7BFF, hi = 0;
    for (int i = 0; i < LUT_MAX_CAND; ++i) {
        const double t = tab[i < nc ? i : nc - 1];      // unused slots repeat the last candidate
        if (!(t >= 1.0) || t > 64.0) return false;
        auto level_of = [&](uint16_t u, int hole_as) { return e2_level(mb, d2h(h2d(u) / t), hole_as); };
        for (int k = 1; k < p->nlev; ++k) {             // smallest u with level >= k (monotone version)
            int a = 0, b = 0x7BFF;                      // invariant: level(a) < k <= level(b)
            if (level_of((uint16_t)b, 2) < k) return false;
            while (b - a > 1) {
                const int mid = (a + b) >> 1;
                if (level_of((uint16_t)mid, 2) >= k) b = mid; else a = mid;
            }
            p->thr[i][k] = (uint16_t)b;
        }
        for (int k = 0; k < p->nlev; ++k) {
            const double v = e2_value(mb, k) * t;
            const uint16_t hb = d2h(v);
            if (h2d(hb) != v) return false;             // level * t must be exact in fp16
            p->val[i][k] = hb;
        }
        int z = 0;
        while (z < 0x0400 && d2h(h2d((uint16_t)(z + 1)) / t) == 0) ++z;
        p->zmax[i] = (uint16_t)z;
        if (mb == 1) {                                  // the E2M1 hole, mapped back to |a|
            const int c = d2h(h2d(0x39FF) * t);
            for (int u = c - 4; u <= c + 4; ++u)
                if (u > 0 && d2h(h2d((uint16_t)u) / t) == 0x39FF && p->nhole[i] < 4)
                    p->hole[i][p->nhole[i]++] = (uint16_t)u;
        }
        if (p->thr[i][1] < lo) lo = p->thr[i][1];
        if (p->thr[i][p->nlev - 1] > hi) hi = p->thr[i][p->nlev - 1];
    }
    p->base = lo - 1;
    p->hi = hi;
    if (!(p->base >= 1 && (p->hi - p->base + 1) <= 8191)) return false;   // byte offsets of the entries must fit 16 bits
    // run starts inside [base, hi], sorted and unique
    int cand[LUT_MAX_CAND * (LUT_MAX_LEVELS + 8) + 1], nb = 0;
    cand[nb++] = p->base;
    for (int i = 0; i < LUT_MAX_CAND; ++i) {
        for (int k = 1; k < p->nlev; ++k) cand[nb++] = p->thr[i][k];
        for (int h = 0; h < p->nhole[i]; ++h) { cand[nb++] = p->hole[i][h]; cand[nb++] = p->hole[i][h] + 1; }
    }
    for (int i = 1; i < nb; ++i) {                      // insertion sort, a few hundred values at most
        const int v = cand[i];
        int j = i - 1;
        while (j >= 0 && cand[j] > v) { cand[j + 1] = cand[j]; --j; }
        cand[j + 1] = v;
    }
    p->nseg = 0;
    for (int i = 0; i < nb; ++i) {
        if (cand[i] < p->base || cand[i] > p->hi) continue;
        if (p->nseg > 0 && p->seg_start[p->nseg - 1] == (uint16_t)cand[i]) continue;
        if (p->nseg == LUT_MAX_SEG) return false;
        p->seg_start[p->nseg++] = (uint16_t)cand[i];
    }
    return true;
}


// ---- kernel arguments -----------------------------------------------------------------------------
struct LutArgs {
    QArgs q;                  // tensor geometry, pointers and output selection (shared helpers use it)
    LutPlan plan;
    uint16_t rm[8];           // fp16(1 / m) for the eight E5M3 mantissas m = 1 + i/8
    uint16_t rt[LUT_MAX_CAND];// fp16(1 / t_i), for the code extraction
    float inv_ele_max;        // 1 / (element max * largest candidate), rounded to fp32
    uint16_t big_l1;          // smallest l1 pattern with l1 * max value > 65504 (fp16 overflow of deq)
    int lpm, log2lpm;         // lanes per micro-block (l2_block_size / 8) and its log2
    int log2cpr;              // log2(chunks per row) when that is a power of two (KV-cache write), else -1
    // second candidate table of the two-table ("Mix") weight formats
    LutPlan plan2;
    float inv_ele_max2;
    uint16_t big_l12;
    int iters;                // chunks per thread
    int64_t step_rows, step_chunks;   // one grid stride of chunks = step_rows rows + step_chunks chunks
};

constexpr int LUT_THREADS = 512;
static_assert(sizeof(LutArgs) <= 4000, "kernel parameters are limited to 4 KB");

// acc_lo += lo(e), acc_hi += hi(e): fp32 accumulation of two fp16 values (one rounding each)
__device__ __forceinline__ void add2_f32_f16(float& acc_lo, float& acc_hi, uint32_t e)
{
    asm("{ .reg .b16 lo, hi;\n mov.b32 {lo, hi}, %2;\n"
        " add.rn.f32.f16 %0, lo, %0;\n add.rn.f32.f16 %1, hi, %1; }"
        : "+f"(acc_lo), "+f"(acc_hi) : "r"(e));
}

// Build the candidate table: entry e covers |a| pattern base + e and holds the 4 candidates' values.
// The table is piecewise constant (a run per threshold of any candidate), so the runs' values are found
// first and then copied out.  Ends without a barrier: callers synchronise before the first lookup.
template <int MB>
__device__ __forceinline__ void lut_build(const LutPlan& plan, uint2* lut, int tid, int nthreads)
{
    __shared__ uint16_t s_seg[LUT_MAX_SEG + 1];
    __shared__ uint2 s_segval[LUT_MAX_SEG];
    // the value of every run: one thread per run finds each candidate's level at the run's first pattern
    for (int sidx = tid; sidx < plan.nseg; sidx += nthreads) {
        const uint32_t u = plan.seg_start[sidx];
        uint32_t v[LUT_MAX_CAND];
        #pragma unroll
        for (int i = 0; i < LUT_MAX_CAND; ++i) {
            int lvl = 0;
            for (int k = 1; k < plan.nlev; ++k) lvl += (u >= plan.thr[i][k]) ? 1 : 0;     // thresholds are sorted
            uint32_t val = plan.val[i][lvl];
            if (MB == 1)
                for (int h = 0; h < plan.nhole[i]; ++h)
                    if (u == plan.hole[i][h]) val = 0;
            v[i] = val;
        }
        s_seg[sidx] = (uint16_t)u;
        s_segval[sidx] = make_uint2(v[0] | (v[1] << 16), v[2] | (v[3] << 16));
    }
    if (tid == 0) s_seg[plan.nseg] = 0xFFFF;
    __syncthreads();
    // fill: a thread takes consecutive entries, finds the run of its first one and walks on from there
    const int n = plan.hi - plan.base + 1;
    const int per = (n + nthreads - 1) / nthreads;
    const int e0 = tid * per, e1 = min(n, e0 + per);
    if (e0 < e1) {
        const uint32_t u0 = (uint32_t)(plan.base + e0);
        int lo = 0, hi = plan.nseg - 1;                     // largest run start <= u0 (run 0 starts at base)
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_seg[mid] <= u0) lo = mid; else hi = mid - 1;
        }
        int sidx = lo;
        for (int e = e0; e < e1; ++e) {
            while ((uint32_t)(plan.base + e) >= s_seg[sidx + 1]) ++sidx;
            lut[e] = s_segval[sidx];
        }
    }
}

// One 8-element chunk of a block through the table: block scale, all candidates' errors, the
// winner's values (dq), its signs (sgo) and, with CODES, its code magnitudes (mag).  The G lanes of
// the block call this together (the maximum and the micro-block error sums are warp shuffles).
template <int MB, bool CODES>
__device__ __forceinline__ void lut_chunk(const LutArgs& a, const uint2* lut, const Chunk& x, uint32_t base2, uint32_t hi2,
                                          __half2* dq, uint32_t* mag, uint32_t* sgo, int& best, uint32_t& l1b)
{
    uint32_t sg[4], ax[4];
    #pragma unroll
    for (int p = 0; p < 4; ++p) { sg[p] = h2_bits(x.h[p]) & 0x80008000u; ax[p] = h2_bits(x.h[p]) & 0x7FFF7FFFu; }

    // -- block maximum and the E5M3 shared scale (round-half-up of the 3-bit mantissa) --
    uint32_t mx = h2_bits(__hmax2(__hmax2(bits_h2(ax[0]), bits_h2(ax[1])), __hmax2(bits_h2(ax[2]), bits_h2(ax[3]))));
    for (int off = a.q.G >> 1; off >= 1; off >>= 1)
        mx = h2_bits(__hmax2(bits_h2(mx), bits_h2(__shfl_xor_sync(0xFFFFFFFFu, mx, off))));
    const uint32_t am16 = max(mx & 0xFFFFu, mx >> 16);
    // amax / ele_max as a multiplication by the rounded reciprocal: exact after the fp16 rounding
    // because ele_max has a short significand (same argument as div2_h)
    const float sf = __half2float(bits_h((uint16_t)am16)) * a.inv_ele_max;
    uint32_t sb = (uint32_t)h_bits(__float2half_rn(sf));
    sb = min(max(sb, 0x0400u), 0x7B80u);
    l1b = (sb + 0x40u) & 0xFF80u;

    // -- a = fp16(|x| / l1): l1 = m * 2^e; |x| is pre-scaled so that the residual of the
    //    division by m stays exact, then the quotient is scaled back (exact unless a < 2^-14) --
    const int e5 = (int)(l1b >> 10) - 15;
    const int s1 = min(15, 8 - e5);
    const uint32_t pre2 = ((uint32_t)(s1 + 15) << 10) * 0x00010001u;
    const uint32_t post2 = ((uint32_t)(15 - (s1 + e5)) << 10) * 0x00010001u;
    const uint32_t nm2 = (0xBC00u | (l1b & 0x03FFu)) * 0x00010001u;          // -m
    const uint32_t rm2 = (uint32_t)a.rm[(l1b >> 7) & 7u] * 0x00010001u;
    const __half2 l1_2 = bits_h2(l1b * 0x00010001u), nl1_2 = bits_h2((l1b | 0x8000u) * 0x00010001u);
    const bool big = l1b >= a.big_l1;

    __half2 aa[4];
    uint32_t w[4];
    #pragma unroll
    for (int p = 0; p < 4; ++p) {
        const __half2 axs = __hmul2(bits_h2(ax[p]), bits_h2(pre2));
        const __half2 q0 = __hmul2(axs, bits_h2(rm2));
        const __half2 r = __hfma2(q0, bits_h2(nm2), axs);
        const __half2 q1 = __hfma2(r, bits_h2(rm2), q0);
        aa[p] = __hmul2(q1, bits_h2(post2));
        // byte offset of the table entry (8 B each; at most 12288 entries, so it fits 16 bits)
        w[p] = (h2_bits(__hmin2(__hmax2(aa[p], bits_h2(base2)), bits_h2(hi2))) - base2) << 3;
    }

    // -- every candidate's squared error, two candidates per half2 --
    uint32_t ct01[8], ct23[8];
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
    if (!big) {
        #pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int p = j >> 1;
            const uint32_t off = (j & 1) ? (w[p] >> 16) : (w[p] & 0xFFFFu);
            const uint2 ent = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(lut) + off);
            ct01[j] = ent.x; ct23[j] = ent.y;
            const __half2 axb = (j & 1) ? __high2half2(bits_h2(ax[p])) : __low2half2(bits_h2(ax[p]));
            const __half2 r01 = __hfma2(bits_h2(ent.x), nl1_2, axb), r23 = __hfma2(bits_h2(ent.y), nl1_2, axb);
            add2_f32_f16(acc0, acc1, h2_bits(__hmul2(r01, r01)));
            add2_f32_f16(acc2, acc3, h2_bits(__hmul2(r23, r23)));
        }
    } else {
        // value * l1 may overflow to infinity here: keep the product's own rounding
        #pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int p = j >> 1;
            const uint32_t off = (j & 1) ? (w[p] >> 16) : (w[p] & 0xFFFFu);
            const uint2 ent = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(lut) + off);
            ct01[j] = ent.x; ct23[j] = ent.y;
            const __half2 axb = (j & 1) ? __high2half2(bits_h2(ax[p])) : __low2half2(bits_h2(ax[p]));
            const __half2 r01 = __hsub2(axb, __hmul2(bits_h2(ent.x), l1_2));
            const __half2 r23 = __hsub2(axb, __hmul2(bits_h2(ent.y), l1_2));
            add2_f32_f16(acc0, acc1, h2_bits(__hmul2(r01, r01)));
            add2_f32_f16(acc2, acc3, h2_bits(__hmul2(r23, r23)));
        }
    }
    for (int off = a.lpm >> 1; off >= 1; off >>= 1) {
        acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, off); acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, off);
        acc2 += __shfl_xor_sync(0xFFFFFFFFu, acc2, off); acc3 += __shfl_xor_sync(0xFFFFFFFFu, acc3, off);
    }
    // first minimum of the fp16-rounded sums (non-negative fp16 patterns order like integers)
    const uint32_t E01 = h2_bits(__floats2half2_rn(acc0, acc1)), E23 = h2_bits(__floats2half2_rn(acc2, acc3));
    uint32_t bv = E01 & 0xFFFFu;
    best = 0;
    if ((E01 >> 16) < bv) { bv = E01 >> 16; best = 1; }
    if ((E23 & 0xFFFFu) < bv) { bv = E23 & 0xFFFFu; best = 2; }
    if ((E23 >> 16) < bv) { bv = E23 >> 16; best = 3; }

    // -- the winner's values, signs and (optionally) codes --
    const uint32_t psel = (best & 1) ? 0x7632u : 0x5410u;
    uint32_t tiny[4];
    #pragma unroll
    for (int p = 0; p < 4; ++p) {
        const uint32_t ra = best < 2 ? ct01[2 * p] : ct23[2 * p], rb = best < 2 ? ct01[2 * p + 1] : ct23[2 * p + 1];
        const __half2 ctw = bits_h2(__byte_perm(ra, rb, psel));
        const __half2 d = __hmul2(ctw, l1_2);
        // negative inputs whose quotient a is tiny: candidates for the reference's "+0" rule below
        tiny[p] = __hle2_mask(aa[p], bits_h2(0x00200020u)) & ((sg[p] >> 15) * 0xFFFFu);
        const uint32_t s = sg[p];
        dq[p] = bits_h2(h2_bits(d) | s);
        sgo[p] = s;
        if (CODES) mag[p] = code2_e2<MB>(__hmul2(ctw, bits_h2((uint32_t)a.rt[best] * 0x00010001u)));
    }

    // The reference returns +0 (not -0) when fp16(a / t) is exactly zero.  Deciding that needs
    // the exact a for tiny quotients, where the scaled division above may be off: rare, so branch.
    if (tiny[0] | tiny[1] | tiny[2] | tiny[3]) {
        const float l1f = __half2float(bits_h((uint16_t)l1b)), t = a.q.tab[0][best < a.q.nc ? best : a.q.nc - 1];
        #pragma unroll
        for (int p = 0; p < 4; ++p)
            #pragma unroll
            for (int h = 0; h < 2; ++h)
                if ((tiny[p] >> (16 * h)) & 1u) {
                    const float xf = __half2float(bits_h((uint16_t)(ax[p] >> (16 * h))));
                    if (rh(__fdiv_rn(rh(__fdiv_rn(xf, l1f)), t)) == 0.f) {
                        const uint32_t clr = ~(0x8000u << (16 * h));
                        dq[p] = bits_h2(h2_bits(dq[p]) & clr);
                        sgo[p] &= clr;
                    }
                }
    }

}

// ---- the kernel -----------------------------------------------------------------------------------
template <int MB, bool CODES>
__global__ void __launch_bounds__(LUT_THREADS, 2) hbq_lut_kernel(const LutArgs a)
{
    extern __shared__ __align__(16) uint2 lut[];
    const QArgs& q = a.q;
    const int tid = threadIdx.x;

    lut_build<MB>(a.plan, lut, tid, LUT_THREADS);
    __syncthreads();

    const int lane = tid & 31;
    const int lig = tid & (q.G - 1);
    const uint32_t base2 = (uint32_t)a.plan.base * 0x00010001u, hi2 = (uint32_t)a.plan.hi * 0x00010001u;
    const int nl2 = q.f.block_size / q.f.l2_block_size;

    int64_t ci = (int64_t)blockIdx.x * LUT_THREADS + tid;
    int64_t row = 0, c = 0;
    split_chunk(q, ci < q.total_chunks ? ci : 0, row, c);
    for (int it = 0; it < a.iters; ++it, ci += (int64_t)gridDim.x * LUT_THREADS) {
        if (it > 0) {                                          // advance (row, chunk-in-row) by one grid stride
            row += a.step_rows; c += a.step_chunks;
            if (c >= q.cpr) { c -= q.cpr; ++row; }
        }
        if (ci - lane >= q.total_chunks) break;                // warp-uniform
        const bool valid = ci < q.total_chunks;
        const int64_t k0 = c * 8;
        Chunk x;
        if (valid) x = load_chunk(q, row, k0);
        else { for (int p = 0; p < 4; ++p) x.h[p] = bits_h2(0u); }
        if (q.rope_cos) rope_chunk(q, x, valid ? row : 0, k0);
        if (q.k_center) center_chunk(q, x, valid ? row : 0, k0);

        __half2 dq[4];
        uint32_t mag[4], sgo[4], l1b;
        int best;
        lut_chunk<MB, CODES>(a, lut, x, base2, hi2, dq, mag, sgo, best, l1b);

        uint32_t l2word = 0;
        const bool mb_leader = (lig & (a.lpm - 1)) == 0;         // first lane of its micro-block
        const int mb_index = lig >> a.log2lpm;
        if (mb_leader) l2word = (uint32_t)best << (mb_index * q.f.l2_sc_bit);
        if (q.out.l2_packed) l2word = group_or(l2word, q.G);

        if (!valid) continue;
        const int64_t kb = c >> q.log2G;
        const int64_t orow = out_row(q, row);
        store_deq(q, orow, k0, dq);
        if (CODES) store_codes<false>(q, orow, k0, mag, sgo);
        if (q.out.l2_idx && mb_leader) q.out.l2_idx[(orow * q.nblk + kb) * nl2 + mb_index] = (uint8_t)best;
        if (lig == 0) {
            store_scale(q, orow, kb, __half2float(bits_h((uint16_t)l1b)));
            if (q.out.scheme) q.out.scheme[orow * q.nblk + kb] = 0;
            if (q.out.l2_packed) {
                const int nbytes = (nl2 * q.f.l2_sc_bit) >> 3;
                uint8_t* lp = q.out.l2_packed + (orow * q.nblk + kb) * nbytes;
                if (nbytes == 4) *reinterpret_cast<uint32_t*>(lp) = l2word;
                else if (nbytes == 2) *reinterpret_cast<uint16_t*>(lp) = (uint16_t)l2word;
                else *lp = (uint8_t)l2word;
            }
        }
    }
}

// ---- the lean kernel: contiguous, aligned tensors, fake-quantised output only ---------------------
// The shape every per-step activation quantize has: K a multiple of the block (no padding), 16-byte
// aligned pointers, no packed or side outputs, no RoPE / permutation.  Chunk ci is then elements
// [8 ci, 8 ci + 8) of both tensors and a thread's lane-in-block never changes, so the row / column
// bookkeeping, the output selection and the dtype branches of the general kernel disappear; the
// per-block division constants come from a second small shared table indexed by the E5M3 scale.
// One CTA of 1024 threads per SM (the candidate table is built once per SM).
constexpr int LEAN_THREADS = 1024;

// One candidate table as the chunk arithmetic sees it.
struct LutView {
    const uint8_t* lutb;          // the table in shared memory
    uint32_t base2, hi2;          // first / last covered |a| pattern, in both halves
    float inv_ele_max;
    uint32_t big_l1;
    const float* tab;             // the candidates (for the rare exact sign-of-zero check)
    int nc;
};

// One 8-element chunk through the tables: xb = the chunk as packed fp16 pairs, dq = its fake-quantised
// values (fp16 pairs, input signs).  The G lanes of a block call this together.  WANT_ERR: also return
// this thread's fp32 sum of the chosen candidates' squared errors (the block total decides between
// the two tables of a "Mix" format).
template <int MB, bool WANT_ERR>
__device__ __forceinline__ void lean_chunk(const LutView& t, const uint4* s_l1c, int lpm, int G, const uint32_t* xb,
                                           uint32_t* dq, float* err)
{
    uint32_t ax[4];
    #pragma unroll
    for (int p = 0; p < 4; ++p) ax[p] = xb[p] & 0x7FFF7FFFu;

    // -- block maximum and the E5M3 shared scale (round-half-up of the 3-bit mantissa) --
    uint32_t mx = h2_bits(__hmax2(__hmax2(bits_h2(ax[0]), bits_h2(ax[1])), __hmax2(bits_h2(ax[2]), bits_h2(ax[3]))));
    for (int off = G >> 1; off >= 1; off >>= 1)
        mx = h2_bits(__hmax2(bits_h2(mx), bits_h2(__shfl_xor_sync(0xFFFFFFFFu, mx, off))));
    const uint32_t am16 = max(mx & 0xFFFFu, mx >> 16);
    const float sf = __half2float(bits_h((uint16_t)am16)) * t.inv_ele_max;
    uint32_t sb = (uint32_t)h_bits(__float2half_rn(sf));
    sb = min(max(sb, 0x0400u), 0x7B80u);
    const uint32_t l1b = (sb + 0x40u) & 0xFF80u;
    const uint4 cst = s_l1c[l1b >> 7];
    const __half2 pre2 = bits_h2(cst.x), post2 = bits_h2(cst.y), nm2 = bits_h2(cst.z), rm2 = bits_h2(cst.w);
    const uint32_t l1u = l1b * 0x00010001u;
    const __half2 l1_2 = bits_h2(l1u), nl1_2 = bits_h2(l1u ^ 0x80008000u);

    // -- a = fp16(|x| / l1) by the pre-scaled Markstein division, and the table offsets --
    __half2 aa[4];
    uint32_t w[4];
    #pragma unroll
    for (int p = 0; p < 4; ++p) {
        const __half2 axs = __hmul2(bits_h2(ax[p]), pre2);
        const __half2 q0 = __hmul2(axs, rm2);
        const __half2 r = __hfma2(q0, nm2, axs);
        const __half2 q1 = __hfma2(r, rm2, q0);
        aa[p] = __hmul2(q1, post2);
        w[p] = (h2_bits(__hmin2(__hmax2(aa[p], bits_h2(t.base2)), bits_h2(t.hi2))) - t.base2) << 3;
    }

    // -- every candidate's squared error, two candidates per half2 --
    uint32_t ct01[8], ct23[8];
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
    const bool small = l1b < t.big_l1;
    if (small) {
        #pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int p = j >> 1;
            const uint32_t off = (j & 1) ? (w[p] >> 16) : (w[p] & 0xFFFFu);
            const uint2 ent = *reinterpret_cast<const uint2*>(t.lutb + off);
            ct01[j] = ent.x; ct23[j] = ent.y;
            const __half2 axb = (j & 1) ? __high2half2(bits_h2(ax[p])) : __low2half2(bits_h2(ax[p]));
            const __half2 r01 = __hfma2(bits_h2(ent.x), nl1_2, axb), r23 = __hfma2(bits_h2(ent.y), nl1_2, axb);
            add2_f32_f16(acc0, acc1, h2_bits(__hmul2(r01, r01)));
            add2_f32_f16(acc2, acc3, h2_bits(__hmul2(r23, r23)));
        }
    } else {
        // value * l1 may overflow to infinity here: keep the product's own rounding
        #pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int p = j >> 1;
            const uint32_t off = (j & 1) ? (w[p] >> 16) : (w[p] & 0xFFFFu);
            const uint2 ent = *reinterpret_cast<const uint2*>(t.lutb + off);
            ct01[j] = ent.x; ct23[j] = ent.y;
            const __half2 axb = (j & 1) ? __high2half2(bits_h2(ax[p])) : __low2half2(bits_h2(ax[p]));
            const __half2 r01 = __hsub2(axb, __hmul2(bits_h2(ent.x), l1_2));
            const __half2 r23 = __hsub2(axb, __hmul2(bits_h2(ent.y), l1_2));
            add2_f32_f16(acc0, acc1, h2_bits(__hmul2(r01, r01)));
            add2_f32_f16(acc2, acc3, h2_bits(__hmul2(r23, r23)));
        }
    }
    for (int off = lpm >> 1; off >= 1; off >>= 1) {
        acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, off); acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, off);
        acc2 += __shfl_xor_sync(0xFFFFFFFFu, acc2, off); acc3 += __shfl_xor_sync(0xFFFFFFFFu, acc3, off);
    }
    // first minimum of the fp16-rounded sums (non-negative fp16 patterns order like integers)
    const uint32_t E01 = h2_bits(__floats2half2_rn(acc0, acc1)), E23 = h2_bits(__floats2half2_rn(acc2, acc3));
    uint32_t bv = E01 & 0xFFFFu;
    int best = 0;
    if ((E01 >> 16) < bv) { bv = E01 >> 16; best = 1; }
    if ((E23 & 0xFFFFu) < bv) { bv = E23 & 0xFFFFu; best = 2; }
    if ((E23 >> 16) < bv) { bv = E23 >> 16; best = 3; }

    // -- the winner's values with the inputs' signs --
    const uint32_t psel = (best & 1) ? 0x7632u : 0x5410u;
    #pragma unroll
    for (int p = 0; p < 4; ++p) {
        const uint32_t ra = best < 2 ? ct01[2 * p] : ct23[2 * p], rb = best < 2 ? ct01[2 * p + 1] : ct23[2 * p + 1];
        const __half2 ctw = bits_h2(__byte_perm(ra, rb, psel));
        const __half2 d = __hmul2(ctw, l1_2);
        dq[p] = h2_bits(d) | (xb[p] & 0x80008000u);
        if (WANT_ERR) {
            const __half2 r = small ? __hfma2(ctw, nl1_2, bits_h2(ax[p])) : __hsub2(bits_h2(ax[p]), d);
            float e0 = 0.f, e1 = 0.f;
            add2_f32_f16(e0, e1, h2_bits(__hmul2(r, r)));
            *err += e0; *err += e1;
        }
    }
    // The reference returns +0 (not -0) when fp16(a / t) is exactly zero.  Only quotients a below
    // 2^-19 can do that; deciding it needs the exact a, where the scaled division may be off: rare.
    const __half2 amin = __hmin2(__hmin2(aa[0], aa[1]), __hmin2(aa[2], aa[3]));
    if (__hle2_mask(amin, bits_h2(0x00200020u)) != 0u) {
        const float l1f = __half2float(bits_h((uint16_t)l1b)), tc = t.tab[best < t.nc ? best : t.nc - 1];
        #pragma unroll
        for (int p = 0; p < 4; ++p)
            #pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t abits = (h2_bits(aa[p]) >> (16 * h)) & 0xFFFFu;
                if (abits <= 0x0020u && ((xb[p] >> (16 * h)) & 0x8000u)) {
                    const float xf = __half2float(bits_h((uint16_t)(ax[p] >> (16 * h))));
                    if (rh(__fdiv_rn(rh(__fdiv_rn(xf, l1f)), tc)) == 0.f) dq[p] &= ~(0x8000u << (16 * h));
                }
            }
    }

}

// Per E5M3 scale (fp16 pattern >> 7): the division constants {2^s1, 2^-(s1+e), -m, fp16(1/m)} as fp16 pairs.
__device__ __forceinline__ void l1_table_build(const LutArgs& a, uint4* s_l1c, int tid)
{
    if (tid < 256) {
        const uint32_t l1b = (uint32_t)tid << 7;
        const int e5 = (int)(l1b >> 10) - 15;
        const int s1 = min(15, 8 - e5);
        uint4 c;
        c.x = ((uint32_t)(s1 + 15) << 10) * 0x00010001u;
        c.y = ((uint32_t)(15 - (s1 + e5)) << 10) * 0x00010001u;
        c.z = (0xBC00u | (l1b & 0x03FFu)) * 0x00010001u;
        c.w = (uint32_t)a.rm[(l1b >> 7) & 7u] * 0x00010001u;
        s_l1c[tid] = c;
    }
}

// KV: the K / post-RoPE Q cache write on the same fast path -- a row is one (token, head) vector of
// D = K elements (D a power of two <= 256, fp16), RoPE is applied on load and the row is stored at its
// (batch, head, token) position.
// MIX: the two-table weight formats -- both tables are evaluated (each with its own block scale) and
// the one with the smaller fp16 total of the chosen candidates' squared errors over the block wins,
// the first on ties (src/quantizer.py:806-840).
// GLU: the tensor to quantise is silu(gate) * x, computed on the fly from two fp16 tensors with the
// roundings of the two separate elementwise ops it replaces (silu in fp32 from the fp16 input, rounded
// to fp16; the product of the two fp16 values rounded to fp16).
template <int MB, bool IN_BF16, bool OUT_BF16, bool KV, bool MIX, bool GLU = false>
__global__ void __launch_bounds__(LEAN_THREADS, 1) hbq_lut_lean_kernel(const LutArgs a)
{
    extern __shared__ __align__(16) uint2 lut[];
    __shared__ uint4 s_l1c[256];             // per E5M3 scale (pattern >> 7): {pre2, post2, -m2, 1/m 2}
    const int tid = threadIdx.x;
    lut_build<MB>(a.plan, lut, tid, LEAN_THREADS);
    l1_table_build(a, s_l1c, tid);
    const int n0 = a.plan.hi - a.plan.base + 1;
    if (MIX) {
        __syncthreads();                     // the builder's staging arrays are reused
        lut_build<MB>(a.plan2, lut + n0, tid, LEAN_THREADS);
    }
    __syncthreads();

    const LutView view0 = {reinterpret_cast<const uint8_t*>(lut), (uint32_t)a.plan.base * 0x00010001u,
                           (uint32_t)a.plan.hi * 0x00010001u, a.inv_ele_max, a.big_l1, a.q.tab[0], a.q.nc};
    const LutView view1 = {reinterpret_cast<const uint8_t*>(lut + n0), (uint32_t)a.plan2.base * 0x00010001u,
                           (uint32_t)a.plan2.hi * 0x00010001u, a.inv_ele_max2, a.big_l12, a.q.tab[1], a.q.nc};
    const uint4* __restrict__ in = reinterpret_cast<const uint4*>(a.q.x);
    const uint4* __restrict__ gate = reinterpret_cast<const uint4*>(a.q.glu_gate);
    uint4* __restrict__ out = reinterpret_cast<uint4*>(a.q.deq);
    const int64_t total = a.q.total_chunks, stride = (int64_t)gridDim.x * LEAN_THREADS;
    const int lane = tid & 31;
    const int G = a.q.G;

    int64_t ci = (int64_t)blockIdx.x * LEAN_THREADS + tid;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u), graw = make_uint4(0u, 0u, 0u, 0u);
    if (ci < total) { raw = __ldg(in + ci); if (GLU) graw = __ldg(gate + ci); }
    for (; ci - lane < total; ci += stride) {
        const bool valid = ci < total;
        uint4 nraw = make_uint4(0u, 0u, 0u, 0u), ngraw = make_uint4(0u, 0u, 0u, 0u);
        if (ci + stride < total) {                                     // next chunk in flight during this one
            nraw = __ldg(in + ci + stride);
            if (GLU) ngraw = __ldg(gate + ci + stride);
        }

        uint32_t xb[4] = {raw.x, raw.y, raw.z, raw.w};
        if (GLU) {
            const uint32_t gb[4] = {graw.x, graw.y, graw.z, graw.w};
            #pragma unroll
            for (int p = 0; p < 4; ++p) {
                const float2 g = __half22float2(bits_h2(gb[p])), u = __half22float2(bits_h2(xb[p]));
                const float s0 = rh(__fdiv_rn(g.x, 1.f + expf(-g.x))), s1 = rh(__fdiv_rn(g.y, 1.f + expf(-g.y)));
                xb[p] = h2_bits(__floats2half2_rn(s0 * u.x, s1 * u.y));      // fp16 x fp16 is exact in fp32
            }
        }
        int64_t oci = ci;                                  // chunk index of the output
        if (KV) {
            const int64_t row = valid ? ci >> a.log2cpr : 0, c = ci & (a.q.cpr - 1);
            Chunk xr;
            #pragma unroll
            for (int p = 0; p < 4; ++p) xr.h[p] = bits_h2(xb[p]);
            if (a.q.rope_cos) rope_chunk(a.q, xr, row, c * 8);
            if (a.q.k_center) center_chunk(a.q, xr, row, c * 8);
            #pragma unroll
            for (int p = 0; p < 4; ++p) xb[p] = h2_bits(xr.h[p]);
            oci = (out_row(a.q, row) << a.log2cpr) + c;
        }
        if (IN_BF16) {
            #pragma unroll
            for (int p = 0; p < 4; ++p)
                xb[p] = h2_bits(__floats2half2_rn(__uint_as_float(xb[p] << 16), __uint_as_float(xb[p] & 0xFFFF0000u)));
        }
        uint32_t dq[4];
        if (!MIX) {
            lean_chunk<MB, false>(view0, s_l1c, a.lpm, G, xb, dq, nullptr);
        } else {
            uint32_t dq1[4];
            float e0 = 0.f, e1 = 0.f;
            lean_chunk<MB, true>(view0, s_l1c, a.lpm, G, xb, dq, &e0);
            lean_chunk<MB, true>(view1, s_l1c, a.lpm, G, xb, dq1, &e1);
            for (int off = G >> 1; off >= 1; off >>= 1) {
                e0 += __shfl_xor_sync(0xFFFFFFFFu, e0, off);
                e1 += __shfl_xor_sync(0xFFFFFFFFu, e1, off);
            }
            if (rh(e1) < rh(e0)) {
                #pragma unroll
                for (int p = 0; p < 4; ++p) dq[p] = dq1[p];
            }
        }
        if (valid) {
            if (OUT_BF16) {
                #pragma unroll
                for (int p = 0; p < 4; ++p) {
                    const float2 f = __half22float2(bits_h2(dq[p]));
                    __nv_bfloat162 bb = __floats2bfloat162_rn(f.x, f.y);
                    dq[p] = *reinterpret_cast<uint32_t*>(&bb);
                }
            }
            out[oci] = make_uint4(dq[0], dq[1], dq[2], dq[3]);
        }
        raw = nraw;
        if (GLU) graw = ngraw;
    }
}

template <int MB>
static int launch_lean(const LutArgs& a, int grid, size_t smem, cudaStream_t stream)
{
    #define HBQ_LAUNCH_LEAN(IB, OB, KVW)                                                                                              \
        { const int rc_ = ensure_dynamic_smem(hbq_lut_lean_kernel<MB, IB, OB, KVW, false>, smem); if (rc_) return rc_; }             \
        hbq_lut_lean_kernel<MB, IB, OB, KVW, false><<<grid, LEAN_THREADS, smem, stream>>>(a);
    #define HBQ_LAUNCH_LEAN_MIX(IB, OB)                                                                                               \
        { const int rc_ = ensure_dynamic_smem(hbq_lut_lean_kernel<MB, IB, OB, false, true>, smem); if (rc_) return rc_; }            \
        hbq_lut_lean_kernel<MB, IB, OB, false, true><<<grid, LEAN_THREADS, smem, stream>>>(a);
    const bool kvw = a.q.rope_cos || a.q.perm_T > 0 || a.q.k_center;
    if (a.q.glu_gate) {
        if (a.q.nscheme == 2 || kvw || a.q.in_bf16 || a.q.out_bf16) return HBQ_ERR_UNSUPPORTED;
        { const int rc_ = ensure_dynamic_smem(hbq_lut_lean_kernel<MB, false, false, false, false, true>, smem); if (rc_) return rc_; }
        hbq_lut_lean_kernel<MB, false, false, false, false, true><<<grid, LEAN_THREADS, smem, stream>>>(a);
    } else if (a.q.nscheme == 2) {
        if (a.q.in_bf16) { if (a.q.out_bf16) { HBQ_LAUNCH_LEAN_MIX(true, true) } else { HBQ_LAUNCH_LEAN_MIX(true, false) } }
        else { if (a.q.out_bf16) { HBQ_LAUNCH_LEAN_MIX(false, true) } else { HBQ_LAUNCH_LEAN_MIX(false, false) } }
    } else if (kvw) { if (a.q.out_bf16) { HBQ_LAUNCH_LEAN(false, true, true) } else { HBQ_LAUNCH_LEAN(false, false, true) } }
    else if (a.q.in_bf16) { if (a.q.out_bf16) { HBQ_LAUNCH_LEAN(true, true, false) } else { HBQ_LAUNCH_LEAN(true, false, false) } }
    else { if (a.q.out_bf16) { HBQ_LAUNCH_LEAN(false, true, false) } else { HBQ_LAUNCH_LEAN(false, false, false) } }
    #undef HBQ_LAUNCH_LEAN
    #undef HBQ_LAUNCH_LEAN_MIX
    HBQ_LAUNCH_CHECK("hbq_lut_lean_kernel");
    return HBQ_OK;
}

// ---- V-cache write: quantisation along the token axis (tile machinery in vcache_dev.cuh) ----------
template <int MB>
struct LutChunkFn {
    LutView view;
    const uint4* s_l1c;
    int lpm, G;
    __device__ __forceinline__ void operator()(const uint32_t* xb, uint32_t* dq) const
    {
        lean_chunk<MB, false>(view, s_l1c, lpm, G, xb, dq, nullptr);
    }
};

template <int MB>
__global__ void __launch_bounds__(V_THREADS, 2) hbq_lut_v_kernel(const LutArgs a, const VArgs v)
{
    extern __shared__ __align__(16) uint2 lut[];
    const int tid = threadIdx.x;
    const int n = a.plan.hi - a.plan.base + 1;
    uint32_t* tile = reinterpret_cast<uint32_t*>(lut + ((n + 1) & ~1));   // 16-byte aligned, after the candidate table
    __shared__ uint4 s_l1c[256];
    lut_build<MB>(a.plan, lut, tid, V_THREADS);
    l1_table_build(a, s_l1c, tid);
    __syncthreads();
    const LutChunkFn<MB> fn = {{reinterpret_cast<const uint8_t*>(lut), (uint32_t)a.plan.base * 0x00010001u,
                                (uint32_t)a.plan.hi * 0x00010001u, a.inv_ele_max, a.big_l1, a.q.tab[0], a.q.nc},
                               s_l1c, a.lpm, a.q.G};
    v_cache_tiles(v, tile, fn);
}

// ---- host side ------------------------------------------------------------------------------------
}  // namespace hbq
#include <mutex>
#include <vector>
namespace hbq {

struct CachedPlan {
    int mb, nc;
    float tab[LUT_MAX_CAND];
    bool ok;
    LutPlan plan;
    uint16_t rm[8], rt[LUT_MAX_CAND], big_l1;       // derived kernel arguments (see LutArgs)
    uint32_t* bytes;                                // byte form of the table (hbq_tab_table), or NULL
    int nbytes_entries;
};
static std::mutex g_plan_mutex;
static std::vector<CachedPlan> g_plans;

// Byte form of a plan's candidate table, for E2M1 / E2M2 elements: entry e (the |a| pattern base + e) holds,
// for each of the four candidates, the TOP BYTE of the fp16 pattern of the element value Q(fp16(a / t_i)) --
// every E2M1 / E2M2 value has at most two mantissa bits, so that byte followed by a zero byte IS the value.
// Padded with copies of the last entry to a multiple of 4 entries (16 bytes, the bulk-copy granule).
static void byte_table_build(CachedPlan& c)
{
    const LutPlan& p = c.plan;
    const int n = p.hi - p.base + 1, npad = (n + 3) & ~3;
    c.bytes = (uint32_t*)malloc(sizeof(uint32_t) * npad);           // kept for the life of the process
    c.nbytes_entries = npad;
    for (int e = 0; e < npad; ++e) {
        const uint32_t u = (uint32_t)(p.base + (e < n ? e : n - 1));
        uint32_t w = 0;
        for (int i = 0; i < LUT_MAX_CAND; ++i) {
            int lvl = 0;
            for (int k = 1; k < p.nlev; ++k) lvl += (u >= p.thr[i][k]) ? 1 : 0;
            uint32_t hb = d2h(e2_value(c.mb, lvl));
            for (int h = 0; h < p.nhole[i]; ++h)
                if (u == p.hole[i][h]) hb = 0;
            w |= (hb >> 8) << (8 * i);
        }
        c.bytes[e] = w;
    }
}

// Plans depend on the format only; building one costs ~2000 scalar quantizer evaluations.
static void plan_to_args(const CachedPlan& c, LutArgs* a)
{
    a->plan = c.plan;
    memcpy(a->rm, c.rm, sizeof(c.rm));
    memcpy(a->rt, c.rt, sizeof(c.rt));
    a->big_l1 = c.big_l1;
}

static bool get_plan(int mb, const float* tab, int nc, LutArgs* out)
{
    std::lock_guard<std::mutex> lock(g_plan_mutex);
    for (const CachedPlan& c : g_plans)
        if (c.mb == mb && c.nc == nc && memcmp(c.tab, tab, sizeof(float) * nc) == 0) {
            if (c.ok) plan_to_args(c, out);
            return c.ok;
        }
    CachedPlan c;
    memset(&c, 0, sizeof(c));
    c.mb = mb; c.nc = nc;
    memcpy(c.tab, tab, sizeof(float) * nc);
    c.ok = lut_plan_build(mb, tab, nc, &c.plan);
    if (c.ok) {
        for (int i = 0; i < 8; ++i) c.rm[i] = d2h(1.0 / (1.0 + i / 8.0));
        double vmax = 0;
        for (int i = 0; i < LUT_MAX_CAND; ++i) {
            c.rt[i] = d2h(1.0 / (double)tab[i < nc ? i : nc - 1]);
            const double v = h2d(c.plan.val[i][c.plan.nlev - 1]);
            if (v > vmax) vmax = v;
        }
        c.big_l1 = 0x7C00;                     // smallest scale whose product with the largest value overflows fp16
        for (int pat = 0x0400; pat <= 0x7B80; pat += 0x80)
            if (h2d((uint16_t)pat) * vmax > 65504.0) { c.big_l1 = (uint16_t)pat; break; }
    }
    if (g_plans.size() < 64) g_plans.push_back(c);
    if (c.ok) plan_to_args(c, out);
    return c.ok;
}

// The byte table of a format for the kernels of quantize_tab.cu; false when the format has none (elements
// wider than E2M2, no table plan, or the cache of plans is full).  `slot` identifies the format among the
// cached ones (stable for the life of the process).
bool hbq_tab_table(int mb, const float* tab, int nc, TabTable* out)
{
    if (mb < 1 || mb > 2) return false;
    LutArgs scratch;
    memset(&scratch, 0, sizeof(scratch));
    if (!get_plan(mb, tab, nc, &scratch)) return false;
    std::lock_guard<std::mutex> lock(g_plan_mutex);
    for (size_t i = 0; i < g_plans.size(); ++i) {
        CachedPlan& c = g_plans[i];
        if (c.ok && c.mb == mb && c.nc == nc && memcmp(c.tab, tab, sizeof(float) * nc) == 0) {
            if (!c.bytes) byte_table_build(c);
            out->slot = (int)i;
            out->host = c.bytes;
            out->entries = c.nbytes_entries;
            out->base = c.plan.base;
            out->hi = c.plan.hi;
            out->big_l1 = c.big_l1;
            memcpy(out->rm, c.rm, sizeof(c.rm));
            return true;
        }
    }
    return false;
}

template <int MB>
static int launch_lut(const LutArgs& a, bool codes, int grid, size_t smem, cudaStream_t stream)
{
    if (codes) {
        { const int rc_ = ensure_dynamic_smem(hbq_lut_kernel<MB, true>, smem); if (rc_) return rc_; }
        hbq_lut_kernel<MB, true><<<grid, LUT_THREADS, smem, stream>>>(a);
    } else {
        { const int rc_ = ensure_dynamic_smem(hbq_lut_kernel<MB, false>, smem); if (rc_) return rc_; }
        hbq_lut_kernel<MB, false><<<grid, LUT_THREADS, smem, stream>>>(a);
    }
    HBQ_LAUNCH_CHECK("hbq_lut_kernel");
    return HBQ_OK;
}

// Runs the table kernel if the (already validated) HBQ arguments fit it.  *launched tells the
// caller whether it did; when it did not, the arithmetic kernel must be used.
// Kernel arguments of the table kernels for a validated HBQ format; false when no table plan fits it.
static bool fill_lut_args(const QArgs& qa, int mb, LutArgs* out)
{
    LutArgs& a = *out;
    memset(&a, 0, sizeof(a));
    if (!get_plan(mb, qa.tab[0], qa.nc, &a)) return false;
    if (qa.nscheme == 2) {                     // second table: through a scratch copy, then into the plan2 fields
        LutArgs b;
        memset(&b, 0, sizeof(b));
        if (!get_plan(mb, qa.tab[1], qa.nc, &b)) return false;
        a.plan2 = b.plan;
        a.big_l12 = b.big_l1;
        a.inv_ele_max2 = 1.f / qa.ele_max[1];
    }
    a.q = qa;
    a.lpm = qa.f.l2_block_size / 8;
    while ((1 << a.log2lpm) < a.lpm) ++a.log2lpm;
    a.inv_ele_max = 1.f / qa.ele_max[0];
    return true;
}

int hbq_lut_try_launch(const QArgs& qa, int mb, cudaStream_t stream, bool* launched)
{
    *launched = false;
    const int L = qa.f.l2_block_size;
    if (qa.nscheme > 2 || qa.nc > LUT_MAX_CAND || !qa.scale_fast_e5m3 || L < 8 || mb < 1 || mb > 3) return HBQ_OK;
    LutArgs a;
    if (!fill_lut_args(qa, mb, &a)) return HBQ_OK;

    int sms = 0;
    { const int rc_ = device_sms(&sms); if (rc_) return rc_; }
    const QArgs& q = qa;
    const bool side_out = q.out.codes || q.out.sign || q.out.scale_u8 || q.out.scale_h || q.out.l2_packed ||
                          q.out.l2_idx || q.out.scheme;
    const bool kvw = q.rope_cos || q.perm_T > 0 || q.k_center;
    a.log2cpr = -1;
    if ((q.cpr & (q.cpr - 1)) == 0) { a.log2cpr = 0; while ((1ll << a.log2cpr) < q.cpr) ++a.log2cpr; }
    // the K-cache write takes the fast path for fp16 rows of a power-of-two length
    const bool mix = q.nscheme == 2;
    if (q.deq && !side_out && q.aligned && q.K == q.Kp && (!kvw || (!mix && !q.in_bf16 && a.log2cpr >= 0))) {
        const int64_t need = (qa.total_chunks + LEAN_THREADS - 1) / LEAN_THREADS;
        const int grid = (int)(need < sms ? need : sms);
        const size_t smem = (size_t)((a.plan.hi - a.plan.base + 1) + (mix ? a.plan2.hi - a.plan2.base + 1 : 0)) * sizeof(uint2);
        int rc;
        switch (mb) {
            case 1: rc = launch_lean<1>(a, grid, smem, stream); break;
            case 2: rc = launch_lean<2>(a, grid, smem, stream); break;
            default: rc = launch_lean<3>(a, grid, smem, stream); break;
        }
        if (rc == HBQ_OK) *launched = true;
        return rc;
    }
    if (q.glu_gate) return HBQ_ERR_UNSUPPORTED;   // the fused silu(gate) * x exists in the lean kernel only
    if (mix) return HBQ_OK;                    // two tables: only the lean kernel; the arithmetic kernel serves the rest
    const int64_t need = (qa.total_chunks + LUT_THREADS - 1) / LUT_THREADS;
    const int grid = (int)(need < 2 * sms ? need : 2 * sms);
    a.iters = (int)((need + grid - 1) / grid);
    a.step_rows = ((int64_t)grid * LUT_THREADS) / qa.cpr;
    a.step_chunks = ((int64_t)grid * LUT_THREADS) % qa.cpr;
    const size_t smem = (size_t)(a.plan.hi - a.plan.base + 1) * sizeof(uint2);
    const bool codes = qa.out.codes != nullptr;
    int rc;
    switch (mb) {
        case 1: rc = launch_lut<1>(a, codes, grid, smem, stream); break;
        case 2: rc = launch_lut<2>(a, codes, grid, smem, stream); break;
        default: rc = launch_lut<3>(a, codes, grid, smem, stream); break;
    }
    if (rc == HBQ_OK) *launched = true;
    return rc;
}


// Launch the V-cache write.  qa carries the validated HBQ format (QArgs as quantize_launch builds it
// for a [rows, block] problem); returns HBQ_ERR_UNSUPPORTED when the format does not fit the table
// kernel (the caller then transposes and uses hbq_quantize like the reference).
int hbq_lut_v_launch(const QArgs& qa, int mb, const void* in, void* out, int in_bf16, int out_bf16,
                     int64_t B, int64_t T, int64_t H, int64_t D, int out_token_major, cudaStream_t stream)
{
    const int L = qa.f.l2_block_size;
    if (qa.nscheme != 1 || qa.nc > LUT_MAX_CAND || !qa.scale_fast_e5m3 || L < 8 || mb < 1 || mb > 3) return HBQ_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) return HBQ_ERR_ALIGN;
    LutArgs a;
    if (!fill_lut_args(qa, mb, &a)) return HBQ_ERR_UNSUPPORTED;

    VArgs v;
    if (!v_args_fill(&v, in, out, in_bf16, out_bf16, B, T, H, D, qa.f.block_size, out_token_major)) return HBQ_ERR_UNSUPPORTED;
    if (v.tiles == 0) return HBQ_OK;
    int sms = 0;
    { const int rc_ = device_sms(&sms); if (rc_) return rc_; }
    const int grid = (int)(v.tiles < 2 * sms ? v.tiles : 2 * sms);
    const size_t smem = (size_t)((a.plan.hi - a.plan.base + 2) & ~1) * sizeof(uint2) + (size_t)V_TILE_BYTES;
    #define HBQ_LAUNCH_V(MBV)                                                                                            \
        { const int rc_ = ensure_dynamic_smem(hbq_lut_v_kernel<MBV>, smem); if (rc_) return rc_; }                    \
        hbq_lut_v_kernel<MBV><<<grid, V_THREADS, smem, stream>>>(a, v);
    switch (mb) {
        case 1: HBQ_LAUNCH_V(1) break;
        case 2: HBQ_LAUNCH_V(2) break;
        default: HBQ_LAUNCH_V(3) break;
    }
    #undef HBQ_LAUNCH_V
    HBQ_LAUNCH_CHECK("hbq_lut_v_kernel");
    return HBQ_OK;
}

}  // namespace hbq
