// HBQ quantize, byte-table kernels: the per-step activation quantizer (one candidate table, E2M1 / E2M2
// elements, up to 4 micro-scale candidates; src/quantizer.py:741-859).
//
// What HBQ asks per element is 2^l2_sc_bit quantise-dequantise-error evaluations with an fp16 rounding
// after every op.  As in quantize_lut.cu the element quantizer is a table lookup keyed by the fp16
// pattern of |a| = |x / l1|, but here
//   * an entry is 4 BYTES: for each candidate the top byte of the fp16 pattern of the element value
//     c_i = Q(fp16(a / t_i)) (E2M1 / E2M2 values have at most two mantissa bits).  Half the shared-memory
//     traffic and bank passes of the 8-byte entries, and a 29 KB table, so that two CTAs fit an SM;
//   * the table is built once per format on the host, kept in a device array of the library image, and
//     each CTA stages it into shared memory with ONE bulk async copy (cp.async.bulk + mbarrier) instead
//     of rebuilding it from thresholds;
//   * the two halves of a half2 are two ELEMENTS, not two candidates: one PRMT builds (c_i(x0), c_i(x1))
//     from the two elements' entries, the candidate's -t_i*l1 is a per-block constant, and
//       r = fma(c, -t*l1, |x|)   e = r*r (fp16)   acc_i += e (fp32)
//     need no broadcast of |x|;
//   * a thread owns C chunks (8 elements each) of ONE block, chunk g + k*Gt for lane g of the block's Gt
//     lanes: the block maximum, the E5M3 scale and the division constants are computed once per C chunks,
//     and every warp load / store still covers whole 32-byte sectors.
// Results are bit-identical to the reference's eager fp16 quantizer (golden vectors + oracle tests).
#include "quantize_tab.cuh"
#include <mutex>
#include <string.h>

namespace hbq {

constexpr int TAB_THREADS = 512;
constexpr int TAB_SLOTS = 32;               // formats that can have a device table at the same time
constexpr int TAB_MAX_ENTRIES = 8192;       // 32 KB per table

// The staged tables.  In host code this name is only a handle for cudaGetSymbolAddress.
static __device__ __align__(128) uint32_t g_tab_slots[TAB_SLOTS][TAB_MAX_ENTRIES];

struct TabArgs {
    const uint4* x;
    const uint4* gate;        // GLU: the tensor to quantise is silu(gate) * x
    uint4* deq;
    hbq_packed_out out;       // SIDE
    const uint32_t* table;    // device address of the format's byte table
    int64_t total_units;      // thread-units of C chunks
    int entries;              // table entries (a multiple of 4)
    uint32_t entry_bytes;     // 4
    uint32_t base2, hi2;      // first / last covered |a| pattern, in both halves
    uint32_t big_l1;
    float inv_ele_max;
    uint32_t nt2[4];          // (-t_i, -t_i) as fp16 pairs
    float tabf[4];            // t_i, for the rare exact sign-of-zero check
    uint16_t rm[8];           // fp16(1 / m) for the eight E5M3 mantissas
    int in_bf16, out_bf16;
    int log2Gt;               // log2(lanes per block)
    int m_lanes, log2m;       // chunks (= lanes) per micro-block
    int l2_sc_bit, nl2, l2_bytes;
};
static_assert(sizeof(TabArgs) <= 4000, "kernel parameters are limited to 4 KB");

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// acc += lo(e); acc += hi(e): fp32 accumulation of two fp16 values, in that order (one rounding each)
__device__ __forceinline__ void acc_pair(float& acc, uint32_t e)
{
    asm("{ .reg .b16 lo, hi;\n mov.b32 {lo, hi}, %1;\n"
        " add.rn.f32.f16 %0, lo, %0;\n add.rn.f32.f16 %0, hi, %0; }"
        : "+f"(acc) : "r"(e));
}
// acc = lo(e) + hi(e), the start of such a sum (lo(e) + 0 is exact)
__device__ __forceinline__ void acc_pair_first(float& acc, uint32_t e)
{
    asm("{ .reg .b16 lo, hi;\n mov.b32 {lo, hi}, %1;\n"
        " add.rn.f32.f16 %0, lo, 0f00000000;\n add.rn.f32.f16 %0, hi, %0; }"
        : "=f"(acc) : "r"(e));
}

// Byte i of both entries as the high bytes of an fp16 pair: (c_i(element 0), c_i(element 1)).  The low
// bytes are filled by sign replication of the (non-negative) value bytes, i.e. with zeros.
__device__ __forceinline__ uint32_t cand_pair(uint32_t e0, uint32_t e1, int i)
{
    return prmt(e0, e1, ((4u + i) << 12) | ((0xCu + i) << 8) | ((uint32_t)i << 4) | (8u + i));
}

// One 8-element chunk (x: its values as fp16 pairs; only |x| is used): every candidate's squared-error sum.
// SMALL: value * t * l1 cannot overflow fp16 for this block, so fma(c, -t*l1, |x|) equals the reference's
// fp16(|x| - fp16(fp16(c*t)*l1)) (both products are exact).  Otherwise the product keeps its own rounding.
template <bool SMALL>
__device__ __forceinline__ void chunk_errors(const uint32_t* ent, const uint32_t* x, const uint32_t* tl, const uint32_t* nt2,
                                             uint32_t l1u, float* acc)
{
    #pragma unroll
    for (int p = 0; p < 4; ++p) {
        #pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 c = bits_h2(cand_pair(ent[2 * p], ent[2 * p + 1], i));
            __half2 r;
            if (SMALL) r = __hfma2(c, bits_h2(tl[i]), __habs2(bits_h2(x[p])));
            else r = __hadd2(__habs2(bits_h2(x[p])), __hmul2(__hmul2(c, bits_h2(nt2[i])), bits_h2(l1u)));
            if (p == 0) acc_pair_first(acc[i], h2_bits(__hmul2(r, r)));
            else acc_pair(acc[i], h2_bits(__hmul2(r, r)));
        }
    }
}

// First minimum among four non-negative fp16 values given as fp32 sums: the sums are rounded to fp16 (as the
// reference rounds them), and since non-negative fp16 patterns order like integers, pattern * 4 + index is a
// key whose minimum is the first minimum.
__device__ __forceinline__ int first_min4(const float* acc)
{
    const uint32_t E01 = h2_bits(__floats2half2_rn(acc[0], acc[1])), E23 = h2_bits(__floats2half2_rn(acc[2], acc[3]));
    const uint32_t k0 = (E01 & 0xFFFFu) * 4u, k1 = (E01 >> 16) * 4u + 1u;
    const uint32_t k2 = (E23 & 0xFFFFu) * 4u + 2u, k3 = (E23 >> 16) * 4u + 3u;
    return (int)(min(min(k0, k1), min(k2, k3)) & 3u);
}

// The C chunks of one thread-unit, after the block scale is known.  SMALL: see chunk_errors (warp-uniform).
// On return xb[k] holds chunk k's fake-quantised values (fp16 pairs with the inputs' signs), `bests` the chosen
// candidate of every chunk (2 bits each) and the return value is the packed minimum of all quotients a.
// The reference returns +0 (not -0) when fp16(a / t) is exactly zero; only quotients a below 2^-19 can do
// that, and deciding it needs the exact a (the scaled division may be off down there), so it is a rare slow
// path.  TINY = 0: the caller runs it (from the returned minimum, re-reading its inputs); 1: it runs here, per
// chunk, before the inputs are overwritten; 2: the inputs are non-negative, the rule cannot apply.
template <int MB, int C, int ML, bool SMALL, bool SIDE, int TINY>
__device__ __forceinline__ uint32_t unit_chunks(const TabArgs& a, const uint32_t tab_addr, const uint32_t* s_nt2,
                                                 const float* s_tabf, uint32_t (*xb)[4], uint32_t l1b, const uint4 cst,
                                                 int m_lanes, uint32_t& bests, uint32_t (*cwout)[4])
{
    const __half2 pre2 = bits_h2(cst.x), post2 = bits_h2(cst.y), nm2 = bits_h2(cst.z), rm2 = bits_h2(cst.w);
    const uint32_t l1u = l1b * 0x00010001u;
    uint32_t tl[4];                                         // (-t_i * l1) pairs; exact products (SMALL only)
    #pragma unroll
    for (int i = 0; i < 4; ++i) tl[i] = h2_bits(__hmul2(bits_h2(l1u), bits_h2(a.nt2[i])));
    uint32_t amin = 0x7C007C00u;
    bests = 0u;
    // byte address of entry (pattern): tab_addr + 4 * (pattern - base)
    const uint32_t addr0 = tab_addr - 4u * (a.base2 & 0xFFFFu);
    #pragma unroll
    for (int k = 0; k < C; ++k) {
        uint32_t ent[8], av[TINY == 1 ? 4 : 1];
        #pragma unroll
        for (int p = 0; p < 4; ++p) {
            // a = fp16(|x| / l1) by the pre-scaled Markstein division (exact for every quotient >= 2^-14)
            const __half2 axs = __hmul2(__habs2(bits_h2(xb[k][p])), pre2);
            const __half2 q0 = __hmul2(axs, rm2);
            const __half2 r = __hfma2(q0, nm2, axs);
            const __half2 q1 = __hfma2(r, rm2, q0);
            const __half2 aa = __hmul2(q1, post2);
            if (TINY == 0) amin = h2_bits(__hmin2(bits_h2(amin), aa));
            if (TINY == 1) av[p] = h2_bits(aa);
            const uint32_t w = h2_bits(__hmin2(__hmax2(aa, bits_h2(a.base2)), bits_h2(a.hi2)));
            uint32_t e0, e1;
            // entry address = pattern * 4 + addr0; the 4 is a kernel argument so that the scaling stays one
            // multiply-add on the (full-rate) FMA pipe instead of shifts on the half-rate ALU pipe
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(e0) : "r"((w & 0xFFFFu) * a.entry_bytes + addr0));
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(e1) : "r"((w >> 16) * a.entry_bytes + addr0));
            ent[2 * p] = e0; ent[2 * p + 1] = e1;
        }
        float acc[4];
        chunk_errors<SMALL>(ent, xb[k], tl, a.nt2, l1u, acc);
        if (ML > 0) {
            #pragma unroll
            for (int off = ML >> 1; off >= 1; off >>= 1) {
                #pragma unroll
                for (int i = 0; i < 4; ++i) acc[i] += __shfl_xor_sync(0xFFFFFFFFu, acc[i], off);
            }
        } else {
            for (int off = m_lanes >> 1; off >= 1; off >>= 1) {
                #pragma unroll
                for (int i = 0; i < 4; ++i) acc[i] += __shfl_xor_sync(0xFFFFFFFFu, acc[i], off);
            }
        }
        const int best = first_min4(acc);
        bests |= (uint32_t)best << (2 * k);
        // the winner's values with the inputs' signs
        const uint32_t wsel = 0x4C08u + (uint32_t)best * 0x1111u;
        const uint32_t ntb = s_nt2[best];
        const __half2 tlb = __hmul2(bits_h2(l1u), bits_h2(ntb));
        uint32_t dq[4];
        #pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint32_t cw = prmt(ent[2 * p], ent[2 * p + 1], wsel);
            if (SIDE) cwout[k][p] = cw;
            const __half2 dneg = SMALL ? __hmul2(bits_h2(cw), tlb)
                                       : __hmul2(__hmul2(bits_h2(cw), bits_h2(ntb)), bits_h2(l1u));
            dq[p] = (h2_bits(dneg) & 0x7FFF7FFFu) | (xb[k][p] & 0x80008000u);
        }
        if (TINY == 1) {
            const __half2 am = __hmin2(__hmin2(bits_h2(av[0]), bits_h2(av[1])), __hmin2(bits_h2(av[2]), bits_h2(av[3])));
            if (__hle2_mask(am, bits_h2(0x00200020u)) != 0u) {
                const float l1f = __half2float(bits_h((uint16_t)l1b)), tc = s_tabf[best];
                #pragma unroll
                for (int p = 0; p < 4; ++p)
                    #pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t xbits = (xb[k][p] >> (16 * h)) & 0xFFFFu;
                        if ((xbits & 0x8000u) && ((av[p] >> (16 * h)) & 0xFFFFu) <= 0x0020u) {
                            const float xf = __half2float(bits_h((uint16_t)(xbits & 0x7FFFu)));
                            if (rh(__fdiv_rn(rh(__fdiv_rn(xf, l1f)), tc)) == 0.f) dq[p] &= ~(0x8000u << (16 * h));
                        }
                    }
            }
        }
        #pragma unroll
        for (int p = 0; p < 4; ++p) xb[k][p] = dq[p];
    }
    return amin;
}

// Stage a format's tables into shared memory; every thread of the CTA calls it.  The candidate table comes
// by ONE bulk async copy whose completion is counted on an mbarrier, with a bounded wait: if the copy has not
// landed by then, every thread loads the table with plain loads (the same values, so a late completion of the
// copy is harmless).  Returns the shared-memory address of the table.
__device__ __forceinline__ uint32_t stage_table(const TabArgs& a, uint32_t* s_tab, uint4* s_l1c, unsigned long long* s_bar,
                                                 uint32_t* s_nt2, float* s_tabf, int nthreads)
{
    const int tid = threadIdx.x;
    if (tid < 4) { s_nt2[tid] = a.nt2[tid]; s_tabf[tid] = a.tabf[tid]; }
    const uint32_t bar = smem_addr(s_bar), dst = smem_addr(s_tab);
    const uint32_t bytes = (uint32_t)a.entries * 4u;
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (tid == 0) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(dst), "l"(a.table), "r"(bytes), "r"(bar) : "memory");
    }
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
    bool landed = false;
    #pragma unroll 1
    for (int it = 0; it < (1 << 20) && !landed; ++it) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], 0;\n selp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(bar) : "memory");
        landed = ok != 0;
    }
    if (!__syncthreads_and(landed ? 1 : 0)) {
        const uint4* src = reinterpret_cast<const uint4*>(a.table);
        uint4* d4 = reinterpret_cast<uint4*>(s_tab);
        for (int i = tid; i < a.entries / 4; i += nthreads) d4[i] = __ldg(src + i);
        __syncthreads();
    }
    return dst;
}

// The block scale of a thread-unit whose C chunks are in xb: the maximum over the block's GT lanes, then the
// E5M3 scale (round-half-up of the 3-bit mantissa).  Returns the scale's fp16 pattern.
template <int C>
__device__ __forceinline__ uint32_t unit_scale(const uint32_t (*xb)[4], int Gt, float inv_ele_max)
{
    uint32_t mx = 0u;
    #pragma unroll
    for (int k = 0; k < C; ++k)
        #pragma unroll
        for (int p = 0; p < 4; ++p) mx = h2_bits(__hmax2(bits_h2(mx), __habs2(bits_h2(xb[k][p]))));
    for (int off = Gt >> 1; off >= 1; off >>= 1)
        mx = h2_bits(__hmax2(bits_h2(mx), bits_h2(__shfl_xor_sync(0xFFFFFFFFu, mx, off))));
    const uint32_t am16 = max(mx & 0xFFFFu, mx >> 16);
    const float sf = __half2float(bits_h((uint16_t)am16)) * inv_ele_max;
    uint32_t sb = (uint32_t)h_bits(__float2half_rn(sf));
    sb = min(max(sb, 0x0400u), 0x7B80u);
    return (sb + 0x40u) & 0xFF80u;
}

// GT / ML: lanes per block / per micro-block as compile-time constants (0: read from the arguments).
template <int MB, int C, int GT, int ML, bool SIDE, bool GLU>
__global__ void __launch_bounds__(TAB_THREADS, 2) hbq_tab_kernel(const TabArgs a)
{
    extern __shared__ __align__(128) uint32_t s_tab[];
    __shared__ uint4 s_l1c[256];             // per E5M3 scale (pattern >> 7): {2^s1, 2^-(s1+e), -m, fp16(1/m)} as fp16 pairs
    __shared__ __align__(8) unsigned long long s_bar;
    __shared__ uint32_t s_nt2[4];            // the candidates, where a run-time index can reach them
    __shared__ float s_tabf[4];
    const int tid = threadIdx.x, lane = tid & 31;
    const uint32_t dst = stage_table(a, s_tab, s_l1c, &s_bar, s_nt2, s_tabf, TAB_THREADS);

    const int log2Gt = GT > 0 ? (GT == 1 ? 0 : GT == 2 ? 1 : GT == 4 ? 2 : GT == 8 ? 3 : GT == 16 ? 4 : 5) : a.log2Gt;
    const int Gt = 1 << log2Gt;
    const int64_t stride = (int64_t)gridDim.x * TAB_THREADS;

    // raw loads of a thread-unit (zeros beyond the end)
    auto load_unit = [&](int64_t uu, uint4* rx, uint4* rg) {
        const bool ok = uu < a.total_units;
        const int64_t cc = (uu >> log2Gt) * (int64_t)(C * Gt) + ((int)uu & (Gt - 1));
        #pragma unroll
        for (int k = 0; k < C; ++k) {
            rx[k] = make_uint4(0u, 0u, 0u, 0u);
            if (ok) rx[k] = __ldg(a.x + cc + k * Gt);
            if (GLU) {
                rg[k] = make_uint4(0u, 0u, 0u, 0u);
                if (ok) rg[k] = __ldg(a.gate + cc + k * Gt);
            }
        }
    };
    #pragma unroll 1
    for (int64_t u = (int64_t)blockIdx.x * TAB_THREADS + tid; u - lane < a.total_units; u += stride) {
        const bool valid = u < a.total_units;
        const int64_t bi = u >> log2Gt;                         // block index (flat over rows)
        const int g = (int)u & (Gt - 1);                        // lane of the block
        const int64_t c0 = bi * (int64_t)(C * Gt) + g;          // chunk k of this thread: c0 + k * Gt

        // ---- the thread's C chunks ----
        uint4 rx[C], rg[GLU ? C : 1];
        load_unit(u, rx, rg);
        uint32_t xb[C][4];
        #pragma unroll
        for (int k = 0; k < C; ++k) {
            xb[k][0] = rx[k].x; xb[k][1] = rx[k].y; xb[k][2] = rx[k].z; xb[k][3] = rx[k].w;
            if (GLU) {
                const uint32_t gb[4] = {rg[k].x, rg[k].y, rg[k].z, rg[k].w};
                #pragma unroll
                for (int p = 0; p < 4; ++p) {
                    const float2 gg = __half22float2(bits_h2(gb[p])), uu = __half22float2(bits_h2(xb[k][p]));
                    const float s0 = rh(__fdiv_rn(gg.x, 1.f + expf(-gg.x))), s1 = rh(__fdiv_rn(gg.y, 1.f + expf(-gg.y)));
                    xb[k][p] = h2_bits(__floats2half2_rn(s0 * uu.x, s1 * uu.y));      // fp16 x fp16 is exact in fp32
                }
            }
        }
        if (a.in_bf16) {
            #pragma unroll
            for (int k = 0; k < C; ++k)
                #pragma unroll
                for (int p = 0; p < 4; ++p)
                    xb[k][p] = h2_bits(__floats2half2_rn(__uint_as_float(xb[k][p] << 16), __uint_as_float(xb[k][p] & 0xFFFF0000u)));
        }

        // ---- block maximum and the E5M3 shared scale (round-half-up of the 3-bit mantissa) ----
        uint32_t mx = 0u;
        #pragma unroll
        for (int k = 0; k < C; ++k)
            #pragma unroll
            for (int p = 0; p < 4; ++p) mx = h2_bits(__hmax2(bits_h2(mx), __habs2(bits_h2(xb[k][p]))));
        if (GT > 0) {
            #pragma unroll
            for (int off = GT >> 1; off >= 1; off >>= 1)
                mx = h2_bits(__hmax2(bits_h2(mx), bits_h2(__shfl_xor_sync(0xFFFFFFFFu, mx, off))));
        } else {
            for (int off = Gt >> 1; off >= 1; off >>= 1)
                mx = h2_bits(__hmax2(bits_h2(mx), bits_h2(__shfl_xor_sync(0xFFFFFFFFu, mx, off))));
        }
        const uint32_t am16 = max(mx & 0xFFFFu, mx >> 16);
        const float sf = __half2float(bits_h((uint16_t)am16)) * a.inv_ele_max;
        uint32_t sb = (uint32_t)h_bits(__float2half_rn(sf));
        sb = min(max(sb, 0x0400u), 0x7B80u);
        const uint32_t l1b = (sb + 0x40u) & 0xFF80u;
        const uint4 cst = s_l1c[l1b >> 7];

        // ---- the chunks: candidates' errors, choice, values ----
        uint32_t bests, amin;
        uint32_t cw[SIDE ? C : 1][4];
        // value * t * l1 overflows fp16 only for blocks whose maximum is within 1 % of fp16's own: one
        // warp-uniform branch between the fused form and the form that keeps each product's rounding
        if (__all_sync(0xFFFFFFFFu, l1b < a.big_l1)) amin = unit_chunks<MB, C, ML, true, SIDE, 0>(a, dst, s_nt2, s_tabf, xb, l1b, cst, a.m_lanes, bests, cw);
        else amin = unit_chunks<MB, C, ML, false, SIDE, 0>(a, dst, s_nt2, s_tabf, xb, l1b, cst, a.m_lanes, bests, cw);

        // The reference returns +0 (not -0) when fp16(a / t) is exactly zero.  Only quotients a below 2^-19
        // can do that; deciding it needs the exact a, where the scaled division may be off: rare, so the
        // inputs are read again and the quotients redone with true divisions.
        if (__hle2_mask(bits_h2(amin), bits_h2(0x00200020u)) != 0u && valid) {
            const float l1f = __half2float(bits_h((uint16_t)l1b));
            #pragma unroll
            for (int k = 0; k < C; ++k) {                  // unrolled: xb must stay in registers
                const float tc = s_tabf[(bests >> (2 * k)) & 3u];
                uint4 raw = __ldg(a.x + c0 + k * Gt);
                uint32_t xr[4] = {raw.x, raw.y, raw.z, raw.w};
                if (GLU) {
                    const uint4 graw = __ldg(a.gate + c0 + k * Gt);
                    const uint32_t gb[4] = {graw.x, graw.y, graw.z, graw.w};
                    for (int p = 0; p < 4; ++p) {
                        const float2 gg = __half22float2(bits_h2(gb[p])), uu = __half22float2(bits_h2(xr[p]));
                        const float s0 = rh(__fdiv_rn(gg.x, 1.f + expf(-gg.x))), s1 = rh(__fdiv_rn(gg.y, 1.f + expf(-gg.y)));
                        xr[p] = h2_bits(__floats2half2_rn(s0 * uu.x, s1 * uu.y));
                    }
                }
                if (a.in_bf16)
                    for (int p = 0; p < 4; ++p)
                        xr[p] = h2_bits(__floats2half2_rn(__uint_as_float(xr[p] << 16), __uint_as_float(xr[p] & 0xFFFF0000u)));
                #pragma unroll
                for (int p = 0; p < 4; ++p)
                    #pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t xbits = (xr[p] >> (16 * h)) & 0xFFFFu;
                        if (xbits & 0x8000u) {
                            const float xf = __half2float(bits_h((uint16_t)(xbits & 0x7FFFu)));
                            if (rh(__fdiv_rn(rh(__fdiv_rn(xf, l1f)), tc)) == 0.f) xb[k][p] &= ~(0x8000u << (16 * h));
                        }
                    }
            }
        }

        // ---- stores ----
        uint32_t l2word = 0u;
        #pragma unroll
        for (int k = 0; k < C; ++k) {
            const int64_t ci = c0 + k * Gt;
            if (SIDE) {
                const int best = (int)((bests >> (2 * k)) & 3u);
                const int cib = g + k * Gt;                      // chunk index inside the block
                const int mbi = cib >> a.log2m;                  // its micro-block
                const bool leader = (g & (a.m_lanes - 1)) == 0;
                if (valid && a.out.codes) {
                    uint32_t wcode = 0u, sbits = 0u;
                    #pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        const uint32_t mag = code2_e2<MB>(bits_h2(cw[k][p]));
                        uint32_t lo = mag & 0xFFFFu, hi = mag >> 16;
                        const uint32_t slo = (xb[k][p] >> 15) & 1u, shi = xb[k][p] >> 31;
                        if (MB == 1) { lo |= slo << 3; hi |= shi << 3; }
                        wcode |= ((lo & 0xFu) | ((hi & 0xFu) << 4)) << (8 * p);
                        sbits |= (slo | (shi << 1)) << (2 * p);
                    }
                    reinterpret_cast<uint32_t*>(a.out.codes)[ci] = wcode;
                    if (MB == 2 && a.out.sign) a.out.sign[ci] = (uint8_t)sbits;
                }
                if (leader) {
                    if (a.out.l2_packed) l2word |= (uint32_t)best << (mbi * a.l2_sc_bit);
                    if (valid && a.out.l2_idx) a.out.l2_idx[bi * a.nl2 + mbi] = (uint8_t)best;
                }
            }
            if (valid) {
                uint32_t dq[4] = {xb[k][0], xb[k][1], xb[k][2], xb[k][3]};
                if (a.out_bf16) {
                    #pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        const float2 f = __half22float2(bits_h2(dq[p]));
                        __nv_bfloat162 bb = __floats2bfloat162_rn(f.x, f.y);
                        dq[p] = *reinterpret_cast<uint32_t*>(&bb);
                    }
                }
                a.deq[ci] = make_uint4(dq[0], dq[1], dq[2], dq[3]);
            }
        }
        if (SIDE) {
            if (a.out.l2_packed) l2word = group_or(l2word, Gt);
            if (valid && g == 0) {
                if (a.out.scale_h) a.out.scale_h[bi] = (uint16_t)l1b;
                if (a.out.scale_u8) a.out.scale_u8[bi] = (uint8_t)(l1b >> 7);
                if (a.out.scheme) a.out.scheme[bi] = 0;
                if (a.out.l2_packed) {
                    uint8_t* lp = a.out.l2_packed + bi * a.l2_bytes;
                    if (a.l2_bytes == 4) *reinterpret_cast<uint32_t*>(lp) = l2word;
                    else if (a.l2_bytes == 2) *reinterpret_cast<uint16_t*>(lp) = (uint16_t)l2word;
                    else *lp = (uint8_t)l2word;
                }
            }
        }
    }
}


// ---- row kernels: a per-row prologue fused in front of the quantizer --------------------------------
// Two activation quantizers of the attention / MLP blocks consume a tensor that only exists to be quantised
// and whose producer needs a whole-row reduction first:
//   RMSNORM  the input of q/k/v_proj and gate/up_proj: aq(weight * rmsnorm(x [+ residual])) (the decoder
//            layer's input_layernorm / post_attention_layernorm followed by _QBaseLinear.forward's
//            self.aq(x), src/module.py:45); the sum x + residual is also written (the new residual stream);
//   SOFTMAX  the attention probabilities: attn_wgt_quantizer.q(softmax(q k^T * scale + bias)) along the key
//            axis (manual_sdpa, src/module.py:108-115).
// One warp owns a row.  It sweeps the row for the reduction (sum of squares; maximum, then sum of exponentials),
// then sweeps it again (from L1 / L2) to form the fp16 values with the reference's per-op roundings and hands
// each 128-element block straight to the table quantizer above -- the normalised tensor / the probabilities
// never go to HBM unquantised.  Geometry: blocks of 128, four lanes per block, four chunks per lane.
enum { ROW_RMSNORM = 0, ROW_SOFTMAX = 1 };
constexpr int ROW_THREADS = 512;
constexpr int ROW_WARPS = ROW_THREADS / 32;

struct RowArgs {
    TabArgs t;                // the quantizer's format (table, candidates); t.x / t.deq unused
    const uint4* in;          // [rows, K] fp16: x (RMSNORM) or the raw scores q k^T (SOFTMAX)
    uint4* out;               // [rows, K] fp16
    int64_t rows;
    int K, nblk;              // row length, 128-element blocks per row
    // RMSNORM
    const uint4* res;         // residual to add first, or NULL
    uint4* x_out;             // where x + residual goes (required with res)
    const uint4* w;           // weight [K] fp16
    float eps;
    // SOFTMAX
    float scale;              // the score scale (a Python float in the reference: applied in fp32)
    int causal;               // key j of query row r is masked when j > (r % L) + key_offset
    int64_t L, HL, key_offset;
    const uint4* mask;        // additive fp16 mask [mask_batches, L, K] or NULL (row r uses batch r / HL, query r % L)
    int64_t mask_batches;
};
static_assert(sizeof(RowArgs) <= 4000, "kernel parameters are limited to 4 KB");

// Reductions over the W lanes that share a row (a whole warp, or one of its halves).
template <int W>
__device__ __forceinline__ float lanes_sum(float v)
{
    #pragma unroll
    for (int off = W / 2; off >= 1; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    return v;
}
template <int W>
__device__ __forceinline__ float lanes_max(float v)
{
    #pragma unroll
    for (int off = W / 2; off >= 1; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
    return v;
}

// -inf into the halves of a packed pair whose key index (j0, j0 + 1) lies beyond the causal limit.
__device__ __forceinline__ uint32_t mask_beyond(uint32_t b, int64_t j0, int64_t limit)
{
    if (j0 > limit) b = (b & 0xFFFF0000u) | 0x0000FC00u;
    if (j0 + 1 > limit) b = (b & 0x0000FFFFu) | 0xFC000000u;
    return b;
}

// The pre-softmax score chunk as the reference's fp16 ops leave it: fp16(fp16(s * scale) + bias), bias = the
// additive mask and / or -inf beyond the causal limit.  cir: chunk index in the row.
__device__ __forceinline__ void score_chunk(const RowArgs& a, const uint4* rin, const uint4* rmask, int cir, int64_t limit,
                                            uint32_t* sv)
{
    const uint4 raw = __ldg(rin + cir);
    const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t m[4] = {0u, 0u, 0u, 0u};
    if (rmask) { const uint4 mv = __ldg(rmask + cir); m[0] = mv.x; m[1] = mv.y; m[2] = mv.z; m[3] = mv.w; }
    #pragma unroll
    for (int p = 0; p < 4; ++p) {
        // tensor * Python scalar: torch multiplies in fp32 with the scalar as fp32 and rounds the product to fp16
        const float2 sf = __half22float2(bits_h2(r[p]));
        __half2 v = __floats2half2_rn(sf.x * a.scale, sf.y * a.scale);
        if (rmask) v = __hadd2(v, bits_h2(m[p]));
        sv[p] = h2_bits(v);
    }
    if ((int64_t)cir * 8 + 7 > limit) {                      // the chunk that holds the causal limit (or lies beyond it)
        #pragma unroll
        for (int p = 0; p < 4; ++p) sv[p] = mask_beyond(sv[p], (int64_t)cir * 8 + 2 * p, limit);
    }
}

// fp32 quotient a / b, correctly rounded, from r = RN(1 / b): first guess, its exact residual, one correction
// (Markstein's sequence).  b is a softmax row sum (>= 1 when finite); NaN and Inf operands end in NaN like a / b.
__device__ __forceinline__ float div_by_sum(float a, float b, float r)
{
    const float q0 = a * r;
    const float rem = fmaf(-q0, b, a);
    return fmaf(rem, r, q0);
}

template <int MB, int ML, int PRO, bool QUANT>
__global__ void __launch_bounds__(ROW_THREADS, 2) hbq_row_kernel(const RowArgs a)
{
    extern __shared__ __align__(128) uint32_t s_tab[];
    __shared__ uint4 s_l1c[256];
    __shared__ __align__(8) unsigned long long s_bar;
    __shared__ uint32_t s_nt2[4];
    __shared__ float s_tabf[4];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t dst = 0u;
    if (QUANT) dst = stage_table(a.t, s_tab, s_l1c, &s_bar, s_nt2, s_tabf, ROW_THREADS);
    // RMSNorm: one row per warp, 8 blocks (1024 elements) per iteration.  Softmax: one row per half-warp, 4 blocks
    // per iteration -- a causal row ends anywhere, and the masked blocks of its last iteration are lanes without
    // work (1.5 blocks on average instead of 3.5).
    constexpr int RPW = PRO == ROW_SOFTMAX ? 2 : 1;          // rows per warp
    constexpr int BPI = 8 / RPW;                             // blocks of a row per iteration
    constexpr int RL = 32 / RPW;                             // lanes of a row
    const int sub = lane / RL;
    const int bl = (lane >> 2) & (BPI - 1), g = lane & 3;    // block of the iteration, lane of the block
    const int cpr = a.K >> 3;                                // chunks per row
    const int iters_all = (a.nblk + BPI - 1) / BPI;

    #pragma unroll 1
    for (int64_t rb = ((int64_t)blockIdx.x * ROW_WARPS + warp) * RPW; rb < a.rows; rb += (int64_t)gridDim.x * ROW_WARPS * RPW) {
        int64_t row = rb + sub;
        const bool live = row < a.rows;                      // odd row count: the idle half repeats the last row, stores nothing
        if (!live) row = a.rows - 1;
        const uint4* rin = a.in + row * cpr;
        uint4* rout = a.out + row * cpr;
        float stat0 = 0.f, stat1 = 0.f;                      // RMSNORM: rstd; SOFTMAX: max, sum
        int iters = iters_all;
        int64_t limit = (int64_t)a.K;                        // SOFTMAX: last unmasked key
        const uint4* rmask = nullptr;
        const uint4* rsrc = rin;                             // what the second sweep reads

        if (PRO == ROW_RMSNORM) {
            float ss = 0.f;
            uint4* rx = a.x_out ? a.x_out + row * cpr : nullptr;
            const uint4* rres = a.res ? a.res + row * cpr : nullptr;
            if (rres) rsrc = rx;
            for (int it = 0; it < iters; ++it) {
                const int blk = it * BPI + bl;
                if (blk < a.nblk) {
                    #pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int ci = blk * 16 + g + 4 * k;
                        if (ci >= cpr) continue;                 // ragged last block (unquantised form only)
                        uint4 v = __ldg(rin + ci);
                        if (rres) {
                            const uint4 rv = __ldg(rres + ci);
                            v.x = h2_bits(__hadd2(bits_h2(v.x), bits_h2(rv.x))); v.y = h2_bits(__hadd2(bits_h2(v.y), bits_h2(rv.y)));
                            v.z = h2_bits(__hadd2(bits_h2(v.z), bits_h2(rv.z))); v.w = h2_bits(__hadd2(bits_h2(v.w), bits_h2(rv.w)));
                            rx[ci] = v;
                        }
                        const uint32_t q[4] = {v.x, v.y, v.z, v.w};
                        #pragma unroll
                        for (int p = 0; p < 4; ++p) {
                            const float2 f = __half22float2(bits_h2(q[p]));
                            ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss);
                        }
                    }
                }
            }
            ss = lanes_sum<32>(ss);
            stat0 = rsqrtf(ss / (float)a.K + a.eps);
        } else {
            const int64_t qpos = row % a.L;
            if (a.causal) limit = qpos + a.key_offset;
            if (limit > (int64_t)a.K - 1) limit = (int64_t)a.K - 1;
            if (a.mask) rmask = a.mask + ((a.mask_batches > 1 ? row / a.HL : 0) * a.L + qpos) * cpr;
            // whole iterations beyond the causal limit hold only masked keys: probabilities 0
            iters = min(iters_all, (int)(limit / (128 * BPI)) + 1);
            float mx = -INFINITY;
            if (!rmask && a.scale > 0.f) {
                // rounding is monotonic, so the largest scaled score is the scaled largest score: one max per pair
                __half2 m2 = bits_h2(0xFC00FC00u);
                for (int it = 0; it < iters; ++it) {
                    const int blk = it * BPI + bl;
                    #pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int ci = blk * 16 + g + 4 * k;
                        const int64_t j0 = (int64_t)ci * 8;
                        if (ci >= cpr || j0 > limit) continue;
                        const uint4 raw = __ldg(rin + ci);
                        uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
                        if (j0 + 7 > limit) {
                            #pragma unroll
                            for (int p = 0; p < 4; ++p) r[p] = mask_beyond(r[p], j0 + 2 * p, limit);
                        }
                        m2 = __hmax2(m2, __hmax2(__hmax2(bits_h2(r[0]), bits_h2(r[1])), __hmax2(bits_h2(r[2]), bits_h2(r[3]))));
                    }
                }
                mx = lanes_max<RL>(fmaxf(__low2float(m2), __high2float(m2)));
                mx = __half2float(__float2half_rn(mx * a.scale));
            } else {
                for (int it = 0; it < iters; ++it) {
                    const int blk = it * BPI + bl;
                    #pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        uint32_t sv[4];
                        const int ci = blk * 16 + g + 4 * k;
                        if (ci >= cpr) continue;
                        score_chunk(a, rin, rmask, ci, limit, sv);
                        const __half2 m2 = __hmax2(__hmax2(bits_h2(sv[0]), bits_h2(sv[1])), __hmax2(bits_h2(sv[2]), bits_h2(sv[3])));
                        mx = fmaxf(mx, fmaxf(__low2float(m2), __high2float(m2)));
                    }
                }
                mx = lanes_max<RL>(mx);
            }
            float sum = 0.f;
            for (int it = 0; it < iters; ++it) {
                const int blk = it * BPI + bl;
                #pragma unroll
                for (int k = 0; k < 4; ++k) {
                    uint32_t sv[4];
                    const int ci = blk * 16 + g + 4 * k;
                    if (ci >= cpr || (int64_t)ci * 8 > limit) continue;      // masked keys add exp(-inf) = 0
                    score_chunk(a, rin, rmask, ci, limit, sv);
                    #pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        const float2 f = __half22float2(bits_h2(sv[p]));
                        sum += expf(f.x - mx); sum += expf(f.y - mx);
                    }
                }
            }
            __syncwarp();
            stat0 = mx;
            stat1 = lanes_sum<RL>(sum);
        }

        // ---- second sweep: the fp16 values, block by block into the quantizer ----
        int iters_w = iters;                                 // the quantizer's shuffles need the whole warp in every iteration
        float rsum = 0.f;
        if (PRO == ROW_SOFTMAX) {
            iters_w = max(iters, __shfl_xor_sync(0xFFFFFFFFu, iters, 16));
            rsum = __frcp_rn(stat1);
        }
        for (int it = 0; it < iters_all; ++it) {
            const int blk = it * BPI + bl;
            const bool valid = blk < a.nblk && live;
            if (PRO == ROW_SOFTMAX && it >= iters_w) {       // only masked keys: zeros (warp-uniform branch)
                if (valid) {
                    #pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (blk * 16 + g + 4 * k < cpr) rout[blk * 16 + g + 4 * k] = make_uint4(0u, 0u, 0u, 0u);
                }
                continue;
            }
            uint32_t xb[4][4];
            #pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int ci = blk * 16 + g + 4 * k;
                #pragma unroll
                for (int p = 0; p < 4; ++p) xb[k][p] = 0u;
                if (blk >= a.nblk || ci >= cpr) continue;
                if (PRO == ROW_RMSNORM) {
                    // weight * fp16(x_f32 * rstd): the rounding points of transformers' LlamaRMSNorm on an fp16 tensor
                    const uint4 v = a.res ? rsrc[ci] : __ldg(rsrc + ci), wv = __ldg(a.w + ci);
                    const uint32_t q[4] = {v.x, v.y, v.z, v.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
                    #pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        const float2 f = __half22float2(bits_h2(q[p]));
                        xb[k][p] = h2_bits(__hmul2(bits_h2(ww[p]), __floats2half2_rn(f.x * stat0, f.y * stat0)));
                    }
                } else {
                    if ((int64_t)ci * 8 > limit) continue;   // masked keys: exp(-inf) / sum = 0
                    uint32_t sv[4];
                    score_chunk(a, rin, rmask, ci, limit, sv);
                    #pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        const float2 f = __half22float2(bits_h2(sv[p]));
                        xb[k][p] = h2_bits(__floats2half2_rn(div_by_sum(expf(f.x - stat0), stat1, rsum),
                                                             div_by_sum(expf(f.y - stat0), stat1, rsum)));
                    }
                }
            }
            if (QUANT) {
                const uint32_t l1b = unit_scale<4>(xb, 4, a.t.inv_ele_max);
                const uint4 cst = s_l1c[l1b >> 7];
                uint32_t bests;
                uint32_t cw[1][4];
                constexpr int TINY = PRO == ROW_SOFTMAX ? 2 : 1;
                if (__all_sync(0xFFFFFFFFu, l1b < a.t.big_l1)) unit_chunks<MB, 4, ML, true, false, TINY>(a.t, dst, s_nt2, s_tabf, xb, l1b, cst, ML, bests, cw);
                else unit_chunks<MB, 4, ML, false, false, TINY>(a.t, dst, s_nt2, s_tabf, xb, l1b, cst, ML, bests, cw);
            }
            if (valid) {
                #pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (blk * 16 + g + 4 * k < cpr) rout[blk * 16 + g + 4 * k] = make_uint4(xb[k][0], xb[k][1], xb[k][2], xb[k][3]);
            }
        }
    }
}

// ---- host side ------------------------------------------------------------------------------------
static std::mutex g_tab_mutex;
static uint32_t* g_tab_dev[kMaxDevices];                 // device address of g_tab_slots, per device
static bool g_tab_ready[kMaxDevices][TAB_SLOTS];         // the slot holds its format's table on that device

// Device address of the format's table on the current device, uploading it at the first use there.  The
// upload is followed by a stream synchronisation (once per format and device), so it cannot happen while
// the stream is being captured: *addr stays NULL then and the caller takes another kernel.
static int table_on_device(const TabTable& t, cudaStream_t stream, const uint32_t** addr)
{
    *addr = nullptr;
    int dev = 0;
    HBQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return HBQ_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(g_tab_mutex);
    if (!g_tab_ready[dev][t.slot]) {
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess) { (void)cudaGetLastError(); return HBQ_OK; }
        if (cs != cudaStreamCaptureStatusNone) return HBQ_OK;
        if (!g_tab_dev[dev]) {
            void* p = nullptr;
            HBQ_CUDA_TRY(cudaGetSymbolAddress(&p, g_tab_slots));
            g_tab_dev[dev] = (uint32_t*)p;
        }
        HBQ_CUDA_TRY(cudaMemcpyAsync(g_tab_dev[dev] + (size_t)t.slot * TAB_MAX_ENTRIES, t.host, (size_t)t.entries * 4,
                                     cudaMemcpyHostToDevice, stream));
        HBQ_CUDA_TRY(cudaStreamSynchronize(stream));
        g_tab_ready[dev][t.slot] = true;
    }
    *addr = g_tab_dev[dev] + (size_t)t.slot * TAB_MAX_ENTRIES;
    return HBQ_OK;
}

template <int MB, int C, int GT, int ML, bool SIDE, bool GLU>
static int launch_tab(const TabArgs& a, size_t smem, cudaStream_t stream)
{
    int sms = 0, per_sm = 0;
    { const int rc = device_sms(&sms); if (rc) return rc; }
    { const int rc = ensure_dynamic_smem(hbq_tab_kernel<MB, C, GT, ML, SIDE, GLU>, smem); if (rc) return rc; }
    { const int rc = resident_ctas(hbq_tab_kernel<MB, C, GT, ML, SIDE, GLU>, TAB_THREADS, smem, &per_sm); if (rc) return rc; }
    const int64_t need = (a.total_units + TAB_THREADS - 1) / TAB_THREADS;
    const int64_t cap = (int64_t)sms * per_sm;
    const int grid = (int)(need < cap ? need : cap);
    hbq_tab_kernel<MB, C, GT, ML, SIDE, GLU><<<grid, TAB_THREADS, smem, stream>>>(a);
    HBQ_LAUNCH_CHECK("hbq_tab_kernel");
    return HBQ_OK;
}

template <int MB, int C, int GT, int ML>
static int launch_tab_variant(const TabArgs& a, bool side, bool glu, size_t smem, cudaStream_t stream)
{
    if (glu) return launch_tab<MB, C, GT, ML, false, true>(a, smem, stream);
    if (side) return launch_tab<MB, C, GT, ML, true, false>(a, smem, stream);
    return launch_tab<MB, C, GT, ML, false, false>(a, smem, stream);
}

// The shipped configurations (block 128: 4 chunks per thread, 4 lanes per block; micro-block 8 or 32) have
// their lane counts compiled in; every other geometry runs the same kernel with run-time loop bounds.
template <int MB>
static int launch_tab_geometry(const TabArgs& a, int C, int Gt, int m, bool side, bool glu, size_t smem, cudaStream_t stream)
{
    if (C == 4 && Gt == 4 && m == 1) return launch_tab_variant<MB, 4, 4, 1>(a, side, glu, smem, stream);
    if (C == 4 && Gt == 4 && m == 4) return launch_tab_variant<MB, 4, 4, 4>(a, side, glu, smem, stream);
    if (C == 4) return launch_tab_variant<MB, 4, 0, 0>(a, side, glu, smem, stream);
    return launch_tab_variant<MB, 2, 0, 0>(a, side, glu, smem, stream);
}

// Fill the format part of the arguments shared by every kernel of this file (table on the device, candidates,
// scale constants).  *ok = false when the format has no byte table or its table cannot be uploaded now.
static int fill_format(const QArgs& q, int mb, cudaStream_t stream, TabArgs* a, bool* ok)
{
    *ok = false;
    TabTable t;
    if (!hbq_tab_table(mb, q.tab[0], q.nc, &t) || t.slot >= TAB_SLOTS || t.entries > TAB_MAX_ENTRIES) return HBQ_OK;
    memset(a, 0, sizeof(*a));
    { const int rc = table_on_device(t, stream, &a->table); if (rc) return rc; }
    if (!a->table) return HBQ_OK;
    a->entries = t.entries;
    a->entry_bytes = 4u;
    a->base2 = (uint32_t)t.base * 0x00010001u;
    a->hi2 = (uint32_t)t.hi * 0x00010001u;
    a->big_l1 = t.big_l1;
    a->inv_ele_max = 1.f / q.ele_max[0];
    for (int i = 0; i < 4; ++i) {
        const float tv = q.tab[0][i < q.nc ? i : q.nc - 1];     // unused slots repeat the last candidate: they never win a tie
        a->tabf[i] = tv;
        a->nt2[i] = (uint32_t)__half_as_ushort(__float2half_rn(-tv)) * 0x00010001u;
    }
    memcpy(a->rm, t.rm, sizeof(a->rm));
    *ok = true;
    return HBQ_OK;
}

template <int MB, int ML, int PRO>
static int launch_row(const RowArgs& a, bool quant, cudaStream_t stream)
{
    int sms = 0;
    { const int rc = device_sms(&sms); if (rc) return rc; }
    const size_t smem = quant ? (size_t)a.t.entries * 4 : 0;
    const int64_t rows_per_cta = ROW_WARPS * (PRO == ROW_SOFTMAX ? 2 : 1);
    const int64_t need = (a.rows + rows_per_cta - 1) / rows_per_cta;
    const int grid = (int)(need < 2ll * sms ? need : 2ll * sms);
    if (quant) {
        { const int rc = ensure_dynamic_smem(hbq_row_kernel<MB, ML, PRO, true>, smem); if (rc) return rc; }
        hbq_row_kernel<MB, ML, PRO, true><<<grid, ROW_THREADS, smem, stream>>>(a);
    } else {
        hbq_row_kernel<MB, ML, PRO, false><<<grid, ROW_THREADS, 0, stream>>>(a);
    }
    HBQ_LAUNCH_CHECK("hbq_row_kernel");
    return HBQ_OK;
}

// q: the validated HBQ format (QArgs as quantize_launch builds it), or NULL for the prologue alone.  Returns
// HBQ_ERR_UNSUPPORTED when the format does not fit the fused kernel (the caller then runs the prologue alone
// and the plain quantizer).
int hbq_row_launch(int pro, const QArgs* q, int mb, RowArgs& a, cudaStream_t stream)
{
    if (a.rows == 0 || a.K == 0) return HBQ_OK;
    if ((a.K % 8) != 0) return HBQ_ERR_UNSUPPORTED;
    a.nblk = (a.K + 127) / 128;
    bool quant = false;
    int ml = 1;
    if (q) {
        const int L = q->f.l2_block_size;
        if (mb < 1 || mb > 2 || q->nscheme != 1 || q->nc > 4 || !q->scale_fast_e5m3 || q->f.block_size != 128 ||
            (L != 8 && L != 32) || (a.K % 128) != 0)
            return HBQ_ERR_UNSUPPORTED;
        bool ok = false;
        { const int rc = fill_format(*q, mb, stream, &a.t, &ok); if (rc) return rc; }
        if (!ok) return HBQ_ERR_UNSUPPORTED;
        quant = true;
        ml = L / 8;
    }
    #define HBQ_ROW(MBV, MLV)                                                                              \
        return pro == ROW_RMSNORM ? launch_row<MBV, MLV, ROW_RMSNORM>(a, quant, stream)                   \
                                  : launch_row<MBV, MLV, ROW_SOFTMAX>(a, quant, stream);
    if (mb == 1) { if (ml == 4) { HBQ_ROW(1, 4) } else { HBQ_ROW(1, 1) } }
    if (ml == 4) { HBQ_ROW(2, 4) } else { HBQ_ROW(2, 1) }
    #undef HBQ_ROW
}

int hbq_format_qargs(const hbq_format* f, QArgs* a, int* mb);      // quantize.cu

int rmsnorm_quantize_launch(const void* x, const void* residual, const void* weight, float eps, int64_t rows, int64_t K,
                            const hbq_format* fmt, void* x_out, void* out, cudaStream_t stream)
{
    if (rows < 0 || K < 0) return HBQ_ERR_ARG;
    if (rows == 0 || K == 0) return HBQ_OK;
    if (!x || !weight || !out || (residual && !x_out) || K > (1 << 24)) return HBQ_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(weight) |
         reinterpret_cast<uintptr_t>(x_out) | reinterpret_cast<uintptr_t>(out)) & 15)
        return HBQ_ERR_ALIGN;
    RowArgs a;
    memset(&a, 0, sizeof(a));
    a.in = (const uint4*)x; a.out = (uint4*)out; a.rows = rows; a.K = (int)K;
    a.res = (const uint4*)residual; a.x_out = residual ? (uint4*)x_out : nullptr; a.w = (const uint4*)weight; a.eps = eps;
    QArgs q;
    int mb = 0;
    if (fmt) { const int rc = hbq_format_qargs(fmt, &q, &mb); if (rc) return rc; }
    return hbq_row_launch(ROW_RMSNORM, fmt ? &q : nullptr, mb ? mb : 2, a, stream);
}

int softmax_quantize_launch(const void* scores, int64_t rows, int64_t S, int64_t L, int64_t heads, float scale, int causal,
                            const void* mask, int64_t mask_batches, const hbq_format* fmt, void* out, cudaStream_t stream)
{
    if (rows < 0 || S < 0 || L <= 0 || heads <= 0) return HBQ_ERR_ARG;
    if (rows == 0 || S == 0) return HBQ_OK;
    if (!scores || !out || S > (1 << 24) || (mask && mask_batches < 1)) return HBQ_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(scores) | reinterpret_cast<uintptr_t>(mask) | reinterpret_cast<uintptr_t>(out)) & 15)
        return HBQ_ERR_ALIGN;
    RowArgs a;
    memset(&a, 0, sizeof(a));
    a.in = (const uint4*)scores; a.out = (uint4*)out; a.rows = rows; a.K = (int)S;
    a.scale = scale;
    a.causal = causal; a.L = L; a.HL = heads * L; a.key_offset = S - L;
    a.mask = (const uint4*)mask; a.mask_batches = mask_batches;
    QArgs q;
    int mb = 0;
    if (fmt) { const int rc = hbq_format_qargs(fmt, &q, &mb); if (rc) return rc; }
    return hbq_row_launch(ROW_SOFTMAX, fmt ? &q : nullptr, mb ? mb : 2, a, stream);
}

int hbq_tab_try_launch(const QArgs& q, int mb, cudaStream_t stream, bool* launched)
{
    *launched = false;
    if (mb < 1 || mb > 2 || q.nscheme != 1 || q.nc > 4 || !q.scale_fast_e5m3) return HBQ_OK;
    if (!q.deq || !q.aligned || q.K != q.Kp) return HBQ_OK;
    if (q.rope_cos || q.perm_T > 0 || q.k_center) return HBQ_OK;
    const bool side = q.out.codes || q.out.sign || q.out.scale_u8 || q.out.scale_h || q.out.l2_packed || q.out.l2_idx ||
                      q.out.scheme;
    const bool glu = q.glu_gate != nullptr;
    if (glu && (side || q.in_bf16 || q.out_bf16)) return HBQ_OK;
    if ((reinterpret_cast<uintptr_t>(q.out.codes) & 3) || (reinterpret_cast<uintptr_t>(q.out.l2_packed) & 3) ||
        (reinterpret_cast<uintptr_t>(q.out.scale_h) & 1))
        return HBQ_OK;
    const int cpb = q.G, L = q.f.l2_block_size;              // chunks per block, elements per micro-block
    if (L < 8) return HBQ_OK;
    const int m = L / 8;
    int C = 0;
    if (cpb % 4 == 0 && m <= cpb / 4) C = 4;
    else if (cpb % 2 == 0 && m <= cpb / 2) C = 2;
    if (C == 0) return HBQ_OK;
    const int Gt = cpb / C;
    if (Gt > 32 || (Gt & (Gt - 1)) || (m & (m - 1))) return HBQ_OK;

    TabTable t;
    if (!hbq_tab_table(mb, q.tab[0], q.nc, &t) || t.slot >= TAB_SLOTS || t.entries > TAB_MAX_ENTRIES) return HBQ_OK;
    TabArgs a;
    memset(&a, 0, sizeof(a));
    { const int rc = table_on_device(t, stream, &a.table); if (rc) return rc; }
    if (!a.table) return HBQ_OK;

    a.x = reinterpret_cast<const uint4*>(q.x);
    a.gate = reinterpret_cast<const uint4*>(q.glu_gate);
    a.deq = reinterpret_cast<uint4*>(q.deq);
    a.out = q.out;
    a.total_units = q.total_chunks / C;
    a.entries = t.entries;
    a.entry_bytes = 4u;
    a.base2 = (uint32_t)t.base * 0x00010001u;
    a.hi2 = (uint32_t)t.hi * 0x00010001u;
    a.big_l1 = t.big_l1;
    a.inv_ele_max = 1.f / q.ele_max[0];
    for (int i = 0; i < 4; ++i) {
        const float tv = q.tab[0][i < q.nc ? i : q.nc - 1];     // unused slots repeat the last candidate: they never win a tie
        a.tabf[i] = tv;
        a.nt2[i] = (uint32_t)__half_as_ushort(__float2half_rn(-tv)) * 0x00010001u;
    }
    memcpy(a.rm, t.rm, sizeof(a.rm));
    a.in_bf16 = q.in_bf16; a.out_bf16 = q.out_bf16;
    while ((1 << a.log2Gt) < Gt) ++a.log2Gt;
    a.m_lanes = m;
    while ((1 << a.log2m) < m) ++a.log2m;
    a.l2_sc_bit = q.f.l2_sc_bit;
    a.nl2 = q.f.block_size / L;
    a.l2_bytes = (a.nl2 * a.l2_sc_bit) >> 3;

    const size_t smem = (size_t)t.entries * 4;
    const int rc = mb == 1 ? launch_tab_geometry<1>(a, C, Gt, m, side, glu, smem, stream)
                           : launch_tab_geometry<2>(a, C, Gt, m, side, glu, smem, stream);
    if (rc == HBQ_OK) *launched = true;
    return rc;
}

}  // namespace hbq
