// tcgen05 / TMEM GEMM with the reference's accumulation models (blockquant_ext_src/gemm.cu).
//
// C[M,N] = A[M,K] * W[N,K]^T, fp16 operands (both K-major), fp16 output.
//
// The reference accumulates exact fp16xfp16 products in fp32 inside a K-chunk of `group_k`
// and then folds the chunk's partial sum into an fp16 running sum, optionally after fake
// quantising it (INT8 / E3M4 with a power-of-two scale per `group_n` columns).  Here each
// K-chunk is one accumulation in tensor memory: kind::f16 MMAs with fp32 accumulators, the
// first MMA of a chunk overwriting.  Two 128x256 fp32 accumulators (all 512 TMEM columns)
// alternate, so the epilogue warps drain chunk c (tcgen05.ld -> round / quantise -> fp16 add
// in registers) while the tensor core computes chunk c+1.
//
// One persistent CTA per SM, 384 threads in three warpgroups:
//   warp 0      TMA producer: 4-stage ring of {A 128x64, W 256x64} fp16 tiles, 128B swizzle
//               (decode-sized M: 6 stages of {A 128x64, W 128x64}, twice the CTAs)
//   warps 1-2   MMA issue (one lane each, alternate chunks); warp 1 also owns the TMEM allocation
//   warp 3      idle (fills the control warpgroup, which gives its registers away)
//   warps 4-11  epilogue: warp w owns TMEM lanes 32*(w%4).. and the 128 columns (w-4)/4; it takes
//               232 registers (setmaxnreg) so that a whole chunk slice (4 TMEM loads, 128 values per
//               thread) is in flight at once and the accumulator goes back to the MMA warps as soon
//               as the loads land, before any arithmetic
// The epilogue is the instruction-issue bottleneck (32768 fp32 values per 128-deep chunk against
// 1024 tensor-pipe cycles), so its arithmetic is packed: fma.rn.f32x2 for the INT8 rounding,
// cvt.rn.f16x2 and half2 min/max/add for the clamp and the fp16 accumulation.
// Every mbarrier wait is bounded: on expiry the kernel records a status word, all roles leave
// their loops, TMEM is freed and the kernel returns.
#include "tc_dev.cuh"
#include <math.h>
#include <atomic>
#include <mutex>

namespace hbq {

constexpr int BM = 128, BK = 64;
constexpr int TMEM_BUF_COLS = 256;                 // column stride of the two accumulators
constexpr int A_BYTES = BM * BK * 2;
// Two tile shapes (template parameters BN, NSTAGE of the kernel):
//   256 columns, 4 stages of 48 KB: the shape for every problem that fills the SMs;
//   128 columns, 6 stages of 32 KB: decode-sized M, where 256-column tiles would leave most SMs without
//   work and the time is the streaming of W -- twice the CTAs, the same bytes in flight per CTA.
constexpr int stage_bytes(int bn) { return A_BYTES + bn * BK * 2; }
constexpr uint32_t smem_bytes(int bn, int nstage) { return nstage * stage_bytes(bn) + 1024 /* alignment slack */ + 256 /* barriers */; }
constexpr int EPW = 8;                         // epilogue warps
constexpr int NTHREADS = 128 + EPW * 32;


// ---- epilogue arithmetic ---------------------------------------------------------------------
// INT8 partial-sum fake quantisation of `n` consecutive columns (gemm.cu:1145-1152, 1198-1249):
// scale = 2^(floor(log2 max|v|) - 6) (1 for an all-zero run), q = clamp(rint(v / scale), +-127).
// v / scale is exact, so rint is one FMA against 1.5 * 2^23.  Non-finite partial sums behave as in the
// reference: a NaN does not count towards the maximum and stays NaN (the clamp is NaN-propagating); an
// infinite maximum makes the reference's scale infinite and with it every value of the run NaN
// (gemm.cu:1145-1152, 1236-1249), which the NaN scale below reproduces.
template <int GN>
__device__ __forceinline__ void psum_int8_accumulate(const float* v, __half2* acc)
{
    float mx = 0.f;
    #pragma unroll
    for (int i = 0; i < GN; i += 2) mx = fmaxf(fmaxf(mx, fabsf(v[i])), fabsf(v[i + 1]));
    const uint32_t e = (__float_as_uint(mx) >> 23) & 0xFFu;
    float scale = mx > 0.f ? __uint_as_float((e - 6u) << 23) : 1.f;
    if (e == 255u) scale = __uint_as_float(0x7FC00000u);
    const float inv = mx > 0.f ? __uint_as_float((260u - e) << 23) : 1.f;
    constexpr float kMagic = 12582912.f;                 // 1.5 * 2^23: v*inv + kMagic rounds to an integer (RNE)
    const float unmagic = -kMagic * scale;               // exact
    // clamp to +-127 after the conversion to fp16: rounding is monotone, so
    // min(fp16(q*s), fp16(127*s)) == fp16(min(q, 127)*s)
    const __half2 lim = __float2half2_rn(127.f * scale);
    const __half2 nlim = bits_h2(h2_bits(lim) ^ 0x80008000u);
    #pragma unroll
    for (int i = 0; i < GN; i += 2) {
        float t0, t1, o0, o1;
        fma2(t0, t1, v[i], v[i + 1], inv, kMagic);
        fma2(o0, o1, t0, t1, scale, unmagic);            // (t - kMagic) * scale, exact
        const __half2 h = __hmin2_nan(__hmax2_nan(__floats2half2_rn(o0, o1), nlim), lim);
        acc[i >> 1] = __hadd2(acc[i >> 1], h);
    }
}

// E3M4 partial-sum fake quantisation (gemm.cu:677-745, 810-887): scale = 2^(floor(log2 max|v|) - 3), so
// y = |v| / scale lies in [0, 16); y is rounded (ties to even) to 4 mantissa bits with the exponent
// clamped at -2 -- a quantum of 2^(e_y - 4), never below 1/64 -- and capped at 15.5.  In fp32 that is one
// magic-number rounding per value with the quantum's exponent taken from the value's own exponent field.
template <int GN>
__device__ __forceinline__ void psum_e3m4_accumulate(const float* v, __half2* acc)
{
    float mx = 0.f;
    #pragma unroll
    for (int i = 0; i < GN; i += 2) mx = fmaxf(fmaxf(mx, fabsf(v[i])), fabsf(v[i + 1]));
    const int se = mx > 0.f ? (int)((__float_as_uint(mx) >> 23) & 0xFFu) - 3 : 127;      // exponent field of the scale
    const float cap = 15.5f * __uint_as_float((uint32_t)se << 23);
    const int qmin = se - 6;                                                               // quantum floor: scale / 64
    float o[GN];
    #pragma unroll
    for (int i = 0; i < GN; ++i) {
        const uint32_t b = __float_as_uint(v[i]);
        const uint32_t ab = b & 0x7FFFFFFFu;
        const int q = max((int)(ab >> 23) - 4, qmin);                                      // exponent field of the quantum
        const float magic = __uint_as_float(((uint32_t)(q + 23) << 23) | 0x00400000u);     // 1.5 * 2^23 quanta
        const float r = fminf((__uint_as_float(ab) + magic) - magic, cap);
        o[i] = __uint_as_float(__float_as_uint(r) | (b & 0x80000000u));
    }
    #pragma unroll
    for (int i = 0; i < GN; i += 2) acc[i >> 1] = __hadd2(acc[i >> 1], __floats2half2_rn(o[i], o[i + 1]));
}

// Fold 32 fp32 partial sums (one TMEM load) of this thread's row into its fp16 running sums.
template <int MODE, int GN>
__device__ __forceinline__ void fold_chunk(const float* v, __half2* acc)
{
    if (MODE == HBQ_ACC_PSUM_INT8) {
        #pragma unroll
        for (int c = 0; c < 32; c += GN) psum_int8_accumulate<GN>(v + c, acc + (c >> 1));
    } else if (MODE == HBQ_ACC_PSUM_E3M4) {
        #pragma unroll
        for (int c = 0; c < 32; c += GN) psum_e3m4_accumulate<GN>(v + c, acc + (c >> 1));
    } else {
        #pragma unroll
        for (int i = 0; i < 16; ++i) {
            const __half2 p = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            acc[i] = (MODE == HBQ_ACC_FP32) ? p : __hadd2(acc[i], p);
        }
    }
}

struct TcArgs {
    __half* C;
    const __half* bias;
    int M, N, K;
    int tiles_m, tiles_n;
    int k_stages;        // ceil(K / 64)
    int chunk_k16;       // MMAs (K = 16 each) per accumulation chunk
    int issuers;         // MMA-issuing warps to use (1 or 2)
    int bn;              // tile width chosen by the host: 256, or 128 for decode-sized M
    uint32_t poll_limit; // polls after which a wait on an mbarrier gives up (kDefaultPollLimit)
    int withhold_loads;  // self-test of the give-up path: the producer issues no load at all, so every
                         // consumer wait runs out with nothing in flight
};
constexpr uint32_t kDefaultPollLimit = 1u << 23;

// ---- the kernel ------------------------------------------------------------------------------
template <int MODE, int GN, int BN, int NSTAGE>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
               const TcArgs args)
{
    constexpr int STAGE_BYTES = A_BYTES + BN * BK * 2;
    // kind::f16: D fp32, A/B fp16, both K-major, M = 128, N = BN
    constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;                  // 1024-byte aligned tile ring
    uint8_t* ctrl = smem_raw + (tiles - raw) + NSTAGE * STAGE_BYTES;
    const uint32_t ctrl_u = tiles + NSTAGE * STAGE_BYTES;
    // control block: full[4] empty[4] tmem_full[2] tmem_empty[2] (8 B each), tmem base, abort flag
    const uint32_t bar_full = ctrl_u, bar_empty = ctrl_u + 8 * NSTAGE;
    const uint32_t bar_tfull = ctrl_u + 16 * NSTAGE, bar_tempty = bar_tfull + 16;
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(ctrl + 16 * NSTAGE + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 16 * NSTAGE + 40);

    constexpr int EPI_COLS = BN / (EPW / 4);
    constexpr int EPI_GROUPS = EPI_COLS / 32;        // TMEM loads (32 columns each) per warp and chunk
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar_tfull + 8 * b, 1); mbar_init(bar_tempty + 8 * b, EPW); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;"
                     ::"r"(smem_u32(tmem_base_smem)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_smem;

    const int total_tiles = args.tiles_m * args.tiles_n;
    const int total_k16 = args.k_stages * (BK / 16);

    // Register re-balancing between the warpgroups: the control warpgroup (warps 0-3) gives registers
    // away, the epilogue warpgroups take them (each setmaxnreg is executed by whole warpgroups).
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok && !args.withhold_loads; t += gridDim.x) {
                const int m0 = (t % args.tiles_m) * BM, n0 = (t / args.tiles_m) * BN;
                for (int ks = 0; ks < args.k_stages; ++ks) {
                    if (!(ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, 1, args.poll_limit))) break;
                    const uint32_t sa = tiles + stage * STAGE_BYTES, sb = sa + A_BYTES;
                    mbar_expect_tx(bar_full + 8 * stage, STAGE_BYTES);
                    tma_load_2d(sa, &mapA, ks * BK, m0, bar_full + 8 * stage);
                    tma_load_2d(sb, &mapB, ks * BK, n0, bar_full + 8 * stage);
                    if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ================= MMA issue =================
        // Two warps issue MMAs, taking alternate chunks: chunk c belongs to warp 1 + (c & 1), which
        // is also the accumulator it fills.  A chunk costs its issuing lane a serial chain of barrier
        // polls, MMA issues and commits that is longer than the chunk's 1024 tensor-pipe cycles; with
        // two warps each chain may take two chunk times.  All 32 lanes run the loop and wait on the
        // barriers together, so that it is warp-uniform code (counters, barrier addresses and matrix
        // descriptors in uniform registers); one fixed lane issues the MMAs and the commits that
        // track them.  MMAs of different chunks go to different accumulators, so their interleaving
        // in the tensor pipe is free; the shared-memory stages are consumed in the producer's order
        // because both warps count every stage.
        const uint32_t mw = (uint32_t)warp - 1u;
        const bool leader = elect_one();
        uint32_t chunk = 0;                  // running chunk counter: buffer = chunk & 1
        uint32_t gks = 0;                    // running k-stage counter: stage = gks % NSTAGE
        bool ok = true;
        if ((args.chunk_k16 % (BK / 16)) == 0) {
            // chunks are whole stages (group_k a multiple of 64, or the fp32 mode)
            const int spc = args.chunk_k16 / (BK / 16);
            // Two issuers only when every stage of the ring always meets the same warp: a warp may wait
            // for a barrier phase only after it has seen the phase before it, or the parity wait
            // aliases.  That holds when chunks are whole, equal and 2 * spc divides the ring; otherwise
            // warp 1 issues everything.
            const bool two = args.issuers == 2 && (NSTAGE % (2 * spc)) == 0 && (args.k_stages % spc) == 0;
            if (!two && mw != 0) ok = false;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                for (int ks0 = 0; ks0 < args.k_stages && ok; ks0 += spc, ++chunk) {
                    const int nst = min(spc, args.k_stages - ks0);
                    if (two && (chunk & 1u) != mw) { gks += nst; continue; }
                    const uint32_t buf = chunk & 1u;
                    uint32_t stage = gks % NSTAGE, phase = (gks / NSTAGE) & 1u;
                    // poll the first stage while waiting for the accumulator
                    bool full_pre = __all_sync(0xFFFFFFFFu, mbar_test(bar_full + 8 * stage, phase));
                    // the epilogue must have drained this accumulator's previous chunk (a fresh
                    // barrier passes the wait for the phase before its first)
                    if (!(ok = mbar_wait_warp(bar_tempty + 8 * buf, ((chunk >> 1) & 1u) ^ 1u, abort_flag, 3, args.poll_limit))) break;
                    const uint32_t d_tmem = tmem_base + buf * TMEM_BUF_COLS;
                    for (int s = 0; s < nst; ++s) {
                        if (!full_pre && !(ok = mbar_wait_warp(bar_full + 8 * stage, phase, abort_flag, 2, args.poll_limit))) break;
                        tc_fence_after();
                        const uint32_t nstage = (stage + 1 == NSTAGE) ? 0u : stage + 1, nphase = (stage + 1 == NSTAGE) ? phase ^ 1u : phase;
                        // poll for the next stage: in flight while the MMAs below are issued, consumed after
                        const bool next_full = (s + 1 < nst) ? mbar_test(bar_full + 8 * nstage, nphase) : false;
                        const uint32_t sa = tiles + stage * STAGE_BYTES, sb = sa + A_BYTES;
                        if (leader) {
                            #pragma unroll
                            for (int kk = 0; kk < BK / 16; ++kk)
                                tc_mma_f16(d_tmem, umma_desc(sa + kk * 32), umma_desc(sb + kk * 32), IDESC,
                                           (s != 0 || kk != 0) ? 1u : 0u);
                            tc_commit(bar_empty + 8 * stage);   // smem slot free once these MMAs retire
                            if (s + 1 == nst) tc_commit(bar_tfull + 8 * buf);
                        }
                        full_pre = __all_sync(0xFFFFFFFFu, next_full);
                        stage = nstage; phase = nphase;
                    }
                    gks += nst;
                }
            }
        } else if (mw == 0) {
            // chunks smaller than a stage (group_k 16 / 32): one warp, general bookkeeping per MMA
            uint32_t stage = 0, phase = 0;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                int in_chunk = 0;
                for (int ks = 0; ks < args.k_stages && ok; ++ks) {
                    if (!(ok = mbar_wait_warp(bar_full + 8 * stage, phase, abort_flag, 2, args.poll_limit))) break;
                    tc_fence_after();
                    const uint32_t sa = tiles + stage * STAGE_BYTES, sb = sa + A_BYTES;
                    #pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        const uint32_t buf = chunk & 1u;
                        if (in_chunk == 0) {
                            // the epilogue must have drained this accumulator's previous chunk
                            if (!(ok = mbar_wait_warp(bar_tempty + 8 * buf, ((chunk >> 1) & 1u) ^ 1u, abort_flag, 3, args.poll_limit))) break;
                            tc_fence_after();
                        }
                        const int k16 = ks * (BK / 16) + kk;
                        const bool last = (in_chunk + 1 == args.chunk_k16) || (k16 + 1 == total_k16);
                        if (leader) {
                            tc_mma_f16(tmem_base + buf * TMEM_BUF_COLS, umma_desc(sa + kk * 32), umma_desc(sb + kk * 32),
                                       IDESC, in_chunk != 0);
                            if (last) tc_commit(bar_tfull + 8 * buf);
                        }
                        __syncwarp();
                        if (last) { in_chunk = 0; ++chunk; } else ++in_chunk;
                    }
                    if (!ok) break;
                    if (leader) tc_commit(bar_empty + 8 * stage);
                    __syncwarp();
                    if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
                }
            }
        }
    }
    } else {
        // ================= epilogue =================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        const int ew = warp - 4;
        const int quarter = warp & 3;            // TMEM lanes this warp may touch
        const int cgrp = ew >> 2;                // which EPI_COLS columns of the 256-wide tile
        const int chunks_per_tile = (total_k16 + args.chunk_k16 - 1) / args.chunk_k16;
        uint32_t chunk = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
            const int m0 = (t % args.tiles_m) * BM, n0 = (t / args.tiles_m) * BN;
            __half2 acc[EPI_COLS / 2];
            #pragma unroll
            for (int i = 0; i < EPI_COLS / 2; ++i) acc[i] = __float2half2_rn(0.f);
            for (int c = 0; c < chunks_per_tile; ++c, ++chunk) {
                const uint32_t buf = chunk & 1u;
                ok = mbar_wait(bar_tfull + 8 * buf, (chunk >> 1) & 1u, abort_flag, 4, args.poll_limit);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * TMEM_BUF_COLS + cgrp * EPI_COLS;
                {
                    // the warp's whole slice of the chunk: all its 32-column loads in flight together
                    uint32_t r[EPI_GROUPS][32];
                    #pragma unroll
                    for (int h = 0; h < EPI_GROUPS; ++h) tc_ld32_issue(taddr + h * 32, r[h]);
                    tc_ld_wait(r[0]);                    // waits for all of them
                    #pragma unroll
                    for (int h = 1; h < EPI_GROUPS; ++h) tc_ld_landed(r[h]);
                    // this warp's reads of the accumulator are complete: hand it back to the MMA warps
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
                    #pragma unroll
                    for (int h = 0; h < EPI_GROUPS; ++h) {
                        float v[32];
                        #pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[h][i]);
                        fold_chunk<MODE, GN>(v, acc + h * 16);
                    }
                }
            }
            if (!ok) break;
            // ---- write the thread's row: EPI_COLS columns starting at n0 + cgrp*EPI_COLS ----
            const int row = m0 + quarter * 32 + lane;
            const int col0 = n0 + cgrp * EPI_COLS;
            if (row < args.M) {
                __half* cp = args.C + (int64_t)row * args.N + col0;
                #pragma unroll
                for (int g = 0; g < EPI_COLS / 8; ++g) {
                    const int col = col0 + g * 8;
                    if (col >= args.N) break;
                    __half2 o[4] = {acc[4 * g], acc[4 * g + 1], acc[4 * g + 2], acc[4 * g + 3]};
                    if (args.bias) {
                        const uint4 bv = *reinterpret_cast<const uint4*>(args.bias + col);
                        o[0] = __hadd2(o[0], bits_h2(bv.x)); o[1] = __hadd2(o[1], bits_h2(bv.y));
                        o[2] = __hadd2(o[2], bits_h2(bv.z)); o[3] = __hadd2(o[3], bits_h2(bv.w));
                    }
                    *reinterpret_cast<uint4*>(cp + g * 8) =
                        make_uint4(h2_bits(o[0]), h2_bits(o[1]), h2_bits(o[2]), h2_bits(o[3]));
                }
            }
        }
    }

    // ---- teardown: every role arrives here, also after an expired wait ----
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // let TMA copies that may still be in flight land before the CTA's smem is released
        const unsigned long long t0 = gtime_ns();
        while (gtime_ns() - t0 < 200000ull) { }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}


// ---- transpose [K,N] -> [N,K] ------------------------------------------------------------------
__global__ void __launch_bounds__(256) transpose_kernel(const __half* __restrict__ in, __half* __restrict__ out,
                                                        int R, int Ccols)
{
    __shared__ __half tile[64][66];
    const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        const int r = i / 64, c = i % 64;
        if (r0 + r < R && c0 + c < Ccols) tile[r][c] = in[(int64_t)(r0 + r) * Ccols + c0 + c];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        const int c = i / 64, r = i % 64;
        if (r0 + r < R && c0 + c < Ccols) out[(int64_t)(c0 + c) * R + r0 + r] = tile[r][c];
    }
}

// ---- host side -----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// fp16 row-major [rows, K] matrix, boxes of box_rows x 64 elements, 128-byte swizzle, zero fill
// Tensor maps depend on (pointer, rows, K, box) only and a serving loop presents the same few operands
// (the weights above all) again and again: a small cache saves the driver call.
struct MapKey { const void* ptr; int64_t rows, K; int box_rows; };
struct MapSlot { MapKey key; CUtensorMap map; bool used; };
static MapSlot g_map_cache[64];
static std::mutex g_map_mutex;

static int make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t K, int box_rows)
{
    const size_t h = ((reinterpret_cast<uintptr_t>(ptr) >> 8) * 0x9E3779B97F4A7C15ull ^ (size_t)rows * 31u ^ (size_t)K ^ (size_t)box_rows) >> 58;
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        const MapSlot& s = g_map_cache[h & 63];
        if (s.used && s.key.ptr == ptr && s.key.rows == rows && s.key.K == K && s.key.box_rows == box_rows) {
            *map = s.map;
            return HBQ_OK;
        }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return HBQ_ERR_CUDA;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return HBQ_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_map_mutex);
    MapSlot& s = g_map_cache[h & 63];
    s.key = {ptr, rows, K, box_rows};
    s.map = *map;
    s.used = true;
    return HBQ_OK;
}

// The same tensor map for the other tensor-core kernels of the library (gemm_packed.cu).
int gemm_make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t K, int box_rows)
{
    return make_map(map, ptr, rows, K, box_rows);
}

bool gemm_tc_eligible(int64_t M, int64_t N, int64_t K, int mode, int group_k, int group_n)
{
    if (M <= 0 || N <= 0 || K <= 0 || M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 30)) return false;
    if ((K % 8) != 0 || (N % 8) != 0) return false;
    if (mode == HBQ_ACC_FP16) return false;                 // the per-product fp16 chain has no tensor-core form
    if (mode == HBQ_ACC_FP32) return true;
    if (group_k < 16 || (group_k % 16) != 0) return false;
    if (mode >= HBQ_ACC_PSUM_INT8 && !(group_n == 4 || group_n == 8 || group_n == 16 || group_n == 32)) return false;
    return true;
}

template <int MODE, int GN>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const TcArgs& args, int grid, cudaStream_t stream)
{
    if (args.bn == 128) {
        { const int rc = ensure_dynamic_smem(gemm_tc_kernel<MODE, GN, 128, 6>, smem_bytes(128, 6)); if (rc) return rc; }
        gemm_tc_kernel<MODE, GN, 128, 6><<<grid, NTHREADS, smem_bytes(128, 6), stream>>>(ma, mb, args);
    } else {
        { const int rc = ensure_dynamic_smem(gemm_tc_kernel<MODE, GN, 256, 4>, smem_bytes(256, 4)); if (rc) return rc; }
        gemm_tc_kernel<MODE, GN, 256, 4><<<grid, NTHREADS, smem_bytes(256, 4), stream>>>(ma, mb, args);
    }
    HBQ_LAUNCH_CHECK("gemm_tc_kernel");
    return HBQ_OK;
}

int transpose_launch(const void* in, void* out, int64_t R, int64_t Ccols, cudaStream_t stream)
{
    const dim3 grid((unsigned)((Ccols + 63) / 64), (unsigned)((R + 63) / 64));
    transpose_kernel<<<grid, 256, 0, stream>>>((const __half*)in, (__half*)out, (int)R, (int)Ccols);
    HBQ_LAUNCH_CHECK("transpose_kernel");
    return HBQ_OK;
}

// SMs that launches leave free for a kernel of another stream (hbq_gemm_reserve_sms)
static std::atomic<int> g_reserved_sms{0};

// A [M,K], W [N,K], both fp16 row-major and 16-byte aligned.
// poll_limit = 0: the default bound; withhold_loads: see TcArgs (the self-test of hbq_gemm_wait_selftest).
int gemm_tc_launch_ex(const void* A, const void* W, void* C, int64_t M, int64_t N, int64_t K, int mode,
                      int group_k, int group_n, const void* bias, cudaStream_t stream, uint32_t poll_limit,
                      int withhold_loads)
{
    if (!gemm_tc_eligible(M, N, K, mode, group_k, group_n)) return HBQ_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(C) |
         reinterpret_cast<uintptr_t>(bias)) & 15)
        return HBQ_ERR_ALIGN;
    CUtensorMap ma, mb;
    int rc = make_map(&ma, A, M, K, BM);
    if (rc) return rc;

    TcArgs args;
    args.C = (__half*)C; args.bias = (const __half*)bias;
    args.M = (int)M; args.N = (int)N; args.K = (int)K;
    int sms = 0;
    { const int rc2 = device_sms(&sms); if (rc2) return rc2; }
    args.tiles_m = (int)((M + BM - 1) / BM);
    // 128-column tiles when 256-column ones would leave more than half of the SMs without work
    // ... or when the whole problem is at most 128 columns wide (a 256-column tile would be half empty)
    args.bn = (N <= 128 || (int64_t)args.tiles_m * ((N + 255) / 256) * 2 <= sms) ? 128 : 256;
    args.tiles_n = (int)((N + args.bn - 1) / args.bn);
    rc = make_map(&mb, W, N, K, args.bn);
    if (rc) return rc;
    args.k_stages = (int)((K + BK - 1) / BK);
    args.chunk_k16 = (mode == HBQ_ACC_FP32) ? args.k_stages * (BK / 16) : group_k / 16;
    args.issuers = 2;
    args.poll_limit = poll_limit ? poll_limit : kDefaultPollLimit;
    args.withhold_loads = withhold_loads;

    const int64_t total = (int64_t)args.tiles_m * args.tiles_n;
    const int usable = sms - g_reserved_sms.load() > 0 ? sms - g_reserved_sms.load() : 1;
    const int grid = (int)(total < usable ? total : usable);

    switch (mode) {
        case HBQ_ACC_FP32: return launch_tc<HBQ_ACC_FP32, 32>(ma, mb, args, grid, stream);
        case HBQ_ACC_GROUPED: return launch_tc<HBQ_ACC_GROUPED, 32>(ma, mb, args, grid, stream);
        case HBQ_ACC_PSUM_INT8:
            switch (group_n) {
                case 4: return launch_tc<HBQ_ACC_PSUM_INT8, 4>(ma, mb, args, grid, stream);
                case 8: return launch_tc<HBQ_ACC_PSUM_INT8, 8>(ma, mb, args, grid, stream);
                case 16: return launch_tc<HBQ_ACC_PSUM_INT8, 16>(ma, mb, args, grid, stream);
                default: return launch_tc<HBQ_ACC_PSUM_INT8, 32>(ma, mb, args, grid, stream);
            }
        case HBQ_ACC_PSUM_E3M4:
            switch (group_n) {
                case 4: return launch_tc<HBQ_ACC_PSUM_E3M4, 4>(ma, mb, args, grid, stream);
                case 8: return launch_tc<HBQ_ACC_PSUM_E3M4, 8>(ma, mb, args, grid, stream);
                case 16: return launch_tc<HBQ_ACC_PSUM_E3M4, 16>(ma, mb, args, grid, stream);
                default: return launch_tc<HBQ_ACC_PSUM_E3M4, 32>(ma, mb, args, grid, stream);
            }
    }
    return HBQ_ERR_ARG;
}

int gemm_tc_launch(const void* A, const void* W, void* C, int64_t M, int64_t N, int64_t K, int mode,
                   int group_k, int group_n, const void* bias, cudaStream_t stream)
{
    return gemm_tc_launch_ex(A, W, C, M, N, K, mode, group_k, group_n, bias, stream, 0, 0);
}

int gemm_tc_reserve_sms(int n)
{
    return g_reserved_sms.exchange(n < 0 ? 0 : n);
}

int gemm_w4_status(int* host_out);          // gemm_packed.cu: that kernel's own status word
int gemm_w4_status_reset();

// Non-zero when a wait gave up in either tensor-core kernel (the packed-weight kernel's codes are offset by 16).
int gemm_tc_status(int* host_out)
{
    int s = 0, p = 0;
    HBQ_CUDA_TRY(cudaMemcpyFromSymbol(&s, g_tc_status, sizeof(int)));
    { const int rc = gemm_w4_status(&p); if (rc) return rc; }
    *host_out = s ? s : (p ? 16 + p : 0);
    return HBQ_OK;
}
int gemm_tc_status_reset()
{
    const int z = 0;
    HBQ_CUDA_TRY(cudaMemcpyToSymbol(g_tc_status, &z, sizeof(int)));
    return gemm_w4_status_reset();
}

}  // namespace hbq
