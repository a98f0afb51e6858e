// Decode-shape GEMM that reads the HBQ weight as packed 4-bit codes and scales (0.5625 B per weight instead of
// the 2 B of the fp16 fake-quantised tensor) and expands them to fp16 in tensor memory in front of the tensor core.
//
//   C[M,N] = X[M,K] * deq(Wp)[N,K]^T     M <= 128 tokens, fp32 accumulation, fp16 output
//
// For M this small the time of the fp16-operand kernel is the streaming of W from HBM.  The reference keeps W as an
// fp16 tensor (src/ptq.py:349) and multiplies with F.linear (src/module.py:64); the values here are the same fp16
// values, rebuilt per tile:  w = fp16(level(code) * t * s)  with level the E2M1 element value, t the micro-scale
// candidate chosen for the element's micro-block and s the E5M3 block scale.  t * s is exact in fp16 (4 + 4
// significant bits), level * t is exact as well, so one multiply by the per-micro-block product t*s rounds exactly
// like the quantizer's fp16(fp16(level * t) * s).
//
// Three kernels share the prepacked weight and its expansion.  One token: gemv_packed_kernel, no tensor core.  Two to
// eight tokens (nibble container): gemm_packed_reg_kernel, mma.sync with the expanded weights as register fragments.
// Everything else, described here: gemm_packed_kernel on tcgen05.
//
// Operands are swapped with respect to gemm_tc.cu: the 128 weight rows of a tile are the M side of the MMA
// (A operand), the tokens its N side (B operand, X through TMA, zero filled beyond M), so the MMA's cost follows the
// token count.  The A operand is read from TENSOR MEMORY: lane = weight row, a 32-bit column = two consecutive k, 64
// columns per stage of 128 k.  The expansion warps write it there with tcgen05.st (each warp the lane quarter it may
// access), so the expanded weights never pass through shared memory: writing 32 KB per stage and having the tensor
// core read it back was, with the record and the X tiles, some 90 KB of shared-memory traffic per 9 KB record and
// the bound of the earlier design.  The accumulator D^T[n, m] sits in tensor memory as well; the SM's 512 columns
// hold four accumulators (two issuers x two segments in flight) of 32 or 64 columns and six or four expanded stages;
// beyond 64 tokens two accumulators of 128 columns (one segment in flight) and four stages.
//
// Prepacked weight (hbq_gemm_w4_prepack): one 9216-byte record per (tile of 128 rows, block of 128 k) -- what one
// pipeline stage consumes, fetched with ONE bulk async copy:
//   [4 pieces][128 rows][16 B]   codes: piece q holds the 32 elements k = 32q..32q+31 of every row, element j of a
//                                32-bit word in nibble j as {sign, e1, e0, m}; rows are contiguous so that a warp's
//                                16-byte reads (one row per lane) hit every bank once
//   [128 rows][8 B]              micro-scale indices (2 bits each, 32 bits), the block scale as fp16, the table bit
// A byte of two codes becomes an fp16 pair with one cvt.rn.f16x2.e2m1x2 (the codes ARE E2M1), then one multiply by the
// packed scale.  With container_bits = 8 each code is stored as the top byte of its value's fp16 pattern
// (17408-byte records): the same values through a byte permute instead of the conversion.
//
// Work split: the (tile, block) records form one sequence of tiles * K/128 stages.  Either every CTA takes whole
// tiles (nothing to fix up), or CTA c of G (one per SM) takes the c-th of G equal runs of the sequence, whatever tile
// boundaries fall inside ("stream-K"), so that every SM streams the same number of bytes.  A shared tile costs a
// chain of dependent round trips through memory (partial sums, fence, count, read back) that is worth about fourteen
// stages, so the host takes equal runs only where they save more than that (few tiles, long K).  In a run, a segment
// that covers its tile's whole K goes straight to C; the others leave fp32 partial sums in a workspace and the CTA
// that completes a tile adds its segments in CTA order (deterministic) and writes C.  A run is processed head of the
// next CTA's tile first and end of the previous CTA's tile last, so that the CTA ending a tile mostly finds the
// partner's partial sums published and completes the tile straight from its accumulator.
//
// 896 threads:
//   warps 0-3    epilogue: one per quarter of the tensor-memory lanes; two accumulator pairs alternate between segments
//   warps 4, 6   record producers (one lane each) of the even / odd stages: one bulk copy of a packed record per stage
//   warps 5, 7   MMA issue (one lane each) on the even / odd stages, an accumulator each; warp 5 owns the tensor-memory
//                allocation
//   warps 8-23   expansion, two groups of eight warps on alternate stages: thread (row r, half hh) turns 64 codes into
//                32 columns of its lane; the groups touch no mbarrier (hardware barriers to their service warps)
//   warps 24-27  waiters (see a stage's record landed and its slot free, release the group, issue the X tiles' TMA
//                loads) and reporters (announce the stored stage to the MMA thread, free the record slot)
// No thread visits every stage: a visit (seeing an mbarrier, arming it, issuing) costs several hundred cycles even
// when nothing blocks, an issued MMA about 90 cycles whatever its width.  What a stage costs now, 0.4 us, is close to
// both the eight MMAs of an issuer and the barrier skeleton alone (measured with the expansion and the MMAs left out).
#include "tc_dev.cuh"
#include <math.h>
#include <mutex>

namespace hbq {

int gemm_make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t K, int box_rows);   // gemm_tc.cu

constexpr int PK_ROWS = 128;                                  // weight rows per tile
constexpr int PK_KB = 128;                                    // k per stage: one quantisation block
constexpr int PK_SIDE_BYTES = PK_ROWS * 8;                    // 1024
// Two containers for the element codes: 4 bits ({sign, e1, e0, m}: 9216-byte records, 0.5625 B per weight) or 8 bits
// (the top byte of the element value's fp16 pattern, sign included -- its low byte is zero: 17408-byte records,
// 1.0625 B per weight).  The 4-bit form costs about 25 instructions per 8 codes to expand, the 8-bit form about 12.
__host__ __device__ constexpr int pk_code_bytes(int cb) { return PK_ROWS * PK_KB * cb / 8; }
__host__ __device__ constexpr int pk_rec_bytes(int cb) { return pk_code_bytes(cb) + PK_SIDE_BYTES; }
constexpr int PK_EXP_BYTES = 2 * PK_ROWS * 128;               // two K-major 128 x 64 fp16 tiles
constexpr int PK_NE = 6;                                      // operand stages when the weight is expanded here (even: two per lane)
constexpr int PK_NE_MAX = 6;                                  // ... when fp16 weight tiles come straight from TMA
constexpr int PK_NL_MAX = 16;                                 // load stages (fewer when X tiles are large)
constexpr int PK_EPI_WARPS = 4;
constexpr int PK_EXP_WARPS = 16;
constexpr int PK_EXP_WARP0 = PK_EPI_WARPS + 4;              // warps 4, 5, 6: record producer, MMA issue, X producer
constexpr int PK_SERVICE0 = PK_EXP_WARP0 + PK_EXP_WARPS;       // warps 24, 25: waiters of expansion groups 0, 1; 26, 27: their reporters
constexpr int PK_THREADS = (PK_SERVICE0 + 4) * 32;
constexpr int PK_CTRL_BYTES = 512;
constexpr int PK_CLUSTER_STAGES = 2;                          // ... what meeting in a cluster's shared memory costs
constexpr int PK_FIXUP_STAGES = 14;                           // what sharing tiles between CTAs costs, in stages

struct PkArgs {
    const uint8_t* wp;          // prepacked weight [tiles][nblk][record]
    __half* C;
    const __half* bias;
    float* ws;                  // [grid][2][m_pad][128] partial sums of segments that do not cover their tile's K
    int* counters;              // [tiles], zero between calls
    int M, N, K;
    int m_pad;                  // tokens rounded up to 16: the MMA's N
    int nblk, tiles, nl;
    int ne;                     // operand stages: 3, or 2 when the tokens' tiles are large
    int total;                  // tiles * nblk stages (below 2^31: a weight of that many records does not fit the device)
    int run_q, run_r;           // equal runs: total / grid and total % grid -- CTA c takes run_q stages, one more if c < run_r
    uint32_t base2[2], step2[2];// micro-scale t = base + idx * step as packed fp16 pairs, per table
    uint32_t acc_cols;          // tensor-memory columns of one accumulator (32, 64 or 128)
    uint32_t acc_bufs;          // accumulator pairs (one per issuer) in flight: 2 (segments alternate), 1 for 128 columns
    uint32_t tmem_cols;         // columns allocated: the accumulators, then (packed weight) `ne` expanded stages of 64
    uint32_t poll_limit;
    int whole_tiles;            // 1: every CTA takes whole tiles (no tile is shared, nothing to fix up)
    int split;                  // S >= 2: a tile's K range is split over the S CTAs of a cluster; 0: no clusters
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// Eight E2M1 codes (nibbles {sign, e1, e0, m} of w) times the packed scale ts2 -> four fp16 pairs.
// Top bytes of the element values 0, .5, 1, 1.5, 2, 3, 4, 6 come from a byte lookup (their low bytes are zero), the
// signs from the nibbles' top bits replicated into byte masks.
template <bool TWO_STEP>
__device__ __forceinline__ void expand8(uint32_t w, uint32_t ts2, uint32_t t2, uint32_t s2, uint32_t* o)
{
    // the conversion unit turns a byte of two E2M1 codes into an fp16 pair (low nibble -> low half), signs included
    uint32_t v[4];
    asm("{ .reg .b8 b0, b1, b2, b3;\n"
        "  mov.b32 {b0, b1, b2, b3}, %4;\n"
        "  cvt.rn.f16x2.e2m1x2 %0, b0;\n"
        "  cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        "  cvt.rn.f16x2.e2m1x2 %2, b2;\n"
        "  cvt.rn.f16x2.e2m1x2 %3, b3; }"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(w));
    #pragma unroll
    for (int p = 0; p < 4; ++p)
        o[p] = TWO_STEP ? h2_bits(__hmul2(__hmul2(bits_h2(v[p]), bits_h2(t2)), bits_h2(s2)))
                        : h2_bits(__hmul2(bits_h2(v[p]), bits_h2(ts2)));
}

// The MMA with its A operand in tensor memory (lane = row, a 32-bit column = two consecutive k), B from shared memory.
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Four 32-bit columns of this thread's tensor-memory lane (warp-collective: every lane, the same columns).
__device__ __forceinline__ void tc_st4(uint32_t taddr, const uint32_t* o)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};"
                 ::"r"(taddr), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
}

// 16 consecutive fp32 columns of this thread's tensor-memory lane
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float* v)
{
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    #pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Bounded waits for the roles that have nothing to do until the barrier completes: mbarrier.try_wait parks the
// thread for a hardware-chosen while instead of spinning, so waiting warps leave the issue slots to the warps that
// expand.  `limit` parked attempts (each ends by itself), then the wait gives up like mbar_wait.
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, uint32_t limit)
{
    #pragma unroll 1
    for (uint32_t it = 0; it < limit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    atomicCAS(&g_tc_status, 0, code);
    return false;
}
// The same for a whole warp: lane 0 waits, the others are held at the shuffle.
__device__ __forceinline__ bool mbar_wait_parked_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, uint32_t limit)
{
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait_parked(bar, parity, abort_flag, code, limit) ? 1 : 0;
    return __shfl_sync(0xFFFFFFFFu, ok, 0) != 0;
}


// Bounded wait of a warp for TWO barriers at once: lane 0 polls (bar0, par0), lane 1 (bar1, par1), the other lanes
// poll nothing; the result is warp-uniform.
__device__ __forceinline__ bool mbar_wait_pair(uint32_t bar0, uint32_t par0, uint32_t bar1, uint32_t par1, volatile int* abort_flag,
                                               int code, uint32_t limit)
{
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t bar = lane == 1 ? bar1 : bar0, par = lane == 1 ? par1 : par0;
    #pragma unroll 1
    for (uint32_t it = 0; it < limit; ++it) {
        const bool t = lane < 2 ? mbar_test(bar, par) : true;
        if (__all_sync(0xFFFFFFFFu, t)) return true;
        if ((it & 127u) == 127u && __any_sync(0xFFFFFFFFu, *abort_flag != 0)) return false;
    }
    if (lane == 0) {
        *abort_flag = 1;
        atomicCAS(&g_tc_status, 0, code);
    }
    __syncwarp();
    return false;
}

// First stage of CTA c's run, and the CTA whose run holds stage g.
__device__ __forceinline__ int run_begin(const PkArgs& a, int c) { return c * a.run_q + min(c, a.run_r); }
__device__ __forceinline__ int cta_of_stage(const PkArgs& a, int g)
{
    const int edge = a.run_r * (a.run_q + 1);
    return g < edge ? g / (a.run_q + 1) : a.run_r + (g - edge) / a.run_q;
}

// Eight element values given as the top bytes of their fp16 patterns (two words) times the packed scale.
template <bool TWO_STEP>
__device__ __forceinline__ void expand8_bytes(uint32_t w0, uint32_t w1, uint32_t ts2, uint32_t t2, uint32_t s2, uint32_t* o)
{
    const uint32_t v[4] = {prmt(w0, 0u, 0x1404u), prmt(w0, 0u, 0x3424u), prmt(w1, 0u, 0x1404u), prmt(w1, 0u, 0x3424u)};
    #pragma unroll
    for (int p = 0; p < 4; ++p)
        o[p] = TWO_STEP ? h2_bits(__hmul2(__hmul2(bits_h2(v[p]), bits_h2(t2)), bits_h2(s2)))
                        : h2_bits(__hmul2(bits_h2(v[p]), bits_h2(ts2)));
}

// MS: log2(chunks of 8 per micro-block): 0 (micro-block 8) or 2 (micro-block 32); CB: bits of the code container
template <int MS, int CB>
__global__ void __launch_bounds__(PK_THREADS, 1)
gemm_packed_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapW, const PkArgs a)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t exp0 = (raw + 1023u) & ~1023u;                    // expanded tiles (1024-byte aligned for the swizzle)
    // operand stage in shared memory: two X tiles, after (fp16 weight) the two weight tiles; the expanded stages of a
    // packed weight live in tensor memory
    constexpr uint32_t WB = CB == 16 ? PK_EXP_BYTES : 0;
    const uint32_t ES = WB + (uint32_t)a.m_pad * 256u;
    constexpr uint32_t LS = pk_rec_bytes(CB);                        // load stage: one packed record
    constexpr uint32_t CODE_BYTES = pk_code_bytes(CB);
    const uint32_t ne = (uint32_t)a.ne;
    const uint32_t ld0 = exp0 + ne * ES;
    const uint32_t ctrl_u = ld0 + (uint32_t)a.nl * LS;
    const uint32_t stg = CB == 16 ? exp0 : ld0;                      // where a cluster's CTAs leave their parts of a tile (free by then)
    uint8_t* ctrl = smem_raw + (ctrl_u - raw);
    // control block: ld_full[16] ld_empty[16] ex_full[6] ex_empty[6] acc_full[2] acc_empty[2] (8 B each), then the
    // tensor-memory base, the abort flag and the "this CTA completes the tile" flag
    const uint32_t bar_lfull = ctrl_u, bar_lempty = ctrl_u + 8 * PK_NL_MAX;
    const uint32_t bar_efull = ctrl_u + 16 * PK_NL_MAX, bar_eempty = bar_efull + 8 * PK_NE_MAX;
    const uint32_t bar_afull = bar_eempty + 8 * PK_NE_MAX, bar_aempty = bar_afull + 16;
    constexpr int CTRL_WORDS = 16 * PK_NL_MAX + 16 * PK_NE_MAX + 32;
    static_assert(CTRL_WORDS + 16 <= PK_CTRL_BYTES, "control block");
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(ctrl + CTRL_WORDS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + CTRL_WORDS + 8);
    volatile int* last_flag = reinterpret_cast<volatile int*>(ctrl + CTRL_WORDS + 12);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x, cta = blockIdx.x;
    // cluster split: CTA `rank` of the S in a cluster takes the rank-th of S equal parts of its tile's K blocks
    const int split_tile = a.split ? cta / a.split : 0, split_rank = a.split ? cta % a.split : 0;
    // (32-bit index arithmetic throughout: a 64-bit division costs hundreds of cycles and several sat in every stage)
    const int g0 = a.split ? split_tile * a.nblk + a.nblk * split_rank / a.split
                 : a.whole_tiles ? a.tiles * cta / G * a.nblk : run_begin(a, cta);
    const int g1 = a.split ? split_tile * a.nblk + a.nblk * (split_rank + 1) / a.split
                 : a.whole_tiles ? a.tiles * (cta + 1) / G * a.nblk : run_begin(a, cta + 1);
    const int nst = g1 - g0;
    // The run's stages are taken in three pieces: the head of the tile that the NEXT CTA completes, the whole tiles, and
    // last the end of the tile that the PREVIOUS CTA began.  A tile shared by two CTAs is thus begun early by one and
    // ended late by the other, whose fix-up then finds the partner's partial sums already published.
    const int e1 = (g0 % a.nblk) == 0 ? g0 : min(g1, (g0 / a.nblk + 1) * a.nblk);
    const int hb = max(e1, g1 - g1 % a.nblk);
    const int pc_s[3] = {hb, e1, g0};
    const int pc_n[3] = {g1 - hb, hb - e1, e1 - g0};
    // stage i of the run in processing order -> its global (tile, block) index
    auto stage_g = [&](int i) -> int {
        if (i < pc_n[0]) return pc_s[0] + i;
        i -= pc_n[0];
        return i < pc_n[1] ? pc_s[1] + i : pc_s[2] + (i - pc_n[1]);
    };
    const uint32_t park_limit = (a.poll_limit >> 6) + 64u;          // parked attempts last far longer than a poll

    if (threadIdx.x == 32) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&mapX) : "memory");
        if (CB == 16) asm volatile("prefetch.tensormap [%0];" ::"l"(&mapW) : "memory");
    }
    if (threadIdx.x < 2 * PK_NL_MAX + 2 * PK_NE_MAX + 4) {
        // one barrier per thread: ld_full / ld_empty (one arrival each), ex_full (two: the stage's reporter or weight
        // bytes, and the X tiles' bytes), ex_empty (one commit), acc_full (both issuers), acc_empty (the epilogue warps)
        const int t = threadIdx.x;
        uint32_t count = 1;
        if (t >= 2 * PK_NL_MAX && t < 2 * PK_NL_MAX + PK_NE_MAX) count = 2;
        else if (t >= 2 * PK_NL_MAX + 2 * PK_NE_MAX) count = t < 2 * PK_NL_MAX + 2 * PK_NE_MAX + 2 ? 2 : PK_EPI_WARPS;
        mbar_init(ctrl_u + 8 * t, count);
        if (t == 0) { *abort_flag = 0; *last_flag = 0; }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_base_smem)), "r"(a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_smem;

    if (warp == 4) {
        // ================= record producer =================
        if (CB == 16) {
            // fp16 weight: its two K-major 128 x 64 tiles go by TMA straight into the operand stage
            if (lane == 0) {
                uint32_t es = 0, eph = 0;
                for (int i = 0; i < nst; ++i) {
                    if (!mbar_wait(bar_eempty + 8 * es, eph ^ 1u, abort_flag, 1, a.poll_limit)) break;
                    const uint32_t dst = exp0 + es * ES, bar = bar_efull + 8 * es;
                    const int g = stage_g(i);
                    const int kb = g % a.nblk, row0 = g / a.nblk * PK_ROWS;
                    mbar_expect_tx(bar, PK_EXP_BYTES);
                    tma_load_2d(dst, &mapW, kb * PK_KB, row0, bar);
                    tma_load_2d(dst + PK_ROWS * 128, &mapW, kb * PK_KB + 64, row0, bar);
                    if (++es == ne) { es = 0; eph ^= 1u; }
                }
            }
        } else if (lane == 0) {
            // packed weight: the records of the EVEN stages (warp 6 takes the odd ones).  One visit of a producing
            // thread to a stage -- seeing the barrier, arming it, issuing the copy -- costs 600-700 cycles even when
            // nothing blocks, so no thread of this kernel visits every stage.
            const uint32_t nl = (uint32_t)a.nl;
            for (int i = 0; i < nst; i += 2) {
                const uint32_t stage = (uint32_t)i % nl, phase = ((uint32_t)i / nl) & 1u;
                if (!mbar_wait(bar_lempty + 8 * stage, phase ^ 1u, abort_flag, 1, a.poll_limit)) break;
                const uint32_t bar = bar_lfull + 8 * stage;
                mbar_expect_tx(bar, LS);
                bulk_load(ld0 + stage * LS, a.wp + stage_g(i) * (int64_t)LS, LS, bar);
            }
        }
    } else if (warp == 6) {
        if (CB == 16) {
            // ================= X producer (fp16 weight): the tokens' tiles travel with the operand stage =================
            if (lane == 0) {
                uint32_t es = 0, eph = 0;
                for (int i = 0; i < nst; ++i) {
                    if (!mbar_wait_parked(bar_eempty + 8 * es, eph ^ 1u, abort_flag, 8, park_limit)) break;
                    const uint32_t dst = exp0 + es * ES + WB, bar = bar_efull + 8 * es;
                    const int kb = stage_g(i) % a.nblk;
                    mbar_expect_tx(bar, (uint32_t)a.m_pad * 256u);
                    tma_load_2d(dst, &mapX, kb * PK_KB, 0, bar);
                    tma_load_2d(dst + (uint32_t)a.m_pad * 128u, &mapX, kb * PK_KB + 64, 0, bar);
                    if (++es == ne) { es = 0; eph ^= 1u; }
                }
            }
        } else if (lane == 0) {
            // ================= record producer of the ODD stages =================
            const uint32_t nl = (uint32_t)a.nl;
            for (int i = 1; i < nst; i += 2) {
                const uint32_t stage = (uint32_t)i % nl, phase = ((uint32_t)i / nl) & 1u;
                if (!mbar_wait(bar_lempty + 8 * stage, phase ^ 1u, abort_flag, 1, a.poll_limit)) break;
                const uint32_t bar = bar_lfull + 8 * stage;
                mbar_expect_tx(bar, LS);
                bulk_load(ld0 + stage * LS, a.wp + stage_g(i) * (int64_t)LS, LS, bar);
            }
        }
    } else if (warp == 5 || warp == 7) {
        // ================= MMA issue =================
        // A visit of an issuing thread to a stage -- seeing the barrier, the MMAs (about 90 cycles each whatever their
        // width), the commits -- is a serial chain of about a thousand cycles, and it bounds the pipeline.  So the two
        // issuers take ALTERNATE stages (issuer p the stages of parity p, all eight MMAs of each) into an accumulator
        // of their own -- MMAs of different threads are not ordered with each other -- and the epilogue adds the two.
        // The operand ring has an even length, so a slot always belongs to the same issuer and its barrier phases are
        // seen one after the other; the test of the next stage's barrier is issued before this stage's MMAs.
        // kind::f16: D fp32, A/B fp16, both K-major, M = 128 weight rows, N = m_pad tokens
        const uint32_t idesc = (1u << 4) | ((uint32_t)(a.m_pad >> 3) << 17) | ((uint32_t)(PK_ROWS >> 4) << 24);
        const int p = warp == 7 ? 1 : 0;
        const bool leader = elect_one();
        bool ok = true;
        bool pre = p < nst && mbar_test(bar_efull + 8 * ((uint32_t)p % ne), ((uint32_t)p / ne) & 1u);
        int j = 0, first = 0;
        for (int pc = 0; pc < 3 && ok; ++pc)
        for (int g = pc_s[pc], gend = pc_s[pc] + pc_n[pc]; g < gend && ok; ++j) {
            const int kb = g % a.nblk;
            const int len = min(a.nblk - kb, gend - g);
            const uint32_t buf = a.acc_bufs == 2u ? (uint32_t)j & 1u : 0u, use = a.acc_bufs == 2u ? (uint32_t)j >> 1 : (uint32_t)j;
            // the epilogue must have drained this accumulator pair's previous segment
            if (!(ok = mbar_wait_warp(bar_aempty + 8 * buf, (use & 1u) ^ 1u, abort_flag, 7, a.poll_limit))) break;
            const uint32_t d_tmem = tmem_base + (2u * buf + (uint32_t)p) * a.acc_cols;
            bool fresh = true;                                   // this issuer's first MMA of the segment overwrites
            for (int i = first + ((p - first) & 1); i < first + len; i += 2) {
                const uint32_t es = (uint32_t)i % ne, eph = ((uint32_t)i / ne) & 1u;
                // weights expanded (or landed) and X tiles landed
                if (!__all_sync(0xFFFFFFFFu, pre) && !(ok = mbar_wait_warp(bar_efull + 8 * es, eph, abort_flag, 3, a.poll_limit))) break;
                tc_fence_after();
                const uint32_t ni = (uint32_t)i + 2u;
                const bool nxt = (int)ni < nst && mbar_test(bar_efull + 8 * (ni % ne), (ni / ne) & 1u);
                if (leader) {
                    const uint32_t wa = exp0 + es * ES, xa = wa + WB;
                    const uint32_t wt = tmem_base + 2u * a.acc_bufs * a.acc_cols + es * 64u;      // the expanded stage in tensor memory
                    #pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        #pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const uint64_t xd = umma_desc(xa + h * ((uint32_t)a.m_pad * 128u) + kk * 32);
                            const uint32_t acc = (!fresh || (h | kk) != 0) ? 1u : 0u;
                            if (CB == 16) tc_mma_f16(d_tmem, umma_desc(wa + h * (PK_ROWS * 128) + kk * 32), xd, idesc, acc);
                            else tc_mma_f16_ts(d_tmem, wt + (uint32_t)(h * 4 + kk) * 8u, xd, idesc, acc);
                        }
                    }
                    tc_commit(bar_eempty + 8 * es);
                }
                __syncwarp();
                fresh = false;
                pre = nxt;
            }
            if (!ok) break;
            // both issuers report the segment, also the one that had no stage in it (its commit completes at once)
            if (leader) tc_commit(bar_afull + 8 * buf);
            __syncwarp();
            first += len;
            g += len;
        }
    } else if (warp >= PK_SERVICE0) {
        // ================= waiter / reporter of expansion group p =================
        // Hardware barriers, three ids per purpose and group, taken in turn by the group's stages: 2 + p + 2k "stage
        // released", 8 + p + 2k "stage stored" (k = 0, 1, 2).  A group owns at most three operand slots, so its waiter is
        // at most two stages ahead of it (a slot frees only after the MMAs of a stage the group has finished) and the
        // group at most two stages ahead of its reporter (the MMAs need the reporter's arrival): an early arrival never
        // falls into a phase of the same barrier that is still open.
        if (CB != 16) {
            const int p = (warp - PK_SERVICE0) & 1;
            const bool reporter = warp >= PK_SERVICE0 + 2;
            const uint32_t nl = (uint32_t)a.nl, odd = (uint32_t)lane & 1u;
            // every operand slot is free at the start: the X tiles of the group's first stages leave at once, under the
            // flight of the first records
            if (!reporter && lane == 0) {
                for (int i = p; i < nst && i < (int)ne; i += 2) {
                    const uint32_t dst = exp0 + (uint32_t)i * ES + WB, bar = bar_efull + 8 * (uint32_t)i;
                    const int kb = stage_g(i) % a.nblk;
                    mbar_expect_tx(bar, (uint32_t)a.m_pad * 256u);
                    tma_load_2d(dst, &mapX, kb * PK_KB, 0, bar);
                    tma_load_2d(dst + (uint32_t)a.m_pad * 128u, &mapX, kb * PK_KB + 64, 0, bar);
                }
            }
            __syncwarp();
            for (int i = p, k = 0; i < nst; i += 2, k = k == 2 ? 0 : k + 1) {
                const uint32_t ls = (uint32_t)i % nl, lph = ((uint32_t)i / nl) & 1u, es = (uint32_t)i % ne, eph = ((uint32_t)i / ne) & 1u;
                if (!reporter) {
                    // lane 0 (and the idle lanes): record landed; lane 1: operand slot free -- one instruction, two addresses
                    const bool ok = mbar_wait_pair(bar_lfull + 8 * ls, lph, bar_eempty + 8 * es, eph ^ 1u, abort_flag, 4, a.poll_limit);
                    asm volatile("bar.arrive %0, 288;" ::"r"(2 + p + 2 * k) : "memory");   // (on failure: the group leaves)
                    if (!ok) break;
                    if (lane == 0 && i >= (int)ne) {
                        // the slot is free: the tokens' two K tiles of this stage go into it; their bytes complete the same
                        // barrier as the reporter's arrival, so an MMA thread waits once per stage
                        const uint32_t dst = exp0 + es * ES + WB, bar = bar_efull + 8 * es;
                        const int kb = stage_g(i) % a.nblk;
                        mbar_expect_tx(bar, (uint32_t)a.m_pad * 256u);
                        tma_load_2d(dst, &mapX, kb * PK_KB, 0, bar);
                        tma_load_2d(dst + (uint32_t)a.m_pad * 128u, &mapX, kb * PK_KB + 64, 0, bar);
                    }
                    __syncwarp();
                } else {
                    asm volatile("bar.sync %0, 288;" ::"r"(8 + p + 2 * k) : "memory");
                    if (*abort_flag) break;
                    if (lane < 2) mbar_arrive(odd ? bar_lempty + 8 * ls : bar_efull + 8 * es);
                }
            }
        }
    } else if (warp >= PK_EXP_WARP0 && CB != 16) {
        // ================= expansion =================
        // Two groups of eight warps take alternate stages, so that one group's arithmetic runs under the other's
        // stores, fence and barrier traffic; thread (row r, half hh) of a group turns 64 codes into the 8 chunks of its
        // row in one of the stage's two 64-wide K tiles.
        const int te = threadIdx.x - PK_EXP_WARP0 * 32;
        const int grp = te >> 8, tg = te & 255;
        const int r = tg & (PK_ROWS - 1), hh = tg >> 7;
        const uint32_t nl = (uint32_t)a.nl;
        // The group touches no mbarrier: a test or an arrival costs the issuing warp several hundred cycles of latency,
        // which with eight per stage was as much as the expansion itself.  Its waiter warp sees the stage's barriers and
        // releases it through a hardware barrier, its reporter warp announces the finished stage.
        for (int i = grp, k = 0; i < nst; i += 2, k = k == 2 ? 0 : k + 1) {
            const uint32_t ls = (uint32_t)i % nl, es = (uint32_t)i % ne;
            asm volatile("bar.sync %0, 288;" ::"r"(2 + grp + 2 * k) : "memory");
            if (*abort_flag) { asm volatile("bar.arrive %0, 288;" ::"r"(8 + grp + 2 * k) : "memory"); break; }
            const uint32_t rec = ld0 + ls * LS;
            // this thread's 64 codes: 16-byte pieces, rows contiguous inside a piece (2 pieces of 32 codes, or 4 of 16)
            constexpr int NP = CB / 2;
            uint32_t l2w, meta, cw[4 * NP];
            asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(l2w), "=r"(meta) : "r"(rec + CODE_BYTES + r * 8));
            #pragma unroll
            for (int p = 0; p < NP; ++p)
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(cw[4 * p]), "=r"(cw[4 * p + 1]), "=r"(cw[4 * p + 2]), "=r"(cw[4 * p + 3])
                             : "r"(rec + ((NP * hh + p) * PK_ROWS + r) * 16));
            const uint32_t sc = meta & 0xFFFFu, s2 = sc * 0x10001u, tb = (meta >> 16) & 1u;
            const uint32_t base2 = tb ? a.base2[1] : a.base2[0], step2 = tb ? a.step2[1] : a.step2[0];
            // a scale in fp16's top binade could overflow t*s where (level*t)*s stays finite: multiply in two steps there
            // (the stores below are warp-collective, so the rare case is a select inside a warp-uniform branch)
            const bool two_step = sc >= 0x7800u;
            const bool any_two = __any_sync(0xFFFFFFFFu, two_step);
            // this half's micro-scale indices: chunk 8hh + c of the block, one index per 2^MS chunks
            const uint32_t l2q = l2w >> (2 * ((8 * hh) >> MS));
            // the stage in tensor memory: lane = weight row (this warp's quarter), 64 columns of two k each; this thread
            // writes columns 32 hh + 4 c + {0..3} for its chunk c
            const uint32_t out = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + 2u * a.acc_bufs * a.acc_cols + es * 64u + (uint32_t)hh * 32u;
            uint32_t t2 = 0u, ts2 = 0u;
            #pragma unroll
            for (int c = 0; c < 8; ++c) {
                if (MS == 0 || (c & 3) == 0) {
                    const uint32_t idx = (l2q >> (2 * (c >> MS))) & 3u;
                    t2 = base2 + idx * step2;
                    ts2 = h2_bits(__hmul2(bits_h2(t2), bits_h2(s2)));
                }
                uint32_t o[4];
                if (CB == 4) expand8<false>(cw[c], ts2, t2, s2, o);
                else expand8_bytes<false>(cw[(2 * c) % (4 * NP)], cw[(2 * c + 1) % (4 * NP)], ts2, t2, s2, o);
                if (any_two) {
                    uint32_t o2[4];
                    if (CB == 4) expand8<true>(cw[c], 0u, t2, s2, o2);
                    else expand8_bytes<true>(cw[(2 * c) % (4 * NP)], cw[(2 * c + 1) % (4 * NP)], 0u, t2, s2, o2);
                    #pragma unroll
                    for (int p = 0; p < 4; ++p) o[p] = two_step ? o2[p] : o[p];
                }
                tc_st4(out + 4u * (uint32_t)c, o);
            }
            // the stores have landed in tensor memory, and are ordered before the arrival that the MMA thread will see
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            asm volatile("bar.arrive %0, 288;" ::"r"(8 + grp + 2 * k) : "memory");
        }
    } else if (warp < PK_EPI_WARPS) {
        // ================= epilogue (warps 0-3: one per quarter of the tensor-memory lanes) =================
        const int quarter = warp, nloc = quarter * 32 + lane;          // this thread's weight row inside the tile
        bool ok = true;
        if (warp == 0 && lane < 12) {
            // The fix-up is a chain of dependent round trips to memory this SM has not touched yet (counters, partial
            // sums, C), and each first touch pays an address-translation miss of a few microseconds.  Touch those pages
            // now, while the first stages are on their way; the values are not used.
            const int ta = g0 / a.nblk, tb = (g1 - 1) / a.nblk;
            const char* pz = nullptr;
            switch (lane) {
            case 0: pz = (const char*)(a.counters + ta); break;
            case 1: pz = (const char*)(a.counters + tb); break;
            case 2: pz = (const char*)(a.ws + (int64_t)cta * 2 * a.m_pad * PK_ROWS); break;
            case 3: pz = (const char*)(a.ws + ((int64_t)cta * 2 + 2) * a.m_pad * PK_ROWS - 1); break;
            case 4: pz = (const char*)(a.ws + (int64_t)max(cta - 2, 0) * 2 * a.m_pad * PK_ROWS); break;
            case 5: pz = (const char*)(a.ws + ((int64_t)min(cta + 2, G - 1) * 2 + 2) * a.m_pad * PK_ROWS - 1); break;
            case 6: pz = (const char*)(a.C + ta * PK_ROWS); break;
            case 7: pz = (const char*)(a.C + (int64_t)(a.M - 1) * a.N + ta * PK_ROWS + PK_ROWS - 1); break;
            case 8: pz = (const char*)(a.C + tb * PK_ROWS); break;
            case 9: pz = (const char*)(a.C + (int64_t)(a.M - 1) * a.N + tb * PK_ROWS + PK_ROWS - 1); break;
            case 10: pz = a.bias ? (const char*)(a.bias + ta * PK_ROWS) : nullptr; break;
            default: pz = a.bias ? (const char*)(a.bias + tb * PK_ROWS) : nullptr; break;
            }
            if (pz) {
                uint32_t unused;
                asm volatile("ld.global.cg.u8 %0, [%1];" : "=r"(unused) : "l"(pz) : "memory");
            }
        }
        int j = 0, first = 0;
        for (int pc = 0; pc < 3 && ok; ++pc)
        for (int g = pc_s[pc], gend = pc_s[pc] + pc_n[pc]; g < gend; ++j) {
            const int tile = g / a.nblk, kb = g % a.nblk;
            const int len = min(a.nblk - kb, gend - g);
            // issuer p accumulated the segment's stages of parity p: a one-stage segment has only one of the two
            const bool has0 = len >= 2 || (first & 1) == 0, has1 = len >= 2 || (first & 1) == 1;
            first += len;
            g += len;
            const uint32_t buf = a.acc_bufs == 2u ? (uint32_t)j & 1u : 0u, use = a.acc_bufs == 2u ? (uint32_t)j >> 1 : (uint32_t)j;
            const bool whole = len == a.nblk;
            // the tile's segments sit in consecutive CTAs
            int c_first = cta, c_last = cta;
            bool closing = false;
            if (!whole && !a.split) {
                c_first = cta_of_stage(a, tile * a.nblk);
                c_last = cta_of_stage(a, tile * a.nblk + a.nblk - 1);
                // This CTA ends the tile: while its MMAs still run, see whether every other CTA of the tile has already
                // published its partial sums.  Then the tile is completed from the accumulator, with no partial sums of
                // this CTA, no fence and no count on the way.
                if (cta == c_last) {
                    if (threadIdx.x == 0) {
                        int seen;
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(a.counters + tile) : "memory");
                        *last_flag = seen == c_last - c_first;
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    closing = *last_flag != 0;
                    asm volatile("bar.sync 1, 128;" ::: "memory");    // everyone has read the flag before its next use
                    if (closing) __threadfence();
                }
            }
            ok = ok && mbar_wait_parked_warp(bar_afull + 8 * buf, use & 1u, abort_flag, 6, park_limit);
            if (!ok) break;
            tc_fence_after();
            const int gn = tile * PK_ROWS + nloc;
            float* part = a.ws + ((int64_t)cta * 2 + (tile == g0 / a.nblk ? 0 : 1)) * a.m_pad * PK_ROWS + nloc;
            const __half bv = a.bias ? a.bias[gn] : __float2half_rn(0.f);
            for (int c0 = 0; c0 < a.m_pad; c0 += 16) {
                float v[16];
                {
                    float v1[16];
                    tc_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (2u * buf) * a.acc_cols + c0, v);
                    tc_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (2u * buf + 1u) * a.acc_cols + c0, v1);
                    #pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = (has0 ? v[i] : 0.f) + (has1 ? v1[i] : 0.f);   // even + odd stages
                }
                if (closing) {
                    // the other CTAs' partial sums in CTA order, this CTA's accumulator last: the order of the fix-up below
                    float acc[16];
                    #pragma unroll
                    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
                    for (int cc = c_first; cc < c_last; ++cc) {
                        const int slot = tile == run_begin(a, cc) / a.nblk ? 0 : 1;
                        const float* q = a.ws + ((int64_t)cc * 2 + slot) * a.m_pad * PK_ROWS + nloc;
                        float w[16];
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) w[i] = c0 + i < a.M ? __ldcg(q + (int64_t)(c0 + i) * PK_ROWS) : 0.f;
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) acc[i] += w[i];
                    }
                    #pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] += acc[i];
                }
                if (a.split) {
                    // the cluster adds the parts of the tile from its CTAs' shared memory (teardown)
                    #pragma unroll
                    for (int i = 0; i < 16; ++i)
                        asm volatile("st.shared.f32 [%0], %1;" ::"r"(stg + (uint32_t)((c0 + i) * PK_ROWS + nloc) * 4u), "f"(v[i]) : "memory");
                } else if (whole || closing) {
                    __half* cp = a.C + (int64_t)c0 * a.N + gn;
                    #pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        __half o = __float2half_rn(v[i]);
                        if (a.bias) o = __hadd(o, bv);
                        if (c0 + i < a.M) cp[(int64_t)i * a.N] = o;
                    }
                } else {
                    #pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (c0 + i < a.M) part[(int64_t)(c0 + i) * PK_ROWS] = v[i];
                }
            }
            // the accumulator has been read: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_aempty + 8 * buf);
            if (closing) {
                if (threadIdx.x == 0) a.counters[tile] = 0;
            } else if (!whole && !a.split) {
                // the CTA that arrives last adds the tile's partial sums in CTA order.
                // Every thread orders its own partial sums before the count (a fence by the counting thread alone, after
                // the barrier, was seen to let a reader on another SM run ahead of a warp's stores)
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 0) {
                    int old;
                    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(a.counters + tile) : "memory");
                    *last_flag = old == c_last - c_first;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const bool last = *last_flag != 0;
                asm volatile("bar.sync 1, 128;" ::: "memory");        // everyone has read the flag before its next use
                if (last) {
                    __threadfence();
                    for (int m0 = 0; m0 < a.M; m0 += 16) {            // sixteen rows, two segments: 32 loads in flight
                        float acc[16];
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) acc[i] = 0.f;
                        for (int cc = c_first; cc <= c_last; cc += 2) {
                            float v[2][16];
                            #pragma unroll
                            for (int u = 0; u < 2; ++u) {
                                const int cu = cc + u <= c_last ? cc + u : c_last;
                                const int slot = tile == run_begin(a, cu) / a.nblk ? 0 : 1;
                                const float* p = a.ws + ((int64_t)cu * 2 + slot) * a.m_pad * PK_ROWS + nloc;
                                #pragma unroll
                                for (int i = 0; i < 16; ++i)
                                    v[u][i] = (cc + u <= c_last && m0 + i < a.M) ? __ldcg(p + (int64_t)(m0 + i) * PK_ROWS) : 0.f;
                            }
                            #pragma unroll
                            for (int u = 0; u < 2; ++u) {
                                #pragma unroll
                                for (int i = 0; i < 16; ++i) acc[i] += v[u][i];
                            }
                        }
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            if (m0 + i >= a.M) break;
                            __half o = __float2half_rn(acc[i]);
                            if (a.bias) o = __hadd(o, bv);
                            a.C[(int64_t)(m0 + i) * a.N + gn] = o;
                        }
                    }
                    if (threadIdx.x == 0) a.counters[tile] = 0;
                }
            }
        }
    }

    // ---- teardown: every role arrives here, also after an expired wait ----
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const unsigned long long t0 = gtime_ns();
        while (gtime_ns() - t0 < 200000ull) { }          // copies that may still be in flight land before smem is released
        __syncthreads();
    }
    if (a.split) {
        // Every CTA of the cluster has left its part of the tile (fp32, [token][row]) at the start of its record ring
        // (fp16 weight: of its operand stages).
        // Each CTA adds a share of the tokens, reading all parts in rank order through distributed shared memory, and
        // writes C; the second barrier keeps every CTA's shared memory alive until all have read it.  Every thread of the
        // cluster reaches both barriers.
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (warp < PK_EPI_WARPS && !*abort_flag) {
            // CTA `rank` adds the tokens of its share, reading every CTA's part in rank order
            const int nloc = threadIdx.x, gn = split_tile * PK_ROWS + nloc;
            const __half bv = a.bias ? a.bias[gn] : __float2half_rn(0.f);
            const int m_lo = a.M * split_rank / a.split, m_hi = a.M * (split_rank + 1) / a.split;
            for (int m0 = m_lo; m0 < m_hi; m0 += 8) {
                float acc[8];
                #pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = 0.f;
                for (int r = 0; r < a.split; r += 2) {
                    float w[2][8];
                    #pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        uint32_t remote;
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(stg + (uint32_t)nloc * 4u), "r"(min(r + u, a.split - 1)));
                        #pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            w[u][i] = 0.f;
                            if (r + u < a.split && m0 + i < m_hi)
                                asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(w[u][i]) : "r"(remote + (uint32_t)((m0 + i) * PK_ROWS) * 4u) : "memory");
                        }
                    }
                    #pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        #pragma unroll
                        for (int i = 0; i < 8; ++i) acc[i] += w[u][i];
                    }
                }
                #pragma unroll
                for (int i = 0; i < 8; ++i) {
                    __half o = __float2half_rn(acc[i]);
                    if (a.bias) o = __hadd(o, bv);
                    if (m0 + i < m_hi) a.C[(int64_t)(m0 + i) * a.N + gn] = o;
                }
            }
        }
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    if (warp == 5) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(a.tmem_cols) : "memory");
    }
}

// ---- one token: no tensor core --------------------------------------------------------------------------------
// For M = 1 the MMA paths' cost per stage (eight MMAs of fixed cost, barriers) is several times the record's time on
// HBM.  Here a warp owns 32 weight rows (lane = row) and every KS-th 128-k block of them: it reads its part of the
// record with plain 16-byte loads (a warp's lanes cover 512 contiguous bytes of a piece), expands eight codes at a
// time exactly as the MMA path does and multiplies with the tokens' values from shared memory (the same address in
// every lane: a broadcast) in fma.rn.f32.f16 -- the product of two fp16 values is exact in fp32, the sum is fp32.
// The KS warps of a CTA meet in shared memory and are added in warp order, so results do not vary from run to run;
// nothing is shared between CTAs.
struct GvArgs {
    const uint8_t* wp;
    const __half* x;            // [M, K]
    __half* C;                  // [M, N]
    const __half* bias;
    int M, N, K, nblk, ks;
    uint32_t base2[2], step2[2];
};

__device__ __forceinline__ void fma2_f32(float& acc, uint32_t w2, uint32_t x2)
{
    asm("{ .reg .b16 wl, wh, xl, xh;\n mov.b32 {wl, wh}, %1;\n mov.b32 {xl, xh}, %2;\n"
        " fma.rn.f32.f16 %0, wl, xl, %0;\n fma.rn.f32.f16 %0, wh, xh, %0; }" : "+f"(acc) : "r"(w2), "r"(x2));
}

template <int MS>
__global__ void __launch_bounds__(512) gemv_packed_kernel(const GvArgs a)
{
    constexpr int MT = 1;                                                       // tokens
    extern __shared__ uint8_t gv_smem[];
    uint4* xs = reinterpret_cast<uint4*>(gv_smem);                               // [MT][K] fp16
    float* red = reinterpret_cast<float*>(gv_smem + (size_t)MT * a.K * 2);        // [ks][MT][32]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    {
        const uint4* src = reinterpret_cast<const uint4*>(a.x);
        const int n16 = a.M * a.K / 8;
        for (int i = threadIdx.x; i < MT * a.K / 8; i += blockDim.x) xs[i] = i < n16 ? __ldg(src + i) : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    const int unit = blockIdx.x, tile = unit >> 2, r = (unit & 3) * 32 + lane;    // this lane's row inside the tile
    const uint8_t* rec0 = a.wp + (int64_t)tile * a.nblk * pk_rec_bytes(4);
    float acc[MT];
    #pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    uint4 cw[4], nw[4];
    uint2 side, nside;
    auto fetch = [&](int kb, uint4* c, uint2& sd) {
        const uint8_t* rec = rec0 + (int64_t)kb * pk_rec_bytes(4);
        #pragma unroll
        for (int q = 0; q < 4; ++q)
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(c[q].x), "=r"(c[q].y), "=r"(c[q].z), "=r"(c[q].w) : "l"(rec + (q * PK_ROWS + r) * 16));
        asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(sd.x), "=r"(sd.y) : "l"(rec + pk_code_bytes(4) + r * 8));
    };
    int kb = warp;
    if (kb < a.nblk) fetch(kb, nw, nside);
    for (; kb < a.nblk; kb += a.ks) {
        #pragma unroll
        for (int q = 0; q < 4; ++q) cw[q] = nw[q];
        side = nside;
        if (kb + a.ks < a.nblk) fetch(kb + a.ks, nw, nside);                      // the next record is on its way under this one
        const uint32_t l2w = side.x, meta = side.y;
        const uint32_t sc = meta & 0xFFFFu, s2 = sc * 0x10001u, tb = (meta >> 16) & 1u;
        const uint32_t base2 = tb ? a.base2[1] : a.base2[0], step2 = tb ? a.step2[1] : a.step2[0];
        const bool two_step = sc >= 0x7800u;                                     // as in the MMA path's expansion
        uint32_t t2 = 0u, ts2 = 0u;
        #pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t w4[4] = {cw[q].x, cw[q].y, cw[q].z, cw[q].w};
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int cb = 4 * q + j;                                        // chunk of 8 k inside the block
                if (MS == 0 || (cb & 3) == 0) {
                    const uint32_t idx = (l2w >> (2 * (cb >> MS))) & 3u;
                    t2 = base2 + idx * step2;
                    ts2 = h2_bits(__hmul2(bits_h2(t2), bits_h2(s2)));
                }
                uint32_t o[4];
                if (!two_step) expand8<false>(w4[j], ts2, t2, s2, o);
                else expand8<true>(w4[j], 0u, t2, s2, o);
                #pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const uint4 xv = xs[(m * a.K + kb * PK_KB + cb * 8) >> 3];
                    fma2_f32(acc[m], o[0], xv.x);
                    fma2_f32(acc[m], o[1], xv.y);
                    fma2_f32(acc[m], o[2], xv.z);
                    fma2_f32(acc[m], o[3], xv.w);
                }
            }
        }
    }
    #pragma unroll
    for (int m = 0; m < MT; ++m) red[(warp * MT + m) * 32 + lane] = acc[m];
    __syncthreads();
    if (warp == 0) {
        const int gn = tile * PK_ROWS + r;
        #pragma unroll
        for (int m = 0; m < MT; ++m) {
            float sum = 0.f;
            for (int w = 0; w < a.ks; ++w) sum += red[(w * MT + m) * 32 + lane];
            __half o = __float2half_rn(sum);
            if (a.bias) o = __hadd(o, a.bias[gn]);
            if (m < a.M) a.C[(int64_t)m * a.N + gn] = o;
        }
    }
}

// ---- two to eight tokens: the warp-level MMA with the weights in registers -----------------------------------
// tcgen05 pays per 128-k stage eight MMAs of fixed cost and a chain of barriers, about twice the record's time on HBM.
// For M <= 8 the product also fits ONE mma.sync m16n8k16 per 16 x 16 weights (a second column tile for 9-16 tokens costs
// more than the tcgen05 path: on B200 this MMA runs at a sixteenth of the tcgen05 rate) with the A operand straight from the expanding thread's
// registers: no shared memory, no barrier, no hand-off between warps.  A warp owns 32 weight rows (two groups of 16)
// and every ks-th 128-k block; lane (g, t) = (lane / 4, lane % 4) loads the 16-byte piece t (32 consecutive codes) of
// rows g and g + 8, expands it as the tcgen05 path does, and uses the four pairs of each word as the A fragments of two
// MMAs.  The MMA adds over its 16 columns whatever k they stand for, so columns (2t, 2t+1, 2t+8, 2t+9) of step s are
// k = 32t + 4s + (0..3), and the B fragment of token n = g is X[n][those k]: one 16-byte load per word serves both steps.  Products are exact in fp32 and the sums are fp32.  The ks warps of a slab meet in shared memory
// and are added in order (results do not vary from run to run); CTAs share nothing.
struct RgArgs {
    const uint8_t* wp;
    const __half* x;            // [M, K]
    __half* C;                  // [M, N]
    const __half* bias;
    int M, N, K, nblk, ks, slabs;
    uint32_t base2[2], step2[2];
};

__device__ __forceinline__ void mma_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int MS>
__global__ void __launch_bounds__(512) gemm_packed_reg_kernel(const RgArgs a)
{
    constexpr int NT = 1;                                                       // column tiles of 8 tokens
    extern __shared__ float rg_red[];                                           // [ks][slabs][32 lanes][8 NT]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int slab = warp % a.slabs, ksp = warp / a.slabs;
    const int row0 = (blockIdx.x * a.slabs + slab) * 32, tile = row0 >> 7, rt = row0 & (PK_ROWS - 1);
    const uint8_t* rec0 = a.wp + (int64_t)tile * a.nblk * pk_rec_bytes(4);
    float c[2][NT][4];
    #pragma unroll
    for (int G2 = 0; G2 < 2; ++G2)
        #pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            #pragma unroll
            for (int i = 0; i < 4; ++i) c[G2][nt][i] = 0.f;
    uint4 cw[2][2], nw[2][2];                                                   // [group][row g / g + 8]: piece t of the row
    uint2 sd[2][2], nsd[2][2];
    auto fetch = [&](int kb, uint4 (*w)[2], uint2 (*s)[2]) {
        const uint8_t* rec = rec0 + (int64_t)kb * pk_rec_bytes(4);
        #pragma unroll
        for (int G2 = 0; G2 < 2; ++G2)
            #pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = rt + 16 * G2 + g + 8 * h;
                asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(w[G2][h].x), "=r"(w[G2][h].y), "=r"(w[G2][h].z), "=r"(w[G2][h].w) : "l"(rec + (t * PK_ROWS + row) * 16));
                asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(s[G2][h].x), "=r"(s[G2][h].y) : "l"(rec + pk_code_bytes(4) + row * 8));
            }
    };
    int kb = ksp;
    if (kb < a.nblk) fetch(kb, nw, nsd);
    for (; kb < a.nblk; kb += a.ks) {
        #pragma unroll
        for (int G2 = 0; G2 < 2; ++G2)
            #pragma unroll
            for (int h = 0; h < 2; ++h) {
                cw[G2][h] = nw[G2][h];
                sd[G2][h] = nsd[G2][h];
            }
        if (kb + a.ks < a.nblk) fetch(kb + a.ks, nw, nsd);                        // the next record is on its way under this one
        // token n = g (+ 8) of this lane: eight consecutive k per word (cached: the slabs of a CTA read the same lines)
        uint4 xv[4][NT];
        #pragma unroll
        for (int q = 0; q < 4; ++q)
            #pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int n = g + 8 * nt;
                xv[q][nt] = n < a.M ? __ldg(reinterpret_cast<const uint4*>(a.x + (int64_t)n * a.K + kb * PK_KB + 32 * t + 8 * q))
                                    : make_uint4(0u, 0u, 0u, 0u);
            }
        #pragma unroll
        for (int G2 = 0; G2 < 2; ++G2) {
            uint32_t s2[2], base2[2], step2[2];
            bool two_step[2];
            #pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t meta = sd[G2][h].y, sc = meta & 0xFFFFu, tb = (meta >> 16) & 1u;
                s2[h] = sc * 0x10001u;
                base2[h] = tb ? a.base2[1] : a.base2[0];
                step2[h] = tb ? a.step2[1] : a.step2[0];
                two_step[h] = sc >= 0x7800u;                                     // as in the tcgen05 path's expansion
            }
            #pragma unroll
            for (int q = 0; q < 4; ++q) {                                        // word q of the lane's piece
                const int cb = 4 * t + q;                                        // its chunk of 8 k inside the block
                uint32_t o[2][4];
                #pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t word = q == 0 ? cw[G2][h].x : q == 1 ? cw[G2][h].y : q == 2 ? cw[G2][h].z : cw[G2][h].w;
                    const uint32_t idx = (sd[G2][h].x >> (2 * (cb >> MS))) & 3u;
                    const uint32_t t2 = base2[h] + idx * step2[h];
                    if (!two_step[h]) expand8<false>(word, h2_bits(__hmul2(bits_h2(t2), bits_h2(s2[h]))), t2, s2[h], o[h]);
                    else expand8<true>(word, 0u, t2, s2[h], o[h]);
                }
                #pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    mma_16816(c[G2][nt], o[0][0], o[1][0], o[0][1], o[1][1], xv[q][nt].x, xv[q][nt].y);
                    mma_16816(c[G2][nt], o[0][2], o[1][2], o[0][3], o[1][3], xv[q][nt].z, xv[q][nt].w);
                }
            }
        }
    }
    float* mine = rg_red + ((size_t)(ksp * a.slabs + slab) * 32 + lane) * (8 * NT);
    #pragma unroll
    for (int G2 = 0; G2 < 2; ++G2)
        #pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            #pragma unroll
            for (int i = 0; i < 4; ++i) mine[(G2 * NT + nt) * 4 + i] = c[G2][nt][i];
    __syncthreads();
    if (ksp == 0) {
        #pragma unroll
        for (int G2 = 0; G2 < 2; ++G2)
            #pragma unroll
            for (int nt = 0; nt < NT; ++nt)
                #pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float sum = 0.f;
                    for (int w = 0; w < a.ks; ++w) sum += rg_red[((size_t)(w * a.slabs + slab) * 32 + lane) * (8 * NT) + (G2 * NT + nt) * 4 + i];
                    const int gn = row0 + 16 * G2 + g + (i >> 1) * 8, m = 8 * nt + 2 * t + (i & 1);
                    __half o = __float2half_rn(sum);
                    if (a.bias) o = __hadd(o, a.bias[gn]);
                    if (m < a.M) a.C[(int64_t)m * a.N + gn] = o;
                }
    }
}

// ---- prepack: the planes of hbq_quantize -> the per-(tile, block) records above --------------------------
struct PrepackArgs {
    const uint8_t* codes;       // [N, K/2]
    const uint8_t* scale_u8;    // [N, nblk]
    const uint8_t* l2;          // [N, nblk, l2_bytes]
    const uint8_t* scheme;      // [N, nblk] or NULL
    uint4* out;
    int64_t total;              // 16-byte slots of the output
    int K, nblk, l2_bytes;
};

template <int CB>
__global__ void __launch_bounds__(256) gemm_w4_prepack_kernel(const PrepackArgs a)
{
    constexpr int CODE_SLOTS = pk_code_bytes(CB) / 16;        // 16-byte slots of codes per record: 512 or 1024
    constexpr int SLOTS = pk_rec_bytes(CB) / 16;              // ... plus 64 of side records
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.total) return;
    const int slot = (int)(i % SLOTS);
    const int64_t rec = i / SLOTS;
    const int kb = (int)(rec % a.nblk);
    const int64_t tile = rec / a.nblk;
    if (slot < CODE_SLOTS) {
        const int q = slot >> 7, r = slot & 127;                                   // piece, row
        const uint8_t* src = a.codes + (tile * PK_ROWS + r) * (int64_t)(a.K / 2) + kb * 64;
        if (CB == 4) {
            a.out[i] = *reinterpret_cast<const uint4*>(src + q * 16);             // 32 codes as they are
        } else {
            // 16 codes -> the top bytes of their E2M1 values 0, .5, 1, 1.5, 2, 3, 4, 6 as fp16, sign in bit 7
            const uint2 nib = *reinterpret_cast<const uint2*>(src + q * 8);
            const unsigned long long n64 = ((unsigned long long)nib.y << 32) | nib.x;
            constexpr unsigned long long LUT = 0x464442403E3C3800ull;
            uint32_t w[4] = {0u, 0u, 0u, 0u};
            #pragma unroll
            for (int e = 0; e < 16; ++e) {
                const uint32_t c = (uint32_t)(n64 >> (4 * e)) & 0xFu;
                const uint32_t b = (uint32_t)(LUT >> (8 * (c & 7u))) & 0xFFu;
                w[e >> 2] |= (b | ((c & 8u) << 4)) << (8 * (e & 3));
            }
            a.out[i] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
        uint32_t w[4];
        #pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int64_t blk = (tile * PK_ROWS + (slot - CODE_SLOTS) * 2 + j) * a.nblk + kb;
            uint32_t l2w = 0;
            for (int b = 0; b < a.l2_bytes; ++b) l2w |= (uint32_t)a.l2[blk * a.l2_bytes + b] << (8 * b);
            w[2 * j] = l2w;
            w[2 * j + 1] = ((uint32_t)a.scale_u8[blk] << 7) | ((a.scheme ? (uint32_t)(a.scheme[blk] & 1u) : 0u) << 16);
        }
        a.out[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// ---- host side ---------------------------------------------------------------------------------------
// Formats the kernel expands: HBQ weights with E2M1 elements, an E5M3 scale per 128 and 2-bit micro-scales per 8 or 32
// whose candidates are base + idx * step in fp16 (the "Mix" pair and its members; not SIG-1 / INT / POT).
static bool w4_format(const hbq_format* f, PkArgs* a, int* micro_shift)
{
    if (!f || f->kind != HBQ_KIND_HBQ || f->ebit != 2 || f->mbit != 1 || f->block_size != 128 || f->sc_ebit != 5 ||
        f->sc_mbit != 3 || f->l2_sc_bit != 2 || (f->l2_block_size != 8 && f->l2_block_size != 32))
        return false;
    uint32_t base[2] = {0x3C00u, 0x3C00u}, step[2] = {0x0100u, 0x0100u};
    switch (f->l2_scheme) {
        case HBQ_L2_FPM1: break;
        case HBQ_L2_FP1: base[0] = 0x3D00u; break;
        case HBQ_L2_FPM10: step[0] = 0x0080u; break;
        case HBQ_L2_FPM100: step[0] = 0x0040u; break;
        case HBQ_L2_MIX: step[1] = 0x0080u; break;
        default: return false;
    }
    if (a) {
        for (int i = 0; i < 2; ++i) { a->base2[i] = base[i] * 0x10001u; a->step2[i] = step[i] * 0x10001u; }
    }
    if (micro_shift) *micro_shift = f->l2_block_size == 8 ? 0 : 2;
    return true;
}

static bool w4_shape(int64_t M, int64_t N, int64_t K)
{
    return M >= 1 && M <= 128 && N >= PK_ROWS && (N % PK_ROWS) == 0 && K >= PK_KB && (K % PK_KB) == 0 &&
           N <= (1ll << 24) && K <= (1ll << 24) && (N / PK_ROWS) * (K / PK_KB) < (1ll << 30);
}

static bool w4_container(int cb) { return cb == 4 || cb == 8; }

int64_t gemm_w4_prepacked_bytes(int64_t N, int64_t K, int container_bits)
{
    if (N <= 0 || K <= 0 || (N % PK_ROWS) || (K % PK_KB) || !w4_container(container_bits)) return -1;
    return (N / PK_ROWS) * (K / PK_KB) * (int64_t)pk_rec_bytes(container_bits);
}

int gemm_w4_prepack(const hbq_packed_out* in, int64_t N, int64_t K, const hbq_format* f, int container_bits, void* out,
                    cudaStream_t stream)
{
    if (!in || !out || !in->codes || !in->scale_u8 || !in->l2_packed) return HBQ_ERR_ARG;
    if (!w4_format(f, nullptr, nullptr) || !w4_shape(1, N, K) || !w4_container(container_bits)) return HBQ_ERR_UNSUPPORTED;
    if (f->l2_scheme == HBQ_L2_MIX && !in->scheme) return HBQ_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(in->codes) | reinterpret_cast<uintptr_t>(out)) & 15) return HBQ_ERR_ALIGN;
    PrepackArgs a;
    a.codes = in->codes; a.scale_u8 = in->scale_u8; a.l2 = in->l2_packed;
    a.scheme = f->l2_scheme == HBQ_L2_MIX ? in->scheme : nullptr;
    a.out = (uint4*)out;
    a.K = (int)K; a.nblk = (int)(K / PK_KB); a.l2_bytes = (128 / f->l2_block_size) * 2 / 8;
    a.total = gemm_w4_prepacked_bytes(N, K, container_bits) / 16;
    const unsigned grid = (unsigned)((a.total + 255) / 256);
    if (container_bits == 4) gemm_w4_prepack_kernel<4><<<grid, 256, 0, stream>>>(a);
    else gemm_w4_prepack_kernel<8><<<grid, 256, 0, stream>>>(a);
    HBQ_LAUNCH_CHECK("gemm_w4_prepack_kernel");
    return HBQ_OK;
}

// The counters come first, so that launches of any token count find them (zeroed) at the same place.
static int64_t w4_counter_bytes(int64_t tiles) { return (tiles * 4 + 255) / 256 * 256; }

int64_t gemm_w4_workspace_bytes(int64_t M, int64_t N, int64_t K)
{
    if (!w4_shape(M, N, K)) return -1;
    int sms = 0;
    if (device_sms(&sms) != HBQ_OK) return -1;
    const int64_t tiles = N / PK_ROWS, m_pad = (M + 15) / 16 * 16;
    return w4_counter_bytes(tiles) + (int64_t)sms * 2 * m_pad * PK_ROWS * 4;   // one counter per tile, two partial-sum slots per CTA
}

template <int MS, int CB>
static int launch_packed(const CUtensorMap& mx, const CUtensorMap& mw, const PkArgs& a, int grid, size_t smem, cudaStream_t stream)
{
    { const int rc = ensure_dynamic_smem(gemm_packed_kernel<MS, CB>, smem); if (rc) return rc; }
    if (a.split) {
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(PK_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = (unsigned)a.split; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        HBQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_packed_kernel<MS, CB>, mx, mw, a));
    } else {
        gemm_packed_kernel<MS, CB><<<grid, PK_THREADS, smem, stream>>>(mx, mw, a);
    }
    HBQ_LAUNCH_CHECK("gemm_packed_kernel");
    return HBQ_OK;
}

// How many clusters of S CTAs of the kernel the device holds at once (0 on error); asked once per (kernel, S, smem).
template <int MS, int CB>
static int max_clusters_of(int S, size_t smem)
{
    static std::mutex mu;
    static int cached[9];
    static size_t cached_smem[9];
    std::lock_guard<std::mutex> lock(mu);
    if (cached_smem[S] == smem && cached[S] != 0) return cached[S] < 0 ? 0 : cached[S];
    if (ensure_dynamic_smem(gemm_packed_kernel<MS, CB>, smem)) return 0;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)(S * 64)); cfg.blockDim = dim3(PK_THREADS); cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)S; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_packed_kernel<MS, CB>, &cfg) != cudaSuccess) { (void)cudaGetLastError(); n = 0; }
    cached[S] = n > 0 ? n : -1;
    cached_smem[S] = smem;
    return n;
}
static int max_clusters(int ms, int cb, int S, size_t smem)
{
    if (cb == 4) return ms == 0 ? max_clusters_of<0, 4>(S, smem) : max_clusters_of<2, 4>(S, smem);
    return ms == 0 ? max_clusters_of<0, 8>(S, smem) : max_clusters_of<2, 8>(S, smem);
}

// Three ways to cut the work, costed in stages per CTA; sets a.split / a.whole_tiles and returns the grid:
//  - equal runs of (tile, block) records per SM: tiles are shared between CTAs, and the fix-up of a shared tile is a
//    chain of dependent round trips through memory worth about fourteen stages at 16 tokens, more with more tokens;
//  - whole tiles per CTA: nothing to fix up, but SMs idle where the tiles do not fill them;
//  - few tiles: a tile's K blocks split over the S CTAs of a thread-block cluster, whose parts meet in distributed
//    shared memory behind a cluster barrier (about two stages); S is the largest size whose clusters all fit on
//    the device at once and whose parts (fp32, m_pad x 128) fit the `staging_bytes` that are free by then.
static int choose_split(PkArgs& a, int sms, int ms, int cb, size_t smem, uint32_t staging_bytes)
{
    int grid = a.total < sms ? a.total : sms;
    a.run_q = a.total / grid;
    a.run_r = a.total % grid;
    const int grid_w = a.tiles < sms ? a.tiles : sms;
    const int64_t stages_w = (int64_t)((a.tiles + grid_w - 1) / grid_w) * a.nblk;
    const int64_t stages_k = (a.total + grid - 1) / grid + (int64_t)PK_FIXUP_STAGES * (a.m_pad / 16);   // partial sums grow with the tokens
    int S = sms / a.tiles;
    if (S > 8) S = 8;
    if (S > a.nblk) S = a.nblk;
    if (staging_bytes < (uint32_t)a.m_pad * PK_ROWS * 4u) S = 0;
    while (S >= 2 && (cb == 16 ? max_clusters_of<0, 16>(S, smem) : max_clusters(ms, cb, S, smem)) < a.tiles) --S;
    const int64_t stages_c = S >= 2 ? (a.nblk + S - 1) / S + PK_CLUSTER_STAGES : (1ll << 40);
    a.split = 0;
    a.whole_tiles = 0;
    if (stages_c < stages_w && stages_c <= stages_k) { a.split = S; grid = a.tiles * S; }
    else if (stages_w <= stages_k) { a.whole_tiles = 1; grid = grid_w; }
    return grid;
}

// The same pipeline on an fp16 weight [N, K] (no expansion: TMA puts the weight tiles straight into the operand
// stages): the fp32-accumulation GEMM for decode-sized M, where giving a CTA whole 128-column tiles over the full K
// would leave most SMs idle.  Equal runs of (tile, block) stages per SM; partial tiles meet in the workspace.
// With 32 KB of weight per stage and SM this form is bound by HBM (per-role cycle stamps: 1350-1550 cycles per stage,
// 4.3 TB/s over the kernel).
bool gemm_w16_eligible(int64_t M, int64_t N, int64_t K)
{
    int sms = 0;
    return w4_shape(M, N, K) && device_sms(&sms) == HBQ_OK && N / PK_ROWS <= sms;
}

int gemm_w16_launch(const void* X, const void* W, void* C, int64_t M, int64_t N, int64_t K, const void* bias, void* workspace,
                    cudaStream_t stream)
{
    if (!X || !W || !C || !workspace) return HBQ_ERR_ARG;
    if (!gemm_w16_eligible(M, N, K)) return HBQ_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(workspace)) & 15)
        return HBQ_ERR_ALIGN;
    if ((reinterpret_cast<uintptr_t>(C) | reinterpret_cast<uintptr_t>(bias)) & 1) return HBQ_ERR_ALIGN;
    PkArgs a;
    memset(&a, 0, sizeof(a));
    int sms = 0;
    { const int rc = device_sms(&sms); if (rc) return rc; }
    a.C = (__half*)C; a.bias = (const __half*)bias;
    a.M = (int)M; a.N = (int)N; a.K = (int)K;
    a.m_pad = (int)((M + 15) / 16 * 16);
    a.nblk = (int)(K / PK_KB); a.tiles = (int)(N / PK_ROWS);
    a.total = a.tiles * a.nblk;
    a.counters = (int*)workspace;
    a.ws = (float*)((uint8_t*)workspace + w4_counter_bytes(a.tiles));
    const uint32_t ES = PK_EXP_BYTES + (uint32_t)a.m_pad * 256u;
    const uint32_t budget = 227u * 1024u - 1024u - PK_CTRL_BYTES;
    a.ne = (int)(budget / ES);
    if (a.ne > PK_NE_MAX) a.ne = PK_NE_MAX;
    a.ne &= ~1;                                            // even: a slot always belongs to the same issuer
    if (a.ne < 2) return HBQ_ERR_UNSUPPORTED;
    a.nl = 0;
    a.acc_cols = a.m_pad <= 32 ? 32u : (a.m_pad <= 64 ? 64u : 128u);
    a.acc_bufs = 2u;
    a.tmem_cols = 4u * a.acc_cols;
    a.poll_limit = 1u << 23;
    CUtensorMap mx, mw;
    { const int rc = gemm_make_map(&mx, X, M, K, a.m_pad); if (rc) return rc; }
    { const int rc = gemm_make_map(&mw, W, N, K, PK_ROWS); if (rc) return rc; }
    const size_t smem = 1024 + (size_t)a.ne * ES + PK_CTRL_BYTES;
    const int grid = choose_split(a, sms, 0, 16, smem, (uint32_t)a.ne * ES);
    // equal runs: the tile counters must read zero; the workspace is the caller's scratch, so they are cleared here
    if (!a.split && !a.whole_tiles) HBQ_CUDA_TRY(cudaMemsetAsync(a.counters, 0, (size_t)a.tiles * 4, stream));
    return launch_packed<0, 16>(mx, mw, a, grid, smem, stream);
}

// workspace: gemm_w4_workspace_bytes() bytes, 16-byte aligned, zeroed once by the caller (the kernel leaves the tile
// counters at zero again); one call at a time per workspace.
// One launch.  The accumulators and the expanded stages share the SM's 512 tensor-memory columns: up to 64 tokens two
// accumulator pairs (segments alternate between them), beyond that one pair of 128 columns.
static int w4_launch_rows(const void* X, const void* Wp, void* C, int64_t M, int64_t N, int64_t K, PkArgs a, int ms,
                          int container_bits, const void* bias, void* workspace, int sms, cudaStream_t stream)
{
    a.wp = (const uint8_t*)Wp; a.C = (__half*)C; a.bias = (const __half*)bias;
    a.M = (int)M; a.N = (int)N; a.K = (int)K;
    a.m_pad = (int)((M + 15) / 16 * 16);
    a.nblk = (int)(K / PK_KB); a.tiles = (int)(N / PK_ROWS);
    a.total = a.tiles * a.nblk;
    a.counters = (int*)workspace;
    a.ws = (float*)((uint8_t*)workspace + w4_counter_bytes(a.tiles));
    const uint32_t LS = (uint32_t)pk_rec_bytes(container_bits), ES = (uint32_t)a.m_pad * 256u;
    // tensor memory: the accumulators, then the expanded stages (64 columns each): six of them, four beyond 32 tokens
    a.acc_cols = a.m_pad <= 32 ? 32u : (a.m_pad <= 64 ? 64u : 128u);
    a.acc_bufs = a.m_pad <= 64 ? 2u : 1u;
    a.tmem_cols = 512u;
    a.ne = (int)((a.tmem_cols - 2u * a.acc_bufs * a.acc_cols) / 64u);
    if (a.ne > PK_NE) a.ne = PK_NE;
    const uint32_t avail = 227u * 1024u - 1024u - (uint32_t)a.ne * ES - PK_CTRL_BYTES;
    a.nl = (int)(avail / LS);
    if (a.nl > PK_NL_MAX) a.nl = PK_NL_MAX;
    // An even count: the two expansion groups take alternate stages, so with an even ring a slot always serves the same
    // group, and a group only ever waits for the fill that follows one it has consumed itself.  (A parity wait cannot
    // tell "this fill has landed" from "the fill before it has not landed yet"; with an odd ring the fill before is the
    // other group's and nothing orders it before the wait.)
    a.nl &= ~1;
    if (a.nl < 2) return HBQ_ERR_UNSUPPORTED;
    CUtensorMap mx;
    { const int rc = gemm_make_map(&mx, X, M, K, a.m_pad); if (rc) return rc; }
    const size_t smem = 1024 + (size_t)a.ne * ES + (size_t)a.nl * LS + PK_CTRL_BYTES;
    const int grid = choose_split(a, sms, ms, container_bits, smem, (uint32_t)a.nl * LS);
    if (container_bits == 4) return ms == 0 ? launch_packed<0, 4>(mx, mx, a, grid, smem, stream) : launch_packed<2, 4>(mx, mx, a, grid, smem, stream);
    return ms == 0 ? launch_packed<0, 8>(mx, mx, a, grid, smem, stream) : launch_packed<2, 8>(mx, mx, a, grid, smem, stream);
}

// One token on the nibble container: the kernel without the tensor core.
static int w4_launch_gemv(const void* X, const void* Wp, void* C, int64_t M, int64_t N, int64_t K, const PkArgs& pa, int ms,
                          const void* bias, int sms, cudaStream_t stream)
{
    GvArgs a;
    memset(&a, 0, sizeof(a));
    a.wp = (const uint8_t*)Wp; a.x = (const __half*)X; a.C = (__half*)C; a.bias = (const __half*)bias;
    a.M = (int)M; a.N = (int)N; a.K = (int)K; a.nblk = (int)(K / PK_KB);
    for (int i = 0; i < 2; ++i) { a.base2[i] = pa.base2[i]; a.step2[i] = pa.step2[i]; }
    const int units = (int)(N / 32);                       // CTAs: 32 weight rows each
    // warps per CTA: enough of them over the GPU to cover the memory latency (about twelve per SM), at most one per block
    int ks = 4;
    while (ks < 16 && (int64_t)units * ks < (int64_t)sms * 12) ks *= 2;
    if (ks > a.nblk) ks = a.nblk;
    a.ks = ks;
    const size_t smem = (size_t)K * 2 + (size_t)ks * 32 * 4;
    auto go = [&](auto kern) -> int {
        { const int rc = ensure_dynamic_smem(kern, smem); if (rc) return rc; }
        kern<<<units, ks * 32, smem, stream>>>(a);
        HBQ_LAUNCH_CHECK("gemv_packed_kernel");
        return HBQ_OK;
    };
    return ms == 0 ? go(gemv_packed_kernel<0>) : go(gemv_packed_kernel<2>);
}

// Two to eight tokens on the nibble container: the warp-level MMA with the weights in registers.
static int w4_launch_reg(const void* X, const void* Wp, void* C, int64_t M, int64_t N, int64_t K, const PkArgs& pa, int ms,
                         const void* bias, int sms, cudaStream_t stream)
{
    RgArgs a;
    memset(&a, 0, sizeof(a));
    a.wp = (const uint8_t*)Wp; a.x = (const __half*)X; a.C = (__half*)C; a.bias = (const __half*)bias;
    a.M = (int)M; a.N = (int)N; a.K = (int)K; a.nblk = (int)(K / PK_KB);
    for (int i = 0; i < 2; ++i) { a.base2[i] = pa.base2[i]; a.step2[i] = pa.step2[i]; }
    // warps of a CTA: slabs of 32 rows x splits of K.  The most slabs that still give every SM a CTA (the slabs of a CTA
    // read the same lines of X), the rest of the warps split K: eight warps, sixteen where the CTAs do not fill the SMs.
    int slabs = 4;
    while (slabs > 1 && N / (32 * slabs) < sms) slabs >>= 1;
    int ks = (N / (32 * slabs) < sms ? 16 : 8) / slabs;
    if (ks > a.nblk) ks = a.nblk;
    a.slabs = slabs; a.ks = ks;
    const int grid = (int)(N / (32 * slabs));
    const size_t smem = (size_t)ks * slabs * 32 * 8 * 4;
    if (ms == 0) gemm_packed_reg_kernel<0><<<grid, ks * slabs * 32, smem, stream>>>(a);
    else gemm_packed_reg_kernel<2><<<grid, ks * slabs * 32, smem, stream>>>(a);
    HBQ_LAUNCH_CHECK("gemm_packed_reg_kernel");
    return HBQ_OK;
}

int gemm_w4_launch(const void* X, const void* Wp, void* C, int64_t M, int64_t N, int64_t K, const hbq_format* f,
                   int container_bits, const void* bias, void* workspace, cudaStream_t stream, uint32_t poll_limit)
{
    PkArgs a;
    memset(&a, 0, sizeof(a));
    int ms = 0;
    if (!X || !Wp || !C || !workspace) return HBQ_ERR_ARG;
    if (!w4_format(f, &a, &ms) || !w4_shape(M, N, K) || !w4_container(container_bits)) return HBQ_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(Wp) | reinterpret_cast<uintptr_t>(workspace)) & 15)
        return HBQ_ERR_ALIGN;
    if ((reinterpret_cast<uintptr_t>(C) | reinterpret_cast<uintptr_t>(bias)) & 1) return HBQ_ERR_ALIGN;
    int sms = 0;
    { const int rc = device_sms(&sms); if (rc) return rc; }
    a.poll_limit = poll_limit ? poll_limit : (1u << 23);
    // the nibble container has two more kernels for the smallest batches (measured on B200, 16 / 8 / 1 tokens x
    // [14336, 4096]: tcgen05 path 20.3 us, warp-level MMA 17.7 us, no tensor core 14.3 us)
    if (M == 1 && container_bits == 4 && K * 2 <= 96 * 1024)
        return w4_launch_gemv(X, Wp, C, M, N, K, a, ms, bias, sms, stream);
    if (M <= 8 && container_bits == 4)
        return w4_launch_reg(X, Wp, C, M, N, K, a, ms, bias, sms, stream);
    return w4_launch_rows(X, Wp, C, M, N, K, a, ms, container_bits, bias, workspace, sms, stream);
}

int gemm_w4_status(int* host_out)
{
    HBQ_CUDA_TRY(cudaMemcpyFromSymbol(host_out, g_tc_status, sizeof(int)));
    return HBQ_OK;
}
int gemm_w4_status_reset()
{
    const int z = 0;
    HBQ_CUDA_TRY(cudaMemcpyToSymbol(g_tc_status, &z, sizeof(int)));
    return HBQ_OK;
}

}  // namespace hbq
