// V-cache write: quantisation along the token axis, shared by the table-driven HBQ kernel and the
// MX / NV kernel.
//
// QLlamaAttention.forward quantises V in blocks of kv_block_size consecutive TOKENS per (batch, head,
// channel) by transposing, quantising and transposing back (src/module.py:163-168).  Here a CTA of 512
// threads takes a tile of 128 tokens x 64 channels of the projection output [B, T, H, D], turns it
// through shared memory so that a thread owns 8 consecutive tokens of one channel (the chunk shape of
// the quantize arithmetic), quantises in place and writes the tile to the cache layout [B, H, T, D].
// Tokens beyond T are the reference's zero padding.
#pragma once
#include "quantize_dev.cuh"

namespace hbq {

struct VArgs {
    const uint16_t* in;
    uint16_t* out;
    int64_t B, T, H, D;
    int in_bf16, out_bf16;
    int out_token_major;      // 0: out is [B,H,T,D] (the cache layout); 1: out keeps the input's [B,T,H,D]
    int64_t tiles;            // B * H * ceil(T/128) * (D/64)
    int tblocks, dslabs;
};
constexpr int VT = 128, VD = 64, V_THREADS = 512;
constexpr int V_TILE_BYTES = (VD / 2) * VT * 4;

// Shared tile of 32-bit words: row = channel pair (d, d+1), column = token, value = the two channels'
// fp16 values of that token.  The 8-token granules of a row are XOR-swizzled with the row's segment
// so that the token-major writes of the load phase spread over the banks, while a thread's 8
// consecutive tokens stay one aligned 32-byte run for the channel-major compute phase.
__device__ __forceinline__ int v_word(int dp, int tk) { return dp * VT + ((((tk >> 3) ^ ((dp >> 2) & 3)) << 3) | (tk & 7)); }

// Persistent loop over this CTA's tiles.  chunk(xb, dq): xb = 8 consecutive tokens of one channel as
// four fp16 pairs, dq = their fake-quantised values; the lanes of a quantisation block (block_size / 8
// consecutive lanes, at most 16) call it together.
template <class ChunkFn>
__device__ __forceinline__ void v_cache_tiles(const VArgs& v, uint32_t* tile, const ChunkFn& chunk)
{
    const int tid = threadIdx.x;
    for (int64_t tl = blockIdx.x; tl < v.tiles; tl += gridDim.x) {
        const int ds = (int)(tl % v.dslabs);
        const int tb = (int)((tl / v.dslabs) % v.tblocks);
        const int64_t bh = tl / ((int64_t)v.dslabs * v.tblocks);
        const int64_t b = bh / v.H, h = bh - b * v.H;
        const int64_t t0 = (int64_t)tb * VT, d0 = (int64_t)ds * VD;

        // -- load [128 tokens][64 channels]: a thread brings 8 channels of one token = 4 words --
        #pragma unroll
        for (int r = 0; r < (VT * VD / 8) / V_THREADS; ++r) {
            const int idx = tid + r * V_THREADS;
            const int tk = idx >> 3, seg = idx & 7;               // token in tile, 8-channel segment
            uint32_t w[4] = {0u, 0u, 0u, 0u};
            if (t0 + tk < v.T) {
                const uint4 g = __ldg(reinterpret_cast<const uint4*>(v.in + (((b * v.T + t0 + tk) * v.H + h) * v.D + d0 + seg * 8)));
                w[0] = g.x; w[1] = g.y; w[2] = g.z; w[3] = g.w;
            }
            #pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (v.in_bf16)
                    w[i] = h2_bits(__floats2half2_rn(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xFFFF0000u)));
                tile[v_word(seg * 4 + i, tk)] = w[i];
            }
        }
        __syncthreads();

        // -- quantise in place: a thread owns 8 consecutive tokens of one channel; lanes 0-15 of a warp
        //    hold an even channel, lanes 16-31 the odd channel of the same words --
        #pragma unroll
        for (int pass = 0; pass < VD / (V_THREADS / 16); ++pass) {
            const int d = pass * (V_THREADS / 16) + (tid >> 4);
            const int lig16 = tid & 15;
            uint32_t* cell = tile + v_word(d >> 1, lig16 * 8);
            const uint4 c0 = *reinterpret_cast<const uint4*>(cell), c1 = *reinterpret_cast<const uint4*>(cell + 4);
            const uint32_t wt[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};      // tokens 0..7, both channels
            const uint32_t pick = (d & 1) ? 0x7632u : 0x5410u;
            uint32_t xb[4], dq[4];
            #pragma unroll
            for (int p = 0; p < 4; ++p) xb[p] = __byte_perm(wt[2 * p], wt[2 * p + 1], pick);   // this channel, tokens 2p, 2p+1
            chunk(xb, dq);
            // rebuild the words with the partner channel's results: the even lane writes tokens 0-3, the odd lane 4-7
            uint32_t ow[4];
            #pragma unroll
            for (int p = 0; p < 2; ++p) {
                const int mine = (d & 1) ? 2 + p : p, theirs = (d & 1) ? p : 2 + p;      // pair index this lane keeps / gives away
                const uint32_t got = __shfl_xor_sync(0xFFFFFFFFu, dq[theirs], 16);      // partner's values for the pair I keep
                const uint32_t ev = (d & 1) ? got : dq[mine], od = (d & 1) ? dq[mine] : got;
                ow[2 * p] = __byte_perm(ev, od, 0x5410u);
                ow[2 * p + 1] = __byte_perm(ev, od, 0x7632u);
            }
            __syncwarp();
            *reinterpret_cast<uint4*>(cell + ((d & 1) ? 4 : 0)) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
        __syncthreads();

        // -- write out[b][h][t][d0 .. d0+64) --
        #pragma unroll
        for (int r = 0; r < (VT * VD / 8) / V_THREADS; ++r) {
            const int idx = tid + r * V_THREADS;
            const int tk = idx >> 3, seg = idx & 7;
            if (t0 + tk < v.T) {
                uint32_t w[4];
                #pragma unroll
                for (int i = 0; i < 4; ++i) {
                    w[i] = tile[v_word(seg * 4 + i, tk)];
                    if (v.out_bf16) {
                        const float2 f = __half22float2(bits_h2(w[i]));
                        __nv_bfloat162 bb = __floats2bfloat162_rn(f.x, f.y);
                        w[i] = *reinterpret_cast<uint32_t*>(&bb);
                    }
                }
                const int64_t orow = v.out_token_major ? (b * v.T + t0 + tk) * v.H + h : (b * v.H + h) * v.T + t0 + tk;
                *reinterpret_cast<uint4*>(v.out + (orow * v.D + d0 + seg * 8)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        __syncthreads();
    }
}

// Tile count and geometry of a [B,T,H,D] V write; false when the shape does not fit the tile kernel.
inline bool v_args_fill(VArgs* v, const void* in, void* out, int in_bf16, int out_bf16, int64_t B, int64_t T, int64_t H,
                        int64_t D, int block_size, int out_token_major)
{
    v->out_token_major = out_token_major;
    if (block_size > VT || block_size < 8 || (VT % block_size) != 0 || (D % VD) != 0) return false;
    v->in = (const uint16_t*)in; v->out = (uint16_t*)out;
    v->B = B; v->T = T; v->H = H; v->D = D; v->in_bf16 = in_bf16; v->out_bf16 = out_bf16;
    v->tblocks = (int)((T + VT - 1) / VT); v->dslabs = (int)(D / VD);
    v->tiles = B * H * v->tblocks * v->dslabs;
    return true;
}

}  // namespace hbq
