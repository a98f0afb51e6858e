// CUDA-core GEMM with the reference's accumulation models, evaluated in the reference's own
// order: products a*b (exact in fp32) are added by sequential fp32 FMAs along k
// (blockquant_ext_src/gemm.cu:225-243, 354-377), so its results are bit-identical to the
// reference extension's.  It serves shapes the tensor-core kernel does not take (unaligned K,
// small group_k, the pure-fp16 chain) and is the on-device cross-check of that kernel.
#include "common.cuh"
#include <math.h>

namespace hbq {

constexpr int ST_M = 64, ST_N = 64, ST_K = 16;

// power-of-two scale of a partial-sum block: 2^(floor(log2 max) - shift)
// (compute_scale_pow2 / compute_scale_pow2_int8, gemm.cu:739-745, 1145-1152)
__device__ __forceinline__ float psum_scale(float max_abs, int shift)
{
    if (!(max_abs > 0.f)) return 1.f;
    return ldexpf(1.f, ilogbf(max_abs) - shift);
}

// INT8 partial-sum fake quantisation, gemm.cu:1236-1249
__device__ __forceinline__ float psum_int8(float g, float scale, float inv)
{
    float v = g * inv;
    if (!isfinite(v)) {
        if (isnan(v)) return NAN;
        v = copysignf(127.f, v);
    }
    float q = nearbyintf(v);
    q = fminf(fmaxf(q, -127.f), 127.f);
    return q * scale;
}

// E3M4 partial-sum fake quantisation (round to nearest even, subnormals down to 2^-6,
// maximum 15.5), gemm.cu:677-737.  Exact arithmetic: the reference build's fast-math
// approximations of the division and log2 are not reproduced.
__device__ float psum_e3m4(float x, float scale)
{
    const float sg = copysignf(1.f, x), a = fabsf(x);
    if (a == 0.f) return copysignf(0.f, x);
    const float y = __fdiv_rn(a, scale);
    if (!isfinite(y)) return isnan(y) ? copysignf(NAN, x) : sg * 15.5f * scale;
    if (y < 0.5f * 0.015625f) return 0.f;
    if (y >= 0.25f) {
        int e = ilogbf(y);
        e = max(-2, min(3, e));
        float p = ldexpf(1.f, e);
        float m = nearbyintf((__fdiv_rn(y, p) - 1.f) * 16.f);
        if (m >= 16.f) { m = 0.f; ++e; if (e > 3) { e = 3; m = 15.f; } p = ldexpf(1.f, e); }
        const float yq = fminf((1.f + m * 0.0625f) * p, 15.5f);
        return sg * yq * scale;
    }
    const float m = nearbyintf(y * 64.f);
    if (m <= 0.f) return 0.f;
    if (m >= 16.f) return sg * 0.25f * scale;
    return sg * (m * 0.0625f) * 0.25f * scale;
}

template <int MODE, bool B_NK>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const __half* __restrict__ A, const __half* __restrict__ B, __half* __restrict__ C,
                 int M, int N, int K, int group_k, int group_n, const __half* __restrict__ bias)
{
    __shared__ __half sA[ST_K][ST_M + 2];
    __shared__ __half sB[ST_K][ST_N + 2];
    __shared__ float sT[(MODE >= HBQ_ACC_PSUM_INT8) ? ST_M : 1][(MODE >= HBQ_ACC_PSUM_INT8) ? ST_N + 1 : 1];

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * ST_M, n0 = blockIdx.x * ST_N;

    float g[4][4];
    __half acc[4][4];
    #pragma unroll
    for (int i = 0; i < 4; ++i)
        #pragma unroll
        for (int j = 0; j < 4; ++j) { g[i][j] = 0.f; acc[i][j] = __float2half(0.f); }

    int cnt = 0;
    for (int k0 = 0; k0 < K; k0 += ST_K) {
        // stage A[m0.., k0..] as sA[k][m] and B as sB[k][n]; out-of-range elements are zero
        #pragma unroll
        for (int t = 0; t < (ST_M * ST_K) / 256; ++t) {
            const int idx = tid + t * 256;
            const int kk = idx % ST_K, mm = idx / ST_K;
            const int gm = m0 + mm, gk = k0 + kk;
            sA[kk][mm] = (gm < M && gk < K) ? A[(int64_t)gm * K + gk] : __float2half(0.f);
        }
        #pragma unroll
        for (int t = 0; t < (ST_N * ST_K) / 256; ++t) {
            const int idx = tid + t * 256;
            if (B_NK) {
                const int kk = idx % ST_K, nn = idx / ST_K;
                const int gn = n0 + nn, gk = k0 + kk;
                sB[kk][nn] = (gn < N && gk < K) ? B[(int64_t)gn * K + gk] : __float2half(0.f);
            } else {
                const int nn = idx % ST_N, kk = idx / ST_N;
                const int gn = n0 + nn, gk = k0 + kk;
                sB[kk][nn] = (gn < N && gk < K) ? B[(int64_t)gk * N + gn] : __float2half(0.f);
            }
        }
        __syncthreads();

        const int kend = min(ST_K, K - k0);
        for (int kk = 0; kk < kend; ++kk) {
            __half ah[4], bh[4];
            #pragma unroll
            for (int i = 0; i < 4; ++i) { ah[i] = sA[kk][ty * 4 + i]; bh[i] = sB[kk][tx * 4 + i]; }
            if constexpr (MODE == HBQ_ACC_FP16) {
                #pragma unroll
                for (int i = 0; i < 4; ++i)
                    #pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = __hfma(ah[i], bh[j], acc[i][j]);
            } else {
            float af[4], bf[4];
            #pragma unroll
            for (int i = 0; i < 4; ++i) { af[i] = __half2float(ah[i]); bf[i] = __half2float(bh[i]); }
            #pragma unroll
            for (int i = 0; i < 4; ++i)
                #pragma unroll
                for (int j = 0; j < 4; ++j) g[i][j] = __fmaf_rn(af[i], bf[j], g[i][j]);
            if (MODE == HBQ_ACC_FP32) continue;

            if (++cnt == group_k || k0 + kk + 1 == K) {
                cnt = 0;
                if (MODE >= HBQ_ACC_PSUM_INT8) {
                    #pragma unroll
                    for (int i = 0; i < 4; ++i)
                        #pragma unroll
                        for (int j = 0; j < 4; ++j) sT[ty * 4 + i][tx * 4 + j] = g[i][j];
                    __syncthreads();
                    const int tileN = min(ST_N, N - n0), tileM = min(ST_M, M - m0);
                    const int gpr = (tileN + group_n - 1) / group_n;
                    for (int q = tid; q < tileM * gpr; q += 256) {
                        const int r = q / gpr, c0 = (q % gpr) * group_n;
                        const int c1 = min(c0 + group_n, tileN);
                        float mx = 0.f;
                        for (int c = c0; c < c1; ++c) { const float av = fabsf(sT[r][c]); if (av > mx) mx = av; }
                        if (MODE == HBQ_ACC_PSUM_INT8) {
                            const float sc = psum_scale(mx, 6), inv = __fdiv_rn(1.f, sc);
                            for (int c = c0; c < c1; ++c) sT[r][c] = psum_int8(sT[r][c], sc, inv);
                        } else {
                            const float sc = psum_scale(mx, 3);
                            for (int c = c0; c < c1; ++c) sT[r][c] = psum_e3m4(sT[r][c], sc);
                        }
                    }
                    __syncthreads();
                    #pragma unroll
                    for (int i = 0; i < 4; ++i)
                        #pragma unroll
                        for (int j = 0; j < 4; ++j) g[i][j] = sT[ty * 4 + i][tx * 4 + j];
                    __syncthreads();
                }
                #pragma unroll
                for (int i = 0; i < 4; ++i)
                    #pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        acc[i][j] = __hadd(acc[i][j], __float2half_rn(g[i][j]));
                        g[i][j] = 0.f;
                    }
            }
            }  // MODE != FP16
        }
        __syncthreads();
    }

    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            __half v = (MODE == HBQ_ACC_FP32) ? __float2half_rn(g[i][j]) : acc[i][j];
            if (bias) v = __hadd(v, bias[gn]);
            C[(int64_t)gm * N + gn] = v;
        }
    }
}

template <int MODE>
static int launch_mode(const __half* A, const __half* B, __half* C, int M, int N, int K, int b_is_nk,
                       int group_k, int group_n, const __half* bias, cudaStream_t stream)
{
    const dim3 grid((N + ST_N - 1) / ST_N, (M + ST_M - 1) / ST_M), block(256);
    if (b_is_nk) gemm_simt_kernel<MODE, true><<<grid, block, 0, stream>>>(A, B, C, M, N, K, group_k, group_n, bias);
    else gemm_simt_kernel<MODE, false><<<grid, block, 0, stream>>>(A, B, C, M, N, K, group_k, group_n, bias);
    HBQ_LAUNCH_CHECK("gemm_simt_kernel");
    return HBQ_OK;
}

int gemm_simt_launch(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                     int b_is_nk, int mode, int group_k, int group_n, const void* bias,
                     cudaStream_t stream)
{
    if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF) return HBQ_ERR_UNSUPPORTED;
    if ((N + ST_N - 1) / ST_N > 0x7FFFFFFF || (M + ST_M - 1) / ST_M > 65535) return HBQ_ERR_UNSUPPORTED;
    const __half* a = (const __half*)A; const __half* b = (const __half*)B; __half* c = (__half*)C;
    const __half* bs = (const __half*)bias;
    switch (mode) {
        case HBQ_ACC_FP32: return launch_mode<HBQ_ACC_FP32>(a, b, c, (int)M, (int)N, (int)K, b_is_nk, 0, 0, bs, stream);
        case HBQ_ACC_FP16: return launch_mode<HBQ_ACC_FP16>(a, b, c, (int)M, (int)N, (int)K, b_is_nk, 0, 0, bs, stream);
        case HBQ_ACC_GROUPED: return launch_mode<HBQ_ACC_GROUPED>(a, b, c, (int)M, (int)N, (int)K, b_is_nk, group_k, 0, bs, stream);
        case HBQ_ACC_PSUM_INT8: return launch_mode<HBQ_ACC_PSUM_INT8>(a, b, c, (int)M, (int)N, (int)K, b_is_nk, group_k, group_n, bs, stream);
        case HBQ_ACC_PSUM_E3M4: return launch_mode<HBQ_ACC_PSUM_E3M4>(a, b, c, (int)M, (int)N, (int)K, b_is_nk, group_k, group_n, bs, stream);
    }
    return HBQ_ERR_ARG;
}

}  // namespace hbq
