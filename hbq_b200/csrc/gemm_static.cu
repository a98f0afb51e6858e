// hbq_gemm_kn_noalloc: the [K,N]-operand GEMM for callers that must not allocate.
//
// hbq_gemm with B given as [K,N] needs device scratch for B transposed and leaves it to the
// caller to provide.  Some callers have no way to do that: code that runs after a serving
// process has frozen its memory pool, a plugin called from inside a framework whose allocator
// it may not touch, a real-time loop where cudaMalloc's implicit synchronisation is not
// acceptable.  For them this file keeps the scratch in a fixed array that is part of the
// library image: every GPU that loads the library holds HBQ_GEMM_NOALLOC_MAX_ELEMS fp16 values
// (8 MiB) until the process exits, and operands with N*K beyond that are refused.
#include "common.cuh"
#include <mutex>

namespace hbq {

int gemm_simt_launch(const void*, const void*, void*, int64_t, int64_t, int64_t, int, int, int, int,
                     const void*, cudaStream_t);
bool gemm_tc_eligible(int64_t, int64_t, int64_t, int, int, int);
int gemm_tc_launch(const void*, const void*, void*, int64_t, int64_t, int64_t, int, int, int, const void*,
                   cudaStream_t);
int transpose_launch(const void*, void*, int64_t, int64_t, cudaStream_t);

// B^T scratch.  In host code this name is only a handle for cudaGetSymbolAddress; the device
// address obtained from it is what the kernels receive.
static __device__ __align__(256) __half g_bt_scratch[HBQ_GEMM_NOALLOC_MAX_ELEMS];

static void* g_scratch_ptr[kMaxDevices];
static std::mutex g_scratch_mutex;

// Device address of the scratch array on the current device; looked up once per device.
static int scratch_address(void** out)
{
    int dev = 0;
    HBQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return HBQ_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[dev]) {
        void* p = nullptr;
        HBQ_CUDA_TRY(cudaGetSymbolAddress(&p, g_bt_scratch));
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return HBQ_OK;
}

}  // namespace hbq

using namespace hbq;

extern "C" int hbq_gemm_kn_noalloc(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                   int mode, int group_k, int group_n, const void* bias, void* stream)
{
    if (!A || !B || !C || M < 0 || N < 0 || K < 0) return HBQ_ERR_ARG;
    if (mode < HBQ_ACC_FP32 || mode > HBQ_ACC_PSUM_E3M4) return HBQ_ERR_ARG;
    if (mode >= HBQ_ACC_GROUPED && group_k <= 0) return HBQ_ERR_ARG;
    if (mode >= HBQ_ACC_PSUM_INT8 && (group_n <= 0 || 64 % group_n != 0)) return HBQ_ERR_ARG;
    // each factor first: N * K itself could wrap for absurd sizes
    if (N > (int64_t)HBQ_GEMM_NOALLOC_MAX_ELEMS || K > (int64_t)HBQ_GEMM_NOALLOC_MAX_ELEMS ||
        N * K > (int64_t)HBQ_GEMM_NOALLOC_MAX_ELEMS)
        return HBQ_ERR_TOO_LARGE;
    if (M == 0 || N == 0) return HBQ_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const bool aligned = (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C | (uintptr_t)bias) & 15) == 0;
    if (K > 0 && aligned && gemm_tc_eligible(M, N, K, mode, group_k, group_n)) {
        void* bt = nullptr;
        int rc = scratch_address(&bt);
        if (rc) return rc;
        // the transpose writes all N*K values the GEMM reads: nothing has to start at zero
        rc = transpose_launch(B, bt, K, N, st);
        if (rc) return rc;
        return gemm_tc_launch(A, bt, C, M, N, K, mode, group_k, group_n, bias, st);
    }
    return gemm_simt_launch(A, B, C, M, N, K, /*b_is_nk=*/0, mode, group_k, group_n, bias, st);
}
