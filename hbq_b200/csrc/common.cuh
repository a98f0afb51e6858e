// Shared helpers of the hbq_b200 CUDA library (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <atomic>
#include "../../include/hbq_b200.h"

namespace hbq {

// Bookkeeping shared by all translation units (defined in api.cu).
void note_launch(int n = 1);
int set_cuda_error(cudaError_t e, const char* where);

// Options of quantize_launch for the fused KV-cache writes.  K (and post-RoPE Q): rotary embedding on load
// and the (b,t,h) -> (b,h,t) row permutation on store; rows = B*T*H, K = D.  V (v_axis != 0): blocks run
// along the token axis of [B,T,H,D].
struct KvWriteOpts {
    const void* cos;
    const void* sin;
    int64_t rope_rows;        // rows of the cos/sin tables: B*T, or T when one table serves every batch
    int64_t B, T, H, D;
    int v_axis;
    const void* center;       // fp16 [B, H, D] subtracted after the rotation (K only), or NULL
    int v_out_token_major;    // V only: write [B,T,H,D] instead of [B,H,T,D]
    const void* glu_gate;     // not a cache write: quantise silu(glu_gate) * x (fp16, same shape as x); the
                              // other fields are then unused
};

#define HBQ_CUDA_TRY(expr)                                                     \
    do {                                                                       \
        cudaError_t _e = (expr);                                               \
        if (_e != cudaSuccess) return ::hbq::set_cuda_error(_e, #expr);        \
    } while (0)

#define HBQ_LAUNCH_CHECK(what)                                                 \
    do {                                                                       \
        cudaError_t _e = cudaGetLastError();                                   \
        if (_e != cudaSuccess) return ::hbq::set_cuda_error(_e, what);         \
        ::hbq::note_launch();                                                  \
    } while (0)

// Host-side per-device caches: the launch paths run tens of thousands of times per second for
// decode-sized tensors, so nothing that can be looked up once is asked of the runtime per call.
constexpr int kMaxDevices = 64;

// Current device and its SM count.
inline int device_sms(int* sms)
{
    static std::atomic<int> cached[kMaxDevices];
    int dev = 0;
    HBQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return HBQ_ERR_DEVICE;
    int v = cached[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        HBQ_CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
        cached[dev].store(v, std::memory_order_relaxed);
    }
    *sms = v;
    return HBQ_OK;
}

// Raise a kernel's dynamic shared-memory limit to `bytes` on the current device, once per kernel,
// device and size (api.cu keeps the table, keyed by the kernel's address).
int ensure_dynamic_smem_impl(const void* kernel, size_t bytes);
template <class Kernel>
inline int ensure_dynamic_smem(Kernel kernel, size_t bytes)
{
    return ensure_dynamic_smem_impl(reinterpret_cast<const void*>(kernel), bytes);
}

// CTAs of `threads` threads and `smem` dynamic bytes that one SM holds at once (the occupancy
// calculator's answer, cached per kernel address and device in api.cu).  A grid-stride kernel sized to
// more CTAs than are resident runs the excess as a thinly occupied second wave.
int resident_ctas_impl(const void* kernel, int threads, size_t smem, int* ctas);
template <class Kernel>
inline int resident_ctas(Kernel kernel, int threads, size_t smem, int* ctas)
{
    return resident_ctas_impl(reinterpret_cast<const void*>(kernel), threads, smem, ctas);
}

__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint16_t h_bits(__half h) { return __half_as_ushort(h); }
__device__ __forceinline__ __half bits_h(uint16_t u) { return __ushort_as_half(u); }

// Round an fp32 value to fp16 and back: the per-op rounding of a torch fp16 elementwise op.
__device__ __forceinline__ float rh(float f) { return __half2float(__float2half_rn(f)); }

}  // namespace hbq
