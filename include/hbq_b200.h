/*
 * hbq_b200 -- C ABI of the B200 (sm_100a) implementation of HBQ's hot path:
 * block quantize-dequantize (MXFP / NVFP / MXINT / HBQ two-level) and the GEMM
 * with modelled low-precision accumulation.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the name ends in _host;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - the calls enqueue work and return; they never synchronise the device;
 *   - return value 0 = success, negative = error (see hbq_error_string);
 *   - no global state besides one device status word (hbq_gemm_status); calls are
 *     re-entrant per stream.
 *
 * Each entry point names the reference interface it replaces (paths inside the
 * HBQ repository).
 */
#ifndef HBQ_B200_H
#define HBQ_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- formats --------------------------------------------------------------------------- */

enum { HBQ_KIND_MXFP = 0, HBQ_KIND_MXINT = 1, HBQ_KIND_HBQ = 2,
       HBQ_KIND_MXEX = 3,   /* MXExQuantizer (src/quantizer.py:541-628): mbit = element bits, sc_ebit = sc_bit,
                               l2_sc_bit, l2_block_size (<= 8); fake-quantised output only */
       HBQ_KIND_VSQ = 4 };  /* VSQQuantizer (src/quantizer.py:630-702): mbit = nbit, sc_mbit; fake-quantised output only */
/* Index into HBQQuantizer.L2_SCHEME, src/quantizer.py:708 */
enum { HBQ_L2_POT = 0, HBQ_L2_INT = 1, HBQ_L2_SIG1 = 2, HBQ_L2_FPM1 = 3,
       HBQ_L2_FP1 = 4, HBQ_L2_FPM10 = 5, HBQ_L2_FPM100 = 6, HBQ_L2_MIX = 7 };
enum { HBQ_DTYPE_F16 = 0, HBQ_DTYPE_BF16 = 1 };

/* Constructor arguments of MXFPQuantizer / MXINTQuantizer / HBQQuantizer
 * (src/quantizer.py:348-357, 431-443, 709-725), same meaning. */
typedef struct hbq_format {
    int32_t kind;                  /* HBQ_KIND_* */
    int32_t ebit, mbit;            /* element format; MXINT: ebit = 0, mbit = nbit */
    int32_t sc_ebit, sc_mbit;      /* shared scale; sc_mbit == 0 => power of two */
    int32_t block_size;            /* 16..256, multiple of 8 */
    int32_t scale_allow_subnormal;
    int32_t use_round;             /* MXFP power-of-two scale: round(log2 max) instead of floor */
    int32_t use_ceil;              /* FP scale: ceil its mantissa */
    int32_t l2_block_size;         /* HBQ micro-block (4, 8, 16, ... block_size) */
    int32_t l2_sc_bit;             /* HBQ: log2(number of micro-scale candidates), 0..4 */
    int32_t l2_scheme;             /* HBQ_L2_* */
    int32_t per_tensor_scale;      /* MXFP only (src/quantizer.py:516-524) */
    int32_t reserved;
} hbq_format;

/* Optional outputs of hbq_quantize; any pointer may be NULL.
 *   Kp = ceil(K / block_size) * block_size, nblk = Kp / block_size, nl2 = block_size / l2_block_size.
 *   codes     element codes, row-major [rows, Kp]:
 *               4-bit elements (E2M1, INT4): two per byte, element 2i in the low nibble;
 *               5-bit elements (E2M2): low 4 bits {exp, mant} packed as above, sign bits in `sign`;
 *               6..8-bit elements: one byte each ({sign, exp, mant} or two's complement).
 *             FP code fields are those of make_fp_quant's detailed output
 *             (src/quantizer.py:249-253): exponent biased by 2^(ebit-1)-1, 0 = subnormal.
 *   sign      [rows, Kp/8] sign bit-plane for 5-bit elements, element i in bit (i % 8).
 *   scale_u8  [rows, nblk] shared scale byte: bits 14..7 of its fp16 pattern, i.e. {exp5, mant3}
 *             with bias 15 (E5M3) or the biased power-of-two exponent << 3.
 *   scale_h   [rows, nblk] shared scale as fp16 (HBQQuantizer.shared_scale).
 *   l2_packed [rows, nblk, nl2*l2_sc_bit/8] micro-scale indices, l2_sc_bit bits each, little
 *             endian; needs nl2*l2_sc_bit to be 8, 16 or 32.
 *   l2_idx    [rows, nblk, nl2] the same indices one per byte (HBQQuantizer.l2_scale).
 *   scheme    [rows, nblk] chosen table of the "Mix" scheme (HBQQuantizer.blk_l2_scheme). */
typedef struct hbq_packed_out {
    uint8_t* codes;
    uint8_t* sign;
    uint8_t* scale_u8;
    uint16_t* scale_h;
    uint8_t* l2_packed;
    uint8_t* l2_idx;
    uint8_t* scheme;
} hbq_packed_out;

/* ---- quantize -------------------------------------------------------------------------- */

/* Replaces _QBase.forward / MXFPQuantizer.q / MXINTQuantizer.q / HBQQuantizer.q
 * (src/quantizer.py:343-345, 415-428, 513-539, 741-859) on a [rows, K] tensor quantised
 * along K.  x has `dtype`, deq `deq_dtype`; bf16 input is converted to fp16 first, the
 * arithmetic is the reference's fp16 arithmetic, and a bf16 deq is the fp16 result rounded to
 * bf16.  deq (the fake-quantised tensor, same shape as x) and `out` may each be NULL.  `tensor_amax` is only read when fmt->per_tensor_scale is set: a device
 * float holding max|x| of the whole tensor (see hbq_absmax). */
int hbq_quantize(const void* x, int dtype, int64_t rows, int64_t K, const hbq_format* fmt,
                 void* deq, int deq_dtype, const hbq_packed_out* out, const float* tensor_amax,
                 void* stream);

/* max|x| over n elements into *amax (device float, overwritten).  Replaces the
 * `xg.abs().max().item()` of the per-tensor scale, src/quantizer.py:519.  `scratch` must
 * hold at least hbq_absmax_scratch_bytes() bytes of device memory. */
int hbq_absmax(const void* x, int dtype, int64_t n, float* amax, void* scratch, void* stream);
int64_t hbq_absmax_scratch_bytes(void);

/* Rebuilds the fake-quantised fp16 tensor [rows, K] from the packed outputs of
 * hbq_quantize (codes, sign, scale_u8, l2_packed, scheme as the format needs them).
 * No reference counterpart: the reference never stores codes (it keeps the fp16
 * fake-quantised weight, src/ptq.py:349). */
int hbq_dequantize(const hbq_packed_out* in, int64_t rows, int64_t K, const hbq_format* fmt,
                   void* deq, int dtype, void* stream);

/* Element quantizer alone over n values (fp16 in, fp16 out): make_fp_quant
 * (src/quantizer.py:187-257) when elem_variant = 1, the free function fp_quant
 * (src/quantizer.py:259-328) when 0. */
int hbq_fp_quant(const void* x, int64_t n, int ebit, int mbit, int allow_subnormal,
                 int use_ceil, int elem_variant, void* out, void* stream);

/* ---- fused KV-cache writes --------------------------------------------------------------- */

/* K-cache (or post-RoPE query) write of QLlamaAttention.forward (src/module.py:147-162) in one
 * pass: k is the k_proj output viewed [B,T,H,D]; the kernel applies the rotary embedding
 * x*cos + rotate_half(x)*sin in fp16 (each product and the sum rounded, as the fp16 tensor ops of
 * apply_rotary_pos_emb round them), quantises along D with `fmt` (D a power of two in [16, 256] and a multiple of block_size) and
 * stores the fake-quantised values in the cache layout [B,H,T,D] -- what the reference does as
 * view + transpose + apply_rotary_pos_emb + kv_quantizer.q.  cos/sin are fp16 [rope_rows, D]
 * tables with rope_rows = B*T, or T when one table serves every batch; both NULL skips the
 * rotation (then k may be bf16).  `center` (fp16 [B,H,D] or NULL) is subtracted after the rotation:
 * the K-cache centring of the Qwen2 attention block (src/module.py:221-244).  Returns HBQ_ERR_UNSUPPORTED for formats outside the fused
 * kernels (callers then run the three steps separately). */
int hbq_kv_write_k(const void* k, int dtype, int64_t B, int64_t T, int64_t H, int64_t D,
                   const void* cos, const void* sin, int64_t rope_rows, const void* center,
                   const hbq_format* fmt, void* out, int out_dtype, void* stream);

/* V-cache write (src/module.py:163-168): v is the v_proj output viewed [B,T,H,D]; blocks of
 * fmt->block_size consecutive TOKENS per (batch, head, channel) are quantised (the tail block
 * zero padded) and the result is stored as [B,H,T,D] -- the reference's transpose, quantise,
 * transpose back.  With out_token_major != 0 the result keeps the input's [B,T,H,D] layout (serving
 * engines with flattened-token caches, vllm/src/hbq_vllm_quant.py:322-345).  Served formats: HBQ with one candidate table, MXFP / NVFP E2Mx and MXINT with a
 * scale inside fp16's range; D a multiple of 64, block_size 16..128.  HBQ_ERR_UNSUPPORTED otherwise. */
int hbq_kv_write_v(const void* v, int dtype, int64_t B, int64_t T, int64_t H, int64_t D,
                   const hbq_format* fmt, void* out, int out_dtype, int out_token_major, void* stream);

/* Gated-MLP activation fused into the quantizer of the down projection's input: what the reference
 * runs as three tensor ops, act_fn(gate_proj(x)) * up_proj(x) (the MLP forward of the patched
 * transformers blocks) followed by down_proj.aq.q(...) (src/module.py:45), in one pass over the two
 * projection outputs.  gate, up and out are fp16 [rows, K], contiguous and 16-byte aligned; act_fn is
 * SiLU.  Roundings are those of the separate ops: silu evaluated in fp32 and rounded to fp16, the
 * product rounded to fp16, then the HBQ quantizer.  Served formats: HBQ with one candidate table,
 * K a multiple of block_size; HBQ_ERR_UNSUPPORTED otherwise (callers then run the steps separately). */
int hbq_swiglu_quantize(const void* gate, const void* up, int64_t rows, int64_t K,
                        const hbq_format* fmt, void* out, void* stream);

/* Normalisation fused into the quantizer of the q/k/v and gate/up projections' input: what the patched decoder
 * layer runs as hidden = hidden + residual_branch, LlamaRMSNorm(hidden) (transformers; weight * fp16(x_f32 *
 * rsqrt(mean(x_f32^2) + eps))) and then _QBaseLinear.forward's self.aq(x) (src/module.py:45), in one kernel: a
 * warp owns a row, sweeps it once for the sum of squares (writing x + residual to x_out when `residual` is
 * given; x_out may be x itself) and once more to normalise and hand each 128-element block to the table
 * quantizer -- the normalised tensor never goes to memory unquantised.  x, residual, x_out, out: fp16 [rows, K],
 * weight fp16 [K], all 16-byte aligned, K a multiple of 8.  fmt = NULL writes the normalised tensor itself (the
 * model's final norm).  Served formats: HBQ with one candidate table, E2M1 / E2M2, block 128, micro-block 8 or
 * 32, K a multiple of 128; HBQ_ERR_UNSUPPORTED otherwise (callers then pass NULL and run hbq_quantize). */
int hbq_rmsnorm_quantize(const void* x, const void* residual, const void* weight, float eps, int64_t rows,
                         int64_t K, const hbq_format* fmt, void* x_out, void* out, void* stream);

/* Attention probabilities with their quantizer: manual_sdpa's attn_weight = softmax(q k^T * scale + bias) and
 * attn_wgt_quantizer.q(attn_weight) (src/module.py:108-115) from the raw scores q k^T (fp16 [rows, S], rows =
 * batch * heads * L query rows) in one kernel.  Rounding points are the reference's: fp16(score * scale) with the product taken in fp32 (a tensor times a Python float),
 * fp16(+ bias), softmax evaluated in fp32 (maximum, exp(x - max), sum, division) and rounded to fp16, then the
 * quantizer along the key axis.  causal != 0 masks key j of query row r when j > (r % L) + (S - L) (is_causal of
 * manual_sdpa; with a key/value cache the new queries are the last L positions); `mask` is an optional additive
 * fp16 mask [mask_batches, L, S] (mask_batches = 1 or batch; `heads` = query rows per batch / L).  Runs of 1024
 * keys that are masked for a row are written as zeros without being evaluated.  out may be scores itself.
 * fmt = NULL writes the probabilities unquantised.  Served formats as hbq_rmsnorm_quantize, S a multiple of 128. */
int hbq_softmax_quantize(const void* scores, int64_t rows, int64_t S, int64_t L, int64_t heads, float scale,
                         int causal, const void* mask, int64_t mask_batches, const hbq_format* fmt, void* out,
                         void* stream);


/* ---- GEMM with modelled accumulation --------------------------------------------------- */

enum { HBQ_ACC_FP32 = 0,       /* gemm_fp32_accum         blockquant_ext.cpp:21-29, gemm.cu:96-303 */
       HBQ_ACC_FP16 = 1,       /* gemm_fp16_accum         blockquant_ext.cpp:31-39, gemm.cu:96-303 */
       HBQ_ACC_GROUPED = 2,    /* gemm_fp16_grouped_accum blockquant_ext.cpp:41-49, gemm.cu:306-553 */
       HBQ_ACC_PSUM_INT8 = 3,  /* gemm_blockquant_mxint8  blockquant_ext.cpp:64-71, gemm.cu:1154-1396 */
       HBQ_ACC_PSUM_E3M4 = 4   /* gemm_blockquant_mxfp8   blockquant_ext.cpp:55-62, gemm.cu:752-1035 */ };

/* C[M,N] = A[M,K] * B, fp16 in, fp16 out, row-major, with the accumulation model `mode`.
 *   b_is_nk = 0: B is [K,N] (the layout the reference extension receives, ops.py:41);
 *   b_is_nk = 1: B is W [N,K] as nn.Linear stores it -- no transpose is needed and this is
 *                the fast path (FP16AccumMatMul.forward, src/ops.py:28-62).
 *   group_k: K-chunk of the fp32 partial sum (modes 2-4); group_n: columns per partial-sum
 *   quantisation block (modes 3-4).  `bias` [N] fp16 or NULL is added in fp16 after the
 *   accumulation (src/ops.py:59-60).
 *   `workspace` / `workspace_bytes`: device scratch, at least hbq_gemm_workspace_bytes(...)
 *   (holds B transposed when b_is_nk = 0 and the tensor-core path is taken; may be NULL if 0). */
int hbq_gemm(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
             int b_is_nk, int mode, int group_k, int group_n, const void* bias,
             void* workspace, int64_t workspace_bytes, void* stream);
int64_t hbq_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int b_is_nk, int mode,
                                 int group_k, int group_n);
/* 1 if hbq_gemm would run the tcgen05 kernel for these arguments, 0 if the SIMT kernel. */
int hbq_gemm_uses_tensor_cores(int64_t M, int64_t N, int64_t K, int b_is_nk, int mode,
                               int group_k, int group_n);
/* Force the SIMT kernel (exact sequential-fp32 model of gemm.cu) regardless of shape. */
int hbq_gemm_simt(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                  int b_is_nk, int mode, int group_k, int group_n, const void* bias,
                  void* stream);

/* Same computation as hbq_gemm with b_is_nk = 0 (B is [K,N]), for callers that cannot hand over
 * device scratch because they cannot allocate any: a plugin running inside a host framework
 * whose memory pool it must not touch, a server that freezes its allocations after start-up,
 * a latency-critical loop that cannot afford cudaMalloc's implicit synchronisation.  The
 * transposed copy of B lives in an array inside the library image instead, so
 *   - every GPU that loads the library holds HBQ_GEMM_NOALLOC_MAX_ELEMS * 2 bytes (8 MiB) for
 *     the life of the process, and N*K above that limit returns HBQ_ERR_TOO_LARGE;
 *   - the call itself performs no cudaMalloc / cudaFree and calls no allocating library routine;
 *   - the first call on each device looks the array's device address up (with that device
 *     current); make that first call before starting any stream capture;
 *   - all calls share the one array, which keeps the previous call's contents: each call
 *     rewrites the N*K values it reads, nothing needs to start at zero, but two calls that
 *     overlap on the GPU (different streams) race on it -- keep them on one stream.
 * This entry point has no counterpart in the reference, whose caller allocates the transposed
 * weight with torch on every call (src/ops.py:41). */
#define HBQ_GEMM_NOALLOC_MAX_ELEMS (4 * 1024 * 1024)
int hbq_gemm_kn_noalloc(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                        int mode, int group_k, int group_n, const void* bias, void* stream);

/* The tensor-core kernel bounds every wait on an mbarrier.  If one expires the kernel stops,
 * frees its tensor memory and records which wait gave up in a device status word; the output
 * of that call is then undefined.  hbq_gemm_status copies the word to the host (it
 * synchronises the device); 0 = no wait has expired since the last reset.
 * No reference counterpart (the reference kernels do not wait on anything). */
int hbq_gemm_status(int* status_host);
int hbq_gemm_status_reset(void);
/* Self-test of that give-up path, for a test suite: launches the tensor-core kernel on the given
 * problem (A [M,K], W [N,K], C [M,N] as for hbq_gemm with b_is_nk = 1; the shape must be one
 * hbq_gemm_uses_tensor_cores accepts) with its loader switched off and the wait bound lowered to
 * `poll_limit` polls (1 .. 2^23).  Nothing is ever in flight, so every wait inside the kernel runs
 * out, every role leaves its loop, tensor memory is freed and the kernel returns normally; afterwards
 * hbq_gemm_status reports a non-zero code (2 = operand wait, 4 = accumulator wait) until
 * hbq_gemm_status_reset.  C is left undefined.  No reference counterpart. */
int hbq_gemm_wait_selftest(const void* A, const void* W, void* C, int64_t M, int64_t N, int64_t K,
                           int mode, int group_k, int group_n, uint32_t poll_limit, void* stream);

/* ---- GEMM on the packed weight (decode shapes) ---------------------------------------------- */

/* C[M,N] = X[M,K] * deq(W)[N,K]^T for M <= 128 tokens, reading W as packed 4-bit codes, block scales and
 * micro-scale indices (0.5625 B per weight) and expanding it to the fp16 fake-quantised values on chip (tensor memory)
 * in front of the tensor core; fp32 accumulation, fp16 output, bias as in hbq_gemm.  Replaces, for a statically
 * quantised HBQ weight (src/ptq.py:349, the fp16 tensor the reference keeps) under fp32 accumulation, the
 * F.linear of _QBaseLinear.forward (src/module.py:64) at decode-sized batches, where the time is the streaming
 * of W: the products are those of the fp16 tensor (each expanded value equals hbq_dequantize's bit for bit).
 *
 * By token count the nibble container runs one of three kernels over the same prepacked weight: one token without the
 * tensor core, two to eight tokens on the warp-level MMA with the expanded weights in registers, more on tcgen05 with
 * the expanded weights in tensor memory.  All add in a fixed order (results do not vary from call to call).
 *
 * Served: HBQ weights with E2M1 elements, block 128 with an E5M3 scale, 2-bit micro-scales per 8 or 32 with the
 * FPM1 / FP1 / FPM10 / FPM100 / Mix tables (every shipped HBQ weight format); N and K multiples of 128;
 * 1 <= M <= 128.  HBQ_ERR_UNSUPPORTED otherwise (callers then use hbq_gemm on the fp16 tensor).
 *
 * hbq_gemm_w4_prepack turns the planes of hbq_quantize (codes, scale_u8, l2_packed, scheme; W is [N, K]) into the
 * kernel's operand, hbq_gemm_w4_prepacked_bytes(N, K, container_bits) bytes, 16-byte aligned: one record per (128 rows,
 * 128 k) -- four 32-element pieces of every row's codes with the rows contiguous, then per row the 32 bits of
 * micro-scale indices, the block scale as fp16 and the table bit.  Done once per weight.
 *
 * container_bits: 4 -- codes as stored, {sign, e1, e0, m} per nibble, records of 9216 bytes (0.5625 B per weight);
 * 8 -- each code as the top byte of its value's fp16 pattern (the low byte is zero for E2M1), records of 17408 bytes
 * (1.0625 B per weight).  Same values either way; the 4-bit form goes through the hardware's E2M1 conversion, the
 * 8-bit form through a byte permute, and on B200 the 4-bit form is the faster one (fewer bytes, as few
 * instructions).  prepack and gemm must be given the same value.
 *
 * workspace: hbq_gemm_w4_workspace_bytes(M, N, K) bytes (-1: shape not served), 16-byte aligned, ZEROED ONCE by
 * the caller before its first use; the kernel leaves it usable for the next call on the same stream, of any M up
 * to the M it was sized for.  Where there are enough tiles every SM takes whole tiles and the workspace is not
 * touched.  Otherwise the work is cut into equal runs of (128 rows, 128 k) records, one run per SM, whatever tile
 * boundaries fall inside a run; the parts of a tile that different SMs computed meet here as fp32 partial sums
 * (two slots per SM) and are added in a fixed order, so results do not vary from run to run; one counter per tile
 * (at the start of the workspace) tells which SM finishes it.  After a
 * call that hbq_gemm_status reports as failed, zero it again. */
int64_t hbq_gemm_w4_prepacked_bytes(int64_t N, int64_t K, int container_bits);
int hbq_gemm_w4_prepack(const hbq_packed_out* in, int64_t N, int64_t K, const hbq_format* fmt, int container_bits,
                        void* out, void* stream);
int64_t hbq_gemm_w4_workspace_bytes(int64_t M, int64_t N, int64_t K);
int hbq_gemm_w4(const void* X, const void* Wp, void* C, int64_t M, int64_t N, int64_t K,
                const hbq_format* fmt, int container_bits, const void* bias, void* workspace,
                int64_t workspace_bytes, void* stream);

/* The tensor-core kernel is persistent: one CTA per SM, each holding most of an SM's shared
 * memory, with a fixed round-robin share of the tiles.  A kernel of another stream that already
 * sits on some SMs (a collective running under the GEMM) keeps those CTAs from starting until it
 * ends, and they still owe their whole share.  hbq_gemm_reserve_sms(n) makes every later launch
 * of this process leave n SMs free for such a neighbour (0 = use all, the default); it returns
 * the previous value.  Host-side setting read at launch time; no reference counterpart. */
int hbq_gemm_reserve_sms(int n);

/* ---- misc ------------------------------------------------------------------------------ */

const char* hbq_error_string(int code);
/* Text of the last failing CUDA runtime/driver call on this thread ("" if none). */
const char* hbq_last_cuda_error(void);
int hbq_version(void);
/* Kernels launched by this library since load (all threads); the benchmark reports it. */
int64_t hbq_launch_count(void);

enum { HBQ_OK = 0, HBQ_ERR_ARG = -1, HBQ_ERR_UNSUPPORTED = -2, HBQ_ERR_CUDA = -3,
       HBQ_ERR_ALIGN = -4, HBQ_ERR_WORKSPACE = -5, HBQ_ERR_DEVICE = -6,
       HBQ_ERR_TOO_LARGE = -7 };

#ifdef __cplusplus
}
#endif
#endif
