/*
 * CPU oracle for the HBQ hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the reference's block quantizers (src/quantizer.py)
 * and of the accumulation models of its GEMM extension
 * (blockquant_ext_src/gemm.cu).  Only the test-suite, the smoke check and the
 * CPU-baseline leg of the benchmark may link or load it; the CUDA library never
 * does.  Parity of this file is pinned by tests/golden/ (vectors produced by
 * importing the reference's own Python quantizers) and, for the GEMM models, by
 * the reference gemm.cu compiled into oracle/_ref/ and run on the GPU.
 *
 * All tensors are fp16 bit patterns (uint16_t), row-major.
 */
#ifndef HBQ_ORACLE_H
#define HBQ_ORACLE_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORC_KIND_MXFP = 0, ORC_KIND_MXINT = 1, ORC_KIND_HBQ = 2,
       ORC_KIND_MXEX = 3,   /* MXExQuantizer: mbit = element bits, sc_ebit = sc_bit, l2_sc_bit, l2_block_size */
       ORC_KIND_VSQ = 4 };  /* VSQQuantizer: mbit = nbit, sc_mbit */
/* Index into HBQQuantizer.L2_SCHEME (quantizer.py:708). */
enum { ORC_L2_POT = 0, ORC_L2_INT = 1, ORC_L2_SIG1 = 2, ORC_L2_FPM1 = 3,
       ORC_L2_FP1 = 4, ORC_L2_FPM10 = 5, ORC_L2_FPM100 = 6, ORC_L2_MIX = 7 };

typedef struct {
    int32_t kind;                  /* ORC_KIND_* */
    int32_t ebit, mbit;            /* element format; MXINT: ebit=0, mbit=nbit */
    int32_t sc_ebit, sc_mbit;      /* shared-scale format; sc_mbit==0 => power of two */
    int32_t block_size;
    int32_t scale_allow_subnormal;
    int32_t use_round;             /* MXFP PoT scale: round(log2) instead of floor */
    int32_t use_ceil;              /* FP scale: ceil the scale mantissa */
    int32_t l2_block_size;         /* HBQ micro-block */
    int32_t l2_sc_bit;             /* HBQ: log2(#candidates) */
    int32_t l2_scheme;             /* ORC_L2_* */
    int32_t per_tensor_scale;      /* MXFP only */
    int32_t reserved;
} orc_format;

/* Quantize-dequantize rows x K fp16 values along K in blocks (zero padded to a
 * multiple of block_size, quantizer.py:67-130).  nblk = ceil(K/block_size).
 *   deq     [rows*K]            dequantised fp16 (required)
 *   scale   [rows*nblk]         shared (L1) scale as fp16 (VSQ: the row's first-level scale), or NULL
 *   l2idx   [rows*nblk*nl2]     HBQ chosen candidate index per micro-block (MXEx: 1 where the
 *                               step-2 grid won; VSQ: the block's second-level scale, nl2 = 1), or NULL
 *   scheme  [rows*nblk]         HBQ "Mix" chosen scheme, or NULL
 *   codes   [rows*nblk*block]   one element code per byte, or NULL:
 *                               FP: {sign, exp field, mantissa} as make_fp_quant's
 *                               detailed output (quantizer.py:249-253); INT: two's complement.
 * Returns 0, or a negative value for an unsupported format. */
int orc_quantize(const uint16_t* x, int64_t rows, int64_t K, const orc_format* fmt,
                 uint16_t* deq, uint16_t* scale, uint8_t* l2idx, uint8_t* scheme,
                 uint8_t* codes);

/* Element quantizer of make_fp_quant (quantizer.py:187-257) applied to n fp16
 * values; elem_variant=1 uses the +0.5004 rounding of the closure, 0 the +0.5
 * of the free function fp_quant (quantizer.py:259-328). */
void orc_fp_quant(const uint16_t* x, int64_t n, int ebit, int mbit, int allow_subnormal,
                  int use_ceil, int elem_variant, uint16_t* out);

/* floor(log2(x)) as the reference evaluates it on an fp16 tensor. */
void orc_floor_log2_h(const uint16_t* x, int64_t n, float* out);

/* GEMM accumulation models, A[M,K] B[K,N] C[M,N] fp16 row-major (gemm.cu). */
enum { ORC_ACC_FP32 = 0, ORC_ACC_FP16 = 1, ORC_ACC_GROUPED = 2,
       ORC_ACC_PSUM_INT8 = 3, ORC_ACC_PSUM_E3M4 = 4 };
int orc_gemm(const uint16_t* A, const uint16_t* B, uint16_t* C, int64_t M, int64_t N,
             int64_t K, int mode, int group_k, int group_n);
/* Same, rows [m0, m1) of C only (bounded CPU-baseline samples). */
int orc_gemm_rows(const uint16_t* A, const uint16_t* B, uint16_t* C, int64_t M, int64_t N,
                  int64_t K, int mode, int group_k, int group_n, int64_t m0, int64_t m1);

int orc_num_threads(void);
/* Launchers such as torchrun export OMP_NUM_THREADS=1; the CPU baseline sets its thread count itself. */
void orc_set_num_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
