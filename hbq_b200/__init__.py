"""hbq_b200 -- B200 (sm_100a) implementation of HBQ's hot path: block quantize-dequantize and the
GEMM with modelled low-precision accumulation, behind the reference's Python interface.

Importing the package does not need a GPU; the CUDA library (``lib/libhbq_b200.so``, built by
``python -m hbq_b200.build``) is loaded on first use and there is no fallback without it.
"""
from . import blockquant_ext  # noqa: F401
from ._lib import HbqError, launch_count  # noqa: F401
from .gemm import gemm, gemm_reserve_sms, gemm_status, gemm_status_reset  # noqa: F401
from .packed_gemm import W4Weight  # noqa: F401
from .fused import rmsnorm_quantize, softmax_quantize  # noqa: F401
from .kvcache import swiglu_quantize, write_k_cache, write_v_cache  # noqa: F401
from .llama import mixtral_8x7b, LlamaArch, QLlamaAttention, QLlamaDecoderLayer, QLlamaMLP, QLlamaModel  # noqa: F401
from .module import QLinear  # noqa: F401
from .ops import FP16AccumMatMul, FP32AccumMatMul  # noqa: F401
from .ptq import PTQConfig, load_quant_config  # noqa: F401
from .ep_moe import ExpertParallelMoE, QuantExpert  # noqa: F401
from .tp_linear import ColumnParallelQLinear, RowParallelQLinear  # noqa: F401
from .quantizer import (HBQQuantizer, MXExQuantizer, MXFPQuantizer, MXINTQuantizer, PackedTensor,  # noqa: F401
                        VSQQuantizer, _QBase,
                        dequantize_packed, get_max_norm, get_min_norm, get_min_subnorm)

__all__ = ["HBQQuantizer", "MXFPQuantizer", "MXINTQuantizer", "MXExQuantizer", "VSQQuantizer", "_QBase", "FP16AccumMatMul", "QLinear",
           "PTQConfig", "load_quant_config", "blockquant_ext", "gemm", "gemm_status", "gemm_status_reset", "PackedTensor",
           "dequantize_packed", "HbqError", "launch_count", "get_max_norm", "get_min_norm", "get_min_subnorm",
           "write_k_cache", "write_v_cache", "swiglu_quantize", "rmsnorm_quantize", "softmax_quantize", "ColumnParallelQLinear", "RowParallelQLinear", "LlamaArch", "mixtral_8x7b", "FP32AccumMatMul", "QLlamaModel", "QLlamaAttention", "QLlamaMLP", "QLlamaDecoderLayer", "ExpertParallelMoE", "QuantExpert", "W4Weight", "gemm_reserve_sms"]
