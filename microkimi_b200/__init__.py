"""microkimi_b200 - the quantized decode hot path of the microkimi engine on
NVIDIA B200 (sm_100a): MXFP4 / q8_0 dequant-fused matvecs, the q8_0 lm_head,
MoE expert dispatch and q8_0 MLA decode attention, as hand-written CUDA behind
the C ABI in include/mk_cuda.h.  `ops` mirrors the engine's operator interface
(same names and argument meaning as the Rust functions it stands in for).
"""
from . import lib  # noqa: F401
from .ops import (Context, F32Weight, KdaLayer, MlaCache, MoeLayer, MxFp4Weight, Q8Head, Vq1Weight, dequant_any, dequant_fp8, matvec, matvec_packed,  # noqa: F401
                  attn_res, quantize_q8, rmsnorm)

__all__ = ["lib", "Context", "F32Weight", "KdaLayer", "MlaCache", "MoeLayer", "MxFp4Weight", "Q8Head", "Vq1Weight", "dequant_any", "dequant_fp8", "matvec", "matvec_packed",
           "attn_res", "quantize_q8", "rmsnorm"]
