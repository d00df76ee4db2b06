"""Operator modules named as in hilda-kernel's ``kernels`` package (kernels/__init__.py:1-12),
restricted to the token-parallel operator path: RMSNorm, FusedAddRMSNorm, RoPE, SwiGLU,
CrossEntropy, FusedLinearCrossEntropy and the GRPO loss, plus GeGLU (same kernels as SwiGLU), the
KL / Jensen-Shannon divergence losses and FusedLinearJSD (the tcgen05 GEMM of FusedLinearCrossEntropy
with a JSD row pass), AttnRes and the paged FP8 decode attention."""
from .rms_norm import HildaRMSNormFunction, hilda_rms_norm, RMSNorm
from .rope import HildaRopeFunction, hilda_rope, RotaryEmbedding
from .cross_entropy import HildaCrossEntropyFunction, hilda_cross_entropy, CrossEntropyLoss
from .swiglu import HildaSwiGLUFunction, hilda_swiglu, SwiGLU
from .geglu import HildaGeGLUFunction, hilda_geglu, GeGLU
from .fused_add_rms_norm import HildaFusedAddRMSNormFunction, hilda_fused_add_rms_norm, FusedAddRMSNorm
from .fused_linear_cross_entropy import (HildaFusedLinearCrossEntropyFunction, hilda_fused_linear_cross_entropy,
                                         FusedLinearCrossEntropyLoss)
from .attn_res import HildaAttnResFunction, hilda_attn_res, AttnRes
from .kl_div import HildaKLDivFunction, hilda_kl_div, KLDivLoss
from .jsd import HildaJSDFunction, hilda_jsd, JSDLoss
from .fused_linear_jsd import HildaFusedLinearJSDFunction, hilda_fused_linear_jsd, FusedLinearJSDLoss
from .grpo_loss import HildaGRPOLossFunction, hilda_grpo_loss, GRPOLoss, fused_selective_log_softmax
from .paged_attention_fp8 import hilda_paged_attention_fp8_decode, reference_paged_attention_decode

__all__ = [
    "HildaRMSNormFunction", "hilda_rms_norm", "RMSNorm",
    "HildaRopeFunction", "hilda_rope", "RotaryEmbedding",
    "HildaCrossEntropyFunction", "hilda_cross_entropy", "CrossEntropyLoss",
    "HildaSwiGLUFunction", "hilda_swiglu", "SwiGLU",
    "HildaGeGLUFunction", "hilda_geglu", "GeGLU",
    "HildaFusedAddRMSNormFunction", "hilda_fused_add_rms_norm", "FusedAddRMSNorm",
    "HildaFusedLinearCrossEntropyFunction", "hilda_fused_linear_cross_entropy", "FusedLinearCrossEntropyLoss",
    "HildaAttnResFunction", "hilda_attn_res", "AttnRes",
    "HildaKLDivFunction", "hilda_kl_div", "KLDivLoss",
    "HildaJSDFunction", "hilda_jsd", "JSDLoss",
    "HildaFusedLinearJSDFunction", "hilda_fused_linear_jsd", "FusedLinearJSDLoss",
    "HildaGRPOLossFunction", "hilda_grpo_loss", "GRPOLoss", "fused_selective_log_softmax",
    "hilda_paged_attention_fp8_decode", "reference_paged_attention_decode",
]
