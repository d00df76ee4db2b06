"""Operator modules named as in hilda-kernel's ``kernels`` package (kernels/__init__.py:1-29): for
every operator the autograd Function, the functional form and the nn.Module, so that
``from kernels import X`` in code written for the reference resolves here unchanged. The token-
parallel path (RMSNorm, FusedAddRMSNorm, RoPE, SwiGLU, CrossEntropy, FusedLinearCrossEntropy, GRPO)
plus GeGLU, the KL / Jensen-Shannon divergence losses, FusedLinearJSD, AttnRes and the paged FP8
decode attention."""
from importlib import import_module

# module -> public names it contributes (the reference's export list, grouped by module)
_EXPORTS = {
    "rms_norm": ("HildaRMSNormFunction", "hilda_rms_norm", "RMSNorm"),
    "fused_add_rms_norm": ("HildaFusedAddRMSNormFunction", "hilda_fused_add_rms_norm", "FusedAddRMSNorm"),
    "rope": ("HildaRopeFunction", "hilda_rope", "RotaryEmbedding"),
    "swiglu": ("HildaSwiGLUFunction", "hilda_swiglu", "SwiGLU"),
    "geglu": ("HildaGeGLUFunction", "hilda_geglu", "GeGLU"),
    "cross_entropy": ("HildaCrossEntropyFunction", "hilda_cross_entropy", "CrossEntropyLoss"),
    "fused_linear_cross_entropy": ("HildaFusedLinearCrossEntropyFunction", "hilda_fused_linear_cross_entropy",
                                   "FusedLinearCrossEntropyLoss"),
    "grpo_loss": ("HildaGRPOLossFunction", "hilda_grpo_loss", "GRPOLoss", "fused_selective_log_softmax"),
    "kl_div": ("HildaKLDivFunction", "hilda_kl_div", "KLDivLoss"),
    "jsd": ("HildaJSDFunction", "hilda_jsd", "JSDLoss"),
    "fused_linear_jsd": ("HildaFusedLinearJSDFunction", "hilda_fused_linear_jsd", "FusedLinearJSDLoss"),
    "attn_res": ("HildaAttnResFunction", "hilda_attn_res", "AttnRes"),
    "paged_attention_fp8": ("hilda_paged_attention_fp8_decode", "reference_paged_attention_decode"),
}

__all__ = []
for _module, _names in _EXPORTS.items():
    _m = import_module(f".{_module}", __name__)
    for _n in _names:
        globals()[_n] = getattr(_m, _n)
        __all__.append(_n)
del _module, _names, _m, _n
