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
if __package__ == "kernels":
    # Imported as the top-level package ``kernels`` (this package's parent directory is on sys.path,
    # the way the reference's bench scripts put ``triton-kernels/`` there, benchmarks/bench_rms_norm.py:17-19):
    # alias the real package and its sub-modules, so that ``from kernels.rope import rope_forward`` works
    # and there is a single copy of every class however it was imported.
    import os as _os
    import sys as _sys
    _root = _os.path.dirname(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))
    if _root not in _sys.path:
        _sys.path.append(_root)
    _real = import_module("hilda_kernel_b200.kernels")
    for _module in _EXPORTS:
        _m = import_module(f"hilda_kernel_b200.kernels.{_module}")
        _sys.modules[f"{__name__}.{_module}"] = _m
        globals()[_module] = _m
    for _n in _real.__all__:
        globals()[_n] = getattr(_real, _n)
        __all__.append(_n)
    del _os, _sys, _root, _real
else:
    for _module, _names in _EXPORTS.items():
        _m = import_module(f".{_module}", __name__)
        for _n in _names:
            globals()[_n] = getattr(_m, _n)
            __all__.append(_n)
    del _names
del _module, _m, _n
