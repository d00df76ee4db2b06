"""AttnRes (attention residuals): softmax attention over the depth of a stack of residual blocks,
behind the reference operator interface.

Mirrors kernels/attn_res.py of hilda-kernel: ``attn_res_forward`` (:213-260), ``attn_res_backward``
(:263-293), ``HildaAttnResFunction`` (:300-319), ``hilda_attn_res`` (:322-334), ``AttnRes`` (:341-352).
``h = sum_i alpha_i v_i`` with ``alpha = softmax_i <w_query, RMSNorm(v_i) * w_norm>`` per token, for
``V = stack(blocks)`` of shape [N, B, T, D] (or [N, B*T, D]), N <= 32. The forward reads every
block row once (online softmax over the blocks); dW_query / dW_norm are summed in a fixed order.
"""
import torch

from .. import _lib as L
from .._lib import device_guard


def attn_res_forward(blocks, w_query, w_norm, eps=1e-6):
    """blocks: list of N tensors [B, T, D] or stacked [N, B, T, D]. Returns (h, V_3d, alpha, rstd):
    h with the blocks' spatial shape, V_3d [N, B*T, D], alpha and rstd [N, B*T] fp32."""
    V = torch.stack(list(blocks)) if isinstance(blocks, (list, tuple)) else blocks
    dev = L.require_cuda(V, w_query, w_norm)
    orig_shape = V.shape
    N, D = V.shape[0], V.shape[-1]
    assert 1 <= N <= 32, "AttnRes supports up to 32 blocks"
    assert w_query.shape == (D,) and w_norm.shape == (D,)
    V_3d = V.reshape(N, -1, D).contiguous()
    n_tokens = V_3d.shape[1]
    w_query, w_norm = w_query.contiguous(), w_norm.contiguous()
    out = torch.empty(n_tokens, D, device=dev, dtype=V.dtype)
    alpha = torch.empty(N, n_tokens, device=dev, dtype=torch.float32)
    rstd = torch.empty(N, n_tokens, device=dev, dtype=torch.float32)
    with device_guard(dev):
        rc = L.lib().hilda_attn_res_fwd(L.ptr(V_3d), L.ptr(w_query), L.ptr(w_norm), L.ptr(out), L.ptr(alpha), L.ptr(rstd),
                                        N, n_tokens, D, float(eps), L.dt(V_3d), L.dt(w_query), L.dt(w_norm), L.stream(dev))
    L.check(rc, "attn_res_fwd")
    return out.view(list(orig_shape[1:])), V_3d, alpha, rstd


def attn_res_backward(dh, V_3d, w_query, w_norm, Alpha, RSTD, eps=1e-6):
    """Returns dV [N, B*T, D], dW_query [D], dW_norm [D]."""
    dev = L.require_cuda(dh, V_3d)
    N, n_tokens, D = V_3d.shape
    dh = dh.contiguous()
    if dh.dtype != V_3d.dtype:
        dh = dh.to(V_3d.dtype)
    w_query, w_norm = w_query.contiguous(), w_norm.contiguous()
    dV = torch.empty_like(V_3d)
    dwq, dwn = torch.empty_like(w_query), torch.empty_like(w_norm)
    lib = L.lib()
    with device_guard(dev):
        ws = torch.empty(max(lib.hilda_attn_res_bwd_workspace_bytes(n_tokens, D) // 4, 64), dtype=torch.float32, device=dev)
        rc = lib.hilda_attn_res_bwd(L.ptr(dh), L.ptr(V_3d), L.ptr(w_query), L.ptr(w_norm), L.ptr(Alpha), L.ptr(RSTD),
                                    L.ptr(dV), L.ptr(dwq), L.ptr(dwn), L.ptr(ws), N, n_tokens, D, L.dt(V_3d),
                                    L.dt(w_query), L.dt(w_norm), L.stream(dev))
    L.check(rc, "attn_res_bwd")
    return dV, dwq, dwn


class HildaAttnResFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, V_stacked, w_query, w_norm, eps):
        ctx.orig_shape = V_stacked.shape
        h, V_3d, Alpha, RSTD = attn_res_forward(V_stacked, w_query, w_norm, eps)
        ctx.save_for_backward(V_3d, w_query, w_norm, Alpha, RSTD)
        ctx.eps = eps
        return h

    @staticmethod
    def backward(ctx, dh):
        V_3d, w_query, w_norm, Alpha, RSTD = ctx.saved_tensors
        dV, dW_query, dW_norm = attn_res_backward(dh, V_3d, w_query, w_norm, Alpha, RSTD, ctx.eps)
        return dV.view(ctx.orig_shape), dW_query, dW_norm, None


def hilda_attn_res(blocks, w_query, w_norm, eps=1e-6):
    """blocks: [N, B, T, D] stacked or a list of [B, T, D]; w_query, w_norm: [D]. Returns [B, T, D]."""
    V = torch.stack(list(blocks)) if isinstance(blocks, (list, tuple)) else blocks
    return HildaAttnResFunction.apply(V, w_query, w_norm, eps)


class AttnRes(torch.nn.Module):
    """Attention residuals module: forward(blocks) -> h."""

    def __init__(self, hidden_dim, eps=1e-6):
        super().__init__()
        self.eps = eps
        self.w_query = torch.nn.Parameter(torch.randn(hidden_dim) * 0.02)
        self.w_norm = torch.nn.Parameter(torch.ones(hidden_dim))

    def forward(self, blocks):
        return hilda_attn_res(blocks, self.w_query, self.w_norm, self.eps)
