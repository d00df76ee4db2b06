"""Fused residual-add + RMSNorm, behind the reference operator interface.

Mirrors kernels/fused_add_rms_norm.py of hilda-kernel: forward (:172-188), backward (:191-232),
``HildaFusedAddRMSNormFunction`` (:239-251), ``hilda_fused_add_rms_norm`` (:254-256),
``FusedAddRMSNorm`` (:263-274).
"""
import torch

from .. import _lib as L
from .._lib import device_guard
from .rms_norm import _norm_backward


def fused_add_rms_norm_forward(X, R, W, eps=1e-6):
    dev = L.require_cuda(X, R, W)
    assert X.shape == R.shape, "X and R must have the same shape"
    assert X.dtype == R.dtype, "X and R must have the same dtype"
    shape = X.shape
    n_cols = shape[-1]
    X_2d = X.reshape(-1, n_cols).contiguous()
    R_2d = R.reshape(-1, n_cols).contiguous()
    W = W.contiguous()
    assert n_cols == W.shape[0], f"Hidden dim mismatch: {n_cols} vs {W.shape[0]}"
    n_rows = X_2d.shape[0]
    Y = torch.empty_like(X_2d)
    S = torch.empty_like(X_2d)
    RSTD = torch.empty(n_rows, dtype=torch.float32, device=dev)
    with device_guard(dev):
        rc = L.lib().hilda_fused_add_rms_norm_fwd(L.ptr(X_2d), L.ptr(R_2d), L.ptr(W), L.ptr(Y), L.ptr(S), L.ptr(RSTD),
                                                  n_rows, n_cols, float(eps), L.dt(X_2d), L.dt(W), L.stream(dev))
    L.check(rc, "fused_add_rms_norm_fwd")
    return Y.view(shape), S.view(shape), RSTD


def fused_add_rms_norm_backward(dY, dS_out, S, W, RSTD, eps=1e-6):
    """Returns (dX, dR, dW); dX and dR are the same tensor, as in the reference (:231-232)."""
    L.require_cuda(dY, dS_out, S, W, RSTD)
    S_2d = S.reshape(-1, S.shape[-1]).contiguous()
    dX, dW = _norm_backward(dY, dS_out, S_2d, W, RSTD, S.shape)
    return dX, dX, dW


class HildaFusedAddRMSNormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, R, W, eps):
        Y, S, RSTD = fused_add_rms_norm_forward(X, R, W, eps)
        ctx.save_for_backward(S, W, RSTD)
        ctx.eps = eps
        # an output nobody differentiates through arrives as None instead of a zero tensor,
        # which saves reading a full tensor of zeros in the backward kernel
        ctx.set_materialize_grads(False)
        return Y, S

    @staticmethod
    def backward(ctx, dY, dS_out):
        S, W, RSTD = ctx.saved_tensors
        dX, dR, dW = fused_add_rms_norm_backward(dY, dS_out, S, W, RSTD, ctx.eps)
        return dX, dR, dW, None


def hilda_fused_add_rms_norm(X, R, W, eps=1e-6):
    """Functional interface: returns (Y, S) where S = X + R, Y = RMSNorm(S) * W."""
    return HildaFusedAddRMSNormFunction.apply(X, R, W, eps)


class FusedAddRMSNorm(torch.nn.Module):
    def __init__(self, hidden_dim, eps=1e-6):
        super().__init__()
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(hidden_dim))

    def forward(self, X, R):
        return hilda_fused_add_rms_norm(X, R, self.weight, self.eps)
