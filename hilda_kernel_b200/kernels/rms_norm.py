"""RMSNorm on hand-written sm_100a kernels, behind the reference operator interface.

Mirrors kernels/rms_norm.py of hilda-kernel: ``rms_norm_forward`` (:261-306), ``rms_norm_backward``
(:309-359), ``HildaRMSNormFunction`` (:366-386), ``hilda_rms_norm`` (:389-391), ``RMSNorm`` (:398-413).
"""
import torch

from .. import _lib as L
from .._lib import device_guard


def rms_norm_forward(X, W, eps=1e-6):
    """Returns (Y, X_flat, RSTD) like the reference; only rstd is saved for the backward."""
    dev = L.require_cuda(X, W)
    shape = X.shape
    hidden_dim = shape[-1]
    X_flat = X.reshape(-1, hidden_dim).contiguous()
    W = W.contiguous()
    n_rows, n_cols = X_flat.shape
    assert n_cols == W.shape[0], f"Hidden dim mismatch: {n_cols} vs {W.shape[0]}"
    Y = torch.empty_like(X_flat)
    RSTD = torch.empty(n_rows, dtype=torch.float32, device=dev)
    with device_guard(dev):
        rc = L.lib().hilda_rms_norm_fwd(L.ptr(X_flat), L.ptr(W), L.ptr(Y), L.ptr(RSTD), n_rows, n_cols, float(eps),
                                        L.dt(X_flat), L.dt(W), L.stream(dev))
    L.check(rc, "rms_norm_fwd")
    return Y.view(*shape), X_flat, RSTD


def _norm_backward(dY, dS, X_flat, W, RSTD, shape):
    dev = X_flat.device
    n_rows, n_cols = X_flat.shape
    dY_flat = dY.reshape(-1, n_cols).contiguous() if dY is not None else None
    dS_flat = dS.reshape(-1, n_cols).contiguous() if dS is not None else None
    W = W.contiguous()
    dX = torch.empty_like(X_flat)
    dW = torch.empty_like(W)
    with device_guard(dev):
        lib = L.lib()
        ws_bytes = lib.hilda_norm_bwd_workspace_bytes(n_rows, n_cols, L.dt(X_flat))
        ws = torch.empty(max(ws_bytes // 4, 4), dtype=torch.float32, device=dev)
        rc = lib.hilda_norm_bwd(L.ptr(dY_flat), L.ptr(dS_flat), L.ptr(X_flat), L.ptr(W), L.ptr(RSTD), L.ptr(dX),
                                L.ptr(dW), L.ptr(ws), n_rows, n_cols, L.dt(X_flat), L.dt(W), L.stream(dev))
    L.check(rc, "norm_bwd")
    return dX.view(*shape), dW


def rms_norm_backward(dY, X, W, RSTD):
    """dX in X's dtype, dW in W's dtype (fp32 partial sums per CTA + a fixed-order second pass)."""
    L.require_cuda(dY, X, W, RSTD)
    X_flat = X.reshape(-1, X.shape[-1])
    return _norm_backward(dY, None, X_flat, W, RSTD, dY.shape)


class HildaRMSNormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, W, eps=1e-6):
        Y, X_flat, RSTD = rms_norm_forward(X, W, eps)
        ctx.save_for_backward(X_flat, W, RSTD)
        return Y

    @staticmethod
    def backward(ctx, dY):
        X_flat, W, RSTD = ctx.saved_tensors
        dX, dW = rms_norm_backward(dY, X_flat, W, RSTD)
        return dX, dW, None


def hilda_rms_norm(X, W, eps=1e-6):
    """Functional interface for RMSNorm."""
    return HildaRMSNormFunction.apply(X, W, eps)


class RMSNorm(torch.nn.Module):
    def __init__(self, hidden_dim, eps=1e-6):
        super().__init__()
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(hidden_dim))

    def forward(self, x):
        return hilda_rms_norm(x, self.weight, self.eps)
