"""KL divergence loss, behind the reference operator interface.

Mirrors kernels/kl_div.py of hilda-kernel: ``kl_div_forward`` (:114-137), ``kl_div_backward`` (:140-165),
``HildaKLDivFunction`` (:172-186), ``hilda_kl_div`` (:189-191), ``KLDivLoss`` (:198-207). Conventions as
``torch.nn.KLDivLoss``: ``y_pred`` holds log-probabilities, ``y_true`` probabilities (log-probabilities
with ``log_target``). As in the reference ``reduction='none'`` returns the per-ROW sums, and its
backward ignores the upstream gradient. Unlike the reference the upstream gradient stays on the
device (no ``float(grad_output)`` host sync).
"""
import torch

from .. import _lib as L
from .._lib import device_guard

_RED = {"none": 0, "sum": 1, "mean": 2, "batchmean": 3}


def kl_div_forward(y_pred, y_true, reduction='batchmean', log_target=False, eps=1e-10):
    assert y_pred.shape == y_true.shape
    assert y_pred.dtype == y_true.dtype, "y_pred and y_true must have the same dtype"
    dev = L.require_cuda(y_pred, y_true)
    y_pred, y_true = y_pred.contiguous(), y_true.contiguous()
    n_cols = y_pred.shape[-1]
    n_rows = y_pred.numel() // max(n_cols, 1)
    loss_rows = torch.empty(n_rows, dtype=torch.float32, device=dev)
    loss_out = torch.empty((), dtype=torch.float32, device=dev)
    with device_guard(dev):
        rc = L.lib().hilda_kl_div_fwd(L.ptr(y_pred), L.ptr(y_true), L.ptr(loss_rows), L.ptr(loss_out), n_rows, n_cols,
                                      _RED[reduction], 1 if log_target else 0, float(eps), L.dt(y_pred), L.stream(dev))
    L.check(rc, "kl_div_fwd")
    return loss_rows if reduction == 'none' else loss_out


def kl_div_backward(y_true, grad_output, reduction='batchmean', log_target=False):
    dev = L.require_cuda(y_true)
    y_true = y_true.contiguous()
    n_cols = y_true.shape[-1]
    n_rows = y_true.numel() // max(n_cols, 1)
    dy_pred = torch.empty_like(y_true)
    g = None
    if reduction != 'none':
        g = torch.as_tensor(grad_output, dtype=torch.float32, device=dev).reshape(-1)[:1].contiguous()
    with device_guard(dev):
        rc = L.lib().hilda_kl_div_bwd(L.ptr(y_true), L.ptr(dy_pred), L.ptr(g), n_rows, n_cols, _RED[reduction],
                                      1 if log_target else 0, L.dt(y_true), L.stream(dev))
    L.check(rc, "kl_div_bwd")
    return dy_pred


class HildaKLDivFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_pred, y_true, reduction, log_target, eps):
        loss = kl_div_forward(y_pred, y_true, reduction, log_target, eps)
        ctx.save_for_backward(y_true)
        ctx.reduction = reduction
        ctx.log_target = log_target
        return loss

    @staticmethod
    def backward(ctx, grad_output):
        y_true, = ctx.saved_tensors
        dy_pred = kl_div_backward(y_true, grad_output, ctx.reduction, ctx.log_target)
        return dy_pred, None, None, None, None


def hilda_kl_div(y_pred, y_true, reduction='batchmean', log_target=False, eps=1e-10):
    """Functional interface: KL(y_true || y_pred). y_pred is log-probs."""
    return HildaKLDivFunction.apply(y_pred, y_true, reduction, log_target, eps)


class KLDivLoss(torch.nn.Module):
    """Drop-in replacement for torch.nn.KLDivLoss."""

    def __init__(self, reduction='batchmean', log_target=False, eps=1e-10):
        super().__init__()
        self.reduction = reduction
        self.log_target = log_target
        self.eps = eps

    def forward(self, y_pred, y_true):
        return hilda_kl_div(y_pred, y_true, self.reduction, self.log_target, self.eps)
