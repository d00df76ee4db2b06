"""Softmax cross entropy with the gradient written in the forward pass.

Mirrors kernels/cross_entropy.py of hilda-kernel: ``cross_entropy_forward`` (:206-249),
``cross_entropy_backward`` (:252-264), ``HildaCrossEntropyFunction`` (:271-290),
``hilda_cross_entropy`` (:293-295), ``CrossEntropyLoss`` (:302-313).
One kernel reads each logits row once (the row lives in the registers of a thread-block cluster)
and writes its gradient row; ignored rows are not read at all.
"""
import torch

from .. import _lib as L
from .._lib import device_guard

_RED = {"none": 0, "mean": 1, "sum": 2}


def _is_unit_scalar(x):
    return x.ndim == 0 and x.dtype == torch.float32 and bool(x == 1.0)


def cross_entropy_forward(logits, targets, ignore_index=-100, reduction='mean', needs_grad=False,
                          n_valid_global=None):
    """Returns (loss, aux, n_valid): aux is the saved dlogits on the training path, lse otherwise.
    n_valid_global (int32 device scalar, optional): divide 'mean' by this count instead of the
    number of valid rows in this call (row-sharded use)."""
    if reduction not in _RED:
        raise ValueError(f"reduction must be one of {list(_RED)}, got {reduction!r}")
    dev = L.require_cuda(logits, targets)
    assert logits.dim() == 2 and targets.dim() == 1 and targets.shape[0] == logits.shape[0], \
        "expects (N, V) logits and (N,) targets"
    logits = logits.contiguous()
    targets = targets.contiguous()
    if targets.dtype != torch.int64:
        targets = targets.long()
    n_rows, n_cols = logits.shape
    per_token_loss = torch.empty(n_rows, dtype=torch.float32, device=dev)
    loss_out = torch.empty((), dtype=torch.float32, device=dev)
    grad = torch.empty_like(logits) if needs_grad else None
    lse = None if needs_grad else torch.empty(n_rows, dtype=torch.float32, device=dev)
    # the reference treats ignore_index == -1 as "nothing ignored" (cross_entropy.py:219-225);
    # no valid target equals -1, so comparing against it is the same thing
    with device_guard(dev):
        lib = L.lib()
        ws = torch.empty(lib.hilda_cross_entropy_workspace_bytes(0) // 4, dtype=torch.int32, device=dev)
        rc = lib.hilda_cross_entropy_fwd(L.ptr(logits), L.ptr(targets), L.ptr(grad), L.ptr(per_token_loss), L.ptr(lse),
                                         L.ptr(loss_out), L.ptr(ws), L.ptr(n_valid_global), n_rows, n_cols, int(ignore_index),
                                         _RED[reduction], L.dt(logits), L.stream(dev))
    L.check(rc, "cross_entropy_fwd")
    L.check_status(ws[2], "cross_entropy_fwd")
    n_valid = ws[0]
    aux = grad if needs_grad else lse
    if reduction == 'none':
        return per_token_loss, aux, n_valid
    return loss_out, aux, n_valid


def cross_entropy_backward(dloss, saved_grad, reduction='mean'):
    """saved_grad already matches the reduction; only a non-unit upstream gradient costs a pass."""
    if reduction != 'none' and _is_unit_scalar(dloss):
        return saved_grad
    dev = saved_grad.device
    n_rows, n_cols = saved_grad.shape
    scale = dloss.to(torch.float32).contiguous()
    per_row = 1 if scale.ndim > 0 else 0
    dlogits = torch.empty_like(saved_grad)
    with device_guard(dev):
        rc = L.lib().hilda_scale_rows(L.ptr(saved_grad), L.ptr(dlogits), L.ptr(scale), per_row, n_rows, n_cols,
                                      L.dt(saved_grad), L.stream(dev))
    L.check(rc, "scale_rows")
    return dlogits


class HildaCrossEntropyFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, ignore_index, reduction):
        needs_grad = logits.requires_grad
        loss, aux, _ = cross_entropy_forward(logits, targets, ignore_index, reduction, needs_grad=needs_grad)
        ctx.reduction = reduction
        ctx.has_saved_grad = needs_grad
        if needs_grad:
            ctx.save_for_backward(aux)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        if not ctx.has_saved_grad:
            return None, None, None, None
        (saved_grad,) = ctx.saved_tensors
        return cross_entropy_backward(dloss, saved_grad, ctx.reduction), None, None, None


def hilda_cross_entropy(logits, targets, ignore_index=-100, reduction='mean'):
    """Functional interface for CrossEntropy."""
    return HildaCrossEntropyFunction.apply(logits, targets, ignore_index, reduction)


class CrossEntropyLoss(torch.nn.Module):
    """Expects (N, V) logits and (N,) targets (flatten bsz*seq before passing)."""

    def __init__(self, ignore_index=-100, reduction='mean'):
        super().__init__()
        self.ignore_index = ignore_index
        self.reduction = reduction

    def forward(self, logits, targets):
        return hilda_cross_entropy(logits, targets, self.ignore_index, self.reduction)
