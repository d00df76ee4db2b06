"""Generalised Jensen-Shannon divergence, behind the reference operator interface.

Mirrors kernels/jsd.py of hilda-kernel: ``jsd_forward`` (:97-135), ``HildaJSDFunction`` (:142-153),
``hilda_jsd`` (:156-158), ``JSDLoss`` (:165-172). X holds the student's log-probabilities (log Q), Y
the teacher's (log P); beta = 0 gives KL(P||Q), beta = 1 KL(Q||P), otherwise
beta KL(P||M) + (1 - beta) KL(Q||M) with M = beta P + (1 - beta) Q. As in the reference one pass
produces the loss and dX, and the backward only multiplies by the upstream gradient. The count of
non-ignored rows stays on the device (the reference reads it back with ``.item()``).
"""
import torch

from .. import _lib as L
from .._lib import device_guard


def jsd_forward(X, Y, beta=0.5, labels=None, ignore_index=-100):
    """X, Y: [BT, V] log-probs; labels: optional [BT]. Returns (loss scalar, dX)."""
    assert X.shape == Y.shape and X.dim() == 2
    assert X.dtype == Y.dtype, "X and Y must have the same dtype"
    dev = L.require_cuda(X, Y)
    X, Y = X.contiguous(), Y.contiguous()
    n_rows, n_cols = X.shape
    if labels is not None:
        L.require_cuda(labels)
        labels = labels.contiguous().long()
    loss_rows = torch.empty(n_rows, dtype=torch.float32, device=dev)
    loss_out = torch.empty((), dtype=torch.float32, device=dev)
    dX = torch.empty_like(X)
    ws = torch.empty(1, dtype=torch.int32, device=dev)
    with device_guard(dev):
        rc = L.lib().hilda_jsd_fwd(L.ptr(X), L.ptr(Y), L.ptr(dX), L.ptr(loss_rows), L.ptr(loss_out), L.ptr(labels),
                                   int(ignore_index), L.ptr(ws), n_rows, n_cols, float(beta), L.dt(X), L.stream(dev))
    L.check(rc, "jsd_fwd")
    return loss_out, dX


class HildaJSDFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, Y, beta, labels, ignore_index):
        loss, dX = jsd_forward(X, Y, beta, labels, ignore_index)
        ctx.save_for_backward(dX)
        return loss

    @staticmethod
    def backward(ctx, grad_output):
        dX, = ctx.saved_tensors
        return dX * grad_output, None, None, None, None


def hilda_jsd(X, Y, beta=0.5, labels=None, ignore_index=-100):
    """Functional interface: JSD(beta)(teacher || student)."""
    return HildaJSDFunction.apply(X, Y, beta, labels, ignore_index)


class JSDLoss(torch.nn.Module):
    """Jensen-Shannon divergence loss."""

    def __init__(self, beta=0.5, ignore_index=-100):
        super().__init__()
        self.beta = beta
        self.ignore_index = ignore_index

    def forward(self, X, Y, labels=None):
        return hilda_jsd(X, Y, self.beta, labels, self.ignore_index)
