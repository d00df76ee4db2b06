"""Fused lm_head projection + cross entropy that never holds the full [BT, V] logits.

Mirrors kernels/fused_linear_cross_entropy.py of hilda-kernel:
``fused_linear_cross_entropy_forward`` (:103-171), ``HildaFusedLinearCrossEntropyFunction`` (:178-210),
``hilda_fused_linear_cross_entropy`` (:213-220), ``FusedLinearCrossEntropyLoss`` (:227-241).
As in the reference, both gradients are produced during the forward pass and the backward only
rescales them when the upstream gradient is not 1. The three GEMMs run on one hand-written
tcgen05/TMEM kernel; the logsumexp statistics come out of the first GEMM's epilogue.
Supported compute dtypes: bfloat16 and float16 (the tensor-core path); hidden dim multiple of 8.
"""
import os

import torch

from .. import _lib as L
from .._lib import device_guard

_RED = {"none": 0, "mean": 1, "sum": 2}

# Rows per chunk; None lets the library choose (scratch <= 1.25 GiB). Exposed for tests and tuning
# (environment HILDA_FLCE_CHUNK_ROWS sets the initial value).
CHUNK_ROWS = int(os.environ["HILDA_FLCE_CHUNK_ROWS"]) if os.environ.get("HILDA_FLCE_CHUNK_ROWS") else None
# Set True to synchronise after each call and raise if a device-side bounded wait ran out.
CHECK_STATUS = False
# Ignored tokens contribute nothing to the loss or to either gradient, so by default their rows are
# compacted away before the three GEMMs run (their d(hidden) rows come back as zeros). The index
# lists, the gather, the GEMM extents and the scatter all follow a count that stays on the device:
# the call makes no host synchronisation (the reference pays one for n_valid,
# fused_linear_cross_entropy.py:121). Set False to run the GEMMs over ignored rows too.
SKIP_IGNORED_ROWS = True
FLCE_COMPACT = 1  # HILDA_FLCE_COMPACT of the C ABI


def fused_linear_cross_entropy_forward(hidden_states, weight, targets, ignore_index=-100, reduction='mean',
                                       compute_grad=True, chunk_rows=None, skip_ignored=None):
    """Returns (loss, grad_input, grad_weight, n_valid); n_valid is a device scalar."""
    if skip_ignored is None:
        skip_ignored = SKIP_IGNORED_ROWS
    if reduction not in _RED:
        raise ValueError(f"reduction must be one of {list(_RED)}, got {reduction!r}")
    dev = L.require_cuda(hidden_states, weight, targets)
    assert hidden_states.dim() == 2 and weight.dim() == 2 and targets.dim() == 1, \
        "expects hidden (BT, H), weight (V, H), targets (BT,)"
    BT, H = hidden_states.shape
    V = weight.shape[0]
    assert weight.shape[1] == H, f"hidden dim mismatch: {H} vs {weight.shape[1]}"
    assert targets.shape[0] == BT
    if hidden_states.dtype != weight.dtype:
        raise TypeError("hidden_states and weight must share a dtype")
    if hidden_states.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("fused_linear_cross_entropy runs on the bf16/fp16 tensor-core path only")
    hidden_states = hidden_states.contiguous()
    weight = weight.contiguous()
    targets = targets.contiguous()
    if targets.dtype != torch.int64:
        targets = targets.long()
    chunk = chunk_rows if chunk_rows is not None else (CHUNK_ROWS or 0)
    flags = FLCE_COMPACT if skip_ignored else 0
    loss_rows = torch.empty(BT, dtype=torch.float32, device=dev) if reduction == 'none' else None
    loss_out = torch.empty((), dtype=torch.float32, device=dev)
    grad_input = torch.empty_like(hidden_states) if compute_grad else None
    grad_weight = torch.empty_like(weight) if compute_grad else None
    with device_guard(dev):
        lib = L.lib()
        nbytes = lib.hilda_flce_workspace_bytes(BT, H, V, chunk, 1 if compute_grad else 0, flags)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        rc = lib.hilda_fused_linear_cross_entropy_fwd(
            L.ptr(hidden_states), L.ptr(weight), L.ptr(targets), L.ptr(loss_out), L.ptr(loss_rows),
            L.ptr(grad_input), L.ptr(grad_weight), L.ptr(ws), BT, H, V, int(ignore_index), _RED[reduction],
            chunk, L.dt(hidden_states), flags, L.stream(dev))
    L.check(rc, "fused_linear_cross_entropy_fwd")
    head = ws[:8].view(torch.int32)
    # a bounded device-side wait that ran out leaves a code here and makes a mean / sum loss NaN;
    # reading the word is a host synchronisation, so only on request
    L.check_status(head[0], "fused_linear_cross_entropy_fwd", force=CHECK_STATUS)
    n_valid = head[1]
    loss = loss_rows if reduction == 'none' else loss_out
    return loss, grad_input, grad_weight, n_valid


def _scale_inplace(t, scale):
    with device_guard(t.device):
        rc = L.lib().hilda_scale_rows(L.ptr(t), L.ptr(t), L.ptr(scale), 0, t.shape[0], t.shape[1], L.dt(t),
                                      L.stream(t.device))
    L.check(rc, "scale_rows")


class HildaFusedLinearCrossEntropyFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden_states, weight, targets, ignore_index, reduction):
        compute_grad = hidden_states.requires_grad or weight.requires_grad
        loss, grad_input, grad_weight, _ = fused_linear_cross_entropy_forward(
            hidden_states, weight, targets, ignore_index, reduction, compute_grad=compute_grad)
        if compute_grad:
            ctx.save_for_backward(grad_input, grad_weight)
        ctx.compute_grad = compute_grad
        ctx.reduction = reduction
        return loss

    @staticmethod
    def backward(ctx, grad_output):
        if not ctx.compute_grad:
            return None, None, None, None, None
        grad_input, grad_weight = ctx.saved_tensors
        if ctx.reduction == 'none':
            raise NotImplementedError(
                "backward through reduction='none' is not provided: the gradients are formed in the "
                "forward pass for a scalar loss (the reference has the same limitation, "
                "fused_linear_cross_entropy.py:192-210)")
        # like the reference (:197-209): rescale the saved gradients in place unless grad_output == 1
        if not bool(grad_output == 1.0):
            scale = grad_output.to(torch.float32).reshape(1).contiguous()
            _scale_inplace(grad_input, scale)
            _scale_inplace(grad_weight, scale)
        return grad_input, grad_weight, None, None, None


def hilda_fused_linear_cross_entropy(hidden_states, weight, targets, ignore_index=-100, reduction='mean'):
    """Functional interface: fused lm_head + CE loss."""
    return HildaFusedLinearCrossEntropyFunction.apply(hidden_states, weight, targets, ignore_index, reduction)


class FusedLinearCrossEntropyLoss(torch.nn.Module):
    """Fused linear projection + cross-entropy loss; weight is an argument of forward."""

    def __init__(self, ignore_index=-100, reduction='mean'):
        super().__init__()
        self.ignore_index = ignore_index
        self.reduction = reduction

    def forward(self, hidden_states, weight, targets):
        return hilda_fused_linear_cross_entropy(hidden_states, weight, targets, self.ignore_index, self.reduction)
