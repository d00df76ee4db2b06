"""GeGLU activation (tanh-approximated GELU gate), behind the reference operator interface.

Mirrors kernels/geglu.py of hilda-kernel: ``geglu_forward`` (:131-143), ``geglu_backward`` (:146-159),
``HildaGeGLUFunction`` (:166-177), ``hilda_geglu`` (:180-182), ``GeGLU`` (:189-192). Same skeleton as
SwiGLU; as in the reference the backward writes da and db over the storage of the saved a and b.
"""
import torch

from .. import _lib as L
from .._lib import device_guard


def geglu_forward(a, b):
    assert a.shape == b.shape, "a and b must have the same shape"
    assert a.dtype == b.dtype, "a and b must have the same dtype"
    dev = L.require_cuda(a, b)
    a, b = a.contiguous(), b.contiguous()
    c = torch.empty_like(b)
    with device_guard(dev):
        rc = L.lib().hilda_geglu_fwd(L.ptr(a), L.ptr(b), L.ptr(c), a.numel(), L.dt(a), L.stream(dev))
    L.check(rc, "geglu_fwd")
    return c


def geglu_backward(a, b, dc):
    """Overwrites a with da and b with db (when they are contiguous) and returns them."""
    dev = L.require_cuda(a, b, dc)
    assert a.shape == b.shape == dc.shape, "a, b and dc must have the same shape"
    dc = dc.contiguous()
    if dc.dtype != a.dtype:
        dc = dc.to(a.dtype)
    a, b = a.contiguous(), b.contiguous()
    with device_guard(dev):
        rc = L.lib().hilda_geglu_bwd(L.ptr(a), L.ptr(b), L.ptr(dc), L.ptr(a), L.ptr(b), a.numel(), L.dt(a),
                                     L.stream(dev))
    L.check(rc, "geglu_bwd")
    return a, b


class HildaGeGLUFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        c = geglu_forward(a, b)
        ctx.save_for_backward(a, b)
        return c

    @staticmethod
    def backward(ctx, dc):
        a, b = ctx.saved_tensors
        da, db = geglu_backward(a, b, dc)
        return da, db


def hilda_geglu(a, b):
    """Functional interface: GeGLU(a, b) = GELU_tanh(a) * b."""
    return HildaGeGLUFunction.apply(a, b)


class GeGLU(torch.nn.Module):
    def forward(self, a, b):
        return hilda_geglu(a, b)
