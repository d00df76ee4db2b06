"""SwiGLU activation, behind the reference operator interface.

Mirrors kernels/swiglu.py of hilda-kernel: ``swiglu_forward`` (:112-124), ``swiglu_backward``
(:127-141), ``HildaSwiGLUFunction`` (:148-159), ``hilda_swiglu`` (:162-164), ``SwiGLU`` (:171-174).
As in the reference, the backward writes da and db over the storage of the saved a and b.
"""
import torch

from .. import _lib as L
from .._lib import device_guard


def swiglu_forward(a, b):
    assert a.shape == b.shape, "a and b must have the same shape"
    assert a.dtype == b.dtype, "a and b must have the same dtype"
    dev = L.require_cuda(a, b)
    a, b = a.contiguous(), b.contiguous()
    c = torch.empty_like(b)
    with device_guard(dev):
        rc = L.lib().hilda_swiglu_fwd(L.ptr(a), L.ptr(b), L.ptr(c), a.numel(), L.dt(a), L.stream(dev))
    L.check(rc, "swiglu_fwd")
    return c


def swiglu_backward(a, b, dc):
    """Overwrites a with da and b with db (when they are contiguous) and returns them."""
    dev = L.require_cuda(a, b, dc)
    assert a.shape == b.shape == dc.shape, "a, b and dc must have the same shape"
    dc = dc.contiguous()
    if dc.dtype != a.dtype:
        dc = dc.to(a.dtype)
    a, b = a.contiguous(), b.contiguous()
    with device_guard(dev):
        rc = L.lib().hilda_swiglu_bwd(L.ptr(a), L.ptr(b), L.ptr(dc), L.ptr(a), L.ptr(b), a.numel(), L.dt(a),
                                      L.stream(dev))
    L.check(rc, "swiglu_bwd")
    return a, b


class HildaSwiGLUFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        c = swiglu_forward(a, b)
        ctx.save_for_backward(a, b)
        return c

    @staticmethod
    def backward(ctx, dc):
        a, b = ctx.saved_tensors
        da, db = swiglu_backward(a, b, dc)
        return da, db


def hilda_swiglu(a, b):
    """Functional interface: SwiGLU(a, b) = SiLU(a) * b."""
    return HildaSwiGLUFunction.apply(a, b)


class SwiGLU(torch.nn.Module):
    def forward(self, a, b):
        return hilda_swiglu(a, b)
