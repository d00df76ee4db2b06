"""Rotate-half RoPE for q and k in one launch, behind the reference operator interface.

Mirrors kernels/rope.py of hilda-kernel: ``rope_forward`` (:113-136), ``rope_backward`` (:139-172),
``HildaRopeFunction`` (:179-197), ``hilda_rope`` (:200-202), ``RotaryEmbedding`` (:209-228).
q and k are indexed (bsz, n_heads, seq_len, head_dim) with arbitrary strides on the first three
dims (a transposed view of (B,S,H,D) memory is used as is, no copy); cos/sin are half-width
tables of shape (1 or bsz, seq_len, head_dim // 2).

Unlike the reference, ``inplace=True`` rotates q and k in their own storage (no output
allocation). The default stays out of place so the function is a drop-in.
"""
import ctypes as C

import torch

from .. import _lib as L
from .._lib import device_guard


def _usable(x):
    """The kernel needs a contiguous last dim and real (non-broadcast) strides."""
    if x.stride(-1) != 1 and x.shape[-1] > 1:
        return False
    return all(st != 0 or sz == 1 for st, sz in zip(x.stride(), x.shape))


def _prep_table(t):
    if t.dim() != 3:
        raise ValueError(f"cos/sin must be (1|bsz, seq, head_dim//2), got {tuple(t.shape)}")
    if t.stride(-1) != 1 and t.shape[-1] > 1:
        t = t.contiguous()
    return t


def _launch(q, k, q_out, k_out, cos, sin, backward):
    dev = L.require_cuda(q, k, cos, sin)
    bsz, n_qh, seq_len, hd = q.shape
    n_kh = k.shape[1]
    assert k.shape[0] == bsz and k.shape[2] == seq_len and k.shape[3] == hd, "q/k shape mismatch"
    assert q.dtype == k.dtype, "q and k must share a dtype"
    assert hd % 2 == 0, "head_dim must be even"
    cos, sin = _prep_table(cos), _prep_table(sin)
    assert cos.shape == sin.shape and cos.dtype == sin.dtype, "cos/sin mismatch"
    assert cos.shape[0] in (1, bsz) and cos.shape[1] >= seq_len and cos.shape[2] == hd // 2, \
        f"cos shape {tuple(cos.shape)} does not match q {tuple(q.shape)}"
    if sin.stride() != cos.stride():
        sin = sin.contiguous()
        cos = cos.contiguous()
    Arr = C.c_int64 * 6
    qs = Arr(q.stride(0), q.stride(1), q.stride(2), q_out.stride(0), q_out.stride(1), q_out.stride(2))
    ks = Arr(k.stride(0), k.stride(1), k.stride(2), k_out.stride(0), k_out.stride(1), k_out.stride(2))
    cos_sb = 0 if cos.shape[0] == 1 else cos.stride(0)
    with device_guard(dev):
        rc = L.lib().hilda_rope(L.ptr(q), L.ptr(q_out), qs, n_qh, L.ptr(k), L.ptr(k_out), ks, n_kh,
                                L.ptr(cos), L.ptr(sin), cos_sb, cos.stride(1), bsz, seq_len, hd,
                                L.dt(q), L.dt(cos), 1 if backward else 0, L.stream(dev))
    L.check(rc, "rope")


def rope_forward(q, k, cos, sin, inplace=False):
    """Returns (q_out, k_out, cos, sin). With inplace=True q_out is q and k_out is k."""
    if not _usable(q):
        q = q.contiguous()
    if not _usable(k):
        k = k.contiguous()
    q_out = q if inplace else torch.empty_like(q)
    k_out = k if inplace else torch.empty_like(k)
    _launch(q, k, q_out, k_out, cos, sin, backward=False)
    return q_out, k_out, cos, sin


def rope_backward(dq, dk, cos, sin):
    """The transpose rotation: the forward kernel with -sin. Returns new tensors (dq_out, dk_out)."""
    if not _usable(dq):
        dq = dq.contiguous()
    if not _usable(dk):
        dk = dk.contiguous()
    dq_out = torch.empty_like(dq)
    dk_out = torch.empty_like(dk)
    _launch(dq, dk, dq_out, dk_out, cos, sin, backward=True)
    return dq_out, dk_out


class HildaRopeFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, cos, sin, inplace=False):
        if inplace:
            if not (_usable(q) and _usable(k)):
                raise ValueError("inplace RoPE needs q and k with a contiguous last dim and no broadcast strides")
            ctx.mark_dirty(q, k)
        q_out, k_out, cos, sin = rope_forward(q, k, cos, sin, inplace=inplace)
        ctx.save_for_backward(cos, sin)
        return q_out, k_out

    @staticmethod
    def backward(ctx, dq, dk):
        cos, sin = ctx.saved_tensors
        dq_out, dk_out = rope_backward(dq, dk, cos, sin)
        return dq_out, dk_out, None, None, None


def hilda_rope(q, k, cos, sin, inplace=False):
    """Functional interface for RoPE."""
    return HildaRopeFunction.apply(q, k, cos, sin, inplace)


class RotaryEmbedding(torch.nn.Module):
    def __init__(self, dim, max_position_embeddings=2048, base=10000, device=None):
        super().__init__()
        self.dim = dim
        inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
        self.register_buffer("inv_freq", inv_freq)
        self._set_cos_sin_cache(max_position_embeddings, device)

    def _set_cos_sin_cache(self, seq_len, device):
        t = torch.arange(seq_len, device=device, dtype=self.inv_freq.dtype)
        freqs = torch.outer(t, self.inv_freq)
        emb = torch.cat((freqs, freqs), dim=-1)
        self.register_buffer("cos_cached", emb.cos()[None, :, :self.dim // 2])
        self.register_buffer("sin_cached", emb.sin()[None, :, :self.dim // 2])

    def forward(self, x, seq_len=None):
        return self.cos_cached[:, :seq_len], self.sin_cached[:, :seq_len]

    def apply_rotary(self, q, k, cos, sin):
        return hilda_rope(q, k, cos, sin)
