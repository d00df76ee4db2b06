"""GRPO PPO-clip loss with fused selective log-softmax.

Mirrors kernels/grpo_loss.py of hilda-kernel: ``fused_selective_log_softmax`` (:65-80),
``grpo_loss_forward`` (:241-297), ``grpo_loss_backward`` (:300-330), ``HildaGRPOLossFunction``
(:337-362), ``hilda_grpo_loss`` (:365-375), ``GRPOLoss`` (:382-397).
When the logits require grad, the forward kernel also writes dlogits for a unit upstream
gradient, so every active logits row is read exactly once; the backward then only rescales when
the upstream gradient is not 1.
"""
import torch

from .. import _lib as L
from .._lib import device_guard


def _mask_f32(mask):
    """The kernels take the mask as fp32: 0 skips the token, any other value is its weight in the
    reductions (the reference tests ``mask == 0`` in its kernels and weights with ``mask.float()``,
    grpo_loss.py:104, :264), so bool, integer and fractional float masks all behave as there."""
    if mask is None:
        return None
    return mask.to(torch.float32).contiguous()


@torch.no_grad()
def fused_selective_log_softmax(logits, input_ids, temperature=1.0, mask=None):
    """log-softmax evaluated only at the token ids: (B, L) fp32 for logits (B, L+1, V)."""
    assert logits.is_contiguous()
    dev = L.require_cuda(logits, input_ids, mask)
    B, L_plus_1, N = logits.shape
    Lc = L_plus_1 - 1
    input_ids = input_ids[:, -Lc:].contiguous() if Lc > 0 else input_ids[:, :0].contiguous()
    if input_ids.dtype != torch.int64:
        input_ids = input_ids.long()
    if mask is not None:
        mask = _mask_f32(mask[:, -Lc:] if Lc > 0 else mask[:, :0])
    log_p = torch.empty(B, Lc, dtype=torch.float32, device=dev)
    with device_guard(dev):
        rc = L.lib().hilda_selective_log_softmax(L.ptr(logits), L.ptr(input_ids), L.ptr(mask), L.ptr(log_p), B, Lc, N,
                                                 float(temperature), L.dt(logits), L.stream(dev))
    L.check(rc, "selective_log_softmax")
    return log_p


def grpo_loss_forward(logits, completion_ids, advantages, old_logp=None, ref_logp=None, completion_mask=None,
                      temperature=1.0, beta=0.0, eps_low=0.2, eps_high=0.2, needs_grad=False, batch_total=None):
    """Returns (loss, kl_mean | None, clip_ratio, lse, mask, dlogits | None). batch_total: number of
    sequences the loss is averaged over when this call sees only a shard of them."""
    assert logits.is_contiguous()
    dev = L.require_cuda(logits, completion_ids, advantages, old_logp, ref_logp, completion_mask)
    B, L_plus_1, N = logits.shape
    Lc = L_plus_1 - 1
    assert completion_ids.shape == (B, Lc), f"completion_ids must be {(B, Lc)}, got {tuple(completion_ids.shape)}"
    if beta != 0.0 and ref_logp is None:
        raise ValueError("ref_logp is required when beta != 0")
    ids = completion_ids.contiguous()
    if ids.dtype != torch.int64:
        ids = ids.long()
    adv = advantages.to(torch.float32).contiguous()
    old = old_logp.to(torch.float32).contiguous() if old_logp is not None else None
    ref = ref_logp.to(torch.float32).contiguous() if ref_logp is not None else None
    mask_i = _mask_f32(completion_mask)
    mask = mask_i if completion_mask is not None else torch.ones(B, Lc, device=dev)

    loss = torch.empty(B, Lc, device=dev, dtype=torch.float32)
    lse = torch.empty_like(loss)
    is_clipped = torch.empty_like(loss)
    kl = torch.empty_like(loss) if beta != 0.0 else None
    scalars = torch.empty(4, device=dev, dtype=torch.float32)
    dlogits = torch.empty_like(logits) if needs_grad else None
    with device_guard(dev):
        lib = L.lib()
        ws = torch.empty(lib.hilda_grpo_workspace_bytes(B) // 4 + 1, dtype=torch.float32, device=dev)
        rc = lib.hilda_grpo_loss_fwd(L.ptr(logits), L.ptr(ids), L.ptr(adv), L.ptr(old), L.ptr(ref), L.ptr(mask_i),
                                     L.ptr(dlogits), L.ptr(loss), L.ptr(kl), L.ptr(is_clipped), L.ptr(lse),
                                     L.ptr(scalars), L.ptr(ws), B, Lc, N, int(batch_total or 0), float(temperature),
                                     float(beta),
                                     float(eps_low), float(eps_high), L.dt(logits), L.stream(dev))
    L.check(rc, "grpo_loss_fwd")
    L.check_status(ws[:1].view(torch.int32)[0], "grpo_loss_fwd")
    kl_mean = scalars[1] if beta != 0.0 else None
    return scalars[0], kl_mean, scalars[2], lse, mask, dlogits


def grpo_loss_backward(grad_output, saved_dlogits):
    """dlogits = saved (unit-gradient) dlogits * grad_output; free when grad_output == 1."""
    if grad_output.ndim == 0 and bool(grad_output == 1.0):
        return saved_dlogits
    dev = saved_dlogits.device
    B, Lp1, N = saved_dlogits.shape
    scale = grad_output.to(torch.float32).reshape(1).contiguous()
    out = torch.empty_like(saved_dlogits)
    with device_guard(dev):
        rc = L.lib().hilda_scale_rows(L.ptr(saved_dlogits), L.ptr(out), L.ptr(scale), 0, B * Lp1, N,
                                      L.dt(saved_dlogits), L.stream(dev))
    L.check(rc, "scale_rows")
    return out


class HildaGRPOLossFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, completion_ids, advantages, old_logp, ref_logp, completion_mask,
                temperature, beta, eps_low, eps_high):
        needs_grad = logits.requires_grad
        loss, kl_mean, clip_ratio, lse, mask, dlogits = grpo_loss_forward(
            logits, completion_ids, advantages, old_logp, ref_logp, completion_mask,
            temperature, beta, eps_low, eps_high, needs_grad=needs_grad)
        ctx.has_saved_grad = needs_grad
        if needs_grad:
            ctx.save_for_backward(dlogits)
        ctx.mark_non_differentiable(clip_ratio)
        if kl_mean is not None:
            ctx.mark_non_differentiable(kl_mean)
        return loss, kl_mean, clip_ratio

    @staticmethod
    def backward(ctx, grad_loss, grad_kl, grad_clip):
        if not ctx.has_saved_grad:
            return (None,) * 10
        (dlogits,) = ctx.saved_tensors
        return (grpo_loss_backward(grad_loss, dlogits),) + (None,) * 9


def hilda_grpo_loss(logits, completion_ids, advantages, old_logp=None, ref_logp=None, completion_mask=None,
                    temperature=1.0, beta=0.0, eps_low=0.2, eps_high=0.2):
    """Functional interface: GRPO loss -> (loss, kl_mean | None, clip_ratio)."""
    return HildaGRPOLossFunction.apply(logits, completion_ids, advantages, old_logp, ref_logp, completion_mask,
                                       temperature, beta, eps_low, eps_high)


class GRPOLoss(torch.nn.Module):
    def __init__(self, temperature=1.0, beta=0.0, eps_low=0.2, eps_high=0.2):
        super().__init__()
        self.temperature = temperature
        self.beta = beta
        self.eps_low = eps_low
        self.eps_high = eps_high

    def forward(self, logits, completion_ids, advantages, old_logp=None, ref_logp=None, completion_mask=None):
        return hilda_grpo_loss(logits, completion_ids, advantages, old_logp, ref_logp, completion_mask,
                               self.temperature, self.beta, self.eps_low, self.eps_high)
