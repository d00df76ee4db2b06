"""Tolerances of the parity tests (fp32 rtol 1e-5; bf16/fp16 outputs and grads rtol 1.6e-2,
atol 1e-2; scalar losses 1e-4 relative)."""
import torch

BF16_RTOL, BF16_ATOL = 1.6e-2, 1e-2
LOSS_REL = 1e-4


def assert_close(actual, expected, dtype=None, scale=None, what="", normalize=False):
    """Compare in fp32. For fp32 data: rtol 1e-5 plus an atol of 1e-5 x the expected tensor's scale
    (results of reductions can cancel to ~0). For 16-bit data: rtol 1.6e-2, atol 1e-2.
    normalize=True first divides both sides by max|expected| (gradients of a mean over many
    tokens are ~1e-4 in size; an absolute 1e-2 would accept anything)."""
    dtype = dtype or actual.dtype
    a = actual.detach().float().cpu()
    e = expected.detach().float().cpu()
    assert a.shape == e.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(e.shape)}"
    if normalize:
        s = max(float(e.abs().max()), 1e-30)
        a, e, scale = a / s, e / s, 1.0
    if dtype == torch.float32:
        sc = scale if scale is not None else max(float(e.abs().max()), 1e-30)
        torch.testing.assert_close(a, e, rtol=1e-5, atol=1e-5 * sc, msg=lambda m: f"{what}: {m}")
    else:
        torch.testing.assert_close(a, e, rtol=BF16_RTOL, atol=BF16_ATOL, msg=lambda m: f"{what}: {m}")


def assert_loss_close(actual, expected, what="loss"):
    a, e = float(actual), float(expected)
    assert abs(a - e) <= LOSS_REL * max(abs(e), 1e-6) + 1e-7, f"{what}: {a} vs {e}"
