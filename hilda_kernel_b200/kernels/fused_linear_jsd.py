"""Fused lm_head projections + JSD distillation loss that never holds the full [BT, V] logits.

Mirrors kernels/fused_linear_jsd.py of hilda-kernel: ``fused_linear_jsd_forward`` (:119-207),
``HildaFusedLinearJSDFunction`` (:214-246), ``hilda_fused_linear_jsd`` (:249-258), ``FusedLinearJSDLoss``
(:265-280). Student: ``student_input @ student_weight.T`` -> log-softmax at ``temperature`` -> X;
teacher the same (no gradient) -> Y; loss = JSD(beta)(P || Q) averaged over the rows whose label is
not ``ignore_index``. Gradients flow to the student's input and weight only, are formed in the
forward pass and, as in the reference, only rescaled by the backward.

Per row chunk: the two logits GEMMs run on the tcgen05 kernel of FusedLinearCrossEntropy with the
online log-sum-exp statistics (taken at 1/temperature) in their epilogues; ONE row kernel replaces
the reference's two log-softmax passes, its JSD kernel and its softmax-gradient kernel, going from
both heads' logits to the student's dlogits in place; two more GEMMs give the gradients. The
student's weight gradient is accumulated across chunks in fp32 (reference: in the 16-bit dtype).
Supported compute dtypes: bfloat16 and float16.
"""
import torch

from .. import _lib as L
from .._lib import device_guard
from .fused_linear_cross_entropy import _scale_inplace

# Rows per chunk; None lets the library choose (the two logits scratches together <= 2.5 GiB).
CHUNK_ROWS = None


def fused_linear_jsd_forward(student_input, student_weight, teacher_input, teacher_weight, labels=None, beta=0.5,
                             temperature=1.0, ignore_index=-100, compute_grad=True, chunk_rows=None):
    """student_input (BT, H), student_weight (V, H), teacher_input (BT, Ht), teacher_weight (V, Ht),
    labels (BT,) optional. Returns (loss, grad_student_input, grad_student_weight)."""
    dev = L.require_cuda(student_input, student_weight, teacher_input, teacher_weight)
    BT, H = student_input.shape
    V = student_weight.shape[0]
    Ht = teacher_input.shape[1]
    assert student_weight.shape[1] == H and teacher_weight.shape == (V, Ht) and teacher_input.shape[0] == BT
    dtype = student_input.dtype
    assert dtype in (torch.bfloat16, torch.float16), "fused linear + JSD runs on the 16-bit tensor-core path"
    assert student_weight.dtype == dtype and teacher_input.dtype == dtype and teacher_weight.dtype == dtype
    assert temperature > 0
    s_in, s_w = student_input.contiguous(), student_weight.contiguous()
    t_in, t_w = teacher_input.contiguous(), teacher_weight.contiguous()
    if labels is not None:
        L.require_cuda(labels)
        labels = labels.contiguous().long()
    lib = L.lib()
    dt = L.dt(s_in)
    inv_t = 1.0 / float(temperature)
    loss_rows = torch.empty(BT, dtype=torch.float32, device=dev)
    dh = torch.empty_like(s_in) if compute_grad else None
    dw = torch.empty_like(s_w) if compute_grad else None
    if BT == 0:
        if compute_grad:
            dw.zero_()
        return loss_rows.sum(), dh, dw
    with device_guard(dev):
        st = L.stream(dev)
        if chunk_rows is None:
            chunk_rows = CHUNK_ROWS or int(lib.hilda_flce_default_chunk_rows(BT, max(H, Ht), V))
        chunk_rows = max(1, min(int(chunk_rows), BT))
        n_chunks = -(-BT // chunk_rows)
        pitch, tiles = lib.hilda_flce_logits_pitch(V), lib.hilda_flce_stat_tiles(V)
        padded = lib.hilda_flce_padded_rows(chunk_rows)
        s_scr = torch.empty(padded * pitch, dtype=dtype, device=dev)
        t_scr = torch.empty(padded * pitch, dtype=dtype, device=dev)
        stats = torch.empty(chunk_rows * tiles * 2, dtype=torch.float32, device=dev)
        head = torch.zeros(2, dtype=torch.int32, device=dev)  # [status, n_valid]
        status_p, n_valid_p = head.data_ptr(), head.data_ptr() + 4
        if labels is not None:
            L.check(lib.hilda_count_valid(L.ptr(labels), BT, int(ignore_index), n_valid_p, st), "count_valid")
        dw32 = torch.empty(V, H, dtype=torch.float32, device=dev) if (compute_grad and n_chunks > 1) else None
        for c in range(n_chunks):
            r0 = c * chunk_rows
            rows = min(chunk_rows, BT - r0)
            sc, tc = s_in[r0:r0 + rows], t_in[r0:r0 + rows]
            lc = labels[r0:r0 + rows] if labels is not None else None
            rs_s = torch.empty(3, rows, dtype=torch.float32, device=dev)
            rs_t = torch.empty(3, rows, dtype=torch.float32, device=dev)
            for x, w, hdim, scr, rs in ((sc, s_w, H, s_scr, rs_s), (tc, t_w, Ht, t_scr, rs_t)):
                L.check(lib.hilda_flce_logits_scaled(L.ptr(x), L.ptr(w), L.ptr(scr), L.ptr(stats), rows, hdim, V, inv_t,
                                                     dt, status_p, st), "flce_logits_scaled")
                L.check(lib.hilda_flce_row_stats(L.ptr(stats), L.ptr(scr), None, L.ptr(rs), rows, V, 0, dt, None, 0, st),
                        "flce_row_stats")
            L.check(lib.hilda_fljsd_dlogits(L.ptr(s_scr), L.ptr(t_scr), L.ptr(rs_s), L.ptr(rs_t), L.ptr(lc),
                                            int(ignore_index), n_valid_p if labels is not None else None, BT,
                                            loss_rows.data_ptr() + 4 * r0, rows, V, float(beta), inv_t, dt, st),
                    "fljsd_dlogits")
            if not compute_grad:
                continue
            L.check(lib.hilda_flce_grad_hidden(L.ptr(s_scr), L.ptr(s_w), dh.data_ptr() + 2 * r0 * H, None, rows, H, V,
                                               dt, status_p, None, 0, st), "flce_grad_hidden")
            mode = 3 if n_chunks == 1 else (0 if c == 0 else (2 if c == n_chunks - 1 else 1))
            L.check(lib.hilda_flce_grad_weight(L.ptr(s_scr), L.ptr(sc), L.ptr(dw32), L.ptr(dw), mode, rows, H, V, dt,
                                               status_p, None, 0, st), "flce_grad_weight")
        # one reduction kernel; the loss comes out NaN if a bounded wait inside a GEMM ran out
        loss = torch.empty((), dtype=torch.float32, device=dev)
        L.check(lib.hilda_flce_sum_loss(L.ptr(loss_rows), BT, None, 0, status_p, L.ptr(loss), st), "flce_sum_loss")
    return loss, dh, dw


class HildaFusedLinearJSDFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, student_input, student_weight, teacher_input, teacher_weight, labels, beta, temperature,
                ignore_index):
        compute_grad = student_input.requires_grad or student_weight.requires_grad
        loss, grad_input, grad_weight = fused_linear_jsd_forward(
            student_input, student_weight, teacher_input, teacher_weight, labels, beta, temperature, ignore_index,
            compute_grad=compute_grad)
        if compute_grad:
            ctx.save_for_backward(grad_input, grad_weight)
        ctx.compute_grad = compute_grad
        return loss

    @staticmethod
    def backward(ctx, grad_output):
        if not ctx.compute_grad:
            return (None,) * 8
        grad_input, grad_weight = ctx.saved_tensors
        # like the reference (:232-245): rescale the saved gradients in place unless grad_output == 1
        if not bool(grad_output == 1.0):
            scale = grad_output.to(torch.float32).reshape(1).contiguous()
            _scale_inplace(grad_input, scale)
            _scale_inplace(grad_weight, scale)
        return grad_input, grad_weight, None, None, None, None, None, None


def hilda_fused_linear_jsd(student_input, student_weight, teacher_input, teacher_weight, labels=None, beta=0.5,
                           temperature=1.0, ignore_index=-100):
    """Functional interface: fused linear + JSD loss."""
    return HildaFusedLinearJSDFunction.apply(student_input, student_weight, teacher_input, teacher_weight, labels,
                                             beta, temperature, ignore_index)


class FusedLinearJSDLoss(torch.nn.Module):
    """Fused linear projection + JSD loss for knowledge distillation."""

    def __init__(self, beta=0.5, temperature=1.0, ignore_index=-100):
        super().__init__()
        self.beta = beta
        self.temperature = temperature
        self.ignore_index = ignore_index

    def forward(self, student_input, student_weight, teacher_input, teacher_weight, labels=None):
        return hilda_fused_linear_jsd(student_input, student_weight, teacher_input, teacher_weight, labels, self.beta,
                                      self.temperature, self.ignore_index)
