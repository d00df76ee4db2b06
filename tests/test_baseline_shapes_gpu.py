"""GPU parity at the FULL benchmark shapes of the token-parallel path (the reference's own bench
configurations: Llama-3-8B block operators at batch 4 x seq 4096, CrossEntropy [8192, 128256],
FusedLinearCE 16384 x 4096 x 128256 with the default row chunking, GRPO [16, 1024, 151936]).

The CPU oracle (oracle/reference_ops.py) needs minutes for the loss operators at these sizes, so it
is used where it finishes in seconds: on every element for the element-wise operators, and on a
seeded sample of rows for the row-independent loss operators (per-row loss / logsumexp, gradient
rows). Quantities that couple all rows (the scalar losses, d(W) of the fused linear operator, the
whole gradient tensors) are compared with the same plain-PyTorch oracle functions evaluated in
fp32 on CUDA tensors, in row chunks. Inputs are generated on the device from a fixed seed and the
sampled rows are copied to the host, so the oracle and the kernels see identical bits.
Tolerances: tests/util.py (fp32 rtol 1e-5; 16-bit rtol 1.6e-2 / atol 1e-2 after normalising by
max|expected|; scalar losses 1e-4 relative)."""
import pytest
import torch

from oracle import reference_ops as R
from tests.util import BF16_ATOL, BF16_RTOL, assert_close, assert_loss_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def dgen(seed):
    return torch.Generator(device=DEV).manual_seed(seed)


def close_on_device(actual, expected, what):
    """The 16-bit criterion of tests/util.assert_close(normalize=True), evaluated on the device in row
    blocks (the tensors are gigabytes): |a - e| <= atol * max|e| + rtol * |e| everywhere."""
    e_max = float(expected.abs().max())
    s = max(e_max, 1e-30)
    worst = 0.0
    a2, e2 = actual.reshape(-1, actual.shape[-1]), expected.reshape(-1, expected.shape[-1])
    step = max(1, (1 << 27) // a2.shape[-1])
    for r0 in range(0, a2.shape[0], step):
        a, e = a2[r0:r0 + step].float(), e2[r0:r0 + step].float()
        worst = max(worst, float((((a - e).abs() - BF16_RTOL * e.abs()) / s).max()))
    assert worst <= BF16_ATOL, f"{what}: worst normalised excess {worst} (max|expected| {e_max})"


def free():
    import gc
    gc.collect()
    torch.cuda.empty_cache()


# ------------------------------------------------------------------ config 2a: FusedAddRMSNorm
def test_fused_add_rms_norm_llama_block_shape():
    import hilda_kernel_b200 as hk
    g = dgen(2)
    x = torch.randn(4, 4096, 4096, device=DEV, generator=g).bfloat16()
    r = torch.randn(4, 4096, 4096, device=DEV, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(4096, device=DEV, generator=g)).bfloat16()
    dy = torch.randn(4, 4096, 4096, device=DEV, generator=g).bfloat16()
    ds = torch.randn(4, 4096, 4096, device=DEV, generator=g).bfloat16()
    xd, rd, wd = x.clone().requires_grad_(True), r.clone().requires_grad_(True), w.clone().requires_grad_(True)
    y, s = hk.hilda_fused_add_rms_norm(xd, rd, wd, 1e-6)
    torch.autograd.backward([y, s], [dy, ds])
    # CPU oracle on every element: forward in the operator's dtype, backward in fp32 from the rounded S
    y_ref, s_ref = R.fused_add_rms_norm(x.cpu(), r.cpu(), w.cpu(), 1e-6)
    assert torch.equal(s.cpu(), s_ref), "S = X + R must be bit-exact"
    assert_close(y, y_ref, torch.bfloat16, what="y")
    s32 = s_ref.float().requires_grad_(True)
    w32 = w.cpu().float().requires_grad_(True)
    y32 = (s32 / torch.sqrt(torch.mean(s32 ** 2, dim=-1, keepdim=True) + 1e-6)) * w32
    y32.backward(dy.cpu().float())
    assert_close(xd.grad, s32.grad + ds.cpu().float(), torch.bfloat16, what="dx")
    assert torch.equal(xd.grad, rd.grad)
    torch.testing.assert_close(wd.grad.float().cpu(), w32.grad, rtol=BF16_RTOL, atol=1e-2 * 16384 ** 0.5)
    free()


# ------------------------------------------------------------------ config 2b: RoPE
@pytest.mark.parametrize("cs_dtype", [torch.bfloat16, torch.float32])
def test_rope_llama_block_shape(cs_dtype):
    import hilda_kernel_b200 as hk
    g = dgen(3)
    # memory order (B, S, H, D), handed over as (B, H, S, D) views, theta = 500000, positions 0..4095
    q = torch.randn(4, 4096, 32, 128, device=DEV, generator=g).bfloat16().transpose(1, 2)
    k = torch.randn(4, 4096, 8, 128, device=DEV, generator=g).bfloat16().transpose(1, 2)
    dq = torch.randn(4, 4096, 32, 128, device=DEV, generator=g).bfloat16().transpose(1, 2)
    dk = torch.randn(4, 4096, 8, 128, device=DEV, generator=g).bfloat16().transpose(1, 2)
    cos, sin = R.rope_tables(4096, 128, base=500000.0, dtype=cs_dtype)
    qd, kd = q.clone().requires_grad_(True), k.clone().requires_grad_(True)
    assert qd.stride() == q.stride()
    qo, ko = hk.hilda_rope(qd, kd, cos.to(DEV), sin.to(DEV))
    torch.autograd.backward([qo, ko], [dq, dk])
    # With bf16 tables the oracle runs in bf16 and the kernel has the same rounding points (bit-exact
    # forward). With fp32 tables the kernel computes in fp32 and rounds once, while autograd through the
    # oracle on bf16 leaves would round each of the two gradient terms to bf16 before adding them (an
    # error of an ulp of the TERMS on a sum that may cancel): there the oracle is evaluated on the
    # same values held in fp32.
    up = (lambda t: t.cpu()) if cs_dtype == torch.bfloat16 else (lambda t: t.cpu().float())
    qr, kr = up(q).requires_grad_(True), up(k).requires_grad_(True)
    q_ref, k_ref = R.rope(qr, kr, cos, sin)
    torch.autograd.backward([q_ref, k_ref], [dq.cpu().to(q_ref.dtype), dk.cpu().to(k_ref.dtype)])
    if cs_dtype == torch.bfloat16:
        assert torch.equal(qo.cpu(), q_ref.detach()) and torch.equal(ko.cpu(), k_ref.detach())
    assert_close(qo, q_ref.to(torch.bfloat16), torch.bfloat16, what="q")
    assert_close(ko, k_ref.to(torch.bfloat16), torch.bfloat16, what="k")
    assert_close(qd.grad, qr.grad, torch.bfloat16, what="dq")
    assert_close(kd.grad, kr.grad, torch.bfloat16, what="dk")
    # in place on the same bits gives the same result
    from hilda_kernel_b200.kernels.rope import rope_forward
    q2, k2 = q.clone(), k.clone()
    qi, ki, _, _ = rope_forward(q2, k2, cos.to(DEV), sin.to(DEV), inplace=True)
    assert qi.data_ptr() == q2.data_ptr() and torch.equal(qi, qo.detach()) and torch.equal(ki, ko.detach())
    free()


# ------------------------------------------------------------------ config 2c: SwiGLU
def test_swiglu_llama_block_shape():
    import hilda_kernel_b200 as hk
    g = dgen(4)
    a = torch.randn(16384, 14336, device=DEV, generator=g).bfloat16()
    b = torch.randn(16384, 14336, device=DEV, generator=g).bfloat16()
    dc = torch.randn(16384, 14336, device=DEV, generator=g).bfloat16()
    a0, b0 = a.clone(), b.clone()
    ad, bd = a.requires_grad_(True), b.requires_grad_(True)
    c = hk.hilda_swiglu(ad, bd)
    c_keep = c.detach().clone()
    c.backward(dc)
    # element-wise, so a seeded sample of 2048 rows through the CPU oracle covers the arithmetic ...
    rows = torch.randperm(16384, generator=torch.Generator().manual_seed(4))[:2048].sort().values
    ar, br = a0[rows.to(DEV)].cpu().requires_grad_(True), b0[rows.to(DEV)].cpu().requires_grad_(True)
    c_ref = R.swiglu(ar, br)
    assert_close(c_keep[rows.to(DEV)], c_ref, torch.bfloat16, what="c")
    a32, b32 = ar.detach().float().requires_grad_(True), br.detach().float().requires_grad_(True)
    (torch.nn.functional.silu(a32) * b32).backward(dc[rows.to(DEV)].cpu().float())
    assert_close(ad.grad[rows.to(DEV)], a32.grad, torch.bfloat16, what="da")
    assert_close(bd.grad[rows.to(DEV)], b32.grad, torch.bfloat16, what="db")
    # ... and the same oracle function on the device covers every element (indexing, tails)
    a1, b1 = a0.float().requires_grad_(True), b0.float().requires_grad_(True)
    close_on_device(c_keep, R.swiglu(a0, b0), "c, every element")
    (torch.nn.functional.silu(a1) * b1).backward(dc.float())
    close_on_device(ad.grad, a1.grad, "da, every element")
    close_on_device(bd.grad, b1.grad, "db, every element")
    free()


# ------------------------------------------------------------------ config 3: CrossEntropy
def test_cross_entropy_benchmark_shape():
    from hilda_kernel_b200.kernels.cross_entropy import cross_entropy_forward
    N, V = 8192, 128256
    g = dgen(5)
    logits = (2 * torch.randn(N, V, device=DEV, generator=g)).bfloat16()
    cg = torch.Generator().manual_seed(5)
    targets = torch.randint(0, V, (N,), generator=cg)
    ignored = torch.randperm(N, generator=cg)[: round(0.1 * N)]
    targets[ignored] = -100
    td = targets.to(DEV)
    loss, grad, n_valid = cross_entropy_forward(logits, td, -100, "mean", needs_grad=True)
    rows_loss, _, _ = cross_entropy_forward(logits, td, -100, "none", needs_grad=False)
    nv = int((targets != -100).sum())
    assert int(n_valid) == nv
    # CPU oracle on 64 sampled rows (48 valid, 16 ignored): per-row loss and gradient rows
    valid = (targets != -100).nonzero().squeeze(1)
    pick = torch.cat([valid[torch.randperm(valid.numel(), generator=cg)[:48]], ignored[:16]])
    lr = logits[pick.to(DEV)].cpu().float().requires_grad_(True)
    per_row = R.cross_entropy_clamped(lr, targets[pick], -100, "none")
    (per_row.sum() / nv).backward()
    torch.testing.assert_close(rows_loss[pick.to(DEV)].cpu(), per_row.detach(), rtol=1e-4, atol=1e-5)
    assert_close(grad[pick.to(DEV)], lr.grad, torch.bfloat16, what="dlogits rows", normalize=True)
    # ignored rows: loss 0 and an exactly zero gradient row, all of them
    assert float(grad[td == -100].abs().max()) == 0.0 and float(rows_loss[td == -100].abs().max()) == 0.0
    # the scalar loss and the whole gradient against the oracle evaluated on the device in row blocks
    total = torch.zeros((), dtype=torch.float64, device=DEV)
    worst, scale = 0.0, None
    for r0 in range(0, N, 1024):
        x = logits[r0:r0 + 1024].float().requires_grad_(True)
        pr = R.cross_entropy_clamped(x, td[r0:r0 + 1024], -100, "none")
        (pr.sum() / nv).backward()
        total += pr.double().sum()
        scale = scale or float(x.grad.abs().max())
        worst = max(worst, float((((grad[r0:r0 + 1024].float() - x.grad).abs() - BF16_RTOL * x.grad.abs()) / scale).max()))
    assert_loss_close(loss, total / nv)
    assert worst <= BF16_ATOL, worst
    free()


# ------------------------------------------------------------------ config 4: FusedLinearCrossEntropy
def _flce_device_oracle(hidden, weight, targets, n_valid, rows_per_block=2048):
    """pytorch_linear_ce (benchmarks/bench_fused_linear_ce.py:36-38) with its matmul's rounding of the
    logits to the compute dtype, evaluated in fp32 on the device in row blocks with hand-written
    gradient formulas of the same loss (autograd would keep every block's logits alive)."""
    W = weight.float()
    dW = torch.zeros_like(W)
    dH = torch.empty(hidden.shape, dtype=torch.float32, device=hidden.device)
    per_row = torch.empty(hidden.shape[0], dtype=torch.float32, device=hidden.device)
    for r0 in range(0, hidden.shape[0], rows_per_block):
        h = hidden[r0:r0 + rows_per_block].float()
        t = targets[r0:r0 + rows_per_block]
        logits = (h @ W.T).to(hidden.dtype).float()
        keep = t != -100
        lse = torch.logsumexp(logits, dim=-1)
        tgt = logits.gather(1, t.clamp_min(0)[:, None]).squeeze(1)
        per_row[r0:r0 + rows_per_block] = torch.where(keep, lse - tgt, torch.zeros_like(lse))
        d = torch.softmax(logits, dim=-1)
        d[torch.arange(d.shape[0], device=d.device)[keep], t[keep]] -= 1.0
        d *= (keep.float() / n_valid)[:, None]
        dH[r0:r0 + rows_per_block] = d @ W
        dW += d.T @ h
    return per_row, dH, dW


def test_fused_linear_cross_entropy_benchmark_shape_default_chunking():
    """hidden [16384, 4096], W [128256, 4096] bf16, 5 % ignored, mean: the operator exactly as the
    benchmark runs it (library-chosen row chunks, fp32 d(W) accumulation over the chunks, ignored
    rows compacted away on the device)."""
    import hilda_kernel_b200._lib as L
    from hilda_kernel_b200.kernels import fused_linear_cross_entropy as F
    BT, H, V = 16384, 4096, 128256
    g = dgen(4)
    hidden = torch.randn(BT, H, device=DEV, generator=g).bfloat16()
    weight = (0.02 * torch.randn(V, H, device=DEV, generator=g)).bfloat16()
    cg = torch.Generator().manual_seed(4)
    targets = torch.randint(0, V, (BT,), generator=cg)
    targets[torch.randperm(BT, generator=cg)[: round(0.05 * BT)]] = -100
    td = targets.to(DEV)
    nv = int((targets != -100).sum())
    assert F.CHUNK_ROWS is None and F.SKIP_IGNORED_ROWS
    chunk = int(L.lib().hilda_flce_default_chunk_rows(BT, H, V))
    assert -(-BT // chunk) >= 3, "the default must split this shape into several row chunks"
    loss, dh, dw, n_valid = F.fused_linear_cross_entropy_forward(hidden, weight, td, -100, "mean", True)
    rows_loss, _, _, _ = F.fused_linear_cross_entropy_forward(hidden, weight, td, -100, "none", False)
    status = int(L.lib().hilda_gemm_get_pair())  # touch the library after the calls; status is checked below
    assert status >= 0 and int(n_valid) == nv
    # (1) CPU oracle on 32 sampled rows: per-row loss and the rows of d(hidden) (a row of d(hidden) needs
    # only that row's logits and the count of valid rows)
    valid = (targets != -100).nonzero().squeeze(1)
    pick = torch.cat([valid[torch.randperm(valid.numel(), generator=cg)[:28]], (targets == -100).nonzero().squeeze(1)[:4]])
    h_s = hidden[pick.to(DEV)].cpu().float().requires_grad_(True)
    w_c = weight.cpu().float()
    lg = h_s @ w_c.T
    lg = lg + (lg.to(torch.bfloat16).float() - lg).detach()
    pr = torch.nn.functional.cross_entropy(lg, targets[pick], ignore_index=-100, reduction="none")
    (pr.sum() / nv).backward()
    diff = (rows_loss[pick.to(DEV)].cpu() - pr.detach()).abs()
    assert float(diff.max()) <= 4 * 2.0 ** -8 * 4.0, float(diff.max())  # one 16-bit ulp of a logit on a rounding boundary
    assert_close(dh[pick.to(DEV)], h_s.grad, torch.bfloat16, what="d hidden rows", normalize=True)
    assert float(dh[td == -100].abs().max()) == 0.0
    # (2) everything that couples the rows: scalar loss, all of d(hidden), all of d(W)
    per_row, dH_ref, dW_ref = _flce_device_oracle(hidden, weight, td, nv)
    assert_loss_close(loss, per_row.double().sum() / nv)
    d2 = (rows_loss - per_row).abs()
    assert float(d2.max()) <= 4 * 2.0 ** -8 * 4.0 and float(d2.mean()) < 1e-4
    close_on_device(dh, dH_ref, "d hidden")
    close_on_device(dw, dW_ref, "d weight")
    # reference bench thresholds (bench_fused_linear_ce.py:41-93) as a floor
    assert float((dh.float() - dH_ref).abs().max()) < 5e-2 and float((dw.float() - dW_ref).abs().max()) < 5e-1
    # (3) the uncompacted path on the same inputs: same results
    loss_u, dh_u, dw_u, _ = F.fused_linear_cross_entropy_forward(hidden, weight, td, -100, "mean", True, skip_ignored=False)
    assert_loss_close(loss_u, loss)
    close_on_device(dh_u, dH_ref, "d hidden, uncompacted")
    close_on_device(dw_u, dW_ref, "d weight, uncompacted")
    free()


# ------------------------------------------------------------------ config 5: GRPO
def test_grpo_benchmark_shape():
    from hilda_kernel_b200.kernels.grpo_loss import grpo_loss_forward
    B, Lc, V = 16, 1023, 151936
    g = dgen(6)
    logits = torch.empty(B, Lc + 1, V, device=DEV, dtype=torch.bfloat16)
    for b in range(B):
        logits[b] = (2 * torch.randn(Lc + 1, V, device=DEV, generator=g)).bfloat16()
    cg = torch.Generator().manual_seed(6)
    ids = torch.randint(0, V, (B, Lc), generator=cg)
    adv = torch.randn(B, generator=cg)
    lens = torch.randint(256, 1025, (B,), generator=cg).clamp(max=Lc)
    mask = (torch.arange(Lc)[None] < lens[:, None]).int()
    idd, advd, maskd = ids.to(DEV), adv.to(DEV), mask.to(DEV)
    # log-probs of the current policy from the oracle, one sequence at a time on the device
    cur = torch.stack([R.selective_log_softmax(logits[b:b + 1].float(), idd[b:b + 1])[0] for b in range(B)])
    old = cur + 0.05 * torch.randn(B, Lc, generator=cg).to(DEV)
    ref = cur + 0.1 * torch.randn(B, Lc, generator=cg).to(DEV)
    loss, kl_mean, clip, lse, _, dlogits = grpo_loss_forward(logits, idd, advd, old, ref, maskd, 1.0, 0.1, 0.2, 0.2,
                                                             needs_grad=True)
    # (1) CPU oracle on sampled active tokens: the row's logsumexp and log-prob
    for b in (0, 7, 15):
        for l in (0, 100, int(lens[b]) - 1):
            row = logits[b, l].cpu().float()
            lse_ref = torch.logsumexp(row, dim=-1)
            assert abs(float(lse[b, l]) - float(lse_ref)) <= 1e-4 * abs(float(lse_ref))
            assert abs(float(cur[b, l]) - float(row[ids[b, l]] - lse_ref)) <= 1e-3
    # (2) the three scalars and the whole gradient: the oracle functions on the device, sequence by
    # sequence (the loss is a mean over sequences of per-sequence masked means)
    total = torch.zeros((), dtype=torch.float64, device=DEV)
    kl_num = torch.zeros((), dtype=torch.float64, device=DEV)
    clip_num = torch.zeros((), dtype=torch.float64, device=DEV)
    worst, scale = 0.0, None
    for b in range(B):
        x = logits[b:b + 1].float().requires_grad_(True)
        lb = R.grpo_loss(x, idd[b:b + 1], advd[b:b + 1], old[b:b + 1], ref[b:b + 1], maskd[b:b + 1], 1.0, 0.1, 0.2, 0.2)
        (lb / B).backward()
        total += lb.double().detach()
        klb, clb = R.grpo_aux(x.detach(), idd[b:b + 1], advd[b:b + 1], old[b:b + 1], ref[b:b + 1], maskd[b:b + 1],
                              1.0, 0.1, 0.2, 0.2)
        kl_num += klb.double() * int(mask[b].sum())
        clip_num += clb.double() * int(mask[b].sum())
        scale = scale or float(x.grad.abs().max())
        worst = max(worst, float((((dlogits[b:b + 1].float() - x.grad).abs() - BF16_RTOL * x.grad.abs()) / scale).max()))
        del x, lb
    assert_loss_close(loss, total / B)
    assert_loss_close(kl_mean, kl_num / int(mask.sum()), "kl_mean")
    assert abs(float(clip) - float(clip_num / int(mask.sum()))) <= 1e-3
    assert worst <= BF16_ATOL, worst
    assert float(dlogits[:, Lc].abs().max()) == 0.0  # the last position carries no gradient
    assert float(dlogits[:, :Lc][maskd == 0].abs().max()) == 0.0  # masked tokens neither
    free()


# ------------------------------------------------------------------ streams and graph replay
def test_operators_on_a_side_stream_and_in_graph_replay():
    """The ABI's contract is "work is enqueued on the given stream": every operator of the path run on
    a non-default stream, and again inside a captured CUDA graph that is replayed on fresh input
    values, must reproduce the default-stream result bit for bit (the kernels are deterministic)."""
    import hilda_kernel_b200 as hk
    from hilda_kernel_b200.kernels import (cross_entropy as CE, fused_add_rms_norm as FA,
                                           fused_linear_cross_entropy as FL, grpo_loss as GR, rms_norm as RN,
                                           rope as RP, swiglu as SW)
    g = dgen(9)
    rn = lambda *s: torch.randn(*s, device=DEV, generator=g)
    x, r, w, dy = rn(512, 2048).bfloat16(), rn(512, 2048).bfloat16(), (1 + 0.1 * rn(2048)).bfloat16(), rn(512, 2048).bfloat16()
    q, k = rn(2, 256, 8, 128).bfloat16().transpose(1, 2), rn(2, 256, 2, 128).bfloat16().transpose(1, 2)
    cos, sin = (t.to(DEV).bfloat16() for t in R.rope_tables(256, 128))
    a, b = rn(512, 3072).bfloat16(), rn(512, 3072).bfloat16()
    logits = (2 * rn(256, 32000)).bfloat16()
    tgt = torch.randint(0, 32000, (256,), device=DEV, generator=g)
    tgt[::9] = -100
    hid, W = rn(700, 512).bfloat16(), (0.05 * rn(3000, 512)).bfloat16()
    ftg = torch.randint(0, 3000, (700,), device=DEV, generator=g)
    ftg[::7] = -100
    gl = (2 * rn(2, 65, 8192)).bfloat16()
    gids = torch.randint(0, 8192, (2, 64), device=DEV, generator=g)
    gadv, gold = rn(2), rn(2, 64) * 0.1 - 9.0
    gmask = (torch.arange(64, device=DEV)[None] < torch.tensor([40, 64], device=DEV)[:, None]).int()

    def run_all():
        out = []
        y, xf, rstd = RN.rms_norm_forward(x, w)
        out += [y, *RN.rms_norm_backward(dy, xf, w, rstd)]
        y2, s2, rstd2 = FA.fused_add_rms_norm_forward(x, r, w)
        out += [y2, s2, *FA.fused_add_rms_norm_backward(dy, dy, s2, w, rstd2)]
        out += list(RP.rope_forward(q, k, cos, sin)[:2]) + list(RP.rope_backward(q, k, cos, sin))
        c = SW.swiglu_forward(a, b)
        out += [c, *SW.swiglu_backward(a.clone(), b.clone(), c)]
        out += list(CE.cross_entropy_forward(logits, tgt, -100, "mean", True)[:2])
        out += list(FL.fused_linear_cross_entropy_forward(hid, W, ftg, -100, "mean", True, chunk_rows=256)[:3])
        lo, kl, cl, lse, _, dl = GR.grpo_loss_forward(gl, gids, gadv, gold, gold + 0.05, gmask, 1.0, 0.1, 0.2, 0.2, True)
        out += [lo, kl, cl, lse, dl]
        return [t for t in out if isinstance(t, torch.Tensor)]

    ref = [t.clone() for t in run_all()]
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        got = run_all()
    side.synchronize()
    assert len(got) == len(ref) >= 25
    for i, (u, v) in enumerate(zip(got, ref)):
        assert torch.equal(u, v), f"side stream: output {i} differs"
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = run_all()
    for t in captured:
        if t.dtype.is_floating_point:
            t.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    for i, (u, v) in enumerate(zip(captured, ref)):
        assert torch.equal(u, v), f"graph replay: output {i} differs"
