"""GPU parity tests: every CUDA operator against the CPU oracle (oracle/reference_ops.py) on
identical seeded inputs, and against the golden outputs of hilda-kernel's reference functions.
All calls go through the Python operator API, which calls the C ABI of libhilda_b200.so."""
import pytest
import torch

from oracle import reference_ops as R
from tests.util import assert_close, assert_loss_close

pytestmark = pytest.mark.gpu

DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16, torch.float16]


def gen(seed):
    return torch.Generator().manual_seed(seed)


def ops():
    import hilda_kernel_b200 as hk
    return hk


# ------------------------------------------------------------------ RMSNorm
@pytest.mark.parametrize("shape", [(2, 128, 1024), (4, 64, 2048), (2, 32, 4096), (1, 16, 8192), (3, 5, 4096),
                                   (1, 1, 4096), (7, 100), (5, 33), (2, 3, 20000), (4, 70000)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_fwd_bwd(shape, dtype):
    hk = ops()
    g = gen(0)
    x = torch.randn(*shape, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(shape[-1], generator=g)).to(dtype)
    dy = torch.randn(*shape, generator=g).to(dtype)
    # oracle in fp32 on the same (already rounded) inputs
    xr, wr = x.float().clone().requires_grad_(True), w.float().clone().requires_grad_(True)
    y_ref = R.rms_norm(xr, wr, 1e-6)
    y_ref.backward(dy.float())
    xd, wd = x.to(DEV).requires_grad_(True), w.to(DEV).requires_grad_(True)
    y = hk.hilda_rms_norm(xd, wd, 1e-6)
    assert y.dtype == dtype and y.shape == x.shape
    y.backward(dy.to(DEV))
    assert_close(y, y_ref, dtype, what="y")
    assert_close(xd.grad, xr.grad, dtype, what="dx")
    assert xd.grad.dtype == dtype and wd.grad.dtype == dtype
    rows = x.numel() // shape[-1]
    if dtype == torch.float32:
        assert_close(wd.grad, wr.grad, dtype, scale=float(rows) ** 0.5 * 3, what="dw")
    else:
        torch.testing.assert_close(wd.grad.float().cpu(), wr.grad, rtol=1.6e-2, atol=1e-2 * max(1.0, rows ** 0.5))


def test_rms_norm_config1_fp32():
    """The reference's RMSNorm benchmark configuration: x [4096,4096] fp32 ~N(0,1), w = 1 + N(0,0.1), eps 1e-6, dY ~N(0,1), seed 0."""
    hk = ops()
    g = gen(0)
    x = torch.randn(4096, 4096, generator=g)
    w = 1 + 0.1 * torch.randn(4096, generator=g)
    dy = torch.randn(4096, 4096, generator=g)
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    y_ref = R.rms_norm(xr, wr, 1e-6)
    y_ref.backward(dy)
    xd, wd = x.to(DEV).requires_grad_(True), w.to(DEV).requires_grad_(True)
    y = hk.hilda_rms_norm(xd, wd, 1e-6)
    y.backward(dy.to(DEV))
    assert_close(y, y_ref, what="y")
    assert_close(xd.grad, xr.grad, what="dx")
    # dW sums 4096 terms of either sign: tie-break against a float64 evaluation
    x64, w64 = x.double().requires_grad_(True), w.double().requires_grad_(True)
    R.rms_norm(x64, w64, 1e-6).backward(dy.double())
    err_ours = (wd.grad.cpu().double() - w64.grad).abs().max()
    err_ref = (wr.grad.double() - w64.grad).abs().max()
    assert err_ours <= max(2 * err_ref, 1e-5 * w64.grad.abs().max()), (float(err_ours), float(err_ref))


def test_rms_norm_golden(golden):
    hk = ops()
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        c = golden[f"rms_norm_{tag}"]
        x, w = c["x"].to(DEV).requires_grad_(True), c["w"].to(DEV).requires_grad_(True)
        y = hk.hilda_rms_norm(x, w, c["eps"])
        y.backward(c["dy"].to(DEV))
        assert_close(y, c["y"].to(dtype), dtype, what="y")
        assert_close(x.grad, c["dx"], dtype, what="dx")
        assert_close(w.grad, c["dw"], dtype, scale=10.0, what="dw")


def test_rms_norm_edge_cases():
    hk = ops()
    # all-zero input (tests/test_rms_norm.py:67-78)
    y = hk.hilda_rms_norm(torch.zeros(2, 64, 1024, device=DEV, dtype=torch.float16),
                          torch.ones(1024, device=DEV, dtype=torch.float16))
    assert float(y.abs().max()) < 1e-3
    # non-contiguous input (tests/test_rms_norm.py:80-95)
    g = gen(1)
    x = torch.randn(4, 256, 2048, generator=g).to(torch.float16)
    w = torch.randn(2048, generator=g).to(torch.float16)
    xt = x.to(DEV).transpose(0, 1)
    assert not xt.is_contiguous()
    y = hk.hilda_rms_norm(xt, w.to(DEV))
    assert_close(y, R.rms_norm_cast(x.transpose(0, 1).contiguous(), w), torch.float16)
    # empty batch
    y = hk.hilda_rms_norm(torch.empty(0, 512, device=DEV), torch.ones(512, device=DEV))
    assert y.shape == (0, 512)
    # fp32 module weight with bf16 activations (the module default), inside nn.Sequential
    m = torch.nn.Sequential(torch.nn.Linear(256, 512), hk.RMSNorm(512)).to(DEV)
    out = m(torch.randn(3, 256, device=DEV))
    out.sum().backward()
    assert out.shape == (3, 512) and m[1].weight.grad is not None
    xb = torch.randn(4, 512, generator=g).to(torch.bfloat16)
    norm = hk.RMSNorm(512).to(DEV)
    yb = norm(xb.to(DEV))
    assert yb.dtype == torch.bfloat16
    assert_close(yb, R.rms_norm_cast(xb, torch.ones(512)), torch.bfloat16)
    assert set(norm.state_dict()) == {"weight"}


def test_rms_norm_dw_deterministic():
    hk = ops()
    g = gen(2)
    x = torch.randn(3000, 4096, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.ones(4096, dtype=torch.bfloat16, device=DEV)
    dy = torch.randn(3000, 4096, generator=g).to(torch.bfloat16).to(DEV)
    outs = []
    for _ in range(2):
        xd, wd = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        hk.hilda_rms_norm(xd, wd).backward(dy)
        outs.append((xd.grad.clone(), wd.grad.clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


def test_norm_backward_ring_and_register_kernels_agree():
    """The backward's kernels (rows staged through a shared-memory ring; register-only, with or without
    the L2 prefetch of upcoming rows) do the same arithmetic in the same order: bit-identical dX and
    dW, with and without dS and dY, for row counts below, at and above the grid size."""
    import hilda_kernel_b200._lib as L
    lib = L.lib()
    assert lib.hilda_norm_bwd_set_path(-1) == 1
    g = gen(17)
    for n_rows, n_cols, dtype in [(5, 4096, torch.float32), (4096, 4096, torch.float32), (1000, 4096, torch.bfloat16),
                                  (9000, 2048, torch.bfloat16), (300, 8192, torch.float16), (777, 1024, torch.float32)]:
        x = torch.randn(n_rows, n_cols, generator=g).to(dtype).to(DEV)
        dy = torch.randn(n_rows, n_cols, generator=g).to(dtype).to(DEV)
        ds = torch.randn(n_rows, n_cols, generator=g).to(dtype).to(DEV)
        w = (1 + 0.1 * torch.randn(n_cols, generator=g)).to(dtype).to(DEV)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
        ws = torch.empty(lib.hilda_norm_bwd_workspace_bytes(n_rows, n_cols, L.dt(x)) // 4, dtype=torch.float32, device=DEV)
        for use_dy, use_ds in ((True, False), (True, True), (False, True)):
            res = []
            for path in (1, 0, 4, 3):
                lib.hilda_norm_bwd_set_path(path)
                try:
                    dx, dw = torch.empty_like(x), torch.empty_like(w)
                    rc = lib.hilda_norm_bwd(dy.data_ptr() if use_dy else None, ds.data_ptr() if use_ds else None,
                                            x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                                            ws.data_ptr(), n_rows, n_cols, L.dt(x), L.dt(w), L.stream(x.device))
                    assert rc == 0
                    torch.cuda.synchronize()
                    res.append((dx, dw))
                finally:
                    lib.hilda_norm_bwd_set_path(1)
            # the explicitly chosen kernels share one thread plan and one grid: bit-identical dX and dW
            for other in res[2:]:
                assert torch.equal(res[1][0], other[0]), (n_rows, n_cols, dtype, use_dy, use_ds)
                assert torch.equal(res[1][1], other[1]), (n_rows, n_cols, dtype, use_dy, use_ds)
            if dtype == torch.float32:
                assert torch.equal(res[0][0], res[1][0]), (n_rows, n_cols, dtype, use_dy, use_ds)
                assert torch.equal(res[0][1], res[1][1]), (n_rows, n_cols, dtype, use_dy, use_ds)
            else:
                # the automatic choice may be the lean 16-bit kernel: its own thread plan (the row sum is
                # grouped differently) and a smaller grid (so are dW's partial sums)
                torch.testing.assert_close(res[0][0].float(), res[1][0].float(), rtol=1.6e-2, atol=1e-2)
                torch.testing.assert_close(res[0][1].float(), res[1][1].float(), rtol=1.6e-2, atol=1e-2 * n_rows ** 0.5)
            assert bool(torch.isfinite(res[0][1].float()).all())


# ------------------------------------------------------------------ FusedAddRMSNorm
@pytest.mark.parametrize("shape", [(2, 64, 4096), (3, 7, 5120), (1, 9, 8192), (5, 100), (300, 1024)])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("use_ds", [True, False])
def test_fused_add_rms_norm(shape, dtype, use_ds):
    hk = ops()
    g = gen(3)
    x = torch.randn(*shape, generator=g).to(dtype)
    r = torch.randn(*shape, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(shape[-1], generator=g)).to(dtype)
    dy = torch.randn(*shape, generator=g).to(dtype)
    ds = torch.randn(*shape, generator=g).to(dtype)
    # forward oracle in the op's dtype (S must be rounded to dtype before the statistics)
    y_ref, s_ref = R.fused_add_rms_norm(x, r, w, 1e-6)
    # backward oracle in fp32, starting from the rounded S
    s32 = s_ref.float().clone().requires_grad_(True)
    w32 = w.float().clone().requires_grad_(True)
    rms = torch.sqrt(torch.mean(s32 ** 2, dim=-1, keepdim=True) + 1e-6)
    y32 = (s32 / rms) * w32
    y32.backward(dy.float())
    dx_ref = s32.grad + (ds.float() if use_ds else 0)

    xd, rd, wd = (t.to(DEV).requires_grad_(True) for t in (x, r, w))
    y, s = hk.hilda_fused_add_rms_norm(xd, rd, wd, 1e-6)
    assert torch.equal(s.cpu(), s_ref), "S = X + R must be bit-exact"
    assert_close(y, y_ref, dtype, what="y")
    if use_ds:
        torch.autograd.backward([y, s], [dy.to(DEV), ds.to(DEV)])
    else:
        y.backward(dy.to(DEV))
    assert_close(xd.grad, dx_ref, dtype, what="dx")
    assert torch.equal(xd.grad, rd.grad)
    rows = x.numel() // shape[-1]
    if dtype == torch.float32:
        assert_close(wd.grad, w32.grad, dtype, scale=float(rows) ** 0.5 * 3, what="dw")
    else:
        torch.testing.assert_close(wd.grad.float().cpu(), w32.grad, rtol=1.6e-2, atol=1e-2 * max(1.0, rows ** 0.5))


def test_fused_add_rms_norm_golden_and_module(golden):
    hk = ops()
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        c = golden[f"fused_add_rms_norm_{tag}"]
        x, r, w = (c[k].to(DEV).requires_grad_(True) for k in ("x", "r", "w"))
        y, s = hk.hilda_fused_add_rms_norm(x, r, w, c["eps"])
        torch.autograd.backward([y, s], [c["dy"].to(DEV), c["ds"].to(DEV)])
        assert torch.equal(s.cpu(), c["s"])
        assert_close(y, c["y"], dtype, what="y")
        assert_close(x.grad, c["dx"], dtype, what="dx")
        assert_close(r.grad, c["dr"], dtype, what="dr")
        assert_close(w.grad, c["dw"], dtype, scale=10.0, what="dw")
    m = hk.FusedAddRMSNorm(256).to(DEV)
    y, s = m(torch.randn(4, 256, device=DEV), torch.randn(4, 256, device=DEV))
    # only S flows back: dY arrives as None
    s.sum().backward()
    assert set(m.state_dict()) == {"weight"}


# ------------------------------------------------------------------ RoPE
def _rope_inputs(bsz, seq, nq, nk, hd, dtype, cs_dtype, seed=4, base=10000.0, layout="bhsd"):
    g = gen(seed)
    if layout == "bhsd":
        q = torch.randn(bsz, nq, seq, hd, generator=g).to(dtype)
        k = torch.randn(bsz, nk, seq, hd, generator=g).to(dtype)
    else:  # memory order (B, S, H, D), handed to the op as a transposed view
        q = torch.randn(bsz, seq, nq, hd, generator=g).to(dtype).transpose(1, 2)
        k = torch.randn(bsz, seq, nk, hd, generator=g).to(dtype).transpose(1, 2)
    cos, sin = R.rope_tables(seq, hd, base=base, dtype=cs_dtype)
    return q, k, cos, sin


@pytest.mark.parametrize("layout", ["bhsd", "bshd"])
@pytest.mark.parametrize("dtype,cs_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                            (torch.bfloat16, torch.float32), (torch.float16, torch.float16)])
@pytest.mark.parametrize("dims", [(2, 64, 8, 2, 128), (1, 33, 3, 1, 64), (2, 17, 4, 4, 20), (1, 700, 2, 1, 128)])
def test_rope_fwd_bwd(layout, dtype, cs_dtype, dims):
    hk = ops()
    bsz, seq, nq, nk, hd = dims
    q, k, cos, sin = _rope_inputs(bsz, seq, nq, nk, hd, dtype, cs_dtype, layout=layout)
    g = gen(5)
    dq = torch.randn(q.shape, generator=g).to(dtype)
    dk = torch.randn(k.shape, generator=g).to(dtype)
    qr, kr = q.clone().requires_grad_(True), k.clone().requires_grad_(True)
    q_ref, k_ref = R.rope(qr, kr, cos, sin)
    torch.autograd.backward([q_ref, k_ref], [dq.to(q_ref.dtype), dk.to(k_ref.dtype)])

    qd = q.to(DEV).requires_grad_(True) if layout == "bhsd" else \
        q.transpose(1, 2).contiguous().to(DEV).transpose(1, 2).requires_grad_(True)
    kd = k.to(DEV).requires_grad_(True) if layout == "bhsd" else \
        k.transpose(1, 2).contiguous().to(DEV).transpose(1, 2).requires_grad_(True)
    assert qd.stride() == q.stride()
    qo, ko = hk.hilda_rope(qd, kd, cos.to(DEV), sin.to(DEV))
    assert qo.dtype == dtype and qo.shape == q.shape
    torch.autograd.backward([qo, ko], [dq.to(DEV), dk.to(DEV)])
    if dtype == cs_dtype:
        # same arithmetic, same rounding points as the PyTorch reference: bit-exact
        assert torch.equal(qo.cpu(), q_ref.detach()) and torch.equal(ko.cpu(), k_ref.detach())
    assert_close(qo, q_ref.to(dtype), dtype, what="q")
    assert_close(ko, k_ref.to(dtype), dtype, what="k")
    assert_close(qd.grad, qr.grad, dtype, what="dq")
    assert_close(kd.grad, kr.grad, dtype, what="dk")


def test_rope_known_answer_and_inplace(golden):
    hk = ops()
    from hilda_kernel_b200.kernels.rope import rope_backward, rope_forward
    # backward of all-ones == cat(cos+sin, cos-sin)  (benchmarks/bench_rope.py:132-146)
    bsz, seq, nq, nk, hd = 2, 256, 32, 8, 128
    cos, sin = R.rope_tables(seq, hd)
    dq_o, dk_o = rope_backward(torch.ones(bsz, nq, seq, hd, device=DEV), torch.ones(bsz, nk, seq, hd, device=DEV),
                               cos.to(DEV), sin.to(DEV))
    exp = R.rope_backward_ones(cos, sin)
    assert float((dq_o.cpu() - exp.expand_as(dq_o)).abs().max()) < 1e-4
    assert float((dk_o.cpu() - exp.expand_as(dk_o)).abs().max()) < 1e-4
    # golden, and in place == out of place
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        c = golden[f"rope_{tag}"]
        q, k = c["q"].to(DEV), c["k"].to(DEV)
        qo, ko, _, _ = rope_forward(q, k, c["cos"].to(DEV), c["sin"].to(DEV))
        assert torch.equal(qo.cpu(), c["q_out"]) and torch.equal(ko.cpu(), c["k_out"])
        q2, k2 = q.clone(), k.clone()
        qi, ki, _, _ = rope_forward(q2, k2, c["cos"].to(DEV), c["sin"].to(DEV), inplace=True)
        assert qi.data_ptr() == q2.data_ptr() and torch.equal(qi, qo) and torch.equal(ki, ko)
        dqo, dko = rope_backward(c["dq"].to(DEV), c["dk"].to(DEV), c["cos"].to(DEV), c["sin"].to(DEV))
        assert_close(dqo, c["dq_in"], dtype, what="dq")
        assert_close(dko, c["dk_in"], dtype, what="dk")
    # autograd through the in-place form on non-leaf tensors, zero-stride upstream grads (sum())
    q, k, cos, sin = _rope_inputs(2, 32, 4, 2, 64, torch.float32, torch.float32)
    ql, kl = q.to(DEV).requires_grad_(True), k.to(DEV).requires_grad_(True)
    qo, ko = hk.hilda_rope(ql * 1.0, kl * 1.0, cos.to(DEV), sin.to(DEV), inplace=True)
    (qo.sum() + ko.sum()).backward()
    qr, kr = q.clone().requires_grad_(True), k.clone().requires_grad_(True)
    a, b = R.rope(qr, kr, cos, sin)
    (a.sum() + b.sum()).backward()
    assert_close(ql.grad, qr.grad, what="dq")
    # per-batch tables and the RotaryEmbedding module
    rot = hk.RotaryEmbedding(64, max_position_embeddings=128, base=500000).to(DEV)
    c2, s2 = rot(None, seq_len=32)
    assert c2.shape == (1, 32, 32) and set(rot.state_dict()) == {"inv_freq", "cos_cached", "sin_cached"}
    cb, sb = c2.expand(2, -1, -1).contiguous(), s2.expand(2, -1, -1).contiguous()
    o1, _ = rot.apply_rotary(q.to(DEV), k.to(DEV), c2, s2)
    o2, _ = hk.hilda_rope(q.to(DEV), k.to(DEV), cb, sb)
    assert torch.equal(o1, o2)


# ------------------------------------------------------------------ SwiGLU
@pytest.mark.parametrize("shape", [(64, 11008), (33, 14336), (7, 200), (5, 33), (1, 1), (3, 4, 1000), (2049, 4096)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(shape, dtype):
    hk = ops()
    g = gen(6)
    a = torch.randn(*shape, generator=g).to(dtype)
    b = torch.randn(*shape, generator=g).to(dtype)
    dc = torch.randn(*shape, generator=g).to(dtype)
    c_ref = R.swiglu(a, b)
    a32, b32 = a.float().clone().requires_grad_(True), b.float().clone().requires_grad_(True)
    R.swiglu(a32, b32).backward(dc.float())
    ad, bd = a.to(DEV).requires_grad_(True), b.to(DEV).requires_grad_(True)
    c = hk.hilda_swiglu(ad, bd)
    assert c.dtype == dtype
    assert_close(c, c_ref, dtype, what="c")
    c.backward(dc.to(DEV))
    assert_close(ad.grad, a32.grad, dtype, what="da")
    assert_close(bd.grad, b32.grad, dtype, what="db")


def test_swiglu_golden_and_inplace_backward(golden):
    from hilda_kernel_b200.kernels.swiglu import swiglu_backward, swiglu_forward
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        c = golden[f"swiglu_{tag}"]
        a, b = c["a"].to(DEV), c["b"].to(DEV)
        out = swiglu_forward(a, b)
        assert_close(out, c["c"], dtype, what="c")
        da, db = swiglu_backward(a, b, c["dc"].to(DEV))
        # the reference overwrites the saved inputs (kernels/swiglu.py:104-105, :141)
        assert da.data_ptr() == a.data_ptr() and db.data_ptr() == b.data_ptr()
        assert_close(da, c["da"], dtype, what="da")
        assert_close(db, c["db"], dtype, what="db")


# ------------------------------------------------------------------ GeGLU
@pytest.mark.parametrize("shape", [(64, 11008), (33, 14336), (7, 200), (5, 33), (3, 4, 1000), (512, 4096)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_geglu(shape, dtype, golden):
    hk = ops()
    g = gen(12)
    a = torch.randn(*shape, generator=g).to(dtype)
    b = torch.randn(*shape, generator=g).to(dtype)
    dc = torch.randn(*shape, generator=g).to(dtype)
    c_ref = R.geglu(a, b)
    a32, b32 = a.float().clone().requires_grad_(True), b.float().clone().requires_grad_(True)
    R.geglu(a32, b32).backward(dc.float())
    ad, bd = a.to(DEV).requires_grad_(True), b.to(DEV).requires_grad_(True)
    c = hk.hilda_geglu(ad, bd)
    assert c.dtype == dtype
    assert_close(c, c_ref, dtype, what="c")
    c.backward(dc.to(DEV))
    assert_close(ad.grad, a32.grad, dtype, what="da")
    assert_close(bd.grad, b32.grad, dtype, what="db")
    if shape == (7, 200) and dtype != torch.float16:
        k = golden["geglu_f32" if dtype == torch.float32 else "geglu_bf16"]
        out = hk.GeGLU()(k["a"].to(DEV), k["b"].to(DEV))
        assert_close(out, k["c"], dtype, what="golden c")


# ------------------------------------------------------------------ CrossEntropy
def _ce_inputs(n, v, dtype, ignore_frac=0.1, seed=7):
    g = gen(seed)
    logits = (2.0 * torch.randn(n, v, generator=g)).to(dtype)
    targets = torch.randint(0, v, (n,), generator=g)
    n_ign = int(round(ignore_frac * n))
    if n_ign:
        targets[torch.randperm(n, generator=g)[:n_ign]] = -100
    return logits, targets


@pytest.mark.parametrize("nv", [(64, 32000), (32, 128256), (64, 4096), (16, 151936), (40, 1000), (9, 50257), (3, 7),
                                (5, 200000), (4, 300000),
                                # one vocabulary per remaining (cluster, register + shared-memory vectors) plan
                                (6, 20000), (6, 28000), (6, 36000), (6, 40000), (6, 50304), (4, 65536), (4, 73728), (4, 81920),
                                (4, 102400)])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_cross_entropy(nv, dtype, reduction):
    hk = ops()
    n, v = nv
    if reduction != "mean" and v > 60000:
        pytest.skip("large-vocabulary cases run with mean only")
    logits, targets = _ce_inputs(n, v, dtype)
    lr = logits.float().clone().requires_grad_(True)
    loss_ref = R.cross_entropy_clamped(lr, targets, -100, reduction)
    g = gen(8)
    up = torch.randn(loss_ref.shape, generator=g) if reduction == "none" else None
    loss_ref.backward(up)
    ld = logits.to(DEV).requires_grad_(True)
    loss = hk.hilda_cross_entropy(ld, targets.to(DEV), -100, reduction)
    assert loss.dtype == torch.float32
    if reduction == "none":
        assert_close(loss, loss_ref.detach(), torch.float32, what="loss rows")
        loss.backward(up.to(DEV))
    else:
        assert_loss_close(loss, loss_ref)
        loss.backward()
    assert ld.grad.dtype == dtype
    assert_close(ld.grad, lr.grad, dtype, what="dlogits", normalize=True)
    ign = targets == -100
    if ign.any():
        assert float(ld.grad[ign.to(DEV)].abs().max()) == 0.0  # ignored rows: exactly zero gradient
    # inference path (no grad): same loss
    loss_inf = hk.hilda_cross_entropy(logits.to(DEV), targets.to(DEV), -100, reduction)
    if reduction == "none":
        assert_close(loss_inf, loss_ref.detach(), torch.float32, what="loss rows (inference)")
    else:
        assert_loss_close(loss_inf, loss_ref)


def test_cross_entropy_golden_and_edges(golden):
    hk = ops()
    c = golden["cross_entropy_f32"]
    ld = c["logits"].to(DEV).requires_grad_(True)
    loss = hk.CrossEntropyLoss()(ld, c["targets"].to(DEV))
    loss.backward()
    assert_loss_close(loss, c["loss"])
    assert float((ld.grad.cpu() - c["dlogits"]).abs().max()) < 1e-4  # bench_cross_entropy.py:108-110
    # non-unit upstream gradient -> one scale pass
    ld2 = c["logits"].to(DEV).requires_grad_(True)
    (hk.hilda_cross_entropy(ld2, c["targets"].to(DEV)) * 3.0).backward()
    assert_close(ld2.grad, 3.0 * c["dlogits"], torch.float32, what="scaled dlogits")
    # every row ignored: loss 0 (clamp), zero grads
    t = torch.full((24,), -100, dtype=torch.long, device=DEV)
    ld3 = c["logits"].to(DEV).requires_grad_(True)
    loss3 = hk.hilda_cross_entropy(ld3, t)
    loss3.backward()
    assert float(loss3) == 0.0 and float(ld3.grad.abs().max()) == 0.0
    # ignore_index = -1 means nothing is ignored (kernels/cross_entropy.py:219-225)
    tt = c["targets"].clamp_min(0)
    l4 = hk.hilda_cross_entropy(c["logits"].to(DEV), tt.to(DEV), -1, "mean")
    assert_loss_close(l4, R.cross_entropy(c["logits"], tt, ignore_index=-1))
    # every cluster/vector plan of the row engine gives the same answer
    import hilda_kernel_b200._lib as L
    logits, targets = _ce_inputs(8, 16384, torch.bfloat16)
    lr = logits.float().clone().requires_grad_(True)
    R.cross_entropy_clamped(lr, targets).backward()
    try:
        for nv_, cl, ns_ in [(8, 1, 0), (8, 8, 0), (10, 8, 0), (8, 1, 4), (8, 1, 6), (8, 2, 6), (8, 4, 6), (8, 8, 6), (8, 1, 8), (10, 1, 9), (8, 2, 4), (8, 2, 8),
                             (10, 2, 9), (8, 4, 4), (8, 4, 8), (10, 4, 9), (8, 8, 4), (8, 8, 8), (10, 8, 9), (51210, 8, 9)]:
            L.lib().hilda_row_engine_force(nv_, cl, ns_)
            ld = logits.to(DEV).requires_grad_(True)
            hk.hilda_cross_entropy(ld, targets.to(DEV)).backward()
            assert_close(ld.grad, lr.grad, torch.bfloat16, what=f"dlogits plan {(nv_, cl, ns_)}", normalize=True)
    finally:
        L.lib().hilda_row_engine_force(0, 0, 0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("v", [50257, 1003, 32001])
def test_cross_entropy_rows_off_the_16_byte_grid(dtype, v):
    """A vocabulary that is not a multiple of the vector width: rows start and end between 16-byte
    boundaries (a different offset in every row). The targets sit on the first and last elements of the
    rows, which the kernel holds as scalars beside the aligned vectors."""
    hk = ops()
    n = 24
    g = gen(31)
    logits = (2.0 * torch.randn(n, v, generator=g)).to(dtype)
    edge = list(range(8)) + [v - 1 - i for i in range(8)]
    targets = torch.tensor([edge[i % len(edge)] for i in range(n)])
    targets[5] = -100
    lr = logits.float().clone().requires_grad_(True)
    loss_ref = R.cross_entropy_clamped(lr, targets, -100, "mean")
    loss_ref.backward()
    ld = logits.to(DEV).requires_grad_(True)
    loss = hk.hilda_cross_entropy(ld, targets.to(DEV), -100, "mean")
    loss.backward()
    assert_loss_close(loss, loss_ref)
    assert_close(ld.grad, lr.grad, dtype, what="dlogits", normalize=True)
    assert float(ld.grad[5].abs().max()) == 0.0
    # the gradient at the target column is softmax - 1: negative, and the largest magnitude of its row
    rows = torch.arange(n)[targets != -100]
    at_t = ld.grad.float().cpu()[rows, targets[rows]]
    assert bool((at_t < 0).all())


# ------------------------------------------------------------------ GRPO
def _grpo_inputs(B, L, V, dtype, seed=9, masked=True):
    g = gen(seed)
    logits = (2.0 * torch.randn(B, L + 1, V, generator=g)).to(dtype)
    ids = torch.randint(0, V, (B, L), generator=g)
    adv = torch.randn(B, generator=g)
    cur = R.selective_log_softmax(logits.float(), ids)
    old = cur + 0.3 * torch.randn(B, L, generator=g)
    ref = cur + 0.1 * torch.randn(B, L, generator=g)
    mask = None
    if masked:
        lens = torch.randint(max(1, L // 4), L + 1, (B,), generator=g)
        mask = (torch.arange(L)[None, :] < lens[:, None]).to(torch.int32)
    return logits, ids, adv, old, ref, mask


@pytest.mark.parametrize("dims", [(4, 32, 32000), (2, 16, 128256), (2, 9, 151936), (3, 12, 300), (2, 5, 1001)])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("beta", [0.0, 0.1])
@pytest.mark.parametrize("masked", [True, False])
def test_grpo(dims, dtype, beta, masked):
    hk = ops()
    B, L, V = dims
    logits, ids, adv, old, ref, mask = _grpo_inputs(B, L, V, dtype, masked=masked)
    lr = logits.float().clone().requires_grad_(True)
    loss_ref = R.grpo_loss(lr, ids, adv, old, ref if beta else None, mask, beta=beta)
    loss_ref.backward()
    kl_ref, clip_ref = R.grpo_aux(logits.float(), ids, adv, old, ref, mask, beta=beta)
    ld = logits.to(DEV).requires_grad_(True)
    md = mask.to(DEV) if mask is not None else None
    loss, kl, clip = hk.hilda_grpo_loss(ld, ids.to(DEV), adv.to(DEV), old.to(DEV), ref.to(DEV) if beta else None, md,
                                        1.0, beta, 0.2, 0.2)
    assert loss.dtype == torch.float32
    assert_loss_close(loss, loss_ref)
    assert abs(float(clip) - float(clip_ref)) < 1e-6 + 1.0 / (B * L)  # a ratio within rounding of a clip edge may flip
    if beta:
        assert_loss_close(kl, kl_ref, "kl_mean")
    else:
        assert kl is None
    loss.backward()
    assert ld.grad.dtype == dtype and ld.grad.shape == logits.shape
    assert_close(ld.grad, lr.grad, dtype, what="dlogits", normalize=True)
    assert float(ld.grad[:, -1, :].abs().max()) == 0.0  # last position never contributes
    if mask is not None:
        dead = (mask == 0).to(DEV)
        assert float(ld.grad[:, :-1, :][dead].abs().max()) == 0.0


def test_grpo_golden_variants(golden):
    hk = ops()
    for tag in ("beta0", "beta01"):
        c = golden[f"grpo_{tag}"]
        ld = c["logits"].to(DEV).requires_grad_(True)
        loss, kl, clip = hk.GRPOLoss(beta=c["beta"])(ld, c["ids"].to(DEV), c["adv"].to(DEV), c["old"].to(DEV),
                                                     c["ref"].to(DEV) if c["beta"] else None, c["mask"].to(DEV))
        loss.backward()
        assert_loss_close(loss, c["loss"])
        assert float((ld.grad.cpu() - c["dlogits"]).abs().max()) < 1e-4  # bench_grpo.py fp32 threshold
    # old_logp=None => ratio 1; temperature != 1; non-unit upstream gradient
    logits, ids, adv, old, ref, mask = _grpo_inputs(2, 8, 4096, torch.float32)
    lr = logits.clone().requires_grad_(True)
    (R.grpo_loss(lr, ids, adv, None, ref, mask, temperature=0.7, beta=0.05) * 2.5).backward()
    ld = logits.to(DEV).requires_grad_(True)
    loss, kl, clip = hk.hilda_grpo_loss(ld, ids.to(DEV), adv.to(DEV), None, ref.to(DEV), mask.to(DEV), 0.7, 0.05)
    (loss * 2.5).backward()
    assert_close(ld.grad, lr.grad, torch.float32, what="dlogits", normalize=True)
    assert float(clip) == 0.0
    # selective log-softmax
    lp = hk.fused_selective_log_softmax(logits.to(DEV), ids.to(DEV), 0.7, mask.to(DEV))
    ref_lp = R.selective_log_softmax(logits, ids, 0.7) * mask
    assert_close(lp, ref_lp, torch.float32, what="logp")
    # no-grad forward gives the same scalars
    with torch.no_grad():
        l2, _, _ = hk.hilda_grpo_loss(logits.to(DEV), ids.to(DEV), adv.to(DEV), None, ref.to(DEV), mask.to(DEV), 0.7, 0.05)
    assert_loss_close(l2, loss)


# ------------------------------------------------------------------ row-sharded normalisation
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_sharded_losses_use_global_counts(dtype):
    """Each shard's kernel divides by the count over ALL shards (valid rows for CE, sequences for
    GRPO), so the shards' losses add up to the unsharded loss and their gradients concatenate to
    the unsharded gradient: what parallel.sharded_cross_entropy / sharded_grpo_loss rely on."""
    from hilda_kernel_b200.kernels.cross_entropy import cross_entropy_forward
    from hilda_kernel_b200.kernels.grpo_loss import grpo_loss_forward
    g = gen(21)
    n, v = 48, 5000
    logits = (2.0 * torch.randn(n, v, generator=g)).to(dtype)
    targets = torch.randint(0, v, (n,), generator=g)
    targets[torch.randperm(n, generator=g)[:9]] = -100
    lr = logits.float().clone().requires_grad_(True)
    ref = R.cross_entropy(lr, targets)
    ref.backward()
    ld, td = logits.to(DEV), targets.to(DEV)
    n_valid = (td != -100).sum(dtype=torch.int32).reshape(1)
    cuts = [0, 20, 48]  # unequal shards, different numbers of ignored rows
    total, grads = 0.0, []
    for a, b in zip(cuts[:-1], cuts[1:]):
        loss, grad, nv_local = cross_entropy_forward(ld[a:b], td[a:b], -100, 'mean', needs_grad=True,
                                                     n_valid_global=n_valid)
        assert int(nv_local) == int((targets[a:b] != -100).sum())
        total += float(loss)
        grads.append(grad)
    assert abs(total - float(ref)) <= 1e-4 * abs(float(ref))
    assert_close(torch.cat(grads), lr.grad, dtype, what="sharded CE dlogits", normalize=True)

    B, L, V = 4, 12, 3000
    logits, ids, adv, old, refp, mask = _grpo_inputs(B, L, V, dtype, seed=22)
    lr = logits.float().clone().requires_grad_(True)
    ref = R.grpo_loss(lr, ids, adv, old, refp, mask, beta=0.1)
    ref.backward()
    kl_ref, clip_ref = R.grpo_aux(logits.float(), ids, adv, old, refp, mask, beta=0.1)
    total, kl_num, clip_num, msum, grads = 0.0, 0.0, 0.0, 0.0, []
    for a, b in ((0, 2), (2, 4)):
        d = lambda t: t[a:b].to(DEV)
        loss, kl, clip, _, m, grad = grpo_loss_forward(d(logits), d(ids), d(adv), d(old), d(refp), d(mask), 1.0, 0.1,
                                                       0.2, 0.2, needs_grad=True, batch_total=B)
        ms = float(m.sum())
        total += float(loss); kl_num += float(kl) * ms; clip_num += float(clip) * ms; msum += ms
        grads.append(grad)
    assert abs(total - float(ref)) <= 1e-4 * abs(float(ref))
    assert abs(kl_num / msum - float(kl_ref)) <= 1e-4 * abs(float(kl_ref))
    assert abs(clip_num / msum - float(clip_ref)) < 1e-6 + 1.0 / (B * L)
    assert_close(torch.cat(grads), lr.grad, dtype, what="sharded GRPO dlogits", normalize=True)
