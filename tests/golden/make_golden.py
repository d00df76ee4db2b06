"""Generate tests/golden/golden.pt from hilda-kernel's OWN PyTorch reference functions.

Run once, in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/hilda-kernel

It imports the reference benchmark modules (``triton-kernels/benchmarks/bench_*.py``; importing them
needs triton but no GPU) and calls the reference implementations they define
(``pytorch_rms_norm``, ``pytorch_fused_add_rms_norm``, ``pytorch_rope``, ``pytorch_swiglu``, ``pytorch_geglu``,
``pytorch_linear_ce``, ``pytorch_grpo_loss``, ``pytorch_jsd``, ``pytorch_linear_jsd``, ``pytorch_attn_res``) plus
``torch.nn.functional.cross_entropy`` exactly as ``bench_cross_entropy.py:77-79`` calls it and
``torch.nn.functional.kl_div`` as ``bench_kl_div.py:45`` does, on small seeded CPU inputs, including their autograd
gradients. Inputs and outputs are stored together so the tests need neither the reference nor
this script at run time.
"""
import contextlib
import io
import os
import sys

import torch


def _import_reference(root):
    tk = os.path.join(root, "triton-kernels")
    sys.path.insert(0, os.path.join(tk, "benchmarks"))
    sys.path.insert(0, tk)
    mods = {}
    with contextlib.redirect_stdout(io.StringIO()):
        for name in ("bench_rms_norm", "bench_fused_add_rms_norm", "bench_rope", "bench_swiglu", "bench_geglu",
                     "bench_fused_linear_ce", "bench_grpo", "bench_jsd", "bench_fused_linear_jsd", "bench_attn_res"):
            mods[name] = __import__(name)
    return mods


def _g(seed):
    return torch.Generator().manual_seed(seed)


def main(root):
    m = _import_reference(root)
    out = {}

    # ---- RMSNorm (fp32 and bf16) with autograd gradients
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        g = _g(0)
        x = torch.randn(6, 256, generator=g).to(dtype)
        w = (1 + 0.1 * torch.randn(256, generator=g)).to(dtype)
        dy = torch.randn(6, 256, generator=g).to(dtype)
        xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        y = m["bench_rms_norm"].pytorch_rms_norm(xr, wr, 1e-6)
        y.backward(dy.to(y.dtype))
        out[f"rms_norm_{tag}"] = dict(x=x, w=w, dy=dy, eps=1e-6, y=y.detach(), dx=xr.grad, dw=wr.grad)

    # ---- FusedAddRMSNorm
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        g = _g(1)
        x = torch.randn(5, 384, generator=g).to(dtype)
        r = torch.randn(5, 384, generator=g).to(dtype)
        w = (1 + 0.1 * torch.randn(384, generator=g)).to(dtype)
        dy = torch.randn(5, 384, generator=g).to(dtype)
        ds = torch.randn(5, 384, generator=g).to(dtype)
        xr, rr, wr = (t.clone().requires_grad_(True) for t in (x, r, w))
        y, s = m["bench_fused_add_rms_norm"].pytorch_fused_add_rms_norm(xr, rr, wr, 1e-6)
        torch.autograd.backward([y, s], [dy, ds])
        out[f"fused_add_rms_norm_{tag}"] = dict(x=x, r=r, w=w, dy=dy, ds=ds, eps=1e-6, y=y.detach(), s=s.detach(),
                                                dx=xr.grad, dr=rr.grad, dw=wr.grad)

    # ---- RoPE (fp32 tables; and bf16 q/k with bf16 tables, the bench convention bench_rope.py:79-80)
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        g = _g(2)
        bsz, seq, nq, nk, hd = 2, 16, 4, 2, 32
        q = torch.randn(bsz, nq, seq, hd, generator=g).to(dtype)
        k = torch.randn(bsz, nk, seq, hd, generator=g).to(dtype)
        inv_freq = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
        freqs = torch.outer(torch.arange(seq, dtype=torch.float32), inv_freq)
        cos, sin = freqs.cos()[None].to(dtype), freqs.sin()[None].to(dtype)
        dq = torch.randn(bsz, nq, seq, hd, generator=g).to(dtype)
        dk = torch.randn(bsz, nk, seq, hd, generator=g).to(dtype)
        qr, kr = q.clone().requires_grad_(True), k.clone().requires_grad_(True)
        qo, ko = m["bench_rope"].pytorch_rope(qr, kr, cos, sin)
        torch.autograd.backward([qo, ko], [dq, dk])
        out[f"rope_{tag}"] = dict(q=q, k=k, cos=cos, sin=sin, dq=dq, dk=dk, q_out=qo.detach(), k_out=ko.detach(),
                                  dq_in=qr.grad, dk_in=kr.grad)

    # ---- SwiGLU
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        g = _g(3)
        a = torch.randn(7, 200, generator=g).to(dtype)
        b = torch.randn(7, 200, generator=g).to(dtype)
        dc = torch.randn(7, 200, generator=g).to(dtype)
        ar, br = a.clone().requires_grad_(True), b.clone().requires_grad_(True)
        c = m["bench_swiglu"].pytorch_swiglu(ar, br)
        c.backward(dc)
        out[f"swiglu_{tag}"] = dict(a=a, b=b, dc=dc, c=c.detach(), da=ar.grad, db=br.grad)

    # ---- GeGLU
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        g = _g(7)
        a = torch.randn(7, 200, generator=g).to(dtype)
        b = torch.randn(7, 200, generator=g).to(dtype)
        dc = torch.randn(7, 200, generator=g).to(dtype)
        ar, br = a.clone().requires_grad_(True), b.clone().requires_grad_(True)
        c = m["bench_geglu"].pytorch_geglu(ar, br)
        c.backward(dc)
        out[f"geglu_{tag}"] = dict(a=a, b=b, dc=dc, c=c.detach(), da=ar.grad, db=br.grad)

    # ---- CrossEntropy: F.cross_entropy(ignore_index=-100, reduction='mean') as bench_cross_entropy.py:77-79
    g = _g(4)
    n, v = 24, 1000
    logits = 2.0 * torch.randn(n, v, generator=g)
    targets = torch.randint(0, v, (n,), generator=g)
    targets[torch.randperm(n, generator=g)[:3]] = -100
    lr = logits.clone().requires_grad_(True)
    loss = torch.nn.functional.cross_entropy(lr, targets, ignore_index=-100, reduction="mean")
    loss.backward()
    out["cross_entropy_f32"] = dict(logits=logits, targets=targets, loss=loss.detach(), dlogits=lr.grad)

    # ---- FusedLinearCE: pytorch_linear_ce takes no ignore arg (bench_fused_linear_ce.py:36-38)
    g = _g(5)
    bt, h, v = 48, 64, 520
    hidden = torch.randn(bt, h, generator=g)
    weight = 0.02 * torch.randn(v, h, generator=g)
    targets = torch.randint(0, v, (bt,), generator=g)
    hr, wr = hidden.clone().requires_grad_(True), weight.clone().requires_grad_(True)
    loss = m["bench_fused_linear_ce"].pytorch_linear_ce(hr, wr, targets)
    loss.backward()
    out["linear_ce_f32"] = dict(hidden=hidden, weight=weight, targets=targets, loss=loss.detach(), dh=hr.grad,
                                dw=wr.grad)

    # ---- GRPO: pytorch_grpo_loss on fp32 logits (the bench passes logits.float(), bench_grpo.py:80)
    for tag, beta in (("beta0", 0.0), ("beta01", 0.1)):
        g = _g(6)
        B, L, V = 3, 12, 300
        logits = 2.0 * torch.randn(B, L + 1, V, generator=g)
        ids = torch.randint(0, V, (B, L), generator=g)
        adv = torch.randn(B, generator=g)
        with torch.no_grad():
            cur = (logits[:, :-1]).log_softmax(-1).gather(-1, ids.unsqueeze(-1)).squeeze(-1)
        old = cur + 0.3 * torch.randn(B, L, generator=g)  # wide enough that some ratios clip
        ref = cur + 0.1 * torch.randn(B, L, generator=g)
        mask = torch.ones(B, L, dtype=torch.int32)
        mask[0, -4:] = 0
        mask[2, -7:] = 0
        lr = logits.clone().requires_grad_(True)
        loss = m["bench_grpo"].pytorch_grpo_loss(lr, ids, adv, old, ref if beta else None, mask, beta=beta)
        loss.backward()
        out[f"grpo_{tag}"] = dict(logits=logits, ids=ids, adv=adv, old=old, ref=ref, mask=mask, beta=beta,
                                  loss=loss.detach(), dlogits=lr.grad)

    # ---- KLDiv: F.kl_div(y_pred, y_true, reduction='batchmean') as bench_kl_div.py:42-45, :62-67
    g = _g(8)
    n, v = 10, 600
    y_pred = torch.randn(n, v, generator=g).log_softmax(-1)
    y_true = torch.randn(n, v, generator=g).softmax(-1)
    yr = y_pred.clone().requires_grad_(True)
    loss = torch.nn.functional.kl_div(yr, y_true, reduction="batchmean")
    loss.backward()
    out["kl_div_f32"] = dict(y_pred=y_pred, y_true=y_true, loss=loss.detach(), dy_pred=yr.grad)

    # ---- JSD: pytorch_jsd at beta 0.5 / 0 / 1 (bench_jsd.py:30-44, :51-58)
    for tag, beta in (("b05", 0.5), ("b0", 0.0), ("b1", 1.0)):
        g = _g(9)
        n, v = 9, 700
        X = torch.randn(n, v, generator=g).log_softmax(-1)
        Y = torch.randn(n, v, generator=g).log_softmax(-1)
        xr = X.clone().requires_grad_(True)
        loss = m["bench_jsd"].pytorch_jsd(xr, Y, beta)
        loss.backward()
        out[f"jsd_{tag}"] = dict(X=X, Y=Y, beta=beta, loss=loss.detach(), dX=xr.grad)

    # ---- FusedLinearJSD: pytorch_linear_jsd on fp32 inputs (bench_fused_linear_jsd.py:31-43, :83-88)
    g = _g(10)
    bt, h, v = 40, 64, 520
    s_in = torch.randn(bt, h, generator=g)
    s_w = 0.05 * torch.randn(v, h, generator=g)
    t_in = torch.randn(bt, h, generator=g)
    t_w = 0.05 * torch.randn(v, h, generator=g)
    sr, wr = s_in.clone().requires_grad_(True), s_w.clone().requires_grad_(True)
    loss = m["bench_fused_linear_jsd"].pytorch_linear_jsd(sr, wr, t_in, t_w, beta=0.5, temperature=2.0)
    loss.backward()
    out["linear_jsd_f32"] = dict(s_in=s_in, s_w=s_w, t_in=t_in, t_w=t_w, beta=0.5, temperature=2.0,
                                 loss=loss.detach(), dh=sr.grad, dw=wr.grad)

    # ---- AttnRes: pytorch_attn_res (bench_attn_res.py:33-51), fp32 and bf16, with autograd gradients
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        g = _g(11)
        nb, bsz, t, d = 5, 2, 7, 256
        V = torch.randn(nb, bsz, t, d, generator=g).to(dtype)
        wq = (0.02 * torch.randn(d, generator=g)).to(dtype)
        wn = (1 + 0.1 * torch.randn(d, generator=g)).to(dtype)
        dh = torch.randn(bsz, t, d, generator=g).to(dtype)
        vr, qr, nr = (x.clone().requires_grad_(True) for x in (V, wq, wn))
        h = m["bench_attn_res"].pytorch_attn_res(vr, qr, nr)
        h.backward(dh)
        out[f"attn_res_{tag}"] = dict(V=V, wq=wq, wn=wn, dh=dh, h=h.detach(), dV=vr.grad, dwq=qr.grad, dwn=nr.grad)

    # ---- paged FP8 decode attention: the reference's own torch evaluation (paged_attention_fp8.py:191-221)
    sys.path.insert(0, os.path.join(root, "triton-kernels"))
    from kernels.paged_attention_fp8 import reference_paged_attention_decode
    g = _g(12)
    batch, nh, nkv, bs, nblk = 3, 8, 2, 16, 9
    q = torch.randn(batch, nh, 128, generator=g).bfloat16()
    kc = torch.randn(nblk, bs, nkv, 128, generator=g).to(torch.float8_e4m3fn)
    vc = torch.randn(nblk, bs, nkv, 128, generator=g).to(torch.float8_e4m3fn)
    bt = torch.tensor([[4, 0, 7], [2, 8, 8], [5, 1, 1]], dtype=torch.int32)
    ctx = torch.tensor([37, 16, 5], dtype=torch.int32)
    o = reference_paged_attention_decode(q, kc, vc, bt, ctx, 128 ** -0.5)
    out["paged_attention_fp8"] = dict(q=q, k_cache=kc.view(torch.uint8), v_cache=vc.view(torch.uint8), block_tables=bt,
                                      context_lens=ctx, scale=128 ** -0.5, out=o)

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.pt")
    torch.save(out, dst)
    print("wrote", dst, os.path.getsize(dst), "bytes;", len(out), "cases")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/hilda-kernel")
    main(sys.argv[1])
