#!/usr/bin/env python
"""Comparators for bench.py's per-operator table, timed on the same GPU, same shapes, same method:

  triton : hilda-kernel's own Triton operators, imported as ``kernels.<op>`` from a copy of the
           reference's ``triton-kernels/kernels`` directory under ``baseline/_ref`` (git-ignored;
           put there by ``python bench.py --install-reference <path to the hilda-kernel checkout>``),
           through their public autograd API and stock code path;
  liger  : Liger-Kernel where the reference's bench scripts compare against it, called as they call it;
  eager  : plain PyTorch on the GPU.

This file never imports hilda_kernel_b200: nothing of this repository's kernels is on these paths.
bench.py runs it as a child process and merges what it prints: ONE JSON LINE PER OPERATOR, flushed as
each finishes, so that a time budget cutting the child short still leaves the finished operators.

Method (the same as bench.py's table): forward+backward through the autograd API on several
rotating buffer sets whose footprint exceeds the 126 MB L2, captured once in a CUDA graph and
replayed between two CUDA events; an implementation that cannot be captured (a host synchronisation
inside it) is timed launch by launch with events instead and marked "eager_launches".
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.nn.functional as F

try:  # Liger 0.8 looks at torch.distributed.tensor.DTensor without importing the sub-module itself
    import torch.distributed.tensor  # noqa: F401
except Exception:
    pass

ROOT = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
DEV = "cuda"


def timed(fns, iters=5):
    """(ms per closure, how) for closures that each run one forward+backward."""
    if not isinstance(fns, (list, tuple)):
        fns = [fns]
    for _ in range(2):  # compiles / autotunes; must happen outside any capture
        for f in fns:
            f()
    torch.cuda.synchronize()
    how = "cuda_graph"
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for f in fns:
                f()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for f in fns:
                f()
        run = graph.replay
    except Exception:
        torch.cuda.synchronize()
        how = "eager_launches"

        def run():
            for f in fns:
                f()
    run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # as in bench.py's table: a warm-up and at least 20 ms of timed work, sized by one timed run
    e0.record()
    run()
    e1.record()
    torch.cuda.synchronize()
    iters = int(min(max(iters, 20.0 / max(e0.elapsed_time(e1), 1e-3)), 2000))
    for _ in range(max(1, iters // 4)):
        run()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (iters * len(fns)), how


def measure(out, key, make_fns, iters=5):
    try:
        ms, how = timed(make_fns(), iters)
        out[key + "_us"] = round(ms * 1e3, 1)
        if how != "cuda_graph":
            out[key + "_timing"] = how
    except Exception as e:  # did not compile / API mismatch / out of memory: say which
        out[key + "_us"] = None
        out[key + "_error"] = f"{type(e).__name__}: {str(e).splitlines()[0][:200] if str(e) else ''}"
        torch.cuda.synchronize()
    finally:
        torch.cuda.empty_cache()


def load_reference():
    if not os.path.isdir(os.path.join(REF_DIR, "kernels")):
        return None, "reference Triton kernels not installed (python bench.py --install-reference <checkout>)"
    sys.path.insert(0, REF_DIR)
    try:
        import kernels  # noqa: F401  (the reference package: triton-kernels/kernels)
        return kernels, None
    except Exception as e:
        return None, f"import failed: {type(e).__name__}: {e}"


def rn(g, *s):
    return torch.randn(*s, device=DEV, generator=g)


def grads(outs, ins, gs):
    torch.autograd.grad(outs, ins, gs)


# ------------------------------------------------------------------ the operators
def op_rms_norm(ref, g):
    out = {}
    w = (1 + 0.1 * rn(g, 4096)).requires_grad_(True)
    sets = [(rn(g, 4096, 4096).requires_grad_(True), rn(g, 4096, 4096)) for _ in range(6)]

    def mk(fn):
        return lambda: [(lambda x=x, dy=dy: grads([fn(x, w)], [x, w], [dy])) for x, dy in sets]
    if ref:
        from kernels.rms_norm import hilda_rms_norm
        measure(out, "triton", mk(lambda x, w_: hilda_rms_norm(x, w_, 1e-6)))
    try:
        from liger_kernel.ops.rms_norm import LigerRMSNormFunction
        measure(out, "liger", mk(lambda x, w_: LigerRMSNormFunction.apply(x, w_, 1e-6)))
    except ImportError as e:
        out["liger_error"] = str(e)
    measure(out, "eager", mk(lambda x, w_: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w_))
    return "rms_norm_fp32_fwd+bwd", out


def op_fused_add_rms_norm(ref, g):
    out = {}
    w = (1 + 0.1 * rn(g, 4096)).bfloat16().requires_grad_(True)
    sets = []
    for _ in range(3):
        x, r = rn(g, 16384, 4096).bfloat16().requires_grad_(True), rn(g, 16384, 4096).bfloat16().requires_grad_(True)
        sets.append((x, r, rn(g, 16384, 4096).bfloat16(), rn(g, 16384, 4096).bfloat16()))

    def mk(fn):
        def one(x, r, dy, ds):
            y, s = fn(x, r, w)
            grads([y, s], [x, r, w], [dy, ds])
        return lambda: [(lambda a=a: one(*a)) for a in sets]
    if ref:
        from kernels.fused_add_rms_norm import hilda_fused_add_rms_norm
        measure(out, "triton", mk(lambda x, r, w_: hilda_fused_add_rms_norm(x, r, w_, 1e-6)))
    try:
        from liger_kernel.ops.fused_add_rms_norm import LigerFusedAddRMSNormFunction
        measure(out, "liger", mk(lambda x, r, w_: LigerFusedAddRMSNormFunction.apply(x, r, w_, 1e-6, 0.0, "llama", False)))
    except ImportError as e:
        out["liger_error"] = str(e)

    def eager(x, r, w_):
        s = x + r
        s32 = s.float()
        return (s32 * torch.rsqrt(s32.pow(2).mean(-1, keepdim=True) + 1e-6)).to(s.dtype) * w_, s
    measure(out, "eager", mk(eager))
    return "fused_add_rms_norm_bf16_fwd+bwd", out


def op_rope(ref, g, bhsd=False):
    out = {}
    inv = 1.0 / (500000.0 ** (torch.arange(0, 128, 2, device=DEV).float() / 128))
    fr = torch.outer(torch.arange(4096, device=DEV).float(), inv)
    cos, sin = fr.cos()[None].bfloat16(), fr.sin()[None].bfloat16()
    cos_full, sin_full = torch.cat([cos, cos], -1), torch.cat([sin, sin], -1)
    sets = []
    for _ in range(4):
        if bhsd:  # the reference bench script's own memory order
            q = rn(g, 4, 32, 4096, 128).bfloat16().requires_grad_(True)
            k = rn(g, 4, 8, 4096, 128).bfloat16().requires_grad_(True)
        else:
            q = rn(g, 4, 4096, 32, 128).bfloat16().transpose(1, 2).requires_grad_(True)
            k = rn(g, 4, 4096, 8, 128).bfloat16().transpose(1, 2).requires_grad_(True)
        sets.append((q, k, torch.randn_like(q), torch.randn_like(k)))

    def mk(fn):
        def one(q, k, dq, dk):
            qo, ko = fn(q, k)
            grads([qo, ko], [q, k], [dq.to(qo.dtype), dk.to(ko.dtype)])
        return lambda: [(lambda a=a: one(*a)) for a in sets]
    if ref:
        from kernels.rope import hilda_rope
        measure(out, "triton", mk(lambda q, k: hilda_rope(q, k, cos, sin)))
    try:
        from liger_kernel.ops.rope import LigerRopeFunction
        measure(out, "liger", mk(lambda q, k: LigerRopeFunction.apply(q, k, cos_full, sin_full)))
    except ImportError as e:
        out["liger_error"] = str(e)

    def eager(q, k):
        def rot(x):
            x1, x2 = x[..., :64], x[..., 64:]
            return torch.cat((-x2, x1), dim=-1)
        c, s = cos_full[:, None], sin_full[:, None]
        return q * c + rot(q) * s, k * c + rot(k) * s
    measure(out, "eager", mk(eager))
    return ("rope_bf16_bhsd_fwd+bwd" if bhsd else "rope_bf16_fwd+bwd"), out


def op_rope_bhsd(ref, g):
    return op_rope(ref, g, bhsd=True)


def op_swiglu(ref, g):
    out = {}
    a = rn(g, 16384, 14336).bfloat16().requires_grad_(True)
    b = rn(g, 16384, 14336).bfloat16().requires_grad_(True)
    dc = rn(g, 16384, 14336).bfloat16()

    # The reference's backward writes da, db over the saved a, b (kernels/swiglu.py:141), so their values
    # change from one repetition to the next; the timing does not depend on the values.
    def mk(fn):
        return lambda: [lambda: grads([fn(a, b)], [a, b], [dc])]
    if ref:
        from kernels.swiglu import hilda_swiglu
        measure(out, "triton", mk(hilda_swiglu))
    try:
        from liger_kernel.ops.swiglu import LigerSiLUMulFunction
        measure(out, "liger", mk(LigerSiLUMulFunction.apply))
    except ImportError as e:
        out["liger_error"] = str(e)
    measure(out, "eager", mk(lambda a_, b_: F.silu(a_) * b_))
    return "swiglu_bf16_fwd+bwd", out


def op_geglu(ref, g):
    out = {}
    a = rn(g, 16384, 14336).bfloat16().requires_grad_(True)
    b = rn(g, 16384, 14336).bfloat16().requires_grad_(True)
    dc = rn(g, 16384, 14336).bfloat16()

    def mk(fn):  # as for SwiGLU: the reference's backward overwrites the saved a, b (kernels/geglu.py:146-159)
        return lambda: [lambda: grads([fn(a, b)], [a, b], [dc])]
    if ref:
        from kernels.geglu import hilda_geglu
        measure(out, "triton", mk(hilda_geglu))
    try:
        from liger_kernel.ops.geglu import LigerGELUMulFunction
        measure(out, "liger", mk(LigerGELUMulFunction.apply))
    except ImportError as e:
        out["liger_error"] = str(e)
    measure(out, "eager", mk(lambda a_, b_: F.gelu(a_, approximate="tanh") * b_))
    return "geglu_bf16_fwd+bwd", out


def op_cross_entropy(ref, g):
    out = {}
    n, v = 8192, 128256
    logits = (2 * rn(g, n, v)).bfloat16().requires_grad_(True)
    t = torch.randint(0, v, (n,), device=DEV, generator=g)
    t[torch.randperm(n, device=DEV, generator=g)[: n // 10]] = -100
    one = torch.ones((), device=DEV)

    def mk(fn):
        return lambda: [lambda: grads([fn(logits, t)], [logits], [one])]
    if ref:
        from kernels.cross_entropy import hilda_cross_entropy
        measure(out, "triton", mk(lambda x, t_: hilda_cross_entropy(x, t_, -100, "mean")))
    try:
        from liger_kernel.ops.cross_entropy import LigerCrossEntropyFunction
        measure(out, "liger", mk(lambda x, t_: LigerCrossEntropyFunction.apply(
            x, t_, None, -100, 0.0, 0.0, "mean", None, False, False)[0]))
    except ImportError as e:
        out["liger_error"] = str(e)
    measure(out, "eager", mk(lambda x, t_: F.cross_entropy(x.float(), t_, ignore_index=-100)))
    return "cross_entropy_bf16_fwd+bwd", out


def op_grpo(ref, g):
    out = {}
    B, Lc, v = 16, 1023, 151936
    logits = torch.empty(B, Lc + 1, v, device=DEV, dtype=torch.bfloat16)
    for b in range(B):
        logits[b] = (2 * rn(g, Lc + 1, v)).bfloat16()
    logits.requires_grad_(True)
    ids = torch.randint(0, v, (B, Lc), device=DEV, generator=g)
    adv = rn(g, B)
    lens = torch.randint(256, 1025, (B,), device=DEV, generator=g).clamp(max=Lc)
    mask = (torch.arange(Lc, device=DEV)[None] < lens[:, None]).int()
    old = rn(g, B, Lc) * 0.05 - 12.0
    ref_lp = old + 0.1 * rn(g, B, Lc)
    one = torch.ones((), device=DEV)
    if ref:
        from kernels.grpo_loss import hilda_grpo_loss
        measure(out, "triton", lambda: [lambda: grads(
            [hilda_grpo_loss(logits, ids, adv, old, ref_lp, mask, 1.0, 0.1, 0.2, 0.2)[0]], [logits], [one])], iters=3)

    def eager():
        lp = logits[:, :-1].float().log_softmax(-1).gather(-1, ids[..., None]).squeeze(-1)
        ratio = torch.exp(lp - old)
        a = adv[:, None]
        ptl = -torch.min(ratio * a, ratio.clamp(0.8, 1.2) * a) + 0.1 * (torch.exp(ref_lp - lp) - (ref_lp - lp) - 1)
        m = mask.float()
        return ((ptl * m).sum(-1) / m.sum(-1).clamp(min=1.0)).mean()
    measure(out, "eager", lambda: [lambda: grads([eager()], [logits], [one])], iters=3)
    out["liger_error"] = "no Liger comparison in the reference's bench_grpo.py"
    return "grpo_bf16_fwd+bwd", out


def op_flce(ref, g):
    out = {}
    bt, h, v = 16384, 4096, 128256
    hidden = rn(g, bt, h).bfloat16().requires_grad_(True)
    weight = (0.02 * rn(g, v, h)).bfloat16().requires_grad_(True)
    t = torch.randint(0, v, (bt,), device=DEV, generator=g)
    t[torch.randperm(bt, device=DEV, generator=g)[: round(0.05 * bt)]] = -100
    one = torch.ones((), device=DEV)

    def mk(fn):
        return lambda: [lambda: grads([fn(hidden, weight, t)], [hidden, weight], [one])]
    if ref:
        from kernels.fused_linear_cross_entropy import hilda_fused_linear_cross_entropy
        measure(out, "triton", mk(lambda a, w, t_: hilda_fused_linear_cross_entropy(a, w, t_, -100, "mean")), iters=3)
    try:
        from liger_kernel.ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction
        measure(out, "liger", mk(lambda a, w, t_: LigerFusedLinearCrossEntropyFunction.apply(
            a, w, t_, None, None, -100, 0.0, 0.0, "mean", None, False)[0]), iters=3)
    except ImportError as e:
        out["liger_error"] = str(e)
    measure(out, "eager", mk(lambda a, w, t_: F.cross_entropy((a @ w.T).float(), t_, ignore_index=-100)), iters=3)
    for k in ("triton", "liger", "eager"):
        if out.get(k + "_us"):
            out[k + "_tokens/s"] = round(bt / (out[k + "_us"] * 1e-6))
    return "fused_linear_cross_entropy_bf16_fwd+bwd", out



def op_attn_res(ref, g):
    """8 blocks of [8192 tokens, 4096] bf16, forward and backward helpers called as bench.py calls its own."""
    out = {}
    nb, ntok, d = 8, 8192, 4096
    wq, wn = (0.02 * rn(g, d)).bfloat16(), (1 + 0.1 * rn(g, d)).bfloat16()
    sets = [(rn(g, nb, ntok, d).bfloat16(), rn(g, ntok, d).bfloat16()) for _ in range(2)]
    if ref:
        from kernels.attn_res import attn_res_backward, attn_res_forward

        def one(Vb, dh):
            _, v3, al, rs = attn_res_forward(Vb, wq, wn)
            attn_res_backward(dh, v3, wq, wn, al, rs)
        measure(out, "triton", lambda: [(lambda a=a: one(*a)) for a in sets])

    def eager(Vb, dh):
        Vb = Vb.detach().requires_grad_(True)
        vf = Vb.float()
        key = (vf * torch.rsqrt(vf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(Vb.dtype) * wn
        alpha = (key.float() * wq.float()).sum(-1).softmax(0)
        h = (alpha.unsqueeze(-1) * vf).sum(0).to(Vb.dtype)
        grads([h], [Vb], [dh])
    measure(out, "eager", lambda: [(lambda a=a: eager(*a)) for a in sets], iters=3)
    return "attn_res_bf16_fwd+bwd", out


def op_paged_attention(ref, g):
    out = {}
    batch, nh, nkv, ctx, bs = 32, 16, 8, 4096, 256
    per_seq = ctx // bs
    sets = []
    for _ in range(3):
        q = rn(g, batch, nh, 128).bfloat16()
        kc = rn(g, batch * per_seq, bs, nkv, 128).to(torch.float8_e4m3fn)
        vc = rn(g, batch * per_seq, bs, nkv, 128).to(torch.float8_e4m3fn)
        bt = torch.randperm(batch * per_seq, device=DEV, generator=g).int().view(batch, per_seq)
        cl = torch.full((batch,), ctx, device=DEV, dtype=torch.int32)
        sets.append((q, kc, vc, bt, cl))
    if ref:
        from kernels.paged_attention_fp8 import hilda_paged_attention_fp8_decode, reference_paged_attention_decode
        measure(out, "triton", lambda: [(lambda a=a: hilda_paged_attention_fp8_decode(*a, 128 ** -0.5)) for a in sets])
        measure(out, "eager", lambda: [(lambda a=a: reference_paged_attention_decode(*a, 128 ** -0.5)) for a in sets],
                iters=3)
    return "paged_attention_fp8_decode", out


def op_kl_div(ref, g):
    out = {}
    n, v = 8192, 128256
    sets = [(rn(g, n, v).log_softmax(-1).bfloat16(), rn(g, n, v).softmax(-1).bfloat16()) for _ in range(2)]
    one = torch.ones((), device=DEV)
    if ref:
        from kernels.kl_div import kl_div_backward, kl_div_forward

        def tri(yp, yt):
            kl_div_forward(yp, yt)
            kl_div_backward(yt, one)
        measure(out, "triton", lambda: [(lambda a=a: tri(*a)) for a in sets])

    def through_autograd(fn):
        def one_(yp, yt):
            yp = yp.detach().requires_grad_(True)
            grads([fn(yp, yt)], [yp], [one.to(torch.float32)])
        return lambda: [(lambda a=a: one_(*a)) for a in sets]
    try:
        from liger_kernel.ops.kl_div import LigerKLDivLossFunction
        measure(out, "liger", through_autograd(lambda yp, yt: LigerKLDivLossFunction.apply(yp, yt, "batchmean", False, 1e-10).float()))
    except ImportError as e:
        out["liger_error"] = str(e)
    measure(out, "eager", through_autograd(lambda yp, yt: F.kl_div(yp.float(), yt.float(), reduction="batchmean")), iters=3)
    return "kl_div_bf16_fwd+bwd", out


def op_jsd(ref, g):
    out = {}
    n, v = 4096, 128256
    sets = [(rn(g, n, v).log_softmax(-1).bfloat16(), rn(g, n, v).log_softmax(-1).bfloat16()) for _ in range(2)]
    if ref:
        from kernels.jsd import jsd_forward
        measure(out, "triton", lambda: [(lambda a=a: jsd_forward(a[0], a[1], 0.5)) for a in sets])
    one = torch.ones((), device=DEV)

    def through_autograd(fn):
        def one_(x, y):
            x = x.detach().requires_grad_(True)
            loss = fn(x, y)
            grads([loss], [x], [one.to(loss.dtype)])
        return lambda: [(lambda a=a: one_(*a)) for a in sets]
    try:
        from liger_kernel.ops.jsd import LigerJSDFunction
        measure(out, "liger", through_autograd(lambda x, y: LigerJSDFunction.apply(x, y, None, 0.5, -100)))
    except ImportError as e:
        out["liger_error"] = str(e)

    def eager(x, y):
        xf, yf = x.float(), y.float()
        m = torch.log(0.5 * (xf.exp() + yf.exp()))
        return 0.5 * (F.kl_div(m, yf, reduction="sum", log_target=True) + F.kl_div(m, xf, reduction="sum", log_target=True)) / x.shape[0]
    measure(out, "eager", through_autograd(eager), iters=3)
    return "jsd_bf16_fwd+bwd", out


def op_fused_linear_jsd(ref, g):
    out = {}
    n, h, v = 2048, 4096, 128256
    si, sw = (0.02 * rn(g, n, h)).bfloat16(), (0.02 * rn(g, v, h)).bfloat16()
    ti, tw = (0.02 * rn(g, n, h)).bfloat16(), (0.02 * rn(g, v, h)).bfloat16()
    if ref:
        from kernels.fused_linear_jsd import fused_linear_jsd_forward
        measure(out, "triton", lambda: [lambda: fused_linear_jsd_forward(si, sw, ti, tw, None, 0.5, 1.0)], iters=3)
    one = torch.ones((), device=DEV)

    def through_autograd(fn):
        def one_():
            a, w = si.detach().requires_grad_(True), sw.detach().requires_grad_(True)
            loss = fn(a, w)
            grads([loss], [a, w], [one.to(loss.dtype)])
        return lambda: [one_]
    try:
        from liger_kernel.ops.fused_linear_jsd import LigerFusedLinearJSDFunction
        measure(out, "liger", through_autograd(lambda a, w: LigerFusedLinearJSDFunction.apply(a, w, ti, tw, None, 0.5, -100, 1.0)), iters=3)
    except ImportError as e:
        out["liger_error"] = str(e)

    def eager(a, w):
        xs = (a @ w.T).float().log_softmax(-1)
        with torch.no_grad():
            ys = (ti @ tw.T).float().log_softmax(-1)
        m = torch.log(0.5 * (xs.exp() + ys.exp()))
        return 0.5 * (F.kl_div(m, ys, reduction="sum", log_target=True) + F.kl_div(m, xs, reduction="sum", log_target=True)) / n
    measure(out, "eager", through_autograd(eager), iters=3)
    return "fused_linear_jsd_bf16_fwd+bwd", out


OPS = {"rms_norm": op_rms_norm, "fused_add_rms_norm": op_fused_add_rms_norm, "rope": op_rope, "rope_bhsd": op_rope_bhsd, "swiglu": op_swiglu, "geglu": op_geglu,
       "cross_entropy": op_cross_entropy, "fused_linear_cross_entropy": op_flce, "grpo": op_grpo,
       "attn_res": op_attn_res, "paged_attention": op_paged_attention, "kl_div": op_kl_div, "jsd": op_jsd,
       "fused_linear_jsd": op_fused_linear_jsd}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default=",".join(OPS))
    args = ap.parse_args()
    assert "hilda_kernel_b200" not in sys.modules
    torch.cuda.set_device(0)
    ref, why = load_reference()
    try:
        import triton
        tv = triton.__version__
    except Exception as e:
        tv = f"unavailable ({e})"
    try:
        import liger_kernel  # noqa: F401
        from importlib.metadata import version
        lv = version("liger_kernel")
    except Exception as e:
        lv = f"unavailable ({e})"
    print(json.dumps({"_meta": {"triton": tv, "liger": lv, "reference_kernels": "installed" if ref else why,
                                "method": "fwd+bwd through the autograd API, CUDA-graph replay between events"}}),
          flush=True)
    g = torch.Generator(device=DEV).manual_seed(1)
    for name in args.ops.split(","):
        if name not in OPS:
            continue
        t0 = time.perf_counter()
        try:
            key, res = OPS[name](ref, g)
        except Exception as e:
            key, res = name, {"error": f"{type(e).__name__}: {e}"}
        if ref is None:
            res["triton_error"] = why
        res["wall_s"] = round(time.perf_counter() - t0, 1)
        print(json.dumps({key: res}), flush=True)
        torch.cuda.empty_cache()
    assert "hilda_kernel_b200" not in sys.modules


if __name__ == "__main__":
    main()
