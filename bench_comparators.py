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


OPS = {"rms_norm": op_rms_norm, "fused_add_rms_norm": op_fused_add_rms_norm, "rope": op_rope, "rope_bhsd": op_rope_bhsd, "swiglu": op_swiglu,
       "cross_entropy": op_cross_entropy, "fused_linear_cross_entropy": op_flce, "grpo": op_grpo}


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
