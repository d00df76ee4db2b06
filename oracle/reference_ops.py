"""CPU oracle for the token-parallel operator path of hilda-kernel.

TEST INFRASTRUCTURE ONLY. Nothing in the shipped package imports this file; only ``tests/``,
``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` do,
and there only as the checker or the CPU baseline, never as the product path.

Each function restates, in plain PyTorch on whatever device its inputs live on (CPU in the
tests), the reference implementation that hilda-kernel's own benchmark scripts compare their
Triton kernels against. Paths are relative to ``triton-kernels/`` in hilda-kernel. Parity is
pinned: ``tests/golden/make_golden.py`` imports those reference functions themselves and stores
their outputs on seeded inputs; ``tests/test_oracle_golden.py`` checks this file against them.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- RMSNorm
def rms_norm(x, weight, eps=1e-6):
    """benchmarks/bench_rms_norm.py:37-41 (``pytorch_rms_norm``). Returns fp32 for 16-bit x
    because of type promotion; callers cast to the operator's output dtype before comparing."""
    variance = x.float().pow(2).mean(-1, keepdim=True)
    x_normed = x * torch.rsqrt(variance + eps)
    return x_normed * weight


def rms_norm_cast(x, weight, eps=1e-6):
    """tests/test_rms_norm.py:22-28 (``pytorch_rms_norm_reference``): all fp32, cast at the end."""
    x_f32 = x.float()
    variance = x_f32.pow(2).mean(-1, keepdim=True)
    x_normed = x_f32 * torch.rsqrt(variance + eps)
    return (x_normed * weight.float()).to(x.dtype)


# --------------------------------------------------------------------------- FusedAddRMSNorm
def fused_add_rms_norm(X, R, W, eps=1e-6):
    """benchmarks/bench_fused_add_rms_norm.py:37-41 (``pytorch_fused_add_rms_norm``)."""
    S = X + R
    rms = torch.sqrt(torch.mean(S.float() ** 2, dim=-1, keepdim=True) + eps)
    Y = (S.float() / rms).to(S.dtype) * W
    return Y, S


# --------------------------------------------------------------------------- RoPE
def rotate_half(x):
    """benchmarks/bench_rope.py:40-43."""
    x1 = x[..., : x.shape[-1] // 2]
    x2 = x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def rope(q, k, cos, sin):
    """benchmarks/bench_rope.py:46-58 (``pytorch_rope``): q, k (bsz, n_h, seq, hd); cos, sin
    half-width (1|bsz, seq, hd//2)."""
    cos_full = torch.cat([cos, cos], dim=-1)
    sin_full = torch.cat([sin, sin], dim=-1)
    cos_4d = cos_full.unsqueeze(1)
    sin_4d = sin_full.unsqueeze(1)
    q_embed = (q * cos_4d) + (rotate_half(q) * sin_4d)
    k_embed = (k * cos_4d) + (rotate_half(k) * sin_4d)
    return q_embed, k_embed


def rope_tables(seq_len, head_dim, base=10000.0, dtype=torch.float32, device=None):
    """kernels/rope.py:209-222 (``RotaryEmbedding``): half-width cos/sin of shape (1, seq, hd//2)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    t = torch.arange(seq_len, device=device, dtype=torch.float32)
    freqs = torch.outer(t, inv_freq)
    return freqs.cos()[None].to(dtype), freqs.sin()[None].to(dtype)


def rope_backward_ones(cos, sin):
    """Known answer of benchmarks/bench_rope.py:132-146: the backward of an all-ones gradient is
    cat(cos + sin, cos - sin) broadcast over batch and heads."""
    c = cos.unsqueeze(1)
    s = sin.unsqueeze(1)
    return torch.cat([c + s, c - s], dim=-1)


# --------------------------------------------------------------------------- SwiGLU
def swiglu(a, b):
    """benchmarks/bench_swiglu.py:46-47 (``pytorch_swiglu``)."""
    return F.silu(a) * b


# --------------------------------------------------------------------------- GeGLU
def geglu(a, b):
    """benchmarks/bench_geglu.py:41-42 (``pytorch_geglu``)."""
    return F.gelu(a, approximate="tanh") * b


# --------------------------------------------------------------------------- CrossEntropy
def cross_entropy(logits, targets, ignore_index=-100, reduction="mean"):
    """benchmarks/bench_cross_entropy.py:77-79, :101-104: ``F.cross_entropy`` with ignore_index.
    Evaluate on ``logits.float()`` for the fp32 scalar check (a bf16 call returns a bf16 loss).
    With no valid row torch gives NaN for 'mean'; the operator (kernels/cross_entropy.py:131-137
    and the clamp at :129) gives 0, which ``cross_entropy_clamped`` restates."""
    return F.cross_entropy(logits, targets, ignore_index=ignore_index, reduction=reduction)


def cross_entropy_clamped(logits, targets, ignore_index=-100, reduction="mean"):
    """The operator's own contract (kernels/cross_entropy.py:114-166, :206-249): per-row loss 0 on
    ignored rows; 'mean' divides by max(n_valid, 1)."""
    per_row = F.cross_entropy(logits, targets, ignore_index=ignore_index, reduction="none")
    if reduction == "none":
        return per_row
    if reduction == "sum":
        return per_row.sum()
    n_valid = (targets != ignore_index).sum().clamp_min(1)
    return per_row.sum() / n_valid.to(per_row.dtype)


# --------------------------------------------------------------------------- FusedLinearCE
def linear_cross_entropy(hidden, weight, targets, ignore_index=-100, reduction="mean"):
    """benchmarks/bench_fused_linear_ce.py:36-38 (``pytorch_linear_ce``) with the ignore_index the
    operator takes (kernels/fused_linear_cross_entropy.py:213-220)."""
    logits = hidden @ weight.T
    return F.cross_entropy(logits, targets, ignore_index=ignore_index, reduction=reduction)


def linear_cross_entropy_fp32_chunked(hidden, weight, targets, ignore_index=-100, reduction="mean", rows=2048):
    """Same quantity evaluated in fp32 in row chunks (full fp32 logits of the benchmark shape are
    8.4 GB). Returns the loss only. 'mean' divides by max(n_valid, 1) like the operator
    (kernels/fused_linear_cross_entropy.py:121-126, :164-165)."""
    w = weight.float()
    total = torch.zeros((), dtype=torch.float64)
    per_row = []
    for s in range(0, hidden.shape[0], rows):
        lg = hidden[s:s + rows].float() @ w.T
        pr = F.cross_entropy(lg, targets[s:s + rows], ignore_index=ignore_index, reduction="none")
        per_row.append(pr)
        total += pr.double().sum()
    if reduction == "none":
        return torch.cat(per_row)
    if reduction == "sum":
        return total.float()
    n_valid = max(int((targets != ignore_index).sum()), 1)
    return (total / n_valid).float()


# --------------------------------------------------------------------------- GRPO
def selective_log_softmax(logits, ids, temperature=1.0):
    """The log-prob gather at the head of ``pytorch_grpo_loss`` (benchmarks/bench_grpo.py:36-40);
    logits (B, L+1, V), ids (B, L) -> (B, L)."""
    L = logits.shape[1] - 1
    lp = (logits[:, :-1, :] / temperature).log_softmax(dim=-1)
    return lp.gather(-1, ids[:, -L:].unsqueeze(-1)).squeeze(-1)


def grpo_loss(logits, completion_ids, advantages, old_logp=None, ref_logp=None, completion_mask=None,
              temperature=1.0, beta=0.0, eps_low=0.2, eps_high=0.2):
    """benchmarks/bench_grpo.py:30-57 (``pytorch_grpo_loss``). The bench feeds it
    ``logits.float()`` (:80, :128)."""
    logp = selective_log_softmax(logits, completion_ids, temperature)
    if old_logp is None:
        old_logp = logp.detach()
    ratio = torch.exp(logp - old_logp)
    ratio_clipped = torch.clamp(ratio, 1 - eps_low, 1 + eps_high)
    adv = advantages.unsqueeze(-1)
    per_token_loss = -torch.min(ratio * adv, ratio_clipped * adv)
    if beta != 0.0 and ref_logp is not None:
        kl = torch.exp(ref_logp - logp) - (ref_logp - logp) - 1
        per_token_loss = per_token_loss + beta * kl
    mask = completion_mask.float() if completion_mask is not None else torch.ones_like(per_token_loss)
    seq_lens = mask.sum(-1).clamp(min=1.0)
    return ((per_token_loss * mask).sum(-1) / seq_lens).mean()


def grpo_aux(logits, completion_ids, advantages, old_logp=None, ref_logp=None, completion_mask=None,
             temperature=1.0, beta=0.0, eps_low=0.2, eps_high=0.2):
    """kl_mean and clip_ratio as the operator reduces them (kernels/grpo_loss.py:140-142 for the
    clip rule, :150 for kl, :290-292 for the masked means), on the oracle's logp."""
    logp = selective_log_softmax(logits, completion_ids, temperature)
    old = logp if old_logp is None else old_logp
    coef_1 = torch.exp(logp - old)
    adv = advantages.unsqueeze(-1)
    is_clipped = ((coef_1 < 1 - eps_low) & (adv < 0)) | ((coef_1 > 1 + eps_high) & (adv > 0))
    mask = completion_mask.float() if completion_mask is not None else torch.ones_like(logp)
    mask_sum = mask.sum().clamp(min=1.0)
    clip_ratio = (is_clipped.float() * mask).sum() / mask_sum
    kl_mean = None
    if beta != 0.0:
        kl = torch.exp(ref_logp - logp) - (ref_logp - logp) - 1
        kl_mean = (kl * mask).sum() / mask_sum
    return kl_mean, clip_ratio


# --------------------------------------------------------------------------- KL divergence
def kl_div(y_pred, y_true, reduction="batchmean", log_target=False):
    """benchmarks/bench_kl_div.py:45, :66: ``torch.nn.functional.kl_div`` (y_pred log-probs,
    y_true probs)."""
    return F.kl_div(y_pred, y_true, reduction=reduction, log_target=log_target)


def kl_div_rows(y_pred, y_true, reduction="batchmean", log_target=False, eps=1e-10):
    """The operator's own contract (kernels/kl_div.py:52-64, :114-137): per-ROW sums of
    t (log max(t, eps) - y) (or exp(t) (t - y) with log_target); 'none' returns the row sums,
    'mean' divides by rows x cols, 'batchmean' by rows."""
    y, t = y_pred.float(), y_true.float()
    y2, t2 = y.reshape(-1, y.shape[-1]), t.reshape(-1, t.shape[-1])
    per_row = (t2.exp() * (t2 - y2)).sum(-1) if log_target else (t2 * (t2.clamp_min(eps).log() - y2)).sum(-1)
    if reduction == "none":
        return per_row
    if reduction == "sum":
        return per_row.sum()
    if reduction == "mean":
        return per_row.sum() / y2.numel()
    return per_row.sum() / y2.shape[0]


# --------------------------------------------------------------------------- JSD
def jsd(X, Y, beta=0.5):
    """benchmarks/bench_jsd.py:30-44 (``pytorch_jsd``): X student, Y teacher log-probs."""
    Q = X.exp()
    P = Y.exp()
    if beta == 0.0:
        loss = (P * (Y - X)).sum(-1)
    elif beta == 1.0:
        loss = (Q * (X - Y)).sum(-1)
    else:
        M = beta * P + (1 - beta) * Q
        log_M = M.log()
        loss = beta * (P * (Y - log_M)).sum(-1) + (1 - beta) * (Q * (X - log_M)).sum(-1)
    return loss.mean()


def jsd_labels(X, Y, beta=0.5, labels=None, ignore_index=-100):
    """The operator's contract with labels (kernels/jsd.py:49-58, :116-120): rows whose label is
    ignore_index contribute nothing; the sum is divided by max(#other rows, 1)."""
    Q, P = X.exp(), Y.exp()
    if beta == 0.0:
        per_row = (P * (Y - X)).sum(-1)
    elif beta == 1.0:
        per_row = (Q * (X - Y)).sum(-1)
    else:
        M = beta * P + (1 - beta) * Q
        log_M = M.log()
        per_row = beta * (P * (Y - log_M)).sum(-1) + (1 - beta) * (Q * (X - log_M)).sum(-1)
    if labels is None:
        return per_row.sum() / X.shape[0]
    keep = labels != ignore_index
    return (per_row * keep).sum() / max(int(keep.sum()), 1)


# --------------------------------------------------------------------------- FusedLinearJSD
def linear_jsd(s_input, s_weight, t_input, t_weight, beta=0.5, temperature=1.0):
    """benchmarks/bench_fused_linear_jsd.py:31-43 (``pytorch_linear_jsd``); the bench feeds it fp32
    copies of the inputs (:60, :83-85)."""
    s_logits = (s_input @ s_weight.t()) / temperature
    t_logits = (t_input @ t_weight.t()) / temperature
    X = s_logits.log_softmax(dim=-1)
    Y = t_logits.log_softmax(dim=-1)
    Q = X.exp()
    P = Y.exp()
    M = beta * P + (1 - beta) * Q
    log_M = M.log()
    loss = beta * (P * (Y - log_M)).sum(-1) + (1 - beta) * (Q * (X - log_M)).sum(-1)
    return loss.mean()


def linear_jsd_labels(s_input, s_weight, t_input, t_weight, labels=None, beta=0.5, temperature=1.0, ignore_index=-100):
    """The operator's contract (kernels/fused_linear_jsd.py:137-141, :182-190): any beta through
    the JSD kernel's three branches, rows with an ignored label dropped, mean over the others."""
    X = ((s_input @ s_weight.t()) / temperature).log_softmax(dim=-1)
    Y = ((t_input @ t_weight.t()) / temperature).log_softmax(dim=-1)
    return jsd_labels(X, Y, beta, labels, ignore_index)


# --------------------------------------------------------------------------- AttnRes
def attn_res(V, w_query, w_norm, eps=1e-6):
    """benchmarks/bench_attn_res.py:33-51 (``pytorch_attn_res``): V [N, B, T, D], w_query, w_norm [D]."""
    V_f32 = V.float()
    rms = torch.sqrt(V_f32.pow(2).mean(dim=-1, keepdim=True) + eps)
    K = (V_f32 / rms).to(V.dtype) * w_norm
    scores = torch.einsum('d, n b t d -> n b t', w_query.float(), K.float())
    alpha = scores.softmax(dim=0)
    h = torch.einsum('n b t, n b t d -> b t d', alpha, V.float()).to(V.dtype)
    return h


# --------------------------------------------------------------------------- paged FP8 decode attention
def paged_attention_decode(q, k_cache, v_cache, block_tables, context_lens, scale):
    """kernels/paged_attention_fp8.py:191-221 (``reference_paged_attention_decode``): q
    [batch, heads, 128] bf16, caches [blocks, block_size, kv_heads, 128] fp8 e4m3; fp32 math,
    bf16 result. Returns the fp32 result as well (second value) for tolerance checks."""
    batch, num_heads, head_dim = q.shape
    _, block_size, num_kv_heads, _ = k_cache.shape
    kv_of_head = torch.arange(num_heads) // (num_heads // num_kv_heads)
    out32 = torch.zeros((batch, num_heads, head_dim), dtype=torch.float32)
    kf, vf = k_cache.float(), v_cache.float()
    for b in range(batch):
        n_ctx = int(context_lens[b])
        if n_ctx == 0:
            continue
        n_blk = -(-n_ctx // block_size)
        ids = block_tables[b, :n_blk].long()
        k = kf.index_select(0, ids).reshape(-1, num_kv_heads, head_dim)[:n_ctx].index_select(1, kv_of_head)
        v = vf.index_select(0, ids).reshape(-1, num_kv_heads, head_dim)[:n_ctx].index_select(1, kv_of_head)
        probs = (torch.einsum('hd,thd->ht', q[b].float(), k) * scale).softmax(dim=-1)
        out32[b] = torch.einsum('ht,thd->hd', probs, v)
    return out32.to(torch.bfloat16), out32
