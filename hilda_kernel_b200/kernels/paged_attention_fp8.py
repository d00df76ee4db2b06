"""Decode attention over a paged FP8 (e4m3) KV cache, behind the reference operator interface.

Mirrors kernels/paged_attention_fp8.py of hilda-kernel: ``hilda_paged_attention_fp8_decode`` (:141-188)
and ``reference_paged_attention_decode`` (:191-221, a plain PyTorch evaluation the reference exports
beside its kernel). q: [batch, heads, 128] (or [batch, 1, heads, 128]) bfloat16; k_cache, v_cache:
[num_blocks, block_size, kv_heads, 128] float8_e4m3fn; block_tables: [batch, max_blocks];
context_lens: [batch]; returns bfloat16 of q's shape. The KV cache is read once per kv head: all
query heads of a GQA group are served by the same CTA, and long contexts are split over CTAs.
"""
import torch

from .. import _lib as L
from .._lib import device_guard


def _as_decode_query(q):
    """[batch, heads, dim] view of a decode query given as that or as [batch, 1, heads, dim];
    the flag says whether the length-1 sequence axis has to be put back on the result."""
    if q.ndim == 3:
        return q, False
    if q.ndim == 4 and q.shape[1] == 1:
        return q[:, 0], True
    raise ValueError(f"a decode query is [batch, heads, dim] or [batch, 1, heads, dim]; got {tuple(q.shape)}")


def _check_decode_inputs(q, k_cache, v_cache, block_tables, context_lens):
    """Same acceptance rules and exception types as the reference (paged_attention_fp8.py:104-137):
    TypeError for dtypes, ValueError for shapes and devices."""
    q3, had_seq_axis = _as_decode_query(q)
    if q3.dtype is not torch.bfloat16:
        raise TypeError(f"the query must be bfloat16, not {q3.dtype}")
    for name, cache in (("k_cache", k_cache), ("v_cache", v_cache)):
        if cache.dtype is not torch.float8_e4m3fn:
            raise TypeError(f"{name} must be float8_e4m3fn, not {cache.dtype}")
        if cache.ndim != 4:
            raise ValueError(f"{name} is [blocks, block_size, kv_heads, head_dim]; got {tuple(cache.shape)}")
    if v_cache.shape != k_cache.shape:
        raise ValueError(f"k_cache {tuple(k_cache.shape)} and v_cache {tuple(v_cache.shape)} differ in shape")
    if block_tables.ndim != 2 or context_lens.ndim != 1:
        raise ValueError("block_tables is [batch, max_blocks] and context_lens is [batch]")
    if not all(t.is_cuda for t in (q3, k_cache, v_cache, block_tables, context_lens)):
        raise ValueError("every tensor has to live on a CUDA device")
    n_seq, n_heads, dim = q3.shape
    n_kv, cache_dim = k_cache.shape[2], k_cache.shape[3]
    if block_tables.shape[0] != n_seq or context_lens.shape[0] != n_seq:
        raise ValueError("q, block_tables and context_lens disagree on the batch size")
    if (dim, cache_dim) != (128, 128):
        raise ValueError("only head_dim = 128 is supported, as in the reference kernel")
    if n_heads % n_kv:
        raise ValueError("the number of query heads must be a multiple of the number of kv heads")
    return q3, had_seq_axis


@torch.inference_mode()
def hilda_paged_attention_fp8_decode(q, k_cache, v_cache, block_tables, context_lens, scale):
    q_3d, restore_seq_dim = _check_decode_inputs(q, k_cache, v_cache, block_tables, context_lens)
    dev = q_3d.device
    if q_3d.stride(-1) != 1:
        q_3d = q_3d.contiguous()
    if k_cache.stride(-1) != 1:
        k_cache = k_cache.contiguous()
    if v_cache.stride(-1) != 1:
        v_cache = v_cache.contiguous()
    block_tables = block_tables.to(torch.int32)
    if block_tables.stride(-1) != 1:
        block_tables = block_tables.contiguous()
    context_lens = context_lens.to(torch.int32).contiguous()
    batch, num_heads, head_dim = q_3d.shape
    _, block_size, num_kv_heads, _ = k_cache.shape
    max_blocks = block_tables.shape[1]
    out = torch.empty((batch, num_heads, head_dim), device=dev, dtype=torch.bfloat16)
    lib = L.lib()
    with device_guard(dev):
        ws = torch.empty(lib.hilda_paged_attention_fp8_workspace_bytes(batch, num_heads, num_kv_heads, max_blocks,
                                                                      block_size) // 4, dtype=torch.float32, device=dev)
        rc = lib.hilda_paged_attention_fp8_decode(
            L.ptr(q_3d), q_3d.stride(0), q_3d.stride(1),
            L.ptr(k_cache), k_cache.stride(0), k_cache.stride(1), k_cache.stride(2),
            L.ptr(v_cache), v_cache.stride(0), v_cache.stride(1), v_cache.stride(2),
            L.ptr(out), out.stride(0), out.stride(1), L.ptr(block_tables), block_tables.stride(0), L.ptr(context_lens),
            L.ptr(ws), float(scale), batch, num_heads, num_kv_heads, head_dim, block_size, max_blocks, L.stream(dev))
    L.check(rc, "paged_attention_fp8_decode")
    return out.unsqueeze(1) if restore_seq_dim else out


@torch.inference_mode()
def reference_paged_attention_decode(q, k_cache, v_cache, block_tables, context_lens, scale):
    """Plain PyTorch evaluation of the same quantity, exported beside the kernel as in the reference
    (paged_attention_fp8.py:191-221): per sequence, gather its blocks, dequantise to fp32, softmax
    attention of every query head over its kv head, result in bfloat16. Runs wherever the tensors are."""
    q3, had_seq_axis = _as_decode_query(q)
    n_seq, n_heads, dim = q3.shape
    block_size, n_kv = k_cache.shape[1], k_cache.shape[2]
    head_to_kv = torch.arange(n_heads, device=q3.device) // (n_heads // n_kv)
    result = q3.new_empty((n_seq, n_heads, dim), dtype=torch.bfloat16)
    for s_idx, n_ctx in enumerate(context_lens.tolist()):
        blocks = block_tables[s_idx, : -(-n_ctx // block_size)].long()
        keys = k_cache[blocks].reshape(-1, n_kv, dim)[:n_ctx].float()[:, head_to_kv]
        vals = v_cache[blocks].reshape(-1, n_kv, dim)[:n_ctx].float()[:, head_to_kv]
        weights = torch.softmax(torch.einsum('hd,thd->ht', q3[s_idx].float(), keys) * scale, dim=-1)
        result[s_idx] = torch.einsum('ht,thd->hd', weights, vals).to(torch.bfloat16)
    return result.unsqueeze(1) if had_seq_axis else result
