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


def _normalize_query_shape(q):
    if q.ndim == 4:
        if q.shape[1] != 1:
            raise ValueError(f'decode query must have shape [batch, 1, heads, dim], got {tuple(q.shape)}')
        return q[:, 0], True
    if q.ndim != 3:
        raise ValueError(f'decode query must have shape [batch, heads, dim], got {tuple(q.shape)}')
    return q, False


def _validate_inputs(q, k_cache, v_cache, block_tables, context_lens):
    q_3d, restore_seq_dim = _normalize_query_shape(q)
    if q_3d.dtype != torch.bfloat16:
        raise TypeError(f'q must be bfloat16, got {q_3d.dtype}')
    if k_cache.dtype != torch.float8_e4m3fn or v_cache.dtype != torch.float8_e4m3fn:
        raise TypeError('k_cache and v_cache must use torch.float8_e4m3fn')
    if k_cache.shape != v_cache.shape:
        raise ValueError('k_cache and v_cache must have the same shape')
    if k_cache.ndim != 4:
        raise ValueError(f'k_cache must be [num_blocks, block_size, num_kv_heads, head_dim], got {tuple(k_cache.shape)}')
    if block_tables.ndim != 2:
        raise ValueError(f'block_tables must be [batch, max_num_blocks], got {tuple(block_tables.shape)}')
    if context_lens.ndim != 1:
        raise ValueError(f'context_lens must be [batch], got {tuple(context_lens.shape)}')
    if not (q_3d.is_cuda and k_cache.is_cuda and v_cache.is_cuda and block_tables.is_cuda and context_lens.is_cuda):
        raise ValueError('all tensors must be on CUDA')
    batch, num_heads, head_dim = q_3d.shape
    _, _, num_kv_heads, cache_head_dim = k_cache.shape
    if batch != block_tables.shape[0] or batch != context_lens.shape[0]:
        raise ValueError('batch dimension mismatch between q, block_tables and context_lens')
    if head_dim != 128 or cache_head_dim != 128:
        raise ValueError('this kernel currently requires head_dim=128')
    if num_heads % num_kv_heads != 0:
        raise ValueError('num_heads must be divisible by num_kv_heads for GQA')
    return q_3d, restore_seq_dim


@torch.inference_mode()
def hilda_paged_attention_fp8_decode(q, k_cache, v_cache, block_tables, context_lens, scale):
    q_3d, restore_seq_dim = _validate_inputs(q, k_cache, v_cache, block_tables, context_lens)
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
    """The plain PyTorch evaluation the reference exports beside its kernel
    (paged_attention_fp8.py:191-221); runs on whatever device the tensors are on."""
    q_3d, restore_seq_dim = _normalize_query_shape(q)
    batch, num_heads, head_dim = q_3d.shape
    _, block_size, num_kv_heads, _ = k_cache.shape
    kv_of_head = torch.arange(num_heads, device=q_3d.device) // (num_heads // num_kv_heads)
    out = torch.empty((batch, num_heads, head_dim), device=q_3d.device, dtype=torch.bfloat16)
    for b in range(batch):
        n_ctx = int(context_lens[b])
        n_blk = -(-n_ctx // block_size)
        ids = block_tables[b, :n_blk].long()
        k = k_cache.index_select(0, ids).reshape(-1, num_kv_heads, head_dim)[:n_ctx].float().index_select(1, kv_of_head)
        v = v_cache.index_select(0, ids).reshape(-1, num_kv_heads, head_dim)[:n_ctx].float().index_select(1, kv_of_head)
        probs = (torch.einsum('hd,thd->ht', q_3d[b].float(), k) * scale).softmax(dim=-1)
        out[b] = torch.einsum('ht,thd->hd', probs, v).to(torch.bfloat16)
    return out.unsqueeze(1) if restore_seq_dim else out
