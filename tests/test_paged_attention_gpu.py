"""GPU parity tests of the paged FP8 decode attention against the CPU oracle (the reference's own
PyTorch evaluation, oracle/reference_ops.py) and its golden output."""
import pytest
import torch

from oracle import reference_ops as R

pytestmark = pytest.mark.gpu

DEV = "cuda"


def gen(seed):
    return torch.Generator().manual_seed(seed)


def _inputs(batch, n_heads, n_kv, ctx_lens, block_size, seed=51, shuffle=True):
    g = gen(seed)
    per_seq = max(1, -(-max(max(ctx_lens), 1) // block_size))
    total = batch * per_seq + 3
    q = torch.randn(batch, n_heads, 128, generator=g).bfloat16()
    kc = torch.randn(total, block_size, n_kv, 128, generator=g).to(torch.float8_e4m3fn)
    vc = torch.randn(total, block_size, n_kv, 128, generator=g).to(torch.float8_e4m3fn)
    ids = torch.randperm(total, generator=g)[: batch * per_seq] if shuffle else torch.arange(batch * per_seq)
    bt = ids.to(torch.int32).view(batch, per_seq).contiguous()
    return q, kc, vc, bt, torch.tensor(ctx_lens, dtype=torch.int32)


def _check(q, kc, vc, bt, ctx, scale):
    import hilda_kernel_b200 as hk
    ref16, ref32 = R.paged_attention_decode(q, kc, vc, bt, ctx, scale)
    out = hk.hilda_paged_attention_fp8_decode(q.to(DEV), kc.to(DEV), vc.to(DEV), bt.to(DEV), ctx.to(DEV), scale)
    assert out.dtype == torch.bfloat16 and out.shape == q.shape
    # bf16 outputs: rtol 1.6e-2 / atol 1e-2 against the fp32 evaluation
    torch.testing.assert_close(out.float().cpu(), ref32, rtol=1.6e-2, atol=1e-2)
    # and within one bf16 rounding of the reference's own rounded result nearly everywhere
    assert float((out.float().cpu() - ref16.float()).abs().max()) < 2e-2
    return out


@pytest.mark.parametrize("cfg", [
    (1, 16, 8, [512], 256), (8, 16, 8, [1024] * 8, 256), (4, 16, 8, [4096, 3000, 17, 1], 256),   # bench shapes (:47-49)
    (3, 8, 2, [37, 16, 5], 16), (2, 32, 8, [700, 300], 64), (2, 8, 8, [129, 128], 128), (2, 24, 8, [100, 260], 32),
    (1, 5, 1, [1000], 16), (2, 12, 4, [0, 50], 16), (1, 64, 8, [333], 16),
    (2, 8, 2, [45, 9], 8), (2, 6, 2, [100, 31], 24), (1, 80, 8, [200], 32), (2, 7, 7, [15, 16], 16)])
def test_paged_attention_decode(cfg):
    batch, n_heads, n_kv, ctx, bs = cfg
    q, kc, vc, bt, cl = _inputs(batch, n_heads, n_kv, ctx, bs)
    out = _check(q, kc, vc, bt, cl, 128 ** -0.5)
    for b, c in enumerate(ctx):
        if c == 0:
            assert float(out[b].abs().max()) == 0.0  # an empty context gives zeros, as in the reference kernel


def test_paged_attention_golden_shapes_and_errors(golden):
    import hilda_kernel_b200 as hk
    c = golden["paged_attention_fp8"]
    kc, vc = c["k_cache"].view(torch.float8_e4m3fn), c["v_cache"].view(torch.float8_e4m3fn)
    out = hk.hilda_paged_attention_fp8_decode(c["q"].to(DEV), kc.to(DEV), vc.to(DEV), c["block_tables"].to(DEV),
                                              c["context_lens"].to(DEV), c["scale"])
    assert float((out.float().cpu() - c["out"].float()).abs().max()) < 2e-2
    # [batch, 1, heads, dim] queries keep their shape (paged_attention_fp8.py:94-101, :186-187)
    out4 = hk.hilda_paged_attention_fp8_decode(c["q"].unsqueeze(1).to(DEV), kc.to(DEV), vc.to(DEV),
                                               c["block_tables"].to(DEV), c["context_lens"].to(DEV), c["scale"])
    assert out4.shape == (3, 1, 8, 128) and torch.equal(out4[:, 0], out)
    # the torch evaluation exported beside the kernel agrees with the oracle
    ref = hk.reference_paged_attention_decode(c["q"], kc, vc, c["block_tables"], c["context_lens"], c["scale"])
    assert torch.equal(ref, c["out"])
    # a strided (non-contiguous over heads) query view and an int64 block table are accepted
    qbig = torch.randn(3, 16, 128, generator=gen(5)).bfloat16().to(DEV)
    o2 = hk.hilda_paged_attention_fp8_decode(qbig[:, ::2], kc.to(DEV), vc.to(DEV), c["block_tables"].long().to(DEV),
                                             c["context_lens"].to(DEV), c["scale"])
    o3 = hk.hilda_paged_attention_fp8_decode(qbig[:, ::2].contiguous(), kc.to(DEV), vc.to(DEV),
                                             c["block_tables"].to(DEV), c["context_lens"].to(DEV), c["scale"])
    assert torch.equal(o2, o3)
    with pytest.raises(TypeError):
        hk.hilda_paged_attention_fp8_decode(c["q"].float().to(DEV), kc.to(DEV), vc.to(DEV), c["block_tables"].to(DEV),
                                            c["context_lens"].to(DEV), c["scale"])
    with pytest.raises(ValueError):
        hk.hilda_paged_attention_fp8_decode(c["q"][:, :7].to(DEV), kc.to(DEV), vc.to(DEV), c["block_tables"].to(DEV),
                                            c["context_lens"].to(DEV), c["scale"])
