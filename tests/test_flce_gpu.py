"""GPU parity tests of FusedLinearCrossEntropy (tcgen05/TMEM GEMMs + fused online-LSE epilogue)
against the CPU oracle, the golden vectors of hilda-kernel's reference, and torch.matmul for the
GEMM kernel itself. All calls go through the C ABI of libhilda_b200.so."""
import pytest
import torch

from oracle import reference_ops as R
from tests.util import assert_close, assert_loss_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gen(seed):
    return torch.Generator().manual_seed(seed)


def _lib():
    import hilda_kernel_b200._lib as L
    return L


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("mnk", [(128, 256, 64), (300, 520, 200), (1000, 1000, 1000), (129, 264, 72), (64, 8, 4096)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("pair", [0, 7])
def test_tcgen05_gemm_layouts(a_mn, b_mn, mnk, dtype, pair):
    """C = A x B through the tcgen05 kernel for K-major and MN-major operands, ragged sizes; as single
    CTAs (128 x 256 tiles) and as CTA pairs (cta_group::2, 256 x 256 tiles)."""
    L = _lib()
    default = L.lib().hilda_gemm_get_pair()
    L.lib().hilda_gemm_set_pair(pair)
    try:
        _gemm_case(L, a_mn, b_mn, mnk, dtype)
    finally:
        L.lib().hilda_gemm_set_pair(default)


def _gemm_case(L, a_mn, b_mn, mnk, dtype):
    M, N, K = mnk
    if (a_mn and M % 8) or (b_mn and N % 8) or ((not a_mn or not b_mn) and K % 8) or N % 8:
        pytest.skip("TMA row pitches and rows of C must be multiples of 16 bytes")
    g = gen(10)
    A = torch.randn(M, K, generator=g).to(dtype)
    B = torch.randn(N, K, generator=g).to(dtype)
    ref = A.float() @ B.float().T
    Ad = (A.T.contiguous() if a_mn else A).to(DEV)
    Bd = (B.T.contiguous() if b_mn else B).to(DEV)
    C = torch.zeros(M, N, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    rc = L.lib().hilda_debug_gemm(Ad.data_ptr(), Ad.stride(0), Bd.data_ptr(), Bd.stride(0), None, C.data_ptr(), N, M, N, K,
                                  a_mn, b_mn, L.dt(dtype), 0, 0, status.data_ptr(), L.stream(C.device))
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    torch.testing.assert_close(C.cpu(), ref, rtol=1e-4, atol=1e-3 * K ** 0.5)
    if N % 8 == 0:
        C16 = torch.zeros(M, N, dtype=dtype, device=DEV)
        rc = L.lib().hilda_debug_gemm(Ad.data_ptr(), Ad.stride(0), Bd.data_ptr(), Bd.stride(0), C16.data_ptr(), None, N, M, N,
                                      K, a_mn, b_mn, L.dt(dtype), 0, 0, status.data_ptr(), L.stream(C.device))
        assert rc == 0
        assert torch.equal(C16.cpu(), ref.to(dtype)) or float((C16.cpu().float() - ref).abs().max()) < 0.02 * K ** 0.5


def _flce_inputs(BT, H, V, dtype, ignore_frac=0.05, seed=11):
    g = gen(seed)
    hidden = torch.randn(BT, H, generator=g).to(dtype)
    weight = (0.02 * torch.randn(V, H, generator=g)).to(dtype)
    targets = torch.randint(0, V, (BT,), generator=g)
    n_ign = int(round(ignore_frac * BT))
    if n_ign:
        targets[torch.randperm(BT, generator=g)[:n_ign]] = -100
    return hidden, weight, targets


def _oracle_grads(hidden, weight, targets, reduction):
    """fp32 autograd of the PyTorch reference on the (already rounded) 16-bit inputs, with the
    logits rounded to the compute dtype as the reference's GEMM does."""
    h, w = hidden.float().clone().requires_grad_(True), weight.float().clone().requires_grad_(True)
    logits = h @ w.T
    logits = logits + (logits.to(hidden.dtype).float() - logits).detach()  # straight-through rounding
    per_row = torch.nn.functional.cross_entropy(logits, targets, ignore_index=-100, reduction="none")
    n_valid = max(int((targets != -100).sum()), 1)
    loss = per_row.sum() / n_valid if reduction == "mean" else per_row.sum()
    loss.backward()
    return loss.detach(), per_row.detach(), h.grad, w.grad


@pytest.mark.parametrize("shape", [(300, 256, 1000), (512, 512, 4096), (1000, 128, 32000), (130, 64, 520),
                                   (257, 4096, 1536), (64, 256, 50257)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("chunk", [None, 128])
def test_flce_fwd_bwd(shape, dtype, chunk):
    import hilda_kernel_b200 as hk
    from hilda_kernel_b200.kernels import fused_linear_cross_entropy as F
    BT, H, V = shape
    if dtype == torch.float16 and V >= 32000:
        # dlogits ~ 1/(V * n_valid) ~ 3e-8 is below fp16's smallest subnormal (6e-8): the 16-bit
        # dlogits buffer (which the reference has too) underflows, so there is nothing to compare
        pytest.skip("fp16 dlogits underflow at this vocabulary size")
    hidden, weight, targets = _flce_inputs(BT, H, V, dtype)
    loss_ref, rows_ref, dh_ref, dw_ref = _oracle_grads(hidden, weight, targets, "mean")
    F.CHUNK_ROWS, F.CHECK_STATUS = chunk, True
    try:
        hd, wd = hidden.to(DEV).requires_grad_(True), weight.to(DEV).requires_grad_(True)
        loss = hk.hilda_fused_linear_cross_entropy(hd, wd, targets.to(DEV), -100, "mean")
        assert loss.dtype == torch.float32
        loss.backward()
        # no-grad forward and reduction='none'
        with torch.no_grad():
            rows = hk.hilda_fused_linear_cross_entropy(hidden.to(DEV), weight.to(DEV), targets.to(DEV), -100, "none")
            lsum = hk.hilda_fused_linear_cross_entropy(hidden.to(DEV), weight.to(DEV), targets.to(DEV), -100, "sum")
    finally:
        F.CHUNK_ROWS, F.CHECK_STATUS = None, False
    # the fp32 chunked oracle (logits not rounded) bounds the effect of the 16-bit logits rounding
    loss_fp32 = R.linear_cross_entropy_fp32_chunked(hidden, weight, targets)
    assert abs(float(loss) - float(loss_fp32)) < 2e-3 * max(1.0, abs(float(loss_fp32)))
    assert_loss_close(loss, loss_ref)
    assert_loss_close(lsum, rows_ref.sum(), "sum")
    # a logit that sits on a rounding boundary of the 16-bit logits may round the other way (the
    # fp32 accumulation order differs), which moves that row's loss by one 16-bit ulp of the logit
    ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    diff = (rows.cpu() - rows_ref).abs()
    assert float(diff.max()) <= 4 * ulp * 4.0 and float(diff.mean()) < 1e-4, (float(diff.max()), float(diff.mean()))
    assert hd.grad.dtype == dtype and wd.grad.dtype == dtype
    assert_close(hd.grad, dh_ref, dtype, what="d hidden", normalize=True)
    assert_close(wd.grad, dw_ref, dtype, what="d weight", normalize=True)
    ign = (targets == -100)
    if ign.any():
        assert float(hd.grad[ign.to(DEV)].abs().max()) == 0.0  # ignored tokens get no gradient


def test_flce_cta_pair_mode_matches_single_cta():
    """The whole operator with the GEMMs run as CTA pairs gives the same loss and gradients."""
    L = _lib()
    from hilda_kernel_b200.kernels.fused_linear_cross_entropy import fused_linear_cross_entropy_forward
    hidden, weight, targets = _flce_inputs(700, 512, 3000, torch.bfloat16)
    hd, wd, td = hidden.to(DEV), weight.to(DEV), targets.to(DEV)
    default = L.lib().hilda_gemm_get_pair()
    L.lib().hilda_gemm_set_pair(0)
    try:
        l0, dh0, dw0, _ = fused_linear_cross_entropy_forward(hd, wd, td, chunk_rows=256)
        L.lib().hilda_gemm_set_pair(7)
        l1, dh1, dw1, _ = fused_linear_cross_entropy_forward(hd, wd, td, chunk_rows=256)
        torch.cuda.synchronize()
    finally:
        L.lib().hilda_gemm_set_pair(default)
    assert_loss_close(l1, l0)
    assert_close(dh1, dh0.float(), torch.bfloat16, what="d hidden", normalize=True)
    assert_close(dw1, dw0.float(), torch.bfloat16, what="d weight", normalize=True)


def test_flce_skip_ignored_rows_matches_full_path():
    """Compacting ignored tokens away before the GEMMs changes nothing but the time."""
    from hilda_kernel_b200.kernels.fused_linear_cross_entropy import fused_linear_cross_entropy_forward
    for frac in (0.0, 0.3, 1.0):
        hidden, weight, targets = _flce_inputs(600, 256, 2000, torch.bfloat16, ignore_frac=frac)
        hd, wd, td = hidden.to(DEV), weight.to(DEV), targets.to(DEV)
        for red in ("mean", "sum", "none"):
            l0, dh0, dw0, n0 = fused_linear_cross_entropy_forward(hd, wd, td, reduction=red, skip_ignored=False)
            l1, dh1, dw1, n1 = fused_linear_cross_entropy_forward(hd, wd, td, reduction=red, skip_ignored=True)
            assert int(n0) == int(n1) == int((targets != -100).sum())
            torch.testing.assert_close(l1, l0, rtol=1e-5, atol=1e-6)
            assert_close(dh1, dh0.float(), torch.bfloat16, what="d hidden", normalize=frac < 1.0)
            assert_close(dw1, dw0.float(), torch.bfloat16, what="d weight", normalize=frac < 1.0)
            if frac > 0:
                assert float(dh1[(targets == -100).to(DEV)].abs().max()) == 0.0


def test_flce_golden_and_upstream_scale(golden):
    import hilda_kernel_b200 as hk
    c = golden["linear_ce_f32"]  # fp32 reference output; inputs rounded to bf16 for the tensor-core path
    hidden, weight = c["hidden"].bfloat16(), c["weight"].bfloat16()
    loss_ref, _, dh_ref, dw_ref = _oracle_grads(hidden, weight, c["targets"], "mean")
    assert abs(float(loss_ref) - float(c["loss"])) < 1e-2  # bf16 inputs move the fp32 golden loss only slightly
    hd, wd = hidden.to(DEV).requires_grad_(True), weight.to(DEV).requires_grad_(True)
    loss = hk.FusedLinearCrossEntropyLoss()(hd, wd, c["targets"].to(DEV))
    (loss * 0.5).backward()
    assert_loss_close(loss, loss_ref)
    assert_close(hd.grad, 0.5 * dh_ref, torch.bfloat16, what="d hidden", normalize=True)
    assert_close(wd.grad, 0.5 * dw_ref, torch.bfloat16, what="d weight", normalize=True)
    assert float((hd.grad.float().cpu() - 0.5 * c["dh"]).abs().max()) < 5e-2   # bench_fused_linear_ce.py thresholds
    assert float((wd.grad.float().cpu() - 0.5 * c["dw"]).abs().max()) < 5e-1
    with pytest.raises(TypeError):
        hk.hilda_fused_linear_cross_entropy(c["hidden"].to(DEV), c["weight"].to(DEV), c["targets"].to(DEV))
    # every target ignored: loss 0 (clamp), zero grads
    t = torch.full_like(c["targets"], -100).to(DEV)
    hd2, wd2 = hidden.to(DEV).requires_grad_(True), weight.to(DEV).requires_grad_(True)
    l2 = hk.hilda_fused_linear_cross_entropy(hd2, wd2, t)
    l2.backward()
    assert float(l2) == 0.0 and float(hd2.grad.abs().max()) == 0.0 and float(wd2.grad.abs().max()) == 0.0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_flce_vocab_parallel_steps_single_gpu(world):
    """The vocab-parallel step API with the ranks emulated one after another on one GPU: shard W by
    rows, combine the per-row (max, sum-exp, target logit) triples as the NCCL path does, and
    compare with the single-shard operator (V/world is not a multiple of the 256-column tile)."""
    import hilda_kernel_b200._lib as L
    from hilda_kernel_b200.kernels.fused_linear_cross_entropy import fused_linear_cross_entropy_forward
    from hilda_kernel_b200.parallel import combine_rowstats, shard_bounds
    BT, H, V, dtype = 384, 256, 4008, torch.bfloat16
    hidden, weight, targets = _flce_inputs(BT, H, V, dtype)
    hd, wd, td = hidden.to(DEV), weight.to(DEV), targets.to(DEV)
    loss1, dh1, dw1, _ = fused_linear_cross_entropy_forward(hd, wd, td)
    lib, st = L.lib(), L.stream(hd.device)
    head = torch.zeros(2, dtype=torch.int32, device=DEV)
    lib.hilda_count_valid(td.data_ptr(), BT, -100, head.data_ptr() + 4, st)
    shards = []
    for r in range(world):
        v0, v1 = shard_bounds(V, world, r, 8)
        Vl = v1 - v0
        ws = wd[v0:v1].contiguous()
        scratch = torch.empty(lib.hilda_flce_padded_rows(BT) * lib.hilda_flce_logits_pitch(Vl), dtype=dtype, device=DEV)
        stats = torch.empty(BT * lib.hilda_flce_stat_tiles(Vl) * 2, dtype=torch.float32, device=DEV)
        rowstat = torch.empty(3, BT, dtype=torch.float32, device=DEV)
        assert lib.hilda_flce_logits(hd.data_ptr(), ws.data_ptr(), scratch.data_ptr(), stats.data_ptr(), BT, H, Vl, 1,
                                     head.data_ptr(), st) == 0
        assert lib.hilda_flce_row_stats(stats.data_ptr(), scratch.data_ptr(), td.data_ptr(), rowstat.data_ptr(), BT, Vl,
                                        v0, 1, st) == 0
        shards.append((v0, Vl, ws, scratch, rowstat))
    rs = combine_rowstats(torch.stack([s[4] for s in shards])).contiguous()
    lse = torch.empty(BT, dtype=torch.float32, device=DEV)
    loss_rows = torch.empty(BT, dtype=torch.float32, device=DEV)
    assert lib.hilda_flce_finalize(rs.data_ptr(), td.data_ptr(), -100, lse.data_ptr(), loss_rows.data_ptr(), BT, st) == 0
    dh = torch.zeros(BT, H, dtype=torch.float32, device=DEV)
    dws = []
    for v0, Vl, ws, scratch, _ in shards:
        assert lib.hilda_flce_dlogits(scratch.data_ptr(), lse.data_ptr(), td.data_ptr(), -100, head.data_ptr() + 4, BT,
                                      Vl, v0, 1, st) == 0
        part = torch.empty(BT, H, dtype=torch.float32, device=DEV)
        assert lib.hilda_flce_grad_hidden(scratch.data_ptr(), ws.data_ptr(), None, part.data_ptr(), BT, H, Vl, 1,
                                          head.data_ptr(), st) == 0
        dh += part
        dw = torch.empty(Vl, H, dtype=dtype, device=DEV)
        assert lib.hilda_flce_grad_weight(scratch.data_ptr(), hd.data_ptr(), None, dw.data_ptr(), 3, BT, H, Vl, 1,
                                          head.data_ptr(), st) == 0
        dws.append(dw)
    torch.cuda.synchronize()
    assert int(head[0]) == 0
    n_valid = int(head[1])
    assert n_valid == int((targets != -100).sum())
    assert_loss_close(loss_rows.sum() / n_valid, loss1)
    assert_close(dh, dh1.float(), torch.bfloat16, what="d hidden", normalize=True)
    assert_close(torch.cat(dws), dw1, torch.bfloat16, what="d weight", normalize=True)
