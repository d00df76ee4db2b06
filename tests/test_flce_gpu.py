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
@pytest.mark.parametrize("compact", [False, True])
def test_flce_vocab_parallel_steps_single_gpu(world, compact):
    """The vocab-parallel step API with the ranks emulated one after another on one GPU: shard W by
    rows, merge the per-row (max, sum-exp, target logit) triples as the NCCL path does (the gathered
    [world, 3, rows] buffer goes straight into the finalize kernel), and compare with the
    single-shard operator (V/world is not a multiple of the 256-column tile). With `compact` the
    ignored rows are dropped by the device-side index lists and every step follows the device-side
    row count, exactly the sequence VocabParallelFLCE issues."""
    import hilda_kernel_b200._lib as L
    from hilda_kernel_b200.kernels.fused_linear_cross_entropy import fused_linear_cross_entropy_forward
    from hilda_kernel_b200.parallel import combine_rowstats, shard_bounds
    # 640 rows, 448 of them valid when compacting: rows 512.. of the compacted buffers are never touched
    BT, H, V, dtype = 640, 256, 4008, torch.bfloat16
    hidden, weight, targets = _flce_inputs(BT, H, V, dtype, ignore_frac=0.3 if compact else 0.05)
    hd, wd, td = hidden.to(DEV), weight.to(DEV), targets.to(DEV)
    loss1, dh1, dw1, _ = fused_linear_cross_entropy_forward(hd, wd, td, skip_ignored=False)
    lib, st = L.lib(), L.stream(hd.device)
    head = torch.zeros(2, dtype=torch.int32, device=DEV)
    nv_p = head.data_ptr() + 4
    dyn = None
    h_use, t_use = hd, td
    if compact:
        idx = torch.empty(BT, dtype=torch.int64, device=DEV)
        inv = torch.empty(BT, dtype=torch.int32, device=DEV)
        t_use = torch.empty(BT, dtype=torch.int64, device=DEV)
        h_use = torch.full_like(hd, float("nan"))  # whatever is not gathered or cleared must never be read
        assert lib.hilda_flce_compact(td.data_ptr(), BT, -100, idx.data_ptr(), inv.data_ptr(), t_use.data_ptr(), nv_p, st) == 0
        assert lib.hilda_gather_valid_rows(hd.data_ptr(), idx.data_ptr(), nv_p, h_use.data_ptr(), BT, H * 2, st) == 0
        keep = (targets != -100).nonzero().squeeze(1)
        assert torch.equal(idx.cpu()[:keep.numel()], keep) and bool((idx.cpu()[keep.numel():] == -1).all())
        assert torch.equal(t_use.cpu()[:keep.numel()], targets[keep]) and bool((t_use.cpu()[keep.numel():] == -100).all())
        assert torch.equal(h_use.cpu()[:keep.numel()], hidden[keep])
        dyn = nv_p
    else:
        lib.hilda_count_valid(td.data_ptr(), BT, -100, nv_p, st)
    shards = []
    for r in range(world):
        v0, v1 = shard_bounds(V, world, r, 8)
        Vl = v1 - v0
        ws = wd[v0:v1].contiguous()
        scratch = torch.empty(lib.hilda_flce_padded_rows(BT) * lib.hilda_flce_logits_pitch(Vl), dtype=dtype, device=DEV)
        stats = torch.empty(BT * lib.hilda_flce_stat_tiles(Vl) * 2, dtype=torch.float32, device=DEV)
        rowstat = torch.zeros(3, BT, dtype=torch.float32, device=DEV)
        assert lib.hilda_flce_logits(h_use.data_ptr(), ws.data_ptr(), scratch.data_ptr(), stats.data_ptr(), BT, H, Vl, 1,
                                     head.data_ptr(), dyn, 0, st) == 0
        assert lib.hilda_flce_row_stats(stats.data_ptr(), scratch.data_ptr(), t_use.data_ptr(), rowstat.data_ptr(), BT, Vl,
                                        v0, 1, dyn, 0, st) == 0
        shards.append((v0, Vl, ws, scratch, rowstat))
    gathered = torch.stack([s[4] for s in shards]).contiguous()  # [world, 3, BT], as all_gather_into_tensor fills it
    lse = torch.empty(BT, dtype=torch.float32, device=DEV)
    loss_rows = torch.empty(BT, dtype=torch.float32, device=DEV)
    assert lib.hilda_flce_finalize(gathered.data_ptr(), world, t_use.data_ptr(), -100, lse.data_ptr(), loss_rows.data_ptr(),
                                   BT, dyn, 0, st) == 0
    # the host-side merge (pure torch, also covered on CPU) and the in-kernel merge agree
    rs = combine_rowstats(gathered).contiguous()
    lse2, loss_rows2 = torch.empty_like(lse), torch.empty_like(loss_rows)
    assert lib.hilda_flce_finalize(rs.data_ptr(), 1, t_use.data_ptr(), -100, lse2.data_ptr(), loss_rows2.data_ptr(), BT,
                                   dyn, 0, st) == 0
    n_live = int((targets != -100).sum()) if compact else BT
    torch.testing.assert_close(loss_rows[:n_live], loss_rows2[:n_live], rtol=1e-6, atol=1e-6)
    dh = torch.zeros(BT, H, dtype=torch.float32, device=DEV)
    dws = []
    for v0, Vl, ws, scratch, _ in shards:
        assert lib.hilda_flce_dlogits(scratch.data_ptr(), lse.data_ptr(), t_use.data_ptr(), -100, nv_p, BT,
                                      Vl, v0, 1, dyn, 0, st) == 0
        part = torch.zeros(BT, H, dtype=torch.float32, device=DEV)
        assert lib.hilda_flce_grad_hidden(scratch.data_ptr(), ws.data_ptr(), None, part.data_ptr(), BT, H, Vl, 1,
                                          head.data_ptr(), dyn, 0, st) == 0
        dh += part
        dw = torch.empty(Vl, H, dtype=dtype, device=DEV)
        assert lib.hilda_flce_grad_weight(scratch.data_ptr(), h_use.data_ptr(), None, dw.data_ptr(), 3, BT, H, Vl, 1,
                                          head.data_ptr(), dyn, 0, st) == 0
        dws.append(dw)
    loss = torch.empty((), dtype=torch.float32, device=DEV)
    assert lib.hilda_flce_sum_loss(loss_rows.data_ptr(), BT, nv_p, 1, head.data_ptr(), loss.data_ptr(), st) == 0
    if compact:
        dh16 = dh.to(dtype)
        dh_full = torch.empty_like(dh16)
        assert lib.hilda_scatter_valid_rows(dh16.data_ptr(), inv.data_ptr(), dh_full.data_ptr(), BT, H * 2, st) == 0
        dh = dh_full.float()
        assert float(dh[(targets == -100).to(DEV)].abs().max()) == 0.0
    torch.cuda.synchronize()
    assert int(head[0]) == 0
    n_valid = int(head[1])
    assert n_valid == int((targets != -100).sum())
    assert_loss_close(loss, loss1)
    assert_close(dh, dh1.float(), torch.bfloat16, what="d hidden", normalize=True)
    assert_close(torch.cat(dws), dw1, torch.bfloat16, what="d weight", normalize=True)


def test_flce_device_side_compaction_edge_counts():
    """The device-side row count at its edges through the single-device operator with several row
    chunks: nothing ignored, everything ignored, a count that ends exactly on a chunk boundary and
    one that leaves whole trailing chunks empty (their d(W) passes add zero)."""
    from hilda_kernel_b200.kernels.fused_linear_cross_entropy import fused_linear_cross_entropy_forward
    BT, H, V = 1024, 128, 1536
    g = gen(21)
    hidden = torch.randn(BT, H, generator=g).bfloat16()
    weight = (0.05 * torch.randn(V, H, generator=g)).bfloat16()
    base = torch.randint(0, V, (BT,), generator=g)
    for n_valid in (BT, 0, 512, 256, 100, 1):
        targets = torch.full((BT,), -100, dtype=torch.int64)
        pick = torch.randperm(BT, generator=g)[:n_valid]
        targets[pick] = base[pick]
        hd, wd, td = hidden.to(DEV), weight.to(DEV), targets.to(DEV)
        for red in ("mean", "none"):
            l0, dh0, dw0, n0 = fused_linear_cross_entropy_forward(hd, wd, td, reduction=red, chunk_rows=256, skip_ignored=False)
            l1, dh1, dw1, n1 = fused_linear_cross_entropy_forward(hd, wd, td, reduction=red, chunk_rows=256, skip_ignored=True)
            assert int(n0) == int(n1) == n_valid
            torch.testing.assert_close(l1, l0, rtol=1e-5, atol=1e-6)
            assert_close(dh1, dh0.float(), torch.bfloat16, what=f"d hidden n_valid={n_valid}", normalize=n_valid > 0)
            assert_close(dw1, dw0.float(), torch.bfloat16, what=f"d weight n_valid={n_valid}", normalize=n_valid > 0)
            assert bool(torch.isfinite(dh1.float()).all()) and bool(torch.isfinite(dw1.float()).all())


def test_flce_makes_no_host_synchronisation():
    """The default path (ignored rows compacted away) only enqueues work: under
    torch.cuda.set_sync_debug_mode('error') any host synchronisation inside the call raises."""
    from hilda_kernel_b200.kernels.fused_linear_cross_entropy import fused_linear_cross_entropy_forward
    hidden, weight, targets = _flce_inputs(600, 256, 2000, torch.bfloat16, ignore_frac=0.2)
    hd, wd, td = hidden.to(DEV), weight.to(DEV), targets.to(DEV)
    fused_linear_cross_entropy_forward(hd, wd, td)  # loads the library, creates the caches
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        loss, dh, dw, n_valid = fused_linear_cross_entropy_forward(hd, wd, td)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    loss_ref, _, dh_ref, dw_ref = _oracle_grads(hidden, weight, targets, "mean")
    assert_loss_close(loss, loss_ref)
    assert_close(dh, dh_ref, torch.bfloat16, what="d hidden", normalize=True)


def test_gemm_bounded_wait_expires_and_the_next_call_is_fine():
    """Failure detection without a fault: a host-set hook makes the TMA producers withhold their
    signals and shortens the wait limit, so every bounded mbarrier wait of the GEMM runs out within
    microseconds. The launch must return, the status word must carry a code, the operator's loss must
    be NaN instead of a plausible number, and the next ordinary call must be correct."""
    L = _lib()
    lib = L.lib()
    from hilda_kernel_b200.kernels import fused_linear_cross_entropy as F
    M, N, K = 512, 512, 1024
    g = gen(5)
    A, B = torch.randn(M, K, generator=g).bfloat16().to(DEV), torch.randn(N, K, generator=g).bfloat16().to(DEV)
    C = torch.zeros(M, N, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    hidden, weight, targets = _flce_inputs(300, 256, 1000, torch.bfloat16)
    hd, wd, td = hidden.to(DEV), weight.to(DEV), targets.to(DEV)
    default_pair = lib.hilda_gemm_get_pair()
    for pair in (7, 0):
        lib.hilda_gemm_set_pair(pair)
        lib.hilda_gemm_set_wait_cap(2048)
        lib.hilda_gemm_set_probe(None, 2)
        try:
            status.zero_()
            rc = lib.hilda_debug_gemm(A.data_ptr(), K, B.data_ptr(), K, None, C.data_ptr(), N, M, N, K, 0, 0, 1, 0, 0,
                                      status.data_ptr(), L.stream(C.device))
            assert rc == 0
            torch.cuda.synchronize()  # returns: nothing hangs, the context stays usable
            assert int(status[0]) != 0
            loss, _, _, _ = F.fused_linear_cross_entropy_forward(hd, wd, td)
            assert bool(torch.isnan(loss))
            F.CHECK_STATUS = True
            with pytest.raises(RuntimeError, match="device status"):
                F.fused_linear_cross_entropy_forward(hd, wd, td)
        finally:
            F.CHECK_STATUS = False
            lib.hilda_gemm_set_probe(None, 0)
            lib.hilda_gemm_set_wait_cap(0)
            lib.hilda_gemm_set_pair(default_pair)
        # the ordinary path right after
        lib.hilda_gemm_set_pair(pair)
        try:
            status.zero_()
            rc = lib.hilda_debug_gemm(A.data_ptr(), K, B.data_ptr(), K, None, C.data_ptr(), N, M, N, K, 0, 0, 1, 0, 0,
                                      status.data_ptr(), L.stream(C.device))
            assert rc == 0
            torch.cuda.synchronize()
            assert int(status[0]) == 0
            torch.testing.assert_close(C, A.float() @ B.float().T, rtol=1e-4, atol=1e-3 * K ** 0.5)
            loss, _, _, _ = F.fused_linear_cross_entropy_forward(hd, wd, td)
            assert_loss_close(loss, _oracle_grads(hidden, weight, targets, "mean")[0])
        finally:
            lib.hilda_gemm_set_pair(default_pair)
