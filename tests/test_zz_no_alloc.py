"""GPU test of hilda_norm_bwd_noalloc, the one entry point that brings its own scratch memory.

It exists for hosts that have no workspace to pass: a plain C/FFI caller without an allocator, or
a server that gave the whole device to its own memory pool and may not call cudaMalloc any more.
The test calls it through the C ABI twice in a row (the second time on different data and a
different shape, so anything left in the shared scratch array by the first call would show) and
requires bit-identical results to hilda_norm_bwd with a caller-supplied workspace (dW within the
tolerance of the other tests where the built-in array forces a smaller grid), and checks that a
call changes neither the driver's free memory nor torch's allocation count. This file is named so
that pytest collects it last."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _run_pair(L, n_rows, n_cols, dtype, seed, with_ds, same_grid=True):
    lib = L.lib()
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n_rows, n_cols, generator=g).to(dtype).to(DEV)
    dy = torch.randn(n_rows, n_cols, generator=g).to(dtype).to(DEV)
    ds = torch.randn(n_rows, n_cols, generator=g).to(dtype).to(DEV) if with_ds else None
    w = (1 + 0.1 * torch.randn(n_cols, generator=g)).to(dtype).to(DEV)
    y = torch.empty_like(x)
    rstd = torch.empty(n_rows, dtype=torch.float32, device=DEV)
    st = L.stream(x.device)
    assert lib.hilda_rms_norm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), n_rows, n_cols, 1e-6,
                                  L.dt(x), L.dt(w), st) == 0
    # existing entry point, caller-owned workspace
    ws = torch.empty(lib.hilda_norm_bwd_workspace_bytes(n_rows, n_cols, L.dt(x)) // 4, dtype=torch.float32, device=DEV)
    dx_a, dw_a = torch.empty_like(x), torch.empty_like(w)
    assert lib.hilda_norm_bwd(dy.data_ptr(), L.ptr(ds), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx_a.data_ptr(),
                              dw_a.data_ptr(), ws.data_ptr(), n_rows, n_cols, L.dt(x), L.dt(w), st) == 0
    # the entry point under test: no workspace argument
    dx_b, dw_b = torch.empty_like(x), torch.empty_like(w)
    assert lib.hilda_norm_bwd_noalloc(dy.data_ptr(), L.ptr(ds), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                      dx_b.data_ptr(), dw_b.data_ptr(), n_rows, n_cols, L.dt(x), L.dt(w), st) == 0
    torch.cuda.synchronize()
    # the entry point's one promise: it takes no device memory, neither from the driver nor from torch
    free0, alloc0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    assert lib.hilda_norm_bwd_noalloc(dy.data_ptr(), L.ptr(ds), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                      dx_b.data_ptr(), dw_b.data_ptr(), n_rows, n_cols, L.dt(x), L.dt(w), st) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_allocated() == alloc0
    assert torch.equal(dx_a, dx_b), "dx differs"
    if same_grid:
        assert torch.equal(dw_a, dw_b), "dw differs"
    else:
        # fewer CTAs than the workspace version: the partial sums are grouped differently
        tol = dict(rtol=1e-5, atol=1e-4) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1e-2 * n_rows ** 0.5)
        torch.testing.assert_close(dw_b.float(), dw_a.float(), **tol)
    assert bool(torch.isfinite(dw_b.float()).all())


def test_norm_bwd_noalloc_matches_workspace_version_twice():
    import hilda_kernel_b200._lib as L
    _run_pair(L, 3000, 4096, torch.bfloat16, seed=21, with_ds=False)
    _run_pair(L, 777, 2048, torch.float32, seed=22, with_ds=True)   # second call: other shape, dtype and data
    _run_pair(L, 3000, 4096, torch.bfloat16, seed=23, with_ds=True)


def test_norm_bwd_noalloc_uses_a_smaller_grid_when_the_default_one_does_not_fit():
    """Hidden size 8192 in bf16: the default plan wants more partial rows than the 16 MiB array holds,
    so fewer CTAs run. dX must not change at all, dW only by the summation grouping."""
    import hilda_kernel_b200._lib as L
    lib = L.lib()
    n_rows, n_cols = 6000, 8192
    grouped = lib.hilda_norm_bwd_workspace_bytes(n_rows, n_cols, 1) > lib.hilda_norm_bwd_noalloc_max_bytes()
    _run_pair(L, n_rows, n_cols, torch.bfloat16, seed=31, with_ds=True, same_grid=not grouped)
    _run_pair(L, 5000, 16384, torch.float32, seed=32, with_ds=False, same_grid=False)


def test_norm_bwd_noalloc_rejects_only_a_row_longer_than_the_array():
    import hilda_kernel_b200._lib as L
    lib = L.lib()
    cap = lib.hilda_norm_bwd_noalloc_max_bytes()
    assert cap == 16 * 1024 * 1024
    n_rows, n_cols = 4, cap // 4 + 8   # one partial row alone exceeds the built-in array
    one = torch.zeros(8, device=DEV)
    rc = lib.hilda_norm_bwd_noalloc(one.data_ptr(), None, one.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(),
                                    one.data_ptr(), n_rows, n_cols, 0, 0, L.stream(one.device))
    assert rc == -3  # HILDA_ERR_SIZE, nothing launched
