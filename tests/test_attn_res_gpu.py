"""GPU parity tests of AttnRes against the CPU oracle (oracle/reference_ops.py, the reference's
pytorch_attn_res) on identical seeded inputs, and against the golden outputs of that function."""
import pytest
import torch

from oracle import reference_ops as R
from tests.util import assert_close

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(params=[0, 1], ids=["cuda_core", "tensor_core"], autouse=True)
def kernel_path(request):
    """Every test runs with both sets of kernels (hilda_attn_res_set_path: the reductions over D on
    the CUDA cores or on the tensor cores); shapes and dtypes the tensor-core kernels do not take
    fall back to the others inside the library."""
    import hilda_kernel_b200._lib as L
    old = L.lib().hilda_attn_res_set_path(request.param)
    yield request.param
    L.lib().hilda_attn_res_set_path(old)


def gen(seed):
    return torch.Generator().manual_seed(seed)


def _oracle(V, wq, wn, dh):
    """fp32 autograd of the reference on the (already rounded) inputs, with the reference's own
    rounding of the normalised keys to the data dtype."""
    v = V.float().clone().requires_grad_(True)
    q = wq.float().clone().requires_grad_(True)
    n = wn.float().clone().requires_grad_(True)
    rms = torch.sqrt(v.pow(2).mean(dim=-1, keepdim=True) + 1e-6)
    kn = v / rms
    kn = kn + (kn.to(V.dtype).float() - kn).detach()          # .to(V.dtype), straight-through
    K = kn * n
    K = K + (K.to(V.dtype).float() - K).detach()              # the 16-bit product
    scores = torch.einsum('d, n b t d -> n b t', q, K)
    alpha = scores.softmax(dim=0)
    h = torch.einsum('n b t, n b t d -> b t d', alpha, v)
    h.backward(dh.float())
    return h.detach(), v.grad, q.grad, n.grad, alpha.detach()


@pytest.mark.parametrize("dims", [(4, 2, 64, 4096), (8, 2, 64, 4096), (8, 1, 40, 8192), (16, 2, 9, 4096), (32, 1, 5, 1024),
                                  (1, 2, 3, 512), (5, 2, 7, 256), (3, 1, 4, 100), (6, 2, 5, 33), (7, 1, 3, 20000), (8, 1, 300, 2048), (3, 2, 50, 1600)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_attn_res_fwd_bwd(dims, dtype):
    import hilda_kernel_b200 as hk
    N, B, T, D = dims
    g = gen(41)
    V = torch.randn(N, B, T, D, generator=g).to(dtype)
    # a query large enough that the softmax over blocks is far from uniform
    wq = (0.3 * torch.randn(D, generator=g) / D ** 0.5 * 8).to(dtype)
    wn = (1 + 0.1 * torch.randn(D, generator=g)).to(dtype)
    dh = torch.randn(B, T, D, generator=g).to(dtype)
    h_ref, dv_ref, dq_ref, dn_ref, alpha_ref = _oracle(V, wq, wn, dh)
    vd, qd, nd = (x.to(DEV).requires_grad_(True) for x in (V, wq, wn))
    h = hk.hilda_attn_res(vd, qd, nd)
    assert h.shape == (B, T, D) and h.dtype == dtype
    h.backward(dh.to(DEV))
    assert_close(h, h_ref, dtype, what="h")
    assert vd.grad.shape == V.shape and vd.grad.dtype == dtype
    assert_close(vd.grad, dv_ref, dtype, what="dV")
    assert_close(qd.grad, dq_ref, dtype, what="dW_query", normalize=True)
    assert_close(nd.grad, dn_ref, dtype, what="dW_norm", normalize=True)
    # the saved softmax weights sum to one over the blocks and match the oracle
    from hilda_kernel_b200.kernels.attn_res import attn_res_forward
    _, _, alpha, rstd = attn_res_forward(V.to(DEV), wq.to(DEV), wn.to(DEV))
    assert float((alpha.sum(0) - 1).abs().max()) < 1e-5
    assert float((alpha.cpu() - alpha_ref.reshape(N, -1)).abs().max()) < (2e-2 if dtype != torch.float32 else 1e-5)


def test_attn_res_golden_list_input_and_determinism(golden):
    import hilda_kernel_b200 as hk
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        c = golden[f"attn_res_{tag}"]
        vd, qd, nd = (c[k].to(DEV).requires_grad_(True) for k in ("V", "wq", "wn"))
        mod = hk.AttnRes(c["V"].shape[-1]).to(DEV)
        with torch.no_grad():
            mod.w_query.copy_(c["wq"].float()); mod.w_norm.copy_(c["wn"].float())
        h = hk.hilda_attn_res(vd, qd, nd)
        h.backward(c["dh"].to(DEV))
        assert_close(h, c["h"], dtype, what="h")
        assert_close(vd.grad, c["dV"], dtype, what="dV")
        assert_close(qd.grad, c["dwq"], dtype, what="dW_query", normalize=True)
        assert_close(nd.grad, c["dwn"], dtype, what="dW_norm", normalize=True)
        # a list of blocks is stacked like the reference does (attn_res.py:226-229)
        h2 = hk.hilda_attn_res([b for b in c["V"].to(DEV)], c["wq"].to(DEV), c["wn"].to(DEV))
        assert torch.equal(h2, h.detach())
        # the module holds fp32 parameters over 16-bit data
        h3 = mod(c["V"].to(DEV))
        assert h3.dtype == dtype and h3.shape == h.shape
        # weight gradients are bit-reproducible (fixed-order sums, no atomics)
        v2, q2, n2 = (c[k].to(DEV).requires_grad_(True) for k in ("V", "wq", "wn"))
        hk.hilda_attn_res(v2, q2, n2).backward(c["dh"].to(DEV))
        assert torch.equal(q2.grad, qd.grad) and torch.equal(n2.grad, nd.grad)
