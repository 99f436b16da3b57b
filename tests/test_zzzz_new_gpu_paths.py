"""GPU tests of paths added after the last run of the suite on hardware (backend selection, the fused SGD kernel,
the relu backward of the linear layer).  They sit in a file that sorts after the others so that, under ``-x``, a
failure here cannot keep the established tests from running."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from fbamtrain_b200.utils.testing import assert_similar  # noqa: E402

DEV = "cuda"
BF = torch.bfloat16


def _nops():
    from fbamtrain_b200.ops import native, native_ops
    return native, native_ops


def test_expected_backends_are_chosen_on_gpu():
    """bf16 CUDA tensors must reach the sm_100a kernels (no silent library fallback), other dtypes the library."""
    _nops()
    from fbamtrain_b200 import ops
    from fbamtrain_b200.ops import dispatch
    x = torch.randn(256, 512, device=DEV).to(BF)
    w = torch.randn(256, 512, device=DEV).to(BF)
    ops.linear(x, w)
    assert dispatch.last_backend("gemm") == "native"
    q, k, v = (torch.randn(2, 128, 2, 64, device=DEV).to(BF) for _ in range(3))
    ops.attention(q, k, v, True)
    assert dispatch.last_backend("mha") == "native"
    img = torch.randn(3, 12, 40, 128, device=DEV).to(BF)
    wt = torch.randn(64, 3, 3, 128, device=DEV).to(BF)
    ops.conv2d_nhwc(img, wt, 1, 1, 1)
    assert dispatch.last_backend("conv2d") == "native"
    ops.linear(x.float(), w.float())
    assert dispatch.last_backend("gemm") == "torch"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("momentum,nesterov", [(0.0, False), (0.9, False), (0.9, True)])
def test_fused_sgd_step_matches_torch_path(dtype, momentum, nesterov):
    _nops()
    from fbamtrain_b200 import ops
    from fbamtrain_b200.optim import SgdOptimizer
    torch.manual_seed(22)
    results = {}
    for backend in ("auto", "torch"):
        p = torch.nn.Parameter(torch.linspace(-1, 1, 1000, device=DEV).to(dtype))
        opt = SgdOptimizer([("w", p)], "optim/t", lr=0.1, momentum=momentum, nesterov=nesterov, weight_decay=0.01)
        ops.set_backend(backend)
        try:
            for k in range(3):
                p.grad = torch.sin(torch.arange(1000, device=DEV) * 0.01 * (k + 1)).to(dtype)
                opt.step()
        finally:
            ops.set_backend("auto")
        results[backend] = (p.detach().float().clone(), {n: t.clone() for n, t in opt.state["w"].items()})
    assert torch.allclose(results["auto"][0], results["torch"][0], atol=1e-6 if dtype == torch.float32 else 1e-2)
    for n, t in results["torch"][1].items():
        assert torch.allclose(results["auto"][1][n], t, atol=1e-5), n


def test_linear_relu_fwd_bwd():
    """``relu(x·Wᵀ + b)``: the epilogue applies the activation, the backward masks by the output's sign."""
    _nops()
    from fbamtrain_b200 import ops
    from fbamtrain_b200.ops import reference as ref
    torch.manual_seed(31)
    x = torch.randn(256, 512, device=DEV).to(BF).requires_grad_(True)
    w = (torch.randn(256, 512, device=DEV) * 0.05).to(BF).requires_grad_(True)
    b = torch.randn(256, device=DEV).to(BF).requires_grad_(True)
    y = ops.linear(x, w, b, "relu")
    g = torch.randn_like(y)
    dx, dw, db = torch.autograd.grad(y, (x, w, b), g)
    xf, wf, bf_ = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yf = ref.linear(xf, wf, bf_, "relu")
    ex, ew, eb = torch.autograd.grad(yf, (xf, wf, bf_), g.float())
    assert_similar(yf.to(BF), y, 3e-2)
    # elements whose pre-activation rounds across zero in bf16 may be masked differently: compare in norm
    for got, exp in ((dx, ex), (dw, ew), (db, eb)):
        assert float((got.float() - exp).norm() / exp.norm()) < 3e-2
