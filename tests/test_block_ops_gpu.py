"""tmw_add_rmsnorm (residual add + RMSNorm in one pass) against the reference's formula in fp32
(titans_core/blocks/norms.py:55-58: ``x / sqrt(mean(x^2) + eps) * scale``)."""

import pytest
import torch

from titanmac_b200 import RMSNorm, _native

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 4e-3}


def reference(x, residual, scale, eps, dtype):
    h = x.float() if residual is None else (x.float() + residual.float()).to(dtype).float()
    rms = torch.sqrt(torch.mean(h ** 2, dim=-1, keepdim=True) + eps)
    return h, h / rms * scale.float()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,dim", [(1, 64), (257, 640), (33, 1024), (19, 2048), (5, 4096), (0, 128)])
@pytest.mark.parametrize("with_residual", [False, True])
def test_add_rmsnorm(dtype, rows, dim, with_residual):
    g = torch.Generator().manual_seed(rows * 131 + dim)
    x = torch.randn(rows, dim, generator=g).to(dtype).to(DEV)
    r = torch.randn(rows, dim, generator=g).to(dtype).to(DEV) if with_residual else None
    scale = (1 + 0.1 * torch.randn(dim, generator=g)).to(dtype).to(DEV)
    h, y = _native.add_rmsnorm(x, r, scale, 1e-5)
    h_ref, y_ref = reference(x, r, scale, 1e-5, dtype)
    assert h.shape == x.shape and y.shape == x.shape and y.dtype == dtype
    if rows:
        assert torch.equal(h.float(), h_ref)  # the sum is rounded once, like the reference's addition
        assert (y.float() - y_ref).abs().max().item() <= TOL[dtype]


def test_in_place_sum_and_leading_axes():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 37, 640, generator=g).to(torch.bfloat16).to(DEV)
    r = torch.randn(2, 37, 640, generator=g).to(torch.bfloat16).to(DEV)
    scale = torch.ones(640, dtype=torch.bfloat16, device=DEV)
    expect_h, expect_y = _native.add_rmsnorm(x.clone(), r, scale, 1e-5)
    h, y = _native.add_rmsnorm(x, r, scale, 1e-5, inplace_sum=True)
    assert h.data_ptr() == x.data_ptr()
    assert torch.equal(x, expect_h) and torch.equal(y, expect_y)


def test_module_uses_the_same_formula_as_eager():
    norm = RMSNorm(640, eps=1e-5).to(DEV)
    with torch.no_grad():
        norm.scale.copy_(1 + 0.1 * torch.randn(640, device=DEV))
    x = torch.randn(4, 50, 640, device=DEV)
    with torch.no_grad():
        fused = norm(x)
    eager = x / torch.sqrt(torch.mean(x ** 2, dim=-1, keepdim=True) + norm.eps) * norm.scale
    assert (fused - eager).abs().max().item() <= 1e-5
    # an input that carries a gradient takes the differentiable PyTorch path
    xg = x.clone().requires_grad_(True)
    norm(xg).sum().backward()
    assert xg.grad is not None


def test_rejects_bad_arguments():
    x = torch.randn(4, 12, device=DEV)  # 12 is not a multiple of 8
    with pytest.raises(_native.TmwError):
        _native.add_rmsnorm(x, None, torch.ones(12, device=DEV), 1e-5)
    with pytest.raises(TypeError):
        _native.add_rmsnorm(torch.randn(4, 16, device=DEV), None, torch.ones(16, device=DEV, dtype=torch.bfloat16), 1e-5)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 2e-2), (torch.float16, 4e-3)])
def test_gelu_is_the_exact_erf_form(dtype, tol):
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(33, 2560, generator=g) * 3).to(dtype)
    x[0, :8] = torch.tensor([0.0, -0.0, 1e-6, -1e-6, 12.0, -12.0, 40.0, -40.0]).to(dtype)
    ref = torch.nn.functional.gelu(x.float())  # approximate="none": 0.5 x (1 + erf(x / sqrt 2)), mlp.py:58-65
    y = _native.gelu(x.to(DEV))
    assert y.dtype == dtype and (y.float().cpu() - ref).abs().max().item() <= tol
    z = x.to(DEV).clone()
    out = _native.gelu(z, inplace=True)
    assert out.data_ptr() == z.data_ptr() and torch.equal(out, y)


def test_gelu_rejects_bad_arguments():
    with pytest.raises(_native.TmwError):
        _native.gelu(torch.randn(12, device=DEV))  # not a multiple of 8
    with pytest.raises(TypeError):
        _native.gelu(torch.randn(4, 16, device=DEV)[:, ::2])
