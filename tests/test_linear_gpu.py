"""The library's tensor-core linear layer (tmw_linear, through the C ABI) against PyTorch in fp32 on the same
bf16-rounded operands: the shapes of the module's projections and of the block's MLP at prefill and decode size,
ragged sizes, bias and the exact-GELU epilogue."""

import pytest
import torch

from titanmac_b200 import _native

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def reference(x, w, b, gelu):
    y = torch.nn.functional.linear(x.float(), w.float(), None if b is None else b.float())
    return torch.nn.functional.gelu(y) if gelu else y


def run_case(m, n, k, bias, gelu, dtype=torch.bfloat16, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = torch.randn(m, k, generator=g, device=DEV).to(dtype)
    w = (torch.randn(n, k, generator=g, device=DEV) * 0.05).to(dtype)
    b = (torch.randn(n, generator=g, device=DEV) * 0.5).to(dtype) if bias else None
    y = _native.linear(x, w, b, gelu=gelu)
    _native.poll_status(torch.device(DEV))
    ref = reference(x, w, b, gelu)
    # one rounding of the result to 16 bits on top of fp32 accumulation in a different order
    tol = (2 ** -8 if dtype == torch.bfloat16 else 2 ** -10) * max(1.0, ref.abs().max().item()) + 1e-3
    err = (y.float() - ref).abs().max().item()
    assert y.shape == (m, n) and y.dtype == dtype
    assert err <= tol, f"m={m} n={n} k={k} bias={bias} gelu={gelu}: observed max-abs error {err:.3e} > {tol:.3e}"


@pytest.mark.parametrize("m", [256, 32896])
@pytest.mark.parametrize("n,k,bias,gelu", [
    (1920, 640, False, False),   # QKV projection
    (640, 640, False, False),    # output projection
    (2560, 640, True, True),     # MLP fc1 + bias + GELU
    (640, 2560, True, False),    # MLP fc2 + bias
])
def test_layer_shapes(m, n, k, bias, gelu):
    run_case(m, n, k, bias, gelu)


@pytest.mark.parametrize("m,n,k", [(1, 8, 8), (127, 136, 72), (129, 264, 200), (300, 50000, 640), (515, 128, 64),
                                   (700, 40, 64), (1000, 1944, 128), (513, 24, 640)])  # narrow last tiles of the pair kernel
def test_ragged_sizes(m, n, k):
    run_case(m, n, k, True, False, seed=m)
    run_case(m, n, k, False, True, seed=m + 1)


def test_fp16_and_strided_input():
    run_case(200, 320, 128, True, True, dtype=torch.float16)
    g = torch.Generator(device=DEV).manual_seed(9)
    big = torch.randn(64, 3, 256, generator=g, device=DEV).to(torch.bfloat16)
    x = big[:, 1]  # rows 768 elements apart
    w = (torch.randn(160, 256, generator=g, device=DEV) * 0.05).to(torch.bfloat16)
    y = _native.linear(x, w)
    assert (y.float() - reference(x, w, None, False)).abs().max().item() <= 2e-2


def test_rejects_what_it_cannot_do():
    x = torch.zeros(4, 12, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(8, 12, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(TypeError):
        _native.linear(x, w)  # k not a multiple of 8
    with pytest.raises(TypeError):
        _native.linear(torch.zeros(4, 16, device=DEV), torch.zeros(8, 16, device=DEV))  # fp32
