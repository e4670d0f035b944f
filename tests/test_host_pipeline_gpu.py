"""HostPipeline: host batches through the module with overlapped copies give the results of plain calls."""

import pytest
import torch

from titanmac_b200 import HostPipeline, WindowConfig, WindowedAttention

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_pipeline_matches_direct_calls():
    torch.manual_seed(0)
    mod = WindowedAttention(WindowConfig(window_size=64, num_heads=4, head_dim=64, n_persistent=8)).eval()
    mod = mod.to(device=DEV, dtype=torch.bfloat16)
    shape = (2, 8 + 300, 256)
    xs = [torch.randn(shape).to(torch.bfloat16).pin_memory() for _ in range(7)]
    ys = [torch.empty(shape, dtype=torch.bfloat16).pin_memory() for _ in range(7)]
    pipe = HostPipeline(mod, shape, torch.bfloat16, torch.device(DEV), depth=2)
    for x, y in zip(xs, ys):
        pipe.submit(x, y)
    pipe.drain()
    for x, y in zip(xs, ys):
        ref = mod(x.to(DEV)).cpu()
        assert torch.equal(y, ref)


def test_pipeline_wants_pinned_memory():
    pipe = HostPipeline(lambda t: t, (4,), torch.float32, torch.device(DEV))
    with pytest.raises(ValueError):
        pipe.submit(torch.zeros(4), torch.zeros(4))
