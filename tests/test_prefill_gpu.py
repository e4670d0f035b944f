"""Parity of the CUDA prefill path (through the C ABI) with the golden vectors and the oracle."""

import pytest
import torch

from conftest import CORE_CASES, FULL_CASES
from oracle import windowed_oracle as wo
from titanmac_b200 import WindowConfig, WindowedAttention, _native

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5   # fp32 contract: max-abs against the reference
BF16_TOL = 2e-2   # bf16 contract: max-abs against the fp32 reference on the same (rounded) inputs
# Module outputs with N(0, 0.02) weights have magnitude ~0.2, where 2e-2 would let a wrong window edge pass: the
# second, tighter bound is what the kernels have been observed to stay under on these cases (the reference's own
# bf16-against-fp32 difference is about 1e-3).
MODULE_REGRESSION_TOL = 5e-3
DEV = "cuda:0"
ALGOS = [_native.ALGO_SIMT, _native.ALGO_TCGEN05]
ALGO_IDS = ["simt", "tcgen05"]


def tc_cases(golden):
    return [c for c in FULL_CASES if golden.meta(c)["dh"] in (64, 128)]


def make_module(m, dtype, w_qkv, w_out, algo=_native.ALGO_AUTO):
    mod = WindowedAttention(WindowConfig(window_size=m["w"], num_heads=m["H"], head_dim=m["dh"],
                                         n_persistent=m["Np"])).eval()
    with torch.no_grad():
        mod.qkv_proj.weight.copy_(w_qkv)
        mod.out_proj.weight.copy_(w_out)
    mod.algo = algo
    return mod.to(device=DEV, dtype=dtype)


@pytest.mark.parametrize("case", FULL_CASES)
def test_module_fp32_matches_reference_output(golden, case):
    m = golden.meta(case)
    mod = make_module(m, torch.float32, golden[case, "w_qkv"], golden[case, "w_out"])
    y = mod(golden[case, "x"].to(DEV))
    assert y.shape == golden[case, "y"].shape and y.dtype == torch.float32
    assert (y.cpu() - golden[case, "y"]).abs().max().item() <= FP32_TOL


@pytest.mark.parametrize("case", CORE_CASES)
def test_core_fp32_matches_reference_core(golden, case):
    m = golden.meta(case)
    q, k, v = (golden[case, f"core_{n}"].to(DEV) for n in "qkv")
    o = _native.prefill(q, k, v, m["w"], m["Np"], algo=_native.ALGO_SIMT)
    assert (o.cpu() - golden[case, "core_o"]).abs().max().item() <= FP32_TOL


def test_config1_fp32_matches_reference_rows(golden):
    case = "config1_fp32"
    m = golden.meta(case)
    x, w_qkv, w_out = wo.layer_inputs(m["B"], m["T"], m["D"], m["Np"], m["seed"])
    mod = make_module(m, torch.float32, w_qkv, w_out)
    y = mod(x.to(DEV)).cpu()
    rows = golden[case, "rows"]
    assert (y[:, rows] - golden[case, "y_rows"]).abs().max().item() <= FP32_TOL
    full = wo.module_forward(x, w_qkv, w_out, m["H"], m["w"], m["Np"])
    assert (y - full).abs().max().item() <= FP32_TOL


@pytest.mark.parametrize("algo", ALGOS, ids=ALGO_IDS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_module_16bit_matches_fp32_reference(golden, dtype, algo):
    for case in tc_cases(golden) + ["config1_fp32"]:
        m = golden.meta(case)
        if case == "config1_fp32":
            x, w_qkv, w_out = wo.layer_inputs(m["B"], m["T"], m["D"], m["Np"], m["seed"])
        else:
            x, w_qkv, w_out = (golden[case, n] for n in ("x", "w_qkv", "w_out"))
        xr, wq, wo_ = (t.to(dtype) for t in (x, w_qkv, w_out))
        ref = wo.module_forward(xr, wq, wo_, m["H"], m["w"], m["Np"])  # fp32 math on the rounded inputs
        mod = make_module(m, dtype, w_qkv, w_out, algo)
        y = mod(xr.to(DEV))
        assert y.dtype == dtype
        err = (y.float().cpu() - ref).abs().max().item()
        assert err <= BF16_TOL, f"{case}: observed max-abs error {err:.3e}"
        assert err <= MODULE_REGRESSION_TOL, f"{case}: observed max-abs error {err:.3e} above the regression bound"


@pytest.mark.parametrize("algo", ALGOS, ids=ALGO_IDS)
@pytest.mark.parametrize("dh,L,w,Np,B,H", [
    (64, 1000, 300, 16, 2, 2),    # several key tiles per query tile, ragged tail
    (64, 257, 512, 0, 1, 3),      # no persistent keys, window longer than the sequence
    (64, 700, 0, 5, 1, 2),        # self-only window
    (64, 513, 127, 130, 1, 1),    # more than one tile of persistent keys
    (128, 900, 256, 16, 1, 2),
    (128, 300, 1024, 1, 2, 1),
    # last 256-row block holds one query tile only, and that tile walks more key tiles than the K/V rings
    # have stages (the absent tile's issuing warp must keep handing stages back in step)
    (64, 16 + 2048, 1024, 16, 1, 2),
    (128, 16 + 2048, 1024, 16, 1, 2),
    (128, 16 + 1280 + 100, 1024, 0, 1, 1),
    (64, 128 + 1500, 640, 128, 1, 1),   # first query tile is persistent rows only
])
def test_core_bf16_unit_variance_inputs(dh, L, w, Np, B, H, algo):
    """N(0,1) q/k/v give O(1) scores: exercises the running-max path, not just a flat softmax."""
    q, k, v = (t.to(torch.bfloat16) for t in wo.qkv_inputs(B, H, L, dh, seed=dh + L))
    ref = wo.attention_core_blockwise(q, k, v, w, Np, block=256)
    if algo == _native.ALGO_TCGEN05 and Np > 128:
        # the tensor-core kernel keeps the persistent keys in one tile of at most 128 rows: pinning it
        # is refused, and the library's own choice falls back to the CUDA-core kernel
        with pytest.raises(_native.TmwError) as e:
            _native.prefill(q.to(DEV), k.to(DEV), v.to(DEV), w, Np, algo=algo)
        assert e.value.status == _native.TMW_ERR_UNSUPPORTED
        algo = _native.ALGO_AUTO
    o = _native.prefill(q.to(DEV), k.to(DEV), v.to(DEV), w, Np, algo=algo)
    _native.poll_status()  # raises if a bounded device-side wait expired
    err = (o.float().cpu() - ref).abs().max().item()
    assert err <= BF16_TOL, err


@pytest.mark.parametrize("algo", ALGOS, ids=ALGO_IDS)
def test_sharded_positions_match_unsharded_rows(algo):
    """q rows [r0, r1) against a K/V buffer [persistent | halo | own rows] equal the same rows of the full call."""
    dh, L, w, Np, B, H = 64, 1200, 200, 16, 1, 2
    q, k, v = (t.to(torch.bfloat16).to(DEV) for t in wo.qkv_inputs(B, H, L, dh, seed=5))
    full = _native.prefill(q, k, v, w, Np, algo=algo)
    for r0, r1 in ((Np + 500, Np + 900), (Np + 900, L), (Np + 100, Np + 101)):
        lo = max(Np, r0 - w)
        kk = torch.cat([k[:, :, :Np], k[:, :, lo:r1]], dim=2).contiguous()
        vv = torch.cat([v[:, :, :Np], v[:, :, lo:r1]], dim=2).contiguous()
        part = _native.prefill(q[:, :, r0:r1].contiguous(), kk, vv, w, Np, q_pos0=r0, k_pos0=lo, algo=algo)
        # same rows, different tile alignment: equal up to the rounding of a different summation order
        assert (part.float() - full[:, :, r0:r1].float()).abs().max().item() <= 1e-2, (r0, r1)


@pytest.mark.parametrize("dh", [64, 128])
def test_rows_behind_a_short_persistent_block_are_never_multiplied(dh):
    """8 persistent keys fill half of the 16-row persistent tile of the tensor-core kernel.  The sequence rows
    right behind them (here: NaN, like a halo that has not arrived yet) lie outside the window of the queries
    asked for, so they must not reach the output - not even as 0 x NaN inside a matrix product."""
    L, w, Np, B, H = 1100, 100, 8, 1, 2
    q, k, v = (t.to(torch.bfloat16) for t in wo.qkv_inputs(B, H, L, dh, seed=11))
    r0 = Np + 8 + w + 5  # the first query whose window starts behind the poisoned rows
    ref = wo.attention_core_rows(q[:, :, r0:].float(), k.float(), v.float(), r0, w, Np)
    kp, vp = k.clone(), v.clone()
    kp[:, :, Np:Np + 8] = float("nan")
    vp[:, :, Np:Np + 8] = float("nan")
    o = _native.prefill(q[:, :, r0:].contiguous().to(DEV), kp.to(DEV), vp.to(DEV), w, Np, q_pos0=r0, k_pos0=Np,
                        algo=_native.ALGO_TCGEN05)
    _native.poll_status()
    assert not torch.isnan(o).any()
    err = (o.float().cpu() - ref).abs().max().item()
    assert err <= BF16_TOL, err


def test_two_kernels_agree_at_full_size_config2_tcgen05():
    """benchmark configuration 2 (B8, L=16+4096, 10 heads x 64, w=512): the two independent CUDA kernels agree,
    and sampled rows agree with the CPU oracle."""
    B, T, D, H, w, Np = 8, 4096, 640, 10, 512, 16
    x, w_qkv, w_out = wo.layer_inputs(B, T, D, Np, seed=0)
    xr, wq = x.to(torch.bfloat16), w_qkv.to(torch.bfloat16)
    qkv = torch.nn.functional.linear(xr.to(DEV), wq.to(DEV))
    L = Np + T
    q, k, v = (qkv.view(B, L, 3, H, 64)[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    o_tc = _native.prefill(q, k, v, w, Np, algo=_native.ALGO_TCGEN05)
    o_simt = _native.prefill(q, k, v, w, Np, algo=_native.ALGO_SIMT)
    assert (o_tc.float() - o_simt.float()).abs().max().item() <= BF16_TOL
    qc, kc, vc = (t.float().cpu() for t in (q, k, v))
    for r0 in (0, 128, 512 + 16 - 3, 2048, L - 64):
        ref = wo.attention_core_rows(qc[:, :, r0:r0 + 64], kc, vc, r0, w, Np)
        assert (o_tc[:, :, r0:r0 + 64].float().cpu() - ref).abs().max().item() <= BF16_TOL
    # rows of a softmax-weighted average stay inside the range of the values they average
    assert o_tc.float().abs().max() <= v.float().abs().max() + 1e-2
    _native.poll_status()


def test_non_contiguous_head_dim_is_rejected():
    q = torch.zeros(1, 1, 16, 128, device=DEV, dtype=torch.bfloat16)[..., ::2]
    with pytest.raises(ValueError):
        _native.prefill(q, q, q, 4, 1)


def test_key_range_error_reaches_python():
    q = torch.zeros(1, 1, 16, 64, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(_native.TmwError) as e:
        _native.prefill(q, q, q, 4, 1, q_pos0=100, k_pos0=1)
    assert e.value.status == _native.TMW_ERR_KEY_RANGE
