"""Benchmark of the WindowedAttention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line.  The default workload is the layer prefill of the reference's
default configuration: bf16, d_model 640, 10 heads x 64, window 512, 16 persistent
tokens, batch 8 per GPU, T = 4096 (L = 4112), seeded synthetic inputs.  A step is
one forward of the module (QKV projection, attention core, output projection) over
one batch.  Across GPUs the batch is sharded (every rank runs its own batch of 8,
weights replicated, no collective on the data path): weak scaling.

``value`` is whole-job TFLOP/s of algorithmic work (masked-out pairs do not count)
with the inputs already in HBM; ``e2e`` is the same through the module's public
``forward`` with host buffers, the copies in both directions inside the timed
region; ``roofline`` describes the attention-core kernel timed in place with CUDA
events; ``cpu_baseline`` is the CPU oracle port timed on a bounded sample.

``--impl reference`` times the reference's CPU path (the oracle port: the same
PyTorch operations the reference issues, all host threads) on a bounded sample of
the same workload.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "titanmac-standalone_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

METRIC = "windowed_attn_layer_prefill_tflops"

WORKLOADS = {
    # name: per-GPU batch, T, d_model, heads, window, n_persistent, dtype
    "config2_layer_prefill": dict(batch=8, T=4096, d_model=640, heads=10, window=512, n_persistent=16,
                                  dtype="bf16"),
    "config1_layer_prefill_fp32": dict(batch=2, T=512, d_model=512, heads=8, window=256, n_persistent=16,
                                       dtype="fp32"),
}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the attention-core kernel,
# taken from the ncu capture summarised under profiles/ (None until captured)
NCU_TRAFFIC_BYTES = {"config2_layer_prefill": None}


def live_pairs(L: int, w: int, Np: int) -> int:
    T = L - Np
    ramp, full = min(T, w), max(0, T - w)
    return ramp * (ramp + 1) // 2 + full * (w + 1) + Np * T + Np * Np


def layer_flops(wl: dict) -> dict:
    B, D, H = wl["batch"], wl["d_model"], wl["heads"]
    L = wl["n_persistent"] + wl["T"]
    dh = D // H
    core = B * H * live_pairs(L, wl["window"], wl["n_persistent"]) * 4 * dh
    qkv = 2 * B * L * D * 3 * D
    out = 2 * B * L * D * D
    return dict(core=core, qkv=qkv, out=out, total=core + qkv + out)


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(source="measured", hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]))
    return dict(source="fallback", hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


class ClockSampler:
    """Polls SM clock and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, index: int, period_s: float = 0.005):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None

    def __enter__(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001 - clocks are reported as unavailable, the run goes on
            self._nv = None
            return self
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:  # noqa: BLE001
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(self.period)

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        return False

    def report(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except (ValueError, IndexError):
            return local_index
    return local_index


# --------------------------------------------------------------------------------------
# CPU side: the reference's path, restated (oracle port)
# --------------------------------------------------------------------------------------


def cpu_reference_sample(wl: dict, iters: int, warmup: int = 1):
    """Times the oracle port on ONE batch element of the workload, fp32 like the reference's default.

    Returns (seconds per forward of one batch element, flops of that forward, cores, description).
    """
    from oracle import windowed_oracle as wo

    torch.set_num_threads(os.cpu_count() or 1)
    one = dict(wl, batch=1)
    x, w_qkv, w_out = wo.layer_inputs(1, wl["T"], wl["d_model"], wl["n_persistent"], seed=0)
    cache = {}
    for _ in range(warmup):  # builds and caches the dense boolean mask like the reference's first call
        wo.module_forward_reference_cost(x, w_qkv, w_out, wl["heads"], wl["window"], wl["n_persistent"], cache)
    times = []
    for _ in range(iters):
        t0 = time.perf_counter()
        wo.module_forward_reference_cost(x, w_qkv, w_out, wl["heads"], wl["window"], wl["n_persistent"], cache)
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    desc = (f"1 of {wl['batch']} batch elements (L={wl['n_persistent'] + wl['T']}), fp32, dense mask + library "
            f"attention like the reference, median of {iters} after {warmup} warm-up (mask build excluded)")
    return sec, layer_flops(one)["total"], torch.get_num_threads(), desc


def run_reference_arm(args, wl_name: str, wl: dict) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sec, flops, cores, desc = cpu_reference_sample(wl, iters=max(1, args.steps), warmup=max(1, args.warmup))
    value = flops / sec / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(workload=wl_name, **wl, step="one batch element per step (bounded sample)"),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# GPU side
# --------------------------------------------------------------------------------------


def run_ours(args, wl_name: str, wl: dict) -> None:
    import torch.distributed as dist

    from oracle import windowed_oracle as wo  # seeded input recipe (and the CPU baseline leg below)
    from titanmac_b200 import WindowConfig, WindowedAttention, _native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path in the product)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    dtype = torch.bfloat16 if wl["dtype"] == "bf16" else torch.float32
    B, T, D, H, w, Np = wl["batch"], wl["T"], wl["d_model"], wl["heads"], wl["window"], wl["n_persistent"]
    L = Np + T
    x_cpu, w_qkv, w_out = wo.layer_inputs(B, T, D, Np, seed=rank)
    mod = WindowedAttention(WindowConfig(window_size=w, num_heads=H, head_dim=D // H, n_persistent=Np)).eval()
    with torch.no_grad():
        mod.qkv_proj.weight.copy_(w_qkv)
        mod.out_proj.weight.copy_(w_out)
    mod = mod.to(device=dev, dtype=dtype)

    # several input sets so that consecutive steps do not find their inputs in L2 (126 MB)
    n_sets = 4
    xs = [(x_cpu.to(dtype) + 0.001 * i).to(dev) for i in range(n_sets)]
    flops = layer_flops(wl)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        mod(xs[i % n_sets])
    _native.poll_status(dev)

    # ---- timed region: inputs resident in HBM --------------------------------------
    mod.core_events = []
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(physical_gpu_index(local)) as clocks:
        barrier()
        start.record()
        for i in range(args.steps):
            mod(xs[i % n_sets])
        end.record()
        barrier()
    elapsed_ms = start.elapsed_time(end)
    core_ms = [a.elapsed_time(b) for a, b in mod.core_events]
    mod.core_events = None
    _native.poll_status(dev)

    # ---- end to end: host buffers, copies inside the timed region -------------------
    x_host = x_cpu.to(dtype).pin_memory()
    y_host = torch.empty((B, L, D), dtype=dtype).pin_memory()
    x_dev = torch.empty((B, L, D), dtype=dtype, device=dev)

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True)
        y = mod(x_dev)
        y_host.copy_(y, non_blocking=True)

    for _ in range(max(3, args.warmup // 4)):
        e2e_step()
    e2e_steps = max(3, min(args.steps, 50))
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for _ in range(e2e_steps):
        e2e_step()
    e2.record()
    barrier()
    e2e_ms = s2.elapsed_time(e2)

    t = torch.tensor([elapsed_ms, e2e_ms, sum(core_ms) / max(1, len(core_ms))], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, core_avg_ms = (float(v) for v in t.cpu())

    if rank == 0:
        peaks = load_peaks()
        value = flops["total"] * world * args.steps / (elapsed_ms * 1e-3) / 1e12
        e2e_value = flops["total"] * world * e2e_steps / (e2e_ms * 1e-3) / 1e12
        achieved = flops["core"] / (core_avg_ms * 1e-3) / 1e12
        peak = peaks["bf16_tflops"]
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
            "config": dict(workload=wl_name, **wl, global_batch=B * world, parallelism=f"batch-sharded x{world}",
                           l2="inputs rotate over 4 sets; x+qkv+o per step = 210 MB > 126 MB L2",
                           flops_per_step_per_gpu=flops),
            "roofline": {"bound": "tensor", "kernel": "attention core (tmw_prefill)", "achieved": achieved,
                         "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "peak_source": f"{peaks['source']} bf16 burst", "avg_launch_ms": core_avg_ms,
                         "traffic": NCU_TRAFFIC_BYTES.get(wl_name),
                         "algorithmic_flops_per_launch": flops["core"]},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": x_host.numel() * x_host.element_size(),
                    "d2h_bytes_per_step": y_host.numel() * y_host.element_size(), "steps": e2e_steps,
                    "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": args.steps,
            "clocks": clocks.report(),
        }
        if world == 1 and not args.no_cpu_baseline:
            sec, cflops, cores, desc = cpu_reference_sample(wl, iters=5, warmup=1)
            line["cpu_baseline"] = {"value": cflops / sec / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": desc}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="config2_layer_prefill")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (N=1 only)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, args.workload, wl)
    else:
        run_ours(args, args.workload, wl)


if __name__ == "__main__":
    main()
