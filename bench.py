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

The ``--steps`` region is repeated until half a second of device time has been
timed; ``ms_per_step`` is the median region (each region counted with its slowest
rank) and ``timing`` holds min / max and every rank's own median.  The default
workload's line also carries, under ``extra``, the benchmark's other
configurations measured in the same run: the decode step of configuration 4
(256 sequences over the GPUs), the long-context core of configuration 5 (on
several GPUs sequence-sharded, with sampled row blocks of the sharded output held
against the CPU oracle) and configuration 2 as one batch of 8 split over the GPUs.

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
    # benchmark configuration 4: 16-layer default model, ring-cache decode; `batch` is the WHOLE-job batch here
    # (256 sequences sharded over the GPUs), prompt 2048 tokens, then `--steps` single-token steps
    "config4_decode": dict(batch=256, T=2048, d_model=640, heads=10, window=512, n_persistent=16, dtype="bf16",
                           layers=16, d_ff=2560, vocab=50000),
    # config 2's layer with the reference's DEFAULT attention class (block-sparse: depthwise convolutions on
    # Q/K/V, block-granular window, global persistent rows), block = max(64, window // 8) = 64
    "config2_block_sparse_layer_prefill": dict(batch=8, T=4096, d_model=640, heads=10, window=512, n_persistent=16,
                                               dtype="bf16", block_size=64, conv_taps=4),
    # config 2's layer, forward + backward (gradients of the input and of both weights)
    "config2_layer_train": dict(batch=8, T=4096, d_model=640, heads=10, window=512, n_persistent=16, dtype="bf16"),
    # the same with the reference's default (block-sparse) attention class
    "config2_block_sparse_layer_train": dict(batch=8, T=4096, d_model=640, heads=10, window=512, n_persistent=16,
                                             dtype="bf16", block_size=64, conv_taps=4),
    # benchmark configuration 3: whole 16-layer model forward (prefill), 2 sequences of 8192 tokens per GPU
    "config3_model_prefill": dict(batch=2, T=8192, d_model=640, heads=10, window=512, n_persistent=16, dtype="bf16",
                                  layers=16, d_ff=2560, vocab=50000),
    # benchmark configuration 5: attention core only, Q/K/V given; the sequence is sharded over the GPUs
    "config5_long_prefill": dict(batch=1, T=131072, d_model=2048, heads=16, window=1024, n_persistent=16,
                                 dtype="bf16"),
}

# DRAM traffic per launch (ncu: dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel, measured on
# exactly the geometry of the workload (config 2: batch 8, L = 4112, 10 heads x 64, window 512: Q + K + V read
# once = 126.4 MB, 24.8 MB of the 42.1 MB of O written back before the kernel ends).  None = not captured for
# the kernel as it is now.
NCU_TRAFFIC_BYTES = {"config2_layer_prefill": 126454528 + 25991680}

MIN_TIMED_SECONDS = 0.5  # the --steps region is repeated until at least this much device time has been timed


def live_pairs(L: int, w: int, Np: int) -> int:
    T = L - Np
    ramp, full = min(T, w), max(0, T - w)
    return ramp * (ramp + 1) // 2 + full * (w + 1) + Np * T + Np * Np


def layer_flops(wl: dict) -> dict:
    B, D, H = wl["batch"], wl["d_model"], wl["heads"]
    L = wl["n_persistent"] + wl["T"]
    dh = D // H
    qkv = 2 * B * L * D * 3 * D
    out = 2 * B * L * D * D
    if "block_size" in wl:
        from oracle import block_sparse_oracle as bo  # pair count only

        core = B * H * bo.live_pairs(L, wl["window"], wl["block_size"], wl["n_persistent"]) * 4 * dh
        conv = 2 * wl["conv_taps"] * B * L * 3 * D
        return dict(core=core, qkv=qkv, out=out, conv=conv, total=core + qkv + out + conv)
    core = B * H * live_pairs(L, wl["window"], wl["n_persistent"]) * 4 * dh
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


def bind_to_gpu_cores(local_index: int) -> dict:
    """Pins this process to the CPU cores that NVML reports as local to its GPU (its NUMA node), so that the
    pinned host buffers allocated afterwards and the threads that drive the copies sit next to the GPU."""
    info = {"bound": False}
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(physical_gpu_index(local_index))
        n_words = (os.cpu_count() + 63) // 64
        words = pynvml.nvmlDeviceGetCpuAffinity(h, n_words)
        cores = [64 * i + b for i, wd in enumerate(words) for b in range(64) if (wd >> b) & 1]
        world_local = int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("WORLD_SIZE", "1")))
        if cores:
            # ranks whose GPUs share a NUMA node share its cores out among themselves
            per = max(1, len(cores) // max(1, world_local))
            mine = cores[(local_index * per) % len(cores):][:per] or cores
            os.sched_setaffinity(0, set(mine))
            info = {"bound": True, "cores": len(mine), "first_core": mine[0], "numa_cores": len(cores)}
            try:
                info["numa_node"] = pynvml.nvmlDeviceGetNumaNodeId(h)
            except Exception:  # noqa: BLE001 - older bindings
                pass
    except Exception as e:  # noqa: BLE001 - binding is an optimisation; the run goes on unbound
        info["error"] = type(e).__name__
    return info


def timed_regions(step, steps: int, barrier, world: int, dev, min_seconds: float = MIN_TIMED_SECONDS,
                  max_regions: int = 200):
    """Times `steps` calls of step(i) with CUDA events, bracketed by barrier() on both sides, as often as it
    takes to cover `min_seconds` of device time (the count is fixed from the first region's time, maximum over
    the ranks, so that every rank runs the same number).  Returns this rank's region times in ms."""
    import torch.distributed as dist

    regions, i, n_regions = [], 0, 1
    while len(regions) < n_regions:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record()
        for _ in range(steps):
            step(i)
            i += 1
        b.record()
        barrier()
        regions.append(a.elapsed_time(b))
        if len(regions) == 1:
            t = torch.tensor([regions[0]], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            n_regions = int(min(max_regions, max(1, math.ceil(min_seconds * 1e3 / max(float(t.item()), 1e-3)))))
    return regions


def gather_ranks(values, world: int, dev):
    """[world, len(values)] float64 tensor on the host: every rank's numbers, for per-rank reporting."""
    import torch.distributed as dist

    t = torch.tensor(values, device=dev, dtype=torch.float64)
    if world == 1:
        return t[None].cpu()
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return torch.stack(out).cpu()


# --------------------------------------------------------------------------------------
# CPU side: the reference's path, restated (oracle port)
# --------------------------------------------------------------------------------------


def block_sparse_conv_weights(wl: dict, seed: int):
    """Seeded depthwise filters ``[D, taps]`` for Q, K and V (N(0, 0.3), CPU generator)."""
    g = torch.Generator(device="cpu").manual_seed(1000 + seed)
    return [torch.randn(wl["d_model"], wl["conv_taps"], generator=g) * 0.3 for _ in range(3)]


def cpu_reference_sample(wl: dict, iters: int, warmup: int = 1):
    """Times the oracle port on ONE batch element of the workload, fp32 like the reference's default.

    Returns (seconds per forward of one batch element, flops of that forward, cores, description).
    """
    from oracle import windowed_oracle as wo

    torch.set_num_threads(os.cpu_count() or 1)
    one = dict(wl, batch=1)
    x, w_qkv, w_out = wo.layer_inputs(1, wl["T"], wl["d_model"], wl["n_persistent"], seed=0)
    if "block_size" in wl:
        from oracle import block_sparse_oracle as bo

        convs = block_sparse_conv_weights(wl, seed=0)

        def forward():
            bo.module_forward_reference_cost(x, w_qkv, *convs, w_out, wl["heads"], wl["window"], wl["block_size"],
                                             wl["n_persistent"])
        how = "library depthwise convolutions + Python loop over query blocks like the reference"
    else:
        cache = {}

        def forward():  # builds and caches the dense boolean mask like the reference's first call
            wo.module_forward_reference_cost(x, w_qkv, w_out, wl["heads"], wl["window"], wl["n_persistent"], cache)
        how = "dense mask + library attention like the reference"
    for _ in range(warmup):
        forward()
    times = []
    for _ in range(iters):
        t0 = time.perf_counter()
        forward()
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    desc = (f"1 of {wl['batch']} batch elements (L={wl['n_persistent'] + wl['T']}), fp32, {how}, "
            f"median of {iters} after {warmup} warm-up (mask build excluded)")
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


_DIST = None


def _dist_setup(args):
    """(dist, world, rank, local, dev); the process group is made once per process."""
    global _DIST
    if _DIST is not None:
        return _DIST
    import torch.distributed as dist

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
    _DIST = (dist, world, rank, local, dev)
    return _DIST


def make_barrier(dist, world):
    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    return barrier


def region_stats(regions, steps: int, world: int, dev) -> dict:
    """Per-step times from every rank's region times: a region counts with its slowest rank; the median region
    is the reported one; the per-rank medians show which GPU (or host) is the slow one."""
    allr = gather_ranks(regions, world, dev) / steps             # [world, regions] ms per step
    worst = allr.max(dim=0).values
    return {"ms_per_step": float(worst.median()), "min": float(worst.min()), "max": float(worst.max()),
            "regions": len(regions), "timed_seconds": float(allr.max(dim=0).values.sum() * steps / 1e3),
            "per_rank_ms_per_step": [round(float(v), 5) for v in allr.median(dim=1).values]}


def pcie_ceiling(nbytes: int, world: int, dev, barrier, iters: int = 10) -> dict:
    """Plain pinned-memory copies of `nbytes`, every rank at the same time and nothing else running: each
    direction alone, then both directions at once on two streams (what the end-to-end leg does in steady state).
    What the host links and the host memory give when all GPUs copy at once is the ceiling of that leg."""
    hosts = [torch.empty(nbytes, dtype=torch.uint8).pin_memory() for _ in range(2)]
    devs = [torch.empty(nbytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    streams = [torch.cuda.Stream(dev) for _ in range(2)]
    out = {}

    def timed(directions):
        for d_ in directions:
            with torch.cuda.stream(streams[d_]):
                (devs[0].copy_(hosts[0], non_blocking=True) if d_ == 0 else hosts[1].copy_(devs[1], non_blocking=True))
        barrier()
        evs = []
        for d_ in directions:
            with torch.cuda.stream(streams[d_]):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(iters):
                    (devs[0].copy_(hosts[0], non_blocking=True) if d_ == 0 else hosts[1].copy_(devs[1], non_blocking=True))
                b.record()
                evs.append((a, b))
        barrier()
        return [nbytes * iters / (a.elapsed_time(b) * 1e-3) / 1e9 for a, b in evs]

    per_rank = lambda v: [round(float(x), 2) for x in gather_ranks([v], world, dev)[:, 0]]  # noqa: E731
    out["h2d_alone_gbs_per_rank"] = per_rank(timed([0])[0])
    out["d2h_alone_gbs_per_rank"] = per_rank(timed([1])[0])
    both = timed([0, 1])
    out["h2d_with_d2h_gbs_per_rank"] = per_rank(both[0])
    out["d2h_with_h2d_gbs_per_rank"] = per_rank(both[1])
    return out


def make_layer(wl: dict, rank: int, dev, dtype):
    from oracle import windowed_oracle as wo  # seeded input recipe
    from titanmac_b200 import WindowConfig, WindowedAttention

    B, T, D, H, w, Np = wl["batch"], wl["T"], wl["d_model"], wl["heads"], wl["window"], wl["n_persistent"]
    x_cpu, w_qkv, w_out = wo.layer_inputs(B, T, D, Np, seed=rank)
    if "block_size" in wl:
        from titanmac_b200 import BlockSparseAttention

        mod = BlockSparseAttention(d_model=D, n_heads=H, window_size=w, block_size=wl["block_size"], n_persistent=Np,
                                   conv_kernel=wl["conv_taps"]).eval()
        with torch.no_grad():
            for conv, wt in zip((mod.conv_q, mod.conv_k, mod.conv_v), block_sparse_conv_weights(wl, seed=rank)):
                conv.weight.copy_(wt[:, None, :])
    else:
        mod = WindowedAttention(WindowConfig(window_size=w, num_heads=H, head_dim=D // H, n_persistent=Np)).eval()
    with torch.no_grad():
        mod.qkv_proj.weight.copy_(w_qkv)
        mod.out_proj.weight.copy_(w_out)
    return mod.to(device=dev, dtype=dtype), x_cpu


def run_ours(args, wl_name: str, wl: dict) -> None:
    from titanmac_b200 import HostPipeline, _native

    dist, world, rank, local, dev = _dist_setup(args)
    affinity = bind_to_gpu_cores(local)  # before any pinned allocation
    barrier = make_barrier(dist, world)
    dtype = torch.bfloat16 if wl["dtype"] == "bf16" else torch.float32
    B, T, D, Np = wl["batch"], wl["T"], wl["d_model"], wl["n_persistent"]
    L = Np + T
    mod, x_cpu = make_layer(wl, rank, dev, dtype)

    # several input sets so that consecutive steps do not find their inputs in L2 (126 MB)
    n_sets = 4
    xs = [(x_cpu.to(dtype) + 0.001 * i).to(dev) for i in range(n_sets)]
    flops = layer_flops(wl)
    for i in range(args.warmup):
        mod(xs[i % n_sets])
    _native.poll_status(dev)

    # ---- timed regions: inputs resident in HBM ---------------------------------------
    mod.core_events = []
    with ClockSampler(physical_gpu_index(local)) as clocks:
        regions = timed_regions(lambda i: mod(xs[i % n_sets]), args.steps, barrier, world, dev)
    core_ms = [a.elapsed_time(b) for a, b in mod.core_events]
    mod.core_events = None
    _native.poll_status(dev)
    stats = region_stats(regions, args.steps, world, dev)
    core_all = gather_ranks([sum(core_ms) / max(1, len(core_ms)), statistics.median(core_ms)], world, dev)
    core_avg_ms = float(core_all[:, 0].max())

    # ---- end to end: host buffers, copies inside the timed region -------------------
    # Every step copies its input from pinned host memory and its output back; HostPipeline (public API)
    # overlaps the two copies and the forward of consecutive steps on three streams.
    x_host = x_cpu.to(dtype).pin_memory()
    y_hosts = [torch.empty((B, L, D), dtype=dtype).pin_memory() for _ in range(2)]
    pipe = HostPipeline(mod, (B, L, D), dtype, dev, depth=2)
    main_stream = torch.cuda.current_stream(dev)
    for i in range(max(3, args.warmup // 4)):
        pipe.submit(x_host, y_hosts[i % 2])
    pipe.drain()
    e2e_steps = max(3, min(args.steps, 50))

    class _Pipe:  # one e2e region = e2e_steps submissions between follow() and join()
        n = 0

    def e2e_region():
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        s2.record(main_stream)
        pipe.follow(main_stream)
        for _ in range(e2e_steps):
            pipe.submit(x_host, y_hosts[_Pipe.n % 2])
            _Pipe.n += 1
        pipe.join(main_stream)
        e2.record(main_stream)
        barrier()
        return s2.elapsed_time(e2)

    first = e2e_region()
    t = torch.tensor([first], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    n_e2e = int(min(50, max(1, math.ceil(MIN_TIMED_SECONDS * 1e3 / max(float(t.item()), 1e-3)))))
    e2e_regions = [first] + [e2e_region() for _ in range(n_e2e - 1)]
    e2e_stats = region_stats(e2e_regions, e2e_steps, world, dev)
    if rank == 0:  # the result really came back: compare the last output with a device-resident forward
        ref = mod(x_host.to(dev)).float().cpu()
        err = (y_hosts[(_Pipe.n - 1) % 2].float() - ref).abs().max().item()
        if not err <= 1e-2:
            raise SystemExit(f"end-to-end output differs from the device-resident forward by {err}")
    h2d_bytes = x_host.numel() * x_host.element_size()
    d2h_bytes = y_hosts[0].numel() * y_hosts[0].element_size()
    pcie = pcie_ceiling(h2d_bytes, world, dev, barrier)
    del pipe, xs

    # ---- the other configurations of the benchmark, carried in the same line ----------
    extra = {}
    if "block_size" not in wl and wl_name == "config2_layer_prefill" and not args.no_extra:
        extra = measure_extras(args, dist, world, rank, local, dev, barrier)

    if rank == 0:
        peaks = load_peaks()
        ms_step = stats["ms_per_step"]
        value = flops["total"] * world / (ms_step * 1e-3) / 1e12
        e2e_value = flops["total"] * world / (e2e_stats["ms_per_step"] * 1e-3) / 1e12
        achieved = flops["core"] / (core_avg_ms * 1e-3) / 1e12
        peak = peaks["bf16_tflops"]
        clk = clocks.report()
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
            "config": dict(workload=wl_name, **wl, global_batch=B * world, parallelism=f"batch-sharded x{world}",
                           l2="inputs rotate over 4 sets; x+qkv+o per step = 210 MB > 126 MB L2",
                           flops_per_step_per_gpu=flops),
            "timing": dict(stats, how=f"regions of {args.steps} steps repeated until {MIN_TIMED_SECONDS} s are timed; a "
                           "region counts with its slowest rank; ms_per_step is the median region",
                           ms_times_median_sm_mhz=(ms_step * clk["sm_mhz"] if clk.get("sm_mhz") else None)),
            "roofline": {"bound": "tensor", "kernel": "attention core (tmw_prefill_block_sparse)"
                         if "block_size" in wl else "attention core (tmw_prefill)", "achieved": achieved,
                         "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "peak_source": f"{peaks['source']} bf16 burst", "avg_launch_ms": core_avg_ms,
                         "avg_launch_ms_per_rank": [round(float(v), 5) for v in core_all[:, 0]],
                         "median_launch_ms_per_rank": [round(float(v), 5) for v in core_all[:, 1]],
                         "traffic": NCU_TRAFFIC_BYTES.get(wl_name),
                         "algorithmic_flops_per_launch": flops["core"]},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps, "ms_per_step": e2e_stats["ms_per_step"],
                    "regions": e2e_stats["regions"], "min_ms_per_step": e2e_stats["min"],
                    "max_ms_per_step": e2e_stats["max"], "per_rank_ms_per_step": e2e_stats["per_rank_ms_per_step"],
                    "per_rank_gbs_each_way": [round(h2d_bytes / (v * 1e-3) / 1e9, 2)
                                              for v in e2e_stats["per_rank_ms_per_step"]],
                    "copy_only_ceiling": pcie, "cpu_affinity": affinity,
                    "how": "HostPipeline: H2D copy, forward and D2H copy of consecutive steps overlap on 3 streams"},
            # this library's kernels per step: the attention core (block-sparse: convolution + two core launches)
            # and, for 16-bit types, the two projections (tmw_linear)
            "gpu_launches": args.steps * stats["regions"] * ((3 if "block_size" in wl else 1) +
                                                              (2 if wl["dtype"] in ("bf16", "fp16") else 0)),
            "clocks": clk,
        }
        if extra:
            line["extra"] = extra
        if world == 1 and not args.no_cpu_baseline:
            sec, cflops, cores, desc = cpu_reference_sample(wl, iters=5, warmup=1)
            line["cpu_baseline"] = {"value": cflops / sec / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": desc}
        print(json.dumps(line), flush=True)


def decode_attention_probe(dev, peaks, batch=256, heads=10, dh=64, window=512, n_persistent=16, layers=4, iters=10):
    """The decode kernel alone on benchmark configuration 4's geometry: one launch = one layer's attention for the whole
    batch.  `layers` independent ring caches are cycled so that a launch never finds its ring in L2."""
    from titanmac_b200 import _native

    caches = [_native.RingCache(batch, heads, dh, window, n_persistent, torch.bfloat16, dev) for _ in range(layers)]
    for c in caches:
        c.k_ring.normal_(); c.v_ring.normal_(); c.k_pers.normal_(); c.v_pers.normal_()
    qkv = torch.randn(batch, 3, heads, dh, device=dev, dtype=torch.bfloat16)
    pos = torch.full((batch,), 2048, dtype=torch.int32, device=dev)
    out = torch.empty(batch, heads, dh, device=dev, dtype=torch.bfloat16)
    for c in caches:
        c.decode(qkv[:, 0], qkv[:, 1], qkv[:, 2], pos, out)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        for c in caches:
            c.decode(qkv[:, 0], qkv[:, 1], qkv[:, 2], pos, out)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / (iters * layers)
    nbytes = batch * heads * (window + 1 + n_persistent) * dh * 2 * 2
    gbs = nbytes / ms / 1e6
    return {"bound": "hbm", "kernel": "decode_stream_kernel (tmw_decode)", "achieved": gbs, "peak": peaks["hbm_gbs"],
            "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "avg_launch_ms": ms,
            "algorithmic_bytes_per_launch": nbytes, "peak_source": f"{peaks['source']} copy bandwidth"}


def random_model(wl: dict, dev, max_seq_len: int):
    """The 16-layer default model with every weight N(0, 0.02), biases 0, norm scales 1 (seeded, CPU generator)."""
    from titanmac_b200 import TitanMAC, TitanMACConfig

    cfg = TitanMACConfig(vocab_size=wl["vocab"], d_model=wl["d_model"], n_heads=wl["heads"], n_layers=wl["layers"],
                         d_ff=wl["d_ff"], max_seq_len=max_seq_len, window_size=wl["window"],
                         n_persistent=wl["n_persistent"], use_block_sparse=False)
    g = torch.Generator(device="cpu").manual_seed(0)
    model = TitanMAC(cfg).eval()
    with torch.no_grad():
        for name, prm in model.named_parameters():
            if name.endswith("scale"):
                prm.fill_(1.0)
            elif name.endswith("bias"):
                prm.zero_()
            else:
                prm.copy_(torch.randn(prm.shape, generator=g) * 0.02)
    return model.to(device=dev, dtype=torch.bfloat16)


def measure_decode(wl_name: str, wl: dict, steps: int, warmup: int, ctx, min_seconds: float = MIN_TIMED_SECONDS):
    """benchmark configuration 4: prompt through the 16-layer model once, then decode steps (CUDA graph).  Returns the
    JSON line as a dict on rank 0, None elsewhere."""
    from titanmac_b200 import _native

    dist, world, rank, local, dev = ctx
    barrier = make_barrier(dist, world)
    if wl["batch"] % world:
        raise SystemExit("the batch must divide by the number of GPUs")
    B = wl["batch"] // world
    max_regions = 8
    e2e_steps = max(3, min(steps, 64))
    # every replayed step moves the position on by one: the position table must cover all of them
    model = random_model(wl, dev, wl["T"] + warmup + steps * max_regions + e2e_steps + 16)
    g = torch.Generator(device="cpu").manual_seed(1 + rank)
    prompt = torch.randint(0, wl["vocab"], (B, wl["T"]), generator=g).to(dev)
    forced = torch.randint(0, wl["vocab"], (B, steps + warmup + 2), generator=g).to(dev)

    chunk = max(1, min(B, 32))  # prompt in slices of the batch: bounds the activation footprint
    caches = model.new_caches(B, dev, torch.bfloat16)
    torch.cuda.synchronize()
    t_pre = time.perf_counter()
    for b0 in range(0, B, chunk):
        sub = model.new_caches(min(chunk, B - b0), dev, torch.bfloat16)
        model.prefill(prompt[b0:b0 + chunk], sub)
        for full, part in zip(caches, sub):
            full.k_ring[b0:b0 + chunk].copy_(part.k_ring); full.v_ring[b0:b0 + chunk].copy_(part.v_ring)
            full.k_pers.copy_(part.k_pers); full.v_pers.copy_(part.v_pers)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t_pre

    tok = forced[:, 0].clone()
    pos = torch.full((B,), wl["T"], dtype=torch.int32, device=dev)
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        model.decode_step(tok, pos, caches)
    torch.cuda.current_stream(dev).wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        logits = model.decode_step(tok, pos, caches)
        pos += 1

    def one_step(i):
        tok.copy_(forced[:, i % forced.shape[1]], non_blocking=True)  # teacher-forced ids, already on the device
        graph.replay()

    for i in range(warmup):
        one_step(i)
    with ClockSampler(physical_gpu_index(local)) as clocks:
        regions = timed_regions(one_step, steps, barrier, world, dev, min_seconds=min_seconds,
                                max_regions=max_regions)
    stats = region_stats(regions, steps, world, dev)
    _native.poll_status(dev)

    # end to end: the step's token ids come from pinned host memory, the greedy choice goes back to the host
    tok_host = forced[:, :8].cpu().pin_memory()
    res_host = torch.empty((B,), dtype=torch.int64).pin_memory()

    def e2e_step(i):
        tok.copy_(tok_host[:, i % 8], non_blocking=True)
        graph.replay()
        res_host.copy_(logits.argmax(dim=-1), non_blocking=True)

    e2e_step(0)
    e2e_stats = region_stats(timed_regions(e2e_step, e2e_steps, barrier, world, dev, min_seconds=0.0), e2e_steps,
                             world, dev)
    peaks = load_peaks()
    L, D, H, w, Np = wl["layers"], wl["d_model"], wl["heads"], wl["window"], wl["n_persistent"]
    probe = decode_attention_probe(dev, peaks, batch=B, heads=H, dh=D // H, window=w, n_persistent=Np)
    n_params = sum(p.numel() for p in model.parameters())
    del graph, caches, model
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    kv_bytes = B * L * (w + 1) * D * 2 * 2
    step_bytes = kv_bytes + n_params * 2
    ms_step = stats["ms_per_step"]
    return {
        "metric": "decode_tokens_per_s", "value": wl["batch"] / (ms_step * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": dict(workload=wl_name, **wl, batch_per_gpu=B, parallelism=f"batch-sharded x{world}",
                       decode="CUDA-graph step, teacher-forced ids", prefill_seconds=prefill_s,
                       l2="ring caches 10.8 GB per 256 sequences >> 126 MB L2",
                       algorithmic_bytes_per_step_per_gpu=step_bytes),
        "timing": stats,
        "roofline": dict(probe, note="decode attention kernel timed alone on this geometry",
                         step_hbm_frac=step_bytes / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"]),
        "e2e": {"value": wl["batch"] / (e2e_stats["ms_per_step"] * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * 8, "steps": e2e_steps,
                "ms_per_step": e2e_stats["ms_per_step"]},
        "gpu_launches": steps * stats["regions"] * L,
        "clocks": clocks.report(),
    }


def run_decode(args, wl_name: str, wl: dict) -> None:
    line = measure_decode(wl_name, wl, args.steps, args.warmup, _dist_setup(args))
    if line is not None:
        print(json.dumps(line), flush=True)


def run_model_prefill(args, wl_name: str, wl: dict) -> None:
    """benchmark configuration 3: forward of the whole default model over `batch` sequences per GPU (weak scaling).

    FLOPs are the reference forward's: per layer the attention module (QKV, live pairs, output projection) and
    the MLP, plus the LM head over all L rows.  The attention core's share of the step is measured with CUDA
    events around every tmw_prefill call."""
    from titanmac_b200 import TitanMAC, TitanMACConfig, _native

    dist, world, rank, local, dev = _dist_setup(args)
    B, T, D, H, w, Np = wl["batch"], wl["T"], wl["d_model"], wl["heads"], wl["window"], wl["n_persistent"]
    L, V, F_, NL = Np + T, wl["vocab"], wl["d_ff"], wl["layers"]
    cfg = TitanMACConfig(vocab_size=V, d_model=D, n_heads=H, n_layers=NL, d_ff=F_, max_seq_len=T, window_size=w,
                         n_persistent=Np, use_block_sparse=False)
    g = torch.Generator(device="cpu").manual_seed(0)
    model = TitanMAC(cfg).eval()
    with torch.no_grad():  # every weight N(0, 0.02), biases 0, norm scales 1
        for name, prm in model.named_parameters():
            if name.endswith("scale"):
                prm.fill_(1.0)
            elif name.endswith("bias"):
                prm.zero_()
            else:
                prm.copy_(torch.randn(prm.shape, generator=g) * 0.02)
    model = model.to(device=dev, dtype=torch.bfloat16)
    g = torch.Generator(device="cpu").manual_seed(1 + rank)
    ids = [torch.randint(0, V, (B, T), generator=g).to(dev) for _ in range(2)]
    lf = layer_flops(wl)
    flops = NL * (lf["total"] + 2 * 2 * B * L * D * F_) + 2 * B * L * D * V
    core_flops = NL * lf["core"]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        model(ids[i % 2])
    events = []
    for layer in model.layers:
        layer.attention.core_events = events
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(physical_gpu_index(local)) as clocks:
        barrier()
        a.record()
        for i in range(args.steps):
            out = model(ids[i % 2])["logits"]
        b.record()
        barrier()
    ms = a.elapsed_time(b)
    core_ms = sum(x.elapsed_time(y) for x, y in events) / args.steps
    for layer in model.layers:
        layer.attention.core_events = None
    _native.poll_status(dev)

    # end to end: token ids from pinned host memory, the last position's logits back to the host
    ids_host = ids[0].cpu().pin_memory()
    ids_dev = torch.empty_like(ids[0])
    last_host = torch.empty((B, V), dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for _ in range(e2e_steps):
        ids_dev.copy_(ids_host, non_blocking=True)
        last_host.copy_(model(ids_dev)["logits"][:, -1], non_blocking=True)
    e2.record()
    barrier()
    e2e_ms = s2.elapsed_time(e2)

    t = torch.tensor([ms, core_ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, core_ms, e2e_ms = (float(v) for v in t.cpu())
    if rank == 0:
        peaks = load_peaks()
        value = flops * world * args.steps / (ms * 1e-3) / 1e12
        achieved = core_flops / (core_ms * 1e-3) / 1e12
        line = {
            "metric": "model_prefill_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": dict(workload=wl_name, **wl, global_batch=B * world, parallelism=f"batch-sharded x{world}",
                           l2="activations and logits per step (> 2 GB) exceed the 126 MB L2",
                           flops_per_step_per_gpu=flops, attention_core_flops_per_step_per_gpu=core_flops),
            "roofline": {"bound": "tensor", "kernel": "attention core (tmw_prefill), 16 launches per step",
                         "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16_tflops"], "peak_source": f"{peaks['source']} bf16 burst",
                         "core_ms_per_step": core_ms, "core_share_of_step": core_ms / (ms / args.steps),
                         "step_frac_of_peak": value / world / peaks["bf16_tflops"], "traffic": None},
            "e2e": {"value": flops * world * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": B * T * 8, "d2h_bytes_per_step": B * V * 2, "steps": e2e_steps,
                    "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": args.steps * NL,
            "clocks": clocks.report(),
        }
        print(json.dumps(line), flush=True)


def train_flops(wl: dict) -> dict:
    """Forward + backward of the layer: every GEMM three times, the core 3.5 times (forward 4 dh per live pair;
    backward recomputes S and forms dP, dV, dQ, dK: 10 dh per live pair)."""
    f = layer_flops(wl)
    return dict(core_fwd=f["core"], core_bwd=f["core"] * 5 // 2, gemm=3 * (f["qkv"] + f["out"]),
                total=f["core"] * 7 // 2 + 3 * (f["qkv"] + f["out"]))


def run_train(args, wl_name: str, wl: dict) -> None:
    """Forward + backward of one attention layer per step (weak scaling, no gradient exchange: the layer is
    timed in isolation).  The backward of the attention core is `tmw_prefill_backward`."""
    from oracle import windowed_oracle as wo
    from titanmac_b200 import WindowConfig, WindowedAttention, _native

    dist, world, rank, local, dev = _dist_setup(args)
    torch.set_grad_enabled(True)
    B, T, D, H, w, Np = wl["batch"], wl["T"], wl["d_model"], wl["heads"], wl["window"], wl["n_persistent"]
    L = Np + T
    x_cpu, w_qkv, w_out = wo.layer_inputs(B, T, D, Np, seed=rank)
    bs = wl.get("block_size", 0)
    if bs:
        from titanmac_b200 import BlockSparseAttention

        mod = BlockSparseAttention(d_model=D, n_heads=H, window_size=w, block_size=bs, n_persistent=Np,
                                   conv_kernel=wl["conv_taps"])
        with torch.no_grad():
            for conv, wt in zip((mod.conv_q, mod.conv_k, mod.conv_v), block_sparse_conv_weights(wl, seed=rank)):
                conv.weight.copy_(wt[:, None, :])
    else:
        mod = WindowedAttention(WindowConfig(window_size=w, num_heads=H, head_dim=D // H, n_persistent=Np))
    with torch.no_grad():
        mod.qkv_proj.weight.copy_(w_qkv)
        mod.out_proj.weight.copy_(w_out)
    mod = mod.to(device=dev, dtype=torch.bfloat16)
    xs = [(x_cpu.to(torch.bfloat16) + 0.001 * i).to(dev).requires_grad_(True) for i in range(4)]
    g = torch.randn(B, L, D, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).to(dev)
    flops = train_flops(wl)

    def step(i):
        x = xs[i % 4]
        x.grad = None
        mod.zero_grad(set_to_none=True)
        mod(x).backward(g)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(physical_gpu_index(local)) as clocks:
        barrier()
        a.record()
        for i in range(args.steps):
            step(i)
        b.record()
        barrier()
    ms = a.elapsed_time(b)
    _native.poll_status(dev)

    # the backward kernels alone (saved tensors of one forward)
    qkv = torch.randn(B, L, 3, H, D // H, device=dev).to(torch.bfloat16)
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    lse = torch.empty(B * H * L, dtype=torch.float32, device=dev)
    o = _native.prefill(q, k, v, w, Np, lse=lse, window_block=bs)
    d_o = torch.empty_like(o)
    d_o.normal_()
    dqkv = torch.empty_like(qkv)
    dq, dk, dv = (dqkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    for _ in range(2):
        _native.prefill_backward(q, k, v, o, d_o, lse, dq, dk, dv, w, Np, window_block=bs)
    c, d_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_core = 5
    c.record()
    for _ in range(n_core):
        _native.prefill_backward(q, k, v, o, d_o, lse, dq, dk, dv, w, Np, window_block=bs)
    d_.record()
    torch.cuda.synchronize()
    core_ms = c.elapsed_time(d_) / n_core

    # end to end: input and output gradient from pinned host memory, input gradient back
    x_host = x_cpu.to(torch.bfloat16).pin_memory()
    g_host = g.cpu().pin_memory()
    dx_host = torch.empty((B, L, D), dtype=torch.bfloat16).pin_memory()
    x_dev = torch.empty((B, L, D), dtype=torch.bfloat16, device=dev, requires_grad=True)
    g_dev = torch.empty_like(g)
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step():
        with torch.no_grad():
            x_dev.copy_(x_host, non_blocking=True)
            g_dev.copy_(g_host, non_blocking=True)
        x_dev.grad = None
        mod.zero_grad(set_to_none=True)
        mod(x_dev).backward(g_dev)
        dx_host.copy_(x_dev.grad, non_blocking=True)

    e2e_step()
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for _ in range(e2e_steps):
        e2e_step()
    e2.record()
    barrier()
    e2e_ms = s2.elapsed_time(e2)

    t = torch.tensor([ms, core_ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, core_ms, e2e_ms = (float(x) for x in t.cpu())
    if rank == 0:
        peaks = load_peaks()
        achieved = flops["core_bwd"] / (core_ms * 1e-3) / 1e12
        line = {
            "metric": "windowed_attn_layer_train_tflops", "value": flops["total"] * world * args.steps / (ms * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": dict(workload=wl_name, **wl, global_batch=B * world, parallelism=f"batch-sharded x{world}",
                           l2="inputs rotate over 4 sets; activations + gradients per step > 126 MB L2",
                           flops_per_step_per_gpu=flops),
            "roofline": {"bound": "tensor", "kernel": "attention-core backward (tmw_prefill_backward / "
                         "tmw_prefill_block_sparse_backward: dQ and dK/dV launches of the tcgen05 kernel)", "achieved": achieved, "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
                         "peak_source": f"{peaks['source']} bf16 burst", "avg_launch_ms": core_ms, "traffic": NCU_TRAFFIC_BYTES.get(wl_name),
                         "algorithmic_flops_per_launch": flops["core_bwd"]},
            "e2e": {"value": flops["total"] * world * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": 2 * x_host.numel() * 2, "d2h_bytes_per_step": dx_host.numel() * 2,
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": args.steps * 3,
            "clocks": clocks.report(),
        }
        print(json.dumps(line), flush=True)


def measure_long(wl_name: str, wl: dict, steps: int, warmup: int, ctx, shard_overlap: int = 0,
                 min_seconds: float = MIN_TIMED_SECONDS, with_e2e: bool = True):
    """benchmark configuration 5: attention core over one long sequence, rows sharded over the GPUs with a K/V halo.

    Every rank draws the SAME whole-length Q, K, V on its own GPU (seeded device generator) and keeps its rows,
    so that after the timed region sampled row blocks of the sharded output - the first rows behind the shard
    boundary, an interior block, the last rows - can be held against the CPU oracle, for both forms of the
    exchange.  The unsharded kernel is timed on the same data (efficiency = its time / (N x the sharded step))."""
    from oracle import windowed_oracle as wo  # checker for the sampled row blocks (outside the timed region)
    from titanmac_b200 import _native, shard

    dist, world, rank, local, dev = ctx
    barrier = make_barrier(dist, world)
    H, w, Np = wl["heads"], wl["window"], wl["n_persistent"]
    dh = wl["d_model"] // H
    Ltot = Np + wl["T"]
    bounds = shard.shard_bounds(Ltot, Np, world)
    r0, r1 = bounds[rank]
    own = r1 - r0
    g = torch.Generator(device=dev).manual_seed(100)
    whole = [torch.randn(1, Ltot, H, dh, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
             .permute(0, 2, 1, 3) for _ in range(3)]
    q, k, v = (t[:, :, r0:r1] for t in whole)
    flops = H * live_pairs(Ltot, w, Np) * 4 * dh

    # the whole sequence on one GPU: the N = 1 kernel time that the sharded step is held against
    for _ in range(2):
        _native.prefill(*whole, w, Np)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(5):
        _native.prefill(*whole, w, Np)
    b.record()
    torch.cuda.synchronize()
    n1_ms = float(gather_ranks([a.elapsed_time(b) / 5], world, dev)[:, 0].median())

    kv = pkv = None
    if world > 1:
        # K and V of this rank live in the sharded buffers from the start (the producer writes them there).
        # Two forms of the step: "push" - every rank's GPU writes the halo / persistent rows into its neighbours'
        # buffers and the attention kernel polls a flag (no host-side collective; the timed form) - and "nccl" -
        # one batch of in-place sends / receives, then the launch(es).
        kv = shard.ShardedKV.allocate(1, H, dh, Ltot, w, Np, torch.bfloat16, dev)
        kv.k_own.copy_(k)
        kv.v_own.copy_(v)
        try:
            pkv = shard.PeerShardedKV.allocate(1, H, dh, Ltot, w, Np, torch.bfloat16, dev)
            pkv.k_own.copy_(k)
            pkv.v_own.copy_(v)
        except ValueError:  # shards shorter than the window
            pkv = None
    form = "single GPU" if world == 1 else ("push" if pkv is not None and not shard_overlap else "nccl")

    def run(which):
        if world == 1:
            return _native.prefill(q, k, v, w, Np)
        if which == "push":
            return shard.pushed_prefill(q, pkv)
        return shard.sharded_prefill(q, None, None, Ltot, w, Np, kv=kv, overlap=(which == "nccl-overlap"))

    timed = form if form != "nccl" else ("nccl-overlap" if shard_overlap else "nccl")
    for _ in range(warmup):
        run(timed)
    with ClockSampler(physical_gpu_index(local)) as clocks:
        regions = timed_regions(lambda i: run(timed), steps, barrier, world, dev, min_seconds=min_seconds,
                                max_regions=20)
    stats = region_stats(regions, steps, world, dev)
    _native.poll_status(dev)
    other = None
    if world > 1 and form == "push":  # the collective form beside it
        for _ in range(2):
            run("nccl")
        other = region_stats(timed_regions(lambda i: run("nccl"), steps, barrier, world, dev, min_seconds=0.0), steps,
                             world, dev)["ms_per_step"]

    # ---- parity of the sharded output (outside the timed region) -------------------------
    worst = 0.0
    blocks = sorted({0, max(0, min(own - 64, w)), max(0, own // 2), max(0, own - 64)})
    kc_pers = [t[:, :, :Np].float().cpu() for t in whole[1:]]
    forms = ["single GPU"] if world == 1 else (["push"] if pkv is not None else []) + ["nccl", "nccl-overlap"]
    for which in forms:
        o = run(which)
        torch.cuda.synchronize()
        _native.poll_status(dev)
        for b0 in blocks:
            row0, n = r0 + b0, min(64, own - b0)
            lo = max(Np, row0 - w)
            # the oracle is given [persistent | the window of these rows]: rows renumbered from Np + (row0 - lo)
            kk, vv = (torch.cat([pers, t[:, :, lo:row0 + n].float().cpu()], dim=2)
                      for pers, t in zip(kc_pers, whole[1:]))
            qq = whole[0][:, :, row0:row0 + n].float().cpu()
            ref = wo.attention_core_rows(qq, kk, vv, Np + (row0 - lo), w, Np) if row0 >= Np else \
                wo.attention_core_rows(qq, kk, vv, row0, w, Np)
            worst = max(worst, (o[:, :, b0:b0 + n].float().cpu() - ref).abs().max().item())
    worst = float(gather_ranks([worst], world, dev)[:, 0].max())

    e2e = None
    if with_e2e:
        # end to end: this rank's rows of Q, K, V from pinned host memory, its rows of O back
        hosts = [x.contiguous().cpu().pin_memory() for x in (q, k, v)]
        devs = [torch.empty_like(x.contiguous()) for x in (q, k, v)]
        o_host = torch.empty((1, H, own, dh), dtype=torch.bfloat16).pin_memory()
        e2e_steps = max(2, min(steps, 5))

        def e2e_step(i):
            for d_, h_ in zip(devs, hosts):
                d_.copy_(h_, non_blocking=True)
            o = _native.prefill(*devs, w, Np) if world == 1 else shard.sharded_prefill(*devs, Ltot, w, Np)
            o_host.copy_(o, non_blocking=True)

        e2e_step(0)
        es = region_stats(timed_regions(e2e_step, e2e_steps, barrier, world, dev, min_seconds=0.0), e2e_steps,
                          world, dev)
        e2e = {"value": flops / (es["ms_per_step"] * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": 3 * hosts[0].numel() * 2, "d2h_bytes_per_step": o_host.numel() * 2,
               "steps": e2e_steps, "ms_per_step": es["ms_per_step"]}
    if pkv is not None:
        pkv.close()
    barrier()
    del whole, kv, pkv
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    peaks = load_peaks()
    ms_step = stats["ms_per_step"]
    value = flops / (ms_step * 1e-3) / 1e12
    line = {
        "metric": "windowed_attn_core_prefill_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": dict(workload=wl_name, **wl, parallelism=f"sequence-sharded x{world}, halo {w} rows",
                       shard_overlap=bool(shard_overlap), exchange=form,
                       exchange_forms="push: tmw_halo_push into the neighbours' buffers + flag polling in the "
                                      "attention kernel; nccl: batch_isend_irecv, then the launch",
                       l2="Q+K+V+O = 2.1 GB per step > 126 MB L2", algorithmic_flops_per_step=flops),
        "timing": stats,
        "unsharded_kernel_ms": n1_ms, "efficiency_vs_unsharded_kernel": n1_ms / (world * ms_step),
        "nccl_exchange_ms_per_step": other,
        "check": {"what": "sampled 64-row blocks of every rank (first rows of the shard, behind the halo, middle, "
                          "last) against the CPU oracle, exchange forms: " + ", ".join(forms),
                  "max_abs_err": worst, "tolerance": 2e-2, "pass": bool(worst <= 2e-2)},
        "roofline": {"bound": "tensor", "kernel": "attention core (tmw_prefill)", "achieved": value / world,
                     "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": value / world / peaks["bf16_tflops"],
                     "peak_source": f"{peaks['source']} bf16 burst", "traffic": None,
                     "note": "per GPU, halo exchange included when sharded"},
        "gpu_launches": steps * stats["regions"] * (1 if world == 1 else 3 if form == "push" else 2 if shard_overlap else 1),
        "clocks": clocks.report(),
    }
    if e2e is not None:
        line["e2e"] = e2e
    return line


def run_long(args, wl_name: str, wl: dict) -> None:
    line = measure_long(wl_name, wl, args.steps, args.warmup, _dist_setup(args), args.shard_overlap)
    if line is not None:
        print(json.dumps(line), flush=True)


def measure_strong_config2(steps: int, warmup: int, ctx) -> dict:
    """benchmark configuration 2 as it is stated: ONE batch of 8 sequences split over the GPUs (8 / N per GPU)."""
    from titanmac_b200 import _native

    dist, world, rank, local, dev = ctx
    barrier = make_barrier(dist, world)
    wl = dict(WORKLOADS["config2_layer_prefill"])
    if wl["batch"] % world:
        return {"unavailable": f"batch {wl['batch']} does not divide by {world} GPUs"}
    whole_flops = layer_flops(wl)["total"]
    wl["batch"] //= world
    mod, x_cpu = make_layer(wl, rank, dev, torch.bfloat16)
    n_sets = max(4, 4 * world)  # 210 MB / N per set: keep the rotation larger than L2
    xs = [(x_cpu.to(torch.bfloat16) + 0.001 * i).to(dev) for i in range(n_sets)]
    for i in range(warmup):
        mod(xs[i % n_sets])
    stats = region_stats(timed_regions(lambda i: mod(xs[i % n_sets]), steps, barrier, world, dev, min_seconds=0.2),
                         steps, world, dev)
    _native.poll_status(dev)
    return {"metric": METRIC, "value": whole_flops / (stats["ms_per_step"] * 1e-3) / 1e12, "unit": "TFLOP/s",
            "scaling": "strong", "global_batch": 8, "batch_per_gpu": wl["batch"], "timing": stats}


def measure_extras(args, dist, world, rank, local, dev, barrier) -> dict:
    """The benchmark's other configurations, measured after the headline workload and carried in its line."""
    ctx = (dist, world, rank, local, dev)
    extra = {}
    d = measure_decode("config4_decode", WORKLOADS["config4_decode"], 64, 5, ctx, min_seconds=0.0)
    lg = measure_long("config5_long_prefill", WORKLOADS["config5_long_prefill"], 10, 3, ctx, min_seconds=0.0,
                      with_e2e=False)
    st = measure_strong_config2(20, 5, ctx)
    if rank == 0:
        extra["config4_decode"] = {"value": d["value"], "unit": d["unit"], "ms_per_step": d["ms_per_step"],
                                   "scaling": "strong", "batch_per_gpu": d["config"]["batch_per_gpu"],
                                   "step_hbm_frac": d["roofline"]["step_hbm_frac"],
                                   "attention_kernel": {k_: d["roofline"][k_] for k_ in
                                                        ("achieved", "peak", "unit", "frac", "avg_launch_ms")},
                                   "timing": d["timing"], "e2e": d["e2e"]}
        key = "config5_core" if world == 1 else "config5_sequence_sharded"
        extra[key] = {"value": lg["value"], "unit": lg["unit"], "ms_per_step": lg["ms_per_step"],
                      "scaling": "strong", "frac_of_bf16_peak_per_gpu": lg["roofline"]["frac"],
                      "unsharded_kernel_ms": lg["unsharded_kernel_ms"],
                      "efficiency_vs_unsharded_kernel": lg["efficiency_vs_unsharded_kernel"],
                      "exchange": lg["config"]["exchange"], "nccl_exchange_ms_per_step": lg["nccl_exchange_ms_per_step"],
                      "check": lg["check"], "timing": lg["timing"]}
        extra["config2_strong"] = st
    return extra


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="config2_layer_prefill")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (N=1 only)")
    ap.add_argument("--no-extra", action="store_true",
                    help="default workload only: skip the decode, long-context and strong-scaling measurements")
    ap.add_argument("--shard-overlap", type=int, choices=[0, 1], default=0,
                    help="config5_long_prefill on several GPUs: 1 = rows that need no halo are launched before the "
                         "halo exchange (two launches), 0 = one exchange, then one launch")
    args = ap.parse_args()
    torch.set_grad_enabled(False)  # inference workloads: nothing is saved for a backward pass
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        if "layer_prefill" not in args.workload:  # (the train, model, decode and long-context workloads)
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable":
                                  "the CPU reference arm is timed on the layer workloads only"}), flush=True)
            return
        run_reference_arm(args, args.workload, wl)
    elif args.workload in ("config2_layer_train", "config2_block_sparse_layer_train"):
        run_train(args, args.workload, wl)
    elif args.workload == "config3_model_prefill":
        run_model_prefill(args, args.workload, wl)
    elif args.workload == "config4_decode":
        run_decode(args, args.workload, wl)
    elif args.workload == "config5_long_prefill":
        run_long(args, args.workload, wl)
    else:
        run_ours(args, args.workload, wl)
    if _DIST is not None and _DIST[1] > 1:
        _DIST[0].destroy_process_group()


if __name__ == "__main__":
    main()
