#!/usr/bin/env python
"""Benchmark of the routed-expert MoE layer (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--no-points]

A step is one forward of the DeepSeek-V3-scale MoE layer (H=7168, I=2048, E=256, top-8) over one
batch of synthetic tokens.  The headline workload is the BF16 decode configuration (T=64, near-uniform
routing): 19.5 GB of expert weights are streamed per step, far more than the 126 MB L2, so no L2
flush is needed between iterations.  At N>1 the same batch is run expert-parallel: experts and tokens
are split evenly over the ranks and rows travel by NCCL all-to-all (strong scaling).

value  : tokens/s with every input resident in HBM, CUDA events on the launch stream, max over ranks.
e2e    : the same metric through the public op (fused_cpp_b200.moe.fused_moe_tiled) with the step's
         activations and top-k arrays copied from pinned host memory and the output copied back, all
         inside the timed region.
roofline: the gate_up grouped GEMM (the dominant kernel), timed per launch by the library's stage
         timer (CUDA events around that kernel) during the timed steps.
cpu_baseline / --impl reference: the CPU port of the reference arithmetic (oracle/) on the host cores,
         on a bounded sample of the same batch.  The reference's native kernels are AArch64-only.
"""
from __future__ import annotations

import argparse
import atexit
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

H, I, E, K = 7168, 2048, 256, 8
WORKLOADS = {
    "bf16_decode_v3_T64": {"kind": "bf16", "tokens": 64, "skew": False},
    "bf16_decode_v3_T32": {"kind": "bf16", "tokens": 32, "skew": False},
    "bf16_decode_v3_T8": {"kind": "bf16", "tokens": 8, "skew": False},
    "bf16_decode_v3_T1": {"kind": "bf16", "tokens": 1, "skew": False},
    "w8a8_decode_v3_T64": {"kind": "int8", "tokens": 64, "skew": False},
    "w8a8_prefill_v3_T8192": {"kind": "int8", "tokens": 8192, "skew": False},
    "w8a8_prefill_v3_T16384": {"kind": "int8", "tokens": 16384, "skew": False},
    "bf16_prefill_v3_T8192": {"kind": "bf16", "tokens": 8192, "skew": False},
    "w8a8_ep_shared_v3_T16384": {"kind": "int8", "tokens": 16384, "skew": False, "shared": True},
    "w8a8_prefill_v3_T2048": {"kind": "int8", "tokens": 2048, "skew": False},
    # Zipf-biased router logits (a few experts take most routes): the compute-bound prefill configuration.
    "w8a8_prefill_zipf_v3_T8192": {"kind": "int8", "tokens": 8192, "skew": True},
    "w8a8_prefill_zipf_v3_T2048": {"kind": "int8", "tokens": 2048, "skew": True},
    "bf16_prefill_zipf_v3_T8192": {"kind": "bf16", "tokens": 8192, "skew": True},
}
DEFAULT_WORKLOAD = "bf16_decode_v3_T64"
EXTRA_POINTS = ["bf16_decode_v3_T1", "bf16_decode_v3_T8", "bf16_decode_v3_T32", "w8a8_decode_v3_T64", "w8a8_prefill_zipf_v3_T8192",
                "w8a8_prefill_v3_T8192"]
CPU_SAMPLE_TOKENS = 16
SEED = 20260101


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as stream:
            data = json.load(stream)
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data.get("bf16_tflops", 0.0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def ncu_traffic_bytes(workload: str) -> float | None:
    """DRAM bytes per launch of the gate_up kernel from the committed ncu summary, if one covers the workload."""
    path = os.path.join(ROOT, "profiles", f"gate_up_gemm_{workload}.md")
    if not os.path.exists(path):
        return None
    with open(path) as stream:
        for line in stream:
            if line.startswith("dram_bytes_per_launch:"):
                return float(line.split(":", 1)[1].split()[0])
    return None


_SAMPLER_CHILD = r"""
import sys, time
import pynvml as nvml
nvml.nvmlInit()
uuid, index, period = sys.argv[1], int(sys.argv[2]), float(sys.argv[3])
try:
    handle = nvml.nvmlDeviceGetHandleByUUID(uuid.encode())
except Exception:
    handle = nvml.nvmlDeviceGetHandleByIndex(index)
print("max", nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM), flush=True)
while True:
    clock = nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM)
    reasons = nvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
    print("s", repr(time.time()), clock, reasons, flush=True)
    time.sleep(period)
"""


class ClockSampler:
    """SM clock and clock-event reasons of one GPU during a timed region, sampled through NVML by a child process
    (a thread of the timing process would compete with the launches for the interpreter lock).  The child is
    started once per GPU and keeps sampling; a region keeps the samples whose time stamps fall inside it."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}
    _children: dict = {}

    def __init__(self, device_index: int, period_s: float = 0.01):
        self.device_index = device_index
        self.period_s = period_s
        self.begin = None
        self.error = None

    def _child(self):
        import queue
        import subprocess
        import threading

        entry = ClockSampler._children.get(self.device_index)
        if entry is not None:
            return entry
        uuid = str(torch.cuda.get_device_properties(self.device_index).uuid)
        if not uuid.startswith("GPU-"):
            uuid = "GPU-" + uuid
        process = subprocess.Popen([sys.executable, "-c", _SAMPLER_CHILD, uuid, str(self.device_index), str(self.period_s)],
                                   stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        lines: "queue.Queue[str]" = queue.Queue()

        def pump():
            for line in process.stdout:
                lines.put(line)

        threading.Thread(target=pump, daemon=True).start()
        entry = {"process": process, "lines": lines, "max": None, "samples": []}
        ClockSampler._children[self.device_index] = entry
        atexit.register(process.kill)
        try:  # wait until the child is sampling, so that a short region is not over before its first sample
            deadline = time.time() + 20.0
            while time.time() < deadline and not entry["samples"]:
                self._drain(entry, block=True)
        except Exception as error:  # noqa: BLE001
            self.error = repr(error)
        return entry

    @staticmethod
    def _drain(entry, block: bool = False) -> None:
        import queue

        while True:
            try:
                line = entry["lines"].get(timeout=0.2) if block else entry["lines"].get_nowait()
            except queue.Empty:
                return
            block = False
            parts = line.split()
            if parts and parts[0] == "max":
                entry["max"] = int(parts[1])
            elif parts and parts[0] == "s":
                entry["samples"].append((float(parts[1]), int(parts[2]), int(parts[3])))

    def prepare(self) -> None:
        """Starts the child if it is not running yet (takes a second or two: call it before the ranks line up)."""
        try:
            self._child()
        except Exception as error:  # noqa: BLE001
            self.error = repr(error)

    def start(self) -> None:
        self.prepare()
        self.begin = time.time()

    def stop(self) -> dict:
        end = time.time()
        entry = ClockSampler._children.get(self.device_index)
        clocks, bits, maximum = [], 0, None
        if entry is not None:
            time.sleep(2.5 * self.period_s)  # let the sample that follows the region arrive
            self._drain(entry)
            maximum = entry["max"]
            inside = [s for s in entry["samples"] if self.begin <= s[0] <= end]
            if not inside:  # a region shorter than the period: the samples next to it
                inside = sorted(entry["samples"], key=lambda s: min(abs(s[0] - self.begin), abs(s[0] - end)))[:2]
            clocks = [s[1] for s in inside]
            for s in inside:
                bits |= s[2]
            entry["samples"] = entry["samples"][-8:]
        reasons = sorted(name for bit, name in self.REASONS.items() if bits & bit)
        result = {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": maximum, "reasons": reasons,
                  "samples": len(clocks), "source": "nvml (child process)"}
        if self.error:
            result["error"] = self.error
        return result


def make_layer(kind: str, device: torch.device, seed: int, experts: int | None = None):
    """Random-init weights of the layer on the device (values do not affect timing; parity is tested elsewhere)."""
    experts = E if experts is None else experts
    generator = torch.Generator(device=device).manual_seed(seed)
    if kind == "int8":
        w13 = torch.randint(-127, 128, (experts, 2 * I, H), generator=generator, dtype=torch.int8, device=device)
        w2 = torch.randint(-127, 128, (experts, H, I), generator=generator, dtype=torch.int8, device=device)
        s13 = (torch.rand((experts, 2 * I), generator=generator, device=device) * 1.5 + 0.5) / (127.0 * H ** 0.5)
        s2 = (torch.rand((experts, H), generator=generator, device=device) * 1.5 + 0.5) / (127.0 * I ** 0.5)
        return {"w13": w13, "w2": w2, "s13": s13, "s2": s2}
    w13 = torch.empty((experts, 2 * I, H), dtype=torch.bfloat16, device=device).normal_(0.0, 0.02, generator=generator)
    w2 = torch.empty((experts, H, I), dtype=torch.bfloat16, device=device).normal_(0.0, 0.02, generator=generator)
    return {"w13": w13, "w2": w2, "s13": None, "s2": None}


def make_batch(tokens: int, skew: bool, seed: int):
    from fused_cpp_b200 import synthetic

    topk_w, topk_ids = synthetic.make_routing(tokens, E, K, seed, skew)
    x = synthetic.make_activations(tokens, H, seed + 1)
    return x, topk_w, topk_ids


def layer_work(kind: str, tokens: int, topk_ids: torch.Tensor) -> dict:
    from fused_cpp_b200 import synthetic

    shape = synthetic.MoEShape(tokens=tokens, hidden=H, inter=I, experts=E, top_k=K)
    return synthetic.algorithmic_work(shape, topk_ids, 1 if kind == "int8" else 2)


def gate_up_roofline(kind: str, nbytes: float, ops: float, ms: float, peaks: dict, traffic) -> dict:
    """Roofline entry of the gate_up grouped GEMM (the dominant kernel) for one launch.

    The bound is whichever of bytes / HBM peak and ops / tensor peak takes longer.  HBM peak and the bf16 tensor
    peak are the measured figures of this pool (a plain copy, a cuBLAS GEMM); the int8 tensor peak is taken as
    twice the measured bf16 one (kind::i8 MMAs run at twice the kind::f16 rate on this part)."""
    seconds = ms * 1e-3
    tensor_peak = peaks["bf16_tflops"] * (2.0 if kind == "int8" else 1.0)
    t_hbm = nbytes / (peaks["hbm_gbs"] * 1e9)
    t_mma = ops / (tensor_peak * 1e12)
    gbs = nbytes / seconds / 1e9 if seconds > 0 else 0.0
    tops = ops / seconds / 1e12 if seconds > 0 else 0.0
    entry = {"kernel": "umma_grouped_gemm_kernel<gate_up> / umma_pair_grouped_gemm_kernel<gate_up>", "traffic": traffic,
             "peak_source": peaks["source"], "algorithmic_bytes_per_launch": nbytes, "ops_per_launch": ops, "ms_per_launch": ms,
             "hbm": {"achieved_gbs": gbs, "peak_gbs": peaks["hbm_gbs"], "frac": gbs / peaks["hbm_gbs"]},
             "tensor": {"achieved_tops": tops, "peak_tops": tensor_peak, "frac": tops / tensor_peak,
                        "peak_note": "measured cuBLAS bf16 burst" + (" x 2 for int8" if kind == "int8" else "")}}
    if t_mma > t_hbm:
        entry.update({"bound": "tensor", "achieved": tops, "peak": tensor_peak, "unit": "TFLOP/s" if kind != "int8" else "TOP/s",
                      "frac": tops / tensor_peak})
    else:
        entry.update({"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"]})
    return entry


def gate_up_bytes(kind: str, tokens: int, active: int) -> float:
    """Algorithmic bytes of one gate_up launch: W13 of the active experts once (+ scales), the sorted
    activation rows in, the bf16 SwiGLU rows out."""
    b = 1 if kind == "int8" else 2
    rows = tokens * K
    total = active * 2 * I * H * b + rows * H * b + rows * I * 2
    if kind == "int8":
        total += active * 2 * I * 4 + rows * 4
    return float(total)


def run_point(name: str, layer: dict, device: torch.device, steps: int, warmup: int, with_e2e: bool, sampler: ClockSampler | None):
    from fused_cpp_b200 import _lib
    from fused_cpp_b200 import moe

    spec = WORKLOADS[name]
    kind, tokens = spec["kind"], spec["tokens"]
    x_host, w_host, ids_host = make_batch(tokens, spec["skew"], SEED)
    x, tw, ids = x_host.to(device), w_host.to(device), ids_host.to(device)
    work = layer_work(kind, tokens, ids_host)
    timer = _lib.StageTimer(steps)

    def step(stage_timer=None):
        return _lib.moe_forward(x, layer["w13"], layer["w2"], tw, ids, s13=layer["s13"], s2=layer["s2"], stage_timer=stage_timer)

    for _ in range(warmup):
        step()
    result = step()
    result.raise_for_status()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    # Timed region 1 (the headline): K steps replayed from a CUDA graph of one forward, so that the host's
    # launch cost (8 launches per step through ctypes) does not sit between the kernels.  The forward makes no
    # host read, so it is capturable as it is.  Falls back to eager launches if capture is refused.
    graph = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        graph.replay()
        torch.cuda.synchronize()
    except Exception as error:  # noqa: BLE001
        graph = None
        sys.stderr.write(f"[bench] CUDA graph capture unavailable, timing eager launches: {error!r}\n")
        torch.cuda.synchronize()
    if sampler is not None:
        sampler.start()
    start.record()
    for _ in range(steps):
        if graph is not None:
            graph.replay()
        else:
            step()
    stop.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler is not None else None
    ms_per_step = start.elapsed_time(stop) / steps

    # Timed region 2: the same K steps launched eagerly with the library's stage timer (CUDA events around
    # every stage on the launch stream); this is where the per-kernel durations of the roofline come from.
    start.record()
    for _ in range(steps):
        step(timer)
    stop.record()
    torch.cuda.synchronize()
    eager_ms_per_step = start.elapsed_time(stop) / steps
    stage_ms = {stage: 0.0 for stage in _lib.STAGES}
    for call in range(timer.calls):
        for stage, value in timer.read(call).items():
            stage_ms[stage] += value / timer.calls
    timer.close()

    peaks = measured_peaks()
    gu_bytes = gate_up_bytes(kind, tokens, work["active_experts"])
    gu_ms = stage_ms["gate_up"]
    traffic = ncu_traffic_bytes(name)
    point = {
        "workload": name, "tokens": tokens, "dtype": "bf16" if kind == "bf16" else "int8(w8a8)", "ms_per_step": ms_per_step,
        "launch_mode": "cuda_graph_replay" if graph is not None else "eager", "eager_ms_per_step": eager_ms_per_step,
        "value": tokens / (ms_per_step * 1e-3), "active_experts": work["active_experts"],
        "stage_ms": {k: round(v, 5) for k, v in stage_ms.items()},
        "roofline": gate_up_roofline(kind, gu_bytes, 2.0 * tokens * K * 2 * I * H, gu_ms, peaks, traffic),
        "layer": {"algorithmic_bytes": work["bytes"], "ops": work["ops"], "hbm_gbs": work["bytes"] / (ms_per_step * 1e-3) / 1e9,
                  "hbm_frac": work["bytes"] / (ms_per_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
                  "tops": work["ops"] / (ms_per_step * 1e-3) / 1e12},
        # route build (1 kernel up to 1024 routes, else 3) + quantise/gather + gate_up (+ requantise) + down + merge
        "gpu_launches_per_step": (1 if tokens * K <= 1024 else 3) + (5 if kind == "int8" else 4),
    }
    if clocks is not None:
        point["clocks"] = clocks

    if with_e2e:
        # Public API, host buffers: H2D of x / top-k weights / ids, the op (with its status check), D2H of out.
        if kind == "int8":
            prepared = moe.PreparedW8A8TiledFusedMoEWeights(w13=(layer["w13"], H, 2 * I, layer["s13"]), w2=(layer["w2"], I, H, layer["s2"]))
        else:
            prepared = moe.PreparedBF16TiledFusedMoEWeights(w13=(layer["w13"], H, 2 * I), w2=(layer["w2"], I, H), fused_silu=True)
        runtime = moe.MoePlannerRuntime(None, hidden_size=H, intermediate_size=I, global_experts=E, local_experts=E)
        previous = moe.set_default_moe_planner_runtime(runtime)
        try:
            x_pin, w_pin, ids_pin = x_host.pin_memory(), w_host.pin_memory(), ids_host.pin_memory()
            out_pin = torch.empty((tokens, H), dtype=torch.bfloat16).pin_memory()
            out_dev = torch.empty((tokens, H), dtype=torch.bfloat16, device=device)

            def e2e_step():
                xd = x_pin.to(device, non_blocking=True)
                wd = w_pin.to(device, non_blocking=True)
                idd = ids_pin.to(device, non_blocking=True)
                kwargs = {"swiglu_limit": 10.0} if kind == "int8" else {}
                moe.fused_moe_tiled(xd, prepared, wd, idd, out=out_dev, **kwargs)
                out_pin.copy_(out_dev, non_blocking=True)

            for _ in range(warmup):
                e2e_step()
            torch.cuda.synchronize()
            start.record()
            for _ in range(steps):
                e2e_step()
            stop.record()
            torch.cuda.synchronize()
            e2e_ms = start.elapsed_time(stop) / steps
        finally:
            moe.set_default_moe_planner_runtime(previous)
        point["e2e"] = {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                        "h2d_bytes_per_step": tokens * H * 2 + tokens * K * 4 + tokens * K * 8,
                        "d2h_bytes_per_step": tokens * H * 2 + 64}
    return point


def cpu_sample_inputs(kind: str, tokens: int, layer: dict | None):
    """The first CPU_SAMPLE_TOKENS tokens of the batch with compacted weights of the experts they hit.
    With `layer` (GPU weights) the experts are copied from the device; otherwise they are generated on the host."""
    x, tw, ids = make_batch(tokens, False, SEED)
    sample = min(CPU_SAMPLE_TOKENS, tokens)
    x, tw, ids = x[:sample].contiguous(), tw[:sample].contiguous(), ids[:sample].contiguous()
    hit = torch.unique(ids)
    remap = torch.full((E,), -1, dtype=torch.int64)
    remap[hit] = torch.arange(hit.numel())
    local_ids = remap[ids]
    if layer is not None:
        index = hit.to(layer["w13"].device)
        weights = {k: (None if v is None else v.index_select(0, index).cpu()) for k, v in layer.items()}
    else:
        generator = torch.Generator().manual_seed(SEED + 7)
        n = hit.numel()
        if kind == "int8":
            base13 = torch.randint(-127, 128, (2 * I, H), generator=generator, dtype=torch.int8)
            base2 = torch.randint(-127, 128, (H, I), generator=generator, dtype=torch.int8)
            weights = {"w13": torch.stack([base13.roll(e, 0) for e in range(n)]), "w2": torch.stack([base2.roll(e, 0) for e in range(n)]),
                       "s13": torch.full((n, 2 * I), 1.0 / (127.0 * H ** 0.5)), "s2": torch.full((n, H), 1.0 / (127.0 * I ** 0.5))}
        else:
            base13 = (torch.randn((2 * I, H), generator=generator) * 0.02).to(torch.bfloat16)
            base2 = (torch.randn((H, I), generator=generator) * 0.02).to(torch.bfloat16)
            weights = {"w13": torch.stack([base13.roll(e, 0) for e in range(n)]), "w2": torch.stack([base2.roll(e, 0) for e in range(n)]),
                       "s13": None, "s2": None}
    return x, tw, local_ids, weights, sample, int(hit.numel())


def time_cpu_port(kind: str, tokens: int, layer: dict | None, warmup: int, passes: int) -> dict:
    """Time `passes` forward passes of the CPU port over one bounded sample (inputs built once)."""
    from oracle import oracle

    x, tw, ids, weights, sample, hit = cpu_sample_inputs(kind, tokens, layer)
    times = []
    for _ in range(warmup + passes):
        begin = time.perf_counter()
        if kind == "int8":
            oracle.w8a8_forward(x, weights["w13"], weights["s13"], weights["w2"], weights["s2"], tw, ids)
        else:
            oracle.bf16_forward(x, weights["w13"], weights["w2"], tw, ids)
        times.append(time.perf_counter() - begin)
    seconds = statistics.mean(times[warmup:])
    cores = len(os.sched_getaffinity(0))
    return {"value": sample / seconds, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"first {sample} of {tokens} tokens ({sample * K} routes, {hit} experts hit); "
                      f"OpenMP C port of the reference arithmetic, mean of {passes} passes after {warmup} warm-up, "
                      f"{seconds * 1e3:.1f} ms per pass",
            "seconds_per_pass": seconds}


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    spec = WORKLOADS[args.workload]
    baseline = time_cpu_port(spec["kind"], spec["tokens"], None, args.warmup, args.steps)
    seconds = baseline.pop("seconds_per_pass")
    value = baseline["value"]
    line = {"impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if spec["kind"] == "bf16" else "int8(w8a8)",
            "data": "synthetic", "config": {"workload": args.workload, "tokens": spec["tokens"], "hidden": H, "inter": I,
                                            "experts": E, "top_k": K, "note": "each step is a bounded sample of the batch on the host cores"},
            "cpu_baseline": baseline,
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_single_gpu(args) -> None:
    from fused_cpp_b200 import _lib

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    if not _lib.device_supported():
        raise SystemExit("bench.py needs a compute-capability-10.x GPU: the library has no other path")
    spec = WORKLOADS[args.workload]
    layers: dict[str, dict] = {}

    def layer_for(kind: str) -> dict:
        if kind not in layers:
            layers[kind] = make_layer(kind, device, SEED + 2)
        return layers[kind]

    sampler = ClockSampler(0)
    head = run_point(args.workload, layer_for(spec["kind"]), device, args.steps, args.warmup, not args.skip_e2e, sampler)
    points = []
    if not args.no_points:
        for name in EXTRA_POINTS:
            if name == args.workload:
                continue
            kind = WORKLOADS[name]["kind"]
            heavy = WORKLOADS[name]["tokens"] > 1024
            point = run_point(name, layer_for(kind), device, max(3, args.steps // 4) if heavy else args.steps, args.warmup, True, None)
            points.append({k: point[k] for k in ("workload", "tokens", "dtype", "ms_per_step", "launch_mode", "eager_ms_per_step", "value",
                                                 "active_experts", "stage_ms", "roofline", "layer", "e2e")})
    cpu = None
    if not args.skip_cpu:
        cpu = time_cpu_port(spec["kind"], spec["tokens"], layer_for(spec["kind"]), 1, 5)
        cpu.pop("seconds_per_pass", None)
    line = {
        "metric": "moe_layer_tokens_per_s", "value": head["value"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": head["dtype"], "data": "synthetic",
        "config": {"workload": args.workload, "tokens": spec["tokens"], "hidden": H, "inter": I, "experts": E, "top_k": K,
                   "routing": "softmax top-8 of N(0,1) logits, renormalised", "parallelism": "single GPU",
                   "l2": "inputs larger than L2: %.1f GB of expert weights are streamed per step" % (head["layer"]["algorithmic_bytes"] / 1e9)},
        "clocks": head.get("clocks"),
        "e2e": {k: head["e2e"][k] for k in ("value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step")} if "e2e" in head else None,
        "gpu_launches": head["gpu_launches_per_step"] * args.steps, "roofline": head["roofline"], "cpu_baseline": cpu,
        "stage_ms": head["stage_ms"], "layer": head["layer"], "launch_mode": head["launch_mode"],
        "eager_ms_per_step": head["eager_ms_per_step"], "points": points,
    }
    print(json.dumps(line), flush=True)


def run_multi_gpu(args) -> None:
    from fused_cpp_b200 import ep

    args.hidden, args.inter, args.top_k = H, I, K
    # "workload:bf16_return" would add the same workload with the opt-in compact return (not bit-identical).
    args.ep_points = os.environ.get("FUSED_CPP_MOE_EP_POINTS", "w8a8_ep_shared_v3_T16384").split(",")
    args.clock_sampler = ClockSampler
    args.roofline = gate_up_roofline
    ep.bench_main(args, WORKLOADS, SEED, measured_peaks())


def main() -> None:
    global E
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    parser.add_argument("--no-points", action="store_true", help="skip the extra single-GPU points")
    parser.add_argument("--ep-impl", default="peer", choices=["peer", "nccl"],
                        help="N > 1: row exchange by the kernels over peer memory (default) or by NCCL all-to-all")
    parser.add_argument("--experts", type=int, default=E, help="shrink the layer (profiling captures only)")
    parser.add_argument("--skip-e2e", action="store_true", help="profiling captures only")
    parser.add_argument("--skip-cpu", action="store_true", help="profiling captures only")
    args = parser.parse_args()
    E = args.experts
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference_arm(args)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 or world > 1:
        run_multi_gpu(args)
    else:
        run_single_gpu(args)


if __name__ == "__main__":
    main()
