#!/usr/bin/env python
"""Benchmark of the routed-expert MoE layer (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--no-points] [--sweep]

A step is one forward of the MoE layer over one batch of synthetic tokens.  The headline workload is the W8A8
decode configuration of the DeepSeek-V3-scale layer (H=7168, I=2048, E=256, top-8, T=64, near-uniform routing):
9.6 GB of int8 expert weights are streamed per step, far more than the 126 MB L2, so no L2 flush is needed
between iterations; workloads whose weights would fit in L2 are timed step by step with an L2 flush in between.
At N>1 the same batch is run expert-parallel: experts and tokens are split evenly over the ranks and rows are
stored by the kernels into peer memory over NVLink (strong scaling).

value  : tokens/s with every input resident in HBM, CUDA events on the launch stream, max over ranks.
e2e    : the same metric through the public op (fused_cpp_b200.moe.fused_moe_tiled) with the step's
         activations and top-k arrays copied from pinned host memory and the output copied back, all
         inside the timed region.
roofline: the gate_up grouped GEMM (the dominant kernel), timed per launch by the library's stage
         timer (CUDA events around that kernel) during the timed steps.
points : the other benchmark configurations (W8A8 prefill T=8192 uniform and Zipf-routed, BF16 decode, the
         routed + shared-expert layer at T=16384, the two small-dimension configurations), same measurements.
cpu_baseline / --impl reference: the CPU port of the reference arithmetic (oracle/) on all host cores, on the
         same batch.  The reference's native kernels are AArch64-only and cannot run on an x86 host.
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
import torch.distributed as dist  # noqa: E402

V3 = {"hidden": 7168, "inter": 2048, "experts": 256, "top_k": 8}
SMALL = {"hidden": 2048, "inter": 1024, "experts": 16, "top_k": 4}
WORKLOADS = {
    "w8a8_decode_v3_T64": {"kind": "int8", "tokens": 64},
    "w8a8_prefill_v3_T8192": {"kind": "int8", "tokens": 8192},
    # The same prefill batch with compact (bf16) route rows: int8 / int32 stages unchanged and bit-exact, the bf16
    # output to tolerance (relative L2 <= 5e-3) instead of bit for bit.  Never the default: a second line.
    "w8a8_prefill_v3_T8192_bf16rows": {"kind": "int8", "tokens": 8192, "route_rows_bf16": True},
    "w8a8_prefill_v3_T16384": {"kind": "int8", "tokens": 16384},
    "w8a8_prefill_v3_T2048": {"kind": "int8", "tokens": 2048},
    # Zipf-biased router logits (a few experts take most routes): the compute-bound prefill configuration.
    "w8a8_prefill_zipf_v3_T8192": {"kind": "int8", "tokens": 8192, "skew": True},
    "w8a8_prefill_zipf_v3_T2048": {"kind": "int8", "tokens": 2048, "skew": True},
    # Routed experts plus one always-active shared expert (expert id E, route K, weight 1).
    "w8a8_ep_shared_v3_T16384": {"kind": "int8", "tokens": 16384, "shared": True},
    # int8 weights, 16-bit activations: the W8A8 layer's weights through the W8A16 entry point, in its default form
    # (activations as 16-bit fixed point per row on the int8 tensor cores) and in the form that keeps the activations
    # bf16 bit for bit and widens the weight tiles on the SM.
    "w8a16_decode_v3_T64": {"kind": "w8a16", "tokens": 64},
    "w8a16_decode_v3_T64_bf16act": {"kind": "w8a16", "tokens": 64, "w8a16_form": "bf16"},
    "bf16_decode_v3_T64": {"kind": "bf16", "tokens": 64},
    "bf16_decode_v3_T32": {"kind": "bf16", "tokens": 32},
    "bf16_decode_v3_T8": {"kind": "bf16", "tokens": 8},
    "bf16_decode_v3_T1": {"kind": "bf16", "tokens": 1},
    "bf16_prefill_v3_T8192": {"kind": "bf16", "tokens": 8192},
    "bf16_prefill_zipf_v3_T8192": {"kind": "bf16", "tokens": 8192, "skew": True},
    # The two small-dimension configurations (H=2048, I=1024, E=16, top-4): 0.1 GB of weights, L2-resident
    # unless flushed, so these are timed per step with an L2 flush between steps.
    "w8a8_small_T16": {"kind": "int8", "tokens": 16, "dims": SMALL},
    "w8a8_small_zipf_T8192": {"kind": "int8", "tokens": 8192, "skew": True, "dims": SMALL},
}
DEFAULT_WORKLOAD = "w8a8_decode_v3_T64"
EXTRA_POINTS = ["w8a8_prefill_v3_T8192", "w8a8_prefill_v3_T8192_bf16rows", "w8a8_prefill_zipf_v3_T8192", "w8a8_ep_shared_v3_T16384", "w8a16_decode_v3_T64", "w8a16_decode_v3_T64_bf16act", "bf16_decode_v3_T64",
                "bf16_decode_v3_T32", "bf16_decode_v3_T8", "bf16_decode_v3_T1", "w8a8_small_T16", "w8a8_small_zipf_T8192"]
EP_POINTS = ["w8a8_ep_shared_v3_T16384", "w8a8_ep_shared_v3_T16384:bf16_return", "bf16_decode_v3_T64"]
SWEEP_TOKENS = (1, 8, 64, 512, 4096, 16384)
SWEEP_TOKENS_MULTI = (64, 4096, 16384)
SEED = 20260101
L2_BYTES = 126 * 1024 * 1024
NOMINAL = {"hbm_gbs": 7700.0, "int8_tops": 4500.0, "bf16_tflops": 2250.0}


def dims_of(spec: dict) -> dict:
    return dict(spec.get("dims", V3))


DTYPE_LABEL = {"int8": "int8(w8a8)", "bf16": "bf16", "w8a16": "16-bit activations x int8 weights (w8a16)"}


def weight_kind(kind: str) -> str:
    """Storage type of the expert weights of a workload kind."""
    return "bf16" if kind == "bf16" else "int8"


def sweep_spec(kind: str, tokens: int, skew: bool) -> tuple[str, dict]:
    name = f"{'w8a8' if kind == 'int8' else 'bf16'}_sweep{'_zipf' if skew else ''}_v3_T{tokens}"
    return name, {"kind": kind, "tokens": tokens, "skew": skew}


def public_config(name: str, spec: dict, n_gpus: int) -> dict:
    """The `config` object of a line: identical for this build's arm and for --impl reference."""
    d = dims_of(spec)
    return {"workload": name, "tokens": spec["tokens"], "hidden": d["hidden"], "inter": d["inter"], "experts": d["experts"],
            "top_k": d["top_k"], "shared_expert": bool(spec.get("shared", False)),
            "routing": ("softmax top-k of N(0,1) logits + Zipf bias 2 ln(1/(rank+1))" if spec.get("skew") else "softmax top-k of N(0,1) logits")
                       + ", weights renormalised", "n_gpus": n_gpus}


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as stream:
            data = json.load(stream)
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data.get("bf16_tflops", 0.0)),
                "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", 0.0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def measure_int8_library_peak(device: torch.device, sustained_seconds: float = 4.0) -> dict | None:
    """Dense int8 tensor rate of a library GEMM on this GPU, by the method the driver's bf16 figures use: torch._int_mm
    (cuBLASLt) on 8192^3, best of 10 single launches (burst) and back-to-back launches for a few seconds (sustained)."""
    try:
        n = 8192
        a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=device)
        b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=device).t().contiguous().t()  # column-major operand
        ops = 2.0 * n * n * n
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = None
        for _ in range(10):
            start.record()
            torch._int_mm(a, b)
            stop.record()
            torch.cuda.synchronize()
            ms = start.elapsed_time(stop)
            best = ms if best is None else min(best, ms)
        launches = max(10, int(sustained_seconds / (best * 1e-3)))
        start.record()
        for _ in range(launches):
            torch._int_mm(a, b)
        stop.record()
        torch.cuda.synchronize()
        sustained_ms = start.elapsed_time(stop) / launches
        return {"burst_tops": ops / (best * 1e-3) / 1e12, "sustained_tops": ops / (sustained_ms * 1e-3) / 1e12,
                "how": f"torch._int_mm int8 {n}^3 -> int32: best of 10 (burst), {launches} back-to-back launches (sustained)"}
    except Exception as error:  # noqa: BLE001
        sys.stderr.write(f"[bench] int8 library GEMM could not be timed: {error!r}\n")
        return None


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
    started once per GPU and keeps sampling; a region keeps the samples whose time stamps fall inside it.
    Reading only: no clock, power or other setting of the GPU is touched."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}
    _children: dict = {}

    def __init__(self, device_index: int, period_s: float = 0.01):
        self.device_index = device_index
        self.period_s = period_s
        self.begin = None
        self.error = None

    def _child(self):
        import queue
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


# ---- synthetic layer and batches ---------------------------------------------------------------------------

def make_experts(kind: str, device: torch.device, seed: int, expert_ids, hidden: int, inter: int) -> dict:
    """Random-init weights of the experts `expert_ids` on the device, one generator seed per GLOBAL expert id, so
    that every world size (and the single-GPU check of the sharded result) sees the same model.  Values do not
    affect timing; parity against the CPU oracle is tested elsewhere on inputs both sides can hold."""
    ids = list(expert_ids)
    count = len(ids)
    if kind == "int8":
        w13 = torch.empty((count, 2 * inter, hidden), dtype=torch.int8, device=device)
        w2 = torch.empty((count, hidden, inter), dtype=torch.int8, device=device)
        s13 = torch.empty((count, 2 * inter), dtype=torch.float32, device=device)
        s2 = torch.empty((count, hidden), dtype=torch.float32, device=device)
    else:
        w13 = torch.empty((count, 2 * inter, hidden), dtype=torch.bfloat16, device=device)
        w2 = torch.empty((count, hidden, inter), dtype=torch.bfloat16, device=device)
        s13 = s2 = None
    generator = torch.Generator(device=device)
    for slot, expert in enumerate(ids):
        generator.manual_seed(seed + int(expert))
        if kind == "int8":
            w13[slot].random_(-127, 128, generator=generator)
            w2[slot].random_(-127, 128, generator=generator)
            s13[slot].uniform_(0.5, 2.0, generator=generator).div_(127.0 * hidden ** 0.5)
            s2[slot].uniform_(0.5, 2.0, generator=generator).div_(127.0 * inter ** 0.5)
        else:
            w13[slot].normal_(0.0, 0.02, generator=generator)
            w2[slot].normal_(0.0, 0.02, generator=generator)
    return {"w13": w13, "w2": w2, "s13": s13, "s2": s2}


def take_experts(layer: dict, count: int) -> dict:
    return {k: (None if v is None else v[:count]) for k, v in layer.items()}


def make_batch(spec: dict, seed: int):
    """(x bf16 [T,H], topk_weights f32 [T,K], topk_ids i64 [T,K]) on the host, routed experts only."""
    from fused_cpp_b200 import synthetic

    d = dims_of(spec)
    topk_w, topk_ids = synthetic.make_routing(spec["tokens"], d["experts"], d["top_k"], seed, bool(spec.get("skew", False)))
    x = synthetic.make_activations(spec["tokens"], d["hidden"], seed + 1)
    return x, topk_w, topk_ids


def with_shared_route(topk_w: torch.Tensor, topk_ids: torch.Tensor, experts: int):
    """The reference's convention for the shared expert: expert id E appended as route K with weight 1."""
    tokens = topk_ids.shape[0]
    ids = torch.cat((topk_ids, torch.full((tokens, 1), experts, dtype=topk_ids.dtype, device=topk_ids.device)), dim=1).contiguous()
    weights = torch.cat((topk_w, torch.ones((tokens, 1), dtype=topk_w.dtype, device=topk_w.device)), dim=1).contiguous()
    return weights, ids


def layer_work(spec: dict, topk_ids: torch.Tensor) -> dict:
    from fused_cpp_b200 import synthetic

    d = dims_of(spec)
    shape = synthetic.MoEShape(tokens=spec["tokens"], hidden=d["hidden"], inter=d["inter"], experts=d["experts"], top_k=d["top_k"])
    return synthetic.algorithmic_work(shape, topk_ids, 2 if spec["kind"] == "bf16" else 1, shared=bool(spec.get("shared", False)))


def gate_up_work(spec: dict, active: int) -> tuple[float, float]:
    """Algorithmic bytes and operations of one gate_up launch: W13 of the active experts once (+ scales), the
    sorted activation rows in, the bf16 SwiGLU rows out; 2 * rows * 2I * H operations."""
    d = dims_of(spec)
    h, i = d["hidden"], d["inter"]
    b = 2 if spec["kind"] == "bf16" else 1           # weight bytes
    a = 1 if spec["kind"] == "int8" else 2           # bytes of an activation element entering the GEMM
    rows = spec["tokens"] * (d["top_k"] + (1 if spec.get("shared") else 0))
    total = active * 2 * i * h * b + rows * h * a + rows * i * 2
    if spec["kind"] != "bf16":
        total += active * 2 * i * 4 + (rows * 4 if spec["kind"] == "int8" else 0)
    return float(total), 2.0 * rows * 2 * i * h


def gate_up_roofline(kind: str, nbytes: float, ops: float, ms: float, peaks: dict, traffic, int8_peak: dict | None = None) -> dict:
    """Roofline entry of the gate_up grouped GEMM (the dominant kernel) for one launch.

    The bound is whichever of bytes / HBM peak and ops / tensor peak takes longer.  HBM peak and the bf16 tensor
    peak are the driver-measured figures (a plain copy, a cuBLAS GEMM).  For int8 the tensor fraction is printed
    against three denominators: a library int8 GEMM timed in this run, twice the measured bf16 burst, and the
    nominal dense figure; `peak` is the library figure when it could be measured, else twice the bf16 burst."""
    seconds = ms * 1e-3
    if kind == "int8":
        twice_bf16 = 2.0 * peaks["bf16_tflops"]
        library = int8_peak["burst_tops"] if int8_peak else None
        tensor_peak = library if library else twice_bf16
        peak_note = "torch._int_mm burst measured in this run" if library else "2 x measured cuBLAS bf16 burst (no int8 library figure)"
        denominators = {"int8_library_burst": library, "int8_library_sustained": int8_peak["sustained_tops"] if int8_peak else None,
                        "twice_bf16_burst": twice_bf16, "nominal": NOMINAL["int8_tops"]}
    else:
        tensor_peak = peaks["bf16_tflops"]
        peak_note = "measured cuBLAS bf16 burst"
        denominators = {"bf16_burst": peaks["bf16_tflops"], "bf16_sustained": peaks.get("bf16_tflops_sustained"), "nominal": NOMINAL["bf16_tflops"]}
    t_hbm = nbytes / (peaks["hbm_gbs"] * 1e9)
    t_mma = ops / (tensor_peak * 1e12)
    gbs = nbytes / seconds / 1e9 if seconds > 0 else 0.0
    tops = ops / seconds / 1e12 if seconds > 0 else 0.0
    entry = {"kernel": "umma_grouped_gemm_kernel<gate_up> / umma_pair_grouped_gemm_kernel<gate_up>", "traffic": traffic,
             "peak_source": peaks["source"], "algorithmic_bytes_per_launch": nbytes, "ops_per_launch": ops, "ms_per_launch": ms,
             "hbm": {"achieved_gbs": gbs, "peak_gbs": peaks["hbm_gbs"], "frac": gbs / peaks["hbm_gbs"], "frac_of_nominal": gbs / NOMINAL["hbm_gbs"]},
             "tensor": {"achieved_tops": tops, "peak_tops": tensor_peak, "frac": tops / tensor_peak, "peak_note": peak_note,
                        "frac_by_denominator": {k: (tops / v if v else None) for k, v in denominators.items()}}}
    if t_mma > t_hbm:
        entry.update({"bound": "tensor", "achieved": tops, "peak": tensor_peak, "unit": "TFLOP/s" if kind != "int8" else "TOP/s",
                      "frac": tops / tensor_peak})
    else:
        entry.update({"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"]})
        if gbs > peaks["hbm_gbs"]:
            # The denominator is a copy (read + write turnaround); a read-only weight stream sustains more.  The
            # bytes are real (DRAM traffic of the launch from ncu = `traffic`); the nominal figure bounds it.
            entry["peak_note"] = ("achieved exceeds the measured copy bandwidth: a read-only stream has no write turnaround; "
                                  f"{gbs / NOMINAL['hbm_gbs']:.3f} of the nominal {NOMINAL['hbm_gbs']:.0f} GB/s")
    return entry


def layer_summary(work: dict, ms: float, peaks: dict, kind: str, int8_peak: dict | None) -> dict:
    """Whole-layer figures: algorithmic bytes and operations over the step time, against both roofs."""
    seconds = ms * 1e-3
    gbs = work["bytes"] / seconds / 1e9
    tops = work["ops"] / seconds / 1e12
    tensor_peak = (int8_peak["burst_tops"] if (kind == "int8" and int8_peak) else peaks["bf16_tflops"] * (2.0 if kind == "int8" else 1.0))
    t_hbm = work["bytes"] / (peaks["hbm_gbs"] * 1e9)
    t_mma = work["ops"] / (tensor_peak * 1e12)
    return {"algorithmic_bytes": work["bytes"], "ops": work["ops"], "hbm_gbs": gbs, "hbm_frac": gbs / peaks["hbm_gbs"], "tops": tops,
            "tensor_frac": tops / tensor_peak, "tensor_frac_of_nominal": tops / (NOMINAL["int8_tops"] if kind == "int8" else NOMINAL["bf16_tflops"]),
            "binding_roof": "tensor" if t_mma > t_hbm else "hbm", "frac_of_binding_roof": max(t_hbm, t_mma) / seconds}


class L2Flush:
    """Writes a buffer twice the size of L2, so that the next step starts with none of its inputs cached."""

    def __init__(self, device: torch.device):
        self.buffer = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=device)

    def __call__(self) -> None:
        self.buffer.fill_(1)


def time_steps(fn, steps: int, flush: L2Flush | None) -> float:
    """ms per step over `steps` calls of fn on the current stream.  Without a flush the steps run back to back
    between one pair of events; with a flush every step has its own pair and the flush runs between them."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if flush is None:
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / steps
    total = 0.0
    for _ in range(steps):
        flush()
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        total += start.elapsed_time(stop)
    return total / steps


def capture_graph(step):
    """A CUDA graph of one forward (the forward makes no host read, so it is capturable as it is), or None."""
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
        return graph
    except Exception as error:  # noqa: BLE001
        sys.stderr.write(f"[bench] CUDA graph capture unavailable, timing eager launches: {error!r}\n")
        torch.cuda.synchronize()
        return None


def run_point(name: str, spec: dict, layer: dict, device: torch.device, steps: int, warmup: int, with_e2e: bool,
              sampler: ClockSampler | None, int8_peak: dict | None, runtime=None):
    from fused_cpp_b200 import _lib
    from fused_cpp_b200 import moe

    kind, tokens = spec["kind"], spec["tokens"]
    d = dims_of(spec)
    hidden, inter, experts, top_k = d["hidden"], d["inter"], d["experts"], d["top_k"]
    shared = bool(spec.get("shared", False))
    x_host, w_host, ids_host = make_batch(spec, SEED)
    x, tw, ids = x_host.to(device), w_host.to(device), ids_host.to(device)
    if shared:
        tw_run, ids_run = with_shared_route(tw, ids, experts)
    else:
        tw_run, ids_run = tw, ids
    weights = take_experts(layer, experts + (1 if shared else 0))
    work = layer_work(spec, ids_host)
    flush = L2Flush(device) if work["bytes"] < 4 * L2_BYTES else None
    timer = _lib.StageTimer(steps)

    def step(stage_timer=None):
        return _lib.moe_forward(x, weights["w13"], weights["w2"], tw_run, ids_run, s13=weights["s13"], s2=weights["s2"], stage_timer=stage_timer,
                                w8a16=kind == "w8a16", route_rows_bf16=bool(spec.get("route_rows_bf16", False)),
                                w8a16_form=_lib.W8A16_BF16_ACTIVATIONS if spec.get("w8a16_form") == "bf16" else _lib.W8A16_FIXED_POINT)

    for _ in range(warmup):
        step()
    result = step()
    result.raise_for_status()
    torch.cuda.synchronize()

    # Timed region 1 (the headline): K replays of a CUDA graph of one forward, so that the host's launch cost
    # (8 launches per step through ctypes) does not sit between the kernels; eager launches if capture is refused.
    graph = capture_graph(step)
    if sampler is not None:
        sampler.start()
    ms_per_step = time_steps(graph.replay if graph is not None else step, steps, flush)
    clocks = sampler.stop() if sampler is not None else None

    # Timed region 2: the same K steps launched eagerly with the library's stage timer (CUDA events around
    # every stage on the launch stream); this is where the per-kernel durations of the roofline come from.
    eager_ms_per_step = time_steps(lambda: step(timer), steps, flush)
    stage_ms = {stage: 0.0 for stage in _lib.STAGES}
    for call in range(timer.calls):
        for stage, value in timer.read(call).items():
            stage_ms[stage] += value / timer.calls
    timer.close()

    peaks = measured_peaks()
    gu_bytes, gu_ops = gate_up_work(spec, work["active_experts"])
    routes = tokens * (top_k + (1 if shared else 0))
    point = {
        "workload": name, "tokens": tokens, "dtype": DTYPE_LABEL[kind], "ms_per_step": ms_per_step,
        "launch_mode": "cuda_graph_replay" if graph is not None else "eager", "eager_ms_per_step": eager_ms_per_step,
        "l2": "flushed between steps (a buffer of twice the L2 is written)" if flush is not None else "inputs larger than L2",
        "route_rows": "bf16 (opt-in compact rows: output to tolerance, not bit-exact)" if spec.get("route_rows_bf16") else "fp32 (the reference's)",
        **({"w8a16_form": "bf16 activations, weights widened on the SM" if spec.get("w8a16_form") == "bf16"
            else "activations as 16-bit fixed point per row (two int8 planes), int8 tensor cores"} if kind == "w8a16" else {}),
        "value": tokens / (ms_per_step * 1e-3), "active_experts": work["active_experts"],
        "stage_ms": {k: round(v, 5) for k, v in stage_ms.items()},
        "roofline": gate_up_roofline(kind, gu_bytes, gu_ops, stage_ms["gate_up"], peaks, ncu_traffic_bytes(name), int8_peak),
        "layer": layer_summary(work, ms_per_step, peaks, kind, int8_peak),
        # route build (1 kernel up to 1024 routes, else 3) + quantise/gather + gate_up (+ requantise) + down + merge;
        # above 64 tokens the two GEMMs are two launches each (thin experts / the others).
        "gpu_launches_per_step": (1 if routes <= 1024 else 3) + (5 if kind == "int8" else 4) + (2 if tokens > 64 else 0),
    }
    if clocks is not None:
        point["clocks"] = clocks

    if with_e2e:
        # Public API, host buffers: H2D of x / top-k weights / ids, the op (with its status check), D2H of out.
        if kind == "w8a16":
            holder = moe.PreparedW8A16TiledFusedMoEWeights(w13=(weights["w13"], hidden, 2 * inter, weights["s13"]),
                                                           w2=(weights["w2"], inter, hidden, weights["s2"]))
            prepared = moe.PreparedW8A16TiledRoutedSharedMoEWeights(packed=holder, routed_experts=experts, shared_expert_id=experts) if shared else holder
        elif kind == "int8":
            holder = moe.PreparedW8A8TiledFusedMoEWeights(w13=(weights["w13"], hidden, 2 * inter, weights["s13"]),
                                                          w2=(weights["w2"], inter, hidden, weights["s2"]))
            prepared = moe.PreparedW8A8TiledRoutedSharedMoEWeights(packed=holder, routed_experts=experts, shared_expert_id=experts) if shared else holder
        else:
            holder = moe.PreparedBF16TiledFusedMoEWeights(w13=(weights["w13"], hidden, 2 * inter), w2=(weights["w2"], inter, hidden), fused_silu=True)
            prepared = moe.PreparedBF16TiledRoutedSharedMoEWeights(packed=holder, routed_experts=experts, shared_expert_id=experts) if shared else holder
        own_runtime = runtime if runtime is not None else moe.MoePlannerRuntime(None, hidden_size=hidden, intermediate_size=inter,
                                                                                  global_experts=experts, local_experts=experts,
                                                                                  shared_experts=1 if shared else 0)
        previous = moe.set_default_moe_planner_runtime(own_runtime)
        previous_rows = os.environ.get("FUSED_CPP_MOE_W2_BF16_ROUTE")
        os.environ["FUSED_CPP_MOE_W2_BF16_ROUTE"] = "1" if spec.get("route_rows_bf16") else "0"
        previous_form = os.environ.get("FUSED_CPP_MOE_W8A16_FORM")
        os.environ["FUSED_CPP_MOE_W8A16_FORM"] = spec.get("w8a16_form", "fixed")
        try:
            x_pin, w_pin, ids_pin = x_host.pin_memory(), w_host.pin_memory(), ids_host.pin_memory()
            out_pin = torch.empty((tokens, hidden), dtype=torch.bfloat16).pin_memory()
            out_dev = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=device)

            def e2e_step():
                xd = x_pin.to(device, non_blocking=True)
                wd = w_pin.to(device, non_blocking=True)
                idd = ids_pin.to(device, non_blocking=True)
                kwargs = {"swiglu_limit": 10.0} if kind == "int8" else {}
                if shared:
                    op = {"int8": moe.fused_moe_w8a8_tiled_with_shared, "w8a16": moe.fused_moe_w8a16_tiled_with_shared,
                          "bf16": moe.fused_moe_bf16_tiled_with_shared}[kind]
                    op(xd, prepared, wd, idd, out=out_dev, **kwargs)
                else:
                    moe.fused_moe_tiled(xd, prepared, wd, idd, out=out_dev, **kwargs)
                out_pin.copy_(out_dev, non_blocking=True)

            for _ in range(warmup):
                e2e_step()
            torch.cuda.synchronize()
            serial_ms = time_steps(e2e_step, steps, flush)
            e2e_ms, e2e_mode = serial_ms, "serial: copy in, forward, copy out on one stream"
            if flush is None:
                # The same work as a two-deep pipeline, the way a serving loop feeds a layer: the next step's inputs
                # travel host-to-device and the previous step's output device-to-host on their own streams while the
                # forward of the current step runs.  Every timed step still has its own two copies inside the timed
                # region (the first step's upload is the prologue, the upload issued in the last step is the extra one).
                forward_stream = torch.cuda.current_stream()
                up_stream, down_stream = torch.cuda.Stream(), torch.cuda.Stream()
                slots = [{"x": torch.empty_like(x_pin, device=device), "w": torch.empty_like(w_pin, device=device),
                          "ids": torch.empty_like(ids_pin, device=device),
                          "out": torch.empty((tokens, hidden), dtype=torch.bfloat16, device=device),
                          "out_pin": torch.empty((tokens, hidden), dtype=torch.bfloat16).pin_memory(),
                          "uploaded": torch.cuda.Event(), "computed": torch.cuda.Event(), "downloaded": torch.cuda.Event()} for _ in range(2)]
                kwargs = {"swiglu_limit": 10.0} if kind == "int8" else {}
                shared_op = {"int8": moe.fused_moe_w8a8_tiled_with_shared, "w8a16": moe.fused_moe_w8a16_tiled_with_shared,
                             "bf16": moe.fused_moe_bf16_tiled_with_shared}[kind]

                def upload(slot):
                    with torch.cuda.stream(up_stream):
                        up_stream.wait_event(slot["computed"])  # the forward that last read these buffers
                        slot["x"].copy_(x_pin, non_blocking=True)
                        slot["w"].copy_(w_pin, non_blocking=True)
                        slot["ids"].copy_(ids_pin, non_blocking=True)
                        slot["uploaded"].record(up_stream)

                counter = {"step": 0}

                def pipelined_step():
                    slot, other = slots[counter["step"] & 1], slots[(counter["step"] & 1) ^ 1]
                    counter["step"] += 1
                    upload(other)
                    forward_stream.wait_event(slot["uploaded"])
                    forward_stream.wait_event(slot["downloaded"])  # its output buffer has been read out
                    if shared:
                        shared_op(slot["x"], prepared, slot["w"], slot["ids"], out=slot["out"], **kwargs)
                    else:
                        moe.fused_moe_tiled(slot["x"], prepared, slot["w"], slot["ids"], out=slot["out"], **kwargs)
                    slot["computed"].record(forward_stream)
                    with torch.cuda.stream(down_stream):
                        down_stream.wait_event(slot["computed"])
                        slot["out_pin"].copy_(slot["out"], non_blocking=True)
                        slot["downloaded"].record(down_stream)

                upload(slots[0])
                for _ in range(warmup):
                    pipelined_step()
                torch.cuda.synchronize()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record(forward_stream)
                for _ in range(steps):
                    pipelined_step()
                forward_stream.wait_event(slots[(counter["step"] - 1) & 1]["downloaded"])
                forward_stream.wait_event(slots[counter["step"] & 1]["uploaded"])
                stop.record(forward_stream)
                torch.cuda.synchronize()
                pipelined_ms = start.elapsed_time(stop) / steps
                if pipelined_ms < serial_ms:
                    e2e_ms = pipelined_ms
                    e2e_mode = ("two-deep pipeline: the next step's upload and the previous step's download on their own streams "
                                "beside the forward; every step's copies are inside the timed region")
            last_plan = dict(own_runtime.last_plan)
        finally:
            moe.set_default_moe_planner_runtime(previous)
            if previous_rows is None:
                os.environ.pop("FUSED_CPP_MOE_W2_BF16_ROUTE", None)
            else:
                os.environ["FUSED_CPP_MOE_W2_BF16_ROUTE"] = previous_rows
            if previous_form is None:
                os.environ.pop("FUSED_CPP_MOE_W8A16_FORM", None)
            else:
                os.environ["FUSED_CPP_MOE_W8A16_FORM"] = previous_form
        point["e2e"] = {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms, "mode": e2e_mode,
                        "serial_value": tokens / (serial_ms * 1e-3), "serial_ms_per_step": serial_ms,
                        "h2d_bytes_per_step": tokens * hidden * 2 + tokens * top_k * 4 + tokens * top_k * 8,
                        "d2h_bytes_per_step": tokens * hidden * 2,
                        "planner": {k: last_plan.get(k) for k in ("planner", "dispatch", "kind", "rows_per_expert", "gate_up_tile", "down_tile", "machine_id", "calibrated") if k in last_plan}}
    return point


# ---- CPU arm ------------------------------------------------------------------------------------------------

def host_cores() -> int:
    return len(os.sched_getaffinity(0))


def cpu_inputs(spec: dict, layer: dict | None):
    """The whole batch of the workload with the weights of the experts it hits, compacted (expert ids remapped to
    0..hit-1).  With `layer` (GPU weights) the experts are copied from the device; otherwise rotated copies of one
    host-generated expert stand in (distinct memory per expert, which is what the CPU timing depends on)."""
    d = dims_of(spec)
    hidden, inter, experts = d["hidden"], d["inter"], d["experts"]
    x, tw, ids = make_batch(spec, SEED)
    if spec.get("shared"):
        tw, ids = with_shared_route(tw, ids, experts)
    hit = torch.unique(ids)
    remap = torch.full((experts + 1,), -1, dtype=torch.int64)
    remap[hit] = torch.arange(hit.numel())
    local_ids = remap[ids]
    kind = weight_kind(spec["kind"])
    if layer is not None:
        index = hit.to(layer["w13"].device)
        weights = {k: (None if v is None else v.index_select(0, index).cpu()) for k, v in layer.items()}
    else:
        generator = torch.Generator().manual_seed(SEED + 7)
        n = int(hit.numel())
        if kind == "int8":
            base13 = torch.randint(-127, 128, (2 * inter, hidden), generator=generator, dtype=torch.int8)
            base2 = torch.randint(-127, 128, (hidden, inter), generator=generator, dtype=torch.int8)
            weights = {"w13": torch.stack([base13.roll(e, 0) for e in range(n)]), "w2": torch.stack([base2.roll(e, 0) for e in range(n)]),
                       "s13": torch.full((n, 2 * inter), 1.0 / (127.0 * hidden ** 0.5)), "s2": torch.full((n, hidden), 1.0 / (127.0 * inter ** 0.5))}
        else:
            base13 = (torch.randn((2 * inter, hidden), generator=generator) * 0.02).to(torch.bfloat16)
            base2 = (torch.randn((hidden, inter), generator=generator) * 0.02).to(torch.bfloat16)
            weights = {"w13": torch.stack([base13.roll(e, 0) for e in range(n)]), "w2": torch.stack([base2.roll(e, 0) for e in range(n)]),
                       "s13": None, "s2": None}
    return x, tw, local_ids, weights, int(hit.numel())


def time_cpu_port(name: str, spec: dict, layer: dict | None, warmup: int, passes: int, budget_s: float = 150.0) -> dict:
    """Time forward passes of the CPU port over the workload's own batch on all host cores (inputs built once).
    The OpenMP thread count is set explicitly: a launcher may export OMP_NUM_THREADS=1 to its children."""
    from oracle import oracle

    cores = host_cores()
    oracle.set_threads(cores)
    x, tw, ids, weights, hit = cpu_inputs(spec, layer)
    tokens = int(x.shape[0])
    routes = int(ids.numel())

    def one_pass() -> float:
        begin = time.perf_counter()
        if spec["kind"] == "int8":
            oracle.w8a8_forward(x, weights["w13"], weights["s13"], weights["w2"], weights["s2"], tw, ids)
        elif spec["kind"] == "w8a16":
            oracle.w8a16_forward(x, weights["w13"], weights["s13"], weights["w2"], weights["s2"], tw, ids)
        else:
            oracle.bf16_forward(x, weights["w13"], weights["w2"], tw, ids)
        return time.perf_counter() - begin

    first = one_pass()
    # Bound the run: as many of the requested passes as fit the time budget (never fewer than one timed pass).
    affordable = max(1, int(budget_s / max(first, 1e-6)) - 1)
    warmup_done = min(max(warmup - 1, 0), max(affordable - 1, 0))
    for _ in range(warmup_done):
        one_pass()
    timed = max(1, min(passes, affordable - warmup_done))
    times = [one_pass() for _ in range(timed)]
    seconds = statistics.mean(times)
    return {"value": tokens / seconds, "unit": "tokens/s", "cores": cores, "kind": "port", "threads": oracle.get_max_threads(),
            "sample": f"the whole batch of {name}: {tokens} tokens, {routes} routes, {hit} experts hit; OpenMP C port of the reference "
                      f"arithmetic on {cores} threads, mean of {timed} passes after {warmup_done + 1} warm-up, {seconds * 1e3:.1f} ms per pass",
            "passes_timed": timed, "seconds_per_pass": seconds}


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    spec = WORKLOADS[args.workload]
    baseline = time_cpu_port(args.workload, spec, None, args.warmup, args.steps)
    seconds = baseline.pop("seconds_per_pass")
    value = baseline["value"]
    line = {"impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": DTYPE_LABEL[spec["kind"]],
            "data": "synthetic", "config": public_config(args.workload, spec, args.gpus),
            "note": "the reference's native kernels are AArch64 SVE/I8MM only; this arm times the CPU port of the same arithmetic "
                    "(oracle/moe_oracle.c) on the host cores, every step the workload's whole batch",
            "cpu_baseline": baseline,
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---- single GPU ---------------------------------------------------------------------------------------------

class LayerCache:
    """One set of device weights per (kind, dims): the V3 layers hold 256 routed experts + the shared one."""

    def __init__(self, device: torch.device):
        self.device = device
        self.layers: dict = {}

    def get(self, spec: dict) -> dict:
        d = dims_of(spec)
        key = (weight_kind(spec["kind"]), d["hidden"], d["inter"], d["experts"])
        if key not in self.layers:
            self.layers[key] = make_experts(key[0], self.device, SEED + 2, range(d["experts"] + 1), d["hidden"], d["inter"])
        return self.layers[key]

    def drop(self) -> None:
        self.layers.clear()
        torch.cuda.empty_cache()


class Runtimes:
    """One planner runtime per (dims, shared expert) for the end-to-end legs.  With calibrate=True the row-tile
    table comes from the library's own quick calibration on this GPU (calibrate_moe_planner_quick on a probe layer
    of the workload's H and I, once per dims); otherwise the runtime carries no table and every call uses the
    library's automatic tiles."""

    def __init__(self, calibrate: bool):
        self.calibrate = calibrate
        self.calibrations: dict = {}
        self.seconds: dict = {}

    def get(self, spec: dict):
        from fused_cpp_b200 import moe
        from fused_cpp_b200.moe import planner_runtime

        d = dims_of(spec)
        key = (d["hidden"], d["inter"], d["experts"])
        if self.calibrate and key not in self.calibrations:
            result = planner_runtime.calibrate_moe_planner_quick(None, _shape=key)
            self.calibrations[key] = result.calibration
            self.seconds[key] = result.elapsed_seconds
        return moe.MoePlannerRuntime(self.calibrations.get(key), hidden_size=d["hidden"], intermediate_size=d["inter"],
                                     global_experts=d["experts"], local_experts=d["experts"], shared_experts=1 if spec.get("shared") else 0)


POINT_KEYS = ("workload", "tokens", "dtype", "ms_per_step", "launch_mode", "eager_ms_per_step", "l2", "route_rows", "value", "active_experts",
              "stage_ms", "roofline", "layer", "e2e")


def run_single_gpu(args) -> None:
    from fused_cpp_b200 import _lib

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    if not _lib.device_supported():
        raise SystemExit("bench.py needs a compute-capability-10.x GPU: the library has no other path")
    spec = WORKLOADS[args.workload]
    if args.experts:
        spec = dict(spec, dims=dict(dims_of(spec), experts=args.experts))
    int8_peak = None if args.skip_peak else measure_int8_library_peak(device)
    runtimes = Runtimes(calibrate=not args.skip_e2e and not args.skip_calibration)
    layers = LayerCache(device)
    sampler = ClockSampler(0)
    head = run_point(args.workload, spec, layers.get(spec), device, args.steps, args.warmup, not args.skip_e2e, sampler, int8_peak,
                     runtimes.get(spec))
    points = []
    if args.sweep:
        for kind in ("int8", "bf16"):
            for skew in (False, True):
                for tokens in SWEEP_TOKENS:
                    name, sweep = sweep_spec(kind, tokens, skew)
                    point = run_point(name, sweep, layers.get(sweep), device, max(3, args.steps // 4) if tokens > 1024 else args.steps,
                                      args.warmup, False, None, int8_peak)
                    points.append({k: point[k] for k in POINT_KEYS if k in point})
            layers.drop()
    elif not args.no_points:
        for name in EXTRA_POINTS:
            if name == args.workload:
                continue
            other = WORKLOADS[name]
            heavy = other["tokens"] > 1024
            point = run_point(name, other, layers.get(other), device, max(3, args.steps // 4) if heavy else args.steps, args.warmup, True,
                              None, int8_peak, runtimes.get(other))
            points.append({k: point[k] for k in POINT_KEYS if k in point})
        for rows, k, n in DENSE_POINTS:
            points.append(run_dense_point(rows, k, n, device, max(3, args.steps // 4) if rows > 1024 else args.steps, args.warmup,
                                          measured_peaks(), int8_peak))
    cpu = None
    if not args.skip_cpu:
        cpu = time_cpu_port(args.workload, spec, layers.get(spec), 1, 3, budget_s=40.0)
        cpu.pop("seconds_per_pass", None)
    work_gb = head["layer"]["algorithmic_bytes"] / 1e9
    line = {
        "metric": "moe_layer_tokens_per_s", "value": head["value"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": head["dtype"], "data": "synthetic",
        "config": public_config(args.workload, spec, 1),
        "parallelism": "single GPU", "l2": f"{head['l2']}: {work_gb:.1f} GB of expert weights and rows are streamed per step",
        "clocks": head.get("clocks"),
        "e2e": {k: head["e2e"][k] for k in ("value", "unit", "ms_per_step", "mode", "serial_value", "h2d_bytes_per_step", "d2h_bytes_per_step", "planner")} if "e2e" in head else None,
        "gpu_launches": head["gpu_launches_per_step"] * args.steps, "roofline": head["roofline"], "cpu_baseline": cpu,
        "int8_library_peak": int8_peak, "planner_calibration_seconds": {"x".join(str(v) for v in k): round(v2, 2) for k, v2 in runtimes.seconds.items()},
        "stage_ms": head["stage_ms"], "layer": head["layer"], "launch_mode": head["launch_mode"],
        "eager_ms_per_step": head["eager_ms_per_step"], "points": points,
    }
    print(json.dumps(line), flush=True)


# ---- dense W8A8 linear (the i8gemm op next to the MoE path) -------------------------------------------------

# (rows, K, N): a decode and a prefill batch through an output projection of the DeepSeek-V3 attention block
# (16384 -> 7168) and through its query up-projection (1536 -> 24576).
DENSE_POINTS = [(64, 16384, 7168), (8192, 16384, 7168), (64, 1536, 24576), (8192, 1536, 24576)]


def run_dense_point(rows: int, k: int, n: int, device: torch.device, steps: int, warmup: int, peaks: dict, int8_peak: dict | None) -> dict:
    """fused_cpp.i8gemm.dynamic_scaled_mm (row quantiser + tcgen05 GEMM with the dense epilogue) on seeded inputs."""
    from fused_cpp_b200 import i8gemm

    generator = torch.Generator().manual_seed(SEED + rows + k + n)
    weight = torch.randint(-127, 128, (n, k), generator=generator, dtype=torch.int8).to(device)
    scale = (torch.rand((n,), generator=generator) * 1.5 + 0.5).div_(127.0 * k ** 0.5).to(device)
    x = torch.randn((rows, k), generator=generator).to(torch.bfloat16).to(device)
    prepared = i8gemm.prepare(weight, scale)
    nbytes = n * k + rows * k * 2 + rows * k + rows * n * 2  # weights, rows in, int8 rows written and re-read once, out
    flush = L2Flush(device) if nbytes < 4 * L2_BYTES else None

    def step():
        return i8gemm.dynamic_scaled_mm(x, prepared, out_dtype=torch.bfloat16)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    # As for the MoE points: the value is timed over replays of a CUDA graph of one call (the host's launch cost of the
    # two launches does not sit between the kernels); the eager figure is reported next to it.
    graph = capture_graph(step)
    ms = time_steps(graph.replay if graph is not None else step, steps, flush)
    eager_ms = ms
    if graph is not None:
        for _ in range(2):  # the allocator settles again after the capture
            step()
        torch.cuda.synchronize()
        eager_ms = time_steps(step, steps, flush)
    ops = 2.0 * rows * n * k
    tensor_peak = int8_peak["burst_tops"] if int8_peak else 2.0 * peaks["bf16_tflops"]
    t_hbm, t_tensor = nbytes / (peaks["hbm_gbs"] * 1e9), ops / (tensor_peak * 1e12)
    bound = "hbm" if t_hbm >= t_tensor else "tensor"
    return {"workload": f"i8gemm_dense_M{rows}_K{k}_N{n}", "tokens": rows, "dtype": "int8(w8a8)", "ms_per_step": ms,
            "value": rows / (ms * 1e-3), "eager_ms_per_step": eager_ms,
            "launch_mode": ("cuda_graph_replay" if graph is not None else "eager") + " (row quantiser + GEMM, two launches; three with the K split of at most 16 rows)",
            "l2": "flushed between steps (a buffer of twice the L2 is written)" if flush is not None else "inputs larger than L2",
            "roofline": {"bound": bound, "achieved": nbytes / (ms * 1e-3) / 1e9 if bound == "hbm" else ops / (ms * 1e-3) / 1e12,
                         "peak": peaks["hbm_gbs"] if bound == "hbm" else tensor_peak, "unit": "GB/s" if bound == "hbm" else "TOP/s",
                         "frac": (t_hbm if bound == "hbm" else t_tensor) / (ms * 1e-3), "whole_op": True,
                         "algorithmic_bytes": nbytes, "ops": ops}}


# ---- expert parallel over the GPUs of one box (launched by torch.distributed.run) ----------------------------

def run_ep_point(name: str, spec: dict, args, rank: int, world: int, device: torch.device, peaks: dict, bf16_return: bool = False) -> dict:
    from fused_cpp_b200 import _lib, ep

    kind, tokens = spec["kind"], spec["tokens"]
    d = dims_of(spec)
    hidden, inter, experts, top_k = d["hidden"], d["inter"], d["experts"], d["top_k"]
    has_shared = bool(spec.get("shared", False))
    per_rank = experts // world
    mine_experts = list(range(rank * per_rank, (rank + 1) * per_rank)) + ([experts] if has_shared else [])
    weights = make_experts(kind, device, SEED + 2, mine_experts, hidden, inter)
    if kind != "int8":
        weights = {k: v for k, v in weights.items() if v is not None}
    x, topk_w, topk_ids = make_batch(spec, SEED)
    mine = ep.shard_rows(tokens, world, rank)
    x_host, w_host, ids_host = x[mine].contiguous(), topk_w[mine].contiguous(), topk_ids[mine].contiguous()
    xd, wd, idd = x_host.to(device), w_host.to(device), ids_host.to(device)
    local_max = (tokens + world - 1) // world
    if args.ep_impl == "peer":
        layer = ep.PeerMemoryExpertParallelMoE(weights, experts, tokens_max=local_max, top_k=top_k, has_shared=has_shared,
                                               return_dtype=torch.bfloat16 if bf16_return else torch.float32)
        exchange = "rows stored by the dispatch kernel and the down-GEMM epilogue into peer memory over NVLink, flag barriers in the same slabs"
        if bf16_return:
            exchange += "; result rows returned as bf16 (opt-in: half the return traffic, outputs within a bf16 step, not bit-identical)"
    else:
        layer = ep.ExpertParallelMoE(weights, experts, has_shared=has_shared)
        exchange = "NCCL all-to-all dispatch/combine"
    kwargs = {"swiglu_limit": 10.0} if kind == "int8" else {}

    def step():
        return layer(xd, wd, idd, **kwargs)

    def timed(fn, steps, warmup, sampler=None):
        if sampler is not None:
            sampler.prepare()
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler is not None:
            sampler.start()
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        clocks = sampler.stop() if sampler is not None else None
        dist.barrier()
        elapsed = torch.tensor([start.elapsed_time(stop) / steps], device=device)
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        return float(elapsed.item()), clocks

    # The peer-memory forward makes no host read and calls no collective library, so one step (kernels, flag barriers
    # included) is captured into a CUDA graph and the timed region replays it; every rank replays the same sequence.
    # Eager launches are timed as well (eager_ms_per_step) and the faster of the two is `value`.
    launch_mode = "eager"
    replay = step
    graph = None
    peer = isinstance(layer, ep.PeerMemoryExpertParallelMoE)
    if peer and os.environ.get("FUSED_CPP_MOE_EP_GRAPH", "1") != "0":
        try:
            side = torch.cuda.Stream(device=device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            replay = graph.replay
            launch_mode = "cuda_graph_replay"
        except Exception as error:  # noqa: BLE001
            launch_mode = f"eager (graph capture failed: {type(error).__name__})"
            replay = step
    captured = torch.tensor([1 if launch_mode == "cuda_graph_replay" else 0], device=device)
    dist.all_reduce(captured, op=dist.ReduceOp.MIN)
    if int(captured.item()) == 0:
        replay = step
        if launch_mode == "cuda_graph_replay":
            launch_mode = "eager (graph capture failed on another rank)"
    new_sampler = (lambda: ClockSampler(device.index)) if rank == 0 else (lambda: None)
    ms, clocks = timed(replay, args.steps, args.warmup, new_sampler())
    eager_ms = ms
    if replay is not step:
        graph_ms = ms
        eager_ms, eager_clocks = timed(step, args.steps, args.warmup, new_sampler())
        if eager_ms < graph_ms:
            ms, clocks, launch_mode = eager_ms, eager_clocks, f"eager (cuda_graph_replay: {graph_ms:.4f} ms)"

    # Per-kernel durations of this rank's expert stage (CUDA events around every stage, a second timed pass).
    roofline = None
    stage_ms = None
    if peer:
        timer = _lib.StageTimer(args.steps)
        layer.stage_timer = timer
        for _ in range(args.steps):
            step()
        torch.cuda.synchronize()
        layer.stage_timer = None
        stage_ms = {stage: 0.0 for stage in _lib.STAGES}
        for call in range(timer.calls):
            for stage, value in timer.read(call).items():
                stage_ms[stage] += value / timer.calls
        timer.close()
        # Algorithmic work of this rank's gate_up launch: the weights of its experts that the batch hits, once,
        # plus the rows it receives in and their SwiGLU rows out.
        owner = topk_ids // per_rank
        local_ids = topk_ids[owner == rank]
        rows = int(local_ids.numel()) + (x_host.shape[0] if has_shared else 0)
        active = int(local_ids.unique().numel()) + (1 if has_shared else 0)
        b = 1 if kind == "int8" else 2
        nbytes = active * 2 * inter * hidden * b + rows * hidden * b + rows * inter * 2 + (active * 2 * inter * 4 + rows * 4 if kind == "int8" else 0)
        roofline = gate_up_roofline(kind, float(nbytes), 2.0 * rows * 2 * inter * hidden, stage_ms["gate_up"], peaks, None)
        roofline["scope"] = f"rank 0 of {world}: {active} active local experts, {rows} received rows"
        dist.barrier()

    x_pin, w_pin, ids_pin = x_host.pin_memory(), w_host.pin_memory(), ids_host.pin_memory()
    out_pin = torch.empty((x_host.shape[0], hidden), dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        out = layer(x_pin.to(device, non_blocking=True), w_pin.to(device, non_blocking=True), ids_pin.to(device, non_blocking=True), **kwargs)
        out_pin.copy_(out, non_blocking=True)

    e2e_ms, _ = timed(e2e_step, args.steps, args.warmup)

    # Check at benchmark scale, outside every timed region: each rank rebuilds the whole model from the per-expert
    # seeds, runs the SINGLE-GPU forward over the whole batch and compares its own shard of that result with what
    # the sharded forward gave it.
    got = layer(xd, wd, idd, **kwargs).clone()
    torch.cuda.synchronize()
    dist.barrier()
    full = make_experts(kind, device, SEED + 2, range(experts + (1 if has_shared else 0)), hidden, inter)
    full_w, full_ids = topk_w.to(device), topk_ids.to(device)
    if has_shared:
        full_w, full_ids = with_shared_route(full_w, full_ids, experts)
    reference = _lib.moe_forward(x.to(device), full["w13"], full["w2"], full_w, full_ids, s13=full["s13"], s2=full["s2"])
    reference.raise_for_status()
    expected = reference.out[mine]
    if bf16_return:
        error = float((got.float() - expected.float()).norm() / expected.float().norm().clamp_min(1e-30))
        agree = torch.tensor([1 if error <= 5e-3 else 0], device=device)
        parity = "relative L2 to the single-GPU forward of the whole batch <= 5e-3 on every rank's shard (bf16 result rows: tolerance, not bit-equality)"
    else:
        agree = torch.tensor([1 if torch.equal(got.view(torch.int16), expected.view(torch.int16)) else 0], device=device)
        parity = "bit-identical to the single-GPU forward of the whole batch, every rank's shard"
    dist.all_reduce(agree, op=dist.ReduceOp.MIN)
    if int(agree.item()) != 1:
        raise RuntimeError(f"{name}: the sharded forward disagrees with the single-GPU forward on at least one rank")
    del full, reference, expected, got
    # Every rank is done with every slab before any of them is unmapped and freed.
    torch.cuda.synchronize()
    dist.barrier()
    replay = None
    graph = None
    if hasattr(layer, "close"):
        layer.raise_for_status()
        layer.close()
    torch.cuda.empty_cache()
    local_tokens = x_host.shape[0]
    # Kernels of this library per forward on one rank, peer form: route build by global expert (1 kernel up to 1024
    # routes, else 3), count barrier, layout, dispatch, barrier | work items, output addresses, gate_up (+ requantise),
    # down, barrier | merge.
    routes_local = local_tokens * (top_k + (1 if has_shared else 0))
    launches_per_step = ((1 if routes_local <= 1024 else 3) + 4) + (5 + (1 if kind == "int8" else 0)) + 1
    work = layer_work(spec, topk_ids)
    config = public_config(name, spec, world)
    return {
        "metric": "moe_layer_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16" if kind == "bf16" else "int8(w8a8)", "data": "synthetic", "config": config,
        "parallelism": f"ep{world}: experts and tokens split evenly, {exchange}",
        "l2": "inputs larger than L2: every rank streams its experts' weights each step",
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": local_tokens * hidden * 2 + local_tokens * top_k * 12,
                "d2h_bytes_per_step": local_tokens * hidden * 2},
        "gpu_launches": launches_per_step * args.steps, "clocks": clocks, "roofline": roofline, "cpu_baseline": None,
        "launch_mode": launch_mode, "eager_ms_per_step": eager_ms, "parity": parity,
        "stage_ms_rank0": {k: round(v, 5) for k, v in stage_ms.items()} if stage_ms else None,
        "layer": {"algorithmic_bytes": work["bytes"], "ops": work["ops"],
                  "hbm_gbs_aggregate": work["bytes"] / (ms * 1e-3) / 1e9, "tops_aggregate": work["ops"] / (ms * 1e-3) / 1e12},
    }


def run_multi_gpu(args) -> None:
    from fused_cpp_b200 import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    try:
        if not _lib.device_supported():
            raise SystemExit("bench.py needs compute-capability-10.x GPUs")
        peaks = measured_peaks()
        entries = [args.workload]
        if args.sweep:
            for kind in ("int8", "bf16"):
                for skew in (False, True):
                    entries += [sweep_spec(kind, tokens, skew) for tokens in SWEEP_TOKENS_MULTI]
        elif not args.no_points:
            entries += os.environ.get("FUSED_CPP_MOE_EP_POINTS", ",".join(EP_POINTS)).split(",")
        lines = []
        for entry in entries:
            if isinstance(entry, tuple):
                name, spec, option = entry[0], entry[1], ""
            else:
                name, _, option = entry.partition(":")  # "workload:bf16_return" = the same workload with the compact return
                spec = WORKLOADS[name]
            if lines and name == args.workload and not option:
                continue
            lines.append(run_ep_point(name + (":" + option if option else ""), spec, args, rank, world, device, peaks, bf16_return=option == "bf16_return"))
        if rank == 0:
            head = lines[0]
            head["points"] = lines[1:]
            print(json.dumps(head), flush=True)
    finally:
        dist.destroy_process_group()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    parser.add_argument("--no-points", action="store_true", help="skip the extra points")
    parser.add_argument("--sweep", action="store_true",
                        help="points = the sweep T x {W8A8, BF16} x {uniform, Zipf} on the V3-scale layer instead of the named configurations")
    parser.add_argument("--ep-impl", default="peer", choices=["peer", "nccl"],
                        help="N > 1: row exchange by the kernels over peer memory (default) or by NCCL all-to-all")
    parser.add_argument("--experts", type=int, default=0, help="shrink the headline layer (profiling captures only)")
    parser.add_argument("--skip-e2e", action="store_true", help="profiling captures only")
    parser.add_argument("--skip-cpu", action="store_true", help="profiling captures only")
    parser.add_argument("--skip-peak", action="store_true", help="profiling captures only: do not time the int8 library GEMM")
    parser.add_argument("--skip-calibration", action="store_true",
                        help="end-to-end legs run under a planner runtime without a calibrated tile table (automatic tiles)")
    args = parser.parse_args()
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
