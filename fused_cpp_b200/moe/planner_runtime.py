"""GPU planner runtime behind the reference's planner entry points.

The reference's quick planner calibrates a CPU cost model and, per call, searches team widths and
lane assignments (src/fused_cpp/moe/planner_runtime.py:35-391; quick calibration in
cpu_moe_schedule_optimization/cost_model/quick_calibration.py:359-426).  None of that has a GPU
meaning.  What carries over is its per-shape geometry table -- bands over the route count that map
to (w13 window, w2 window) with 0 = default (planners/stage_window_policy.py:34-97) -- so here:

  * calibrate_moe_planner_quick() times the candidate row tiles of the tcgen05 grouped GEMM on the
    current GPU for a ladder of rows-per-expert buckets (the reference's bucket list,
    planners/planned_moe.py:14) and writes a JSON profile (atomic, refuses to overwrite);
  * MoePlannerRuntime looks the bucket up from the call's shape alone -- it never reads topk_ids on
    the host -- and returns a one-task strict Plan V2 whose window fields carry the two row tiles;
  * enable_moe_planner_quick() = calibrate, construct, install, in that order (install only after
    both succeeded), as the reference does.
"""
from __future__ import annotations

import json
import os
import tempfile
import threading
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable, Sequence

import torch

from .plan import AsyncMoEPlanV2, gpu_placeholder_plan

DEFAULT_MOE_COST_CACHE_DIR = Path(os.environ.get("FUSED_CPP_MOE_COST_CACHE_DIR", Path.home() / ".cache" / "fused_cpp_b200" / "moe"))
ROUTE_BUCKETS = (1, 2, 4, 8, 12, 24, 48, 96, 192, 384, 768, 1536, 2040, 4096, 8192)
# 0 = the library's automatic choice (by batch size, and above 64 tokens a per-expert split made on the device);
# 512 = the two-SM (cta_group::2) kernel with 256-row items for every expert.
CANDIDATE_TILES = (0, 16, 32, 64, 128, 256, 512)
PROFILE_SCHEMA = 1


@dataclass(frozen=True)
class GpuTileCalibration:
    """Row-tile table of one GPU: kind ('int8'|'bf16') -> {bucket: (gate_up_tile, down_tile)}."""
    machine_id: str
    gpu_name: str
    sm_count: int
    tiles: dict = field(default_factory=dict)
    timings_ms: dict = field(default_factory=dict)
    schema: int = PROFILE_SCHEMA

    def lookup(self, kind: str, rows_per_expert: int) -> tuple[int, int]:
        table = self.tiles.get(kind, {})
        best = None
        for bucket in sorted(int(b) for b in table):
            best = bucket
            if rows_per_expert <= bucket:
                break
        if best is None:
            # No measurement for this kind: 0 = the library's own choice (by batch size up to 64 tokens, above that a
            # per-expert split between the one-SM and the two-SM kernel made on the device from the actual routing).
            return 0, 0
        pair = table.get(best, table.get(str(best)))
        return int(pair[0]), int(pair[1])

    def to_json(self) -> str:
        payload = asdict(self)
        payload["tiles"] = {k: {str(b): list(v) for b, v in t.items()} for k, t in self.tiles.items()}
        payload["timings_ms"] = {k: {str(b): v for b, v in t.items()} for k, t in self.timings_ms.items()}
        return json.dumps(payload, indent=1, sort_keys=True)

    @classmethod
    def from_json(cls, text: str) -> "GpuTileCalibration":
        payload = json.loads(text)
        if int(payload.get("schema", -1)) != PROFILE_SCHEMA:
            raise ValueError(f"unsupported GPU tile profile schema {payload.get('schema')!r}")
        tiles = {k: {int(b): tuple(v) for b, v in t.items()} for k, t in payload.get("tiles", {}).items()}
        timings = {k: {int(b): v for b, v in t.items()} for k, t in payload.get("timings_ms", {}).items()}
        return cls(machine_id=str(payload["machine_id"]), gpu_name=str(payload["gpu_name"]), sm_count=int(payload["sm_count"]),
                   tiles=tiles, timings_ms=timings)


@dataclass(frozen=True)
class QuickMoeCalibrationResult:
    calibration: GpuTileCalibration
    output_path: Path | None
    cpu_ids: tuple[int, ...]
    service_widths: tuple[int, ...]
    supported_widths: tuple[int, ...]
    elapsed_seconds: float
    fit_report: dict


# Device memory the probe layer's weights may take (bytes): the layer keeps the caller's H and I and as many of its
# local experts as fit, so that tile timings are taken at the real operand widths.
PROBE_WEIGHT_BYTES = 3 << 30
DEFAULT_PROBE_SHAPE = (2048, 1024, 32)  # (hidden, inter, experts) when no layer shape is given
CALIBRATION_BUCKETS = (1, 2, 4, 8, 24, 48, 96, 192, 384)


def _probe_layer(kind: str, hidden: int, inter: int, experts: int, device: torch.device, seed: int) -> dict:
    """Random weights of the probe layer, generated on the device (values do not affect timing)."""
    per_expert = 3 * hidden * inter * (1 if kind == "int8" else 2)
    experts = max(2, min(int(experts), PROBE_WEIGHT_BYTES // per_expert))
    generator = torch.Generator(device=device).manual_seed(seed)
    if kind == "int8":
        return {"experts": experts,
                "w13": torch.randint(-127, 128, (experts, 2 * inter, hidden), generator=generator, dtype=torch.int8, device=device),
                "w2": torch.randint(-127, 128, (experts, hidden, inter), generator=generator, dtype=torch.int8, device=device),
                "s13": torch.full((experts, 2 * inter), 1e-3, device=device), "s2": torch.full((experts, hidden), 1e-3, device=device)}
    return {"experts": experts,
            "w13": torch.empty((experts, 2 * inter, hidden), dtype=torch.bfloat16, device=device).normal_(0.0, 0.02, generator=generator),
            "w2": torch.empty((experts, hidden, inter), dtype=torch.bfloat16, device=device).normal_(0.0, 0.02, generator=generator),
            "s13": None, "s2": None}


def _probe_routing(rows_per_expert: int, experts: int, skewed: bool, seed: int):
    """(tokens, top-k ids [T, K]) with `rows_per_expert` routes per expert on average.  Uniform: every expert gets
    exactly that many.  Skewed: softmax top-k of N(0,1) logits plus the Zipf-like bias 2 ln(1/(rank+1)), the
    benchmark's skewed router, so a few experts take most routes and some take none."""
    top_k = min(8, experts)
    routes = max(top_k, rows_per_expert * experts)
    tokens = max(1, routes // top_k)
    if not skewed:
        ids = (torch.arange(tokens * top_k, dtype=torch.int64) % experts).reshape(tokens, top_k)
        return tokens, ids
    generator = torch.Generator(device="cpu").manual_seed(seed)
    rank = torch.randperm(experts, generator=generator).to(torch.float32)
    logits = torch.randn((tokens, experts), generator=generator) + 2.0 * torch.log(1.0 / (rank + 1.0))
    return tokens, torch.topk(logits, top_k, dim=-1).indices.to(torch.int64).contiguous()


def _probe_tiles(kind: str, rows_per_expert: int, tiles: Sequence[int], seed: int, hidden: int, inter: int, experts: int,
                 repeats: int = 8, _cache: dict | None = None) -> dict[int, float]:
    """Time one forward per candidate tile on a probe layer of the caller's H and I: the sum of a uniformly routed
    batch and a skewed one with `rows_per_expert` routes per expert on average (ms)."""
    from .. import _lib

    device = torch.device("cuda", torch.cuda.current_device())
    cache = _cache if _cache is not None else {}
    key = (kind, hidden, inter, experts)
    if key not in cache:
        cache.clear()  # one probe layer at a time on the device
        cache[key] = _probe_layer(kind, hidden, inter, experts, device, seed)
    layer = cache[key]
    result: dict[int, float] = {int(tile): 0.0 for tile in tiles}
    for skewed in (False, True):
        tokens, ids = _probe_routing(rows_per_expert, layer["experts"], skewed, seed + 1)
        ids = ids.to(device)
        generator = torch.Generator(device=device).manual_seed(seed + 2)
        x = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=device).normal_(0.0, 1.0, generator=generator)
        weights = torch.full(ids.shape, 1.0 / ids.shape[1], dtype=torch.float32, device=device)
        for tile in tiles:
            def run():
                return _lib.moe_forward(x, layer["w13"], layer["w2"], weights, ids, s13=layer["s13"], s2=layer["s2"],
                                        gate_up_tile=tile, down_tile=tile)
            run()
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(repeats):
                run()
            stop.record()
            torch.cuda.synchronize()
            result[int(tile)] += start.elapsed_time(stop) / repeats
    return result


def calibrate_moe_planner_quick(cpu_ids: Sequence[int] | None = None, *, output: str | Path | None = None,
                                supported_widths: Sequence[int] | None = None, machine_id: str | None = None,
                                overwrite: bool = False, seed: int = 20260814, report: Callable[[str], None] | None = None,
                                _probe: Callable[..., dict[int, float]] | None = None,
                                _buckets: Sequence[int] | None = None,
                                _shape: tuple[int, int, int] | None = None) -> QuickMoeCalibrationResult:
    """Time the grouped GEMM's row tiles per rows-per-expert bucket on this GPU and write the profile.

    Signature of the reference's quick calibration (quick_calibration.py:359-368).  `cpu_ids` is kept
    for compatibility and recorded only; `supported_widths` names the candidate row tiles
    (default: automatic and 16..512).  `_shape` = (hidden, inter, local experts) of the layer the table is for
    (enable_moe_planner_quick passes its own; a bare call probes a small default layer); `_probe` lets tests
    substitute synthetic timings.
    """
    begin = time.perf_counter()
    path = Path(output) if output is not None else None
    if path is not None and path.exists() and not overwrite:
        raise FileExistsError(f"{path} already exists; pass overwrite=True to replace it")
    tiles = tuple(int(t) for t in (supported_widths or CANDIDATE_TILES))
    if any(t not in CANDIDATE_TILES for t in tiles):
        raise ValueError(f"supported_widths (row tiles) must be drawn from {CANDIDATE_TILES}")
    hidden, inter, experts = (int(v) for v in (_shape or DEFAULT_PROBE_SHAPE))
    probe = _probe
    probe_kwargs: dict = {}
    if probe is None:
        from .. import _lib

        if not _lib.device_supported():
            raise RuntimeError("quick calibration requires a compute-capability-10.x CUDA device")
        probe = _probe_tiles
        probe_kwargs = {"_cache": {}}
        gpu_name = torch.cuda.get_device_name()
        sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    else:
        gpu_name, sm_count = "synthetic", 0
    buckets = tuple(_buckets) if _buckets is not None else CALIBRATION_BUCKETS
    table: dict[str, dict[int, tuple[int, int]]] = {}
    timings: dict[str, dict[int, dict[int, float]]] = {}
    for kind in ("int8", "bf16"):
        table[kind], timings[kind] = {}, {}
        for bucket in buckets:
            measured = probe(kind, bucket, tiles, seed, hidden, inter, experts, **probe_kwargs)
            best = min(measured, key=lambda t: (measured[t], t))
            # A fixed tile that is not clearly faster on the probe batches is not worth giving up the automatic
            # choice, which adapts to the routing of every batch.
            if 0 in measured and measured[0] <= 1.05 * measured[best]:
                best = 0
            table[kind][int(bucket)] = (int(best), int(best))
            timings[kind][int(bucket)] = {int(t): float(v) for t, v in measured.items()}
            if report is not None:
                report(f"[quick-calibration] {kind} H={hidden} I={inter} rows/expert<={bucket}: tile {best} ({measured[best]:.3f} ms)")
    probe_kwargs.clear()
    calibration = GpuTileCalibration(machine_id=machine_id or gpu_name, gpu_name=gpu_name, sm_count=int(sm_count), tiles=table,
                                     timings_ms=timings)
    if path is not None:
        path.parent.mkdir(parents=True, exist_ok=True)
        handle, temp_name = tempfile.mkstemp(prefix=path.name + ".", suffix=".tmp", dir=str(path.parent))
        try:
            with os.fdopen(handle, "w") as stream:
                stream.write(calibration.to_json())
            os.replace(temp_name, path)
        except BaseException:
            if os.path.exists(temp_name):
                os.unlink(temp_name)
            raise
    resolved_cpus = tuple(int(c) for c in cpu_ids) if cpu_ids is not None else tuple(sorted(os.sched_getaffinity(0)))
    return QuickMoeCalibrationResult(calibration=calibration, output_path=path, cpu_ids=resolved_cpus, service_widths=tiles,
                                     supported_widths=tiles, elapsed_seconds=time.perf_counter() - begin,
                                     fit_report={"buckets": list(buckets), "kinds": ["int8", "bf16"], "probe_shape": [hidden, inter, experts],
                                                 "routings": ["uniform", "zipf"]})


class MoePlannerRuntime:
    """Thread-safe tile chooser for one GPU and one expert shape (interface of planner_runtime.py:35-317)."""

    def __init__(self, calibration: GpuTileCalibration | str | Path | None, *, hidden_size: int, intermediate_size: int,
                 global_experts: int, local_experts: int, mode: str = "standalone", degree: int = 1, concurrent_ranks: int = 1,
                 cpu_ids: Sequence[int] | None = None, shared_experts: int = 0,
                 cost_cache_dir: str | Path | None = DEFAULT_MOE_COST_CACHE_DIR) -> None:
        if int(shared_experts) not in (0, 1):
            raise ValueError("shared_experts must be 0 or 1")
        if mode not in ("standalone", "tp", "ep"):
            raise ValueError(f"unsupported mode {mode!r}")
        if isinstance(calibration, (str, Path)):
            calibration = GpuTileCalibration.from_json(Path(calibration).read_text())
        if calibration is None:
            calibration = GpuTileCalibration(machine_id="builtin", gpu_name="builtin", sm_count=0)
        self.calibration = calibration
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.global_experts = int(global_experts)
        self.local_experts = int(local_experts)
        self.shared_experts = int(shared_experts)
        self.mode = str(mode)
        self.degree = int(degree)
        self.concurrent_ranks = int(concurrent_ranks)
        self.cpu_ids = tuple(int(c) for c in cpu_ids) if cpu_ids is not None else ()
        self.num_cores = len(self.cpu_ids)
        self.cost_cache_dir = None if cost_cache_dir is None else Path(cost_cache_dir)
        self._lock = threading.RLock()
        self._last: dict[str, object] = {}

    def initialize_planner(self, max_routes: int) -> dict[str, object]:
        if int(max_routes) <= 0:
            raise ValueError(f"max_routes must be positive, got {max_routes}")
        return {"initialized": True, "max_routes": int(max_routes), "generated_entries": 0, "total_entries": 0, "elapsed_ms": 0.0}

    def _shape_ok(self, packed: Any, experts: int) -> bool:
        return (int(packed.w13[0].shape[0]) == experts and int(packed.w13[1]) == self.hidden_size
                and int(packed.w13[2]) == 2 * self.intermediate_size and int(packed.w2[1]) == self.intermediate_size
                and int(packed.w2[2]) == self.hidden_size)

    def _plan(self, packed: Any, topk_ids: torch.Tensor, experts: int, label: str) -> AsyncMoEPlanV2:
        if type(packed).__name__.startswith("PreparedW8A16"):
            kind = "w8a16"  # no tile table of its own: the library's automatic choice
        else:
            kind = "int8" if packed.w13[0].dtype == torch.int8 else "bf16"
        routes = int(topk_ids.shape[0]) * int(topk_ids.shape[1])
        rows_per_expert = max(1, -(-routes // max(1, experts)))
        gate_up_tile, down_tile = self.calibration.lookup(kind, rows_per_expert)
        with self._lock:
            self._last = {"planner": "gpu_tile_table", "dispatch": label, "kind": kind, "routes": routes,
                          "rows_per_expert": rows_per_expert, "gate_up_tile": gate_up_tile, "down_tile": down_tile,
                          "machine_id": self.calibration.machine_id, "calibrated": bool(self.calibration.tiles.get(kind))}
        return gpu_placeholder_plan(gate_up_tile, down_tile)

    def plan_for_dispatch(self, weights: Any, topk_ids: torch.Tensor, *, num_threads: int, activation: Any,
                          global_num_experts: int) -> AsyncMoEPlanV2 | None:
        """A plan when this runtime owns the call, else None.  Uses shapes only: no host read of topk_ids."""
        activation_name = getattr(activation, "value", activation)
        effective = self.global_experts if int(global_num_experts) < 0 else int(global_num_experts)
        if (self.shared_experts != 0 or str(activation_name) != "silu" or effective != self.global_experts
                or not self._shape_ok(weights, self.local_experts) or topk_ids.dim() != 2 or topk_ids.numel() == 0):
            return None
        return self._plan(weights, topk_ids, self.local_experts, "routed")

    def plan_for_shared_dispatch(self, weights: Any, combined_topk_ids: torch.Tensor, *, num_threads: int,
                                 activation: Any) -> AsyncMoEPlanV2 | None:
        activation_name = getattr(activation, "value", activation)
        packed = getattr(weights, "packed", None)
        if (self.shared_experts != 1 or packed is None or str(activation_name) != "silu"
                or int(getattr(weights, "routed_experts", -1)) != self.local_experts
                or int(getattr(weights, "shared_expert_id", -1)) != self.local_experts
                or not self._shape_ok(packed, self.local_experts + 1) or combined_topk_ids.dim() != 2
                or combined_topk_ids.numel() == 0):
            return None
        return self._plan(packed, combined_topk_ids, self.local_experts + 1, "routed+shared")

    @property
    def last_plan(self) -> dict[str, object]:
        with self._lock:
            return dict(self._last)


_default_runtime_lock = threading.RLock()
_default_runtime: MoePlannerRuntime | None = None


def set_default_moe_planner_runtime(runtime: MoePlannerRuntime | None) -> MoePlannerRuntime | None:
    """Install `runtime` for normal fused-MoE dispatch and return the previous one."""
    if runtime is not None and not isinstance(runtime, MoePlannerRuntime):
        raise TypeError("runtime must be a MoePlannerRuntime or None")
    global _default_runtime
    with _default_runtime_lock:
        previous, _default_runtime = _default_runtime, runtime
        return previous


def get_default_moe_planner_runtime() -> MoePlannerRuntime | None:
    with _default_runtime_lock:
        return _default_runtime


def enable_moe_planner_quick(*, hidden_size: int, intermediate_size: int, global_experts: int, local_experts: int,
                             cpu_ids: Sequence[int] | None = None, mode: str = "standalone", degree: int = 1,
                             concurrent_ranks: int = 1, shared_experts: int = 0,
                             cost_cache_dir: str | Path | None = DEFAULT_MOE_COST_CACHE_DIR, output: str | Path | None = None,
                             supported_widths: Sequence[int] | None = None, machine_id: str | None = None,
                             overwrite: bool = False, seed: int = 20260814,
                             report: Callable[[str], None] | None = None) -> MoePlannerRuntime:
    """Calibrate, construct and install the default planner runtime (planner_runtime.py:348-391)."""
    result = calibrate_moe_planner_quick(cpu_ids, output=output, supported_widths=supported_widths, machine_id=machine_id,
                                         overwrite=overwrite, seed=seed, report=report,
                                         _shape=(int(hidden_size), int(intermediate_size), int(local_experts) + int(shared_experts)))
    runtime = MoePlannerRuntime(result.calibration, hidden_size=hidden_size, intermediate_size=intermediate_size,
                                global_experts=global_experts, local_experts=local_experts, mode=mode, degree=degree,
                                concurrent_ranks=concurrent_ranks, cpu_ids=result.cpu_ids, shared_experts=shared_experts,
                                cost_cache_dir=cost_cache_dir)
    set_default_moe_planner_runtime(runtime)
    return runtime


__all__ = ["DEFAULT_MOE_COST_CACHE_DIR", "GpuTileCalibration", "MoePlannerRuntime", "QuickMoeCalibrationResult",
           "calibrate_moe_planner_quick", "enable_moe_planner_quick", "get_default_moe_planner_runtime",
           "set_default_moe_planner_runtime"]
