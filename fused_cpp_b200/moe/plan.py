"""Plan V2: the versioned execution-plan record that rides through the fused-MoE op signatures.

Field names, defaults and acceptance rules follow the reference's plan carrier
(src/fused_cpp/moe/plan.py:79-405) so that plans produced for it load here unchanged.  On the GPU
the CPU placement fields (cores, widths, dependencies) are validated for shape and otherwise
ignored; `task_w13_window_tiles[0]` / `task_w2_window_tiles[0]` keep their role as per-stage
geometry selectors and carry the row-tile of the gate_up / down grouped GEMM (0 = automatic).
"""
from __future__ import annotations

import functools

from dataclasses import dataclass, fields
from typing import Mapping, Sequence

import torch

ASYNC_MOE_PLAN_VERSION = 2
ASYNC_MOE_EXECUTION_STRICT = "strict"
ASYNC_MOE_EXECUTION_TAIL_POOL = "tail_pool"
ASYNC_MOE_PLACEMENT_FIXED = 0
ASYNC_MOE_PLACEMENT_TAIL_POOL = 1
ASYNC_MOE_STAGE_EXPERT = 0
ASYNC_MOE_RESIZE_NONE = 0
ASYNC_MOE_FULL_EXPERT_RANGE = 0

_INT_DTYPES = (torch.int8, torch.int16, torch.int32, torch.int64)
_PER_TASK = ("task_core_begins", "task_threads", "task_preferred_threads", "task_min_threads", "task_max_threads",
             "task_placement_modes", "task_numa_nodes", "task_stage_ids", "task_resize_points",
             "task_range_granularities", "task_w13_window_tiles", "task_w2_window_tiles")
_REQUIRED_VECTORS = ("thread_cpu_ids", "task_expert_ids", "task_core_begins", "task_threads", "task_dep_offsets",
                     "task_deps", "task_preferred_threads", "task_min_threads", "task_max_threads",
                     "task_allowed_thread_offsets", "task_allowed_threads", "task_placement_modes", "task_numa_nodes",
                     "task_stage_ids", "task_resize_points", "task_range_granularities")
_OPTIONAL_VECTORS = ("task_w13_window_tiles", "task_w2_window_tiles")
_RETIRED = ("task_release_ns", "task_resize_timeout_ns", "task_preferred_core_begins")


def _as_vector(value: object, name: str) -> torch.Tensor:
    if isinstance(value, torch.Tensor):
        if value.device.type != "cpu":
            raise ValueError(f"{name} must be a CPU tensor")
        if value.dtype not in _INT_DTYPES:
            raise TypeError(f"{name} must use an integer dtype, got {value.dtype}")
        if value.dim() != 1:
            raise ValueError(f"{name} must be 1-D")
        return value.to(torch.int64).contiguous()
    if isinstance(value, (str, bytes)) or not isinstance(value, Sequence):
        raise TypeError(f"{name} must be a 1-D integer sequence or tensor")
    try:
        return torch.tensor([int(v) for v in value], dtype=torch.int64)
    except (TypeError, ValueError) as error:
        raise TypeError(f"{name} must contain integers") from error


def _check_csr(offsets: list[int], payload: list[int], tasks: int, name: str) -> None:
    if len(offsets) != tasks + 1:
        raise ValueError(f"{name} must have num_tasks + 1 entries")
    if offsets[0] != 0:
        raise ValueError(f"{name}[0] must be 0")
    if offsets[-1] != len(payload):
        raise ValueError(f"last {name} entry must equal the length of its payload")
    if any(a > b for a, b in zip(offsets, offsets[1:])):
        raise ValueError(f"{name} must be non-decreasing")


@dataclass(frozen=True)
class AsyncMoEPlanV2:
    num_threads: int
    execution_mode: str
    thread_cpu_ids: torch.Tensor
    task_expert_ids: torch.Tensor
    task_core_begins: torch.Tensor
    task_threads: torch.Tensor
    task_dep_offsets: torch.Tensor
    task_deps: torch.Tensor
    task_preferred_threads: torch.Tensor
    task_min_threads: torch.Tensor
    task_max_threads: torch.Tensor
    task_allowed_thread_offsets: torch.Tensor
    task_allowed_threads: torch.Tensor
    task_placement_modes: torch.Tensor
    task_numa_nodes: torch.Tensor
    task_stage_ids: torch.Tensor
    task_resize_points: torch.Tensor
    task_range_granularities: torch.Tensor
    task_w13_window_tiles: torch.Tensor | None = None
    task_w2_window_tiles: torch.Tensor | None = None
    early_merge: bool | None = None

    @property
    def plan_version(self) -> int:
        return ASYNC_MOE_PLAN_VERSION

    @property
    def native_execution_mode(self) -> int:
        return 0 if self.execution_mode == ASYNC_MOE_EXECUTION_STRICT else 1

    @property
    def native_early_merge(self) -> int:
        return -1 if self.early_merge is None else int(self.early_merge)

    def __post_init__(self) -> None:
        tasks = int(self.task_expert_ids.numel()) if isinstance(self.task_expert_ids, torch.Tensor) else 0
        for name in _OPTIONAL_VECTORS:
            if getattr(self, name) is None:
                object.__setattr__(self, name, torch.zeros(tasks, dtype=torch.int64))
        self.validate()

    @classmethod
    def from_dict(cls, plan: Mapping[str, object]) -> "AsyncMoEPlanV2":
        retired = sorted(set(_RETIRED) & set(plan))
        if retired:
            raise ValueError(f"{', '.join(retired)} has been retired from Plan V2")
        version = int(plan.get("plan_version", -1))
        if version != ASYNC_MOE_PLAN_VERSION:
            raise ValueError(f"plan_version must be {ASYNC_MOE_PLAN_VERSION}, got {version}")
        missing = [name for name in ("num_threads", "execution_mode", *_REQUIRED_VECTORS) if name not in plan]
        if missing:
            raise ValueError(f"Plan V2 is missing required fields: {', '.join(missing)}")
        vectors = {name: _as_vector(plan[name], name) for name in _REQUIRED_VECTORS}
        tasks = int(vectors["task_expert_ids"].numel())
        for name in _OPTIONAL_VECTORS:
            vectors[name] = _as_vector(plan.get(name, [0] * tasks), name)
        early_merge = plan.get("early_merge")
        if early_merge is not None and type(early_merge) is not bool:
            raise TypeError("early_merge must be a bool or None")
        return cls(num_threads=int(plan["num_threads"]), execution_mode=str(plan["execution_mode"]),
                   early_merge=early_merge, **vectors)

    @classmethod
    def _from_planner_bridge(cls, plan: Mapping[str, object]) -> "AsyncMoEPlanV2":
        """Materialise a bridge that this package's own planner built (plan.py:182-199 of the reference skips the
        per-element conversion and the validation for those, about 1 ms per call on its CPU path).  The GPU planner's
        plans are single-task placeholders, so the ordinary constructor is fast enough and is what runs here."""
        return cls.from_dict(plan)

    def validate(self) -> None:
        if self.execution_mode not in (ASYNC_MOE_EXECUTION_STRICT, ASYNC_MOE_EXECUTION_TAIL_POOL):
            raise ValueError(f"execution_mode must be 'strict' or 'tail_pool', got {self.execution_mode!r}")
        if self.num_threads <= 0:
            raise ValueError(f"num_threads must be positive, got {self.num_threads}")
        if self.early_merge is not None and type(self.early_merge) is not bool:
            raise TypeError("early_merge must be a bool or None")
        lists: dict[str, list[int]] = {}
        for field in fields(self):
            if field.name in ("num_threads", "execution_mode", "early_merge"):
                continue
            tensor = getattr(self, field.name)
            if not isinstance(tensor, torch.Tensor):
                raise TypeError(f"{field.name} must be a tensor in a materialized plan")
            if tensor.device.type != "cpu":
                raise ValueError(f"{field.name} must be a CPU tensor")
            if tensor.dtype not in _INT_DTYPES:
                raise TypeError(f"{field.name} must use an integer dtype, got {tensor.dtype}")
            if tensor.dim() != 1:
                raise ValueError(f"{field.name} must be 1-D")
            lists[field.name] = [int(v) for v in tensor.tolist()]

        cpus = lists["thread_cpu_ids"]
        if len(cpus) != self.num_threads:
            raise ValueError(f"thread_cpu_ids must have exactly num_threads entries: got {len(cpus)} vs {self.num_threads}")
        if any(cpu < 0 for cpu in cpus):
            raise ValueError("thread_cpu_ids must be non-negative")
        if len(set(cpus)) != len(cpus):
            raise ValueError("thread_cpu_ids must not contain duplicates")
        experts = lists["task_expert_ids"]
        tasks = len(experts)
        if tasks == 0:
            raise ValueError("Plan V2 must contain at least one task")
        if any(e < 0 for e in experts):
            raise ValueError("task_expert_ids must be non-negative")
        for name in _PER_TASK:
            if len(lists[name]) != tasks:
                raise ValueError(f"{name} must have one entry per task: got {len(lists[name])} vs {tasks}")
        strict = self.execution_mode == ASYNC_MOE_EXECUTION_STRICT
        grains = lists["task_range_granularities"]
        if any(g < 0 for g in grains):
            raise ValueError("task_range_granularities must be non-negative")
        for name in _OPTIONAL_VECTORS:
            if any(w < 0 for w in lists[name]):
                raise ValueError(f"{name} must be non-negative, 0 meaning the full stripe")
        by_expert: dict[int, list[int]] = {}
        for task, expert in enumerate(experts):
            by_expert.setdefault(expert, []).append(task)
        for expert, ids in by_expert.items():
            kinds = {grains[t] for t in ids}
            if len(ids) == 1:
                if kinds != {ASYNC_MOE_FULL_EXPERT_RANGE}:
                    raise ValueError(f"single-task expert {expert} must use the full-expert range")
            else:
                if not strict:
                    raise ValueError("route-sliced experts currently require strict execution")
                if len(kinds) != 1 or ASYNC_MOE_FULL_EXPERT_RANGE in kinds:
                    raise ValueError(f"route-sliced expert {expert} must use one shared positive granularity")
        begins, widths, modes = lists["task_core_begins"], lists["task_threads"], lists["task_placement_modes"]
        for task in range(tasks):
            if widths[task] <= 0:
                raise ValueError(f"task_threads[{task}] must be positive")
            if modes[task] == ASYNC_MOE_PLACEMENT_FIXED:
                if begins[task] < 0:
                    raise ValueError(f"fixed task_core_begins[{task}] must be non-negative")
                if begins[task] + widths[task] > self.num_threads:
                    raise ValueError(f"task {task} interval [{begins[task]}, {begins[task] + widths[task]}) exceeds "
                                     f"num_threads={self.num_threads}")
            elif modes[task] == ASYNC_MOE_PLACEMENT_TAIL_POOL:
                if begins[task] != -1:
                    raise ValueError(f"tail-pool task_core_begins[{task}] must be -1")
            else:
                raise ValueError(f"task_placement_modes[{task}] has unsupported value {modes[task]}")
        if strict and any(m != ASYNC_MOE_PLACEMENT_FIXED for m in modes):
            raise ValueError("strict Plan V2 requires every task placement to be fixed")
        if any(n != -1 for n in lists["task_numa_nodes"]):
            raise ValueError("strict and tail_pool Plan V2 require task_numa_nodes=-1")
        if any(s != ASYNC_MOE_STAGE_EXPERT for s in lists["task_stage_ids"]):
            raise ValueError("Plan V2 currently only supports whole-expert tasks")
        if any(p != ASYNC_MOE_RESIZE_NONE for p in lists["task_resize_points"]):
            raise ValueError("strict and tail_pool Plan V2 do not support resize points")
        if not strict and any(g != ASYNC_MOE_FULL_EXPERT_RANGE for g in grains):
            raise ValueError("tail-pool Plan V2 requires full-expert task ranges")

        dep_offsets, deps = lists["task_dep_offsets"], lists["task_deps"]
        _check_csr(dep_offsets, deps, tasks, "task_dep_offsets")
        for task in range(tasks):
            mine = deps[dep_offsets[task]:dep_offsets[task + 1]]
            if any(d < 0 or d >= task for d in mine):
                raise ValueError(f"task {task} dependencies must refer to earlier task ids")
            if modes[task] == ASYNC_MOE_PLACEMENT_TAIL_POOL and mine:
                raise ValueError(f"tail-pool task {task} must not have dependencies")
            if modes[task] == ASYNC_MOE_PLACEMENT_FIXED and any(modes[d] == ASYNC_MOE_PLACEMENT_TAIL_POOL for d in mine):
                raise ValueError(f"fixed task {task} must not depend on a tail-pool task")

        allowed_offsets, allowed = lists["task_allowed_thread_offsets"], lists["task_allowed_threads"]
        _check_csr(allowed_offsets, allowed, tasks, "task_allowed_thread_offsets")
        preferred, lows, highs = lists["task_preferred_threads"], lists["task_min_threads"], lists["task_max_threads"]
        for task in range(tasks):
            mine = allowed[allowed_offsets[task]:allowed_offsets[task + 1]]
            if not mine:
                raise ValueError(f"task {task} must allow at least one thread width")
            if any(w <= 0 or w > self.num_threads for w in mine):
                raise ValueError(f"task {task} allowed widths are out of range")
            if any(a >= b for a, b in zip(mine, mine[1:])):
                raise ValueError(f"task {task} allowed widths must be strictly increasing")
            if widths[task] not in mine:
                raise ValueError(f"task_threads[{task}] is not present in its allowed widths")
            if preferred[task] not in mine:
                raise ValueError(f"task_preferred_threads[{task}] is not in its allowed widths")
            if lows[task] != mine[0]:
                raise ValueError(f"task_min_threads[{task}] does not match its allowed widths")
            if highs[task] != mine[-1]:
                raise ValueError(f"task_max_threads[{task}] does not match its allowed widths")
            if modes[task] == ASYNC_MOE_PLACEMENT_FIXED and begins[task] + mine[-1] > self.num_threads:
                raise ValueError(f"task {task} allowed widths exceed its fixed logical-core placement")
        if not strict:
            pooled = [t for t in range(tasks) if modes[t] == ASYNC_MOE_PLACEMENT_TAIL_POOL]
            if not pooled:
                raise ValueError("tail_pool execution requires at least one pooled task")
            pool_widths = {widths[t] for t in pooled}
            if len(pool_widths) != 1:
                raise ValueError("all tail-pool tasks must use the same selected width")
            pool = pool_widths.pop()
            if pool > self.num_threads or self.num_threads % pool != 0:
                raise ValueError(f"tail-pool task width must divide num_threads: pool_width={pool}, num_threads={self.num_threads}")
            for task in range(tasks):
                if modes[task] == ASYNC_MOE_PLACEMENT_FIXED and (begins[task] % pool or widths[task] % pool):
                    raise ValueError(f"fixed task intervals must align to the tail-pool width: task={task}")

    def legacy_schedule(self):
        if self.execution_mode != ASYNC_MOE_EXECUTION_STRICT:
            raise RuntimeError("only strict Plan V2 can be lowered to the legacy executor")
        return (self.task_expert_ids, self.task_core_begins, self.task_threads, self.task_dep_offsets, self.task_deps)


def upgrade_legacy_async_plan(plan: Mapping[str, object]) -> dict[str, object]:
    """Lift a legacy fixed-width async bridge (src/fused_cpp/moe/plan.py:428-447) to strict Plan V2."""
    widths = [int(w) for w in plan["task_threads"]]  # type: ignore[index]
    tasks = len(widths)
    upgraded = dict(plan)
    upgraded.update(
        plan_version=ASYNC_MOE_PLAN_VERSION, execution_mode=ASYNC_MOE_EXECUTION_STRICT,
        task_preferred_threads=list(widths), task_min_threads=list(widths), task_max_threads=list(widths),
        task_allowed_thread_offsets=list(range(tasks + 1)), task_allowed_threads=list(widths),
        task_placement_modes=[ASYNC_MOE_PLACEMENT_FIXED] * tasks, task_numa_nodes=[-1] * tasks,
        task_stage_ids=[ASYNC_MOE_STAGE_EXPERT] * tasks, task_resize_points=[ASYNC_MOE_RESIZE_NONE] * tasks,
        task_range_granularities=[ASYNC_MOE_FULL_EXPERT_RANGE] * tasks, early_merge=None)
    return upgraded


def gpu_placeholder_plan(gate_up_tile: int = 0, down_tile: int = 0) -> AsyncMoEPlanV2:
    """The one-task strict plan a GPU runtime hands to the op: no CPU placement, tile ids in the window fields.
    One (immutable) object per tile pair: building and validating twenty small tensors per forward is measurable
    next to a decode layer of 1.4 ms."""
    return _cached_placeholder_plan(int(gate_up_tile), int(down_tile))


@functools.lru_cache(maxsize=256)
def _cached_placeholder_plan(gate_up_tile: int, down_tile: int) -> AsyncMoEPlanV2:
    return AsyncMoEPlanV2(
        num_threads=1, execution_mode=ASYNC_MOE_EXECUTION_STRICT,
        thread_cpu_ids=torch.zeros(1, dtype=torch.int64), task_expert_ids=torch.zeros(1, dtype=torch.int64),
        task_core_begins=torch.zeros(1, dtype=torch.int64), task_threads=torch.ones(1, dtype=torch.int64),
        task_dep_offsets=torch.zeros(2, dtype=torch.int64), task_deps=torch.zeros(0, dtype=torch.int64),
        task_preferred_threads=torch.ones(1, dtype=torch.int64), task_min_threads=torch.ones(1, dtype=torch.int64),
        task_max_threads=torch.ones(1, dtype=torch.int64),
        task_allowed_thread_offsets=torch.tensor([0, 1], dtype=torch.int64),
        task_allowed_threads=torch.ones(1, dtype=torch.int64),
        task_placement_modes=torch.zeros(1, dtype=torch.int64), task_numa_nodes=torch.full((1,), -1, dtype=torch.int64),
        task_stage_ids=torch.zeros(1, dtype=torch.int64), task_resize_points=torch.zeros(1, dtype=torch.int64),
        task_range_granularities=torch.zeros(1, dtype=torch.int64),
        task_w13_window_tiles=torch.tensor([int(gate_up_tile)], dtype=torch.int64),
        task_w2_window_tiles=torch.tensor([int(down_tile)], dtype=torch.int64), early_merge=False)


__all__ = [
    "ASYNC_MOE_EXECUTION_STRICT", "ASYNC_MOE_EXECUTION_TAIL_POOL", "ASYNC_MOE_FULL_EXPERT_RANGE",
    "ASYNC_MOE_PLACEMENT_FIXED", "ASYNC_MOE_PLACEMENT_TAIL_POOL", "ASYNC_MOE_PLAN_VERSION", "ASYNC_MOE_RESIZE_NONE",
    "ASYNC_MOE_STAGE_EXPERT", "AsyncMoEPlanV2", "upgrade_legacy_async_plan", "gpu_placeholder_plan",
]
