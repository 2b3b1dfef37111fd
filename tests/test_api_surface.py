"""The Python surface that mirrors fused_cpp.moe: exports, plan carrier, planner runtime, calibration
files, dispatch logic with fakes (no GPU), and that the C-ABI library exports what the header declares."""
from __future__ import annotations

import ctypes
import os
import re

import pytest
import torch

import fused_cpp_b200.moe as moe
from fused_cpp_b200 import _lib
from fused_cpp_b200.moe import bf16_tiled as module
from fused_cpp_b200.moe import planner_runtime
from fused_cpp_b200.moe.plan import AsyncMoEPlanV2, gpu_placeholder_plan, upgrade_legacy_async_plan

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

REFERENCE_EXPORTS = """ASYNC_MOE_EXECUTION_STRICT ASYNC_MOE_EXECUTION_TAIL_POOL ASYNC_MOE_FULL_EXPERT_RANGE ASYNC_MOE_PLACEMENT_FIXED
ASYNC_MOE_PLACEMENT_TAIL_POOL ASYNC_MOE_PLAN_VERSION ASYNC_MOE_RESIZE_NONE ASYNC_MOE_STAGE_EXPERT AsyncMoEPlanV2
DEFAULT_MOE_COST_CACHE_DIR MoePlannerRuntime PreparedBF16TiledFusedMoEWeights PreparedBF16TiledRoutedSharedMoEWeights
PreparedW8A16TiledFusedMoEWeights PreparedW8A8TiledFusedMoEWeights PreparedW8A16TiledRoutedSharedMoEWeights
PreparedW8A8TiledRoutedSharedMoEWeights _HAS_BF16_TILED_FUSED_MOE _HAS_W8A8_TILED_FUSED_MOE
available_fused_moe_bf16_tiled_backends calibrate_moe_planner_quick enable_moe_planner_quick fused_moe_bf16_tiled
fused_moe_bf16_tiled_with_shared fused_moe_bf16_tiled_scheduled fused_moe_bf16_tiled_async fused_moe_bf16_tiled_async_plan
fused_moe_bf16_tiled_planned_staged fused_moe_bf16_tiled_vllm_staged fused_moe_tiled fused_moe_w8a16_tiled
fused_moe_w8a16_tiled_async_plan fused_moe_w8a8_tiled fused_moe_w8a8_tiled_async_plan fused_moe_w8a16_tiled_with_shared
fused_moe_w8a8_tiled_with_shared shared_mlp_bf16_tiled fused_moe_naive get_default_moe_planner_runtime bf16_tiled_fused_moe
bf16_tiled_fused_moe_scheduled bf16_tiled_fused_moe_async bf16_tiled_fused_moe_async_plan bf16_tiled_fused_moe_planned_staged
bf16_tiled_fused_moe_vllm_staged naive_fused_moe prepare_fused_moe_bf16_tiled_weights prepare_fused_moe_w8a16_tiled_weights
prepare_fused_moe_w8a16_tiled_quantized_weights prepare_fused_moe_w8a8_tiled_weights
prepare_fused_moe_w8a8_tiled_quantized_weights prepare_routed_shared_moe_bf16_tiled_weights
prepare_routed_shared_moe_w8a16_tiled_quantized_weights prepare_routed_shared_moe_w8a8_tiled_quantized_weights
prepare_shared_mlp_bf16_tiled_weights prepare_bf16_tiled_fused_moe_weights set_default_moe_planner_runtime
upgrade_legacy_async_plan""".split()


def test_every_reference_export_exists():
    """The export list of src/fused_cpp/moe/__init__.py:67-126."""
    missing = [name for name in REFERENCE_EXPORTS if not hasattr(moe, name)]
    assert not missing, missing


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "fused_moe_b200.h")).read()
    declared = set(re.findall(r"FMOE_API\s+[\w\s\*]+?\b(fmoe_\w+)\s*\(", header))
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.fmoe_abi_version() == 2


def test_workspace_layout_needs_no_gpu():
    layout = _lib.workspace_layout(True, 16, 4, 16, 2048, 1024)
    assert layout.total_bytes > 64 * 2048 * 4 and layout.status == 0 and layout.route_out % 256 == 0
    with pytest.raises(ValueError, match="multiples of 16"):
        _lib.workspace_layout(True, 16, 4, 16, 2050, 1024)


def _legacy(experts: int, width: int) -> dict:
    tasks = list(range(experts))
    return {"num_threads": experts * width, "thread_cpu_ids": list(range(experts * width)), "task_expert_ids": tasks,
            "task_core_begins": [t * width for t in tasks], "task_threads": [width] * experts,
            "task_dep_offsets": [0] * (experts + 1), "task_deps": []}


def test_plan_v2_round_trip_and_rejections():
    plan = AsyncMoEPlanV2.from_dict(upgrade_legacy_async_plan(_legacy(3, 2)))
    assert plan.plan_version == 2 and plan.native_execution_mode == 0 and plan.native_early_merge == -1
    assert plan.task_w13_window_tiles.tolist() == [0, 0, 0]
    bad = upgrade_legacy_async_plan(_legacy(2, 1))
    bad["plan_version"] = 1
    with pytest.raises(ValueError, match="plan_version must be 2"):
        AsyncMoEPlanV2.from_dict(bad)
    bad = upgrade_legacy_async_plan(_legacy(2, 1))
    bad["task_release_ns"] = [0, 0]
    with pytest.raises(ValueError, match="retired"):
        AsyncMoEPlanV2.from_dict(bad)
    bad = upgrade_legacy_async_plan(_legacy(2, 1))
    bad["thread_cpu_ids"] = [0, 0]
    with pytest.raises(ValueError, match="duplicates"):
        AsyncMoEPlanV2.from_dict(bad)
    bad = upgrade_legacy_async_plan(_legacy(2, 1))
    bad["task_numa_nodes"] = [0, -1]
    with pytest.raises(ValueError, match="task_numa_nodes=-1"):
        AsyncMoEPlanV2.from_dict(bad)
    bad = upgrade_legacy_async_plan(_legacy(2, 1))
    bad["task_w2_window_tiles"] = [-1, 0]
    with pytest.raises(ValueError, match="non-negative"):
        AsyncMoEPlanV2.from_dict(bad)
    bad = upgrade_legacy_async_plan(_legacy(2, 2))
    bad["task_core_begins"] = [0, 3]
    with pytest.raises(ValueError, match="exceeds num_threads"):
        AsyncMoEPlanV2.from_dict(bad)
    placeholder = gpu_placeholder_plan(32, 64)
    assert placeholder.task_w13_window_tiles.tolist() == [32] and placeholder.task_w2_window_tiles.tolist() == [64]


def _w8a8_weights(experts=1, hidden=16, inter=16):
    tensor = torch.empty((experts, 2 * inter, hidden), dtype=torch.int8)
    return moe.PreparedW8A8TiledFusedMoEWeights(w13=(tensor, hidden, 2 * inter, torch.ones((experts, 2 * inter))),
                                                w2=(torch.empty((experts, hidden, inter), dtype=torch.int8), inter, hidden,
                                                    torch.ones((experts, hidden))))


def test_prepared_weight_contract():
    weights = _w8a8_weights()
    assert weights.fused_silu and weights.backend_n_tile == 128 and weights.backend_name == "cuda_sm100_w8a8_tcgen05"


def test_fused_moe_tiled_dispatches_on_weight_type(monkeypatch):
    weights = _w8a8_weights()
    expected = torch.zeros((1, 16), dtype=torch.bfloat16)
    monkeypatch.setattr(module, "fused_moe_w8a8_tiled", lambda *a, **k: expected)
    assert module.fused_moe_tiled(expected, weights, torch.ones((1, 1)), torch.zeros((1, 1), dtype=torch.int64),
                                  swiglu_limit=10.0) is expected
    with pytest.raises(ValueError, match="w13_bias"):
        module.fused_moe_tiled(expected, weights, torch.ones((1, 1)), torch.zeros((1, 1), dtype=torch.int64),
                               w13_bias=torch.zeros(1))
    with pytest.raises(TypeError, match="weights must be"):
        module.fused_moe_tiled(expected, object(), torch.ones((1, 1)), torch.zeros((1, 1), dtype=torch.int64))


def test_w8a8_requires_installed_runtime(monkeypatch):
    monkeypatch.setattr(module, "_require_backend", lambda: None)
    previous = moe.set_default_moe_planner_runtime(None)
    try:
        with pytest.raises(RuntimeError, match="requires an installed MoePlannerRuntime"):
            module.fused_moe_w8a8_tiled(torch.zeros((1, 16), dtype=torch.bfloat16), _w8a8_weights(), torch.ones((1, 1)),
                                        torch.zeros((1, 1), dtype=torch.int64))
    finally:
        moe.set_default_moe_planner_runtime(previous)


def test_w8a8_rejects_unclamped_activation():
    class FakeCuda(torch.Tensor):
        pass
    x = torch.zeros((1, 16), dtype=torch.bfloat16, device="meta")
    # device check comes first for non-CUDA tensors; the limit check is reached with a CUDA-typed stub
    with pytest.raises((TypeError, ValueError)):
        module.fused_moe_w8a8_tiled_async_plan(x, _w8a8_weights(), torch.ones((1, 1)), torch.zeros((1, 1), dtype=torch.int64),
                                               gpu_placeholder_plan(), swiglu_limit=0.0)


def test_routed_shared_wrapper_appends_one_all_token_route(monkeypatch):
    """Mirror of tests/test_moe_w8a8.py:105-162 of the reference, with fakes for the runtime and executor."""
    packed = _w8a8_weights(experts=3)
    weights = moe.PreparedW8A8TiledRoutedSharedMoEWeights(packed=packed, routed_experts=2, shared_expert_id=2)
    captured = {}

    class FakeRuntime:
        def plan_for_shared_dispatch(self, _weights, combined_ids, **kwargs):
            captured["planned_ids"] = combined_ids.clone()
            return object()

    def fake_execute(_input, _packed, combined_weights, combined_ids, _plan, **kwargs):
        captured["ids"], captured["weights"], captured["kwargs"] = combined_ids.clone(), combined_weights.clone(), kwargs
        return expected

    expected = torch.empty((2, 16), dtype=torch.bfloat16)
    monkeypatch.setattr(module, "_require_backend", lambda: None)
    monkeypatch.setattr(module, "_check_shared_call", lambda *a: 1.0)
    monkeypatch.setattr("fused_cpp_b200.moe.planner_runtime.get_default_moe_planner_runtime", lambda: FakeRuntime())
    monkeypatch.setattr(module, "fused_moe_w8a8_tiled_async_plan", fake_execute)
    ids = torch.tensor([[0, 1], [1, 0]], dtype=torch.int64)
    w = torch.tensor([[0.7, 0.3], [0.4, 0.6]], dtype=torch.float32)
    actual = module.fused_moe_w8a8_tiled_with_shared(torch.zeros((2, 16), dtype=torch.bfloat16), weights, w, ids, num_threads=4,
                                                     swiglu_limit=10.0, out=expected)
    assert actual is expected
    assert torch.equal(captured["ids"], torch.tensor([[0, 1, 2], [1, 0, 2]]))
    assert torch.equal(captured["planned_ids"], captured["ids"])
    torch.testing.assert_close(captured["weights"], torch.tensor([[0.7, 0.3, 1.0], [0.4, 0.6, 1.0]]))
    assert captured["kwargs"]["global_num_experts"] == -1


def _synthetic_probe(kind, bucket, tiles, seed, hidden, inter, experts):
    # pretend the best tile is the smallest one that holds the bucket
    return {t: (1.0 if t >= bucket else 5.0) + t * 1e-3 for t in tiles}


def test_quick_calibration_writes_atomically_and_refuses_overwrite(tmp_path):
    output = tmp_path / "profile.json"
    messages = []
    result = moe.calibrate_moe_planner_quick(None, output=output, machine_id="test-gpu", report=messages.append,
                                             _probe=_synthetic_probe)
    assert output.exists() and result.output_path == output and messages
    assert not [p for p in tmp_path.iterdir() if p.name.endswith(".tmp")]
    loaded = planner_runtime.GpuTileCalibration.from_json(output.read_text())
    assert loaded.machine_id == "test-gpu" and loaded.lookup("int8", 8) == (16, 16) and loaded.lookup("bf16", 100) == (256, 256)
    with pytest.raises(FileExistsError, match="already exists"):
        moe.calibrate_moe_planner_quick(None, output=output, _probe=_synthetic_probe)
    moe.calibrate_moe_planner_quick(None, output=output, overwrite=True, _probe=_synthetic_probe)


def test_enable_quick_installs_only_after_success(monkeypatch, tmp_path):
    order = []
    real_calibrate = planner_runtime.calibrate_moe_planner_quick

    def calibrate(*args, **kwargs):
        order.append("calibrate")
        return real_calibrate(*args, _probe=_synthetic_probe, **kwargs)

    monkeypatch.setattr(planner_runtime, "calibrate_moe_planner_quick", calibrate)
    previous = moe.set_default_moe_planner_runtime(None)
    try:
        runtime = planner_runtime.enable_moe_planner_quick(hidden_size=64, intermediate_size=32, global_experts=4, local_experts=4,
                                                           output=tmp_path / "p.json")
        assert order == ["calibrate"] and moe.get_default_moe_planner_runtime() is runtime
        moe.set_default_moe_planner_runtime(None)
        monkeypatch.setattr(planner_runtime, "MoePlannerRuntime", lambda *a, **k: (_ for _ in ()).throw(ValueError("boom")))
        with pytest.raises(ValueError, match="boom"):
            planner_runtime.enable_moe_planner_quick(hidden_size=64, intermediate_size=32, global_experts=4, local_experts=4)
        assert moe.get_default_moe_planner_runtime() is None
    finally:
        moe.set_default_moe_planner_runtime(previous)


def test_runtime_plans_from_shapes_only():
    calibration = planner_runtime.GpuTileCalibration(machine_id="m", gpu_name="g", sm_count=148,
                                                     tiles={"int8": {8: (16, 16), 96: (128, 64)}})
    runtime = moe.MoePlannerRuntime(calibration, hidden_size=16, intermediate_size=16, global_experts=4, local_experts=4)
    weights = _w8a8_weights(experts=4)

    class NoHostRead(torch.Tensor):
        pass

    ids = torch.zeros((4, 2), dtype=torch.int64, device="meta")  # a meta tensor cannot be read on the host
    plan = runtime.plan_for_dispatch(weights, ids, num_threads=1, activation="silu", global_num_experts=-1)
    assert plan.task_w13_window_tiles.tolist() == [16] and runtime.last_plan["rows_per_expert"] == 2
    big = torch.zeros((160, 2), dtype=torch.int64, device="meta")
    plan = runtime.plan_for_dispatch(weights, big, num_threads=1, activation="silu", global_num_experts=-1)
    assert (plan.task_w13_window_tiles.tolist(), plan.task_w2_window_tiles.tolist()) == ([128], [64])
    assert runtime.plan_for_dispatch(_w8a8_weights(experts=3), ids, num_threads=1, activation="silu", global_num_experts=-1) is None
    assert runtime.plan_for_dispatch(weights, ids, num_threads=1, activation="gelu", global_num_experts=-1) is None
    with pytest.raises(TypeError):
        moe.set_default_moe_planner_runtime(object())


def test_naive_matches_explicit_loop():
    generator = torch.Generator().manual_seed(5)
    x = torch.randn((6, 16), generator=generator)
    w13 = torch.randn((3, 8, 16), generator=generator)
    w2 = torch.randn((3, 16, 4), generator=generator)
    ids = torch.tensor([[0, 2], [1, 0], [2, 1], [0, 1], [2, 0], [1, 2]])
    w = torch.softmax(torch.randn((6, 2), generator=generator), -1)
    expected = torch.zeros((6, 16))
    for t in range(6):
        for s in range(2):
            e = int(ids[t, s])
            gate_up = w13[e] @ x[t]
            mid = torch.nn.functional.silu(gate_up[:4]) * gate_up[4:]
            expected[t] += w[t, s] * (w2[e] @ mid)
    torch.testing.assert_close(moe.fused_moe_naive(x, w13, w2, w, ids), expected, rtol=1e-5, atol=1e-5)


def test_router_and_projection_helpers_have_no_cpu_path():
    """The router front-end and the dense projection helpers import without a GPU and refuse CPU tensors loudly."""
    from fused_cpp_b200 import deepseek_v4_w8a8, router

    with pytest.raises(ValueError, match="CUDA tensor"):
        router.router_topk(torch.zeros((2, 8)), 2)
    with pytest.raises(ValueError, match="scoring"):
        router.router_topk(torch.zeros((2, 8)), 2, scoring="tanh")
    weight = deepseek_v4_w8a8.PreparedDeepSeekV4W8A8LinearWeight.__new__(deepseek_v4_w8a8.PreparedDeepSeekV4W8A8LinearWeight)
    with pytest.raises(TypeError, match="CUDA torch.bfloat16"):
        deepseek_v4_w8a8.deepseek_v4_w8a8_linear(torch.zeros((2, 8), dtype=torch.bfloat16), weight)
    assert set(deepseek_v4_w8a8.__all__) == {
        "PreparedDeepSeekV4W8A8LinearWeight", "_HAS_DEEPSEEK_V4_W8A8", "deepseek_v4_w8a8_linear", "deepseek_v4_w8a8_linear_pair",
        "deepseek_v4_wo_b_w8a8", "prepare_deepseek_v4_w8a8_linear_quantized_weight", "prepare_deepseek_v4_w8a8_linear_weight"}
