"""The repurposed planner entry points on the GPU: enable_moe_planner_quick really times the row tiles of the
grouped GEMMs on a probe layer of the caller's shape (uniform and skewed routing), writes the JSON profile,
refuses to overwrite it, installs the runtime, and fused_moe_tiled then runs under the tiles the table holds and
reports them through runtime.last_plan.  Reference behaviour kept: install-after-success ordering and file
semantics of src/fused_cpp/moe/planner_runtime.py:348-391 and
cpu_moe_schedule_optimization/cost_model/quick_calibration.py:343-426.
"""
from __future__ import annotations

import json

import pytest
import torch

from fused_cpp_b200 import moe, synthetic
from fused_cpp_b200.moe import planner_runtime
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_enable_quick_calibrates_on_the_gpu_and_the_forward_uses_the_table(cuda_device, tmp_path):
    shape = synthetic.CONFIG_SMALL_W8A8  # T=16, H=2048, I=1024, E=16, top-4
    output = tmp_path / "tiles.json"
    messages = []
    previous = moe.set_default_moe_planner_runtime(None)
    try:
        runtime = moe.enable_moe_planner_quick(hidden_size=shape.hidden, intermediate_size=shape.inter, global_experts=shape.experts,
                                               local_experts=shape.experts, output=output, report=messages.append)
        assert moe.get_default_moe_planner_runtime() is runtime
        profile = json.loads(output.read_text())
        buckets = {str(b) for b in planner_runtime.CALIBRATION_BUCKETS}
        for kind in ("int8", "bf16"):
            assert set(profile["tiles"][kind]) == buckets
            for bucket, timings in profile["timings_ms"][kind].items():
                assert set(int(t) for t in timings) == set(planner_runtime.CANDIDATE_TILES)
                assert all(v > 0.0 for v in timings.values()), (kind, bucket, timings)
                chosen = profile["tiles"][kind][bucket][0]
                assert timings[str(chosen)] <= 1.05 * min(timings.values()) + 1e-9
        assert profile["gpu_name"] == torch.cuda.get_device_name() and profile["sm_count"] > 0
        assert len(messages) == 2 * len(buckets) and all(f"H={shape.hidden} I={shape.inter}" in m for m in messages)
        with pytest.raises(FileExistsError, match="already exists"):
            moe.enable_moe_planner_quick(hidden_size=shape.hidden, intermediate_size=shape.inter, global_experts=shape.experts,
                                         local_experts=shape.experts, output=output)

        # A forward through the public op under the installed runtime: the tiles it ran with are the table's entry
        # for this batch's rows per expert, and the result is still the oracle's, bit for bit.
        case = synthetic.make_w8a8_case(shape, seed=synthetic.SEED_BASE)
        prepared = moe.prepare_fused_moe_w8a8_tiled_quantized_weights(case["w13"], case["s13"], case["w2"], case["s2"])
        out = moe.fused_moe_tiled(case["x"].to(cuda_device), prepared, case["topk_weights"].to(cuda_device),
                                  case["topk_ids"].to(cuda_device), swiglu_limit=10.0)
        plan = runtime.last_plan
        rows_per_expert = -(-shape.tokens * shape.top_k // shape.experts)
        assert plan["kind"] == "int8" and plan["rows_per_expert"] == rows_per_expert and plan["calibrated"] is True
        assert (plan["gate_up_tile"], plan["down_tile"]) == runtime.calibration.lookup("int8", rows_per_expert)
        expected = oracle.w8a8_forward(case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"], case["topk_ids"])
        assert torch.equal(out.cpu().view(torch.int16), expected.view(torch.int16))
    finally:
        moe.set_default_moe_planner_runtime(previous)
