"""Generate the golden fixtures in this directory from the REFERENCE's own Python functions.

Run in a container that has the reference checkout:

    REFERENCE_ROOT=/path/to/fused_cpp python tests/golden/make_golden.py

It imports, unmodified,
  * tests/test_moe_w8a8.py::_quantize_row and ::_reference   (the W8A8 per-token reference), and
  * src/fused_cpp/moe/naive.py::fused_moe_naive               (the BF16 reference, also with biases, gelu and swigluoai),
  * tests/test_i8gemm.py::_reference_dynamic_scaled_mm        (the dense W8A8 linear reference),
runs them on seeded inputs from fused_cpp_b200.synthetic (plus the input recipe of the reference's
own W8A8 test), and stores ONLY their outputs (inputs are regenerated from the seeds by the tests).
The reference cannot travel to the GPU machine; these files can.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)

from fused_cpp_b200 import synthetic  # noqa: E402
from tests import cases  # noqa: E402


def _load_reference():
    root = os.environ.get("REFERENCE_ROOT", "/root/reference")
    sys.path.insert(0, os.path.join(root, "src"))
    sys.path.insert(0, root)
    spec = importlib.util.spec_from_file_location("ref_test_moe_w8a8", os.path.join(root, "tests", "test_moe_w8a8.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    from fused_cpp.moe.naive import fused_moe_naive
    spec = importlib.util.spec_from_file_location("ref_test_i8gemm", os.path.join(root, "tests", "test_i8gemm.py"))
    dense = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(dense)
    return module._quantize_row, module._reference, fused_moe_naive, dense._reference_dynamic_scaled_mm


def main() -> None:
    quantize_row, reference, fused_moe_naive, dense_reference = _load_reference()
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    for name in cases.W8A8_CASES:
        case = cases.w8a8_case(name)
        rows = [quantize_row(case["x"][t]) for t in range(case["x"].shape[0])]
        golden = {
            "xq": torch.stack([r[0] for r in rows]).to(torch.int8),
            "a": torch.tensor([r[1] for r in rows], dtype=torch.float64),
            "out": reference(case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"],
                             case["topk_ids"]),
        }
        torch.save(golden, os.path.join(HERE, f"w8a8_{name}.pt"))
        print("w8a8", name, tuple(golden["out"].shape))
    for name in cases.BF16_CASES:
        case = cases.bf16_case(name)
        out = fused_moe_naive(case["x"].float(), case["w13"].float(), case["w2"].float(), case["topk_weights"],
                              case["topk_ids"]).to(torch.bfloat16)
        torch.save({"out": out}, os.path.join(HERE, f"bf16_{name}.pt"))
        print("bf16", name, tuple(out.shape))


    # BF16 op variants: biases, gelu, swigluoai through the same fused_moe_naive
    for name in cases.BF16_VARIANTS:
        case = cases.bf16_variant_case(name)
        bias13 = None if case["w13_bias"] is None else case["w13_bias"].float()
        bias2 = None if case["w2_bias"] is None else case["w2_bias"].float()
        out = fused_moe_naive(case["x"].float(), case["w13"].float(), case["w2"].float(), case["topk_weights"], case["topk_ids"],
                              w13_bias=bias13, w2_bias=bias2, activation=case["activation"]).to(torch.bfloat16)
        torch.save({"out": out}, os.path.join(HERE, f"bf16_variant_{name}.pt"))
        print("bf16 variant", name, tuple(out.shape))

    # W8A16: fused_moe_naive on the dequantised weights (q * scale in fp32) of the W8A8 cases
    for name in cases.W8A16_CASES:
        case = cases.w8a8_case(name)
        w13 = case["w13"].float() * case["s13"].reshape(case["w13"].shape[0], -1, 1)
        w2 = case["w2"].float() * case["s2"].reshape(case["w2"].shape[0], -1, 1)
        out = fused_moe_naive(case["x"].float(), w13, w2, case["topk_weights"], case["topk_ids"]).to(torch.bfloat16)
        torch.save({"out": out}, os.path.join(HERE, f"w8a16_{name}.pt"))
        print("w8a16", name, tuple(out.shape))

    # appended: dense W8A8 linear, tests/test_i8gemm.py::_reference_dynamic_scaled_mm of the reference
    for name in cases.I8GEMM_CASES:
        case = cases.i8gemm_case(name)
        out = dense_reference(case["x"], case["weight"], case["weight_scale"], bias=case["bias"], out_dtype=case["out_dtype"])
        torch.save({"out": out}, os.path.join(HERE, f"i8gemm_{name}.pt"))
        print("i8gemm", name, tuple(out.shape))


if __name__ == "__main__":
    main()
