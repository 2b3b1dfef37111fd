"""Import alias for callers written against the reference's package name.

vLLM's DeepSeek-V4 adapter and the reference's own Python planner do `import fused_cpp.moe`,
`from fused_cpp.moe.bf16_tiled import ...`, `importlib.import_module("fused_cpp._moe_C")` and
`from fused_cpp._C import i8gemm_prepare` (src/fused_cpp/__init__.py, src/fused_cpp/i8gemm.py:21-33,
cpu_moe_schedule_optimization/planners/interval_planner.py:229-235).  With this directory on the path
those imports resolve to the modules of `fused_cpp_b200`: the same module objects under a second name,
so monkeypatching or reading state through either name sees the other.

Only the routed-expert MoE path, the dense W8A8 linear and the DeepSeek-V4 W8A8 projection wrappers exist
in this build; the reference's sibling operators (bf16_linear, sparse_mla, mHC, ...) are not aliased and
importing them raises ImportError as on any build that lacks them.
"""
import sys as _sys

import fused_cpp_b200 as _impl
from fused_cpp_b200 import deepseek_v4_w8a8, i8gemm, moe  # noqa: F401
from fused_cpp_b200.moe import _moe_C, bf16_tiled, naive, plan, planner_runtime  # noqa: F401

__version__ = _impl.__version__

_sys.modules[__name__ + ".moe"] = moe
_sys.modules[__name__ + ".moe.bf16_tiled"] = bf16_tiled
_sys.modules[__name__ + ".moe.naive"] = naive
_sys.modules[__name__ + ".moe.plan"] = plan
_sys.modules[__name__ + ".moe.planner_runtime"] = planner_runtime
_sys.modules[__name__ + ".i8gemm"] = i8gemm
_sys.modules[__name__ + ".deepseek_v4_w8a8"] = deepseek_v4_w8a8
# The two native extension modules of the reference: the MoE op table, and the module that holds the i8gemm ops.
_sys.modules[__name__ + "._moe_C"] = _moe_C
_sys.modules[__name__ + "._C"] = i8gemm
_C = i8gemm

__all__ = ["deepseek_v4_w8a8", "i8gemm", "moe"]
