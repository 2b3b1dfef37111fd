"""Dense W8A8 linear with dynamic per-row activation quantisation: the surface of the reference's
`fused_cpp.i8gemm` (src/fused_cpp/i8gemm.py:41-199) on the B200 tensor cores.

    packed = i8gemm.prepare(weight_int8, weight_scale)
    out = i8gemm.dynamic_scaled_mm(x_cuda, packed, bias=None, out_dtype=torch.bfloat16)

Arithmetic follows the reference's scalar statement (csrc/i8gemm.cpp:384-399, :147-165): scale =
amax/127 (1 for a zero row), q = clamp(nearbyint(x/scale), -128, 127), out = (acc * x_scale) * w_scale
(+ bias); int32 accumulation is exact on tcgen05 `kind::i8`.  The packed weight on this backend is the
[N, K] matrix zero-padded to K % 16 == 0 and resident on the GPU.  `nthreads` is accepted and ignored.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

BACKEND = "cuda_sm100_tcgen05"
_supports_i8gemm = _lib.device_supported()


def _require_backend() -> None:
    if not _lib.device_supported():
        raise RuntimeError("i8gemm backend unavailable: no compute-capability-10.x CUDA device (there is no CPU path)")


@dataclass(frozen=True)
class PreparedI8GEMMWeight:
    packed_weight: torch.Tensor
    weight_scale: torch.Tensor
    k: int
    n: int
    k_padded: int
    n_padded: int
    backend: str


def i8gemm_prepare(weight: torch.Tensor, weight_scale: torch.Tensor, backend: str = "auto"):
    """-> (packed[N, Kp] int8 on the GPU, scale_f32[N], K, N, Kp, Np, backend); csrc/i8gemm.cpp:280-316."""
    if backend not in ("auto", BACKEND):
        raise RuntimeError(f"i8gemm.prepare: unknown backend {backend!r}; available: {BACKEND}")
    n, k = int(weight.shape[0]), int(weight.shape[1])
    if n <= 0 or k <= 0:
        raise RuntimeError(f"i8gemm.prepare: N and K must be positive, got N={n} K={k}")
    device = torch.device("cuda", torch.cuda.current_device())
    k_padded = max(16, (k + 15) // 16 * 16)
    packed = torch.zeros((n, k_padded), dtype=torch.int8, device=device)
    packed[:, :k] = weight.to(device)
    scale = weight_scale.to(device=device, dtype=torch.float32).reshape(-1)
    if scale.numel() == 1:
        scale = scale.expand(n)
    return packed, scale.contiguous(), k, n, k_padded, n, BACKEND


def _workspace(rows: int, k: int, n: int, device: torch.device) -> torch.Tensor:
    return _lib.get_workspace(int(_lib.load().fmoe_i8gemm_workspace_bytes(rows, k, n)), device)


def i8gemm_dynamic_scaled_mm(output, input, packed_weight, weight_scale, bias, K, N, Kp, Np, nthreads=0) -> None:
    """Writes `output` in place (csrc/module.cpp:220-233 op; csrc/i8gemm.cpp:318)."""
    if input.dim() != 2 or input.device.type != "cuda" or not input.is_contiguous():
        raise RuntimeError("i8gemm.dynamic_scaled_mm: input must be a contiguous 2D CUDA tensor [M, K]")
    if input.dtype not in (torch.float32, torch.bfloat16) or output.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("i8gemm.dynamic_scaled_mm: input/output dtype must be float32/bfloat16")
    rows = int(input.shape[0])
    if int(input.shape[1]) != K or tuple(output.shape) != (rows, N) or tuple(packed_weight.shape) != (N, Kp):
        raise RuntimeError("i8gemm.dynamic_scaled_mm: shape mismatch")
    bias_f32 = None if bias is None else bias.to(device=input.device, dtype=torch.float32).contiguous()
    workspace = _workspace(rows, K, N, input.device)
    _lib.check(_lib.load().fmoe_i8gemm_dynamic_scaled_mm(
        _lib._ptr(input), 1 if input.dtype == torch.bfloat16 else 0, rows, K, _lib._ptr(packed_weight), _lib._ptr(weight_scale),
        _lib._ptr(bias_f32), N, _lib._ptr(output), 1 if output.dtype == torch.bfloat16 else 0, _lib._ptr(workspace),
        workspace.numel(), _lib._stream()))


def i8gemm_dynamic_scaled_mm_pair(first_output, second_output, input, first_packed_weight, first_weight_scale, K, first_N, Kp,
                                  first_Np, second_packed_weight, second_weight_scale, second_N, second_Np, nthreads=0) -> None:
    """Two bf16 GEMMs sharing one activation quantisation (csrc/i8gemm.cpp:454)."""
    rows = int(input.shape[0])
    workspace = _workspace(rows, K, max(first_N, second_N), input.device)
    _lib.check(_lib.load().fmoe_i8gemm_dynamic_scaled_mm_pair(
        _lib._ptr(input), rows, K, _lib._ptr(first_packed_weight), _lib._ptr(first_weight_scale), first_N, _lib._ptr(first_output),
        _lib._ptr(second_packed_weight), _lib._ptr(second_weight_scale), second_N, _lib._ptr(second_output), _lib._ptr(workspace),
        workspace.numel(), _lib._stream()))


def prepare(weight_int8: torch.Tensor, weight_scale: torch.Tensor, *, backend: str = "auto") -> PreparedI8GEMMWeight:
    """Prepare an int8 [N, K] linear weight for repeated GEMMs."""
    _require_backend()
    if weight_int8.dim() != 2:
        raise RuntimeError(f"i8gemm.prepare: weight_int8 must be 2D [N, K], got {weight_int8.dim()}D")
    if weight_int8.dtype != torch.int8:
        raise RuntimeError(f"i8gemm.prepare: weight_int8 dtype must be torch.int8, got {weight_int8.dtype}")
    if weight_scale.numel() not in (1, int(weight_int8.shape[0])):
        raise RuntimeError("i8gemm.prepare: weight_scale must be scalar or shape [N]")
    packed, scale, k, n, k_padded, n_padded, selected = i8gemm_prepare(weight_int8.contiguous(), weight_scale.contiguous(), str(backend))
    return PreparedI8GEMMWeight(packed, scale, int(k), int(n), int(k_padded), int(n_padded), str(selected))


def dynamic_scaled_mm(x: torch.Tensor, packed: PreparedI8GEMMWeight, *, bias: Optional[torch.Tensor] = None,
                      out_dtype: torch.dtype = torch.bfloat16, nthreads: int = 0) -> torch.Tensor:
    """x @ weight.T with dynamic per-row int8 quantisation; returns float32 or bfloat16."""
    _require_backend()
    if not isinstance(packed, PreparedI8GEMMWeight):
        raise RuntimeError("i8gemm.dynamic_scaled_mm: packed must come from i8gemm.prepare")
    if x.shape[-1] != packed.k:
        raise RuntimeError(f"i8gemm.dynamic_scaled_mm: x last dim must be K={packed.k}, got {x.shape[-1]}")
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError(f"i8gemm.dynamic_scaled_mm: x dtype must be float32/bfloat16, got {x.dtype}")
    if out_dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError(f"i8gemm.dynamic_scaled_mm: out_dtype must be float32/bfloat16, got {out_dtype}")
    if bias is not None and (bias.dim() != 1 or int(bias.shape[0]) != packed.n):
        raise RuntimeError(f"i8gemm.dynamic_scaled_mm: bias must be shape [{packed.n}]")
    out_shape = (*tuple(x.shape[:-1]), packed.n)
    if x.numel() == 0:
        return torch.empty(out_shape, dtype=out_dtype, device=x.device)
    x_2d = x.contiguous().reshape(-1, packed.k)
    out_2d = torch.empty((x_2d.shape[0], packed.n), dtype=out_dtype, device=x.device)
    i8gemm_dynamic_scaled_mm(out_2d, x_2d, packed.packed_weight, packed.weight_scale, bias, packed.k, packed.n, packed.k_padded,
                             packed.n_padded, int(nthreads))
    return out_2d.reshape(out_shape)


mm = dynamic_scaled_mm


def dynamic_scaled_mm_pair(x: torch.Tensor, first: PreparedI8GEMMWeight, second: PreparedI8GEMMWeight, *, nthreads: int = 0):
    """Two BF16-output GEMMs sharing the dynamic per-row activation quantisation."""
    _require_backend()
    if not isinstance(first, PreparedI8GEMMWeight) or not isinstance(second, PreparedI8GEMMWeight):
        raise TypeError("first and second must be PreparedI8GEMMWeight")
    if x.device.type != "cuda" or x.dtype != torch.bfloat16 or x.dim() != 2:
        raise TypeError("i8gemm.dynamic_scaled_mm_pair input must be CUDA BF16 [M, K]")
    if first.k != second.k or first.k_padded != second.k_padded or x.shape[1] != first.k:
        raise ValueError("paired i8gemm weights and input must share K and Kp")
    if int(nthreads) < 0:
        raise ValueError("nthreads must be non-negative; zero selects the backend default")
    x = x.contiguous()
    first_output = torch.empty((x.shape[0], first.n), dtype=torch.bfloat16, device=x.device)
    second_output = torch.empty((x.shape[0], second.n), dtype=torch.bfloat16, device=x.device)
    i8gemm_dynamic_scaled_mm_pair(first_output, second_output, x, first.packed_weight, first.weight_scale, first.k, first.n,
                                  first.k_padded, first.n_padded, second.packed_weight, second.weight_scale, second.n,
                                  second.n_padded, int(nthreads))
    return first_output, second_output


__all__ = ["PreparedI8GEMMWeight", "_supports_i8gemm", "dynamic_scaled_mm", "dynamic_scaled_mm_pair", "mm", "prepare"]
