"""Explicit W8A8 linear selection for the DeepSeek-V4 attention projections: the surface of the reference's
`fused_cpp.deepseek_v4_w8a8` (src/fused_cpp/deepseek_v4_w8a8.py:29-160) on the GPU path.

These are the callers next to the dense `i8gemm`: a bf16 [N, K] projection weight is quantised per output channel
once (scale = amax / 127, 1 for a zero row; round-half-even of w / scale clamped to +-127, `:43-53`), then every
call fuses dynamic per-row activation quantisation, the int8 GEMM, channel dequantisation and the bf16 store;
`deepseek_v4_w8a8_linear_pair` runs the main and the indexer Q projection on one shared activation quantisation.
Same names, argument meaning and error types as the reference; tensors live on the GPU and `num_threads` is
accepted and ignored.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib, i8gemm

_HAS_DEEPSEEK_V4_W8A8 = _lib.device_supported()


@dataclass(frozen=True)
class PreparedDeepSeekV4W8A8LinearWeight:
    """Opaque per-output-channel W8 weight for dynamic per-row A8 GEMM."""

    packed: i8gemm.PreparedI8GEMMWeight

    @property
    def k(self) -> int:
        return self.packed.k

    @property
    def n(self) -> int:
        return self.packed.n


def _quantize_weight_per_output_channel(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    if weight.dtype != torch.bfloat16:
        raise TypeError("DeepSeek V4 W8A8 source weight must be a torch.bfloat16 tensor")
    if weight.dim() != 2:
        raise ValueError(f"DeepSeek V4 W8A8 source weight must be [N, K], got {tuple(weight.shape)}")
    device = torch.device("cuda", torch.cuda.current_device())
    rows, cols = weight.shape
    padded = (cols + 15) // 16 * 16  # the row quantiser works on 16-column vectors; zero columns change nothing
    source = weight.to(device)
    if padded != cols:
        source = torch.nn.functional.pad(source, (0, padded - cols))
    quantized, scale = _lib.quantize_rows(source.contiguous(), weight_mode=True)
    return quantized[:, :cols].contiguous(), scale.contiguous()


def prepare_deepseek_v4_w8a8_linear_weight(weight: torch.Tensor, *, backend: str = "auto") -> PreparedDeepSeekV4W8A8LinearWeight:
    """Quantize one BF16 ``[N, K]`` attention weight (CPU or CUDA) and keep it on the GPU."""
    quantized, scale = _quantize_weight_per_output_channel(weight)
    return prepare_deepseek_v4_w8a8_linear_quantized_weight(quantized, scale, backend=backend)


def prepare_deepseek_v4_w8a8_linear_quantized_weight(weight: torch.Tensor, scale: torch.Tensor, *,
                                                     backend: str = "auto") -> PreparedDeepSeekV4W8A8LinearWeight:
    """Take a checkpoint INT8 ``[N, K]`` weight with FP32 channel scales."""
    if weight.dtype != torch.int8 or weight.dim() != 2:
        raise TypeError("DeepSeek V4 quantized weight must be a torch.int8 [N, K] tensor")
    if scale.dtype != torch.float32:
        raise TypeError("DeepSeek V4 W8 scale must be a torch.float32 tensor")
    if scale.numel() != weight.shape[0]:
        raise ValueError(f"DeepSeek V4 W8 scale must contain N={weight.shape[0]} values")
    if backend == "sve":  # the reference's default backend name; there is one backend here
        backend = "auto"
    return PreparedDeepSeekV4W8A8LinearWeight(packed=i8gemm.prepare(weight.contiguous(), scale.reshape(-1).contiguous(), backend=backend))


def deepseek_v4_w8a8_linear(input: torch.Tensor, weight: PreparedDeepSeekV4W8A8LinearWeight, *, num_threads: int = 0,
                            out: torch.Tensor | None = None) -> torch.Tensor:
    """Fuse dynamic A8 quantization, the int8 GEMM, channel dequant, and BF16 store."""
    if not isinstance(weight, PreparedDeepSeekV4W8A8LinearWeight):
        raise TypeError("weight must be PreparedDeepSeekV4W8A8LinearWeight")
    if input.device.type != "cuda" or input.dtype != torch.bfloat16:
        raise TypeError("DeepSeek V4 W8A8 input must be a CUDA torch.bfloat16 tensor")
    if input.shape[-1] != weight.k:
        raise ValueError(f"DeepSeek V4 W8A8 input K must be {weight.k}, got {input.shape[-1]}")
    if int(num_threads) < 0:
        raise ValueError("num_threads must be non-negative; zero selects the backend default")
    result = i8gemm.dynamic_scaled_mm(input, weight.packed, out_dtype=torch.bfloat16, nthreads=int(num_threads))
    if out is None:
        return result
    if out.device != result.device or out.dtype != result.dtype or out.shape != result.shape or not out.is_contiguous():
        raise ValueError("out must be contiguous CUDA BF16 with shape [*, N]")
    out.copy_(result)
    return out


def deepseek_v4_w8a8_linear_pair(input: torch.Tensor, first: PreparedDeepSeekV4W8A8LinearWeight,
                                 second: PreparedDeepSeekV4W8A8LinearWeight, *, num_threads: int = 0):
    """Run main/indexer Q projections with one shared activation quantization."""
    if not isinstance(first, PreparedDeepSeekV4W8A8LinearWeight) or not isinstance(second, PreparedDeepSeekV4W8A8LinearWeight):
        raise TypeError("paired weights must be PreparedDeepSeekV4W8A8LinearWeight")
    if input.device.type != "cuda" or input.dtype != torch.bfloat16 or input.dim() != 2:
        raise TypeError("DeepSeek V4 paired W8A8 input must be CUDA BF16 [M, K]")
    if first.k != second.k or input.shape[1] != first.k:
        raise ValueError("paired W8A8 weights and input must share K")
    if int(num_threads) < 0:
        raise ValueError("num_threads must be non-negative; zero selects the backend default")
    return i8gemm.dynamic_scaled_mm_pair(input, first.packed, second.packed, nthreads=int(num_threads))


def deepseek_v4_wo_b_w8a8(input: torch.Tensor, weight: PreparedDeepSeekV4W8A8LinearWeight, *, num_threads: int = 0,
                          out: torch.Tensor | None = None) -> torch.Tensor:
    """Run the TP-local ``attn.wo_b`` projection; collective reduction stays external."""
    return deepseek_v4_w8a8_linear(input, weight, num_threads=num_threads, out=out)


__all__ = [
    "PreparedDeepSeekV4W8A8LinearWeight",
    "_HAS_DEEPSEEK_V4_W8A8",
    "deepseek_v4_w8a8_linear",
    "deepseek_v4_w8a8_linear_pair",
    "deepseek_v4_wo_b_w8a8",
    "prepare_deepseek_v4_w8a8_linear_quantized_weight",
    "prepare_deepseek_v4_w8a8_linear_weight",
]
