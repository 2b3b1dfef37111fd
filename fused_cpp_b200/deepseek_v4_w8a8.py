"""W8A8 attention projections of DeepSeek-V4 on the GPU: the callers that sit next to the dense `i8gemm`.

An adaptation of the reference's `fused_cpp.deepseek_v4_w8a8` (src/fused_cpp/deepseek_v4_w8a8.py:29-160), which is
itself a thin validation layer over `i8gemm`; the public names, argument meaning and exception types are kept so that
its callers need no change, everything behind them is this package's.

What the functions do.  A bf16 projection weight [N, K] becomes int8 once, per output channel (scale = amax / 127, or 1
for an all-zero row; q = round-half-even(w / scale) clamped to +-127, `:43-53` of the reference) -- here on the GPU by
the library's row quantiser.  Every forward call then quantises the activation rows dynamically, multiplies on the int8
tensor cores, applies row scale x channel scale and stores bf16, in one C-ABI call
(fmoe_i8gemm_dynamic_scaled_mm).  The paired form runs the main and the indexer Q projection over ONE activation
quantisation (fmoe_i8gemm_dynamic_scaled_mm_pair).  Tensors live on the GPU; `num_threads` is validated and unused.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib, i8gemm

_HAS_DEEPSEEK_V4_W8A8 = _lib.device_supported()
_QUANTISER_COLUMN_QUANTUM = 16  # the row quantiser reads 16-column vectors


@dataclass(frozen=True)
class PreparedDeepSeekV4W8A8LinearWeight:
    """GPU-resident int8 [N, K] projection weight with its fp32 channel scales (opaque to callers)."""

    packed: i8gemm.PreparedI8GEMMWeight

    @property
    def k(self) -> int:
        return self.packed.k

    @property
    def n(self) -> int:
        return self.packed.n


def _check_threads(num_threads) -> int:
    threads = int(num_threads)
    if threads < 0:
        raise ValueError("num_threads must be non-negative; zero selects the backend default")
    return threads


def _check_prepared(*weights) -> None:
    if not all(isinstance(w, PreparedDeepSeekV4W8A8LinearWeight) for w in weights):
        raise TypeError("weight must be PreparedDeepSeekV4W8A8LinearWeight" if len(weights) == 1
                        else "paired weights must be PreparedDeepSeekV4W8A8LinearWeight")


def _is_cuda_bf16(tensor: torch.Tensor) -> bool:
    return tensor.device.type == "cuda" and tensor.dtype == torch.bfloat16


def _quantize_weight_per_output_channel(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 [N, K] -> (int8 [N, K], fp32 scale [N]) with the library's weight quantiser.  K is padded with zero columns
    to the quantiser's vector width first; zeros change neither the row maximum nor any quantised value."""
    if weight.dtype != torch.bfloat16:
        raise TypeError("DeepSeek V4 W8A8 source weight must be a torch.bfloat16 tensor")
    if weight.dim() != 2:
        raise ValueError(f"DeepSeek V4 W8A8 source weight must be [N, K], got {tuple(weight.shape)}")
    columns = int(weight.shape[1])
    on_gpu = weight.to(torch.device("cuda", torch.cuda.current_device()))
    tail = -columns % _QUANTISER_COLUMN_QUANTUM
    if tail:
        on_gpu = torch.nn.functional.pad(on_gpu, (0, tail))
    quantised, scale = _lib.quantize_rows(on_gpu.contiguous(), weight_mode=True)
    return quantised[:, :columns].contiguous(), scale.contiguous()


def prepare_deepseek_v4_w8a8_linear_quantized_weight(weight: torch.Tensor, scale: torch.Tensor, *,
                                                     backend: str = "auto") -> PreparedDeepSeekV4W8A8LinearWeight:
    """Checkpoint-native route: an int8 [N, K] weight and its N fp32 channel scales, kept as they are."""
    if weight.dtype != torch.int8 or weight.dim() != 2:
        raise TypeError("DeepSeek V4 quantized weight must be a torch.int8 [N, K] tensor")
    if scale.dtype != torch.float32:
        raise TypeError("DeepSeek V4 W8 scale must be a torch.float32 tensor")
    channels = int(weight.shape[0])
    if scale.numel() != channels:
        raise ValueError(f"DeepSeek V4 W8 scale must contain N={channels} values")
    # "sve" is the reference's name for its only production backend; callers that pass it get this build's only one.
    selected = "auto" if backend == "sve" else backend
    return PreparedDeepSeekV4W8A8LinearWeight(packed=i8gemm.prepare(weight.contiguous(), scale.reshape(-1).contiguous(), backend=selected))


def prepare_deepseek_v4_w8a8_linear_weight(weight: torch.Tensor, *, backend: str = "auto") -> PreparedDeepSeekV4W8A8LinearWeight:
    """bf16 route: quantise [N, K] per output channel on the GPU, then as the checkpoint-native route."""
    quantised, scale = _quantize_weight_per_output_channel(weight)
    return prepare_deepseek_v4_w8a8_linear_quantized_weight(quantised, scale, backend=backend)


def deepseek_v4_w8a8_linear(input: torch.Tensor, weight: PreparedDeepSeekV4W8A8LinearWeight, *, num_threads: int = 0,
                            out: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 [*, K] x prepared [N, K]^T -> bf16 [*, N]; with `out`, the result is written there and `out` returned."""
    _check_prepared(weight)
    if not _is_cuda_bf16(input):
        raise TypeError("DeepSeek V4 W8A8 input must be a CUDA torch.bfloat16 tensor")
    if input.shape[-1] != weight.k:
        raise ValueError(f"DeepSeek V4 W8A8 input K must be {weight.k}, got {input.shape[-1]}")
    threads = _check_threads(num_threads)
    product = i8gemm.dynamic_scaled_mm(input, weight.packed, out_dtype=torch.bfloat16, nthreads=threads)
    if out is None:
        return product
    acceptable = (out.device == product.device and out.dtype == product.dtype and out.shape == product.shape and out.is_contiguous())
    if not acceptable:
        raise ValueError("out must be contiguous CUDA BF16 with shape [*, N]")
    return out.copy_(product)


def deepseek_v4_w8a8_linear_pair(input: torch.Tensor, first: PreparedDeepSeekV4W8A8LinearWeight,
                                 second: PreparedDeepSeekV4W8A8LinearWeight, *, num_threads: int = 0):
    """Two projections of the same rows (main Q and indexer Q) sharing the activation quantisation: (first, second)."""
    _check_prepared(first, second)
    if not _is_cuda_bf16(input) or input.dim() != 2:
        raise TypeError("DeepSeek V4 paired W8A8 input must be CUDA BF16 [M, K]")
    if first.k != second.k or input.shape[1] != first.k:
        raise ValueError("paired W8A8 weights and input must share K")
    return i8gemm.dynamic_scaled_mm_pair(input, first.packed, second.packed, nthreads=_check_threads(num_threads))


def deepseek_v4_wo_b_w8a8(input: torch.Tensor, weight: PreparedDeepSeekV4W8A8LinearWeight, *, num_threads: int = 0,
                          out: torch.Tensor | None = None) -> torch.Tensor:
    """The tensor-parallel-local `attn.wo_b` projection; the reduction across ranks stays with the caller."""
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
