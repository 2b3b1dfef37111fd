"""Checkpoint-format side of the prepared weights: compressed-tensors int8 expert tensors -> prepare_*.

The reference leaves this step to its caller: "for compressed-tensors checkpoints which already store symmetric
channel-wise INT8 expert weights, use prepare_fused_moe_w8a16_tiled_quantized_weights; pass raw INT8 W13 / W2 and
their FP32 per-output-channel scales directly" (docs/vllm_bf16_tiled_moe_integration.md:246-259).  What a
checkpoint actually holds is one tensor per expert and projection,

    <prefix>.<expert>.gate_proj.weight        int8  [F, H]        <prefix>.<expert>.gate_proj.weight_scale  [F, 1] or [F]
    <prefix>.<expert>.up_proj.weight          int8  [F, H]        <prefix>.<expert>.up_proj.weight_scale
    <prefix>.<expert>.down_proj.weight        int8  [H, F]        <prefix>.<expert>.down_proj.weight_scale  [H, 1] or [H]

(the channel-wise "pack-quantized"/"int-quantized" layout of compressed-tensors; scales in fp32, bf16 or fp16).  The
functions here stack them into the layouts prepare_* take -- w13 [E, 2F, H] with gate rows then up rows and
scales [E, 2F]; w2 [E, H, F] and scales [E, H] -- without ever materialising bf16 weights, and hand them to the
W8A16 or W8A8 preparation.  Tensors are taken from any mapping (a safetensors file handle's get_tensor works through
`lambda name: handle.get_tensor(name)` wrapped in a dict-like, a torch state dict does as it is).
"""
from __future__ import annotations

from typing import Callable, Mapping

import torch

PROJECTIONS = ("gate_proj", "up_proj", "down_proj")


def _fetch(source, name: str) -> torch.Tensor:
    tensor = source(name) if callable(source) else source[name]
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} is not a tensor")
    return tensor


def _channel_scale(source, name: str, channels: int) -> torch.Tensor:
    scale = _fetch(source, name).to(torch.float32).reshape(-1)
    if scale.numel() != channels:
        raise ValueError(f"{name} must hold one scale per output channel ({channels}), got {scale.numel()} values: "
                         "only channel-wise symmetric int8 is supported (no group or tensor-wise scales)")
    return scale


def _int8_weight(source, name: str) -> torch.Tensor:
    weight = _fetch(source, name)
    if weight.dtype != torch.int8 or weight.dim() != 2:
        raise TypeError(f"{name} must be a 2-D torch.int8 tensor, got {weight.dtype} {tuple(weight.shape)}")
    return weight


def stack_compressed_tensors_experts(source: Mapping[str, torch.Tensor] | Callable[[str], torch.Tensor], prefix: str, experts: int,
                                     *, first_expert: int = 0):
    """Stack the experts [first_expert, first_expert + experts) under `prefix` (e.g. "model.layers.3.mlp.experts").

    Returns (w13 int8 [E, 2F, H], w13_scale fp32 [E, 2F], w2 int8 [E, H, F], w2_scale fp32 [E, H])."""
    if experts <= 0:
        raise ValueError("experts must be positive")
    w13 = s13 = w2 = s2 = None
    for slot in range(experts):
        base = f"{prefix}.{first_expert + slot}"
        gate = _int8_weight(source, f"{base}.gate_proj.weight")
        up = _int8_weight(source, f"{base}.up_proj.weight")
        down = _int8_weight(source, f"{base}.down_proj.weight")
        inter, hidden = gate.shape
        if tuple(up.shape) != (inter, hidden) or tuple(down.shape) != (hidden, inter):
            raise ValueError(f"{base}: gate/up must be [F, H] and down [H, F], got {tuple(gate.shape)}, {tuple(up.shape)}, {tuple(down.shape)}")
        if w13 is None:
            w13 = torch.empty((experts, 2 * inter, hidden), dtype=torch.int8)
            s13 = torch.empty((experts, 2 * inter), dtype=torch.float32)
            w2 = torch.empty((experts, hidden, inter), dtype=torch.int8)
            s2 = torch.empty((experts, hidden), dtype=torch.float32)
        elif tuple(w13.shape[1:]) != (2 * inter, hidden):
            raise ValueError(f"{base}: expert shapes differ inside one layer")
        w13[slot, :inter].copy_(gate)
        w13[slot, inter:].copy_(up)
        s13[slot, :inter].copy_(_channel_scale(source, f"{base}.gate_proj.weight_scale", inter))
        s13[slot, inter:].copy_(_channel_scale(source, f"{base}.up_proj.weight_scale", inter))
        w2[slot].copy_(down)
        s2[slot].copy_(_channel_scale(source, f"{base}.down_proj.weight_scale", hidden))
    return w13, s13, w2, s2


def prepare_moe_from_compressed_tensors(source, prefix: str, experts: int, *, mode: str = "w8a16", first_expert: int = 0,
                                        shared_prefix: str | None = None):
    """Prepared weights for fused_moe_tiled straight from a compressed-tensors checkpoint.

    mode "w8a16" (the reference's route for these checkpoints) or "w8a8" (dynamic int8 activations on the same
    tensors).  shared_prefix (e.g. "model.layers.3.mlp.shared_experts") adds the always-active shared expert as
    expert id E and returns the routed + shared holder for fused_moe_*_with_shared."""
    from . import moe

    if mode not in ("w8a16", "w8a8"):
        raise ValueError("mode must be 'w8a16' or 'w8a8'")
    w13, s13, w2, s2 = stack_compressed_tensors_experts(source, prefix, experts, first_expert=first_expert)
    if shared_prefix is None:
        prepare = (moe.prepare_fused_moe_w8a16_tiled_quantized_weights if mode == "w8a16"
                   else moe.prepare_fused_moe_w8a8_tiled_quantized_weights)
        return prepare(w13, s13, w2, s2)

    class _Shared:  # the shared expert's tensors have no expert index: present them as expert 0 of their own prefix
        def __call__(self, name: str):
            return _fetch(source, name.replace(f"{shared_prefix}.0.", f"{shared_prefix}.", 1))

    sw13, ss13, sw2, ss2 = stack_compressed_tensors_experts(_Shared(), shared_prefix, 1)
    prepare = (moe.prepare_routed_shared_moe_w8a16_tiled_quantized_weights if mode == "w8a16"
               else moe.prepare_routed_shared_moe_w8a8_tiled_quantized_weights)
    return prepare(w13, s13, w2, s2, sw13[0], ss13[0], sw2[0], ss2[0])


__all__ = ["prepare_moe_from_compressed_tensors", "stack_compressed_tensors_experts"]
