"""ctypes front-end of the CPU oracle (oracle/moe_oracle.c).

Test infrastructure only.  Tensors are torch CPU tensors; bf16 tensors are passed as their
16-bit patterns.  Every function cites the C routine it calls; the C file cites the reference.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import build as _build

NUMERICS_TORCHREF = 0
NUMERICS_NATIVE = 1

_LIB = None


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = _build.LIB
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(_build.SRC):
            path = _build.build()
        _LIB = ctypes.CDLL(path)
        _LIB.fmoe_oracle_expneg.restype = ctypes.c_float
        _LIB.fmoe_oracle_expneg.argtypes = [ctypes.c_float]
        _LIB.fmoe_oracle_f32_to_bf16.restype = ctypes.c_uint16
        _LIB.fmoe_oracle_f32_to_bf16.argtypes = [ctypes.c_float]
    return _LIB


def set_threads(count: int) -> None:
    """OpenMP thread count of the oracle's parallel loops (omp_set_num_threads of the runtime the library links).

    A launcher may export OMP_NUM_THREADS=1 to its children (torch.distributed.run does); a timing that is meant
    to use every host core sets the count here instead of trusting the environment."""
    lib().omp_set_num_threads(ctypes.c_int(max(1, int(count))))


def get_max_threads() -> int:
    fn = lib().omp_get_max_threads
    fn.restype = ctypes.c_int
    return int(fn())


def _ptr(tensor: torch.Tensor | None) -> ctypes.c_void_p:
    if tensor is None:
        return ctypes.c_void_p(0)
    assert tensor.device.type == "cpu" and tensor.is_contiguous()
    return ctypes.c_void_p(tensor.data_ptr())


def expneg(gate: float) -> float:
    return float(lib().fmoe_oracle_expneg(ctypes.c_float(gate)))


def route_build(topk_ids: torch.Tensor, experts: int):
    """fmoe_oracle_route_build: (counts[E], offsets[E+1], sorted flat route ids[T*K])."""
    ids = topk_ids.to(torch.int64).contiguous().reshape(-1)
    counts = torch.zeros(experts, dtype=torch.int32)
    offsets = torch.zeros(experts + 1, dtype=torch.int32)
    order = torch.zeros(max(ids.numel(), 1), dtype=torch.int32)
    status = lib().fmoe_oracle_route_build(_ptr(ids), ctypes.c_int64(ids.numel()), ctypes.c_int(experts),
                                           _ptr(counts), _ptr(offsets), _ptr(order))
    if status != 0:
        raise ValueError("topk expert id is out of range")
    return counts, offsets, order[: ids.numel()]


def quantize_rows(x_bf16: torch.Tensor, numerics: int = NUMERICS_TORCHREF):
    """fmoe_oracle_quantize_rows: bf16 [rows, cols] -> (int8 [rows, cols], fp32 scale [rows])."""
    assert x_bf16.dtype == torch.bfloat16 and x_bf16.dim() == 2
    x = x_bf16.contiguous()
    q = torch.empty(x.shape, dtype=torch.int8)
    scale = torch.empty(x.shape[0], dtype=torch.float32)
    lib().fmoe_oracle_quantize_rows(_ptr(x), ctypes.c_int64(x.shape[0]), ctypes.c_int(x.shape[1]),
                                    ctypes.c_int(numerics), _ptr(q), _ptr(scale))
    return q, scale


def w8a8_forward(x, w13, s13, w2, s2, topk_w, topk_ids, numerics: int = NUMERICS_TORCHREF, dumps: bool = False):
    """fmoe_oracle_w8a8_forward.  Returns out bf16 [T,H], or (out, dict of intermediates) with dumps=True.

    Intermediates: xq[T,H], a[T] per token; acc1[TK,2I], y[TK,I] bf16, yq[TK,I], a2[TK], acc2[TK,H],
    route_out[TK,H], all indexed by flat route id t*K+slot.
    """
    tokens, hidden = x.shape
    experts, two_i, _ = w13.shape
    inter = two_i // 2
    top_k = topk_ids.shape[1]
    routes = tokens * top_k
    x = x.contiguous()
    w13 = w13.contiguous()
    w2 = w2.contiguous()
    s13 = s13.to(torch.float32).reshape(experts, two_i).contiguous()
    s2 = s2.to(torch.float32).reshape(experts, hidden).contiguous()
    topk_w = topk_w.to(torch.float32).contiguous()
    ids = topk_ids.to(torch.int64).contiguous()
    out = torch.empty((tokens, hidden), dtype=torch.bfloat16)
    d = {}
    if dumps:
        d = {
            "xq": torch.empty((tokens, hidden), dtype=torch.int8),
            "a": torch.empty(tokens, dtype=torch.float32),
            "acc1": torch.empty((routes, two_i), dtype=torch.int32),
            "y": torch.empty((routes, inter), dtype=torch.bfloat16),
            "yq": torch.empty((routes, inter), dtype=torch.int8),
            "a2": torch.empty(routes, dtype=torch.float32),
            "acc2": torch.empty((routes, hidden), dtype=torch.int32),
            "route_out": torch.empty((routes, hidden), dtype=torch.float32),
        }
    status = lib().fmoe_oracle_w8a8_forward(
        _ptr(x), _ptr(w13), _ptr(s13), _ptr(w2), _ptr(s2), _ptr(topk_w), _ptr(ids),
        ctypes.c_int64(tokens), ctypes.c_int(top_k), ctypes.c_int(experts), ctypes.c_int(hidden), ctypes.c_int(inter),
        ctypes.c_int(numerics), _ptr(out),
        _ptr(d.get("xq")), _ptr(d.get("a")), _ptr(d.get("acc1")), _ptr(d.get("y")), _ptr(d.get("yq")),
        _ptr(d.get("a2")), _ptr(d.get("acc2")), _ptr(d.get("route_out")))
    if status != 0:
        raise ValueError("topk expert id is out of range")
    return (out, d) if dumps else out


def bf16_forward(x, w13, w2, topk_w, topk_ids, swiglu_limit: float = 0.0, dumps: bool = False, activation: int = 0,
                 w13_bias=None, w2_bias=None):
    """fmoe_oracle_bf16_forward_ex.  Returns out bf16 [T,H] (and {y, route_out} with dumps=True).
    activation: 0 SiLU (with swiglu_limit), 2 gelu, 3 swigluoai; biases fp32 [E,2I] / [E,H] or None.
    w13 holds gate rows [0,I) then up rows [I,2I) for every activation."""
    tokens, hidden = x.shape
    experts, two_i, _ = w13.shape
    inter = two_i // 2
    top_k = topk_ids.shape[1]
    routes = tokens * top_k
    out = torch.empty((tokens, hidden), dtype=torch.bfloat16)
    d = {}
    if dumps:
        d = {"y": torch.empty((routes, inter), dtype=torch.bfloat16),
             "route_out": torch.empty((routes, hidden), dtype=torch.float32)}
    x, w13, w2 = x.contiguous(), w13.contiguous(), w2.contiguous()
    topk_w, topk_ids = topk_w.to(torch.float32).contiguous(), topk_ids.to(torch.int64).contiguous()
    b13 = None if w13_bias is None else w13_bias.to(torch.float32).reshape(experts, two_i).contiguous()
    b2 = None if w2_bias is None else w2_bias.to(torch.float32).reshape(experts, hidden).contiguous()
    status = lib().fmoe_oracle_bf16_forward_ex(
        _ptr(x), _ptr(w13), _ptr(w2), _ptr(topk_w), _ptr(topk_ids),
        ctypes.c_int64(tokens), ctypes.c_int(top_k), ctypes.c_int(experts), ctypes.c_int(hidden), ctypes.c_int(inter),
        ctypes.c_float(swiglu_limit), ctypes.c_int(activation), _ptr(b13), _ptr(b2), _ptr(out), _ptr(d.get("y")),
        _ptr(d.get("route_out")))
    if status != 0:
        raise ValueError("topk expert id is out of range")
    return (out, d) if dumps else out


def w8a16_forward(x, w13, s13, w2, s2, topk_w, topk_ids, swiglu_limit: float = 0.0, dumps: bool = False, activation: int = 0,
                  fixed_point: bool = False):
    """fmoe_oracle_w8a16_forward: int8 weights + per-channel scales, bf16 activations.  Returns out bf16 [T,H]
    (and {y, route_out} with dumps=True).  fixed_point=True: fmoe_oracle_w8a16_fixed_forward, the activations as
    16-bit fixed point per row with exact integer dot products (the CUDA library's default W8A16 form)."""
    tokens, hidden = x.shape
    experts, two_i, _ = w13.shape
    inter = two_i // 2
    top_k = topk_ids.shape[1]
    routes = tokens * top_k
    out = torch.empty((tokens, hidden), dtype=torch.bfloat16)
    d = {}
    if dumps:
        d = {"y": torch.empty((routes, inter), dtype=torch.bfloat16),
             "route_out": torch.empty((routes, hidden), dtype=torch.float32)}
    x, w13, w2 = x.contiguous(), w13.contiguous(), w2.contiguous()
    s13 = s13.to(torch.float32).reshape(experts, two_i).contiguous()
    s2 = s2.to(torch.float32).reshape(experts, hidden).contiguous()
    topk_w, topk_ids = topk_w.to(torch.float32).contiguous(), topk_ids.to(torch.int64).contiguous()
    entry = lib().fmoe_oracle_w8a16_fixed_forward if fixed_point else lib().fmoe_oracle_w8a16_forward
    status = entry(
        _ptr(x), _ptr(w13), _ptr(s13), _ptr(w2), _ptr(s2), _ptr(topk_w), _ptr(topk_ids),
        ctypes.c_int64(tokens), ctypes.c_int(top_k), ctypes.c_int(experts), ctypes.c_int(hidden), ctypes.c_int(inter),
        ctypes.c_float(swiglu_limit), ctypes.c_int(activation), _ptr(out), _ptr(d.get("y")), _ptr(d.get("route_out")))
    if status != 0:
        raise ValueError("topk expert id is out of range")
    return (out, d) if dumps else out


def merge_bf16_path(route_out: torch.Tensor, topk_w: torch.Tensor) -> torch.Tensor:
    """fmoe_oracle_merge_bf16_path: route_out fp32 [T,K,H] + weights [T,K] -> bf16 [T,H]."""
    tokens, top_k, hidden = route_out.shape
    out = torch.empty((tokens, hidden), dtype=torch.bfloat16)
    route_out, topk_w = route_out.contiguous(), topk_w.to(torch.float32).contiguous()
    lib().fmoe_oracle_merge_bf16_path(_ptr(route_out), _ptr(topk_w),
                                      ctypes.c_int64(tokens), ctypes.c_int(top_k), ctypes.c_int(hidden), _ptr(out))
    return out


def i8gemm_dynamic(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor, bias=None,
                   out_dtype=torch.float32, clamp_low: int = -128) -> torch.Tensor:
    """fmoe_oracle_i8gemm_dynamic: dense dynamic-quant W8A8 linear (scalar-fallback arithmetic)."""
    rows, k = x.shape
    n = weight.shape[0]
    out = torch.empty((rows, n), dtype=out_dtype)
    # keep every converted operand alive until the call returns
    x32 = x.to(torch.float32).contiguous()
    w = weight.contiguous()
    scale = weight_scale.to(torch.float32).reshape(-1).expand(n).contiguous()
    bias32 = None if bias is None else bias.to(torch.float32).contiguous()
    lib().fmoe_oracle_i8gemm_dynamic(_ptr(x32), ctypes.c_int64(rows), ctypes.c_int(k), _ptr(w), _ptr(scale), ctypes.c_int(n),
                                     _ptr(bias32), _ptr(out), ctypes.c_int(1 if out_dtype == torch.bfloat16 else 0),
                                     ctypes.c_int(clamp_low))
    return out


def w8a8_route_rows(rows_q, rows_scale, rows_expert, w13, s13, w2, s2, numerics: int = NUMERICS_TORCHREF) -> torch.Tensor:
    """fmoe_oracle_w8a8_route_rows: pre-quantised rows [R,H] + scales + expert ids -> route_out fp32 [R,H]."""
    rows, hidden = rows_q.shape
    experts, two_i, _ = w13.shape
    out = torch.empty((rows, hidden), dtype=torch.float32)
    rows_q, rows_scale = rows_q.contiguous(), rows_scale.to(torch.float32).contiguous()
    rows_expert, w13, w2 = rows_expert.to(torch.int64).contiguous(), w13.contiguous(), w2.contiguous()
    s13 = s13.to(torch.float32).reshape(experts, two_i).contiguous()
    s2 = s2.to(torch.float32).reshape(experts, hidden).contiguous()
    status = lib().fmoe_oracle_w8a8_route_rows(
        _ptr(rows_q), _ptr(rows_scale), _ptr(rows_expert), ctypes.c_int64(rows), _ptr(w13), _ptr(s13), _ptr(w2), _ptr(s2),
        ctypes.c_int(experts),
        ctypes.c_int(hidden), ctypes.c_int(two_i // 2), ctypes.c_int(numerics), _ptr(out))
    if status != 0:
        raise ValueError("row expert id is out of range")
    return out


def merge_w8a8_path(route_out: torch.Tensor, topk_w: torch.Tensor) -> torch.Tensor:
    """fmoe_oracle_merge_w8a8_path: route_out fp32 [T,K,H] + weights [T,K] -> bf16 [T,H]."""
    tokens, top_k, hidden = route_out.shape
    out = torch.empty((tokens, hidden), dtype=torch.bfloat16)
    route_out, topk_w = route_out.contiguous(), topk_w.to(torch.float32).contiguous()
    lib().fmoe_oracle_merge_w8a8_path(_ptr(route_out), _ptr(topk_w),
                                      ctypes.c_int64(tokens), ctypes.c_int(top_k), ctypes.c_int(hidden), _ptr(out))
    return out
