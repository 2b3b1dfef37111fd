"""ctypes binding of libfused_moe_b200.so (the C ABI declared in include/fused_moe_b200.h).

There is no fallback: if the library is missing, cannot be loaded, or the current device is not a
B200-class GPU, calls raise.  Tensors are torch CUDA tensors; only their device pointers cross the
ABI.  Workspaces come from torch's caching allocator and are cached per (device, size class).
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import torch

OK = 0
ERR_INVALID_ARGUMENT = 1
ERR_CUDA = 2
ERR_WORKSPACE = 3
ERR_EXPERT_ID_RANGE = 4
ERR_DEVICE_WAIT = 5
ERR_UNSUPPORTED_DEVICE = 6

NUMERICS_TORCHREF = 0
NUMERICS_NATIVE = 1
GEMM_AUTO = 0
GEMM_SIMT = 1  # the CUDA-core cross-check GEMM: exists only in the diagnostic library (load_diag)
GEMM_UMMA = 2
ACTIVATION_SILU = 0
ACTIVATION_GELU = 2
ACTIVATION_SWIGLUOAI = 3

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libfused_moe_b200.so")
DIAG_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libfused_moe_b200_diag.so")

EXPORTS = (
    "fmoe_abi_version", "fmoe_last_error", "fmoe_device_supported", "fmoe_read_status",
    "fmoe_w8a8_workspace_layout", "fmoe_w8a8_forward", "fmoe_quantize_weight_rows", "fmoe_quantize_rows",
    "fmoe_bf16_workspace_layout", "fmoe_bf16_forward", "fmoe_w8a16_forward", "fmoe_i8gemm_workspace_bytes", "fmoe_i8gemm_dynamic_scaled_mm",
    "fmoe_stage_timer_create", "fmoe_stage_timer_destroy", "fmoe_stage_timer_reset", "fmoe_stage_timer_calls",
    "fmoe_stage_timer_read", "fmoe_route_build_noalloc", "fmoe_ep_dispatch_workspace_bytes", "fmoe_ep_dispatch_prepare",
    "fmoe_w8a8_expert_rows_forward", "fmoe_bf16_expert_rows_forward", "fmoe_ep_combine_finish",
    "fmoe_i8gemm_dynamic_scaled_mm_pair",
    "fmoe_router_topk",
    "fmoe_ep_peer_create", "fmoe_ep_peer_handle", "fmoe_ep_peer_connect", "fmoe_ep_peer_destroy", "fmoe_ep_peer_slab_bytes",
    "fmoe_ep_peer_dispatch", "fmoe_ep_peer_experts", "fmoe_ep_peer_combine", "fmoe_ep_peer_read_status",
    "fmoe_ep_peer_slab_address", "fmoe_ep_peer_connect_addresses",
)
STAGES = ("route", "quant_in", "gate_up", "quant_mid", "down", "merge")


W8A16_FIXED_POINT = 0
W8A16_BF16_ACTIVATIONS = 1


def w8a16_form_from_env() -> int:
    """FUSED_CPP_MOE_W8A16_FORM: "fixed" (default; activations as 16-bit fixed point on the int8 tensor cores) or "bf16"
    (activations stay bf16, weights widened on the SM)."""
    value = os.environ.get("FUSED_CPP_MOE_W8A16_FORM", "fixed").strip().lower()
    if value in ("fixed", "fixed_point", "0", ""):
        return W8A16_FIXED_POINT
    if value in ("bf16", "bf16_activations", "1"):
        return W8A16_BF16_ACTIVATIONS
    raise ValueError(f"FUSED_CPP_MOE_W8A16_FORM must be 'fixed' or 'bf16', got {value!r}")


class Config(ctypes.Structure):
    _fields_ = [
        ("numerics", ctypes.c_int32), ("gemm_impl", ctypes.c_int32), ("gate_up_tile", ctypes.c_int32),
        ("down_tile", ctypes.c_int32), ("swiglu_limit", ctypes.c_float), ("activation", ctypes.c_int32),
        ("stage_timer", ctypes.c_void_p), ("dump_acc1", ctypes.c_void_p), ("dump_acc2", ctypes.c_void_p),
        ("w13_bias", ctypes.c_void_p), ("w2_bias", ctypes.c_void_p), ("route_rows_bf16", ctypes.c_int32),
        ("w8a16_form", ctypes.c_int32),
    ]


class WorkspaceLayout(ctypes.Structure):
    _fields_ = [(name, ctypes.c_size_t) for name in (
        "total_bytes", "status", "counts", "offsets", "sorted_routes", "row_expert", "items", "scratch", "a_rows",
        "a_scale", "y", "yq", "y_scale", "route_out", "route_pos")]


class FusedMoEError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


_LIB = None
_DIAG_LIB = None


def load() -> ctypes.CDLL:
    """Load the shared library; raise (never fall back) if it is absent."""
    global _LIB
    if _LIB is None:
        _LIB = _open(LIB_PATH)
    return _LIB


def load_diag() -> ctypes.CDLL:
    """The diagnostic twin of the library (same ABI plus the CUDA-core GEMM, the MMA-rate probe and the stage
    switches of FUSED_CPP_MOE_GEMM_DIAG).  For tests and measurements; the package's forward path never loads it."""
    global _DIAG_LIB
    if _DIAG_LIB is None:
        _DIAG_LIB = _open(DIAG_LIB_PATH)
        _DIAG_LIB.fmoe_probe_mma_rate.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                                  ctypes.POINTER(ctypes.c_float)]
    return _DIAG_LIB


def _open(path: str) -> ctypes.CDLL:
    if not os.path.exists(path):
        raise FusedMoEError(ERR_CUDA, f"{path} is missing: build it with `python -m fused_cpp_b200.build` "
                                      "(there is no CPU or PyTorch fallback for this path)")
    lib = ctypes.CDLL(path)
    lib.fmoe_last_error.restype = ctypes.c_char_p
    lib.fmoe_i8gemm_workspace_bytes.restype = ctypes.c_size_t
    lib.fmoe_i8gemm_workspace_bytes.argtypes = [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32]
    p, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
    lib.fmoe_device_supported.argtypes = [ctypes.c_int]
    lib.fmoe_read_status.argtypes = [p, p, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]
    for name in ("fmoe_w8a8_workspace_layout", "fmoe_bf16_workspace_layout"):
        getattr(lib, name).argtypes = [i64, i32, i32, i32, i32, ctypes.POINTER(WorkspaceLayout)]
    lib.fmoe_w8a8_forward.argtypes = [p, p, p, p, p, p, p, i64, i32, i32, i32, i32, ctypes.POINTER(Config), p, p,
                                      ctypes.c_size_t, p]
    lib.fmoe_bf16_forward.argtypes = [p, p, p, p, p, i64, i32, i32, i32, i32, ctypes.POINTER(Config), p, p,
                                      ctypes.c_size_t, p]
    lib.fmoe_w8a16_forward.argtypes = lib.fmoe_w8a8_forward.argtypes
    lib.fmoe_quantize_weight_rows.argtypes = [p, i64, i32, p, p, p]
    lib.fmoe_quantize_rows.argtypes = [p, i64, i32, i32, p, p, p]
    lib.fmoe_stage_timer_create.argtypes = [i32, ctypes.POINTER(ctypes.c_void_p)]
    lib.fmoe_stage_timer_destroy.argtypes = [p]
    lib.fmoe_stage_timer_reset.argtypes = [p]
    lib.fmoe_stage_timer_calls.argtypes = [p]
    lib.fmoe_stage_timer_read.argtypes = [p, i32, ctypes.POINTER(ctypes.c_float)]
    lib.fmoe_ep_dispatch_workspace_bytes.restype = ctypes.c_size_t
    lib.fmoe_ep_dispatch_workspace_bytes.argtypes = [i64, i32, i32]
    lib.fmoe_ep_dispatch_prepare.argtypes = [p, p, i64, i32, i32, i32, i32, i32, i32, i32, p, p, p, p, p, p, ctypes.c_size_t, p]
    lib.fmoe_w8a8_expert_rows_forward.argtypes = [p, p, p, i64, p, p, p, p, i32, i32, i32, ctypes.POINTER(Config), p, p,
                                                  ctypes.c_size_t, p]
    lib.fmoe_bf16_expert_rows_forward.argtypes = [p, p, i64, p, p, i32, i32, i32, ctypes.POINTER(Config), p, p, ctypes.c_size_t, p]
    lib.fmoe_ep_combine_finish.argtypes = [p, p, p, i64, i32, i32, i32, p, p, p]
    lib.fmoe_route_build_noalloc.argtypes = [p, i64, i32, i32, p, p, p, p, p, p]
    lib.fmoe_i8gemm_dynamic_scaled_mm.argtypes = [p, i32, i64, i32, p, p, p, i32, p, i32, p, ctypes.c_size_t, p]
    lib.fmoe_i8gemm_dynamic_scaled_mm_pair.argtypes = [p, i64, i32, p, p, i32, p, p, p, i32, p, p, ctypes.c_size_t, p]
    lib.fmoe_router_topk.argtypes = [p, p, i64, i32, i32, i32, i32, ctypes.c_float, p, p, p]
    lib.fmoe_ep_peer_create.argtypes = [i32, i32, i64, i32, i32, i32, i32, i32, i32, ctypes.POINTER(ctypes.c_void_p)]
    lib.fmoe_ep_peer_handle.argtypes = [p, p]
    lib.fmoe_ep_peer_connect.argtypes = [p, p]
    lib.fmoe_ep_peer_destroy.argtypes = [p]
    lib.fmoe_ep_peer_destroy.restype = None
    lib.fmoe_ep_peer_slab_address.argtypes = [p]
    lib.fmoe_ep_peer_slab_address.restype = ctypes.c_void_p
    lib.fmoe_ep_peer_connect_addresses.argtypes = [p, ctypes.POINTER(ctypes.c_void_p)]
    lib.fmoe_ep_peer_slab_bytes.argtypes = [p]
    lib.fmoe_ep_peer_slab_bytes.restype = ctypes.c_int64
    lib.fmoe_ep_peer_dispatch.argtypes = [p, p, p, i64, i32, i32, i32, p]
    lib.fmoe_ep_peer_experts.argtypes = [p, p, p, p, p, ctypes.POINTER(Config), p]
    lib.fmoe_ep_peer_combine.argtypes = [p, p, i64, i32, p, p]
    lib.fmoe_ep_peer_read_status.argtypes = [p, p, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]
    return lib


def check(code: int, lib: ctypes.CDLL | None = None) -> None:
    if code != OK:
        message = (lib or load()).fmoe_last_error().decode("utf-8", "replace")
        error_type = ValueError if code == ERR_INVALID_ARGUMENT else FusedMoEError
        if error_type is ValueError:
            raise ValueError(message)
        raise FusedMoEError(code, message)


def device_supported(device: int | None = None) -> bool:
    if not torch.cuda.is_available():
        return False
    index = torch.cuda.current_device() if device is None else int(device)
    return bool(load().fmoe_device_supported(index))


def _ptr(tensor: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if tensor is None else tensor.data_ptr())


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def workspace_layout(int8: bool, tokens: int, top_k: int, experts: int, hidden: int, inter: int) -> WorkspaceLayout:
    layout = WorkspaceLayout()
    fn = load().fmoe_w8a8_workspace_layout if int8 else load().fmoe_bf16_workspace_layout
    check(fn(tokens, top_k, experts, hidden, inter, ctypes.byref(layout)))
    return layout


_WORKSPACES: dict[tuple[int, int], torch.Tensor] = {}


def get_workspace(nbytes: int, device: torch.device) -> torch.Tensor:
    """A cached uint8 workspace of at least nbytes (grown geometrically, one per device).

    Like the reference's per-thread RuntimeScratch (csrc/moe/arm/i8mm_w8a8/kernels.cpp:177-182) it is
    reused across calls, so calls on one device must be serialised by the caller (one stream).
    """
    key = (device.index if device.index is not None else torch.cuda.current_device(), 0)
    current = _WORKSPACES.get(key)
    if current is None or current.numel() < nbytes:
        size = max(nbytes, 0 if current is None else int(current.numel() * 1.5))
        _WORKSPACES.pop(key, None)
        current = torch.empty(size + 256, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = current
    offset = (-current.data_ptr()) % 256
    return current[offset:offset + nbytes]


@dataclass
class ForwardResult:
    out: torch.Tensor
    workspace: torch.Tensor
    layout: WorkspaceLayout
    acc1: torch.Tensor | None = None
    acc2: torch.Tensor | None = None

    def region(self, name: str, dtype: torch.dtype, shape) -> torch.Tensor:
        count = 1
        for dim in shape:
            count *= int(dim)
        begin = getattr(self.layout, name)
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        return self.workspace[begin:begin + nbytes].view(dtype).reshape(shape)

    def status(self) -> tuple[int, int]:
        error, detail = ctypes.c_int32(0), ctypes.c_int32(0)
        check(load().fmoe_read_status(_ptr(self.workspace), _stream(), ctypes.byref(error), ctypes.byref(detail)))
        return error.value, detail.value

    def status_word(self, index: int) -> int:
        """One int32 word of the status block (2, 5: work items of the two GEMMs; 6, 7: those of the experts routed to
        the two-SM kernel when the tiles are automatic; 3: active experts).  Synchronises."""
        torch.cuda.current_stream().synchronize()
        return int(self.workspace[: 64].view(torch.int32)[index].item())

    def raise_for_status(self) -> None:
        error, detail = self.status()
        if error == ERR_EXPERT_ID_RANGE:
            raise FusedMoEError(error, f"topk expert id is out of range (flat route {detail})")
        if error != OK:
            raise FusedMoEError(error, load().fmoe_last_error().decode("utf-8", "replace"))


class StageTimer:
    """Per-stage CUDA-event timer handed to moe_forward(stage_timer=...): the GPU form of the
    reference's FUSED_CPP_MOE_STAGE_TIMING report."""

    def __init__(self, max_calls: int):
        self.handle = ctypes.c_void_p(0)
        check(load().fmoe_stage_timer_create(int(max_calls), ctypes.byref(self.handle)))

    def reset(self) -> None:
        check(load().fmoe_stage_timer_reset(self.handle))

    @property
    def calls(self) -> int:
        return int(load().fmoe_stage_timer_calls(self.handle))

    def read(self, call: int) -> dict[str, float]:
        values = (ctypes.c_float * len(STAGES))()
        check(load().fmoe_stage_timer_read(self.handle, int(call), values))
        return {name: float(values[i]) for i, name in enumerate(STAGES)}

    def close(self) -> None:
        if self.handle:
            load().fmoe_stage_timer_destroy(self.handle)
            self.handle = ctypes.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _require_cuda(name: str, tensor: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if tensor.device.type != "cuda":
        raise ValueError(f"{name} must be a CUDA tensor (this build has no CPU path)")
    if tensor.dtype != dtype:
        raise TypeError(f"{name} must have dtype {dtype}, got {tensor.dtype}")
    return tensor.contiguous()


def moe_forward(x, w13, w2, topk_weights, topk_ids, *, s13=None, s2=None, numerics: int = NUMERICS_TORCHREF,
                gemm_impl: int = GEMM_AUTO, gate_up_tile: int = 0, down_tile: int = 0, swiglu_limit: float | None = None,
                out: torch.Tensor | None = None, dump: bool = False, workspace: torch.Tensor | None = None,
                stage_timer: "StageTimer | None" = None, diagnostic: bool = False, activation: int = ACTIVATION_SILU,
                w13_bias: torch.Tensor | None = None, w2_bias: torch.Tensor | None = None, w8a16: bool = False,
                route_rows_bf16: bool = False, w8a16_form: int | None = None) -> ForwardResult:
    """One routed-expert MoE forward through the C ABI.  int8 weights (with s13/s2) select W8A8, or, with
    w8a16=True, the W8A16 path (16-bit activations; w8a16_form picks W8A16_FIXED_POINT, the default, or
    W8A16_BF16_ACTIVATIONS; None reads FUSED_CPP_MOE_W8A16_FORM = "fixed" | "bf16").
    diagnostic=True (or gemm_impl=GEMM_SIMT) runs the call in the diagnostic library instead of the product one."""
    quantised_weights = w13.dtype == torch.int8
    if w8a16 and not quantised_weights:
        raise TypeError("w8a16 needs int8 weights with s13 / s2")
    int8 = quantised_weights and not w8a16
    x = _require_cuda("input", x, torch.bfloat16)
    w13 = _require_cuda("w13", w13, torch.int8 if quantised_weights else torch.bfloat16)
    w2 = _require_cuda("w2", w2, torch.int8 if quantised_weights else torch.bfloat16)
    topk_weights = _require_cuda("topk_weights", topk_weights, torch.float32)
    topk_ids = _require_cuda("topk_ids", topk_ids, torch.int64)
    tokens, hidden = x.shape
    experts, two_i, _ = w13.shape
    inter = two_i // 2
    top_k = topk_ids.shape[1]
    if quantised_weights:
        s13 = _require_cuda("w13_scale", s13, torch.float32)
        s2 = _require_cuda("w2_scale", s2, torch.float32)
    if out is None:
        out = torch.empty_like(x)
    layout = workspace_layout(int8, tokens, top_k, experts, hidden, inter)
    if workspace is None:
        workspace = get_workspace(layout.total_bytes, x.device)
    forced = os.environ.get("FUSED_CPP_MOE_FORCE_TILES")  # "gate_up,down": diagnostic override of the row tiles
    if forced and gate_up_tile == 0 and down_tile == 0:
        gate_up_tile, down_tile = (int(v) for v in forced.split(","))
    config = Config()
    config.numerics = numerics
    config.gemm_impl = gemm_impl
    config.gate_up_tile = gate_up_tile
    config.down_tile = down_tile
    config.swiglu_limit = (10.0 if int8 else 0.0) if swiglu_limit is None else float(swiglu_limit)
    config.activation = int(activation)
    config.route_rows_bf16 = 1 if route_rows_bf16 else 0
    config.w8a16_form = w8a16_form_from_env() if w8a16_form is None else int(w8a16_form)
    if w13_bias is not None:
        w13_bias = _require_cuda("w13_bias", w13_bias, torch.float32)
        if tuple(w13_bias.shape) != (experts, two_i):
            raise ValueError("w13_bias must be [E, 2I]")
        config.w13_bias = w13_bias.data_ptr()
    if w2_bias is not None:
        w2_bias = _require_cuda("w2_bias", w2_bias, torch.float32)
        if tuple(w2_bias.shape) != (experts, hidden):
            raise ValueError("w2_bias must be [E, H]")
        config.w2_bias = w2_bias.data_ptr()
    if stage_timer is not None:
        config.stage_timer = stage_timer.handle
    acc1 = acc2 = None
    if dump:
        acc_dtype = torch.int32 if int8 else torch.float32
        acc1 = torch.zeros((max(tokens * top_k, 1), two_i), dtype=acc_dtype, device=x.device)
        acc2 = torch.zeros((max(tokens * top_k, 1), hidden), dtype=acc_dtype, device=x.device)
        config.dump_acc1 = acc1.data_ptr()
        config.dump_acc2 = acc2.data_ptr()
    # The CUDA-core cross-check and the stage switches exist only in the diagnostic library.
    lib = load_diag() if (gemm_impl == GEMM_SIMT or diagnostic) else load()
    if quantised_weights:
        entry = lib.fmoe_w8a16_forward if w8a16 else lib.fmoe_w8a8_forward
        code = entry(_ptr(x), _ptr(w13), _ptr(s13), _ptr(w2), _ptr(s2), _ptr(topk_weights), _ptr(topk_ids),
                     tokens, top_k, experts, hidden, inter, ctypes.byref(config), _ptr(out),
                     _ptr(workspace), workspace.numel(), _stream())
    else:
        code = lib.fmoe_bf16_forward(_ptr(x), _ptr(w13), _ptr(w2), _ptr(topk_weights), _ptr(topk_ids), tokens, top_k,
                                     experts, hidden, inter, ctypes.byref(config), _ptr(out), _ptr(workspace),
                                     workspace.numel(), _stream())
    check(code, lib)
    return ForwardResult(out=out, workspace=workspace, layout=layout, acc1=acc1, acc2=acc2)


def quantize_rows(x: torch.Tensor, numerics: int = NUMERICS_TORCHREF, weight_mode: bool = False):
    """bf16 [rows, cols] -> (int8 [rows, cols], fp32 scale [rows]) on the GPU."""
    x = _require_cuda("x", x, torch.bfloat16)
    rows, cols = x.shape
    q = torch.empty((rows, cols), dtype=torch.int8, device=x.device)
    scale = torch.empty(rows, dtype=torch.float32, device=x.device)
    lib = load()
    if weight_mode:
        check(lib.fmoe_quantize_weight_rows(_ptr(x), rows, cols, _ptr(q), _ptr(scale), _stream()))
    else:
        check(lib.fmoe_quantize_rows(_ptr(x), rows, cols, numerics, _ptr(q), _ptr(scale), _stream()))
    return q, scale


def route_build_noalloc(topk_ids: torch.Tensor, experts: int):
    """Route lists through the allocation-free entry point (scratch inside the library, nothing allocated by it).

    For hosts that cannot allocate device memory while serving.  The output tensors here are the caller's
    (this helper makes them with torch for convenience); limits: T*K <= 131072, experts <= 512.
    Returns (counts[E], offsets[E+1], sorted_routes[T*K], row_expert[T*K], status[2]) on the device.
    """
    topk_ids = _require_cuda("topk_ids", topk_ids, torch.int64)
    tokens, top_k = topk_ids.shape
    device = topk_ids.device
    counts = torch.empty(experts, dtype=torch.int32, device=device)
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=device)
    order = torch.empty(max(tokens * top_k, 1), dtype=torch.int32, device=device)
    row_expert = torch.empty(max(tokens * top_k, 1), dtype=torch.int32, device=device)
    status = torch.empty(2, dtype=torch.int32, device=device)
    check(load().fmoe_route_build_noalloc(_ptr(topk_ids), tokens, top_k, experts, _ptr(counts), _ptr(offsets), _ptr(order),
                                          _ptr(row_expert), _ptr(status), _stream()))
    return counts, offsets, order[: tokens * top_k], row_expert[: tokens * top_k], status


# ---- expert-parallel building blocks (used by fused_cpp_b200.ep) ---------------------------------

def ep_dispatch_prepare(x, topk_ids, experts_global: int, world: int, shared_rank: int, int8: bool,
                        numerics: int = NUMERICS_TORCHREF):
    """Sort this rank's routes by destination rank and lay out the payload (fmoe_ep_dispatch_prepare).

    Returns dict(dest_counts int32[W], send_order int32[TK], send_rows [TK,H] int8|bf16, send_scale f32[TK]|None,
    send_expert int64[TK], workspace)."""
    x = _require_cuda("input", x, torch.bfloat16)
    topk_ids = _require_cuda("topk_ids", topk_ids, torch.int64)
    tokens, hidden = x.shape
    top_k = topk_ids.shape[1]
    routes = tokens * top_k
    device = x.device
    lib = load()
    workspace = torch.empty(lib.fmoe_ep_dispatch_workspace_bytes(tokens, top_k, world) + 256, dtype=torch.uint8, device=device)
    offset = (-workspace.data_ptr()) % 256
    ws = workspace[offset:]
    out = {
        "dest_counts": torch.empty(world, dtype=torch.int32, device=device),
        "send_order": torch.empty(max(routes, 1), dtype=torch.int32, device=device),
        "send_rows": torch.empty((max(routes, 1), hidden), dtype=torch.int8 if int8 else torch.bfloat16, device=device),
        "send_scale": torch.empty(max(routes, 1), dtype=torch.float32, device=device) if int8 else None,
        "send_expert": torch.empty(max(routes, 1), dtype=torch.int64, device=device),
        "workspace": ws,
    }
    check(lib.fmoe_ep_dispatch_prepare(_ptr(x), _ptr(topk_ids), tokens, top_k, experts_global, world, shared_rank, hidden,
                                       1 if int8 else 0, numerics, _ptr(out["dest_counts"]), _ptr(out["send_order"]),
                                       _ptr(out["send_rows"]), _ptr(out["send_scale"]), _ptr(out["send_expert"]), _ptr(ws),
                                       ws.numel(), _stream()))
    for name in ("send_order", "send_rows", "send_scale", "send_expert"):
        if out[name] is not None:
            out[name] = out[name][:routes]
    return out


def expert_rows_forward(rows, rows_scale, rows_expert, w13, w2, s13=None, s2=None, *, numerics: int = NUMERICS_TORCHREF,
                        gemm_impl: int = GEMM_AUTO, gate_up_tile: int = 0, down_tile: int = 0, swiglu_limit: float | None = None):
    """Grouped GEMMs over received rows (fmoe_*_expert_rows_forward).  Returns route_out fp32 [R, H] in row order."""
    int8 = w13.dtype == torch.int8
    count = rows.shape[0]
    experts, two_i, hidden = w13.shape
    inter = two_i // 2
    device = w13.device
    route_out = torch.empty((count, hidden), dtype=torch.float32, device=device)
    if count == 0:
        return route_out
    layout = workspace_layout(int8, count, 1, experts, hidden, inter)
    workspace = get_workspace(layout.total_bytes, device)
    config = Config()
    config.numerics = numerics
    config.gemm_impl = gemm_impl
    config.gate_up_tile = gate_up_tile
    config.down_tile = down_tile
    config.swiglu_limit = (10.0 if int8 else 0.0) if swiglu_limit is None else float(swiglu_limit)
    lib = load()
    rows = rows.contiguous()
    rows_expert = rows_expert.contiguous()
    if int8:
        rows_scale = rows_scale.contiguous()
        code = lib.fmoe_w8a8_expert_rows_forward(_ptr(rows), _ptr(rows_scale), _ptr(rows_expert), count, _ptr(w13), _ptr(s13),
                                                 _ptr(w2), _ptr(s2), experts, hidden, inter, ctypes.byref(config), _ptr(route_out),
                                                 _ptr(workspace), workspace.numel(), _stream())
    else:
        code = lib.fmoe_bf16_expert_rows_forward(_ptr(rows), _ptr(rows_expert), count, _ptr(w13), _ptr(w2), experts, hidden, inter,
                                                 ctypes.byref(config), _ptr(route_out), _ptr(workspace), workspace.numel(), _stream())
    check(code)
    return route_out


def ep_combine_finish(returned_rows, send_order, topk_weights, tokens: int, top_k: int, tree_merge: bool, out=None):
    """Scatter the returned fp32 route rows to flat-route order and merge (fmoe_ep_combine_finish)."""
    hidden = returned_rows.shape[1]
    device = returned_rows.device
    if out is None:
        out = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=device)
    route_out = torch.empty((max(tokens * top_k, 1), hidden), dtype=torch.float32, device=device)
    returned_rows, topk_weights = returned_rows.contiguous(), topk_weights.contiguous()
    check(load().fmoe_ep_combine_finish(_ptr(returned_rows), _ptr(send_order), _ptr(topk_weights), tokens, top_k,
                                        hidden, 1 if tree_merge else 0, _ptr(route_out), _ptr(out), _stream()))
    return out


def router_topk(logits: torch.Tensor, top_k: int, *, scoring: str = "softmax", selection_bias: torch.Tensor | None = None,
                renormalize: bool = True, routed_scaling_factor: float = 1.0):
    """Expert scores -> (topk_weights fp32 [T, K], topk_ids int64 [T, K]) on the GPU (fmoe_router_topk)."""
    if scoring not in ("softmax", "sigmoid"):
        raise ValueError("scoring must be 'softmax' or 'sigmoid'")
    logits = _require_cuda("logits", logits, torch.float32)
    if logits.dim() != 2:
        raise ValueError("logits must be [tokens, experts]")
    tokens, experts = logits.shape
    bias = None
    if selection_bias is not None:
        bias = _require_cuda("selection_bias", selection_bias, torch.float32)
        if bias.shape != (experts,):
            raise ValueError("selection_bias must be [experts]")
    weights = torch.empty((tokens, top_k), dtype=torch.float32, device=logits.device)
    ids = torch.empty((tokens, top_k), dtype=torch.int64, device=logits.device)
    check(load().fmoe_router_topk(_ptr(logits), _ptr(bias), tokens, experts, top_k, 1 if scoring == "sigmoid" else 0,
                                  1 if renormalize else 0, float(routed_scaling_factor), _ptr(weights), _ptr(ids), _stream()))
    return weights, ids


class PeerContext:
    """One rank's side of the peer-memory expert-parallel exchange (fmoe_ep_peer_*): owns the slab that the other
    ranks write into.  The caller exchanges the 64-byte handles and provides the collectives between the stages."""

    def __init__(self, world: int, rank: int, tokens_max: int, top_k: int, hidden: int, inter: int, local_experts: int, int8: bool,
                 return_bf16: bool = False):
        self.world, self.rank, self.top_k, self.hidden, self.int8 = world, rank, top_k, hidden, int8
        self.tokens_max = tokens_max
        handle = ctypes.c_void_p()
        check(load().fmoe_ep_peer_create(world, rank, tokens_max, top_k, hidden, inter, local_experts, 1 if int8 else 0,
                                         1 if return_bf16 else 0, ctypes.byref(handle)))
        self.handle = handle

    def ipc_handle(self) -> bytes:
        buffer = ctypes.create_string_buffer(64)
        check(load().fmoe_ep_peer_handle(self.handle, buffer))
        return buffer.raw

    def connect(self, handles: list) -> None:
        blob = b"".join(bytes(h) for h in handles)
        if len(blob) != 64 * self.world:
            raise ValueError("expected one 64-byte handle per rank")
        check(load().fmoe_ep_peer_connect(self.handle, ctypes.create_string_buffer(blob, len(blob))))

    @property
    def slab_address(self) -> int:
        return int(load().fmoe_ep_peer_slab_address(self.handle) or 0)

    def connect_addresses(self, addresses: list) -> None:
        """Connect ranks that can already address one another's slabs (contexts of one process)."""
        if len(addresses) != self.world:
            raise ValueError("expected one slab address per rank")
        table = (ctypes.c_void_p * self.world)(*[ctypes.c_void_p(int(a)) for a in addresses])
        check(load().fmoe_ep_peer_connect_addresses(self.handle, table))

    @property
    def slab_bytes(self) -> int:
        return int(load().fmoe_ep_peer_slab_bytes(self.handle))

    def dispatch(self, x, topk_ids, experts_global: int, shared_rank: int, numerics: int) -> None:
        check(load().fmoe_ep_peer_dispatch(self.handle, _ptr(x), _ptr(topk_ids), x.shape[0], experts_global, shared_rank, numerics,
                                           _stream()))

    def experts(self, w13, s13, w2, s2, config: "Config") -> None:
        check(load().fmoe_ep_peer_experts(self.handle, _ptr(w13), _ptr(s13), _ptr(w2), _ptr(s2), ctypes.byref(config), _stream()))

    def combine(self, topk_weights, tokens: int, tree_merge: bool, out) -> None:
        check(load().fmoe_ep_peer_combine(self.handle, _ptr(topk_weights), tokens, 1 if tree_merge else 0, _ptr(out), _stream()))

    def read_status(self) -> tuple[int, int]:
        first, second = ctypes.c_int32(0), ctypes.c_int32(0)
        check(load().fmoe_ep_peer_read_status(self.handle, _stream(), ctypes.byref(first), ctypes.byref(second)))
        return int(first.value), int(second.value)

    def close(self) -> None:
        if self.handle:
            load().fmoe_ep_peer_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def probe_mma_rate(int8: bool, n: int = 256, iterations: int = 20000, *, nonzero: bool = False, commit_every: int = 0,
                   second_issuer: bool = False, alternate: bool = False, two_sm: bool = False, round_trips: bool = False) -> float:
    """Measured dense tensor-core peak (tera-ops/s) for a 128 x n MMA tile on the current GPU.

    nonzero: operands hold a non-zero pattern instead of zeros; commit_every: a tcgen05.commit after every c MMAs;
    second_issuer: two threads of different warps issue half of the MMAs each, into separate accumulators;
    alternate: the one issuing thread alternates between two accumulators; two_sm: cta_group::2 MMAs of 256 x n issued
    by the leader of every two-CTA cluster; round_trips (needs commit_every = c): rounds of c MMAs, a commit and a wait
    for it, so that c x the time per MMA is the latency of one pipeline stage."""
    value = ctypes.c_float(0.0)
    mode = ((1 if nonzero else 0) | (2 if second_issuer else 0) | (4 if alternate else 0) | (8 if two_sm else 0) | (16 if round_trips else 0)
            | (commit_every << 8))
    check(load_diag().fmoe_probe_mma_rate(1 if int8 else 0, n, iterations, mode, ctypes.byref(value)), load_diag())
    return float(value.value)
