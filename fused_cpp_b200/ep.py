"""Expert-parallel routed-expert MoE over one NVLink/NVSwitch box.

One process per GPU (torch.distributed, NCCL).  Rank r owns experts [r*E/W, (r+1)*E/W) and, if there is
one, a replica of the shared expert; tokens stay data-parallel.  One forward is

    source rank : quantise / copy each route's token row, sort routes by destination rank   (CUDA)
    exchange    : counts, then rows + (scale, local expert id) by all-to-all-v               (NCCL)
    expert rank : grouped gate_up / down GEMMs over the received rows -> fp32 route rows      (CUDA, tcgen05)
    exchange    : fp32 route rows back by the mirrored all-to-all-v                           (NCCL)
    source rank : scatter to flat-route order, merge in the reference's slot order            (CUDA)

Each route keeps the single-GPU arithmetic and the merge order is unchanged, so the sharded result is
bit-identical to the single-GPU one (int8 path and bf16 path alike).  The reference has no expert
parallelism to be compatible with (csrc/moe/arm/i8mm_w8a8/kernels.cpp:488 rejects it).

The device steps sit behind a small backend object so that the exchange logic can be tested with CPU
ranks (gloo) and a stand-in backend; the product backend is CudaBackend and nothing else is shipped.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


class CudaBackend:
    """The three device steps through the C ABI (fused_cpp_b200._lib)."""

    def __init__(self, numerics: int = 0, gate_up_tile: int = 0, down_tile: int = 0):
        self.numerics = numerics
        self.gate_up_tile = gate_up_tile
        self.down_tile = down_tile

    def dispatch_prepare(self, x, topk_ids, experts_global, world, shared_rank, int8):
        from . import _lib

        return _lib.ep_dispatch_prepare(x, topk_ids, experts_global, world, shared_rank, int8, self.numerics)

    def expert_rows_forward(self, rows, scale, expert, weights, swiglu_limit):
        from . import _lib

        return _lib.expert_rows_forward(rows, scale, expert, weights["w13"], weights["w2"], weights.get("s13"), weights.get("s2"),
                                        numerics=self.numerics, gate_up_tile=self.gate_up_tile, down_tile=self.down_tile,
                                        swiglu_limit=swiglu_limit)

    def combine_finish(self, returned, send_order, topk_weights, tokens, top_k, tree_merge, out):
        from . import _lib

        return _lib.ep_combine_finish(returned, send_order, topk_weights, tokens, top_k, tree_merge, out)


def validate_expert_split(experts_global: int, world: int, local_experts: int, has_shared: bool) -> int:
    """Experts per rank, after checking that every rank holds the same contiguous share."""
    if world <= 0 or experts_global <= 0 or experts_global % world != 0:
        raise ValueError(f"{experts_global} experts do not split evenly over {world} ranks")
    per_rank = experts_global // world
    expected = per_rank + (1 if has_shared else 0)
    if local_experts != expected:
        raise ValueError(f"this rank holds {local_experts} expert weight blocks, expected {expected} "
                         f"({per_rank} routed{' + 1 shared' if has_shared else ''})")
    return per_rank


@dataclass
class ExchangePlan:
    send_splits: list
    recv_splits: list

    @property
    def received(self) -> int:
        return sum(self.recv_splits)


def exchange_counts(dest_counts: torch.Tensor, expected_routes: int, group) -> ExchangePlan:
    """All-to-all of the per-destination route counts; the split sizes are needed on the host.

    Every rank also tells every other whether its dispatch dropped routes (an expert id out of range), so
    that all ranks raise together before the row exchange instead of one rank leaving the others waiting.
    """
    send = dest_counts.to(torch.int64)
    dropped = (send.sum() != expected_routes).to(torch.int64)
    message = torch.stack((send, dropped.expand_as(send)), dim=1).contiguous()
    reply = torch.empty_like(message)
    dist.all_to_all_single(reply, message, group=group)
    send_splits = [int(v) for v in send.tolist()]
    recv_splits = [int(v) for v in reply[:, 0].tolist()]
    failed = [rank for rank, flag in enumerate(reply[:, 1].tolist()) if flag]
    if sum(send_splits) != expected_routes and dist.get_rank(group) not in failed:
        failed.append(dist.get_rank(group))
    if failed:
        raise RuntimeError(f"expert-parallel dispatch dropped routes on rank(s) {sorted(failed)}: an expert id was out of range")
    return ExchangePlan(send_splits, recv_splits)


def _all_to_all_rows(rows: torch.Tensor, out_rows: int, send_splits, recv_splits, group) -> torch.Tensor:
    received = torch.empty((out_rows,) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(received, rows.contiguous(), output_split_sizes=recv_splits, input_split_sizes=send_splits, group=group)
    return received


class ExpertParallelMoE:
    """Routed (+ optional shared) expert layer sharded by expert over the ranks of `group`.

    weights: dict with this rank's blocks w13[E/W (+1), 2I, H], w2[E/W (+1), H, I] (int8 or bf16) and, for int8,
    s13 / s2; when has_shared the shared expert is the last local block.
    """

    def __init__(self, weights: dict, experts_global: int, *, has_shared: bool = False, group=None, backend=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.weights = weights
        self.int8 = weights["w13"].dtype == torch.int8
        self.has_shared = bool(has_shared)
        self.experts_global = int(experts_global)
        self.per_rank = validate_expert_split(self.experts_global, self.world, int(weights["w13"].shape[0]), self.has_shared)
        self.backend = backend if backend is not None else CudaBackend()
        self.last_exchange: ExchangePlan | None = None

    def forward(self, x, topk_weights, topk_ids, *, routed_scaling_factor: float = 1.0, swiglu_limit: float | None = None, out=None):
        tokens = x.shape[0]
        if self.has_shared:
            # The reference's convention: the shared expert is expert id E, appended as route K with weight 1.
            shared = torch.full((tokens, 1), self.experts_global, dtype=topk_ids.dtype, device=topk_ids.device)
            topk_ids = torch.cat((topk_ids, shared), dim=1).contiguous()
            ones = torch.ones((tokens, 1), dtype=topk_weights.dtype, device=topk_weights.device)
            topk_weights = torch.cat((topk_weights * routed_scaling_factor, ones), dim=1).contiguous()
        elif routed_scaling_factor != 1.0:
            topk_weights = topk_weights * routed_scaling_factor
        top_k = topk_ids.shape[1]
        prepared = self.backend.dispatch_prepare(x, topk_ids, self.experts_global, self.world,
                                                 self.rank if self.has_shared else -1, self.int8)
        plan = exchange_counts(prepared["dest_counts"], tokens * top_k, self.group)
        self.last_exchange = plan
        rows = _all_to_all_rows(prepared["send_rows"], plan.received, plan.send_splits, plan.recv_splits, self.group)
        meta = prepared["send_expert"].reshape(-1, 1)
        if self.int8:
            meta = torch.cat((meta, prepared["send_scale"].view(torch.int32).to(torch.int64).reshape(-1, 1)), dim=1)
        meta = _all_to_all_rows(meta.contiguous(), plan.received, plan.send_splits, plan.recv_splits, self.group)
        expert = meta[:, 0].contiguous()
        scale = meta[:, 1].to(torch.int32).view(torch.float32).contiguous() if self.int8 else None
        route_rows = self.backend.expert_rows_forward(rows, scale, expert, self.weights, swiglu_limit)
        returned = _all_to_all_rows(route_rows, tokens * top_k, plan.recv_splits, plan.send_splits, self.group)
        return self.backend.combine_finish(returned, prepared["send_order"], topk_weights.to(torch.float32), tokens, top_k,
                                           not self.int8, out)

    __call__ = forward


class PeerMemoryExpertParallelMoE:
    """The same sharded layer with the row exchanges done by the kernels over peer memory (fmoe_ep_peer_*).

    Each rank owns a slab that every other rank of the box maps: the dispatch kernel stores quantised rows straight
    into the expert ranks' slabs and the down GEMM's epilogue stores the fp32 result rows straight back; two flag
    barriers through the same slabs order the stages.  After set-up (one exchange of IPC handles through
    torch.distributed) a forward involves no collective library and no host synchronisation.  Bit-identical to
    ExpertParallelMoE and to the single-GPU forward; with return_dtype=torch.bfloat16 (opt-in) the result rows travel
    back rounded to bf16: half the traffic, outputs within a bf16 step of the exact ones, no longer bit-identical.  tokens_max bounds the tokens any rank passes to forward();
    every rank must call forward() the same number of times.
    """

    def __init__(self, weights: dict, experts_global: int, *, tokens_max: int, top_k: int, has_shared: bool = False, group=None,
                 numerics: int = 0, gate_up_tile: int = 0, down_tile: int = 0, return_dtype: torch.dtype = torch.float32):
        from . import _lib

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.weights = weights
        self.int8 = weights["w13"].dtype == torch.int8
        self.has_shared = bool(has_shared)
        self.experts_global = int(experts_global)
        local_experts, two_inter, hidden = (int(v) for v in weights["w13"].shape)
        self.per_rank = validate_expert_split(self.experts_global, self.world, local_experts, self.has_shared)
        self.top_k = int(top_k) + (1 if self.has_shared else 0)
        self.hidden = hidden
        self.numerics = numerics
        self.tiles = (gate_up_tile, down_tile)
        if return_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("return_dtype must be torch.float32 (bit-identical to one GPU) or torch.bfloat16 (half the return traffic)")
        self.return_dtype = return_dtype
        self.context = _lib.PeerContext(self.world, self.rank, int(tokens_max), self.top_k, hidden, two_inter // 2, local_experts, self.int8,
                                        return_bf16=return_dtype == torch.bfloat16)
        handles = [None] * self.world
        dist.all_gather_object(handles, self.context.ipc_handle(), group=group)
        self.context.connect(handles)
        self.stage_timer = None  # optional _lib.StageTimer: per-kernel CUDA events of the expert stage
        dist.barrier(group=group)  # every rank has mapped every slab before anyone writes

    def forward(self, x, topk_weights, topk_ids, *, routed_scaling_factor: float = 1.0, swiglu_limit: float | None = None, out=None):
        from . import _lib

        tokens = x.shape[0]
        if self.has_shared:
            shared = torch.full((tokens, 1), self.experts_global, dtype=topk_ids.dtype, device=topk_ids.device)
            topk_ids = torch.cat((topk_ids, shared), dim=1)
            ones = torch.ones((tokens, 1), dtype=topk_weights.dtype, device=topk_weights.device)
            topk_weights = torch.cat((topk_weights * routed_scaling_factor, ones), dim=1)
        elif routed_scaling_factor != 1.0:
            topk_weights = topk_weights * routed_scaling_factor
        if topk_ids.shape[1] != self.top_k:
            raise ValueError(f"top_k is {topk_ids.shape[1]}, the context was built for {self.top_k}")
        x = x.contiguous()
        topk_ids = topk_ids.contiguous()
        topk_weights = topk_weights.to(torch.float32).contiguous()
        if out is None:
            out = torch.empty((tokens, self.hidden), dtype=torch.bfloat16, device=x.device)
        config = _lib.Config()
        config.numerics = self.numerics
        config.gate_up_tile, config.down_tile = self.tiles
        config.swiglu_limit = (10.0 if self.int8 else 0.0) if swiglu_limit is None else float(swiglu_limit)
        if self.stage_timer is not None:
            config.stage_timer = self.stage_timer.handle
        context = self.context
        context.dispatch(x, topk_ids, self.experts_global, self.rank if self.has_shared else -1, self.numerics)
        context.experts(self.weights["w13"], self.weights.get("s13"), self.weights["w2"], self.weights.get("s2"), config)
        context.combine(topk_weights, tokens, not self.int8, out)
        return out

    __call__ = forward

    def raise_for_status(self) -> None:
        """Synchronises; raises if the last forward dropped a route (expert id out of range) or a kernel gave up a wait."""
        from . import _lib

        dispatch_error, expert_error = self.context.read_status()
        for where, code in (("dispatch", dispatch_error), ("expert stage", expert_error)):
            if code != 0:
                text = _lib.load().fmoe_last_error().decode("utf-8", "replace")
                raise _lib.FusedMoEError(code, f"expert-parallel {where} reported device-side error {code} on rank {self.rank}: {text}")

    def close(self) -> None:
        self.context.close()


def shard_rows(total: int, world: int, rank: int) -> slice:
    """Contiguous even split of `total` tokens (the first total % world ranks take one more)."""
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return slice(begin, begin + base + (1 if rank < extra else 0))
