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

import json
import os
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
                raise _lib.FusedMoEError(code, f"expert-parallel {where} reported device-side error {code} on rank {self.rank}")

    def close(self) -> None:
        self.context.close()


def shard_rows(total: int, world: int, rank: int) -> slice:
    """Contiguous even split of `total` tokens (the first total % world ranks take one more)."""
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return slice(begin, begin + base + (1 if rank < extra else 0))


# ---- multi-GPU benchmark leg (called by bench.py under torchrun) -----------------------------------

def bench_main(args, workloads: dict, seed: int, peaks: dict) -> None:
    from . import _lib, synthetic

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    try:
        if not _lib.device_supported():
            raise SystemExit("bench.py needs compute-capability-10.x GPUs")
        hidden, inter, experts, top_k = args.hidden, args.inter, args.experts, args.top_k
        lines = []
        for entry in [args.workload] + ([] if args.no_points else list(args.ep_points)):
            name, _, option = entry.partition(":")  # "workload:bf16_return" = the same workload with the compact return
            spec = workloads[name]
            lines.append(_bench_one(name, spec, args, rank, world, device, hidden, inter, experts, top_k, seed, peaks,
                                    has_shared=spec.get("shared", False), bf16_return=option == "bf16_return"))
        if rank == 0:
            head = lines[0]
            head["points"] = lines[1:]
            print(json.dumps(head), flush=True)
    finally:
        dist.destroy_process_group()


def _bench_one(name, spec, args, rank, world, device, hidden, inter, experts, top_k, seed, peaks, has_shared, bf16_return=False):
    from . import synthetic

    kind, tokens = spec["kind"], spec["tokens"]
    per_rank = experts // world
    generator = torch.Generator(device=device).manual_seed(seed + 2 + rank)
    local = per_rank + (1 if has_shared else 0)
    if kind == "int8":
        weights = {"w13": torch.randint(-127, 128, (local, 2 * inter, hidden), generator=generator, dtype=torch.int8, device=device),
                   "w2": torch.randint(-127, 128, (local, hidden, inter), generator=generator, dtype=torch.int8, device=device),
                   "s13": (torch.rand((local, 2 * inter), generator=generator, device=device) * 1.5 + 0.5) / (127.0 * hidden ** 0.5),
                   "s2": (torch.rand((local, hidden), generator=generator, device=device) * 1.5 + 0.5) / (127.0 * inter ** 0.5)}
    else:
        weights = {"w13": torch.empty((local, 2 * inter, hidden), dtype=torch.bfloat16, device=device).normal_(0, 0.02, generator=generator),
                   "w2": torch.empty((local, hidden, inter), dtype=torch.bfloat16, device=device).normal_(0, 0.02, generator=generator)}
    topk_w, topk_ids = synthetic.make_routing(tokens, experts, top_k, seed, spec.get("skew", False))
    x = synthetic.make_activations(tokens, hidden, seed + 1)
    mine = shard_rows(tokens, world, rank)
    x_host, w_host, ids_host = x[mine].contiguous(), topk_w[mine].contiguous(), topk_ids[mine].contiguous()
    xd, wd, idd = x_host.to(device), w_host.to(device), ids_host.to(device)
    local_max = (tokens + world - 1) // world
    if getattr(args, "ep_impl", "peer") == "peer":
        layer = PeerMemoryExpertParallelMoE(weights, experts, tokens_max=local_max, top_k=top_k, has_shared=has_shared,
                                            return_dtype=torch.bfloat16 if bf16_return else torch.float32)
        exchange = "rows stored by the dispatch kernel and the down-GEMM epilogue into peer memory over NVLink, flag barriers in the same slabs"
        if bf16_return:
            exchange += "; result rows returned as bf16 (opt-in: half the return traffic, outputs within a bf16 step, not bit-identical)"
    else:
        layer = ExpertParallelMoE(weights, experts, has_shared=has_shared)
        exchange = "NCCL all-to-all dispatch/combine"
    kwargs = {"swiglu_limit": 10.0} if kind == "int8" else {}

    def step():
        return layer(xd, wd, idd, **kwargs)

    def timed(fn, steps, warmup, sampler=None):
        if sampler is not None:
            sampler.prepare()
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler is not None:
            sampler.start()
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        clocks = sampler.stop() if sampler is not None else None
        dist.barrier()
        elapsed = torch.tensor([start.elapsed_time(stop) / steps], device=device)
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        return float(elapsed.item()), clocks

    # The forward makes no host read and calls no collective library, so one step (kernels, flag barriers included)
    # is captured into a CUDA graph and the timed region replays it; every rank replays the same sequence.  Eager
    # launches are timed as well (eager_ms_per_step).
    launch_mode = "eager"
    replay = step
    graph = None
    if isinstance(layer, PeerMemoryExpertParallelMoE) and os.environ.get("FUSED_CPP_MOE_EP_GRAPH", "1") != "0":
        try:
            side = torch.cuda.Stream(device=device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            replay = graph.replay
            launch_mode = "cuda_graph_replay"
        except Exception as error:  # noqa: BLE001
            launch_mode = f"eager (graph capture failed: {type(error).__name__})"
            replay = step
    captured = torch.tensor([1 if launch_mode == "cuda_graph_replay" else 0], device=device)
    dist.all_reduce(captured, op=dist.ReduceOp.MIN)
    if int(captured.item()) == 0:
        replay = step
        if launch_mode == "cuda_graph_replay":
            launch_mode = "eager (graph capture failed on another rank)"
    sampler_class = getattr(args, "clock_sampler", None)
    ms, clocks = timed(replay, args.steps, args.warmup, sampler_class(device.index) if (sampler_class and rank == 0) else None)
    eager_ms = ms
    if replay is not step:
        # Both ways of launching are timed under the same rules; the line reports the faster one as `value`
        # (with few ranks the eager launches already keep the GPU busy and the captured collectives cost more).
        graph_ms = ms
        eager_ms, eager_clocks = timed(step, args.steps, args.warmup, sampler_class(device.index) if (sampler_class and rank == 0) else None)
        if eager_ms < graph_ms:
            ms, clocks, launch_mode = eager_ms, eager_clocks, f"eager (cuda_graph_replay: {graph_ms:.4f} ms)"

    # Per-kernel durations of this rank's expert stage (CUDA events around every stage, a second timed pass).
    roofline = None
    stage_ms = None
    if isinstance(layer, PeerMemoryExpertParallelMoE) and getattr(args, "roofline", None) is not None:
        from . import _lib

        timer = _lib.StageTimer(args.steps)
        layer.stage_timer = timer
        for _ in range(args.steps):
            step()
        torch.cuda.synchronize()
        layer.stage_timer = None
        stage_ms = {stage: 0.0 for stage in _lib.STAGES}
        for call in range(timer.calls):
            for stage, value in timer.read(call).items():
                stage_ms[stage] += value / timer.calls
        timer.close()
        # Algorithmic work of this rank's gate_up launch: the weights of its experts that the batch hits, once,
        # plus the rows it receives in and their SwiGLU rows out.
        owner = topk_ids // per_rank
        local_ids = topk_ids[owner == rank]
        rows = int(local_ids.numel()) + (x_host.shape[0] if has_shared else 0)
        active = int(local_ids.unique().numel()) + (1 if has_shared else 0)
        b = 1 if kind == "int8" else 2
        nbytes = active * 2 * inter * hidden * b + rows * hidden * b + rows * inter * 2 + (active * 2 * inter * 4 + rows * 4 if kind == "int8" else 0)
        roofline = args.roofline(kind, float(nbytes), 2.0 * rows * 2 * inter * hidden, stage_ms["gate_up"], peaks, None)
        roofline["scope"] = f"rank 0 of {world}: {active} active local experts, {rows} received rows"
        dist.barrier()

    x_pin, w_pin, ids_pin = x_host.pin_memory(), w_host.pin_memory(), ids_host.pin_memory()
    out_pin = torch.empty((x_host.shape[0], hidden), dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        out = layer(x_pin.to(device, non_blocking=True), w_pin.to(device, non_blocking=True), ids_pin.to(device, non_blocking=True), **kwargs)
        out_pin.copy_(out, non_blocking=True)

    e2e_ms, _ = timed(e2e_step, args.steps, args.warmup)
    # Cross-check at benchmark scale: the peer-memory forward against the NCCL all-to-all form on the same batch
    # (each is bit-identical to the single-GPU forward in the tests; here they must agree with each other).
    parity = None
    if isinstance(layer, PeerMemoryExpertParallelMoE):
        other = ExpertParallelMoE(weights, experts, has_shared=has_shared)
        expected = other(xd, wd, idd, **kwargs)
        got = layer(xd, wd, idd, **kwargs)
        if bf16_return:
            error = float((got.float() - expected.float()).norm() / expected.float().norm().clamp_min(1e-30))
            agree = torch.tensor([1 if error <= 5e-3 else 0], device=device)
            parity = "relative L2 to the NCCL all-to-all form on this batch <= 5e-3"
        else:
            agree = torch.tensor([1 if torch.equal(got.view(torch.int16), expected.view(torch.int16)) else 0], device=device)
            parity = "bit-identical to the NCCL all-to-all form on this batch, every rank"
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        if int(agree.item()) != 1:
            raise RuntimeError(f"{name}: the peer-memory forward disagrees with the NCCL form on at least one rank")
        del other, expected, got
    # Every rank is done with every slab before any of them is unmapped and freed.
    torch.cuda.synchronize()
    dist.barrier()
    replay = None
    graph = None
    if hasattr(layer, "close"):
        layer.close()
    local_tokens = x_host.shape[0]
    # Kernels of this library per forward on one rank, peer form: route build by global expert (1 kernel up to 1024
    # routes, else 3), count barrier, layout, dispatch, barrier | work items, output addresses, gate_up (+ requantise),
    # down, barrier | merge.  (The NCCL form has no barriers but a route build, gathers and a scatter on the expert side.)
    routes_local = local_tokens * (top_k + (1 if has_shared else 0))
    launches_per_step = ((1 if routes_local <= 1024 else 3) + 4) + (5 + (1 if kind == "int8" else 0)) + 1
    work = synthetic.algorithmic_work(synthetic.MoEShape(tokens, hidden, inter, experts, top_k), topk_ids, 1 if kind == "int8" else 2,
                                      shared=has_shared)
    return {
        "metric": "moe_layer_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16" if kind == "bf16" else "int8(w8a8)", "data": "synthetic",
        "config": {"workload": name, "tokens": tokens, "hidden": hidden, "inter": inter, "experts": experts, "top_k": top_k,
                   "shared_expert": has_shared, "parallelism": f"ep{world}: experts and tokens split evenly, {exchange}",
                   "l2": "inputs larger than L2: every rank streams its experts' weights each step"},
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": local_tokens * hidden * 2 + local_tokens * top_k * 12,
                "d2h_bytes_per_step": local_tokens * hidden * 2},
        "gpu_launches": launches_per_step * args.steps, "clocks": clocks, "roofline": roofline, "cpu_baseline": None,
        "launch_mode": launch_mode, "eager_ms_per_step": eager_ms, "parity": parity,
        "stage_ms_rank0": {k: round(v, 5) for k, v in stage_ms.items()} if stage_ms else None,
        "layer": {"algorithmic_bytes": work["bytes"], "ops": work["ops"],
                  "hbm_gbs_aggregate": work["bytes"] / (ms * 1e-3) / 1e9, "tops_aggregate": work["ops"] / (ms * 1e-3) / 1e12},
    }
