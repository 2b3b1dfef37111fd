"""Expert-parallel exchange logic on CPU ranks (gloo, world size 2), with the CPU oracle standing in for
the three device steps.  Checks that the sharded layer returns the single-rank result bit for bit, with and
without the shared expert, and that host-side failures surface on every rank instead of hanging."""
from __future__ import annotations

import os
import socket
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fused_cpp_b200 import ep, synthetic
from oracle import oracle
from tests import cases


class OracleBackend:
    """CPU stand-in for ep.CudaBackend built from the oracle's pieces (test infrastructure only)."""

    def dispatch_prepare(self, x, topk_ids, experts_global, world, shared_rank, int8):
        assert int8
        tokens, top_k = topk_ids.shape
        per_rank = experts_global // world
        flat = topk_ids.reshape(-1)
        dest = torch.where(flat == experts_global, torch.full_like(flat, shared_rank), flat // per_rank)
        valid = (flat >= 0) & ((flat < experts_global) | ((flat == experts_global) & (shared_rank >= 0)))
        order = torch.argsort(torch.where(valid, dest, torch.full_like(dest, world)), stable=True)
        order = order[: int(valid.sum())]
        xq, scale = oracle.quantize_rows(x)
        token = order // top_k
        local = torch.where(flat[order] == experts_global, torch.full_like(flat[order], per_rank), flat[order] % per_rank)
        return {"dest_counts": torch.bincount(dest[valid], minlength=world).to(torch.int32), "send_order": order.to(torch.int32),
                "send_rows": xq[token].contiguous(), "send_scale": scale[token].contiguous(), "send_expert": local.contiguous()}

    def expert_rows_forward(self, rows, scale, expert, weights, swiglu_limit):
        if rows.shape[0] == 0:
            return torch.empty((0, rows.shape[1]), dtype=torch.float32)
        return oracle.w8a8_route_rows(rows, scale, expert, weights["w13"], weights["s13"], weights["w2"], weights["s2"])

    def combine_finish(self, returned, send_order, topk_weights, tokens, top_k, tree_merge, out):
        route_out = torch.empty_like(returned)
        route_out[send_order.long()] = returned
        merge = oracle.merge_bf16_path if tree_merge else oracle.merge_w8a8_path
        return merge(route_out.view(tokens, top_k, -1), topk_weights)


def _by_value(payload):
    """Tensors leave a rank as numpy arrays: a torch tensor put on a multiprocessing queue travels as a handle that
    the receiver has to fetch from the sender, and a rank that has already exited cannot serve it."""
    if isinstance(payload, torch.Tensor):
        return ("tensor", payload.detach().cpu().contiguous().numpy())
    if isinstance(payload, (tuple, list)):
        return type(payload)(_by_value(item) for item in payload)
    return payload


def _from_value(payload):
    if isinstance(payload, tuple) and len(payload) == 2 and isinstance(payload[0], str) and payload[0] == "tensor":
        return torch.from_numpy(payload[1])
    if isinstance(payload, (tuple, list)):
        return type(payload)(_from_value(item) for item in payload)
    return payload


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, scenario, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        import datetime
        try:
            dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
        except Exception as error:  # noqa: BLE001 - the rendezvous itself failed: the runner tries again on a fresh port
            queue.put((rank, "rendezvous", f"{type(error).__name__}: {error}"))
            return
        queue.put((rank, "ok", _by_value(scenario(rank, world))))
    except Exception as error:  # noqa: BLE001
        queue.put((rank, "error", f"{type(error).__name__}: {error}\n{traceback.format_exc()[-600:]}"))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


_RENDEZVOUS_TROUBLE = ("Address already in use", "Connection refused", "Connection reset", "timed out", "Timed out")


def _run_once(scenario, world):
    context = mp.get_context("spawn")
    queue = context.Queue()
    port = _free_port()
    procs = [context.Process(target=_worker, args=(r, world, port, scenario, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    return {rank: (status, _from_value(payload) if status == "ok" else payload) for rank, status, payload in results}


def _run(scenario, world=2):
    # The port is picked before the ranks start, so another process can take it in between; a run whose rendezvous
    # failed (and only that: the scenario never started on that rank) is tried again on a fresh port, twice at most.
    for _ in range(3):
        results = _run_once(scenario, world)
        trouble = [payload for status, payload in results.values()
                   if status == "rendezvous" or (status == "error" and any(t in str(payload) for t in _RENDEZVOUS_TROUBLE))]
        if not trouble:
            break
    return results


def _shard(case, rank, world, shared=None):
    experts = case["w13"].shape[0]
    per = experts // world
    block = slice(rank * per, (rank + 1) * per)
    weights = {k: case[k][block].contiguous() for k in ("w13", "s13", "w2", "s2")}
    if shared is not None:
        weights = {k: torch.cat((weights[k], shared[k][None]), 0) for k in weights}
    rows = ep.shard_rows(case["x"].shape[0], world, rank)
    return weights, rows


def scenario_plain(rank, world):
    case = cases.w8a8_case("tiny")
    weights, rows = _shard(case, rank, world)
    layer = ep.ExpertParallelMoE(weights, 4, backend=OracleBackend())
    out = layer(case["x"][rows], case["topk_weights"][rows], case["topk_ids"][rows])
    return out.view(torch.int16), (rows.start, rows.stop), layer.last_exchange.send_splits


def scenario_shared(rank, world):
    case = cases.w8a8_case("ragged")
    case["topk_ids"] = case["topk_ids"] % 6  # 6 routed experts split over 2 ranks
    for key in ("w13", "s13", "w2", "s2"):
        case[key] = case[key][:6]
    w13, s13, w2, s2 = synthetic.make_int8_expert(144, 80, 99)
    shared = {"w13": w13, "s13": s13, "w2": w2, "s2": s2}
    weights, rows = _shard(case, rank, world, shared)
    layer = ep.ExpertParallelMoE(weights, 6, has_shared=True, backend=OracleBackend())
    out = layer(case["x"][rows], case["topk_weights"][rows], case["topk_ids"][rows], routed_scaling_factor=2.5)
    return out.view(torch.int16), (rows.start, rows.stop), None


def scenario_bad_id(rank, world):
    case = cases.w8a8_case("tiny")
    weights, rows = _shard(case, rank, world)
    if rank == 1:
        case["topk_ids"][rows.start, 0] = 17
    layer = ep.ExpertParallelMoE(weights, 4, backend=OracleBackend())
    layer(case["x"][rows], case["topk_weights"][rows], case["topk_ids"][rows])
    return None


def scenario_bad_split(rank, world):
    case = cases.w8a8_case("tiny")
    weights, _ = _shard(case, rank, world)
    ep.ExpertParallelMoE(weights, 5, backend=OracleBackend())
    return None


def test_ep_two_ranks_match_single_rank_bit_for_bit():
    results = _run(scenario_plain)
    case = cases.w8a8_case("tiny")
    expected = oracle.w8a8_forward(case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"], case["topk_ids"])
    for rank, (status, payload) in results.items():
        assert status == "ok", payload
        out, (begin, end), splits = payload
        assert torch.equal(out, expected[begin:end].view(torch.int16)), f"rank {rank}"
        assert sum(splits) == (end - begin) * 2


def test_ep_with_shared_expert_matches_single_rank():
    results = _run(scenario_shared)
    case = cases.w8a8_case("ragged")
    ids = case["topk_ids"] % 6
    w13, s13, w2, s2 = synthetic.make_int8_expert(144, 80, 99)
    tokens = ids.shape[0]
    full_ids = torch.cat((ids, torch.full((tokens, 1), 6)), 1)
    full_w = torch.cat((case["topk_weights"] * 2.5, torch.ones((tokens, 1))), 1)
    expected = oracle.w8a8_forward(case["x"], torch.cat((case["w13"][:6], w13[None])), torch.cat((case["s13"][:6], s13[None])),
                                   torch.cat((case["w2"][:6], w2[None])), torch.cat((case["s2"][:6], s2[None])), full_w, full_ids)
    for rank, (status, payload) in results.items():
        assert status == "ok", payload
        out, (begin, end), _ = payload
        assert torch.equal(out, expected[begin:end].view(torch.int16)), f"rank {rank}"


def test_ep_out_of_range_id_raises_on_every_rank():
    results = _run(scenario_bad_id)
    for rank, (status, payload) in results.items():
        assert status == "error" and "dropped routes on rank(s) [1]" in payload, (rank, payload)


def test_ep_rejects_uneven_expert_split():
    results = _run(scenario_bad_split)
    for rank, (status, payload) in results.items():
        assert status == "error" and "do not split evenly" in payload


def test_shard_rows_covers_everything():
    for total, world in ((64, 8), (7, 3), (2, 4), (0, 2)):
        pieces = [ep.shard_rows(total, world, r) for r in range(world)]
        assert pieces[0].start == 0 and pieces[-1].stop == total
        assert all(a.stop == b.start for a, b in zip(pieces, pieces[1:]))
    with pytest.raises(ValueError, match="expected 3"):
        ep.validate_expert_split(4, 2, 2, True)
