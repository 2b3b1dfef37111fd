"""Expert-parallel layer on GPUs, both exchanges (NCCL all-to-all and the kernels' own stores into peer memory)
against the single-GPU forward (bit-exact), on a one-rank NCCL group always and on two GPUs when the box has them."""
from __future__ import annotations

import datetime
import os
import tempfile
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fused_cpp_b200 import _lib, ep, synthetic
from tests import cases

pytestmark = pytest.mark.gpu



def _single_gpu(case, device, shared=None, scaling=1.0):
    c = {k: v.to(device) for k, v in case.items()}
    ids, w = c["topk_ids"], c["topk_weights"]
    w13, s13, w2, s2 = c["w13"], c.get("s13"), c["w2"], c.get("s2")
    if shared is not None:
        tokens = ids.shape[0]
        ids = torch.cat((ids, torch.full((tokens, 1), w13.shape[0], dtype=torch.int64, device=device)), 1)
        w = torch.cat((w * scaling, torch.ones((tokens, 1), device=device)), 1)
        w13 = torch.cat((w13, shared["w13"][None].to(device)))
        w2 = torch.cat((w2, shared["w2"][None].to(device)))
        if s13 is not None:
            s13 = torch.cat((s13, shared["s13"][None].to(device)))
            s2 = torch.cat((s2, shared["s2"][None].to(device)))
    return _lib.moe_forward(c["x"], w13, w2, w.contiguous(), ids.contiguous(), s13=s13, s2=s2).out


def _ep_worker(rank, world, store_path, kind, with_shared, impl, queue):
    try:
        os.environ.update(NCCL_NVLS_ENABLE="0")
        device = torch.device("cuda", rank)
        torch.cuda.set_device(device)
        # Rendezvous through a file: a TCP port picked by the parent can be taken again before rank 0 listens on it.
        dist.init_process_group("nccl", init_method=f"file://{store_path}", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=120), device_id=device)
        case = cases.w8a8_case("wide") if kind == "int8" else cases.bf16_case("top8")
        experts = case["w13"].shape[0]
        if kind == "int8" and experts % world:
            experts = experts - experts % world
        keys = ("w13", "s13", "w2", "s2") if kind == "int8" else ("w13", "w2")
        case["topk_ids"] = case["topk_ids"] % experts
        for k in keys:
            case[k] = case[k][:experts]
        shared = None
        if with_shared:
            hidden, inter = case["x"].shape[1], case["w13"].shape[1] // 2
            if kind == "int8":
                a, b, c, d = synthetic.make_int8_expert(hidden, inter, 4242)
                shared = {"w13": a, "s13": b, "w2": c, "s2": d}
            else:
                a, c = synthetic.make_bf16_expert(hidden, inter, 4242, 0.05)
                shared = {"w13": a, "w2": c}
        per = experts // world
        weights = {k: case[k][rank * per:(rank + 1) * per].to(device) for k in keys}
        if shared is not None:
            weights = {k: torch.cat((weights[k], shared[k][None].to(device))) for k in keys}
        rows = ep.shard_rows(case["x"].shape[0], world, rank)
        if impl in ("peer", "peer_bf16"):
            most = max(ep.shard_rows(case["x"].shape[0], world, r).stop - ep.shard_rows(case["x"].shape[0], world, r).start for r in range(world))
            layer = ep.PeerMemoryExpertParallelMoE(weights, experts, tokens_max=most, top_k=case["topk_ids"].shape[1], has_shared=with_shared,
                                                   return_dtype=torch.bfloat16 if impl == "peer_bf16" else torch.float32)
        else:
            layer = ep.ExpertParallelMoE(weights, experts, has_shared=with_shared)
        expected = _single_gpu(case, device, shared, 1.5)[rows]
        same = True
        for _ in range(1 if impl == "nccl" else 8):  # later calls reuse the slabs and the barrier epochs
            out = layer(case["x"][rows].to(device), case["topk_weights"][rows].to(device), case["topk_ids"][rows].to(device),
                        routed_scaling_factor=1.5 if with_shared else 1.0)
            if impl == "peer_bf16":
                # Result rows rounded to bf16 on the way back: close to the exact result (relative L2 within 5e-3,
                # every element within two bf16 steps of its magnitude plus a small absolute term), not bit-equal.
                difference = (out.float() - expected.float()).abs()
                relative_l2 = float(difference.norm() / expected.float().norm())
                bound = expected.float().abs() * 2.0 ** -6 + 1e-2 * expected.float().abs().mean()
                same = same and relative_l2 <= 5e-3 and bool((difference <= bound).all())
            else:
                same = same and torch.equal(out.view(torch.int16), expected.view(torch.int16))
        if impl != "nccl":
            layer.raise_for_status()
            torch.cuda.synchronize()
            dist.barrier()
            layer.close()
        queue.put((rank, "ok" if same else "mismatch", float((out.float() - expected.float()).abs().max())))
    except Exception as error:  # noqa: BLE001
        queue.put((rank, "error", f"{type(error).__name__}: {error}\n{traceback.format_exc()[-800:]}"))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _run_ep(world, kind, with_shared, impl="nccl"):
    context = mp.get_context("spawn")
    queue = context.Queue()
    with tempfile.TemporaryDirectory() as folder:
        store_path = os.path.join(folder, "rendezvous")
        procs = [context.Process(target=_ep_worker, args=(r, world, store_path, kind, with_shared, impl, queue)) for r in range(world)]
        for p in procs:
            p.start()
        results = [queue.get(timeout=300) for _ in procs]
        for p in procs:
            p.join(timeout=60)
    for rank, status, detail in results:
        assert status == "ok", (rank, status, detail)


@pytest.mark.parametrize("impl", ["nccl", "peer", "peer_bf16"])
@pytest.mark.parametrize("kind", ["int8", "bf16"])
@pytest.mark.parametrize("with_shared", [False, True], ids=["routed", "routed+shared"])
def test_ep_one_rank_equals_plain_forward(cuda_device, kind, with_shared, impl):
    """World size 1: every route is 'sent' to the own rank, so this isolates the CUDA entry points."""
    _run_ep(1, kind, with_shared, impl)


@pytest.mark.parametrize("impl", ["nccl", "peer", "peer_bf16"])
@pytest.mark.parametrize("kind", ["int8", "bf16"])
@pytest.mark.parametrize("with_shared", [False, True], ids=["routed", "routed+shared"])
def test_ep_two_gpus_equal_single_gpu(cuda_device, kind, with_shared, impl):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run_ep(2, kind, with_shared, impl)
