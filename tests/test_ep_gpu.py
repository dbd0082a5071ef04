"""GPU tests of expert parallelism.  The regroup / row-move kernels run on one GPU; the two-rank
layer (NCCL all-to-all over NVLink) needs two GPUs and is skipped otherwise.  The two-rank result
must equal the one-GPU layer bit for bit: every row goes through the same kernels, only on
another GPU."""
import os
import socket
import traceback

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from netra_kernel_b200 import synth
from netra_kernel_b200.ep import ExpertParallelMoELayer, ExpertParallelPlan, shard_expert_weights

pytestmark = pytest.mark.gpu


def test_regroup_and_move_rows_kernels_match_the_host_index_math():
    from netra_kernel_b200 import abi
    lib = abi.load()
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(3)
    for world, e_l in ((2, 128), (8, 32), (4, 64)):
        plan = ExpertParallelPlan(world, 0)
        counts = torch.randint(0, 40, (world, e_l), generator=g, dtype=torch.int32)
        counts[:, 5] = 0                                            # an expert nobody sends to
        want_index, want_off = plan.regroup_reference(counts, extra_rows=77)
        total = int(counts.sum())
        src_base = torch.zeros(world * e_l, dtype=torch.int32, device=dev)
        dst_base = torch.zeros_like(src_base)
        offsets = torch.zeros(e_l + 2, dtype=torch.int32, device=dev)
        index = torch.full((total + 16,), -1, dtype=torch.int32, device=dev)
        abi.check(lib.netra_ep_regroup_launch(src_base.data_ptr(), dst_base.data_ptr(), offsets.data_ptr(), index.data_ptr(),
                                              counts.to(dev).data_ptr(), world, e_l, 77, total + 16, None), "regroup")
        torch.cuda.synchronize()
        assert torch.equal(offsets.cpu(), want_off) and torch.equal(index[:total].cpu(), want_index)
        assert torch.all(index[total:] == -1)
        rows = torch.randint(0, 255, (total, 2048), dtype=torch.uint8, device=dev)
        scattered = torch.zeros_like(rows)
        abi.check(lib.netra_moe_move_rows_launch(scattered.data_ptr(), rows.data_ptr(), index.data_ptr(), total, 2048, 1, None), "scatter")
        back = torch.zeros_like(rows)
        abi.check(lib.netra_moe_move_rows_launch(back.data_ptr(), scattered.data_ptr(), index.data_ptr(), total, 2048, 0, None), "gather")
        torch.cuda.synchronize()
        assert torch.equal(scattered[want_index.long().to(dev)], rows) and torch.equal(back, rows)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ep_rank(rank, world, port, tokens, results):
    try:
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        weights = synth.make_expert_weights(0)
        hidden, router_w, bias = synth.make_activations(tokens, 0.6, seed=2)
        plan = ExpertParallelPlan(world, rank)
        local = tuple(t.to(dev) for t in shard_expert_weights(weights, plan))
        t_l = tokens // world
        layer = ExpertParallelMoELayer(plan, router_w.to(dev), *local, max_local_tokens=t_l, router_bias=bias.to(dev))
        mine = hidden[rank * t_l:(rank + 1) * t_l].to(dev)
        out = layer(mine)
        out2 = layer(mine)                                   # a second call reuses every buffer
        torch.cuda.synchronize()
        layer.check_status()
        results[rank] = {"out": out.cpu(), "same": bool(torch.equal(out, out2)), "recv": layer.last_splits.recv}
        if rank == 0:                                        # one-GPU layer over all tokens, same weights
            from netra_kernel_b200.moe import RoutedMoELayer
            full = RoutedMoELayer(router_w.to(dev), *(t.to(dev) for t in weights), tokens, bias.to(dev))
            results["ref"] = full(hidden.to(dev)).cpu()
            full.check_status()
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        results[rank] = "error: " + traceback.format_exc()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_expert_parallel_layer_equals_the_one_gpu_layer():
    world, tokens = 2, 512
    manager = mp.Manager()
    results = manager.dict()
    port = _free_port()
    procs = [mp.get_context("spawn").Process(target=_ep_rank, args=(r, world, port, tokens, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
        if p.is_alive():
            p.kill()
    res = dict(results)
    assert all(isinstance(res.get(r), dict) for r in range(world)), res
    got = torch.cat([res[r]["out"] for r in range(world)])
    assert all(res[r]["same"] for r in range(world))
    assert torch.equal(got.view(torch.int16), res["ref"].view(torch.int16))
    assert sum(res[0]["recv"]) + sum(res[1]["recv"]) == tokens * 8
