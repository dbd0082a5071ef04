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
    for world, e_l, slot, shared_first in ((2, 128, 0, False), (8, 32, 0, True), (4, 64, 1600, True), (2, 128, 3000, False), (8, 32, 512, True)):
        plan = ExpertParallelPlan(world, 0)
        counts = torch.randint(0, 40, (world, e_l), generator=g, dtype=torch.int32)
        counts[:, 5] = 0                                            # an expert nobody sends to
        want_index, want_off = plan.regroup_reference(counts, extra_rows=77, slot_rows=slot, shared_first=shared_first)
        total = int((want_index >= 0).sum())                        # rows delivered (a slot that is too small truncates)
        rows_in = world * slot if slot else total
        src_base = torch.zeros(world * e_l, dtype=torch.int32, device=dev)
        dst_base = torch.zeros_like(src_base)
        offsets = torch.zeros(e_l + 2, dtype=torch.int32, device=dev)
        index_rows = rows_in if slot else rows_in + 16                 # without slots the tail past the routed rows is -1
        index = torch.full((index_rows,), 12345, dtype=torch.int32, device=dev)
        abi.check(lib.netra_ep_regroup_launch(src_base.data_ptr(), dst_base.data_ptr(), offsets.data_ptr(), index.data_ptr(),
                                              counts.to(dev).data_ptr(), world, e_l, 77, index_rows, slot, int(shared_first), None),
                  "regroup")
        torch.cuda.synchronize()
        assert torch.equal(offsets.cpu(), want_off)
        assert torch.equal(index[:rows_in].cpu(), want_index) and torch.all(index[rows_in:] == -1)
        # rows with a 2112-byte pitch on the source-major side, 2048-byte rows on the expert-major side
        rows = torch.randint(0, 255, (rows_in, 2112), dtype=torch.uint8, device=dev)
        block = torch.zeros(total + 77, 2048, dtype=torch.uint8, device=dev)
        abi.check(lib.netra_moe_move_rows_launch(block.data_ptr(), rows.data_ptr(), index.data_ptr(), rows_in, 2048, 2048, 2112, 0, 0, 1, None),
                  "scatter")
        tail = torch.zeros(total + 77, 64, dtype=torch.uint8, device=dev)
        abi.check(lib.netra_moe_move_rows_launch(tail.data_ptr(), rows.data_ptr(), index.data_ptr(), rows_in, 64, 64, 2112, 0, 2048, 1, None),
                  "scatter tail")
        back = torch.zeros(rows_in, 2048, dtype=torch.uint8, device=dev)
        abi.check(lib.netra_moe_move_rows_launch(back.data_ptr(), block.data_ptr(), index.data_ptr(), rows_in, 2048, 2048, 2048, 0, 0, 0, None),
                  "gather")
        torch.cuda.synchronize()
        used = (want_index >= 0).to(dev)
        where = want_index.long().to(dev)[used]
        assert torch.equal(block[where], rows[used][:, :2048]) and torch.equal(tail[where], rows[used][:, 2048:])
        assert torch.equal(back[used], rows[used][:, :2048]) and torch.all(back[~used] == 0)


def test_pack_and_unpack_slot_rows():
    from netra_kernel_b200 import abi
    lib = abi.load()
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(5)
    world, e_l, slot = 4, 64, 96
    counts = torch.randint(0, 3, (world * e_l,), generator=g, dtype=torch.int32)
    offsets = torch.zeros(world * e_l + 2, dtype=torch.int32)
    offsets[1:-1] = torch.cumsum(counts, 0)
    pairs = int(offsets[-2])
    offsets[-1] = pairs + 10
    a = torch.randint(0, 255, (pairs, 2048), dtype=torch.uint8, device=dev)
    a_s = torch.rand(pairs, 16, device=dev)
    send = torch.zeros(world * slot, 2112, dtype=torch.uint8, device=dev)
    overflow = torch.zeros(1, dtype=torch.int32, device=dev)
    abi.check(lib.netra_ep_pack_rows_launch(send.data_ptr(), a.data_ptr(), a_s.data_ptr(), offsets.to(dev).data_ptr(), world, e_l, slot,
                                            overflow.data_ptr(), None), "pack")
    down = torch.zeros(pairs, 2048, dtype=torch.float32, device=dev)
    back = torch.randn(world * slot, 2048, device=dev)
    abi.check(lib.netra_ep_unpack_rows_launch(down.data_ptr(), back.data_ptr(), offsets.to(dev).data_ptr(), world, e_l, slot, None), "unpack")
    torch.cuda.synchronize()
    per_rank = counts.view(world, e_l).sum(1).tolist()
    assert max(per_rank) <= slot and int(overflow) == 0
    pos = 0
    for r, n in enumerate(per_rank):
        got = send[r * slot:r * slot + n]
        assert torch.equal(got[:, :2048], a[pos:pos + n])
        assert torch.equal(got[:, 2048:].contiguous().view(torch.float32), a_s[pos:pos + n])
        assert torch.equal(down[pos:pos + n], back[r * slot:r * slot + n])
        pos += n
    # a slot that is too small is reported, and nothing is written past it
    small = min(per_rank) - 1
    send2 = torch.zeros(world * small + 8, 2112, dtype=torch.uint8, device=dev)
    abi.check(lib.netra_ep_pack_rows_launch(send2.data_ptr(), a.data_ptr(), a_s.data_ptr(), offsets.to(dev).data_ptr(), world, e_l, small,
                                            overflow.data_ptr(), None), "pack small")
    torch.cuda.synchronize()
    assert int(overflow) == max(per_rank) and torch.all(send2[world * small:] == 0)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ep_rank(rank, world, port, tokens, exchange, results):
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
        layer = ExpertParallelMoELayer(plan, router_w.to(dev), *local, max_local_tokens=t_l, router_bias=bias.to(dev),
                                       exchange=exchange, slot_rows=t_l * 8)   # skewed routing: size the slots for the worst case
        mine = hidden[rank * t_l:(rank + 1) * t_l].to(dev)
        out = layer(mine)
        out2 = layer(mine)                                   # a second call reuses every buffer
        torch.cuda.synchronize()
        layer.check_status()
        results[rank] = {"out": out.cpu(), "same": bool(torch.equal(out, out2)), "recv": layer.last_splits.recv if exchange == "exact" else None}
        if exchange == "fixed":                              # a slot too small for the routed rows is reported, not hidden
            tiny = ExpertParallelMoELayer(plan, router_w.to(dev), *local, max_local_tokens=t_l, router_bias=bias.to(dev),
                                          exchange="fixed", slot_rows=64)
            tiny(mine)
            torch.cuda.synchronize()
            try:
                tiny.check_status()
                results[rank] = dict(results[rank], overflow_reported=False)
            except Exception as exc:
                results[rank] = dict(results[rank], overflow_reported="slot holds 64" in str(exc))
            tiny.close()
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
@pytest.mark.parametrize("exchange", ["fixed", "exact"])
def test_two_gpu_expert_parallel_layer_equals_the_one_gpu_layer(exchange):
    world, tokens = 2, 512
    manager = mp.Manager()
    results = manager.dict()
    port = _free_port()
    procs = [mp.get_context("spawn").Process(target=_ep_rank, args=(r, world, port, tokens, exchange, results)) for r in range(world)]
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
    if exchange == "exact":
        assert sum(res[0]["recv"]) + sum(res[1]["recv"]) == tokens * 8
    else:
        assert all(res[r]["overflow_reported"] for r in range(world))
