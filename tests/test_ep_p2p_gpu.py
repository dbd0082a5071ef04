"""GPU tests of expert parallelism over peer memory (netra_ep_layer_*).

On one GPU several ranks are emulated in one process: each rank has its own layer object, weights
shard, window and workspace, and the ranks' calls are issued stage by stage on ONE stream, so every
wait finds its flags already raised (kernels that wait on one another are never in flight
together).  The result must equal the one-GPU layer bit for bit.  The two-GPU test runs one process
per GPU with CUDA IPC windows, directly and as a replayed CUDA graph.
"""
import os
import socket
import traceback

import pytest
import torch
import torch.multiprocessing as mp

from netra_kernel_b200 import synth
from netra_kernel_b200.ep import (ExpertParallelPlan, PeerExpertParallelLayer, default_row_capacity, ep_sizes,
                                  shard_expert_weights)

pytestmark = pytest.mark.gpu


def _aligned_window(nbytes, dev):
    buf = torch.zeros(nbytes + 1024, dtype=torch.uint8, device=dev)
    return buf, (buf.data_ptr() + 1023) // 1024 * 1024


def _emulated_ranks(world, tokens, weights, router_w, bias, dev, row_capacity=None, timeout_s=2.0):
    t_l = tokens // world
    cap = row_capacity or default_row_capacity(world, t_l)
    _, win_bytes = ep_sizes(world, t_l, cap)
    keep, ptrs = [], []
    for _ in range(world):
        buf, ptr = _aligned_window(win_bytes, dev)
        keep.append(buf)
        ptrs.append(ptr)
    layers = []
    for r in range(world):
        plan = ExpertParallelPlan(world, r)
        local = tuple(t.to(dev) for t in shard_expert_weights(weights, plan))
        layers.append(PeerExpertParallelLayer(plan, router_w, *local, max_local_tokens=t_l, router_bias=bias, row_capacity=cap,
                                              wait_timeout_s=timeout_s, windows=ptrs))
    return layers, keep


def _interleaved_call(layers, hidden_parts, outs):
    for stage in range(layers[0].stage_count):
        for r, layer in enumerate(layers):
            layer.launch_stage(stage, hidden_parts[r], outs[r])


@pytest.mark.parametrize("world,tokens,alpha", [(1, 64, 0.0), (2, 256, 0.6), (4, 512, 0.0), (8, 2048, 0.3), (2, 4096, 0.3)])
def test_emulated_ranks_equal_the_one_gpu_layer(expert_weights, world, tokens, alpha):
    from netra_kernel_b200.moe import RoutedMoELayer
    dev = torch.device("cuda", 0)
    hidden, router_w, bias = synth.make_activations(tokens, alpha or None, seed=4)
    hidden, router_w = hidden.to(dev), router_w.to(dev)
    bias = bias.to(dev) if bias is not None else None
    shared_w = torch.rand(tokens, device=dev) + 0.5
    layers, keep = _emulated_ranks(world, tokens, expert_weights, router_w, bias, dev)
    t_l = tokens // world
    parts = [hidden[r * t_l:(r + 1) * t_l].contiguous() for r in range(world)]
    outs = [torch.zeros_like(p) for p in parts]
    # per-rank shared weights are passed through launch_stage's optional argument
    for call in range(2):                                           # the second call reuses every buffer and flag
        for stage in range(layers[0].stage_count):
            for r, layer in enumerate(layers):
                layer.launch_stage(stage, parts[r], outs[r], shared_w[r * t_l:(r + 1) * t_l].contiguous())
        torch.cuda.synchronize()
        for layer in layers:
            layer.check_status()
        if call == 0:
            first = torch.cat(outs).clone()
    full = RoutedMoELayer(router_w, *(t.to(dev) for t in expert_weights), tokens, bias)
    want = full(hidden, shared_w)
    torch.cuda.synchronize()
    full.check_status()
    got = torch.cat(outs)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert torch.equal(first.view(torch.int16), want.view(torch.int16))
    for layer in layers:
        layer.close()
    full.close()


@pytest.mark.parametrize("world,tokens,alpha", [(1, 1024, 0.0), (2, 4096, 0.3), (4, 2048, 0.6), (8, 2048, 0.0)])
def test_emulated_ranks_with_fp16_partial_rows_equal_the_one_gpu_layer(expert_weights, world, tokens, alpha):
    """The prefill contract across ranks: the block's down rows as FP16 partials, sent home by the return pass in the
    receiver's panel layout, reduced by the FP16 reducer - bit for bit the one-GPU layer with the same setting."""
    from netra_kernel_b200.moe import RoutedMoELayer
    dev = torch.device("cuda", 0)
    hidden, router_w, bias = synth.make_activations(tokens, alpha or None, seed=9)
    hidden, router_w = hidden.to(dev), router_w.to(dev)
    bias = bias.to(dev) if bias is not None else None
    layers, keep = _emulated_ranks(world, tokens, expert_weights, router_w, bias, dev)
    for layer in layers:
        layer.set_partial_format(1)
    t_l = tokens // world
    parts = [hidden[r * t_l:(r + 1) * t_l].contiguous() for r in range(world)]
    outs = [torch.zeros_like(p) for p in parts]
    for call in range(2):                                           # the second call reuses every buffer and flag
        _interleaved_call(layers, parts, outs)
        torch.cuda.synchronize()
        for layer in layers:
            layer.check_status()
        if call == 0:
            first = torch.cat(outs).clone()
    full = RoutedMoELayer(router_w, *(t.to(dev) for t in expert_weights), tokens, bias)
    full.set_partial_format(1)
    want = full(hidden)
    torch.cuda.synchronize()
    full.check_status()
    assert torch.equal(torch.cat(outs).view(torch.int16), want.view(torch.int16))
    assert torch.equal(first.view(torch.int16), want.view(torch.int16))
    full.set_partial_format(0)
    assert not torch.equal(full(hidden).view(torch.int16), want.view(torch.int16))     # the two contracts do differ
    # a small call under the same setting keeps the FP32 rows (swap-AB forms), as the one-GPU layer does
    small = [p[:8].contiguous() for p in parts]
    small_out = [torch.zeros_like(p) for p in small]
    _interleaved_call(layers, small, small_out)
    torch.cuda.synchronize()
    for layer in layers:
        layer.check_status()
    want_small = full(torch.cat(small))
    assert torch.equal(torch.cat(small_out).view(torch.int16), want_small.view(torch.int16))
    for layer in layers:
        layer.close()
    full.close()


def test_block_that_needs_more_rows_than_its_capacity_is_reported(expert_weights):
    dev = torch.device("cuda", 0)
    world, tokens = 2, 256
    hidden, router_w, _ = synth.make_activations(tokens, None, seed=4)
    hidden, router_w = hidden.to(dev), router_w.to(dev)
    t_l = tokens // world
    layers, keep = _emulated_ranks(world, tokens, expert_weights, router_w, None, dev, row_capacity=t_l + 256)
    parts = [hidden[r * t_l:(r + 1) * t_l].contiguous() for r in range(world)]
    outs = [torch.zeros_like(p) for p in parts]
    _interleaved_call(layers, parts, outs)
    torch.cuda.synchronize()                                        # nothing was written past the blocks: the context is intact
    for layer in layers:
        words = layer.status()
        assert words[2] > t_l + 256 and words[0] == words[1] == words[3] == 0
        with pytest.raises(Exception, match="row_capacity"):
            layer.check_status()
        layer.close()


def test_missing_peer_ends_in_a_reported_timeout(expert_weights):
    """Rank 0 of a world of two runs alone: the flags of rank 1 are never raised, every wait gives up
    after its limit and the call completes with the time-out recorded (nothing hangs or faults)."""
    dev = torch.device("cuda", 0)
    world, tokens = 2, 64
    hidden, router_w, _ = synth.make_activations(tokens, None, seed=4)
    hidden, router_w = hidden.to(dev), router_w.to(dev)
    layers, keep = _emulated_ranks(world, tokens, expert_weights, router_w, None, dev, timeout_s=0.05)
    t_l = tokens // world
    out = torch.zeros(t_l, 2048, dtype=torch.bfloat16, device=dev)
    layers[0](hidden[:t_l].contiguous(), out=out)
    torch.cuda.synchronize()
    words = layers[0].status()
    assert words[3] == (1 << 1) | (1 << 9) | (1 << 17) and words[2] == 0
    with pytest.raises(Exception, match="timed out"):
        layers[0].check_status()
    assert torch.isfinite(torch.ones(4, device=dev).sum()).item()   # the context still works
    for layer in layers:
        layer.close()


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _peer_rank(rank, world, port, tokens, results, partial_format=0):
    try:
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)     # host plumbing only: handles and barriers
        weights = synth.make_expert_weights(0)
        hidden, router_w, bias = synth.make_activations(tokens, 0.6, seed=2)
        plan = ExpertParallelPlan(world, rank)
        local = tuple(t.to(dev) for t in shard_expert_weights(weights, plan))
        t_l = tokens // world
        layer = PeerExpertParallelLayer(plan, router_w.to(dev), *local, max_local_tokens=t_l, router_bias=bias.to(dev))
        layer.set_partial_format(partial_format)
        mine = hidden[rank * t_l:(rank + 1) * t_l].to(dev)
        stream = torch.cuda.Stream(device=dev)
        torch.cuda.synchronize(dev)
        dist.barrier()                                       # every rank is ready before the first call's bounded waits start
        with torch.cuda.stream(stream):
            out = layer(mine)
            out2 = layer(mine)
            stream.synchronize()
            layer.check_status()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            out3 = torch.zeros_like(out)
            with torch.cuda.graph(graph, stream=stream):
                layer(mine, out=out3)
            for _ in range(3):
                graph.replay()
            stream.synchronize()
            layer.check_status()
        results[rank] = {"out": out.cpu(), "same": bool(torch.equal(out, out2) and torch.equal(out, out3))}
        if rank == 0:                                        # one-GPU layer over all tokens, same weights
            from netra_kernel_b200.moe import RoutedMoELayer
            full = RoutedMoELayer(router_w.to(dev), *(t.to(dev) for t in weights), tokens, bias.to(dev))
            full.set_partial_format(partial_format)
            results["ref"] = full(hidden.to(dev)).cpu()
            full.check_status()
        dist.barrier()
        layer.close()
        dist.destroy_process_group()
    except Exception:
        results[rank] = "error: " + traceback.format_exc()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("tokens,partial_format", [(512, 0), (2048, 0), (2048, 1)])      # 2,048 tokens: 64 rows per expert, the
def test_two_gpu_peer_memory_layer_equals_the_one_gpu_layer(tokens, partial_format):       # token-major GEMMs; 1: FP16 rows sent home
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    port = _free_port()
    procs = [mp.get_context("spawn").Process(target=_peer_rank, args=(r, world, port, tokens, results, partial_format)) for r in range(world)]
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
