"""CPU tests of the expert-parallel host logic with two gloo ranks: count exchange, variable
all-to-all dispatch, source-major -> expert-major regrouping, return and combine must reproduce
the single-process CPU checker; inconsistent sizes and a missing rank are reported as errors on
the host (no GPU is involved, nothing hangs)."""
import datetime
import os
import socket
import traceback

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from netra_kernel_b200 import synth
from netra_kernel_b200.ep import ExpertParallelPlan
from oracle import moe_ref as R
from tests import helpers

WORLD = 2
TOKENS = 32


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _random_weights(path):
    """Random FP8 codes (no NaN patterns) and positive scales: plumbing tests need no trained-like values."""
    g = np.random.default_rng(7)
    def codes(shape):
        c = g.integers(0, 256, size=shape, dtype=np.uint8)
        c[(c & 0x7F) == 0x7F] = 0x38
        return c
    np.save(path / "w13.npy", codes((257, 1024, 2048)))
    np.save(path / "w2.npy", codes((257, 2048, 512)))
    np.save(path / "w13_s.npy", (g.random((257, 8, 16), dtype=np.float32) * 4e-4 + 1e-4))
    np.save(path / "w2_s.npy", (g.random((257, 16, 4), dtype=np.float32) * 4e-4 + 1e-4))


def _load(path):
    return [np.load(path / f"{n}.npy", mmap_mode="r") for n in ("w13", "w13_s", "w2", "w2_s")]


def _ep_rank(rank, port, path, mode, results):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=WORLD, timeout=datetime.timedelta(seconds=8))
        plan = ExpertParallelPlan(WORLD, rank)
        w13, w13_s, w2, w2_s = _load(path)
        hidden, router_w, _ = synth.make_activations(TOKENS)
        t_l = TOKENS // WORLD
        mine = slice(rank * t_l, (rank + 1) * t_l)
        hb, rb = helpers.bits(hidden)[mine], helpers.bits(router_w)
        ids, w = R.route_topk(R.router_logits(hb, rb))
        ids9, w9 = R.append_shared(ids, w, np.ones(t_l, np.float32))
        perm, counts, offsets = R.sort_pairs(ids)
        aq, a_s = R.quant_fp8_group128(R.bf16_bits_to_f32(hb))
        sorted_rows, sorted_scales = aq[perm // 8], a_s[perm // 8]
        counts_t = torch.from_numpy(counts)
        if mode == "missing_rank" and rank == 1:
            results[rank] = "left"
            return                                   # never joins the collective
        recv_counts = plan.exchange_counts(counts_t)
        splits = plan.splits(counts_t, recv_counts)
        if mode == "bad_sizes":
            with pytest.raises(ValueError, match="split sizes"):
                plan.all_to_all_rows(torch.from_numpy(sorted_rows[:-1].copy()), splits.send, splits.recv)
            results[rank] = "refused"
            return
        recv_a = plan.all_to_all_rows(torch.from_numpy(sorted_rows), splits.send, splits.recv).numpy()
        recv_s = plan.all_to_all_rows(torch.from_numpy(sorted_scales), splits.send, splits.recv).numpy()
        index, off = plan.regroup_reference(recv_counts, extra_rows=t_l)
        index, off = index.numpy(), off.numpy()
        r = splits.total_recv
        blk_a, blk_s = np.zeros((r + t_l, 2048), np.uint8), np.zeros((r + t_l, 16), np.float32)
        blk_a[index], blk_s[index] = recv_a, recv_s
        blk_a[r:], blk_s[r:] = aq, a_s
        down = np.zeros((r + t_l, 2048), np.float32)
        e_l = plan.experts_per_rank
        for g in range(e_l + 1):
            lo, hi = off[g], off[g + 1]
            if hi > lo:
                e = plan.local_expert_range().start + g if g < e_l else 256
                down[lo:hi], _, _ = R.expert_mlp(blk_a[lo:hi], blk_s[lo:hi], w13[e], w13_s[e], w2[e], w2_s[e])
        back = plan.all_to_all_rows(torch.from_numpy(down[index]), splits.recv, splits.send).numpy()
        rows = np.zeros((t_l, 9, 2048), np.float32)
        inv = np.empty_like(perm)
        inv[perm] = np.arange(perm.size)
        rows[:, :8] = back[inv].reshape(t_l, 8, 2048)
        rows[:, 8] = down[r:]
        results[rank] = {"out": R.combine(rows, w9), "recv": splits.recv, "send": splits.send, "ids": ids9,
                         "expert_major_ok": bool(np.all(np.diff(off) >= 0)) and off[e_l] == r}
    except Exception:
        results[rank] = "error: " + traceback.format_exc()
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _run(mode, path):
    manager = mp.Manager()
    results = manager.dict()
    port = _free_port()
    procs = [mp.get_context("spawn").Process(target=_ep_rank, args=(r, port, path, mode, results)) for r in range(WORLD)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        if p.is_alive():
            p.kill()
    return dict(results)


@pytest.fixture(scope="module")
def weight_dir(tmp_path_factory):
    path = tmp_path_factory.mktemp("ep_weights")
    _random_weights(path)
    return path


def test_two_rank_dispatch_and_combine_reproduce_the_single_process_checker(weight_dir):
    res = _run("ok", weight_dir)
    assert set(res) == {0, 1} and all(isinstance(v, dict) for v in res.values()), res
    w13, w13_s, w2, w2_s = _load(weight_dir)
    hidden, router_w, _ = synth.make_activations(TOKENS)
    ref = R.moe_layer(helpers.bits(hidden), helpers.bits(router_w), w13, w13_s, w2, w2_s)
    got = np.concatenate([res[0]["out"], res[1]["out"]])
    assert np.array_equal(np.concatenate([res[0]["ids"], res[1]["ids"]]), ref["topk_ids"])
    m = R.parity_metrics(got, ref["out"])
    assert m["rel_l2"] < 1e-4 and m["exact_fraction"] > 0.99, m
    assert res[0]["send"][1] == res[1]["recv"][0] and res[1]["send"][0] == res[0]["recv"][1]
    assert sum(res[0]["send"]) == TOKENS // WORLD * 8 and res[0]["expert_major_ok"] and res[1]["expert_major_ok"]


def test_inconsistent_payload_is_refused_before_the_collective(weight_dir):
    assert _run("bad_sizes", weight_dir) == {0: "refused", 1: "refused"}


def test_missing_rank_ends_in_a_timeout_error_not_a_hang(weight_dir):
    res = _run("missing_rank", weight_dir)
    assert res[1] == "left"
    assert isinstance(res[0], str) and res[0].startswith("error:"), res[0]


def test_plan_ownership_and_regroup_index():
    plan = ExpertParallelPlan(8, 3)
    assert plan.experts_per_rank == 32 and plan.owner(95) == 2 and plan.owner(96) == 3
    assert list(plan.local_expert_range())[:2] == [96, 97]
    with pytest.raises(ValueError):
        ExpertParallelPlan(3, 0)
    counts = torch.tensor([[2, 0, 1], [1, 3, 0]], dtype=torch.int32)      # 2 sources x 3 local experts
    small = ExpertParallelPlan(2, 0, n_routed=6)
    index, off = small.regroup_reference(counts, extra_rows=4)
    # source-major rows: s0:[e0,e0,e2] s1:[e0,e1,e1,e1] -> expert-major: e0:[s0,s0,s1] e1:[s1,s1,s1] e2:[s0]
    assert index.tolist() == [0, 1, 6, 2, 3, 4, 5] and off.tolist() == [0, 3, 6, 7, 11]
    # shared expert's rows first, fixed slots of 5 rows per source (unused slot rows are -1)
    index, off = small.regroup_reference(counts, extra_rows=4, slot_rows=5, shared_first=True)
    assert index.tolist() == [4, 5, 10, -1, -1, 6, 7, 8, 9, -1] and off.tolist() == [0, 4, 7, 10, 11]
    # a slot of 3 rows truncates source 1 to its first three rows: nothing points past world * slot rows
    index, off = small.regroup_reference(counts, extra_rows=4, slot_rows=3, shared_first=True)
    assert index.tolist() == [4, 5, 9, 6, 7, 8] and off.tolist() == [0, 4, 7, 9, 10]
    assert ExpertParallelPlan(8, 0).slot_rows_for(2048) % 64 == 0 and ExpertParallelPlan(8, 0).slot_rows_for(2048) < 2048 * 8 // 4
    world1 = ExpertParallelPlan(1, 0)
    c = torch.arange(256, dtype=torch.int32)
    assert torch.equal(world1.exchange_counts(c).view(-1), c)


def test_peer_memory_layer_sizes_and_capacity_rules():
    """Host-side parts of the peer-memory layer that need no GPU: size queries through the C ABI, capacity rules,
    argument errors."""
    import ctypes
    from netra_kernel_b200 import abi
    from netra_kernel_b200.ep import default_row_capacity, ep_sizes
    assert default_row_capacity(1, 256) == 256 * 9
    assert default_row_capacity(8, 256) == 256 + 8 * 256 * 8                       # worst case: every pair routed to one rank
    tight = default_row_capacity(8, 256, headroom=8.0)
    assert 256 + 2048 < tight < default_row_capacity(8, 256) and (tight - 256) % 64 == 0
    ws, win = ep_sizes(8, 256, default_row_capacity(8, 256))
    ws2, win2 = ep_sizes(8, 256, tight)
    assert ws > ws2 > 0 and win > win2 > 0 and ws % 1024 == 0 and win % 1024 == 0
    # the window holds at least the activation block, its scales and the FP32 return buffer
    assert win2 >= tight * 2048 + tight * 64 + 256 * 9 * 8192
    lib = abi.load()
    a, b = ctypes.c_uint64(), ctypes.c_uint64()
    assert lib.netra_ep_sizes_query(3, 256, 4096, ctypes.byref(a), ctypes.byref(b)) != 0       # 3 does not divide 256
    assert b"world" in lib.netra_moe_last_error()
    assert lib.netra_ep_sizes_query(8, 256, 100, ctypes.byref(a), ctypes.byref(b)) != 0        # cannot hold the rank's own tokens
    assert lib.netra_ep_layer_stage_count() == 9
