"""Multi-rank host logic on CPU: two gloo ranks shard a Q8_0 matmul by weight row, compute their
shards with the oracle (the device kernels are covered by the -m gpu tests), all-gather and
un-shard; the result must equal the unsharded matmul bit for bit."""
import os
import socket
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n, k, m, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from __graft_entry__ import load_package
    from oracle import orc
    pkg = load_package()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        s, e = pkg.sharding.shard_rows(n, world, rank)
        shard = pkg.synth.q8_0_weight_rows(n, k, seed=5, row_begin=s, row_end=e)
        x = pkg.synth.normal((m, k), seed=6)                       # replicated activation
        local = orc.q8_forward_batched(shard, x, k, e - s, orc.SEM_AVX2)
        full = pkg.sharding.all_gather_cols_cpu(local)
        whole = pkg.synth.q8_0_weight_rows(n, k, seed=5, row_begin=0, row_end=n)
        ref = orc.q8_forward_batched(whole, x, k, n, orc.SEM_AVX2)
        q.put((rank, bool(np.array_equal(full.view(np.uint32), ref.view(np.uint32))), full.shape))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("m", [1, 5])
def test_two_gloo_ranks_row_sharded_matmul_equals_unsharded(m):
    world, n, k = 2, 256, 128
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, k, m, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in res) == [0, 1]
    assert all(r[1] for r in res) and all(r[2] == (m, n) for r in res)


def test_shard_rows_cover_and_match_the_reference_partition(rmi):
    for n in (0, 1, 7, 1024, 32768, 151936):
        for g in (1, 2, 4, 8):
            rows = [rmi.sharding.shard_rows(n, g, r) for r in range(g)]
            assert rows[0][0] == 0 and rows[-1][1] == n
            assert all(rows[i][1] == rows[i + 1][0] for i in range(g - 1))
            per = (n + g - 1) // g
            assert all(e - s <= per for s, e in rows)


def test_unshard_numpy_layout(rmi):
    g, m, npr = 4, 3, 5
    full = np.arange(m * g * npr, dtype=np.float32).reshape(m, g * npr)
    gathered = np.stack([full[:, r * npr:(r + 1) * npr] for r in range(g)])
    assert np.array_equal(rmi.sharding.unshard_numpy(gathered), full)


def test_sharded_weight_generator_is_shard_consistent(rmi):
    whole = rmi.synth.q8_0_weight_rows(3000, 64, seed=9, row_begin=0, row_end=3000)
    rb = 64 // 32 * 34
    for s, e in ((0, 1024), (1000, 2100), (2999, 3000), (1024, 2048)):
        part = rmi.synth.q8_0_weight_rows(3000, 64, seed=9, row_begin=s, row_end=e)
        assert np.array_equal(part, whole[s * rb:e * rb])


def _handle_worker(rank, world, port, q):
    """The peer-store variant's host logic: handle exchange and pointer tables over gloo, with
    fake handles and a fake opener (no GPU)."""
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        mine = bytes([rank + 1]) * 64
        table = pkg.sharding.exchange_handles(mine, rank, world, dist.all_gather_object)
        ptrs = pkg.sharding.peer_pointer_table(table, rank, own_ptr=1000 + rank, open_handle=lambda h: 2000 + h[0])
        q.put((rank, table, ptrs, pkg.sharding.rotate_own_first(ptrs, rank)))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_exchange_ipc_handles_and_build_pointer_tables():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_handle_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        rank, table, ptrs, fan = q.get(timeout=120)
        got[rank] = (table, ptrs, fan)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank in range(world):
        table, ptrs, fan = got[rank]
        assert table == [bytes([1]) * 64, bytes([2]) * 64]
        # own allocation for itself, the opener's mapping for the peer
        assert ptrs[rank] == 1000 + rank and ptrs[1 - rank] == 2000 + (2 - rank)
        assert fan[0] == ptrs[rank] and sorted(fan) == sorted(ptrs)


def test_exchange_handles_rejects_duplicates_and_gaps():
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    pkg = load_package()

    def dup(out, obj):
        out[0], out[1] = (0, b"a"), (0, b"b")

    def gap(out, obj):
        out[0], out[1] = (0, b"a"), (1, None)

    with pytest.raises(ValueError):
        pkg.sharding.exchange_handles(b"a", 0, 2, dup)
    with pytest.raises(ValueError):
        pkg.sharding.exchange_handles(b"a", 0, 2, gap)
    assert pkg.sharding.rotate_own_first([10, 11, 12, 13], 2) == [12, 13, 10, 11]


def _plan_worker(rank, world, port, n, k, m, q):
    """Each rank builds the TensorSplit plan itself (it is deterministic), takes the rows the plan puts on its
    device, computes them with the oracle and all-gathers."""
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from __graft_entry__ import load_package
    from oracle import orc
    pkg = load_package()
    lp = pkg.load_plan
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        idx = lp.PackageIndex.from_tensor_table([("token_embd.weight", [32], 0), ("blk.0.ffn_up.weight", [k, n], 8)], 1)
        devices = lp.balanced_devices(idx, world)
        plan = lp.build_load_plan(idx, [0], devices, devices[0].id, lp.TENSOR_SPLIT)
        (rows,) = plan.rows_on("blk.0.ffn_up.weight", devices[rank].id)
        s, e = rows
        shard = pkg.synth.q8_0_weight_rows(n, k, seed=5, row_begin=s, row_end=e)
        x = pkg.synth.normal((m, k), seed=6)
        local = orc.q8_forward_batched(shard, x, k, e - s, orc.SEM_AVX2)
        full = pkg.sharding.all_gather_cols_cpu(local)
        whole = pkg.synth.q8_0_weight_rows(n, k, seed=5, row_begin=0, row_end=n)
        ref = orc.q8_forward_batched(whole, x, k, n, orc.SEM_AVX2)
        q.put((rank, (s, e), bool(np.array_equal(full.view(np.uint32), ref.view(np.uint32)))))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_take_their_rows_from_a_tensor_split_plan():
    world, n, k, m = 2, 256, 128, 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_plan_worker, args=(r, world, port, n, k, m, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [r[1] for r in res] == [(0, 128), (128, 256)]
    assert all(r[2] for r in res)
