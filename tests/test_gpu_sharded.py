"""Device side of the sharded matmul on one GPU: every rank's shard computed in turn, the
un-shard kernel, and equality with the unsharded result."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m", [1, 16, 130])
def test_row_shards_gathered_on_the_device_equal_the_full_matmul(rmi, m):
    torch = pytest.importorskip("torch")
    ctx = rmi.context(0)
    ctx.set_semantics(rmi.SEM_NEON)
    n, k, g = 1024, 256, 4
    whole = rmi.synth.q8_0_weight_rows(n, k, seed=3, row_begin=0, row_end=n)
    x = torch.from_numpy(rmi.synth.normal((m, k), seed=4)).cuda()
    full_w = rmi.QuantizedTensor.from_bytes(whole, rmi.GGML_Q8_0, k, n)
    ref = torch.empty((m, n), dtype=torch.float32, device="cuda")
    rmi.matmul_q8_0_dev(full_w, x.data_ptr(), m, ref.data_ptr())
    gathered = torch.empty((g, m, n // g), dtype=torch.float32, device="cuda")
    for r in range(g):   # what each rank would compute; here one GPU plays every rank in turn
        s, e = rmi.sharding.shard_rows(n, g, r)
        shard = rmi.QuantizedTensor.from_bytes(rmi.synth.q8_0_weight_rows(n, k, seed=3, row_begin=s, row_end=e),
                                               rmi.GGML_Q8_0, k, e - s)
        rmi.matmul_q8_0_dev(shard, x.data_ptr(), m, gathered[r].data_ptr())
    out = torch.empty((m, n), dtype=torch.float32, device="cuda")
    rmi.unshard_cols_dev(ctx, gathered.data_ptr(), g, m, n // g, out.data_ptr())
    ctx.sync()
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int32), ref.view(torch.int32))
    assert np.array_equal(rmi.sharding.unshard_numpy(gathered.cpu().numpy()), out.cpu().numpy())
    ctx.set_semantics(rmi.SEM_AVX2)


def test_sharded_linear_single_rank(rmi):
    torch = pytest.importorskip("torch")
    ctx = rmi.context(0)
    ctx.set_semantics(rmi.SEM_NEON)
    n, k, m = 512, 128, 7
    wb = rmi.synth.q8_0_weight_rows(n, k, seed=8, row_begin=0, row_end=n)
    lin = rmi.sharding.ShardedLinear(rmi, wb, k, n, rank=0, world=1)
    x = torch.from_numpy(rmi.synth.normal((m, k), seed=9)).cuda()
    out_local = torch.empty((m, n), dtype=torch.float32, device="cuda")
    gathered = torch.empty((1, m, n), dtype=torch.float32, device="cuda")
    out_full = torch.empty((m, n), dtype=torch.float32, device="cuda")
    ctx.sync()
    torch.cuda.synchronize()
    lin.forward_dev(x, out_local, gathered, out_full)
    ctx.sync()
    torch.cuda.synchronize()
    assert torch.equal(out_full, out_local)
    ctx.set_semantics(rmi.SEM_AVX2)


@pytest.mark.parametrize("sem", ["SEM_NEON", "SEM_AVX2"])
@pytest.mark.parametrize("m", [1, 2, 16, 130])
def test_fanout_stores_land_in_every_buffer(rmi, m, sem):
    """One GPU plays every rank in turn; each rank's matmul stores its column slice into all g
    'final' buffers (here local allocations).  Every buffer must equal the unsharded matmul."""
    torch = pytest.importorskip("torch")
    ctx = rmi.context(0)
    ctx.set_semantics(getattr(rmi, sem))
    n, k, g = 1024, 256, 4
    x = torch.from_numpy(rmi.synth.normal((m, k), seed=4)).cuda()
    full_w = rmi.QuantizedTensor.from_bytes(rmi.synth.q8_0_weight_rows(n, k, seed=3, row_begin=0, row_end=n),
                                            rmi.GGML_Q8_0, k, n)
    ref = torch.empty((m, n), dtype=torch.float32, device="cuda")
    rmi.matmul_q8_0_dev(full_w, x.data_ptr(), m, ref.data_ptr())
    finals = [torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda") for _ in range(g)]
    torch.cuda.synchronize()
    for r in range(g):
        s, e = rmi.sharding.shard_rows(n, g, r)
        shard = rmi.QuantizedTensor.from_bytes(rmi.synth.q8_0_weight_rows(n, k, seed=3, row_begin=s, row_end=e),
                                               rmi.GGML_Q8_0, k, e - s)
        fan = rmi.sharding.rotate_own_first([f.data_ptr() for f in finals], r)
        rmi.matmul_q8_0_fanout_dev(shard, x.data_ptr(), m, fan, n, s)
        ctx.sync()
        shard.free()
    for f in finals:
        assert torch.equal(f.view(torch.int32), ref.view(torch.int32))
    full_w.free()
    ctx.set_semantics(rmi.SEM_AVX2)


def test_fanout_rejects_bad_arguments(rmi):
    ctx = rmi.context(0)
    w = rmi.QuantizedTensor.from_bytes(rmi.synth.q8_0_weight_rows(64, 64, seed=1, row_begin=0, row_end=64),
                                       rmi.GGML_Q8_0, 64, 64)
    buf = ctx.dev_alloc(64 * 64 * 4)
    with pytest.raises(rmi.RmiError):
        rmi.matmul_q8_0_fanout_dev(w, buf, 1, [], 64, 0)                 # no outputs
    with pytest.raises(rmi.RmiError):
        rmi.matmul_q8_0_fanout_dev(w, buf, 1, [buf] * 9, 64, 0)          # too many
    with pytest.raises(rmi.RmiError):
        rmi.matmul_q8_0_fanout_dev(w, buf, 1, [buf], 64, 32)             # columns past the stride
    ctx.dev_free(buf)
    w.free()


@pytest.mark.parametrize("m", [7, 1300])
def test_peer_sharded_linear_single_rank_and_flag_round(rmi, m):
    """world = 1: the fan-out is this rank's own buffer and the flag round completes on its own flag; both
    exchanges, alternating result buffers, a different x every round (m = 1300 runs two slabs of the
    peer-copy exchange)."""
    torch = pytest.importorskip("torch")
    ctx = rmi.context(0)
    ctx.set_semantics(rmi.SEM_NEON)
    n, k = 512, 128
    wb = rmi.synth.q8_0_weight_rows(n, k, seed=8, row_begin=0, row_end=n)
    lin = rmi.sharding.PeerShardedLinear(rmi, wb, k, n, rank=0, world=1, m_max=m)
    seen = set()
    for rnd in range(4):
        x = torch.from_numpy(rmi.synth.normal((m, k), seed=9 + rnd)).cuda()
        ref = torch.empty((m, n), dtype=torch.float32, device="cuda")
        rmi.matmul_q8_0_dev(lin.weight, x.data_ptr(), m, ref.data_ptr())
        ptr = lin.forward_dev(x.data_ptr(), m, (rmi.EXCHANGE_FUSED_STORES, rmi.EXCHANGE_PEER_COPY, rmi.EXCHANGE_PEER_PUSH)[rnd % 3])
        ctx.check_status()
        got = np.empty((m, n), np.float32)
        ctx.d2h(got, ptr)
        assert np.array_equal(got.view(np.uint32), ref.cpu().numpy().view(np.uint32)), rnd
        seen.add(ptr)
    assert lin.epoch == 4 and len(seen) == 2
    with pytest.raises(ValueError):
        lin.forward_dev(0, m + 1)
    lin.close()
    ctx.set_semantics(rmi.SEM_AVX2)


def test_flag_wait_runs_out_and_reports_timeout(rmi):
    """A rank that never signals: world = 2 with both flag arrays local and slot 1 never written.  The wait
    kernel returns after the context's limit (20 ms here), the status call reports RMI_ERR_TIMEOUT once and
    clears the word, and the context stays usable.  Nothing hangs or faults: the wait is a bounded poll."""
    ctx = rmi.context(0)
    f0, f1 = ctx.dev_alloc(256), ctx.dev_alloc(256)
    zeros = np.zeros(64, np.uint32)
    ctx.h2d(f0, zeros)
    ctx.h2d(f1, zeros)
    ctx.set_wait_limit_ms(20)
    try:
        rmi.peer_signal_wait_dev(ctx, [f0, f1], rank=0, epoch=1)
        with pytest.raises(rmi.RmiError) as e:
            ctx.check_status()
        assert e.value.status == 5 and "site 20" in e.value.message
        ctx.check_status()                      # cleared: the next check is clean
        got = np.zeros(64, np.uint32)
        ctx.d2h(got, f1)
        assert got[0] == 1                      # this rank's own signal did go out
        # the slot gets written: the same round now completes
        ctx.h2d(f0, np.array([1, 1] + [0] * 62, np.uint32))
        rmi.peer_signal_wait_dev(ctx, [f0, f1], rank=0, epoch=1)
        ctx.check_status()
        with pytest.raises(rmi.RmiError):
            ctx.set_wait_limit_ms(0)
    finally:
        ctx.set_wait_limit_ms(2000)
        ctx.dev_free(f0)
        ctx.dev_free(f1)


def test_unshard_vectorised_and_ragged(rmi):
    torch = pytest.importorskip("torch")
    ctx = rmi.context(0)
    for g, m, npr in [(4, 9, 1024), (3, 5, 30), (2, 1, 8)]:
        gathered = torch.arange(g * m * npr, dtype=torch.float32, device="cuda").reshape(g, m, npr)
        out = torch.empty((m, g * npr), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        rmi.unshard_cols_dev(ctx, gathered.data_ptr(), g, m, npr, out.data_ptr())
        ctx.sync()
        assert np.array_equal(out.cpu().numpy(), rmi.sharding.unshard_numpy(gathered.cpu().numpy()))


def test_ipc_export_gives_a_64_byte_handle(rmi):
    ctx = rmi.context(0)
    p = ctx.dev_alloc(4096)
    h = ctx.ipc_export(p)
    assert isinstance(h, bytes) and len(h) == 64 and any(h)
    ctx.dev_free(p)


_TWO_RANK_SCRIPT = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["RMI_REPO"])
from __graft_entry__ import load_package
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo", rank=rank, world_size=world)
pkg = load_package()
ctx = pkg.context(rank)
ctx.set_semantics(pkg.SEM_NEON)
n, k = 2048, 512
s, e = pkg.sharding.shard_rows(n, world, rank)
shard = pkg.synth.q8_0_weight_rows(n, k, seed=3, row_begin=s, row_end=e)
lin = pkg.sharding.PeerShardedLinear(pkg, shard, k, n, rank, world, m_max=1200)
full = pkg.QuantizedTensor.from_bytes(pkg.synth.q8_0_weight_rows(n, k, seed=3, row_begin=0, row_end=n), pkg.GGML_Q8_0, k, n)
def bcast(obj):
    box = [obj]
    dist.broadcast_object_list(box, src=0)
    return box[0]
comm = pkg.NcclComm(ctx, world, rank, bcast)
nccl_lin = pkg.sharding.ShardedLinear(pkg, shard, k, n, rank, world, comm=comm)
ok = True
for m in (1, 16, 160, 1200):
    # three rounds back to back, a different x each, no host barrier in between: a stale or overwritten
    # result buffer shows up as a bit mismatch.  Each round's result is read back (enqueued on the
    # context's stream) before the next round is called, which is the documented contract.
    xs = [torch.from_numpy(pkg.synth.normal((m, k), seed=4 + 10 * r)).cuda() for r in range(3)]
    refs = []
    for x in xs:
        ref = torch.empty((m, n), dtype=torch.float32, device="cuda")
        pkg.matmul_q8_0_dev(full, x.data_ptr(), m, ref.data_ptr())
        refs.append(ref)
    ctx.sync()
    for exchange in (pkg.EXCHANGE_FUSED_STORES, pkg.EXCHANGE_PEER_COPY, pkg.EXCHANGE_PEER_PUSH):
        for x, ref in zip(xs, refs):
            ptr = lin.forward_dev(x.data_ptr(), m, exchange)
            got = np.empty((m, n), np.float32)
            ctx.d2h(got, ptr)
            ctx.check_status()
            ok = ok and np.array_equal(got.view(np.uint32), ref.cpu().numpy().view(np.uint32))
    out_local = torch.empty((m, n // world), dtype=torch.float32, device="cuda")
    gathered = torch.empty((world, m, n // world), dtype=torch.float32, device="cuda")
    out_full = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    nccl_lin.forward_dev(xs[0], out_local, gathered, out_full)
    ctx.sync()
    ok = ok and torch.equal(out_full.view(torch.int32), refs[0].view(torch.int32))
    dist.barrier()
comm.destroy()
lin.close()
dist.destroy_process_group()
print("RANK_OK" if ok else "RANK_MISMATCH", flush=True)
sys.exit(0 if ok else 1)
"""


def test_two_ranks_on_two_gpus_store_into_each_other(rmi, tmp_path):
    """Needs two GPUs: the ranks wait on each other's flags, so they must not share a device."""
    torch = pytest.importorskip("torch")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs (ranks that wait on one another never share one GPU)")
    import os, subprocess, sys, socket
    script = tmp_path / "two_ranks.py"
    script.write_text(_TWO_RANK_SCRIPT)
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   RMI_REPO=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    for p, out in zip(procs, outs):
        assert p.returncode == 0 and "RANK_OK" in out, out[-2000:]


@pytest.mark.parametrize("world", [2, 3])
def test_load_plan_row_ranges_uploaded_from_gguf_equal_the_full_matmul(rmi, tmp_path, world):
    """A TensorSplit plan over `world` logical devices, every device's placements executed on this GPU through
    the GGUF upload entry point: the per-device matmuls, laid side by side, are the unsharded matmul (oracle
    checked), and the unsplit tensors come back as mapped bytes."""
    from oracle import orc
    lp, g = rmi.load_plan, rmi.gguf
    ctx = rmi.context(0)
    ctx.set_semantics(rmi.SEM_AVX2)
    n, k, m = 96, 128, 5
    w = rmi.synth.q8_0_weight_rows(n, k, seed=21, row_begin=0, row_end=n)
    norm = rmi.synth.normal((k,), seed=22)
    path = str(tmp_path / "plan.gguf")
    g.write_gguf(path, [("general.architecture", g.T_STR, "qwen3"), ("qwen3.block_count", g.T_U32, 1)],
                 [("token_embd.weight", [32], g.GGML_F32, np.zeros(128, np.uint8)),
                  ("blk.0.attn_norm.weight", [k], g.GGML_F32, norm.view(np.uint8)),
                  ("blk.0.ffn_up.weight", [k, n], g.GGML_Q8_0, w)])
    idx = lp.PackageIndex.from_gguf_file(path)
    devices = lp.balanced_devices(idx, world, slack_rows=1)
    plan = lp.build_load_plan(idx, [0], devices, "cuda0", lp.TENSOR_SPLIT)
    loader = rmi.GGUFLoader.from_file(path)
    x = rmi.synth.normal((m, k), seed=23)
    out = np.zeros((m, n), np.float32)
    covered = 0
    seen_norm = 0
    for d in devices:
        got = lp.execute_plan(rmi, loader, plan, idx, d.id, ctx=ctx)
        for s, e, wt in got.get("blk.0.ffn_up.weight", []):
            assert s == covered and wt.n_out == e - s and wt.n_in == k
            out[:, s:e] = rmi.matmul_q8_0(wt, x)
            covered = e
        for s, e, raw in got.get("blk.0.attn_norm.weight", []):
            assert (s, e) == (0, 1) and np.array_equal(np.asarray(raw).view(np.float32), norm)
            seen_norm += 1
    assert covered == n and seen_norm == 1
    ref = orc.q8_forward_batched(w, x, k, n, orc.SEM_AVX2)
    assert np.array_equal(out.view(np.uint32), ref.view(np.uint32))
    loader.close()
