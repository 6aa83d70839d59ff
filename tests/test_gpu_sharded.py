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
