"""Column-sharded matmul across GPUs (one process per GPU).

The path shards by weight row (= output column): rank r of g holds rows [r*N/g, (r+1)*N/g) -- the
partition the reference uses across threads (src/ops/kernel/q8_0/parallel.rs:124-139) and plans
across devices (PlacementSlice::Rows, src/format/load_plan.rs:19-22).  The activation is
replicated and quantized locally (deterministic, so identical on every rank); the only exchange
is an all-gather of the [M, N/g] results, after which a device kernel restores row-major [M, N].
"""
from __future__ import annotations

import numpy as np


def shard_rows(n_rows: int, world: int, rank: int) -> tuple[int, int]:
    """Rows of rank `rank`: ceil(n/world) per rank, the last ranks may get fewer (or none),
    as in the reference's thread partition."""
    per = (n_rows + world - 1) // world
    s = min(rank * per, n_rows)
    return s, min(s + per, n_rows)


def unshard_numpy(gathered: np.ndarray) -> np.ndarray:
    """[g, M, N/g] -> [M, N]; what rmi_unshard_cols_dev computes on the device."""
    g, m, npr = gathered.shape
    return np.ascontiguousarray(gathered.transpose(1, 0, 2)).reshape(m, g * npr)


def all_gather_cols_cpu(local: np.ndarray, group=None) -> np.ndarray:
    """Host-side exchange used by the CPU (gloo) tests: all-gather [M, N/g] -> [M, N]."""
    import torch
    import torch.distributed as dist
    t = torch.from_numpy(np.ascontiguousarray(local))
    out = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
    dist.all_gather(out, t, group=group)
    return unshard_numpy(np.stack([o.numpy() for o in out]))


class ShardedLinear:
    """One rank's shard of a Q8_0 weight plus the gather step (NCCL, device buffers)."""

    def __init__(self, pkg, weight_bytes_of_shard, n_in: int, n_out: int, rank: int, world: int, group=None):
        self.pkg, self.rank, self.world, self.group = pkg, rank, world, group
        self.n_in, self.n_out = n_in, n_out
        self.row_begin, self.row_end = shard_rows(n_out, world, rank)
        if n_out % world != 0:
            raise ValueError("the gather assumes equal shards: n_out must be a multiple of the world size")
        self.weight = pkg.QuantizedTensor.from_bytes(weight_bytes_of_shard, pkg.GGML_Q8_0, n_in,
                                                     self.row_end - self.row_begin)

    def forward_dev(self, x, out_local, gathered=None, out_full=None):
        """x [M, n_in] f32 cuda tensor; out_local [M, n_out/g]; optional gather into out_full [M, n_out]."""
        import torch.distributed as dist
        m = x.shape[0]
        self.pkg.matmul_q8_0_dev(self.weight, x.data_ptr(), m, out_local.data_ptr())
        if gathered is None:
            return out_local
        if self.world > 1:
            dist.all_gather_into_tensor(gathered, out_local, group=self.group)
        else:
            gathered.copy_(out_local.reshape(gathered.shape))
        self.pkg.unshard_cols_dev(self.pkg.context(), gathered.data_ptr(), self.world, m, self.n_out // self.world,
                                  out_full.data_ptr())
        return out_full
