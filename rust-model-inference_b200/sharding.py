"""Column-sharded matmul across GPUs (one process per GPU).

The path shards by weight row (= output column): rank r of g holds rows [r*N/g, (r+1)*N/g) -- the
partition the reference uses across threads (src/ops/kernel/q8_0/parallel.rs:124-139) and plans
across devices (PlacementSlice::Rows, src/format/load_plan.rs:19-22).  The activation is
replicated and quantized locally (deterministic, so identical on every rank); the only exchange
is an all-gather of the [M, N/g] results, after which a device kernel restores row-major [M, N]
(ShardedLinear), or -- fused -- the matmul stores its column slice straight into every rank's
[M, N] buffer through peer-mapped pointers, or the copy engines push it there slab by slab behind
the next slab's matmul, and a flag round closes the step (PeerShardedLinear over rmi_shard_group).
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
    """One rank's shard of a Q8_0 weight plus the NCCL gather step (device buffers).  With `comm` (an
    NcclComm of the package) the gather and the un-shard run inside the library (rmi_allgather_cols_dev);
    without it torch.distributed's all-gather is used and only the un-shard is the library's."""

    def __init__(self, pkg, weight_bytes_of_shard, n_in: int, n_out: int, rank: int, world: int, group=None, comm=None):
        self.pkg, self.rank, self.world, self.group, self.comm = pkg, rank, world, group, comm
        self.n_in, self.n_out = n_in, n_out
        self.row_begin, self.row_end = shard_rows(n_out, world, rank)
        if n_out % world != 0:
            raise ValueError("the gather assumes equal shards: n_out must be a multiple of the world size")
        self.weight = pkg.QuantizedTensor.from_bytes(weight_bytes_of_shard, pkg.GGML_Q8_0, n_in,
                                                     self.row_end - self.row_begin)

    def forward_dev(self, x, out_local, gathered=None, out_full=None):
        """x [M, n_in] f32 cuda tensor; out_local [M, n_out/g]; optional gather into out_full [M, n_out]."""
        m = x.shape[0]
        self.pkg.matmul_q8_0_dev(self.weight, x.data_ptr(), m, out_local.data_ptr())
        if gathered is None:
            return out_local
        if self.comm is not None:
            self.comm.allgather_cols_dev(out_local.data_ptr(), m, self.n_out // self.world, gathered.data_ptr(),
                                         out_full.data_ptr())
            return out_full
        if self.world > 1:
            import torch.distributed as dist
            dist.all_gather_into_tensor(gathered, out_local, group=self.group)
        else:
            gathered.copy_(out_local.reshape(gathered.shape))
        self.pkg.unshard_cols_dev(self.pkg.context(), gathered.data_ptr(), self.world, m, self.n_out // self.world,
                                  out_full.data_ptr())
        return out_full


def exchange_handles(local: bytes, rank: int, world: int, all_gather_object) -> list:
    """Every rank contributes one opaque handle; returns the list indexed by rank.
    `all_gather_object(out_list, obj)` has torch.distributed's signature."""
    out = [None] * world
    all_gather_object(out, (rank, local))
    table = [None] * world
    for r, h in out:
        if table[r] is not None:
            raise ValueError(f"rank {r} reported twice")
        table[r] = h
    if any(h is None for h in table):
        raise ValueError("a rank did not report its handle")
    return table


def peer_pointer_table(handles: list, rank: int, own_ptr: int, open_handle) -> list:
    """Pointer of every rank's buffer as seen from `rank`: its own allocation, IPC mappings for the others."""
    return [own_ptr if r == rank else open_handle(h) for r, h in enumerate(handles)]


def rotate_own_first(ptrs: list, rank: int) -> list:
    """Fan-out order: this rank's buffer first (the primary store), then the peers starting at
    rank+1 so that the ranks do not all write to the same peer at the same time."""
    return [ptrs[(rank + i) % len(ptrs)] for i in range(len(ptrs))]


class PeerShardedLinear:
    """Row-sharded Q8_0 linear whose result lands complete on every rank without a collective call
    (rmi_shard_group): either the matmul's epilogue stores this rank's columns into all ranks' result
    buffers (EXCHANGE_FUSED_STORES), or the copy engines push them slab by slab while the next slab is
    computed (EXCHANGE_PEER_COPY).  Result buffers alternate by round."""

    def __init__(self, pkg, weight_bytes_of_shard, n_in: int, n_out: int, rank: int, world: int, m_max: int, group=None):
        if n_out % world != 0:
            raise ValueError("equal shards: n_out must be a multiple of the world size")
        if world > 8:
            raise ValueError("at most 8 ranks (one NVSwitch domain)")
        self.pkg, self.rank, self.world, self.group = pkg, rank, world, group
        self.n_in, self.n_out, self.m_max = n_in, n_out, m_max
        self.row_begin, self.row_end = shard_rows(n_out, world, rank)
        self.ctx = pkg.context()
        self.weight = pkg.QuantizedTensor.from_bytes(weight_bytes_of_shard, pkg.GGML_Q8_0, n_in,
                                                     self.row_end - self.row_begin)
        self.shard_group = pkg.ShardGroup(self.ctx, world, rank, n_out, m_max)
        if world > 1:
            import torch.distributed as dist
            gather = lambda out, obj: dist.all_gather_object(out, obj, group=group)
            self.shard_group.connect(exchange_handles(self.shard_group.export(), rank, world, gather))
            dist.barrier(group=group)  # every rank has mapped every buffer before the first store
        self.out_ptr = None

    @property
    def epoch(self) -> int:
        return self.shard_group.epoch

    def forward_dev(self, x_ptr: int, m: int, exchange: int = 0) -> int:
        """x [m, n_in] f32 on the device -> pointer of this round's [m, n_out] buffer, complete (all ranks'
        columns) once the enqueued work has run.  Reads of a round's result must be enqueued on the context's
        stream before the next call; the buffer then stays intact until the call after that."""
        if m > self.m_max:
            raise ValueError("m exceeds m_max")
        self.out_ptr = self.shard_group.matmul_dev(self.weight, x_ptr, m, exchange)
        return self.out_ptr

    def close(self):
        self.ctx.sync()
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(group=self.group)  # no peer is still storing into a buffer that is about to go
        self.shard_group.free()
        self.weight.free()
