"""N-sharding of Y = X * W^T across the GPUs of one node (one process per GPU).

Rank r holds the contiguous weight rows W[r*N/g : (r+1)*N/g, :] and the full X, computes its
M x N/g column block of Y with a kernel plugin, and one NCCL all-gather over NVLink collects
the blocks; a device interleave kernel turns the gathered [g][M][N/g] buffer into the
row-major M x N result every rank ends up with.  K is never split across GPUs, so there is no
reduction.  The reference is single-GPU (device 0 hard-coded, src/bf16_gemm.cuh:531); this
module has no counterpart there.
"""
from __future__ import annotations

import os

from dataclasses import dataclass


@dataclass(frozen=True)
class ShardPlan:
    world: int
    rank: int
    N: int
    row_start: int   # first weight row (= first Y column) of this rank
    rows: int        # weight rows (= Y columns) of this rank


def shard_plan(N: int, world: int, rank: int) -> ShardPlan:
    """Equal contiguous row blocks.  A shape shards only when every block keeps a 16-byte
    row pitch (N/g a multiple of 8 bf16 elements)."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    if N % world != 0 or (N // world) % 8 != 0:
        raise ValueError(f"N={N} does not shard across {world} GPUs in multiples of 8 columns")
    nb = N // world
    return ShardPlan(world, rank, N, rank * nb, nb)


def blocked_to_row_major_index(plan_world: int, M: int, nb: int, m: int, n: int) -> int:
    """Flat index into the gathered [g][M][nb] buffer of the element that belongs at Y[m, n]
    (the mapping the interleave kernel implements)."""
    r, j = divmod(n, nb)
    assert r < plan_world
    return (r * M + m) * nb + j


def destination_order(rank: int, world: int, rotate: bool = True, peers=None) -> list[int]:
    """Ranks whose Y the peer-store epilogue writes, in store order.  Rotated: own rank first, then rank+1, ...
    (mod world), so that ranks walking their tiles in step address different GPUs at any moment.  ``peers``
    overrides the list (a subset is only good for timing: [rank] stores nothing remotely)."""
    if peers is not None:
        order = [int(r) for r in peers]
        if not order or len(order) > 8 or any(not (0 <= r < world) for r in order) or len(set(order)) != len(order):
            raise ValueError(f"bad destination list {order} for {world} ranks")
        return order
    return [(rank + i) % world if rotate else i for i in range(world)]


class FusedNShardedGemm:
    """Per-rank GEMM whose epilogue stores its column block straight into the row-major Y of every
    rank (TMA stores over NVLink into a symmetric buffer, or multimem stores to its NVSwitch multicast
    address), so the all-gather overlaps the math tile by tile and no interleave pass is needed.
    ``run`` ends with a cross-rank barrier on the stream: after it, this rank's ``Y`` holds every rank's
    block.  Needs a TMA-store configuration (``e1``, no split-K).

    Ordering between steps.  A step's stores land in the OTHER ranks' memory, so a rank that is quick out of
    the barrier could start the next step and overwrite a result a slower rank is still reading.  With
    ``double_buffer=True`` (default) two symmetric buffers are used in turn: step i+1 writes the buffer step i
    did not use, and step i+2 can only begin after step i+1's barrier, which every rank reaches on its stream
    after whatever it queued to read step i's result.  So a consumer that reads ``Y`` in stream order, before
    it calls ``run`` again, is safe without a second barrier.  With ``double_buffer=False`` there is one buffer
    and ``run`` opens with a barrier of its own instead (every rank is done with the previous result first)."""

    def __init__(self, kernel, M: int, N: int, K: int, rank: int, world: int, group=None, rotate: bool = True, peers=None,
                 multicast: bool = True, double_buffer: bool = True, forward: bool = False):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        from . import GemmArgs

        if kernel.config.epi != 1 or kernel.config.split_k != 1:
            raise ValueError(f"{kernel.config.name()} has no TMA-store epilogue")
        self.torch = torch
        self.kernel = kernel
        self.M, self.N, self.K = M, N, K
        self.plan = shard_plan(N, world, rank)
        if not kernel.can_run(M, self.plan.rows, K):
            raise ValueError(f"{kernel.config.name()} cannot run the {M}x{self.plan.rows}x{K} shard")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.double_buffer = bool(double_buffer)
        # multicast runs of the 256 x 256 plugins: store each tile locally and let the kernel's sender warps forward it
        # from L2 in 512-byte rows, instead of sending 128-byte pieces from the epilogue (the 512 x 256 plugins always forward)
        self.forward = bool(forward)
        self.buffers, self.handles, self.args_list = [], [], []
        # Destination order: own buffer first, then rank+1, rank+2, ... so that at any moment the ranks
        # (which walk their tiles in step) send to eight different GPUs instead of all to the same one.
        order = destination_order(rank, world, rotate, peers)
        self.multicast = None
        for _ in range(2 if self.double_buffer else 1):
            Y = symm_mem.empty((M, N), dtype=torch.bfloat16, device=dev)       # same buffer on every rank
            handle = symm_mem.rendezvous(Y, group if group is not None else dist.group.WORLD)
            ptrs = list(handle.buffer_ptrs)
            assert len(ptrs) == world <= 8
            # With an NVSwitch multicast mapping of the buffer one store reaches every rank, and each result byte
            # leaves this GPU once instead of world-1 times; without one (or with fewer destinations than ranks)
            # the epilogue stores to each peer in turn.
            mc = int(getattr(handle, "multicast_ptr", 0) or 0)
            use_mc = bool(multicast and mc and peers is None and self.plan.rows % 8 == 0 and os.environ.get("SM100_GEMM_MULTICAST", "1") != "0")
            self.multicast = use_mc if self.multicast is None else (self.multicast and use_mc)
            self.buffers.append(Y)
            self.handles.append(handle)
            self.args_list.append((ptrs, mc))
        self.order = order
        self.step = 0
        self.Y = self.buffers[0]            # the buffer the most recent run() filled (the first one before any run)
        self.handle = self.handles[0]
        self._GemmArgs = GemmArgs

    def _args(self, buf: int, row0: int, rows: int, X_ptr: int, W_ptr: int, stream: int):
        """GemmArgs of one launch that computes Y rows [row0, row0 + rows) into buffer `buf` of every rank."""
        ptrs, mc = self.args_list[buf]
        a = self._GemmArgs()
        a.M, a.N, a.K = rows, self.plan.rows, self.K
        a.x_scale_f = a.w_scale_f = 1.0
        a.y_num_peers, a.y_col_offset, a.y_ld = len(self.order), self.plan.row_start, self.N
        off = row0 * self.N * 2
        order = self.order
        if self.multicast and order[0] != self.plan.rank:
            # with a multicast address the first destination must be this rank's own matrix: the two-row-block kernels
            # store a tile there first and forward it from there
            order = [self.plan.rank] + [r for r in order if r != self.plan.rank]
        for i, r in enumerate(order):
            a.y_peers[i] = ptrs[r] + off
        a.y_multicast = (mc + off) if self.multicast else None
        a.y_forward = 1 if (self.multicast and self.forward) else 0
        a.X, a.W, a.stream = X_ptr, W_ptr, stream
        return a

    def run(self, X, W_shard):
        from . import dispatch_ex

        buf = self.step % len(self.buffers)
        self.step += 1
        if not self.double_buffer:
            self.handles[buf].barrier()    # nobody still reads the previous result
        dispatch_ex(self.kernel, self._args(buf, 0, self.M, X.data_ptr(), W_shard.data_ptr(), self.torch.cuda.current_stream().cuda_stream))
        self.handles[buf].barrier()        # every rank's stores have landed before anyone reads Y
        self.Y, self.handle = self.buffers[buf], self.handles[buf]
        return 1


class NShardedGemm:
    """Per-rank GEMM + all-gather + interleave on the current CUDA device.

    ``kernel`` is a LoadedKernel; tensors are torch CUDA tensors (bf16).  The all-gather is
    issued on ``comm_stream`` when given so that it can overlap the next compute step.
    """

    def __init__(self, kernel, M: int, N: int, K: int, rank: int, world: int, group=None):
        import torch

        from . import util_lib

        self.torch = torch
        self.kernel = kernel
        self.M, self.N, self.K = M, N, K
        self.plan = shard_plan(N, world, rank)
        self.group = group
        self.util = util_lib()
        if not kernel.can_run(M, self.plan.rows, K):
            raise ValueError(f"{kernel.config.name()} cannot run the {M}x{self.plan.rows}x{K} shard")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.y_local = torch.empty((M, self.plan.rows), dtype=torch.bfloat16, device=dev)
        self.blocked = torch.empty((world, M, self.plan.rows), dtype=torch.bfloat16, device=dev) if world > 1 else None
        wsb = kernel.workspace_bytes(M, self.plan.rows, K)
        self.ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
        self.ws_ptr = self.ws.data_ptr() if wsb else 0

    def run(self, X, W_shard, Y_out):
        """Y_out (M x N, row-major) <- X @ W^T, where this rank passes only its rows of W."""
        import torch.distributed as dist

        from . import dispatch

        t = self.torch
        stream = t.cuda.current_stream().cuda_stream
        if self.plan.world == 1:
            dispatch(self.kernel, self.M, self.N, self.K, X.data_ptr(), W_shard.data_ptr(), Y_out.data_ptr(), self.ws_ptr, stream)
            return 1
        dispatch(self.kernel, self.M, self.plan.rows, self.K, X.data_ptr(), W_shard.data_ptr(), self.y_local.data_ptr(),
                 self.ws_ptr, stream)
        dist.all_gather_into_tensor(self.blocked, self.y_local, group=self.group)
        rc = self.util.gemm_interleave_blocks(self.blocked.data_ptr(), Y_out.data_ptr(), self.plan.world, self.M, self.plan.rows, 2,
                                              stream)
        if rc != 0:
            raise RuntimeError(f"gemm_interleave_blocks failed with CUDA error {rc}")
        return 2  # kernels of this library launched (GEMM + interleave); split-K adds its reduce
