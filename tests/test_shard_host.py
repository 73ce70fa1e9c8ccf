"""Host-side logic of the N-sharded multi-GPU run, on CPU with two gloo ranks: the shard plan,
the all-gather of per-rank column blocks and the block -> row-major index mapping that the
interleave kernel implements.  The per-rank GEMM is done by the CPU oracle here (test
infrastructure); the product path has no CPU compute."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sm120_gemm_b200.shard import blocked_to_row_major_index, shard_plan


def test_shard_plan_rules():
    p = shard_plan(16384, 8, 3)
    assert (p.row_start, p.rows) == (3 * 2048, 2048)
    assert [shard_plan(64, 4, r).row_start for r in range(4)] == [0, 16, 32, 48]
    with pytest.raises(ValueError):
        shard_plan(100, 8, 0)          # not divisible
    with pytest.raises(ValueError):
        shard_plan(48, 4, 0)           # 12 columns per rank: pitch not a multiple of 16 bytes
    with pytest.raises(ValueError):
        shard_plan(64, 4, 4)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, M, N, K, out_dir):
    from oracle import oracle as o

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    X, W = o.make_inputs(M, N, K, seed=2, dist="normal")          # every rank draws the same inputs
    plan = shard_plan(N, world, rank)
    y_local = o.gemm_bf16(X, W[plan.row_start:plan.row_start + plan.rows])     # this rank's M x N/g block
    y_local = torch.from_numpy(o.f32_to_bf16_bits(y_local).astype(np.int32))   # gloo has no 16-bit integer type
    blocked = torch.empty((world * M, plan.rows), dtype=torch.int32)       # [g][M][N/g], flattened over g
    dist.all_gather_into_tensor(blocked, y_local.contiguous())
    flat = blocked.numpy().reshape(-1)
    idx = np.array([[blocked_to_row_major_index(world, M, plan.rows, m, n) for n in range(N)] for m in range(M)])
    Y = flat[idx].astype(np.uint16)
    ref = o.f32_to_bf16_bits(o.gemm_bf16(X, W))
    np.save(os.path.join(out_dir, f"ok_{rank}.npy"), np.array([np.array_equal(Y, ref)]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gather_reassembles_row_major_result(tmp_path):
    world, M, N, K = 2, 24, 64, 96
    mp.spawn(_worker, args=(world, _free_port(), M, N, K, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert np.load(tmp_path / f"ok_{r}.npy")[0], f"rank {r} did not reassemble the unsharded result"


def test_destination_order_of_the_peer_store_gather():
    from sm120_gemm_b200.shard import destination_order

    for world in (1, 2, 4, 8):
        firsts = set()
        for rank in range(world):
            order = destination_order(rank, world)
            assert order[0] == rank and sorted(order) == list(range(world))
            firsts.add(order[1 % world])
        assert len(firsts) == world              # at every position the ranks address different GPUs
        assert destination_order(world - 1, world, rotate=False) == list(range(world))
    assert destination_order(3, 8, peers=[3]) == [3]
    for bad in ([], [9], [1, 1], list(range(9))):
        with pytest.raises(ValueError):
            destination_order(0, 8, peers=bad)
