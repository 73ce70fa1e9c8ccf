"""N-sharded GEMM on 2 GPUs (skipped when fewer are visible): every gather path -- epilogue TMA
stores into each rank's Y, epilogue multimem stores to the NVSwitch multicast address of Y, and NCCL
all-gather + interleave -- must reproduce, bit for bit, the result of the same plugin run unsharded
on one GPU, on every rank."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
KERNELS = ["bf16_bm256_bn256_bk64_s6_cg2_sk1_ab0_e1", "bf16_bm512_bn256_bk64_s4_cg2_sk1_ab0_e1"]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, M, N, K, out_dir, multicast, kernel):
    import torch.distributed as dist

    import sm120_gemm_b200 as g
    from sm120_gemm_b200.shard import FusedNShardedGemm, NShardedGemm, shard_plan

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if not multicast:
        os.environ.update(TORCH_SYMM_MEM_DISABLE_MULTICAST="1", NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    k = g.load_plugin(os.path.join(g.KERNEL_DIR, f"libgemm_{kernel}.so"))
    gen = torch.Generator(device=dev); gen.manual_seed(7)          # same stream on every rank
    X = torch.randn((M, K), device=dev, generator=gen).to(torch.bfloat16)
    W = torch.randn((N, K), device=dev, generator=gen).to(torch.bfloat16)
    st = torch.cuda.current_stream().cuda_stream
    Yref = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    g.dispatch(k, M, N, K, X.data_ptr(), W.data_ptr(), Yref.data_ptr(), 0, st)     # unsharded, this GPU alone
    plan = shard_plan(N, world, rank)
    Wr = W[plan.row_start:plan.row_start + plan.rows].contiguous()
    fused = FusedNShardedGemm(k, M, N, K, rank, world, multicast=multicast)
    fused.Y.fill_(float("nan"))
    dist.barrier()
    fused.run(X, Wr)
    Yn = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
    NShardedGemm(k, M, N, K, rank, world).run(X, Wr, Yn)
    torch.cuda.synchronize()
    k.check_status()
    ok = [bool(torch.equal(fused.Y, Yref)), bool(torch.equal(Yn, Yref)), bool(fused.multicast)]
    np.save(os.path.join(out_dir, f"ok_{rank}.npy"), np.array(ok))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("kernel", KERNELS, ids=["tile256x256", "tile512x256"])
@pytest.mark.parametrize("multicast", [False, True], ids=["peer_stores", "multicast_stores"])
def test_two_gpu_sharded_equals_unsharded(tmp_path, multicast, kernel):
    import torch.multiprocessing as mp

    world, M, N, K = 2, 1024 + 64, 2048, 1536       # M is not a tile multiple: the last row block is clipped
    mp.spawn(_worker, args=(world, _free_port(), M, N, K, str(tmp_path), multicast, kernel), nprocs=world, join=True)
    used = []
    for r in range(world):
        ok = np.load(tmp_path / f"ok_{r}.npy")
        assert ok[0], f"rank {r}: fused-epilogue result differs from the unsharded one"
        assert ok[1], f"rank {r}: NCCL all-gather result differs from the unsharded one"
        used.append(bool(ok[2]))
    if multicast and not all(used):
        pytest.skip("no multicast mapping of symmetric memory on this node: the peer-store path ran instead")
    assert all(used) == multicast
