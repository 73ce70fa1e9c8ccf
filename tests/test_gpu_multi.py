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


def _worker(rank, world, port, M, N, K, out_dir, multicast, kernel, forward):
    import torch.distributed as dist

    import sm120_gemm_b200 as g
    from sm120_gemm_b200.host_gemm import ShardedHostGemm
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
    # a second, different problem for the step that follows immediately
    X2 = torch.randn((M, K), device=dev, generator=gen).to(torch.bfloat16)
    Yref2 = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    g.dispatch(k, M, N, K, X2.data_ptr(), W.data_ptr(), Yref2.data_ptr(), 0, st)
    ok = []
    for double_buffer in (True, False):
        fused = FusedNShardedGemm(k, M, N, K, rank, world, multicast=multicast, double_buffer=double_buffer, forward=forward)
        for b in fused.buffers:
            b.fill_(float("nan"))
        dist.barrier()
        # two steps back to back with a read of the first result between them, in stream order and with no extra
        # barrier: the second step's remote stores must not disturb what a slower rank is still reading
        fused.run(X, Wr)
        y1 = fused.Y.clone()
        if rank == 0:
            torch.cuda._sleep(20_000_000)          # rank 0 dawdles (about 10 ms) before its copy is queued behind the clone
            y1b = fused.Y.clone()
        else:
            y1b = y1
        fused.run(X2, Wr)
        y2 = fused.Y.clone()
        torch.cuda.synchronize()
        ok += [bool(torch.equal(y1, Yref)), bool(torch.equal(y1b, Yref)), bool(torch.equal(y2, Yref2))]
        used_multicast = bool(fused.multicast)
        if double_buffer:
            # host buffers in (this rank's rows of X, exchanged over NVLink; its weight rows), its rows of Y out
            shg = ShardedHostGemm(fused, chunk_rows=M // world // 2)
            r0 = rank * (M // world)
            Xh, Wh = X[r0:r0 + M // world].cpu().pin_memory(), Wr.cpu().pin_memory()      # this rank's rows of X only
            Yh = torch.empty((M // world, N), dtype=torch.bfloat16).pin_memory()
            shg.run(Xh, Wh, Yh)
            torch.cuda.synchronize()
            r0 = rank * (M // world)
            ok.append(bool(torch.equal(Yh.cuda(), Yref[r0:r0 + M // world])))
        dist.barrier()
        del fused
    Yn = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
    NShardedGemm(k, M, N, K, rank, world).run(X, Wr, Yn)
    torch.cuda.synchronize()
    k.check_status()
    ok += [bool(torch.equal(Yn, Yref)), used_multicast]
    np.save(os.path.join(out_dir, f"ok_{rank}.npy"), np.array(ok))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("kernel,shape,forward", [(KERNELS[0], (1024 + 64, 2048, 1536), False), (KERNELS[0], (1024 + 64, 4096, 1536), True),
                                                  (KERNELS[1], (1024 + 64, 2048, 1536), False), (KERNELS[1], (2560 + 64, 8192, 512), False)],
                         ids=["tile256x256", "tile256x256_forwarded_from_l2", "tile512x256", "tile512x256_halved_last_wave"])
@pytest.mark.parametrize("multicast", [False, True], ids=["peer_stores", "multicast_stores"])
def test_two_gpu_sharded_equals_unsharded(tmp_path, multicast, kernel, shape, forward):
    import torch.multiprocessing as mp

    # M is not a tile multiple: the last row block is clipped.  The third case gives every rank 6 x 16 = 96 tiles of 512 x 256
    # on 74 clusters: the 22 tiles of the second round go out as 44 halves of 256 rows
    world, (M, N, K) = 2, shape
    mp.spawn(_worker, args=(world, _free_port(), M, N, K, str(tmp_path), multicast, kernel, forward), nprocs=world, join=True)
    used = []
    for r in range(world):
        ok = np.load(tmp_path / f"ok_{r}.npy")
        names = ["two buffers: step 1", "two buffers: step 1 read late", "two buffers: step 2", "host-buffer sharded call",
                 "one buffer: step 1", "one buffer: step 1 read late", "one buffer: step 2", "NCCL all-gather + interleave"]
        for i, what in enumerate(names):
            assert ok[i], f"rank {r}: {what} differs from the unsharded result"
        used.append(bool(ok[len(names)]))
    if multicast and not all(used):
        pytest.skip("no multicast mapping of symmetric memory on this node: the peer-store path ran instead")
    assert all(used) == multicast
