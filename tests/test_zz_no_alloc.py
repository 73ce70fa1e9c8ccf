"""gemm_run_no_alloc: the split-K GEMM entry point for callers that cannot allocate device
memory (its FP32 partial sums live in a fixed array inside the plugin).  Collected last on
purpose.  The GPU test calls it through the C ABI twice in a row, with different inputs, and
demands the same bits as gemm_run with a caller-owned workspace: both run the same kernels, so
any difference would mean stale scratch contents or a wrong scratch address."""
import numpy as np
import pytest

import sm120_gemm_b200 as g

NAME = "bf16_bm128_bn128_bk64_s7_cg1_sk4_ab0_e0"


def test_no_alloc_rejects_what_it_cannot_hold(registry):
    """Size and configuration checks happen before any CUDA call, so they run without a GPU."""
    k = registry.find(NAME)
    assert g.NO_ALLOC_SCRATCH_BYTES == 16 << 20
    # 4 splits x 2048 x 2048 floats = 64 MiB > 16 MiB
    assert k.lib.gemm_run_no_alloc(2048, 2048, 1024, 16, 16, 16, 0) == 4
    msg = k.last_error()[1]
    assert "16777216" in msg and "caller-owned workspace" in msg
    assert k.lib.gemm_run_no_alloc(128, 130, 1024, 16, 16, 16, 0) == 1          # unsupported shape
    # the limit itself: 4 x 128 x 8192 floats are exactly 16 MiB (accepted by the size check: what stops the call here is
    # the missing device or the null operands, not the workspace), one 8-column step more is over
    assert k.workspace_bytes(128, 8192, 2048) == g.NO_ALLOC_SCRATCH_BYTES
    assert k.lib.gemm_run_no_alloc(128, 8192, 2048, 0, 0, 0, 0) in (2, 6)
    assert k.lib.gemm_run_no_alloc(128, 8200, 2048, 16, 16, 16, 0) == 4
    direct = registry.find("bf16_bm128_bn128_bk64_s6_cg1_sk1_ab0_e1")
    assert direct.lib.gemm_run_no_alloc(128, 128, 1024, 16, 16, 16, 0) == 6      # no scratch in this plugin


@pytest.mark.gpu
def test_no_alloc_matches_caller_workspace_twice(registry, cuda_device):
    import torch

    from oracle import oracle as o
    from tests.gpu_util import run_bf16, to_bits, to_dev

    k = registry.find(NAME)
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row, different data and sizes: half of the array, then all of it (the exact-fit shape)
    for seed, (M, N, K) in ((21, (128, 4096, 2048)), (22, (128, 8192, 2048))):
        assert k.workspace_bytes(M, N, K) <= g.NO_ALLOC_SCRATCH_BYTES
        X, W = o.make_inputs(M, N, K, seed=seed, dist="normal")
        Xd, Wd = to_dev(X), to_dev(W)
        expect = run_bf16(k, Xd, Wd)             # existing entry point, workspace from the caller
        Y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = k.lib.gemm_run_no_alloc(M, N, K, Xd.data_ptr(), Wd.data_ptr(), Y.data_ptr(), stream)
        assert rc == 0, k.last_error()
        torch.cuda.synchronize()
        k.check_status()
        assert np.array_equal(to_bits(Y), to_bits(expect))
        ref = o.gemm_bf16(X, W)
        assert o.check_dense(to_bits(Y), ref, K, float(np.abs(o.bf16_bits_to_f32(X)).max()),
                             float(np.abs(o.bf16_bits_to_f32(W)).max()))["ok"]
    if torch.cuda.device_count() >= 2:
        # the array's address is looked up per device, with that device current
        with torch.cuda.device(1):
            X, W = o.make_inputs(128, 4096, 2048, seed=23, dist="normal")
            Xd, Wd = to_dev(X).to("cuda:1"), to_dev(W).to("cuda:1")
            Y = torch.full((128, 4096), float("nan"), dtype=torch.bfloat16, device="cuda:1")
            assert k.lib.gemm_run_no_alloc(128, 4096, 2048, Xd.data_ptr(), Wd.data_ptr(), Y.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
            torch.cuda.synchronize()
            k.check_status()
            assert o.check_dense(to_bits(Y), o.gemm_bf16(X, W), 2048, float(np.abs(o.bf16_bits_to_f32(X)).max()),
                                 float(np.abs(o.bf16_bits_to_f32(W)).max()))["ok"]
