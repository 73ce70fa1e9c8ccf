"""Helpers shared by the GPU tests: move bf16 bit patterns to the device and call a plugin
through its C ABI (raw device addresses, the current torch stream)."""
import numpy as np
import torch

import sm120_gemm_b200 as g


def to_dev(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16)


def to_bits(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def run_bf16(k: g.LoadedKernel, X: torch.Tensor, W: torch.Tensor, fill_nan: bool = True) -> torch.Tensor:
    M, K = X.shape
    N = W.shape[0]
    Y = torch.empty((M, N), dtype=torch.bfloat16, device=X.device)
    if fill_nan:
        Y.fill_(float("nan"))          # an element the kernel fails to write stays NaN and fails the check
    wsb = k.workspace_bytes(M, N, K)
    ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=X.device)
    g.dispatch(k, M, N, K, X.data_ptr(), W.data_ptr(), Y.data_ptr(), ws.data_ptr() if wsb else 0,
               torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    k.check_status()
    return Y
