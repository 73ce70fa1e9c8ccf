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


def run_ex(k: g.LoadedKernel, M: int, N: int, K: int, X: torch.Tensor, W: torch.Tensor, x_scale=None, w_scale=None,
           x_scale_f: float = 1.0, w_scale_f: float = 1.0, group_size: int = 0) -> torch.Tensor:
    """gemm_run_ex for the non-bf16 plugins: X, W (and scale arrays) are device tensors in the
    layouts include/sm100_gemm.h documents; returns the bf16 M x N result."""
    Y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=X.device)
    wsb = k.workspace_bytes(M, N, K)
    ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=X.device)
    a = g.GemmArgs()
    a.M, a.N, a.K, a.group_size = M, N, K, group_size
    a.X, a.W, a.Y = X.data_ptr(), W.data_ptr(), Y.data_ptr()
    a.x_scale = x_scale.data_ptr() if x_scale is not None else None
    a.w_scale = w_scale.data_ptr() if w_scale is not None else None
    a.x_scale_f, a.w_scale_f = x_scale_f, w_scale_f
    a.workspace, a.workspace_bytes = (ws.data_ptr() if wsb else None), wsb
    a.sm_limit = 0
    a.stream = torch.cuda.current_stream().cuda_stream
    g.dispatch_ex(k, a)
    torch.cuda.synchronize()
    k.check_status()
    return Y
