"""Y = X * W^T with HOST buffers: the end-to-end call a caller without device-resident data makes.

Pinned host X (M x K), W (N x K) in, pinned host Y (M x N) out, bf16.  W goes to the device
first (every output row needs all of it); X then travels in row chunks, and for each chunk the
copy in, the kernel-plugin call and the copy of the finished Y rows out run on three streams,
so PCIe in, the tensor cores and PCIe out overlap.  The reference has no such call (its bench
keeps everything on the device, src/bench.cu:353-395); this is the plugin C ABI with the copies
a host-side caller needs around it.
"""
from __future__ import annotations


class HostGemm:
    def __init__(self, kernel, M: int, N: int, K: int, chunk_rows: int = 2048, device_X=None, device_W=None, device_Y=None):
        import torch

        self.torch = torch
        self.kernel = kernel
        self.M, self.N, self.K = M, N, K
        self.chunk = min(chunk_rows, M)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.X = device_X if device_X is not None else torch.empty((M, K), dtype=torch.bfloat16, device=dev)
        self.W = device_W if device_W is not None else torch.empty((N, K), dtype=torch.bfloat16, device=dev)
        self.Y = device_Y if device_Y is not None else torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        wsb = max(kernel.workspace_bytes(self.chunk, N, K), 16)
        self.ws = torch.empty(wsb, dtype=torch.uint8, device=dev)
        self.ws_ptr = self.ws.data_ptr() if kernel.workspace_bytes(self.chunk, N, K) else 0
        self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
        if not kernel.can_run(self.chunk, N, K):
            raise ValueError(f"{kernel.config.name()} cannot run {self.chunk}x{N}x{K}")

    def run(self, Xh, Wh, Yh) -> int:
        """Enqueues everything; returns the number of kernel launches.  The result is complete in Yh
        once the current stream has been synchronised."""
        from . import dispatch

        t = self.torch
        cur = t.cuda.current_stream()
        self.s_in.wait_stream(cur)          # buffers may still be in use by earlier work on the caller's stream
        self.s_out.wait_stream(cur)
        launches = 0
        with t.cuda.stream(self.s_in):
            self.W.copy_(Wh, non_blocking=True)
        for r0 in range(0, self.M, self.chunk):
            r1 = min(r0 + self.chunk, self.M)
            with t.cuda.stream(self.s_in):
                self.X[r0:r1].copy_(Xh[r0:r1], non_blocking=True)
                landed = t.cuda.Event()
                landed.record(self.s_in)
            cur.wait_event(landed)
            dispatch(self.kernel, r1 - r0, self.N, self.K, self.X[r0:r1].data_ptr(), self.W.data_ptr(), self.Y[r0:r1].data_ptr(),
                     self.ws_ptr, cur.cuda_stream)
            launches += 2 if self.kernel.config.split_k != 1 else 1
            done = t.cuda.Event()
            done.record(cur)
            self.s_out.wait_event(done)
            with t.cuda.stream(self.s_out):
                Yh[r0:r1].copy_(self.Y[r0:r1], non_blocking=True)
        cur.wait_stream(self.s_out)         # the caller's stream completes when the last rows are back on the host
        return launches
