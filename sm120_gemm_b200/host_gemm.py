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


class ShardedHostGemm:
    """The same host-buffer call on the N-sharded path (one process per GPU).  Nothing is sent from the host twice:
    every rank brings its own 1/world of the ROWS of X and its own weight rows from pinned host memory, the X
    slices are exchanged between the GPUs by one NCCL all-gather over NVLink (each rank needs all of X), the row
    chunks then run through the fused GEMM + all-gather of the result (``FusedNShardedGemm``: every rank's device Y
    receives every column block), and each rank returns only its 1/world slice of the rows of Y to the host.  Host
    traffic of the whole job per call: M*K*2 + N*K*2 bytes up, M*N*2 bytes down, whatever the number of GPUs.
    The copy out of a chunk overlaps the kernels of the next ones; a chunk is copied out after the cross-rank
    barrier that follows its GEMM."""

    def __init__(self, fused, chunk_rows: int = 2048, device_X=None, device_W=None, group=None):
        import torch

        self.torch = torch
        self.f = fused
        self.group = group
        M, world = fused.M, fused.plan.world
        if M % world != 0:
            raise ValueError(f"M={M} rows do not split over {world} ranks")
        self.slice_rows = M // world
        self.row0 = fused.plan.rank * self.slice_rows
        self.chunk = min(chunk_rows, self.slice_rows)
        if self.slice_rows % self.chunk != 0:
            raise ValueError(f"chunk of {self.chunk} rows does not divide the {self.slice_rows}-row slice of a rank")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.X = device_X if device_X is not None else torch.empty((M, fused.K), dtype=torch.bfloat16, device=dev)
        self.W = device_W if device_W is not None else torch.empty((fused.plan.rows, fused.K), dtype=torch.bfloat16, device=dev)
        self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
        self.h2d_bytes = (self.slice_rows + fused.plan.rows) * fused.K * 2
        self.d2h_bytes = self.slice_rows * fused.N * 2

    def run(self, Xh_slice, Wh_shard, Yh_slice) -> int:
        """Xh_slice: pinned (M/world) x K, rows [rank*M/world, (rank+1)*M/world) of X; Wh_shard: pinned (N/world) x K;
        Yh_slice: pinned (M/world) x N, receives the same rows of Y.  Returns the number of GEMM launches."""
        import torch.distributed as dist

        from . import dispatch_ex

        t, f = self.torch, self.f
        cur = t.cuda.current_stream()
        self.s_in.wait_stream(cur)
        self.s_out.wait_stream(cur)
        buf = f.step % len(f.buffers)
        f.step += 1
        Y, handle = f.buffers[buf], f.handles[buf]
        if not f.double_buffer:
            handle.barrier()
        mine = self.X[self.row0:self.row0 + self.slice_rows]
        with t.cuda.stream(self.s_in):
            mine.copy_(Xh_slice, non_blocking=True)
            x_landed = t.cuda.Event()
            x_landed.record(self.s_in)
            self.W.copy_(Wh_shard, non_blocking=True)
            w_landed = t.cuda.Event()
            w_landed.record(self.s_in)
        cur.wait_event(x_landed)
        dist.all_gather_into_tensor(self.X, mine, group=self.group)     # in place: each rank's slice is already where it belongs
        cur.wait_event(w_landed)
        launches = 0
        for r0 in range(0, f.M, self.chunk):
            r1 = r0 + self.chunk
            dispatch_ex(f.kernel, f._args(buf, r0, r1 - r0, self.X[r0:r1].data_ptr(), self.W.data_ptr(), cur.cuda_stream))
            launches += 1
            handle.barrier()                      # every rank's blocks of these rows have landed here
            if self.row0 <= r0 < self.row0 + self.slice_rows:
                done = t.cuda.Event()
                done.record(cur)
                self.s_out.wait_event(done)
                with t.cuda.stream(self.s_out):
                    Yh_slice[r0 - self.row0:r1 - self.row0].copy_(Y[r0:r1], non_blocking=True)
        cur.wait_stream(self.s_out)
        f.Y, f.handle = Y, handle
        return launches
