"""Fused transform + quantize for activations that live in host memory.

The kernel turns 2 bytes per element into 0.53, at several TB/s; a host round trip is bound by the PCIe link
(about 55 GB/s per direction).  Rows are independent, so the input is cut into row chunks and three streams
overlap the upload of chunk i+1, the kernel on chunk i and the download of chunk i-1 on double-buffered device
staging: the whole pass then costs about as much as the upload alone instead of upload + kernel + download.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib


class HostQuantizer:
    """Reusable pipeline: ``hq(x_host, q_host, sf_host)`` enqueues the whole pass and returns; the results are
    complete after ``hq.synchronize()`` (or once the current stream has waited on ``hq.done``).

    x_host   bf16 [rows, cols], pinned
    q_host   uint8 [rows, cols/2], pinned       packed E2M1, element 2i in the low nibble
    sf_host  uint8 [rows, cols/G], pinned       E8M0 / E4M3 scale bytes, row-major
    matrix   bf16 [G, cols] per-group transform (or [G, G] shared) on the device
    """

    def __init__(self, cols: int, matrix: torch.Tensor, fmt: str = "mx", global_scale: Optional[torch.Tensor] = None,
                 chunk_rows: int = 2048, device=None):
        if fmt not in ("mx", "nv"):
            raise ValueError(fmt)
        if not matrix.is_cuda:
            raise _lib.WushB200Error("wush_b200 ops need CUDA tensors; there is no CPU fallback")
        self.dev = torch.device(device) if device is not None else matrix.device
        self.fmt, self.cols, self.group = fmt, cols, 32 if fmt == "mx" else 16
        if cols % 32 or chunk_rows % 128:
            raise ValueError("cols must be a multiple of 32 and chunk_rows of 128")
        self.matrix = matrix.to(torch.bfloat16).contiguous()
        self.gs = None
        if fmt == "nv":
            self.gs = global_scale.to(device=self.dev, dtype=torch.float32).reshape(-1)[:1].contiguous()
        self.chunk = chunk_rows
        self.groups = cols // self.group
        self.sf_cols = (self.groups + 3) // 4 * 4
        mk = lambda *shape, dt: [torch.empty(*shape, dtype=dt, device=self.dev) for _ in range(2)]
        self.xd = mk(chunk_rows, cols, dt=torch.bfloat16)
        self.qd = mk(chunk_rows, cols // 2, dt=torch.uint8)
        self.sd = [torch.zeros(chunk_rows, self.sf_cols, dtype=torch.uint8, device=self.dev) for _ in range(2)]
        self.s_in, self.s_k, self.s_out = (torch.cuda.Stream(device=self.dev) for _ in range(3))
        self.done = torch.cuda.Event()
        self.launches = 0

    def __call__(self, x_host: torch.Tensor, q_host: torch.Tensor, sf_host: torch.Tensor) -> None:
        rows = x_host.shape[0]
        if x_host.dtype != torch.bfloat16 or tuple(x_host.shape) != (rows, self.cols) or not x_host.is_contiguous():
            raise ValueError("x_host must be a contiguous bf16 [rows, cols] tensor")
        if tuple(q_host.shape) != (rows, self.cols // 2) or tuple(sf_host.shape) != (rows, self.groups):
            raise ValueError("output shapes must be [rows, cols/2] and [rows, cols/G]")
        lib = _lib.load()
        start = torch.cuda.Event()
        start.record(torch.cuda.current_stream(self.dev))
        for s in (self.s_in, self.s_k, self.s_out):
            s.wait_event(start)
        ev_in, ev_k, ev_out = {}, {}, {}
        n_chunks = (rows + self.chunk - 1) // self.chunk
        for c in range(n_chunks):
            r0 = c * self.chunk
            n = min(self.chunk, rows - r0)
            b = c & 1
            with torch.cuda.stream(self.s_in):
                if c >= 2:
                    self.s_in.wait_event(ev_k[c - 2])           # the kernel that read this staging buffer is done
                self.xd[b][:n].copy_(x_host[r0:r0 + n], non_blocking=True)
                ev_in[c] = torch.cuda.Event()
                ev_in[c].record(self.s_in)
            with torch.cuda.stream(self.s_k):
                self.s_k.wait_event(ev_in[c])
                if c >= 2:
                    self.s_k.wait_event(ev_out[c - 2])          # its previous results have left the device
                with torch.cuda.device(self.dev):
                    if self.fmt == "mx":
                        rc = lib.wush_fused_quantize_mx(self.xd[b].data_ptr(), self.matrix.data_ptr(), self.matrix.shape[1],
                                                        self.qd[b].data_ptr(), self.sd[b].data_ptr(), self.sf_cols,
                                                        _lib.SF_ROW_MAJOR, n, self.cols, 0, self.s_k.cuda_stream)
                    else:
                        rc = lib.wush_fused_quantize_nv(self.xd[b].data_ptr(), self.matrix.data_ptr(), self.matrix.shape[1],
                                                        self.gs.data_ptr(), self.qd[b].data_ptr(), self.sd[b].data_ptr(),
                                                        self.sf_cols, _lib.SF_ROW_MAJOR, n, self.cols, 0,
                                                        self.s_k.cuda_stream)
                _lib.check(rc, f"wush_fused_quantize_{self.fmt}")
                self.launches += 1
                ev_k[c] = torch.cuda.Event()
                ev_k[c].record(self.s_k)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_k[c])
                q_host[r0:r0 + n].copy_(self.qd[b][:n], non_blocking=True)
                sf_host[r0:r0 + n].copy_(self.sd[b][:n, : self.groups], non_blocking=True)
                ev_out[c] = torch.cuda.Event()
                ev_out[c].record(self.s_out)
        self.done = ev_out[n_chunks - 1] if n_chunks else start
        torch.cuda.current_stream(self.dev).wait_event(self.done)

    def synchronize(self) -> None:
        self.done.synchronize()
        _lib.check_status(self.dev, "host-streamed quantize")
