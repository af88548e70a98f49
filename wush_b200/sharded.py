"""FP4 linear layer with column-sharded weights: the output features (weight rows) are split over the ranks of
a process group, activations are replicated, and every rank ends up with the complete output.

The GEMM kernel's epilogue writes each finished tile into the same place of every rank's output buffer (torch
symmetric memory, plain NVLink stores), so the all-gather of the output columns happens inside the GEMM instead
of after it; two symmetric-memory barriers fence the buffers.  ``peer=False`` (or a failed symmetric-memory
set-up, or a CPU stand-in for the kernel) selects the baseline: local GEMM, then an NCCL all-gather.

The reference is single-GPU; this is the multi-GPU form of its ``forward_gemm``
(inference_lib/src/fp_quant/module/linear_fns.py:65-76) for layers too large for one GPU.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib


def shard_bounds(n_total: int, world: int, rank: int) -> tuple[int, int]:
    """Output features [begin, end) of `rank`: equal shards, which must be multiples of 8 columns."""
    if n_total % (8 * world):
        raise ValueError(f"out_features ({n_total}) must be a multiple of 8 * world ({8 * world})")
    per = n_total // world
    return rank * per, (rank + 1) * per


class ColumnShardedFP4Linear:
    """y = alpha * deq(x) @ deq(W)^T with W's rows sharded over the group.

    qweight_shard  uint8 [N/world, K/2]   this rank's packed E2M1 rows
    scales_shard   uint8 / float8 [N/world, K/G] this rank's scales, row-major (swizzled once here)
    """

    def __init__(self, qweight_shard: torch.Tensor, scales_shard: torch.Tensor, n_total: int, fmt: str = "mx",
                 alpha: float = 1.0 / 9.0, group=None, max_tokens: int = 32768, peer: bool | None = None, gemm_fn=None):
        import torch.distributed as dist
        self.fmt, self.n_total, self.group = fmt, n_total, group
        self.dev = qweight_shard.device
        on = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if on else 1
        self.rank = dist.get_rank(group) if on else 0
        self.col0, col1 = shard_bounds(n_total, self.world, self.rank)
        self.n_shard = col1 - self.col0
        if qweight_shard.shape[0] != self.n_shard:
            raise ValueError("qweight_shard must hold this rank's N/world rows")
        self.k = qweight_shard.shape[1] * 2
        self.qweight = qweight_shard.contiguous()
        self._gemm_fn = gemm_fn
        if gemm_fn is None:
            from . import qutlass_ops as ops
            self.ws = ops.to_blocked(scales_shard.view(torch.uint8)).view(-1)
        else:
            self.ws = scales_shard
        self.alpha = torch.tensor([alpha], dtype=torch.float32, device=self.dev)
        self.max_tokens = max_tokens
        if peer is None:
            peer = os.environ.get("WUSH_B200_GEMM_PEER", "1") != "0"
        self._handle = None
        if peer and self.world > 1 and self.dev.type == "cuda" and gemm_fn is None:
            try:
                import torch.distributed._symmetric_memory as symm
                os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only
                grp = group if group is not None else dist.group.WORLD
                self._flat = symm.empty(max_tokens * n_total, dtype=torch.bfloat16, device=self.dev)
                self._handle = symm.rendezvous(self._flat, group=grp)
                ptrs = [int(p) for p in self._handle.buffer_ptrs]
                self._ptr_array = (ctypes.c_void_p * self.world)(*ptrs)
            except Exception as exc:   # symmetric memory not available for this group/device
                import warnings
                warnings.warn(f"peer-memory output buffers unavailable ({exc}); using NCCL all-gather")
                self._handle = None

    @property
    def fused(self) -> bool:
        return self._handle is not None

    def forward(self, xq: torch.Tensor, xs_blocked: torch.Tensor) -> torch.Tensor:
        """xq: uint8 [M, K/2] packed activations (replicated on every rank), xs_blocked: their scales in the
        blocked layout.  Returns bf16 [M, N] -- with peer memory a view of the layer's output buffer, valid
        until the next forward()."""
        m = xq.shape[0]
        if self._handle is not None:
            if m > self.max_tokens:
                raise ValueError(f"{m} tokens exceed the output buffer ({self.max_tokens})")
            lib = _lib.load()
            fmt = _lib.FORMAT_MXFP4 if self.fmt == "mx" else _lib.FORMAT_NVFP4
            self._handle.barrier(channel=0)       # nobody still reads the previous output
            with torch.cuda.device(self.dev):
                rc = lib.wush_gemm_fp4_bf16_tn_sharded(fmt, xq.data_ptr(), self.qweight.data_ptr(), xs_blocked.data_ptr(),
                                                       self.ws.data_ptr(), self.alpha.data_ptr(), self._ptr_array,
                                                       self.world, self.rank, self.n_total, self.col0, m, self.n_shard,
                                                       self.k, _lib.status_word(self.dev).data_ptr(),
                                                       torch.cuda.current_stream().cuda_stream)
            _lib.check(rc, "wush_gemm_fp4_bf16_tn_sharded")
            self._handle.barrier(channel=1)       # every rank's columns have landed everywhere
            return self._flat[: m * self.n_total].view(m, self.n_total)
        # baseline: local GEMM, then all-gather of the column shards
        if self._gemm_fn is not None:
            y_local = self._gemm_fn(xq, self.qweight, xs_blocked, self.ws)
        else:
            from . import qutlass_ops as ops
            y_local = ops.matmul_fp4_blocked(xq, self.qweight, xs_blocked, self.ws, self.alpha, self.fmt)
        if self.world == 1:
            return y_local
        import torch.distributed as dist
        gathered = torch.empty(self.world * m, self.n_shard, dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(gathered, y_local.contiguous(), group=self.group)
        return gathered.view(self.world, m, self.n_shard).permute(1, 0, 2).reshape(m, self.n_total)
