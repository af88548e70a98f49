"""One decoder block with all seven linear layers in W4A4 and their weights column-sharded over the GPUs of a
process group -- the multi-GPU form of the reference's quantized layer (FPQuantLinear / FPQuant4x16NoMasterFn,
inference_lib/src/fp_quant/module/linear.py:267-386, linear_fns.py:494-539) for models whose layers are spread
over a node (hidden 8192, 64 query / 8 key-value heads, FFN 28672 by default).  The reference is single-GPU; what
is kept from it is the per-layer arithmetic: fused transform + quantize of the layer input, block-scaled FP4 GEMM,
bias / residual.

Partitioning.  Every linear layer is split by OUTPUT features (weight rows), and the residual stream is kept
column-sharded: rank r holds columns [r, r+1) * hidden / world of every token.
  * q/k/v: rank r owns the rows of its own heads (64/world query heads, 8/world key-value heads), so attention
    runs on local heads only and its output is exactly rank r's column shard of the o_proj input;
  * gate/up: rank r owns rows [r, r+1) * ffn / world of both, so SwiGLU is local and its output is rank r's column
    shard of the down_proj input;
  * o_proj / down_proj: rank r owns output columns [r, r+1) * hidden / world = its shard of the residual stream, and
    adds the residual in the GEMM's epilogue.
What a GEMM needs from the other ranks is the rest of its K dimension.  Scale groups never straddle a shard, so
every rank runs the fused transform + quantize kernel on the columns it holds and ships FP4 codes + scale bytes
(0.53 bytes per element instead of 2 for bf16) into the same slot of every rank's operand buffer: one contiguous
device-to-device copy per peer, which the copy engines carry over NVLink while the SMs multiply.  The GEMM reads its
activations as a stack of K shards (`rows=` of qutlass_ops.matmul_fp4_blocked).  RMSNorm needs the sum of squares of
whole rows: the per-rank partial sums (4 bytes per token) travel the same way, and the normalisation itself is folded
into the quantize kernel (its row_scale / col_scale prologue), as SwiGLU is a single pass.

Overlap.  The tokens are cut into micro-batches that run on separate streams: while one micro-batch multiplies, the
codes of the other are in flight.  Buffers live in torch symmetric memory; a stage's exchange ends with one
cross-rank barrier on its stream.  No collective library call and no multicast is involved.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import _lib
from . import qutlass_ops as ops


@dataclass
class BlockConfig:
    hidden: int = 8192
    n_heads: int = 64
    n_kv_heads: int = 8
    ffn: int = 28672
    head_dim: int = 128
    fmt: str = "mx"               # "mx" (MXFP4) or "nv" (NVFP4)
    rms_eps: float = 1e-5

    @property
    def group(self) -> int:
        return 32 if self.fmt == "mx" else 16


LAYERS = ("qkv", "o", "gate_up", "down")


def quantize_block_weights(cfg: BlockConfig, weights: dict, transforms: dict, device) -> dict:
    """Quantize the seven bf16 weight matrices of a block with the fused kernel (rows are independent, so a row
    shard of the result is the result of the row shard).  weights: 'q','k','v','o','gate','up','down' [out, in];
    transforms: 'attn_in' (shared by q/k/v), 'o', 'mlp_in' (shared by gate/up), 'down': bf16 [G, in] per-group
    matrices or [G, G] shared.  Returns name -> (codes u8 [out, in/2], scales u8 [out, in/G])."""
    gs = torch.tensor([10.0], device=device) if cfg.fmt == "nv" else None
    tmap = {"q": "attn_in", "k": "attn_in", "v": "attn_in", "o": "o", "gate": "mlp_in", "up": "mlp_in", "down": "down"}
    out = {}
    for name, w in weights.items():
        q, sf = ops._quantize(w.to(device), transforms[tmap[name]].to(device), cfg.fmt, gs)
        out[name] = (q, sf[: w.shape[0], : w.shape[1] // cfg.group].contiguous())
    return out


def _broadcast(flat: torch.Tensor, handle, peers, rank: int, world: int, lo: int, hi: int, table) -> None:
    """Elements [lo, hi) of this rank's symmetric buffer `flat` into the same place of every other rank's buffer on
    the current stream.  Default: one device-to-device copy per peer, carried by
    the copy engines while the SMs multiply.  WUSH_B200_BLOCK_BROADCAST=1: one kernel launch instead, through the
    buffer's multicast address when it has one (the data leaves this GPU once and the NVSwitch replicates it;
    WUSH_B200_BLOCK_MULTIMEM=0: plain stores to each peer).  Measured per block: 2 GPUs 9.6 ms (copies) / 10.0 (plain
    stores) / 10.6 (multicast); 8 GPUs 4.68 / 4.60 / 4.55 ms -- the SM-driven forms take time from the GEMMs and only
    pay once seven copies per exchange are replaced."""
    import os
    if os.environ.get("WUSH_B200_BLOCK_BROADCAST", "0") != "1":
        for i in range(1, world):
            p = (rank + i) % world                                          # every rank starts with another peer
            peers[p][lo:hi].copy_(flat[lo:hi], non_blocking=True)
        return
    esz = flat.element_size()
    mc = int(getattr(handle, "multicast_ptr", 0) or 0) if os.environ.get("WUSH_B200_BLOCK_MULTIMEM", "1") == "1" else 0
    lib = _lib.load()
    with torch.cuda.device(flat.device):
        rc = lib.wush_peer_broadcast(flat.data_ptr() + lo * esz, (mc + lo * esz) if mc else None,
                                     None if mc else table(lo), 0 if mc else world - 1, (hi - lo) * esz,
                                     torch.cuda.current_stream(flat.device).cuda_stream)
    _lib.check(rc, "wush_peer_broadcast")


def _peer_table(peers, rank: int, world: int):
    """lo -> ctypes array of the other ranks' addresses of element `lo` (cached per offset)."""
    import ctypes
    cache = {}

    def table(lo: int):
        t = cache.get(lo)
        if t is None:
            esz = peers[0].element_size()
            t = cache[lo] = (ctypes.c_void_p * (world - 1))(*[peers[(rank + i) % world].data_ptr() + lo * esz
                                                              for i in range(1, world)])
        return t
    return table


class _Exchange:
    """Operand buffer of one GEMM input in symmetric memory: `world` slots, slot s holding the codes and the blocked
    scale bytes rank s produced for its K shard.  put(): quantize the local columns into the own slot, copy the slot
    into every peer's buffer, barrier."""

    def __init__(self, rows: int, k_shard: int, group_size: int, world: int, rank: int, device, pg):
        self.rows, self.ks, self.g, self.world, self.rank = rows, k_shard, group_size, world, rank
        pitch = k_shard // 2
        code_bytes = rows * pitch
        sf_bytes = (rows + 127) // 128 * 128 * (k_shard // group_size)
        slot = code_bytes + sf_bytes
        slot = (slot + pitch * 16 - 1) // (pitch * 16) * (pitch * 16)     # whole rows of the code matrix, 16-byte multiple
        self.slot, self.code_bytes, self.pitch = slot, code_bytes, pitch
        self.rows_per_slot = slot // pitch
        if world > 1:
            import torch.distributed._symmetric_memory as symm
            self.flat = symm.empty(world * slot, dtype=torch.uint8, device=device)
            self.handle = symm.rendezvous(self.flat, group=pg)
            self.peers = [self.handle.get_buffer(p, (world * slot,), torch.uint8) for p in range(world)]
            self.table = _peer_table(self.peers, rank, world)
        else:
            self.flat = torch.empty(slot, dtype=torch.uint8, device=device)
            self.handle, self.peers = None, [self.flat]
        mine = self.flat[rank * slot:(rank + 1) * slot]
        self.my_codes = mine[:code_bytes].view(rows, pitch)
        self.my_scales = mine[code_bytes:code_bytes + sf_bytes]
        self.codes = self.flat.view(world, self.rows_per_slot, pitch)      # the GEMM's stacked operand
        self.scales = self.flat[code_bytes:]                               # first scale tensor; the others `slot` bytes on

    def put(self, x: torch.Tensor, matrix: torch.Tensor, fmt: str, gs, row_scale=None, col_scale=None) -> None:
        m = x.shape[0]
        ops.fused_quantize_into(x, matrix, fmt, gs, self.my_codes[:m], self.my_scales, col0=0, sf_layout=_lib.SF_BLOCKED,
                                row_scale=row_scale, col_scale=col_scale)
        if self.world > 1:
            lo, hi = self.rank * self.slot, (self.rank + 1) * self.slot
            _broadcast(self.flat, self.handle, self.peers, self.rank, self.world, lo, hi, self.table)
            self.handle.barrier(channel=0)

    def gemm(self, m: int, w: torch.Tensor, ws_blocked: torch.Tensor, alpha: torch.Tensor, fmt: str, **kw) -> torch.Tensor:
        if self.world == 1:
            return ops.matmul_fp4_blocked(self.my_codes[:m], w, self.my_scales, ws_blocked, alpha, fmt, **kw)
        return ops.matmul_fp4_blocked(self.codes, w, self.scales, ws_blocked, alpha, fmt, rows=m,
                                      scale_shard_bytes=self.slot, **kw)


class _RowSums:
    """Sum over the ranks of one fp32 value per token (the squared norm of a row of the sharded residual stream)."""

    def __init__(self, rows: int, world: int, rank: int, device, pg):
        self.rows, self.world, self.rank = rows, world, rank
        if world > 1:
            import torch.distributed._symmetric_memory as symm
            self.flat = symm.empty(world * rows, dtype=torch.float32, device=device)
            self.handle = symm.rendezvous(self.flat, group=pg)
            self.peers = [self.handle.get_buffer(p, (world * rows,), torch.float32) for p in range(world)]
            self.table = _peer_table(self.peers, rank, world)

    def total(self, partial: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return partial
        m = partial.shape[0]
        lo = self.rank * self.rows
        self.flat[lo:lo + m].copy_(partial)
        _broadcast(self.flat, self.handle, self.peers, self.rank, self.world, lo, lo + m, self.table)
        self.handle.barrier(channel=0)
        return self.flat.view(self.world, self.rows)[:, :m].sum(0)          # fixed order: the same bits on every rank


class ShardedDecoderBlock:
    """forward(h_local) for one decoder block; h_local is this rank's column shard [tokens, hidden / world] of the
    residual stream (bf16), tokens = sequences * seq_len, and is updated in place.

    qweights   what quantize_block_weights returned for the FULL matrices (every rank passes the same; the rows of
               its own shard are taken here), or already the shard when `presharded`
    transforms 'attn_in', 'o', 'mlp_in', 'down': bf16 [G, in_features] per-group matrices or [G, G] shared
    """

    def __init__(self, cfg: BlockConfig, qweights: dict, transforms: dict, gammas: tuple, seq_len: int,
                 max_tokens: int, device, group=None, micro_batches: int = 2, local_only: bool = False):
        import torch.distributed as dist
        # local_only: the whole block on this GPU even inside a multi-GPU job (e.g. as the comparison for the sharded one)
        on = dist.is_available() and dist.is_initialized() and not local_only
        self.world = dist.get_world_size(group) if on else 1
        self.rank = dist.get_rank(group) if on else 0
        pg = (group if group is not None else dist.group.WORLD) if on else None
        self.cfg, self.dev, self.seq_len = cfg, torch.device(device), seq_len
        w, r, d = self.world, self.rank, cfg.head_dim
        if cfg.n_kv_heads % w or cfg.n_heads % w or (cfg.hidden // w) % 256 or (cfg.ffn // w) % 256:
            raise ValueError("heads must divide evenly and hidden / world, ffn / world must be multiples of 256")
        self.hq, self.hkv = cfg.n_heads // w, cfg.n_kv_heads // w
        self.hs, self.fs = cfg.hidden // w, cfg.ffn // w                     # shard widths of hidden and ffn
        rows = lambda t, n: t[r * n:(r + 1) * n]
        cat = lambda parts: tuple(torch.cat([p[i] for p in parts]).contiguous() for i in (0, 1))
        shard = {
            "qkv": cat([tuple(rows(t, self.hq * d) for t in qweights["q"]), tuple(rows(t, self.hkv * d) for t in qweights["k"]),
                        tuple(rows(t, self.hkv * d) for t in qweights["v"])]),
            "o": tuple(rows(t, self.hs).contiguous() for t in qweights["o"]),
            "gate_up": cat([tuple(rows(t, self.fs) for t in qweights["gate"]), tuple(rows(t, self.fs) for t in qweights["up"])]),
            "down": tuple(rows(t, self.hs).contiguous() for t in qweights["down"]),
        }
        self.w = {k: (q, ops.to_blocked(s).view(-1)) for k, (q, s) in shard.items()}
        # this rank's columns of every input transform (per-group matrices are column-local; a shared one is kept)
        cols = {"attn_in": self.hs, "o": self.hs, "mlp_in": self.hs, "down": self.fs}
        self.t = {k: (m if m.shape[1] == cfg.group else m[:, r * cols[k]:(r + 1) * cols[k]]).to(self.dev).contiguous()
                  for k, m in transforms.items()}
        self.gamma = tuple(g[r * self.hs:(r + 1) * self.hs].to(self.dev).contiguous() for g in gammas)
        gsv = 3.0 if cfg.fmt == "mx" else 10.0
        self.alpha = torch.tensor([1.0 / (gsv * gsv)], dtype=torch.float32, device=self.dev)
        self.gs = torch.tensor([10.0], device=self.dev) if cfg.fmt == "nv" else None
        if max_tokens % (micro_batches * seq_len):
            raise ValueError("max_tokens must be a multiple of micro_batches * seq_len")
        self.mb_rows = max_tokens // micro_batches
        self.streams = [torch.cuda.Stream(device=self.dev) for _ in range(micro_batches)]
        mk = lambda ks: _Exchange(self.mb_rows, ks, cfg.group, w, r, self.dev, pg)
        # per micro-batch: two hidden-wide operand buffers used alternately (a peer may already be filling the next
        # one while this rank still multiplies from the previous one), one ffn-wide, one row-sum buffer per norm
        self.slots = [{"h": (mk(self.hs), mk(self.hs)), "f": mk(self.fs),
                       "ssq": (_RowSums(self.mb_rows, w, r, self.dev, pg), _RowSums(self.mb_rows, w, r, self.dev, pg))}
                      for _ in range(micro_batches)]

    # -- pieces ---------------------------------------------------------------------------------------------
    def _rstd(self, h: torch.Tensor, sums: _RowSums) -> torch.Tensor:
        """1 / rms of every WHOLE row of the residual stream: local sums of squares, added over the ranks.  The
        scaling itself (and the norm's weight) is applied inside the quantize kernel that follows."""
        total = sums.total(ops.row_sumsq(h))
        return torch.rsqrt(total / self.cfg.hidden + self.cfg.rms_eps)

    def _attention(self, qkv: torch.Tensor) -> torch.Tensor:
        d, s = self.cfg.head_dim, self.seq_len
        b = qkv.shape[0] // s
        t = qkv.view(b, s, self.hq + 2 * self.hkv, d)
        q = t[:, :, : self.hq].transpose(1, 2)
        k = t[:, :, self.hq: self.hq + self.hkv].transpose(1, 2)
        v = t[:, :, self.hq + self.hkv:].transpose(1, 2)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.hq != self.hkv)
        return o.transpose(1, 2).reshape(qkv.shape[0], self.hq * d)

    def _micro_batch(self, h: torch.Tensor, slot: dict) -> None:
        cfg, fmt, m = self.cfg, self.cfg.fmt, h.shape[0]
        a, b = slot["h"]
        # attention half
        a.put(h, self.t["attn_in"], fmt, self.gs, row_scale=self._rstd(h, slot["ssq"][0]), col_scale=self.gamma[0])
        qkv = a.gemm(m, *self.w["qkv"], self.alpha, fmt)
        b.put(self._attention(qkv), self.t["o"], fmt, self.gs)
        b.gemm(m, *self.w["o"], self.alpha, fmt, residual=h, out=h)            # h += o_proj(...) in the epilogue
        # MLP half
        a.put(h, self.t["mlp_in"], fmt, self.gs, row_scale=self._rstd(h, slot["ssq"][1]), col_scale=self.gamma[1])
        gu = a.gemm(m, *self.w["gate_up"], self.alpha, fmt)
        slot["f"].put(ops.swiglu(gu[:, : self.fs], gu[:, self.fs:]), self.t["down"], fmt, self.gs)
        slot["f"].gemm(m, *self.w["down"], self.alpha, fmt, residual=h, out=h)
        del cfg

    def forward(self, h_local: torch.Tensor) -> torch.Tensor:
        if h_local.dtype != torch.bfloat16 or h_local.shape[1] != self.hs or not h_local.is_contiguous():
            raise ValueError(f"h_local must be a contiguous bfloat16 [tokens, {self.hs}] tensor")
        tokens = h_local.shape[0]
        if tokens % self.seq_len or tokens > self.mb_rows * len(self.streams):
            raise ValueError("tokens must be whole sequences and fit the buffers")
        seqs = tokens // self.seq_len
        per = -(-seqs // len(self.streams)) * self.seq_len
        main = torch.cuda.current_stream(self.dev)
        for j, st in enumerate(self.streams):
            lo, hi = j * per, min((j + 1) * per, tokens)
            if lo >= hi:
                # every rank issues the same barriers: an empty micro-batch still takes part in none, because all
                # ranks see the same token count
                continue
            st.wait_stream(main)
            with torch.cuda.stream(st):
                self._micro_batch(h_local[lo:hi], self.slots[j])
        for st in self.streams:
            main.wait_stream(st)
        return h_local
