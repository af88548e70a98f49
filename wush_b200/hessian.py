"""Hessian accumulation for GPTQ/WUSH calibration, backed by the sm_100a tensor-core kernel.

``accumulate_hessian`` keeps the signature and in-place semantics of the reference's wrapper at
src/quantization/accumulate_hessian.py:112-148.
"""
from __future__ import annotations

import torch

from . import _lib


def accumulate_hessian(mat_hessian: torch.Tensor, mat_input: torch.Tensor, save_lower_only: bool = False,
                       compute_lower_only: bool = True) -> torch.Tensor:
    """In place ``mat_hessian += mat_input^T @ mat_input``; returns ``mat_hessian``.

    mat_hessian: ([meta,] hidden, hidden) fp32, contiguous, on a CUDA device.
    mat_input:   ([meta,] tokens, hidden) bf16, or fp32 (then the products are formed in TF32, like the
                 reference's kernel when its caller passes fp32), contiguous.
    save_lower_only: update only the lower triangle (incl. diagonal) and leave the rest untouched.
    compute_lower_only: kept for signature compatibility; the kernel always computes the lower
        triangle and mirrors it, which gives the same (symmetric) result.
    """
    assert compute_lower_only or not save_lower_only, "compute_lower_only must be True when save_lower_only is True"
    assert mat_hessian.is_contiguous() and mat_input.is_contiguous()
    if not (mat_hessian.is_cuda and mat_input.is_cuda):
        raise _lib.WushB200Error("accumulate_hessian needs CUDA tensors; there is no CPU fallback")
    if mat_hessian.dtype != torch.float32:
        raise ValueError("mat_hessian must be float32")
    if mat_input.dtype not in (torch.bfloat16, torch.float32):
        raise NotImplementedError(f"mat_input dtype {mat_input.dtype}: the kernel takes bfloat16 or float32 activations")
    *meta, tokens, hidden = mat_input.shape
    if tuple(mat_hessian.shape) != (*meta, hidden, hidden):
        raise ValueError(f"shape mismatch: hessian {tuple(mat_hessian.shape)} vs input {tuple(mat_input.shape)}")
    h3 = mat_hessian.view(-1, hidden, hidden)
    x3 = mat_input.view(-1, tokens, hidden)
    lib = _lib.load()
    flags = _lib.HESSIAN_LOWER_ONLY if save_lower_only else 0
    if mat_input.dtype == torch.float32:
        flags |= _lib.HESSIAN_INPUT_F32
    with torch.cuda.device(mat_input.device):
        stream = torch.cuda.current_stream().cuda_stream
        for b in range(h3.shape[0]):
            rc = lib.wush_hessian_accumulate(h3[b].data_ptr(), x3[b].data_ptr(), tokens, hidden, flags,
                                             _lib.status_word(mat_input.device).data_ptr(), stream)
            _lib.check(rc, "wush_hessian_accumulate")
    return mat_hessian


def _hessian_flags(x: torch.Tensor, lower_only: bool, overwrite: bool) -> int:
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise NotImplementedError(f"activation dtype {x.dtype}: the kernel takes bfloat16 or float32")
    return ((_lib.HESSIAN_LOWER_ONLY if lower_only else 0) | (_lib.HESSIAN_INPUT_F32 if x.dtype == torch.float32 else 0)
            | (_lib.HESSIAN_OVERWRITE if overwrite else 0))


def _kernel_accumulate(h: torch.Tensor, x: torch.Tensor, row_begin: int, row_end: int, lower_only: bool,
                       overwrite: bool = False) -> None:
    lib = _lib.load()
    flags = _hessian_flags(x, lower_only, overwrite)
    with torch.cuda.device(x.device):
        rc = lib.wush_hessian_accumulate_rows(h.data_ptr(), x.data_ptr(), x.shape[0], x.shape[1], row_begin, row_end,
                                              flags, _lib.status_word(x.device).data_ptr(),
                                              torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "wush_hessian_accumulate_rows")


def _kernel_accumulate_tiles(h: torch.Tensor, x: torch.Tensor, tile_begin: int, tile_end: int, overwrite: bool) -> None:
    lib = _lib.load()
    flags = _hessian_flags(x, True, overwrite)
    with torch.cuda.device(x.device):
        rc = lib.wush_hessian_accumulate_tiles(h.data_ptr(), x.data_ptr(), x.shape[0], x.shape[1], tile_begin, tile_end,
                                               flags, _lib.status_word(x.device).data_ptr(),
                                               torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "wush_hessian_accumulate_tiles")


def _kernel_finalize(h: torch.Tensor, scale: float) -> None:
    with torch.cuda.device(h.device):
        rc = _lib.load().wush_hessian_finalize(h.data_ptr(), h.shape[0], scale, torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "wush_hessian_finalize")


def _kernel_finalize_count(h: torch.Tensor, count: torch.Tensor) -> None:
    with torch.cuda.device(h.device):
        rc = _lib.load().wush_hessian_finalize_count(h.data_ptr(), h.shape[0], count.data_ptr(),
                                                     torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "wush_hessian_finalize_count")


SEGMENT_TOKENS = 32768


def token_segments(tokens: int) -> list[tuple[int, int]]:
    """(first token, count) of the launches a long input is cut into: 32768 tokens each, the last one up to half
    as much again (the rule the library applies inside one call)."""
    out, t0 = [], 0
    while t0 < tokens:
        left = tokens - t0
        n = left if left < SEGMENT_TOKENS + SEGMENT_TOKENS // 2 else SEGMENT_TOKENS
        out.append((t0, n))
        t0 += n
    return out


def tile_panels(n_tiles: int, per_wave: int, max_panels: int = 7, ratio: float = 2.0,
                max_waves: int = 3) -> list[tuple[int, int]]:
    """Cut the tile list [0, n_tiles) into launches whose cross-GPU combine can overlap the next launch.

    A launch works on `per_wave` tiles side by side, so a launch over a multiple of per_wave tiles wastes
    nothing.  The last panel is the (possibly partly filled) last wave: its combine is the only one nothing
    hides, so it is kept as small as the tile count allows.  The combine of a panel runs while the NEXT panel is
    multiplied and costs (measured, co-resident with the multiply kernel) a bit under half of the panel's own
    multiply time, so the panels before the last shrink geometrically towards the end (each `ratio` times the
    next, whole waves): one wave before the last, then two, four, ... and the first panel takes what is left.
    No panel is longer than `max_waves` waves (longer ones are cut into equal pieces): the combine reads the
    panel's tiles back from every rank, and it runs several times faster while they still sit in the L2 caches
    that the multiply kernel wrote them through (measured at hidden 14336: 0.8 us per tile for a panel of 75 MB
    combined right after it was written, 4.7 us per tile for 113 MB that had been evicted by the next panel's
    input stream -- enough for the side stream to fall behind the multiply kernel)."""
    per_wave = max(1, per_wave)
    waves = -(-n_tiles // per_wave)
    if waves <= 1 or max_panels <= 1:
        return [(0, n_tiles)] if n_tiles else []
    head = waves - 1                                   # full waves before the last one
    sizes, size = [], 1.0
    while head > 0 and len(sizes) < max_panels - 2:
        take = min(head, max(1, int(round(size))))
        sizes.append(take)
        head -= take
        size *= ratio
    if head > 0:
        sizes.append(head)
    sizes.reverse()
    if max_waves >= 1:
        capped = []
        for w in sizes:
            pieces = -(-w // max_waves)
            capped += [w // pieces + (1 if i < w % pieces else 0) for i in range(pieces)]
        sizes = capped
    cuts = [0]
    for w in sizes:
        cuts.append(cuts[-1] + w * per_wave)
    return [(a, b) for a, b in zip(cuts[:-1], cuts[1:])] + [(cuts[-1], n_tiles)]


class _PeerBuffers:
    """A Hessian buffer in symmetric (peer-addressable) memory plus the device-side pointer tables the
    peer-reduce kernel needs.  Creating one is a collective over the group; instances are pooled and
    reused because the rendezvous costs milliseconds.

    When the GPUs sit behind an NVSwitch that can reduce in flight, torch binds the buffer to a multicast
    address as well (`mc_ptr`); the reduce kernel then uses multimem instructions.  WUSH_B200_HESSIAN_MULTIMEM=0
    (or TORCH_SYMM_MEM_DISABLE_MULTICAST=1) keeps it on plain peer loads and stores."""

    _pool: dict = {}

    def __init__(self, hidden: int, device: torch.device, group):
        import os
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        grp = group if group is not None else dist.group.WORLD
        n = hidden * hidden
        # behind the matrix: the int64 token count (16 bytes) and 16 uint32 slots of the in-kernel barrier
        self.flat = symm.empty(n + 4 + 16, dtype=torch.float32, device=device)
        self.handle = symm.rendezvous(self.flat, group=grp)
        self.h = self.flat[:n].view(hidden, hidden)
        self.count = self.flat[n:n + 2].view(torch.int64)
        ptrs = [int(x) for x in self.handle.buffer_ptrs]
        self.rank, self.world = self.handle.rank, self.handle.world_size
        self.buf_table = torch.tensor(ptrs, dtype=torch.int64, device=device)
        self.count_table = torch.tensor([x + 4 * n for x in ptrs], dtype=torch.int64, device=device)
        self.slot_table = torch.tensor([x + 4 * (n + 4) for x in ptrs], dtype=torch.int64, device=device)
        self.flat[n + 4:].zero_()
        torch.cuda.synchronize(device)
        self.handle.barrier(channel=0)            # nobody signals before every rank's slots are zero
        self.epoch = 0
        self.kernel_barrier = os.environ.get("WUSH_B200_HESSIAN_KERNEL_BARRIER", "1") != "0"
        self.mc_ptr = 0
        if os.environ.get("WUSH_B200_HESSIAN_MULTIMEM", "1") != "0":
            try:
                self.mc_ptr = int(self.handle.multicast_ptr or 0)
            except Exception:
                self.mc_ptr = 0
        self.side = torch.cuda.Stream(device=device)
        self.key = (hidden, device.index, id(grp))

    @classmethod
    def acquire(cls, hidden: int, device: torch.device, group):
        import torch.distributed as dist
        grp = group if group is not None else dist.group.WORLD
        free = cls._pool.setdefault((hidden, device.index, id(grp)), [])
        return free.pop() if free else cls(hidden, device, group)

    def release(self) -> None:
        self._pool.setdefault(self.key, []).append(self)

    def combine(self, hidden: int, tile_begin: int, tile_end: int, channel: int, mirror: bool = True) -> None:
        """On the current stream: wait until every rank's partial sums of the tile range are complete, sum them
        across the ranks (scaled by 1 / total tokens), wait until every rank has delivered, rebuild the mirror
        image of the range locally.  The two waits are barriers the reduce and the mirror kernel run themselves
        (WUSH_B200_HESSIAN_KERNEL_BARRIER=0: separate symmetric-memory barrier kernels on `channel`)."""
        lib = _lib.load()
        dev = self.flat.device
        stream = torch.cuda.current_stream(dev).cuda_stream
        status = _lib.status_word(dev).data_ptr()
        slots = self.slot_table.data_ptr() if self.kernel_barrier else None
        if not self.kernel_barrier:
            self.handle.barrier(channel=channel)
        self.epoch += 1
        with torch.cuda.device(dev):
            rc = lib.wush_hessian_peer_reduce(self.buf_table.data_ptr(), self.mc_ptr or None, self.count_table.data_ptr(),
                                              self.rank, self.world, hidden, tile_begin, tile_end, slots, self.epoch,
                                              status, stream)
        _lib.check(rc, "wush_hessian_peer_reduce")
        if mirror:
            self.mirror(hidden, tile_begin, tile_end, channel)

    def mirror(self, hidden: int, tile_begin: int, tile_end: int, channel: int) -> None:
        """On the current stream: wait until every rank has delivered the sums it owns (a barrier the mirror kernel
        runs itself), then rebuild the mirror image of the tile range locally."""
        lib = _lib.load()
        dev = self.flat.device
        stream = torch.cuda.current_stream(dev).cuda_stream
        status = _lib.status_word(dev).data_ptr()
        slots = self.slot_table.data_ptr() if self.kernel_barrier else None
        if not self.kernel_barrier:
            self.handle.barrier(channel=channel)
        self.epoch += 1
        with torch.cuda.device(dev):
            rc = lib.wush_hessian_mirror_tiles(self.h.data_ptr(), hidden, tile_begin, tile_end, self.rank, self.world,
                                               slots, self.epoch, status, stream)
        _lib.check(rc, "wush_hessian_mirror_tiles")


def panel_bounds(hidden: int, panels: int, align: int = 256) -> list[tuple[int, int]]:
    """Row panels of roughly equal lower-triangle area, boundaries on multiples of `align`."""
    cuts = [0]
    for p in range(1, panels):
        r = int(round(hidden * (p / panels) ** 0.5 / align)) * align
        r = min(max(r, cuts[-1]), hidden)
        if r > cuts[-1]:
            cuts.append(r)
    if cuts[-1] < hidden:
        cuts.append(hidden)
    return list(zip(cuts[:-1], cuts[1:]))


class DistributedHessian:
    """Second moment H = (1/N) sum_tokens x^T x with the calibration tokens sharded over the ranks of a
    process group: what ``WUSH.update`` (src/quantization/wush_gptq.py:456-469) maintains on one GPU.

    Each rank adds its own tokens into a raw fp32 sum (lower triangle only, bf16 inputs are not
    rescaled per call, so their products stay exact); the ranks are combined once per Hessian and the
    1/N factor and the mirror image are applied once at the end.

    ``update(x)`` mirrors the calibration hook (one sequence per call).  ``accumulate_overlapped(x)``
    takes all local tokens at once; on several GPUs it cuts the last pass over the tile list into panels and
    combines every finished panel across the GPUs on a side stream while the next one is being multiplied, so
    that only the combine of the last (smallest) panel is not hidden.

    `accumulate_fn` / `finalize_fn` exist so that the host logic can be exercised on CPU ranks
    (gloo) with a stand-in for the CUDA kernels; the defaults call the kernels and need a GPU.
    """

    def __init__(self, hidden: int, device, group=None, panels: int = 7, accumulate_fn=None, finalize_fn=None,
                 peer: bool | None = None, stage_tokens: int | None = None):
        import os
        import torch.distributed as dist
        self.hidden, self.device, self.group, self.panels = hidden, torch.device(device), group, panels
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        # Multi-GPU on CUDA: keep the sum in peer-addressable memory and combine the ranks with the
        # peer-reduce kernel (NVLink / NVSwitch, fused with the scaling).  peer=False, the environment switch
        # WUSH_B200_HESSIAN_PEER=0, injected stand-in functions or a failed symmetric-memory set-up select
        # the NCCL all-reduce of row panels instead.
        if peer is None:
            peer = os.environ.get("WUSH_B200_HESSIAN_PEER", "1") != "0"
        self._peer = None
        kernels = accumulate_fn is None and finalize_fn is None
        if peer and self.world > 1 and self.device.type == "cuda" and kernels:
            try:
                self._peer = _PeerBuffers.acquire(hidden, self.device, group)
            except Exception as exc:   # symmetric memory not available for this group/device
                import warnings
                warnings.warn(f"peer-memory Hessian reduce unavailable ({exc}); using NCCL all-reduce")
        # The kernels' first launch overwrites instead of adding (no zero-fill pass over the buffer); the NCCL
        # path all-reduces rectangular panels, which include never-written entries, and the stand-ins add.
        self._fresh = self._peer is not None or (kernels and self.world == 1 and self.device.type == "cuda")
        if self._peer is not None:
            self.raw = self._peer.h
        elif self._fresh:
            self.raw = torch.empty(hidden, hidden, dtype=torch.float32, device=self.device)
        else:
            self.raw = torch.zeros(hidden, hidden, dtype=torch.float32, device=self.device)
        self.local_tokens = 0
        self._reduced = False
        self._tail = None                     # peer path: tile range whose combine is still to be done
        self._accumulate = accumulate_fn or _kernel_accumulate
        self._finalize = finalize_fn or _kernel_finalize
        self._comm_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        # update() collects short inputs (one calibration sequence per call) in a staging buffer and runs the
        # kernel once per `stage_tokens` tokens: a 2048-token launch spends half its time on the read-modify-
        # write of H and on partly filled waves, a 32768-token one runs at the tensor-core rate.  The buffer is
        # capped at 1 GiB; stage_tokens=0 launches on every call.  All calls must be on one stream.
        self._stage_cap = 32768 if stage_tokens is None else int(stage_tokens)
        self._stage = None
        self._staged = 0
        # measurement hook: a list that receives one (start, end) pair of timing events around the accumulation
        # launches of every accumulate_overlapped() call (the tensor-core part of the job, on its own stream)
        self.profile: list | None = None

    def _add(self, x: torch.Tensor, r0: int, r1: int) -> None:
        """raw (+)= x^T x for rows [r0, r1), lower triangle; the very first launch overwrites."""
        if self._fresh:
            self._accumulate(self.raw, x, r0, r1, True, True)
            self._fresh = False
        else:
            self._accumulate(self.raw, x, r0, r1, True)

    # -- per-call path (calibration hook) ----------------------------------------------------------
    def update(self, x: torch.Tensor) -> None:
        x = x.reshape(-1, x.shape[-1])
        if not x.is_contiguous():
            x = x.contiguous()
        assert not self._reduced, "update after the cross-rank reduction"
        n = x.shape[0]
        cap = min(self._stage_cap, (1 << 30) // max(1, self.hidden * x.element_size()))
        if n == 0:
            return
        if 2 * n > cap:
            # long inputs go straight to the kernel
            self._flush()
            self._add(x, 0, self.hidden)
        else:
            if self._stage is not None and (self._stage.dtype != x.dtype or self._staged + n > self._stage.shape[0]):
                self._flush()
            if self._stage is None or self._stage.dtype != x.dtype:
                self._stage = torch.empty(cap, self.hidden, dtype=x.dtype, device=self.device)
            self._stage[self._staged:self._staged + n].copy_(x)
            self._staged += n
        self.local_tokens += n

    def _flush(self) -> None:
        if self._staged:
            self._add(self._stage[:self._staged], 0, self.hidden)
            self._staged = 0

    # -- all local tokens at once, reduction overlapped with compute --------------------------------
    def accumulate_overlapped(self, x: torch.Tensor) -> None:
        x = x.reshape(-1, x.shape[-1])
        assert not self._reduced
        self._flush()
        cuda = self._comm_stream is not None
        if self.profile is not None and cuda:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
            self.profile.append(ev)
        if self._peer is not None and x.shape[0] > 0:
            self._accumulate_peer(x)
            if self.profile is not None:
                self.profile[-1][1].record()
            return
        if self.world == 1:
            self._add(x, 0, self.hidden)
            self.local_tokens += x.shape[0]
            self._reduced = True
            if self.profile is not None and cuda:
                self.profile[-1][1].record()
            return
        for (r0, r1) in panel_bounds(self.hidden, self.panels):
            self._accumulate(self.raw, x, r0, r1, True)
            if cuda:
                done = torch.cuda.Event()
                done.record()
                self._comm_stream.wait_event(done)
                with torch.cuda.stream(self._comm_stream):
                    self._reduce_panel(r0, r1)
            else:
                self._reduce_panel(r0, r1)
        if self.profile is not None and cuda:
            self.profile[-1][1].record()
        if cuda and self.world > 1:
            torch.cuda.current_stream(self.device).wait_stream(self._comm_stream)
        self.local_tokens += x.shape[0]
        self._reduced = True

    def _accumulate_peer(self, x: torch.Tensor) -> None:
        """Peer-memory path: all but the last 32768-token segment are plain launches over the whole tile list;
        the last segment is launched panel by panel, and every panel but the last is combined across the GPUs
        on the side stream (barrier, reduce kernel, barrier, mirror) while the next panel is multiplied."""
        pb, lib = self._peer, _lib.load()
        self.local_tokens += x.shape[0]
        pb.count.fill_(self.local_tokens)       # read by every rank's reduce kernel after the first barrier
        segs = token_segments(x.shape[0])
        for (t0, n) in segs[:-1]:
            self._add(x[t0:t0 + n], 0, self.hidden)
        t0, n = segs[-1]
        xl = x[t0:t0 + n]
        n_tiles = int(lib.wush_hessian_tile_count(self.hidden))
        import os
        with torch.cuda.device(self.device):
            # WUSH_B200_HESSIAN_TILES_PER_PANEL overrides the device's wave size (small matrices in tests)
            per_wave = int(os.environ.get("WUSH_B200_HESSIAN_TILES_PER_PANEL", "0")) or int(lib.wush_hessian_tiles_per_wave())
        main = torch.cuda.current_stream(self.device)
        panels = tile_panels(n_tiles, per_wave, self.panels,
                             max_waves=int(os.environ.get("WUSH_B200_HESSIAN_PANEL_WAVES", "3")))
        # With many panels the mirror images wait for one pass over the whole matrix at the end: beside the multiply
        # kernel the mirror kernel crawls like the reduce kernel (measured at hidden 14336: together 1.5 ms for a
        # panel the multiply kernel needs 0.75 ms for, so the side stream fell 0.4-0.7 ms behind), alone it moves
        # the 2 x 411 MB in under 0.2 ms.  Small matrices (one or two panels) keep the per-panel mirror, which the
        # next panel hides completely.
        self._mirror_all = len(panels) > 2
        pb.side.wait_stream(main)               # the side stream starts behind everything issued so far
        for i, (a, b) in enumerate(panels):
            _kernel_accumulate_tiles(self.raw, xl, a, b, self._fresh)
            if i + 1 < len(panels):
                done = torch.cuda.Event()
                done.record(main)
                pb.side.wait_event(done)
                with torch.cuda.stream(pb.side):
                    pb.combine(self.hidden, a, b, channel=0, mirror=not self._mirror_all)
        self._fresh = False
        self._tail = panels[-1]
        self._reduced = True

    def _reduce_panel(self, r0: int, r1: int) -> None:
        import torch.distributed as dist
        # only columns [0, r1) of these rows hold data: pack them so the wire carries no zeros
        staged = self.raw[r0:r1, :r1].contiguous()
        dist.all_reduce(staged, group=self.group)
        self.raw[r0:r1, :r1].copy_(staged)

    # -- result ---------------------------------------------------------------------------------------
    def finalize(self) -> torch.Tensor:
        import torch.distributed as dist
        self._flush()
        total = self.local_tokens
        if self._peer is not None:
            pb = self._peer
            main = torch.cuda.current_stream(self.device)
            if self._tail is None:
                # nothing combined yet (update() path, or no tokens at all): one combine over the whole list
                if self._fresh:
                    self.raw.zero_()
                    self._fresh = False
                pb.count.fill_(self.local_tokens)
                self._tail = (0, int(_lib.load().wush_hessian_tile_count(self.hidden)))
            else:
                main.wait_stream(pb.side)       # the earlier panels are combined and mirrored
            defer = getattr(self, "_mirror_all", False)
            pb.combine(self.hidden, self._tail[0], self._tail[1], channel=1, mirror=not defer)
            if defer:
                pb.mirror(self.hidden, 0, int(_lib.load().wush_hessian_tile_count(self.hidden)), channel=1)
                self._mirror_all = False
            self._tail = None
            self._reduced = True
            self._count = None                    # total is computed on demand (num_samples)
            return self.raw
        if self._fresh:
            self.raw.zero_()
            self._fresh = False
        if self.world > 1:
            if not self._reduced:
                for (r0, r1) in panel_bounds(self.hidden, self.panels):
                    self._reduce_panel(r0, r1)
                self._reduced = True
            n = torch.tensor([self.local_tokens], dtype=torch.int64, device=self.device)
            dist.all_reduce(n, group=self.group)
            self._count = n
            if self._finalize is _kernel_finalize:
                # the count stays on the device: no host synchronisation inside the job
                _kernel_finalize_count(self.raw, n)
                return self.raw
            total = int(n.item())
        self._finalize(self.raw, 1.0 / max(total, 1))
        self._count = total
        return self.raw

    @property
    def num_samples(self) -> int:
        """Tokens over all ranks (reads the device-side count if the reduction left it there).  A host
        synchronisation point: a device-side timeout reported by any of the kernels raises here."""
        c = getattr(self, "_count", self.local_tokens)
        if c is None:
            import torch.distributed as dist
            n = torch.tensor([self.local_tokens], dtype=torch.int64, device=self.device)
            dist.all_reduce(n, group=self.group)
            c = self._count = int(n.item())
        if self.device.type == "cuda" and self._accumulate is _kernel_accumulate:
            _lib.check_status(self.device, "Hessian accumulation")
        return int(c.item()) if isinstance(c, torch.Tensor) else int(c)

    def release(self) -> None:
        """Give a peer-memory buffer back to the pool (the matrix returned by finalize() is then reused by
        the next DistributedHessian of the same size).  No-op for ordinary buffers."""
        if self._peer is not None:
            self._peer.release()
            self._peer = None
