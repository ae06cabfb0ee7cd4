"""Multi-GPU use of the operator: one process per GPU, ``torch.distributed`` for the plumbing.

Two ways the path shards (the reference itself is single-GPU, so this is new):

* **Data parallel over scenes** (``SceneParallelLayer``): every rank holds its own point cloud and a
  replica of the weights.  Forward and dgrad need no communication.  The weight gradient is the
  one real exchange step: each rank's fp32 partial ``[k_vol, c_in, c_out]`` is summed with a single
  all-reduce (NCCL over NVLink on GPUs, gloo on CPU in the tests) and then folded into the
  caller's ``kernel_grad``.
* **One scene split over ranks** (``shard_pairs_by_rows``): the pair list of a kernel map is cut by
  *output-row range* for the forward (each rank owns a contiguous block of output rows, so no two
  ranks ever accumulate into the same row) and by *input-row range* for dgrad; any disjoint cut
  serves wgrad, whose partial sums are all-reduced as above.  Range boundaries are placed on the
  cumulative pair histogram so that ranks get equal pair counts, not equal row counts.

The host-side index work here is NumPy; the per-rank compute is the CUDA operator.
"""
from __future__ import annotations

import numpy as np

from .maps import KernelMap

__all__ = ["balanced_row_ranges", "shard_pairs_by_rows", "shard_map_device", "MapShard", "allreduce_sum_",
           "SceneParallelLayer", "BoundSceneLayer", "PeerExchange"]


def balanced_row_ranges(rows: np.ndarray, n_rows: int, world: int) -> np.ndarray:
    """Boundaries ``b[0]=0 <= ... <= b[world]=n_rows`` such that the number of pairs whose row
    falls in ``[b[r], b[r+1])`` is as equal as a contiguous cut allows."""
    hist = np.bincount(rows, minlength=n_rows).astype(np.int64) if rows.size else np.zeros(n_rows, np.int64)
    cum = np.concatenate([[0], np.cumsum(hist)])
    total = int(cum[-1])
    bounds = np.zeros(world + 1, dtype=np.int64)
    bounds[world] = n_rows
    for r in range(1, world):
        bounds[r] = int(np.searchsorted(cum, total * r / world, side="left"))
    return np.maximum.accumulate(np.minimum(bounds, n_rows))


def shard_pairs_by_rows(km: KernelMap, world: int, by: str = "out"):
    """Cut a kernel map into ``world`` kernel maps over the same voxel rows.

    ``by="out"``: rank r gets exactly the pairs whose output row lies in its range (forward);
    ``by="in"``: the same by input row (dgrad).  Offset-major order and the order inside each
    offset are kept, and ``kpos`` is re-derived per rank.  Returns ``(shards, bounds)``.
    """
    key = km.omap if by == "out" else km.imap
    n_rows = km.n_out if by == "out" else km.n_in
    bounds = balanced_row_ranges(key, n_rows, world)
    seg = np.repeat(np.arange(km.k_vol), km.knnz)
    owner = np.searchsorted(bounds, key, side="right") - 1
    owner = np.clip(owner, 0, world - 1)
    shards = []
    for r in range(world):
        sel = owner == r
        knnz = np.bincount(seg[sel], minlength=km.k_vol).astype(np.int32)
        kpos = np.zeros(km.k_vol + 1, dtype=np.int32)
        np.cumsum(knnz, out=kpos[1:])
        shards.append(KernelMap(km.n_in, km.n_out, km.k_vol, knnz, kpos,
                                np.ascontiguousarray(km.imap[sel]), np.ascontiguousarray(km.omap[sel]),
                                km.out_coords))
    return shards, bounds


class MapShard:
    """One rank's cut of a kernel map, as tensors on the device of the map it was cut from."""

    def __init__(self, kpos, imap, omap, row_range):
        self.kpos, self.imap, self.omap, self.row_range = kpos, imap, omap, row_range

    @property
    def pairs(self) -> int:
        return int(self.imap.numel())


def shard_map_device(kpos, imap, omap, n_rows: int, rank: int, world: int, by: str = "out") -> MapShard:
    """``shard_pairs_by_rows`` for one rank, computed where the map lives (tensor operations on the map's own
    device; nothing is copied to the host but the two range boundaries).

    The row ranges are the same balanced ones: boundaries on the cumulative pair histogram of the key map
    (``out_map`` for ``by="out"``, ``in_map`` for ``by="in"``).  The rank keeps the pairs whose key row falls
    in its range, in their original order, and ``kpos`` is re-derived from the per-offset counts of the kept
    pairs.  Every rank computes the same boundaries from the same map, so no communication is needed."""
    import torch
    key = omap if by == "out" else imap
    k_vol = kpos.numel() - 1
    pairs = key.numel()
    key64 = key.long()
    hist = torch.bincount(key64, minlength=n_rows) if pairs else torch.zeros(n_rows, dtype=torch.long, device=key.device)
    cum = torch.cat([hist.new_zeros(1), torch.cumsum(hist, 0)])
    total = int(pairs)
    # first row index whose cumulative count reaches total * r / world  (numpy: searchsorted(cum, x, side="left"))
    targets = torch.tensor([total * r / world for r in (rank, rank + 1)], dtype=torch.float64, device=key.device)
    b = torch.searchsorted(cum.double(), targets, right=False).clamp(max=n_rows).tolist()
    lo = 0 if rank == 0 else int(b[0])
    hi = n_rows if rank == world - 1 else int(b[1])
    hi = max(hi, lo)
    keep = (key64 >= lo) & (key64 < hi)
    seg = torch.searchsorted(kpos[1:].long().contiguous(), torch.arange(pairs, device=key.device), right=True)
    knnz = torch.bincount(seg[keep], minlength=k_vol)[:k_vol]
    new_kpos = torch.cat([knnz.new_zeros(1), torch.cumsum(knnz, 0)]).to(torch.int32)
    return MapShard(new_kpos.contiguous(), imap[keep].contiguous(), omap[keep].contiguous(), (lo, hi))


def world_size(group=None) -> int:
    """Ranks in ``group`` (1 outside an initialised process group)."""
    import torch.distributed as dist

    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def allreduce_sum_(tensor, group=None):
    """In-place sum over all ranks; a no-op outside an initialised process group."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=group)
    return tensor


class PeerExchange:
    """Sum of every rank's fp32 partial sums over peer memory instead of an NCCL all-reduce
    (``fgms_b200_peer_exchange``, ``csrc/peer_exchange.cuh``).

    The ranks' buffers come from PyTorch's symmetric-memory allocator (one allocation per rank, mapped into every
    process of ``group``); the library's kernel reads and writes them with plain loads and stores.  ``sums`` is
    this rank's input (use it as the weight-gradient workspace), ``reduced`` receives the totals.  ``run()``
    enqueues the kernel on ``stream`` — meant to be a side stream, so that the kernel (a few small CTAs) runs
    beside the input-gradient kernel where NCCL's would wait for its SMs.

    With one rank (or ``buffers`` given: pointer tables of an emulated group on one device, used by the tests)
    no symmetric memory is involved.
    """

    def __init__(self, count: int, device, group=None, ctas: int = 0, wait_limit_cycles: int = 0, buffers=None):
        import ctypes
        import torch
        from . import _lib
        self._L, self._check = _lib.lib, _lib.check
        self.device = torch.device(device)
        self.count = (int(count) + 3) // 4 * 4
        self.group = group
        # CTAs of 128 threads and 32 registers, one per 2048 values of the buffer: between 16 and 128 (at most one per
        # SM, resident all at once beside a persistent kernel) for buffers of up to 4 MB; up to 512 for larger ones,
        # which are bound by the bytes in flight over the link (a few of these CTAs fit an SM beside a persistent one)
        self.ctas = int(ctas) if ctas else max(16, min(128 if self.count <= (1 << 20) else 512, self.count // 2048))
        self.wait_limit = int(wait_limit_cycles)
        if buffers is not None:
            self.rank, self.world, sums, reduced, flags = buffers
            self.sums, self.reduced = sums[self.rank], reduced[self.rank]
            ptrs = ([t.data_ptr() for t in sums], [t.data_ptr() for t in reduced], [t.data_ptr() for t in flags])
            self._keep = (sums, reduced, flags)
        else:
            self.world = world_size(group)
            flag_bytes = self._L.fgms_b200_peer_exchange_flag_bytes(max(self.world, 1))
            n_flag = flag_bytes // 4
            total = 2 * self.count + n_flag
            if self.world > 1:
                import torch.distributed as dist
                import torch.distributed._symmetric_memory as symm_mem
                self.rank = dist.get_rank(group)
                buf = symm_mem.empty(total, dtype=torch.float32, device=self.device)
                buf.zero_()
                handle = symm_mem.rendezvous(buf, group if group is not None else dist.group.WORLD)
                torch.cuda.synchronize(self.device)
                dist.barrier(group)  # every rank's flags are zero before anyone's first call
                base = [int(p) for p in handle.buffer_ptrs]
                self._keep = (buf, handle)
            else:
                self.rank = 0
                buf = torch.zeros(total, dtype=torch.float32, device=self.device)
                base = [buf.data_ptr()]
                self._keep = (buf,)
            self.sums, self.reduced = buf[: self.count], buf[self.count: 2 * self.count]
            ptrs = (base, [b + 4 * self.count for b in base], [b + 8 * self.count for b in base])
        self._ptrs = ptrs
        self._ranges = {}

    def _tables(self, lo: int, hi: int):
        """Pointer tables of the element range [lo, hi) of every rank's buffers (built once per range)."""
        import ctypes
        t = self._ranges.get((lo, hi))
        if t is None:
            arr = ctypes.c_void_p * self.world
            t = (arr(*[b + 4 * lo for b in self._ptrs[0]]), arr(*[b + 4 * lo for b in self._ptrs[1]]), arr(*self._ptrs[2]))
            self._ranges[(lo, hi)] = t
        return t

    def run(self, stream=None, lo: int = 0, hi: int | None = None):
        """Enqueue one exchange of the elements [lo, hi) (default: all).  Every rank of the group must make the
        same calls in the same order; calls on one object must be enqueued on one stream."""
        import torch
        hi = self.count if hi is None else hi
        if lo % 4 or hi % 4 or not 0 <= lo <= hi <= self.count:
            raise ValueError("range bounds must be multiples of 4 inside the buffer")
        sums, reduced, flags = self._tables(lo, hi)
        st = (stream if stream is not None else torch.cuda.current_stream(self.device)).cuda_stream
        with torch.cuda.device(self.device):
            # epoch 0: the kernel numbers its calls on the device, so the launch may be replayed from a CUDA graph
            self._check(self._L.fgms_b200_peer_exchange(sums, reduced, flags, self.rank, self.world, hi - lo, 0,
                                                        self.wait_limit, self.ctas, st))


class SceneParallelLayer:
    """One sparse-convolution layer trained data-parallel: each rank its own scene.

    ``forward`` / ``backward`` run the CUDA operator on the local scene; ``backward`` sums the fp32
    weight-gradient partials of all ranks with one all-reduce before adding them to ``w_grad``.
    """

    def __init__(self, kpos, imap, omap, qsum: int, arch80: bool, group=None):
        self.kpos, self.imap, self.omap, self.qsum, self.arch80, self.group = kpos, imap, omap, qsum, arch80, group

    def forward(self, feats, weights, out):
        from . import backend
        backend.fgms_fusion_fwd_cuda(feats, weights, self.qsum, out, self.kpos, None, self.imap, self.omap,
                                     False, self.arch80)
        return out

    def backward(self, grad_out, feats, weights, in_grad, w_grad):
        """wgrad first, so that the all-reduce of its fp32 sums runs beside dgrad."""
        import torch
        import torch.distributed as dist
        from . import backend
        multi = world_size(self.group) > 1
        work = part = None
        if feats.dtype == torch.float16 and not multi:
            # nothing to exchange: single launch, straight into w_grad
            backend.fgms_wgrad_cuda(feats, grad_out, w_grad, self.kpos, self.imap, self.omap, self.arch80)
        elif feats.dtype == torch.float16:
            ws = backend.fgms_wgrad_cuda(feats, grad_out, w_grad, self.kpos, self.imap, self.omap, self.arch80,
                                         workspace=backend.wgrad_workspace(w_grad.size(1), w_grad.size(2), w_grad.size(0),
                                                                           feats.device), accumulate=False)
            part = ws[: w_grad.numel()]
        else:
            part = torch.zeros_like(w_grad)
            backend.fgms_wgrad_cuda(feats, grad_out, part, self.kpos, self.imap, self.omap, self.arch80)
        if multi:
            work = dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        backend.fgms_dgrad_cuda(grad_out, weights, in_grad, self.kpos, self.imap, self.omap, self.arch80)
        if work is not None:
            work.wait()
        if part is not None:
            if feats.dtype == torch.float16:
                backend.wgrad_finalize(w_grad, part)
            else:
                w_grad += part
        return in_grad, w_grad


class BoundSceneLayer:
    """A :class:`SceneParallelLayer` step bound to fixed tensors: arguments are validated once, every later
    ``forward()`` / ``backward()`` goes straight to the C ABI with the stored pointers.

    The checked Python entry points cost about 20 us of host time per call; with a collective in the step
    that makes the host, not the GPU, the bottleneck.  Binding is for training loops that reuse their buffers
    (the tensors must stay alive and keep their storage while the object is used).
    """

    def __init__(self, feats, weights, grad_out, out, in_grad, w_grad, kpos, imap, omap, arch80: bool, group=None,
                 exchange: bool = True, transport: str = "nccl"):
        import torch
        from . import _lib, backend
        k_vol = backend._common(feats, weights, kpos, imap, omap)
        backend._check_feat("out", out, feats.dtype)
        backend._check_feat("grad_out", grad_out, feats.dtype)
        backend._check_feat("in_grad", in_grad, feats.dtype)
        backend._check_feat("w_grad", w_grad, feats.dtype, dim=3)
        if in_grad.shape != feats.shape or w_grad.shape != weights.shape or out.shape != grad_out.shape \
                or out.size(1) != weights.size(2):
            raise ValueError("output / gradient buffers do not match the shapes of feats, weights and grad_out")
        self._keep = (feats, weights, grad_out, out, in_grad, w_grad, kpos, imap, omap)
        self._L, self._check, self.group = _lib.lib, _lib.check, group
        self.device = feats.device
        self.fp16 = feats.dtype == torch.float16
        dtype, math = backend._dtype_math(feats, arch80)
        self.multi = world_size(group) > 1
        # exchange = False keeps the multi-rank form of the step (fp32 sums, final addition) but skips the
        # all-reduce: the step's kernels alone, which is how the collective's exposed time is measured
        self.exchange = exchange and self.multi
        # transport: "nccl" = all-reduce of the fp32 sums; "peer" = the library's own kernel over peer memory on a side
        # stream (PeerExchange), which can run beside the input-gradient kernel
        if transport not in ("nccl", "peer"):
            raise ValueError("transport must be 'nccl' or 'peer'")
        self.px = None
        n_in, n_out, c_in, c_out = feats.size(0), out.size(0), weights.size(1), weights.size(2)
        p = lambda t: t.data_ptr() if t.numel() > 0 else None
        pairs = imap.numel()
        self._fwd_args = (p(feats), p(weights), p(out), p(kpos), None, p(imap), p(omap), pairs, n_in, n_out, c_in, c_in,
                          c_out, k_vol, 0, dtype, math, 0)
        self._dgrad_args = (p(grad_out), p(weights), p(in_grad), p(kpos), p(imap), p(omap), pairs, n_in, n_out, c_in, c_out,
                            k_vol, dtype, math)
        self.w_grad, self.part, ws_ptr, ws_bytes, accumulate = w_grad, None, None, 0, 1
        if self.multi and self.exchange and transport == "peer":
            self.px = PeerExchange(w_grad.numel(), feats.device, group)
            self._side = torch.cuda.Stream(device=feats.device, priority=-1)  # its few CTAs go first when room frees up
            self._ev_sums, self._ev_total = torch.cuda.Event(), torch.cuda.Event()
        if self.fp16 and (self.multi or backend.kernel_family("wgrad", c_in, c_out, feats.dtype, arch80, k_vol) != "tcgen05"):
            ws = self.px.sums if self.px is not None else backend.wgrad_workspace(c_in, c_out, k_vol, feats.device)
            ws_ptr, ws_bytes = ws.data_ptr(), ws.numel() * 4
            if self.multi:
                self.part, accumulate = ws[: w_grad.numel()], 0  # fp32 sums, all-reduced, then added to w_grad
        elif not self.fp16 and self.multi:
            # fp32 storage: sums of this rank, all-reduced, then added
            self.part = self.px.sums[: w_grad.numel()].view_as(w_grad) if self.px is not None else torch.zeros_like(w_grad)
        target = self.part if (self.part is not None and not self.fp16) else w_grad
        self._wgrad_args = (p(feats), p(grad_out), p(target), p(kpos), p(imap), p(omap), pairs, n_in, n_out, c_in, c_out,
                            k_vol, dtype, math, ws_ptr, ws_bytes, accumulate)

    def _stream(self):
        import torch
        return torch.cuda.current_stream(self.device).cuda_stream

    def forward(self):
        import torch
        with torch.cuda.device(self.device):  # the library launches on the current device
            self._check(self._L.fgms_b200_fusion_fwd(*self._fwd_args, self._stream()))

    def backward(self):
        """wgrad first, its all-reduce beside dgrad, then the sums are added to ``w_grad``."""
        import torch
        import torch.distributed as dist
        with torch.cuda.device(self.device):  # the library launches on the current device
            st = self._stream()
            if self.part is not None and not self.fp16:
                self.part.zero_()
            self._check(self._L.fgms_b200_wgrad(*self._wgrad_args, st))
            work, total = None, self.part
            if self.px is not None:
                main = torch.cuda.current_stream(self.device)
                self._ev_sums.record(main)
                self._side.wait_event(self._ev_sums)
                self.px.run(self._side)
                self._ev_total.record(self._side)
                total = self.px.reduced[: self.w_grad.numel()]
            elif self.exchange:
                work = dist.all_reduce(self.part, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
            self._check(self._L.fgms_b200_dgrad(*self._dgrad_args, st))
            if work is not None:
                work.wait()
            if self.px is not None:
                torch.cuda.current_stream(self.device).wait_event(self._ev_total)
            if self.multi:
                if self.fp16:
                    self._check(self._L.fgms_b200_wgrad_finalize(self.w_grad.data_ptr(), total.data_ptr(), self.w_grad.numel(), st))
                else:
                    self.w_grad += total.view_as(self.w_grad)
