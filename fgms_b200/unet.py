"""A MinkUNet-style encoder-decoder stack of sparse convolutions, run as one training step.

The reference's benchmark driver walks the layer list of a whole network and calls the operator once
per layer (``spconv-test.py:51-126``, default network ``minkunet-semantickitti``); the kernel maps of
those layers come from files that are not available offline.  Here the same kind of stack is built from
a voxel cloud alone:

* stem: submanifold 3x3x3, ``c_in -> widths[0]``;
* four encoder stages: a 2x2x2 stride-2 convolution to the next resolution and channel width, then two
  submanifold 3x3x3 convolutions;
* a mirrored decoder: a transposed 2x2x2 convolution back to the finer voxels, the encoder's features of
  that resolution added to it (additive skip), then two submanifold 3x3x3 convolutions.

25 operator layers for the default widths (32, 32, 64, 128, 256).  Layers of one resolution share one
kernel map, and a transposed layer reuses its downsampling layer's pairs with the roles swapped — the map
reuse a dgSPARSE-style caller does.  There are no normalisation or activation layers: they are not part of
the operator the path covers.

``UNetStep`` binds such a network to fixed buffers and runs forward + backward as a flat list of C-ABI
calls: every layer's forward, then in reverse order every layer's weight gradient and input gradient.
With several ranks (one scene or batch per rank) the fp32 weight-gradient sums of all layers live in one
flat buffer cut into buckets in backward order; a bucket's all-reduce is started as soon as its last
weight gradient is enqueued and runs beside the backward of the layers before it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

__all__ = ["LayerSpec", "minkunet_spec", "UNetMaps", "build_unet_maps", "build_unet_maps_host", "unet_weights",
           "UNetStep", "layer_flops", "step_flops", "flat_layout", "plan_buckets"]


@dataclass(frozen=True)
class LayerSpec:
    name: str
    kind: str      # "subm" (3x3x3, same voxels) | "down" (2x2x2 stride 2) | "up" (transposed 2x2x2)
    c_in: int
    c_out: int
    res_in: int    # resolution level of the input voxels (0 = finest)
    res_out: int
    src: str       # name of the value the layer reads
    dst: str       # name of the value it produces
    skip: str | None = None  # value added to the layer's output (decoder skip connection)

    @property
    def k_vol(self) -> int:
        return 27 if self.kind == "subm" else 8


def minkunet_spec(c_in: int = 4, widths=(32, 32, 64, 128, 256)) -> list[LayerSpec]:
    """Layer list of the stack: ``widths[0]`` is the stem width, ``widths[s]`` the width of encoder stage s."""
    L = [LayerSpec("stem", "subm", c_in, widths[0], 0, 0, "input", "e0")]
    levels = len(widths) - 1
    for s in range(1, levels + 1):
        a, b = widths[s - 1], widths[s]
        L.append(LayerSpec(f"enc{s}.down", "down", a, b, s - 1, s, f"e{s - 1}", f"e{s}d"))
        L.append(LayerSpec(f"enc{s}.conv1", "subm", b, b, s, s, f"e{s}d", f"e{s}a"))
        L.append(LayerSpec(f"enc{s}.conv2", "subm", b, b, s, s, f"e{s}a", f"e{s}"))
    prev = f"e{levels}"
    for s in range(levels, 0, -1):
        a, b = widths[s], widths[s - 1]
        L.append(LayerSpec(f"dec{s - 1}.up", "up", a, b, s, s - 1, prev, f"d{s - 1}u", skip=f"e{s - 1}"))
        L.append(LayerSpec(f"dec{s - 1}.conv1", "subm", b, b, s - 1, s - 1, f"d{s - 1}u", f"d{s - 1}a"))
        L.append(LayerSpec(f"dec{s - 1}.conv2", "subm", b, b, s - 1, s - 1, f"d{s - 1}a", f"d{s - 1}"))
        prev = f"d{s - 1}"
    return L


@dataclass
class UNetMaps:
    """Kernel maps of every resolution: ``subm[r]`` (27 offsets), ``down[r]`` (r -> r + 1, 8 offsets) and
    ``up[r]`` (r + 1 -> r, the transposed map).  Entries are ``maps.KernelMap`` (host) or
    ``gpu_maps.DeviceKernelMap`` (device)."""

    subm: list
    down: list
    up: list

    def of(self, layer: LayerSpec):
        if layer.kind == "subm":
            return self.subm[layer.res_in]
        if layer.kind == "down":
            return self.down[layer.res_in]
        return self.up[layer.res_out]

    @property
    def voxels(self) -> list[int]:
        return [m.n_in for m in self.subm]


def build_unet_maps(coords, levels: int = 4) -> UNetMaps:
    """All maps of the stack on the device (``coords``: CUDA int32 ``[n, 3]``, no voxel twice)."""
    from . import gpu_maps
    subm, down, up = [], [], []
    c = coords
    for r in range(levels + 1):
        subm.append(gpu_maps.build_submanifold_map(c, 3))
        if r < levels:
            d = gpu_maps.build_strided_map(c, 2)
            down.append(d)
            up.append(gpu_maps.transpose_map(d, c))
            c = d.out_coords
    return UNetMaps(subm, down, up)


def build_unet_maps_host(coords: np.ndarray, levels: int = 4) -> UNetMaps:
    """The same maps from the host builders (the oracle's inputs; the device builders match them bit for bit)."""
    from . import maps
    subm, down, up = [], [], []
    c = maps.unique_coords(coords)
    for r in range(levels + 1):
        subm.append(maps.build_submanifold_map(c, 3))
        if r < levels:
            d = maps.build_strided_map(c, 2, 2)
            down.append(d)
            up.append(maps.transpose_map(d, c))
            c = d.out_coords
    return UNetMaps(subm, down, up)


def unet_weights(spec, umaps: UNetMaps, seed: int, dtype=np.float16) -> list[np.ndarray]:
    """Seeded weights ``[k_vol, c_in, c_out]`` per layer, uniform with the bound that keeps the variance of the
    features about constant through the stack: ``sqrt(3 / (c_in * pairs per output voxel))`` (the usual
    kaiming-uniform bound assumes all 27 neighbours exist; on a surface cloud about a third do, and a stack of
    25 layers without normalisation would otherwise underflow fp16).  A layer whose output also receives a
    skip connection gets ``1 / sqrt(2)`` of that."""
    rng = np.random.default_rng(seed)
    out = []
    for layer in spec:
        km = umaps.of(layer)
        pairs = int(km.pairs)
        ppo = max(pairs / max(km.n_out, 1), 1.0)
        bound = math.sqrt(3.0 / (layer.c_in * ppo)) * (2 ** -0.5 if layer.skip else 1.0)
        out.append(rng.uniform(-bound, bound, size=(layer.k_vol, layer.c_in, layer.c_out)).astype(dtype))
    return out


def layer_flops(layer: LayerSpec, pairs: int, first: bool) -> float:
    """Effective flops of one step of a layer: 2 * pairs * c_in * c_out per pass; forward, weight gradient and
    (except for the first layer, whose input needs no gradient) input gradient."""
    return 2.0 * pairs * layer.c_in * layer.c_out * (2 if first else 3)


def step_flops(spec, umaps: UNetMaps) -> float:
    return sum(layer_flops(l, int(umaps.of(l).pairs), i == 0) for i, l in enumerate(spec))


def flat_layout(spec, align: int = 128):
    """Where every layer's ``[k_vol, c_in, c_out]`` block sits in the flat weight / weight-gradient buffers: layers in
    BACKWARD order (the order their gradients become ready), every block padded to a multiple of ``align`` elements.
    Returns ``({layer index: (first element, one past the padded block)}, total elements)``."""
    off, where = 0, {}
    for i in range(len(spec) - 1, -1, -1):
        n = spec[i].k_vol * spec[i].c_in * spec[i].c_out
        size = (n + align - 1) // align * align
        where[i] = (off, off + size)
        off += size
    return where, off


def plan_buckets(spec, where, bucket_bytes: int, tail_bytes: int = 0):
    """Cut the flat buffer into buckets of consecutive layers (backward order), each closed once it holds at least
    ``bucket_bytes`` of fp32 sums (the last one takes what is left).  Returns ``[(first element, one past the last,
    index of the layer whose weight gradient completes the bucket)]``: that layer's gradient is the last of the bucket to
    be enqueued, so the bucket's exchange can start right after it.

    Nothing is left to run beside the exchange of the LAST bucket, so it should be small: with ``tail_bytes`` the
    layers at the end of the backward (the first layers of the network) whose sums together fit ``tail_bytes`` form
    a bucket of their own, and only the layers before them are cut greedily."""
    order = list(range(len(spec) - 1, -1, -1))
    size = lambda i: (where[i][1] - where[i][0]) * 4
    n_tail, acc = 0, 0
    for i in reversed(order):
        if tail_bytes <= 0 or acc + size(i) > tail_bytes:
            break
        acc += size(i)
        n_tail += 1
    head = order[:len(order) - n_tail] if n_tail < len(order) else []
    tail = order[len(head):]
    buckets, start, acc = [], 0, 0
    for i in head:
        lo, hi = where[i]
        acc += (hi - lo) * 4
        if acc >= bucket_bytes or i == head[-1]:
            buckets.append((start, hi, i))
            start, acc = hi, 0
    if tail:
        buckets.append((start, where[tail[-1]][1], tail[-1]))
    return buckets


class UNetStep:
    """Forward + backward of the stack over fixed device buffers, as straight C-ABI calls.

    ``feats`` ``[n0, c_in]`` and ``grad_out`` ``[n0, widths[0]]`` are the step's inputs; after ``run()`` the flat
    fp16 ``w_grad`` holds every layer's weight gradient (``w_grads[i]`` is the view of layer i), summed over
    the ranks of ``group`` when there are several.  The first layer's input gradient is not computed.

    The stem's few input channels (4) are padded with zero channels to 16 inside the step: 8-byte rows cannot be
    gathered in 16-byte pieces and would run on the CUDA-core kernels, 32-byte rows run on the tensor cores.  The
    padded weight rows multiply zeros and their gradient is zero; ``weights[0]`` / ``w_grads[0]`` show the real
    ``c_in`` rows only.  ``set_input`` refreshes the padded copy when the caller's features change.
    """

    def __init__(self, spec, umaps: UNetMaps, weights, feats, grad_out, group=None, bucket_bytes: int = 6 << 20,
                 arch80: bool = True, exchange: bool | None = None, transport: str = "nccl"):
        import torch
        from . import _lib, backend
        from .dist import world_size
        self.spec, self.umaps, self.group = list(spec), umaps, group
        self.device = feats.device
        # the layers as they are run: the stem with its input channels padded to a multiple of 16
        from dataclasses import replace
        self._cin0 = self.spec[0].c_in
        run_spec = list(self.spec)
        if self._cin0 % 16:
            run_spec[0] = replace(run_spec[0], c_in=(self._cin0 + 15) // 16 * 16)
        report_spec, self.spec = self.spec, run_spec
        # exchange: None = the data-parallel form (fp32 sums in buckets, all-reduced, added to w_grad at the end)
        # when the process group has several ranks; False = this rank alone, whatever the group; True = the
        # data-parallel form even with one rank (the collective is then skipped)
        self.multi = world_size(group) > 1 if exchange is None else bool(exchange)
        self._collective = self.multi and world_size(group) > 1
        self._L, self._check = _lib.lib, _lib.check
        dt = feats.dtype
        if dt != torch.float16:
            raise ValueError("UNetStep runs fp16 storage (the configuration the stack is specified in)")
        dtype, math_ = backend._dtype_math(feats, arch80)
        dev = self.device
        n_vox = umaps.voxels
        if feats.size(0) != n_vox[0] or grad_out.size(0) != n_vox[0]:
            raise ValueError("feats / grad_out rows differ from the finest kernel map's voxel count")

        # ---- values (activations) and their gradients: one flat buffer each, zeroed once per step -------------
        width = {"input": spec[0].c_in}
        level = {"input": 0}
        for l in self.spec:
            width[l.dst], level[l.dst] = l.c_out, l.res_out
        names = [n for n in width if n != "input"]
        sizes = {n: n_vox[level[n]] * width[n] for n in names}
        pad = lambda x: (x + 127) // 128 * 128  # keeps every view 256-byte aligned (fp16)
        total = sum(pad(sizes[n]) for n in names)
        self._act_flat = torch.zeros(total, dtype=dt, device=dev)
        self._grad_flat = torch.zeros(total, dtype=dt, device=dev)
        if run_spec[0].c_in != self._cin0:
            self._input = torch.zeros((feats.size(0), run_spec[0].c_in), dtype=dt, device=dev)
            self._input[:, : self._cin0].copy_(feats)
        else:
            self._input = feats
        self.val, self.grad = {"input": self._input}, {}
        off = 0
        for n in names:
            shape = (n_vox[level[n]], width[n])
            self.val[n] = self._act_flat[off: off + sizes[n]].view(shape)
            self.grad[n] = self._grad_flat[off: off + sizes[n]].view(shape)
            off += pad(sizes[n])
        self.out_name = self.spec[-1].dst
        self.grad_out = grad_out

        # ---- weights and weight gradients, flat, in BACKWARD order (the order the gradients become ready) -----
        order = list(range(len(self.spec)))[::-1]
        where, w_total = flat_layout(self.spec)
        w_sizes = [where[i][1] - where[i][0] for i in order]
        self._w_flat = torch.zeros(w_total, dtype=dt, device=dev)
        self.w_grad = torch.zeros(w_total, dtype=dt, device=dev)
        # transport of the buckets' sums between ranks: "nccl" = all-reduce; "peer" = the library's kernel over
        # peer-mapped memory on a side stream (dist.PeerExchange), whose few small CTAs run beside the backward kernels
        if transport not in ("nccl", "peer"):
            raise ValueError("transport must be 'nccl' or 'peer'")
        self.px = None
        if self._collective and transport == "peer":
            from .dist import PeerExchange
            self.px = PeerExchange(w_total, dev, group)
            self._dw32, self._total32 = self.px.sums[:w_total], self.px.reduced[:w_total]
            self._side = torch.cuda.Stream(device=dev, priority=-1)
            self._ev_bucket = [torch.cuda.Event() for _ in range(64)]
            self._ev_done = torch.cuda.Event()
        else:
            self._dw32 = torch.zeros(w_total, dtype=torch.float32, device=dev) if self.multi else None
            self._total32 = self._dw32
        self.weights, self.w_grads, self._dw32_views = [None] * len(self.spec), [None] * len(self.spec), [None] * len(self.spec)
        self._w_off = {}
        off = 0
        for i, sz in zip(order, w_sizes):
            l = self.spec[i]
            n = l.k_vol * l.c_in * l.c_out
            shape = (l.k_vol, l.c_in, l.c_out)
            self.weights[i] = self._w_flat[off: off + n].view(shape)
            w_src = torch.as_tensor(weights[i]).to(dev, dt)
            self.weights[i][:, : w_src.size(1), :].copy_(w_src)  # (padded input channels keep zero weights)
            self.w_grads[i] = self.w_grad[off: off + n].view(shape)
            if self.multi:
                self._dw32_views[i] = self._dw32[off: off + n]
            self._w_off[i] = (off, off + sz)
            off += sz
        # buckets: consecutive layers in backward order, closed when they reach `bucket_bytes` of fp32 sums
        self.buckets = plan_buckets(self.spec, where, bucket_bytes, tail_bytes=min(1 << 20, bucket_bytes // 4)) if self.multi else []

        # a small fp32 workspace for layers whose weight gradient has no single-launch fp16 form (single rank only)
        self._ws = None
        p = lambda t: t.data_ptr() if t.numel() > 0 else None
        self._fwd, self._bwd = [], []
        for i, l in enumerate(self.spec):
            km = umaps.of(l)
            pairs = int(km.pairs)
            src, dst = self.val[l.src], self.val[l.dst]
            self._fwd.append((l, (p(src), p(self.weights[i]), p(dst), p(km.kpos), None, p(km.imap), p(km.omap), pairs,
                                  km.n_in, km.n_out, l.c_in, l.c_in, l.c_out, l.k_vol, 0, dtype, math_, 0)))
            g_dst = self.grad[l.dst]
            single = backend.kernel_family("wgrad", l.c_in, l.c_out, dt, arch80, l.k_vol) == "tcgen05"
            if self.multi:
                ws, ws_bytes, accumulate = self._dw32_views[i].data_ptr(), self._dw32_views[i].numel() * 4, 0
            elif single:
                ws, ws_bytes, accumulate = None, 0, 1
            else:
                if self._ws is None or self._ws.numel() < l.k_vol * l.c_in * l.c_out:
                    self._ws = torch.empty(max(l.k_vol * l.c_in * l.c_out, 64), dtype=torch.float32, device=dev)
                ws, ws_bytes, accumulate = "ws", 0, 1  # patched below, once the largest workspace is known
            wgrad = [p(src), p(g_dst), p(self.w_grads[i]), p(km.kpos), p(km.imap), p(km.omap), pairs, km.n_in, km.n_out,
                     l.c_in, l.c_out, l.k_vol, dtype, math_, ws, ws_bytes, accumulate]
            dgrad = None
            if i > 0:
                dgrad = (p(g_dst), p(self.weights[i]), p(self.grad[l.src]), p(km.kpos), p(km.imap), p(km.omap), pairs,
                         km.n_in, km.n_out, l.c_in, l.c_out, l.k_vol, dtype, math_)
            self._bwd.append((l, wgrad, dgrad))
        for _, wgrad, _ in self._bwd:
            if wgrad[14] == "ws":
                wgrad[14], wgrad[15] = self._ws.data_ptr(), self._ws.numel() * 4
        self._bucket_end = {last: (lo, hi) for lo, hi, last in self.buckets}
        self.launches_per_step = len(self.spec) * 3 - 1
        # what the caller sees: the layer list as given, the stem's real input channels only
        self.run_spec, self.spec = self.spec, report_spec
        self._w_run = list(self.weights)
        self.weights[0] = self.weights[0][:, : self._cin0, :]
        self.w_grads[0] = self.w_grads[0][:, : self._cin0, :]

    def set_input(self, feats):
        """Copy new input features ``[n0, c_in]`` into the step's (channel-padded) input buffer."""
        if self._input is feats:
            return
        self._input[:, : self._cin0].copy_(feats)

    def _stream(self):
        import torch
        return torch.cuda.current_stream(self.device).cuda_stream

    def forward(self):
        L, check, st = self._L, self._check, self._stream()
        self._act_flat.zero_()
        for l, args in self._fwd:
            if l.skip is not None:
                self.val[l.dst].copy_(self.val[l.skip])  # the layer accumulates on top of the skip features
            check(L.fgms_b200_fusion_fwd(*args, st))
        return self.val[self.out_name]

    def backward(self):
        import torch
        import torch.distributed as dist
        L, check, st = self._L, self._check, self._stream()
        main = torch.cuda.current_stream(self.device)
        self._grad_flat.zero_()
        self.w_grad.zero_()
        self.grad[self.out_name].copy_(self.grad_out)
        works, n_bucket = [], 0
        for i in range(len(self.spec) - 1, -1, -1):
            l, wgrad, dgrad = self._bwd[i]
            if l.skip is not None:
                # the skip source's gradient starts as this layer's output gradient; the encoder layer that
                # reads the skip source adds its input gradient later in this loop
                self.grad[l.skip].copy_(self.grad[l.dst])
            check(L.fgms_b200_wgrad(*wgrad, st))
            if self._collective and i in self._bucket_end:
                lo, hi = self._bucket_end[i]
                if self.px is not None:
                    ev = self._ev_bucket[n_bucket % len(self._ev_bucket)]
                    ev.record(main)
                    self._side.wait_event(ev)
                    self.px.run(self._side, lo, hi)
                    n_bucket += 1
                else:
                    works.append(dist.all_reduce(self._dw32[lo:hi], op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            if dgrad is not None:
                check(L.fgms_b200_dgrad(*dgrad, st))
        for w in works:
            w.wait()
        if self.px is not None:
            self._ev_done.record(self._side)
            main.wait_event(self._ev_done)
        if self.multi:
            check(L.fgms_b200_wgrad_finalize(self.w_grad.data_ptr(), self._total32.data_ptr(), self.w_grad.numel(), st))

    def run(self):
        import torch
        with torch.cuda.device(self.device):
            self.forward()
            self.backward()

    def profile(self, reps: int = 5, flush=None):
        """Per-call device times of the step (mean over ``reps`` steps, CUDA events around every operator call):
        a list of ``{layer, pass, ms}`` in execution order.  ``flush`` (a callable) runs before every step,
        untimed.  Single rank only; meant for reports, not for the timed benchmark."""
        import torch
        if self.multi:
            raise ValueError("profile() times the kernels of one rank: build the step with exchange=False")
        L, check = self._L, self._check
        ev = lambda: torch.cuda.Event(enable_timing=True)
        rows, sums = [], []
        with torch.cuda.device(self.device):
            st = self._stream()
            for rep in range(reps + 1):  # the first repetition warms up
                if flush is not None:
                    flush()
                marks = []
                self._act_flat.zero_()
                for l, args in self._fwd:
                    if l.skip is not None:
                        self.val[l.dst].copy_(self.val[l.skip])
                    a, b = ev(), ev()
                    a.record(); check(L.fgms_b200_fusion_fwd(*args, st)); b.record()
                    marks.append((l.name, "fwd", a, b))
                self._grad_flat.zero_(); self.w_grad.zero_()
                self.grad[self.out_name].copy_(self.grad_out)
                for i in range(len(self.spec) - 1, -1, -1):
                    l, wgrad, dgrad = self._bwd[i]
                    if l.skip is not None:
                        self.grad[l.skip].copy_(self.grad[l.dst])
                    a, b = ev(), ev()
                    a.record(); check(L.fgms_b200_wgrad(*wgrad, st)); b.record()
                    marks.append((l.name, "wgrad", a, b))
                    if dgrad is not None:
                        a, b = ev(), ev()
                        a.record(); check(L.fgms_b200_dgrad(*dgrad, st)); b.record()
                        marks.append((l.name, "dgrad", a, b))
                torch.cuda.synchronize(self.device)
                if rep == 0:
                    continue
                ms = [a.elapsed_time(b) for _, _, a, b in marks]
                if not sums:
                    rows, sums = [(n, p) for n, p, _, _ in marks], ms
                else:
                    sums = [x + y for x, y in zip(sums, ms)]
        return [{"layer": n, "pass": p, "ms": t / reps} for (n, p), t in zip(rows, sums)]
