"""Multi-GPU host logic on CPU ranks: pair sharding by row range and the weight-gradient exchange
(gloo, world_size 2).  No GPU is involved; the per-rank compute is the oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fgms_b200 import clouds, maps
from fgms_b200.dist import allreduce_sum_, balanced_row_ranges, shard_pairs_by_rows
from oracle import spconv_oracle as orc


def _problem():
    coords = clouds.surface_cloud(2500, 40, 31)
    km = maps.build_submanifold_map(coords)
    f, w, g = clouds.make_tensors(km.n_in, km.n_out, 12, 20, km.k_vol, 31)
    return km, f, w, g


@pytest.mark.parametrize("world", [1, 2, 3, 8])
@pytest.mark.parametrize("by", ["out", "in"])
def test_shards_partition_the_pairs_and_own_disjoint_rows(world, by):
    km, f, w, g = _problem()
    shards, bounds = shard_pairs_by_rows(km, world, by)
    assert bounds[0] == 0 and bounds[-1] == (km.n_out if by == "out" else km.n_in)
    assert sum(s.pairs for s in shards) == km.pairs
    for r, s in enumerate(shards):
        s.validate()
        key = s.omap if by == "out" else s.imap
        if key.size:
            assert bounds[r] <= key.min() and key.max() < bounds[r + 1]
        # order inside every offset is preserved
        for k in range(km.k_vol):
            a, b = s.kpos[k], s.kpos[k + 1]
            assert (np.diff(s.omap[a:b]) > 0).all()
    sizes = np.array([s.pairs for s in shards])
    assert sizes.max() - sizes.min() <= 0.15 * km.pairs / world + 64  # balanced by pair count


def test_sharded_forward_and_dgrad_need_no_exchange():
    km, f, w, g = _problem()
    full_out = orc.fwd(f, w, km.n_out, km.kpos, km.imap, km.omap)
    shards, bounds = shard_pairs_by_rows(km, 4, "out")
    out = np.zeros_like(full_out)
    for r, s in enumerate(shards):
        part = orc.fwd(f, w, km.n_out, s.kpos, s.imap, s.omap)
        assert np.abs(part[: bounds[r]]).max(initial=0) == 0 and np.abs(part[bounds[r + 1]:]).max(initial=0) == 0
        out[bounds[r]: bounds[r + 1]] = part[bounds[r]: bounds[r + 1]]  # each rank owns its rows outright
    assert np.array_equal(out, full_out)
    full_ig = orc.dgrad(g, w, km.n_in, km.kpos, km.imap, km.omap)
    shards, bounds = shard_pairs_by_rows(km, 4, "in")
    ig = np.zeros_like(full_ig)
    for r, s in enumerate(shards):
        ig[bounds[r]: bounds[r + 1]] = orc.dgrad(g, w, km.n_in, s.kpos, s.imap, s.omap)[bounds[r]: bounds[r + 1]]
    assert np.array_equal(ig, full_ig)


def test_balanced_ranges_edge_cases():
    assert balanced_row_ranges(np.zeros(0, np.int32), 10, 4).tolist() == [0, 0, 0, 0, 10]
    b = balanced_row_ranges(np.array([5] * 100, np.int32), 10, 2)  # all pairs on one row
    assert b[0] == 0 and b[-1] == 10 and (np.diff(b) >= 0).all()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        km, f, w, g = _problem()
        shards, _ = shard_pairs_by_rows(km, world, "out")
        s = shards[rank]
        part = torch.from_numpy(orc.wgrad(f, g, km.k_vol, s.kpos, s.imap, s.omap))  # this rank's partial sums
        allreduce_sum_(part)                                                        # the one exchange step
        ref = orc.wgrad(f, g, km.k_vol, km.kpos, km.imap, km.omap)
        q.put((rank, float(np.abs(part.numpy() - ref).max()), float(np.abs(ref).max())))
    finally:
        dist.destroy_process_group()


def test_weight_gradient_allreduce_two_ranks():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, scale in results:
        assert err <= 1e-12 * max(scale, 1.0), (rank, err)


def test_allreduce_is_a_noop_without_a_process_group():
    t = torch.ones(4)
    assert allreduce_sum_(t) is t and t.sum() == 4


@pytest.mark.parametrize("world", [1, 2, 5, 8])
@pytest.mark.parametrize("by", ["out", "in"])
def test_tensor_side_cut_equals_the_numpy_cut(world, by):
    """``shard_map_device`` (tensor operations on the map's device; CPU tensors here) gives every rank exactly the
    shard ``shard_pairs_by_rows`` gives it."""
    from fgms_b200.dist import shard_map_device
    km, *_ = _problem()
    shards, bounds = shard_pairs_by_rows(km, world, by)
    t = lambda a: torch.from_numpy(a)
    n_rows = km.n_out if by == "out" else km.n_in
    for r, s in enumerate(shards):
        cut = shard_map_device(t(km.kpos), t(km.imap), t(km.omap), n_rows, r, world, by)
        assert cut.row_range == (int(bounds[r]), int(bounds[r + 1]))
        assert np.array_equal(cut.kpos.numpy(), s.kpos)
        assert np.array_equal(cut.imap.numpy(), s.imap) and np.array_equal(cut.omap.numpy(), s.omap)


def _unet_rank(rank, world, port, out_dir):
    """One CPU rank of the data-parallel stack: its own scene, the oracle as the per-layer compute, the weight-gradient
    sums of all layers in one flat buffer exchanged bucket by bucket as the buckets complete in the backward."""
    from fgms_b200 import unet
    from oracle import unet_oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    spec = unet.minkunet_spec(4, (16, 16, 32))
    coords = clouds.surface_cloud(500, 32, 40 + rank)
    um = unet.build_unet_maps_host(coords, levels=2)
    w = unet.unet_weights(spec, unet.build_unet_maps_host(clouds.surface_cloud(500, 32, 40), levels=2), 3, dtype=np.float64)  # same on all ranks
    rng = np.random.default_rng(rank)
    f, g = rng.standard_normal((um.voxels[0], 4)), rng.standard_normal((um.voxels[0], 16))
    val = unet_oracle.forward(spec, um, w, f)
    _, w_grads = unet_oracle.backward(spec, um, w, val, g)
    where, total = unet.flat_layout(spec)
    buckets = unet.plan_buckets(spec, where, bucket_bytes=40_000)
    flat = torch.zeros(total, dtype=torch.float64)
    ends = {last: (lo, hi) for lo, hi, last in buckets}
    works = []
    for i in range(len(spec) - 1, -1, -1):            # backward order: layer i's gradient becomes ready
        lo, _ = where[i]
        flat[lo: lo + w_grads[i].size] = torch.from_numpy(w_grads[i].ravel())
        if i in ends:
            a, b = ends[i]
            works.append(dist.all_reduce(flat[a:b], async_op=True))
    for wk in works:
        wk.wait()
    np.save(os.path.join(out_dir, f"own{rank}.npy"), np.concatenate([x.ravel() for x in w_grads]))
    np.save(os.path.join(out_dir, f"flat{rank}.npy"), flat.numpy())
    dist.destroy_process_group()


def test_bucketed_exchange_of_a_stack_on_cpu_ranks(tmp_path):
    from fgms_b200 import unet
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_unet_rank, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    spec = unet.minkunet_spec(4, (16, 16, 32))
    where, total = unet.flat_layout(spec)
    buckets = unet.plan_buckets(spec, where, bucket_bytes=40_000)
    assert len(buckets) >= 2 and buckets[0][0] == 0 and buckets[-1][1] == total
    assert all(a[1] == b[0] for a, b in zip(buckets, buckets[1:]))
    own = [np.load(tmp_path / f"own{r}.npy") for r in range(world)]
    flats = [np.load(tmp_path / f"flat{r}.npy") for r in range(world)]
    assert np.array_equal(flats[0], flats[1])
    pos = 0
    for i, l in enumerate(spec):                        # `own` is in layer order, the flat buffer in backward order
        n = l.k_vol * l.c_in * l.c_out
        lo = where[i][0]
        assert np.allclose(flats[0][lo: lo + n], own[0][pos: pos + n] + own[1][pos: pos + n], rtol=1e-12, atol=1e-12), l.name
        pos += n


def test_bucket_plan_keeps_the_last_bucket_small():
    """Nothing runs beside the last bucket's exchange: with ``tail_bytes`` the network's first layers (the end of the
    backward) get a bucket of their own that fits it, and the cut still covers the buffer without gaps."""
    from fgms_b200 import unet
    spec = unet.minkunet_spec(4, (32, 64, 128, 256))
    where, total = unet.flat_layout(spec)
    plain = unet.plan_buckets(spec, where, bucket_bytes=6 << 20)
    tailed = unet.plan_buckets(spec, where, bucket_bytes=6 << 20, tail_bytes=1 << 20)
    for b in (plain, tailed):
        assert b[0][0] == 0 and b[-1][1] == total and all(x[1] == y[0] for x, y in zip(b, b[1:]))
        assert [last for _, _, last in b] == sorted((last for _, _, last in b), reverse=True)  # backward order
    assert (tailed[-1][1] - tailed[-1][0]) * 4 <= 1 << 20 < (plain[-1][1] - plain[-1][0]) * 4
    assert tailed[-1][2] == 0 and len(tailed) == len(plain) + 1
    # a tail that nothing fits, and one that everything fits
    assert unet.plan_buckets(spec, where, 6 << 20, tail_bytes=16) == plain
    assert unet.plan_buckets(spec, where, 6 << 20, tail_bytes=1 << 30) == [(0, total, 0)]
