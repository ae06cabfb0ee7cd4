"""The peer-memory sum of the ranks' weight-gradient sums (``fgms_b200_peer_exchange``) on ONE device.

The kernels of different ranks wait for one another, so they never run here as separate launches on one GPU.  The
arithmetic and addressing of a two-rank group are checked with the other rank's flags set by the host (as if it had
arrived), one rank's call at a time; the bounded wait is checked with a flag that nothing sets.  The real exchange
between GPUs is checked by the benchmark's ``multi_gpu_check`` on 2 to 8 GPUs."""
import pytest
import torch

from fgms_b200 import _lib

pytestmark = pytest.mark.gpu


def _group(world, count, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    n_flag = _lib.lib.fgms_b200_peer_exchange_flag_bytes(world) // 4
    sums = [torch.randn(count, device="cuda", generator=g) for _ in range(world)]
    reduced = [torch.full((count,), float("nan"), device="cuda") for _ in range(world)]
    flags = [torch.zeros(n_flag, dtype=torch.int32, device="cuda") for _ in range(world)]
    return sums, reduced, flags


def test_one_rank_copies_its_sums():
    from fgms_b200 import backend
    from fgms_b200.dist import PeerExchange
    px = PeerExchange(27 * 64 * 64, "cuda")
    backend.device_status(reset=True)
    for call in range(3):
        px.sums.normal_()
        px.run()
        torch.cuda.synchronize()
        assert torch.equal(px.reduced, px.sums), f"call {call}"
    assert backend.device_status() == 0


@pytest.mark.parametrize("world", [2, 8])
def test_emulated_group_sums_in_rank_order(world):
    """Every rank's call in turn, the flags of the ranks that are not running set by the host beforehand."""
    from fgms_b200 import backend
    from fgms_b200.dist import PeerExchange
    count = 27 * 32 * 32
    sums, reduced, flags = _group(world, count)
    ranks = [PeerExchange(count, "cuda", buffers=(r, world, sums, reduced, flags)) for r in range(world)]
    backend.device_status(reset=True)
    for epoch in (1, 2):
        for f in flags:
            f[: 2 * world] = epoch  # every rank "has arrived" and "has finished": no call waits for another
        for r in ranks:
            r.run()
        torch.cuda.synchronize()
        total = sums[0].clone()
        for s in sums[1:]:
            total += s             # the same order of additions as the kernel's
        for r in range(world):
            assert torch.equal(reduced[r], total), f"epoch {epoch}, rank {r}"
        for s in sums:
            s.mul_(-0.5)
    assert backend.device_status() == 0


def test_a_wait_that_nothing_ends_runs_out_and_is_reported():
    """Rank 0 of a two-rank group whose other rank never calls: the wait gives up after its limit, the kernel
    returns, the problem is counted and the context stays usable."""
    from fgms_b200 import backend
    from fgms_b200.dist import PeerExchange
    count = 4096
    sums, reduced, flags = _group(2, count)
    px = PeerExchange(count, "cuda", buffers=(0, 2, sums, reduced, flags), wait_limit_cycles=2_000_000, ctas=4)
    backend.device_status(reset=True)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(); px.run(); end.record()
    torch.cuda.synchronize()
    assert start.elapsed_time(end) < 100.0          # about a millisecond of waiting, not a hang
    assert backend.device_status() >= 1
    assert int(flags[1][0]) == 1                      # it did announce itself to the other rank
    x = torch.ones(8, device="cuda") * 2              # the context still works
    assert float(x.sum()) == 16.0
