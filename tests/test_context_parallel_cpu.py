"""Host-side logic of the context-parallel wrapper on two CPU ranks (gloo): the token gather puts chunks in sequence
order for both layouts and its backward returns the rank-summed gradient of the local tokens."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, zigzag, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nsa_b200.context_parallel import _GatherTokens, chunk_layout
    B, T, H, D = 2, 16 * world, 2, 4
    full = torch.arange(B * T * H * D, dtype=torch.float32).reshape(B, T, H, D)
    layout = chunk_layout(world, zigzag)
    cl = T // (world * len(layout[0]))
    local = torch.cat([full[:, c * cl:(c + 1) * cl] for c in layout[rank]], 1).clone().requires_grad_(True)
    gathered = _GatherTokens.apply(local, None, zigzag)
    ok = torch.equal(gathered, full)
    w = torch.arange(T, dtype=torch.float32).view(1, T, 1, 1) * (rank + 1)   # a different loss on every rank
    (gathered * w).sum().backward()
    expect_full = torch.arange(T, dtype=torch.float32).view(1, T, 1, 1) * sum(r + 1 for r in range(world))
    expect = torch.cat([expect_full[:, c * cl:(c + 1) * cl] for c in layout[rank]], 1).expand_as(local)
    ok = ok and torch.equal(local.grad, expect)
    ret[rank] = bool(ok)
    dist.destroy_process_group()


def _run(zigzag, port):
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, zigzag, ret), nprocs=world, join=True)
    assert all(ret[r] for r in range(world)), dict(ret)


def test_gather_tokens_contiguous_layout():
    _run(False, 29611)


def test_gather_tokens_zigzag_layout():
    _run(True, 29612)


def _rows_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nsa_b200.context_parallel import _GatherRows, _compressed_ranges
    Tc, H, D = 13, 2, 3                      # 13 compressed positions over 2 ranks: 7 + 6 (uneven)
    ranges = _compressed_ranges(Tc, world)
    counts = [hi - lo for lo, hi in ranges]
    full = torch.arange(Tc * H * D, dtype=torch.float32).reshape(1, Tc, H, D)
    lo, hi = ranges[rank]
    local = full[:, lo:hi].clone().requires_grad_(True)
    gathered = _GatherRows.apply(local, counts, None)
    ok = torch.equal(gathered, full)
    w = torch.arange(Tc, dtype=torch.float32).view(1, Tc, 1, 1) * (rank + 1)
    (gathered * w).sum().backward()
    expect = (torch.arange(Tc, dtype=torch.float32).view(1, Tc, 1, 1) * sum(r + 1 for r in range(world)))[:, lo:hi]
    ok = ok and torch.equal(local.grad, expect.expand_as(local))
    ret[rank] = bool(ok)
    dist.destroy_process_group()


def test_gather_rows_uneven_counts():
    """The all-gather of the sharded compressed K/V and its reduce-scatter backward, with ranks owning 7 and 6 rows."""
    from nsa_b200.context_parallel import _compressed_ranges
    assert _compressed_ranges(4095, 8)[0] == (0, 512) and _compressed_ranges(4095, 8)[-1] == (3584, 4095)
    assert _compressed_ranges(3, 8)[-1] == (3, 3)
    ret = mp.Manager().dict()
    mp.spawn(_rows_worker, args=(2, 29613, ret), nprocs=2, join=True)
    assert all(ret[r] for r in range(2)), dict(ret)


def test_chunk_layout_balances_causal_work():
    from nsa_b200.context_parallel import chunk_layout
    P = 8
    lay = chunk_layout(P, True)
    assert sorted(c for r in lay for c in r) == list(range(2 * P))
    work = [sum(2 * c + 1 for c in chunks) for chunks in lay]      # causal work of chunk c grows like 2c+1
    assert max(work) == min(work)
