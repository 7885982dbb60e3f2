"""Stand-alone all-to-all / all-to-all + segment sum / gather + all-to-all (the reference's LCCL operators) on gloo ranks."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from recsdk_b200.parallel.lccl import lccl_all_to_all, lccl_all_uss, lccl_gather_all, unsorted_segment_sum

DIM = 4
COUNTS = [[2, 3], [1, 4]]          # COUNTS[s][d]: rows rank s sends to rank d


def _send_rows(rank):
    n = sum(COUNTS[rank])
    return (torch.arange(n * DIM, dtype=torch.float32).view(n, DIM) + 1000 * rank)


def _expected_recv(rank, world=2):
    parts = []
    for s in range(world):
        rows = _send_rows(s)
        start = sum(COUNTS[s][:rank])
        parts.append(rows[start:start + COUNTS[s][rank]])
    return torch.cat(parts)


def _worker(rank, world, init_file, ret):
    dist.init_process_group("gloo", init_method="file://" + init_file, rank=rank, world_size=world)
    try:
        kw = dict(rank=rank, rank_size=world, dim=DIM)
        want = _expected_recv(rank)
        got = lccl_all_to_all(_send_rows(rank), COUNTS, [want.shape[0]], None, **kw)
        ok = torch.equal(got, want)
        # segment sum of the received rows: duplicates of an id are summed
        restore = torch.arange(want.shape[0]) % 2
        uss = lccl_all_uss(_send_rows(rank), torch.tensor(COUNTS), [2], None, restore, **kw)
        ref = torch.zeros(2, DIM).index_add_(0, restore, want)
        ok = ok and torch.allclose(uss, ref)
        # gather + exchange: the table rows that lookup names, in destination order
        table = torch.arange(10 * DIM, dtype=torch.float32).view(10, DIM) + 100 * rank
        lookup = torch.arange(sum(COUNTS[rank])) * 2 % 10
        ga = lccl_gather_all(table, lookup, COUNTS, None, None, **kw)
        parts = []
        for s in range(world):
            t = torch.arange(10 * DIM, dtype=torch.float32).view(10, DIM) + 100 * s
            lk = torch.arange(sum(COUNTS[s])) * 2 % 10
            start = sum(COUNTS[s][:rank])
            parts.append(t[lk][start:start + COUNTS[s][rank]])
        ok = ok and torch.equal(ga, torch.cat(parts))
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_lccl_ops_two_gloo_ranks():
    with tempfile.TemporaryDirectory() as d:
        ret = mp.Manager().dict()
        mp.spawn(_worker, args=(2, os.path.join(d, "init"), ret), nprocs=2, join=True)
        assert ret.get(0) and ret.get(1)


def test_single_rank_and_argument_checks(monkeypatch):
    rows = torch.randn(5, DIM)
    out = lccl_all_to_all(rows, [[5]], None, None, rank=0, rank_size=1, dim=DIM)
    assert torch.equal(out, rows) and out.data_ptr() != rows.data_ptr()
    assert torch.equal(lccl_all_to_all(rows.reshape(-1), [[5]], None, None, rank=0, rank_size=1, dim=DIM), rows)   # flat input
    with pytest.raises(ValueError, match="sends 4"):
        lccl_all_to_all(rows, [[4]], None, None, rank=0, rank_size=1, dim=DIM)
    with pytest.raises(ValueError, match="rank_size x rank_size"):
        lccl_all_to_all(rows, [[5, 1]], None, None, rank=0, rank_size=1, dim=DIM)
    with pytest.raises(ValueError, match="shape_vec says 7"):
        lccl_all_to_all(rows, [[5]], [7], None, rank=0, rank_size=1, dim=DIM)
    with pytest.raises(ValueError, match="needs shape_vec"):
        lccl_all_uss(rows, [[5]], None, None, torch.zeros(5, dtype=torch.int64), rank=0, rank_size=1, dim=DIM)
    with pytest.raises(ValueError, match="outside"):
        lccl_gather_all(torch.randn(3, DIM), torch.tensor([0, 3]), [[2]], None, None, rank=0, rank_size=1, dim=DIM)
    with pytest.raises(ValueError, match="restore index outside"):
        unsorted_segment_sum(rows, torch.tensor([0, 1, 2, 3, 9]), 4)

    restore = torch.tensor([2, 0, 2, 2, 0])
    ref = torch.zeros(4, DIM).index_add_(0, restore, rows)
    assert torch.allclose(unsorted_segment_sum(rows, restore, 4, deterministic=False), ref)
    monkeypatch.setenv("LCCL_DETERMINISTIC", "1")
    det = lccl_all_uss(rows, [[5]], [4], None, restore, rank=0, rank_size=1, dim=DIM)
    assert torch.allclose(det, ref) and det.shape == (4, DIM) and bool((det[1] == 0).all()) and bool((det[3] == 0).all())
    # the deterministic sum is a fixed left-to-right order per segment
    assert torch.equal(det[2], (rows[0] + rows[2]) + rows[3])
    assert unsorted_segment_sum(rows[:0], restore[:0], 3).shape == (3, DIM)
