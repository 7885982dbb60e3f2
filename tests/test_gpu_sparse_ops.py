"""Sparse preprocessing kernels against their CPU statements (same module, CPU tensors)."""
import pytest
import torch

from recsdk_b200.ops import sparse_ops as S


def _kjt(F, B, max_len, n_ids, seed):
    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(0, max_len + 1, (F * B,), generator=g)
    ids = torch.randint(-5, n_ids, (int(lengths.sum()),), generator=g)
    return lengths, ids


def test_cpu_paths_consistent():
    lengths, ids = _kjt(3, 8, 5, 40, 0)
    offs = torch.zeros(25, dtype=torch.int64)
    torch.cumsum(lengths, 0, out=offs[1:])
    ub, inv, nl, no, uo = S.dedup_input_indices(ids, offs, [0, 2, 3], 8)
    assert torch.equal(ub[inv], ids) and int(nl.sum()) == int(uo[-1]) and no[-1] == uo[-1]
    out, cnt = S.select(ids, ids > 10)
    assert torch.equal(out[: int(cnt)], ids[ids > 10])


@pytest.mark.gpu
def test_segmented_unique_gpu():
    g = torch.Generator().manual_seed(1)
    keys = torch.randint(-3, 5000, (200_000,), generator=g)
    keys[::1001] = torch.iinfo(torch.int64).min                      # the hash set's sentinel is a legal key
    offs = torch.tensor([0, 70_000, 70_000, 150_000, 200_000])
    ub, inv, uo, cnt = S.segmented_unique(keys.cuda(), offs, with_counts=True)
    rb, rinv, ruo, rcnt = S.segmented_unique(keys, offs, with_counts=True)
    assert torch.equal(uo.cpu(), ruo)
    ub, inv, cnt = ub.cpu(), inv.cpu(), cnt.cpu()
    assert torch.equal(ub[inv], keys)
    for t in range(4):
        a, b = int(ruo[t]), int(ruo[t + 1])
        order = torch.argsort(ub[a:b])
        assert torch.equal(ub[a:b][order], rb[a:b])
        assert torch.equal(cnt[a:b][order], rcnt[a:b])
        seg = inv[int(offs[t]):int(offs[t + 1])]
        assert seg.numel() == 0 or (int(seg.min()) >= a and int(seg.max()) < b)
    u, i = S.unique(keys.cuda())
    assert torch.equal(torch.sort(u.cpu()).values, torch.unique(keys))


@pytest.mark.gpu
@pytest.mark.parametrize("world,blocks", [(4, False), (8, True), (40, False)])
def test_bucketize_gpu(world, blocks):
    F, B = 5, 257
    lengths, ids = _kjt(F, B, 70, 100_000, 2)
    ids = ids.abs()
    w = torch.rand(ids.numel())
    bs = torch.tensor([100_000 // world + 1] * F) if blocks else None
    ref = S.block_bucketize_sparse_features(lengths, ids, world, F, B, bs, w, local_rows=True)
    got = S.block_bucketize_sparse_features(lengths.cuda(), ids.cuda(), world, F, B, None if bs is None else bs.cuda(), w.cuda(),
                                            local_rows=True)
    for r, o in zip(ref, got):
        assert torch.equal(r, o.cpu()) if r.dtype != torch.float32 else torch.allclose(r, o.cpu())


@pytest.mark.gpu
def test_select_range_lengths_gpu():
    g = torch.Generator().manual_seed(3)
    v = torch.randint(0, 1 << 40, (100_003,), generator=g)
    f = torch.rand(100_003, generator=g) < 0.3
    out, cnt = S.select(v.cuda(), f.cuda())
    assert torch.equal(out[: int(cnt)].cpu(), v[f])
    out, cnt = S.select_index(f.cuda())
    assert torch.equal(out[: int(cnt)].cpu(), f.nonzero().squeeze(1))
    lengths, ids = _kjt(6, 64, 9, 500, 4)
    offs = torch.zeros(6 * 64 + 1, dtype=torch.int64)
    torch.cumsum(lengths, 0, out=offs[1:])
    fo = [0, 1, 4, 6]
    assert torch.equal(S.get_table_range(offs.cuda(), fo, 64).cpu(), S.get_table_range(offs, fo, 64))
    ub, inv, nl, no, uo = S.dedup_input_indices(ids.cuda(), offs.cuda(), fo, 64)
    rub, rinv, rnl, rno, ruo = S.dedup_input_indices(ids, offs, fo, 64)
    assert torch.equal(nl.cpu(), rnl) and torch.equal(no.cpu(), rno) and torch.equal(uo.cpu(), ruo)
    assert torch.equal(ub[inv].cpu(), ids)


@pytest.mark.gpu
@pytest.mark.parametrize("mean", [False, True])
@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
def test_pooled_segment_add_matches_index_add(mean, gdtype):
    """Sorted run-length reduction of bag gradients onto unique rows (skewed ids: a few rows span many groups of 64 pairs)."""
    from recsdk_b200.ops import _lib

    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(3)
    batch, F, D, U = 512, 3, 64, 2000
    bags = batch * F
    lengths = torch.randint(0, 9, (bags,), generator=g)
    n = int(lengths.sum())
    inv = torch.where(torch.rand(n, generator=g) < 0.3, torch.randint(0, 3, (n,), generator=g), torch.randint(0, U, (n,), generator=g))
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), lengths.cumsum(0)]).to(dev)
    grad = torch.randn(batch, F * D, generator=g).to(gdtype).to(dev)
    inv_d = inv.to(dev)
    bag_of = torch.repeat_interleave(torch.arange(bags, dtype=torch.int32, device=dev), lengths.to(dev))
    L = _lib.lib()
    keys_sorted, bags_sorted = torch.empty_like(inv_d), torch.empty_like(bag_of)
    tb = int(L.rb_sort_segments_temp_bytes(n))
    temp = torch.empty(tb, dtype=torch.uint8, device=dev)
    st = _lib.stream_ptr(dev)
    _lib.check(L.rb_sort_pairs_i64_i32(inv_d.data_ptr(), bag_of.data_ptr(), n, U.bit_length(), keys_sorted.data_ptr(),
                                       bags_sorted.data_ptr(), temp.data_ptr(), tb, st), "sort")
    assert bool((keys_sorted[1:] >= keys_sorted[:-1]).all())
    red = torch.zeros(U, D, device=dev)
    _lib.check(L.rb_pooled_segment_add(grad.data_ptr(), _lib.dtype_code(gdtype), grad.stride(0), keys_sorted.data_ptr(),
                                       bags_sorted.data_ptr(), offsets.data_ptr(), n, batch, D, int(mean), red.data_ptr(), st), "add")
    gg = grad.float().view(batch, F, D).permute(1, 0, 2).reshape(bags, D)
    if mean:
        gg = gg / lengths.to(dev).clamp(min=1).float()[:, None]
    want = torch.zeros(U, D, device=dev).index_add_(0, inv_d, gg[bag_of.long()])
    torch.testing.assert_close(red, want, rtol=1e-4, atol=1e-3)
    _lib.check_status()
