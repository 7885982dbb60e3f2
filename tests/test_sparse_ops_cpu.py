"""The host path of the id-preprocessing ops (the oracle the GPU kernels are compared with), checked against
hand-written expectations: segmented unique, bucketisation by owner, compaction, table ranges."""
import torch

from recsdk_b200.ops import sparse_ops as S


def _t(*a, dtype=torch.int64):
    return torch.tensor(list(a), dtype=dtype)


def test_segmented_unique_per_table():
    keys = _t(5, 3, 5, 9, 3, 3, 7, 7)               # table 0: first five ids, table 1: the rest
    ub, inv, uo, cnt = S.segmented_unique(keys, _t(0, 5, 8), with_counts=True)
    assert uo.tolist() == [0, 3, 5]
    assert ub[:3].tolist() == [3, 5, 9] and ub[3:5].tolist() == [3, 7]      # the same id is distinct per table
    assert torch.equal(ub[inv], keys) and ub.numel() == keys.numel()
    assert cnt[:5].tolist() == [2, 2, 1, 1, 2]
    assert S.segmented_unique(keys, _t(0, 5, 8))[3] is None
    ub, inv, uo, _ = S.segmented_unique(_t(4, 4), _t(0, 0, 2))               # an empty table in front
    assert uo.tolist() == [0, 0, 1] and ub[0] == 4 and inv.tolist() == [0, 0]
    u, inv, c = S.unique(_t(2, 1, 2, 2), with_counts=True)
    assert u.tolist() == [1, 2] and inv.tolist() == [1, 0, 1, 1] and c.tolist() == [1, 3]
    u, inv = S.unique(torch.empty(0, dtype=torch.int64))
    assert u.numel() == 0 and inv.numel() == 0


def test_block_bucketize_round_robin_and_blocks():
    # F = 2 features, B = 2 samples; bags: f0b0=[0,5] f0b1=[2] f1b0=[] f1b1=[7,8,1]
    lengths, ids = _t(2, 1, 0, 3), _t(0, 5, 2, 7, 8, 1)
    nl, ni, nw, perm = S.block_bucketize_sparse_features(lengths, ids, 2, 2, 2)
    # bucket-major: [rank0: f0b0 f0b1 f1b0 f1b1 | rank1: ...]
    assert nl.tolist() == [1, 1, 0, 1, 1, 0, 0, 2] and nw is None
    assert ni.tolist() == [0, 2, 8, 5, 7, 1]                                 # ids keep their value, order inside a bag is kept
    assert ni[perm].tolist() == ids.tolist()                                 # the permutation undoes the bucketisation
    nl2, ni2, _, _ = S.block_bucketize_sparse_features(lengths, ids, 2, 2, 2, local_rows=True)
    assert nl2.tolist() == nl.tolist() and ni2.tolist() == [0, 1, 4, 2, 3, 0]   # id // world on the owner
    # contiguous blocks: feature 0 in blocks of 3 rows, feature 1 in blocks of 5; ids past the last block stay on the last rank
    nl3, ni3, nw3, perm3 = S.block_bucketize_sparse_features(lengths, ids, 2, 2, 2, block_sizes=_t(3, 5),
                                                             weights=torch.arange(6, dtype=torch.float32), want_permute=False)
    assert nl3.tolist() == [1, 1, 0, 1, 1, 0, 0, 2] and perm3 is None
    assert ni3.tolist() == [0, 2, 1, 5, 7, 8] and nw3.tolist() == [0.0, 2.0, 5.0, 1.0, 3.0, 4.0]
    nl4, ni4, _, _ = S.block_bucketize_sparse_features(lengths, ids, 2, 2, 2, block_sizes=_t(3, 5), local_rows=True)
    assert ni4.tolist() == [0, 2, 1, 2, 2, 3]                                # id - rank * block
    far = S.block_bucketize_sparse_features(_t(1), _t(100), 2, 1, 1, block_sizes=_t(3))
    assert far[0].tolist() == [0, 1]                                         # clamped to the last rank


def test_select_and_table_range_and_new_lengths():
    flags = torch.tensor([1, 0, 1, 1, 0], dtype=torch.bool)
    out, n = S.select(_t(10, 11, 12, 13, 14), flags)
    assert int(n) == 3 and out[:3].tolist() == [10, 12, 13] and out.numel() == 5
    pos, n = S.select_index(flags)
    assert int(n) == 3 and pos[:3].tolist() == [0, 2, 3]
    none, n0 = S.select(None, torch.zeros(4, dtype=torch.bool))
    assert int(n0) == 0 and none.numel() == 4
    # three features, the first two share a table; B = 2
    offsets = _t(0, 2, 3, 3, 6, 7, 9)
    assert S.get_table_range(offsets, [0, 2, 3], 2).tolist() == [0, 6, 9]
    assert S.get_table_range(offsets.int(), [0, 1, 2, 3], 2).tolist() == [0, 3, 6, 9]
    nl, no = S.get_new_length_and_offsets(_t(0, 3, 3), [0, 2, 3], 2)
    assert nl.tolist() == [1, 1, 1, 0, 0, 0] and no.tolist() == [0, 1, 2, 3, 3, 3, 3]


def test_workspace_grows_and_is_reused():
    dev = torch.device("cpu")
    a = S._ws(dev, "probe", 10, torch.int32)
    assert a.numel() >= 1024 and S._ws(dev, "probe", 100, torch.int32) is a
    b = S._ws(dev, "probe", 5000, torch.int32)
    assert b is not a and b.numel() >= 5000 and S._ws(dev, "probe", 10, torch.int64) is not b
