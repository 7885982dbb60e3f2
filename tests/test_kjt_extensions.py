import torch

from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor
from recsdk_b200.sparse.kjt_extensions import (ExtendedJaggedTensor, KeyedJaggedTensorWithCount, KeyedJaggedTensorWithLookHelper,
                                               KeyedJaggedTensorWithTimestamp)


def test_side_tensors_follow_values():
    vals = torch.tensor([10, 11, 12, 13, 14, 15])
    lens = torch.tensor([1, 2, 0, 3])                      # 2 keys x batch 2
    k = KeyedJaggedTensorWithLookHelper(["a", "b"], vals, lengths=lens, hash_indices=vals * 2, unique_inverse=vals - 10,
                                        unique_indices=torch.tensor([7, 8]), unique_offset=torch.tensor([0, 1, 2]))
    a, b = k.split([1, 1])
    assert a.hash_indices.tolist() == [20, 22, 24] and b.hash_indices.tolist() == [26, 28, 30]
    assert b.unique_indices.tolist() == [7, 8] and isinstance(b, KeyedJaggedTensorWithLookHelper)
    p = k.permute([1, 0])
    assert p.keys() == ["b", "a"] and p.values().tolist() == [13, 14, 15, 10, 11, 12] and p.unique_inverse.tolist() == [3, 4, 5, 0, 1, 2]
    moved = k.to(torch.device("cpu"))
    assert moved.hash_indices.tolist() == k.hash_indices.tolist() and moved["a"].values().tolist() == [10, 11, 12]
    t = KeyedJaggedTensorWithTimestamp(["a", "b"], vals, lengths=lens, timestamps=vals + 100)
    assert t.split([1, 1])[1].timestamps.tolist() == [113, 114, 115]
    try:
        KeyedJaggedTensorWithTimestamp(["a"], vals, lengths=torch.tensor([6]), timestamps=vals[:2])
        assert False
    except ValueError:
        pass


def test_dedup_with_counts_and_extended_jt():
    k = KeyedJaggedTensor(["a"], torch.tensor([5, 5, 7, 9, 9, 9]), lengths=torch.tensor([3, 3]))
    d = KeyedJaggedTensorWithCount.dedup(k)
    assert d.values().tolist() == [5, 7, 9] and d.counts.tolist() == [2, 1, 3] and d.lengths().tolist() == [2, 1]
    e = ExtendedJaggedTensor(torch.arange(4.), lengths=torch.tensor([1, 3]), extras={"ts": torch.arange(4) + 50})
    assert e.to(torch.device("cpu")).extras["ts"].tolist() == [50, 51, 52, 53]


def test_side_tensor_kjt_concat_dict_dist_roundtrip_and_validation():
    import pytest
    import torch

    from recsdk_b200.sparse.kjt_extensions import (KeyedExtendedJaggedTensor, KeyedJaggedTensorWithCount,
                                                   KeyedJaggedTensorWithTimestamp)

    a = KeyedJaggedTensorWithCount.from_lengths_sync(["f0", "f1"], torch.tensor([5, 6, 7, 8, 9]), torch.tensor([1, 2, 0, 2]),
                                                     counts=torch.tensor([1, 1, 2, 3, 1]))
    b = KeyedJaggedTensorWithCount.from_lengths_sync(["f2"], torch.tensor([1, 2, 3]), torch.tensor([3, 0]), counts=torch.tensor([4, 4, 4]))
    c = KeyedJaggedTensorWithCount.concat([a, b])
    assert c.keys() == ["f0", "f1", "f2"] and c.counts.tolist() == [1, 1, 2, 3, 1, 4, 4, 4]
    d = c.to_dict()
    assert d["f1"].values().tolist() == [8, 9] and d["f1"].extras["counts"].tolist() == [3, 1]
    # what an all-to-all carries, and the batch rebuilt from it
    assert c.dist_labels() == ["lengths", "values", "counts"]
    assert c.dist_splits([2, 1]) == [[4, 2], [5, 3], [5, 3]]
    r = KeyedJaggedTensorWithCount.dist_init(c.keys(), c.dist_tensors(), c.dist_labels(), c.stride())
    assert r.values().tolist() == c.values().tolist() and r.counts.tolist() == c.counts.tolist()
    e = KeyedJaggedTensorWithTimestamp.empty_like(c)
    assert e.values().numel() == 0 and e.stride() == 2 and e.timestamps.numel() == 0
    assert "counts=(8,)" in str(c)
    x = KeyedExtendedJaggedTensor(["k0", "k1"], torch.arange(4), lengths=torch.tensor([1, 1, 1, 1]), extra=torch.tensor([.1, .2, .3, .4]))
    p0, p1 = x.split([1, 1])
    assert p1.extra.tolist() == pytest.approx([.3, .4]) and x.to_base().keys() == ["k0", "k1"]
    with pytest.raises(ValueError):
        KeyedExtendedJaggedTensor(["k", "k"], torch.arange(2), lengths=torch.tensor([1, 1]))
    with pytest.raises(TypeError):
        KeyedExtendedJaggedTensor(["k"], torch.arange(2), lengths=torch.tensor([2]), length_per_key=[2.0])
    with pytest.raises(ValueError):
        KeyedExtendedJaggedTensor(["k"], torch.arange(2), lengths=torch.tensor([2]), extra=torch.arange(3))
    with pytest.raises(ValueError):
        KeyedExtendedJaggedTensor(["k"], torch.arange(2))


def test_generic_forms_that_take_the_class_to_build():
    """``split_extend`` / ``permute_extend`` / ``pin_memory_extend`` (``extended_jagged_tensor.py:288-580`` of the reference) and
    the single ``extra`` of an extended jagged tensor."""
    import pytest
    import torch

    from recsdk_b200.sparse import (ExtendedJaggedTensor, KeyedExtendedJaggedTensor, KeyedJaggedTensorWithCount)

    k = KeyedJaggedTensorWithCount(["a", "b"], torch.tensor([1, 2, 3]), lengths=torch.tensor([2, 0, 0, 1]), counts=torch.tensor([7, 8, 9]))
    head, tail = k.split_extend([1, 1])
    assert isinstance(tail, KeyedJaggedTensorWithCount) and tail.counts.tolist() == [9] and head.counts.tolist() == [7, 8]
    as_ext = k.split_extend([2], lambda **kw: KeyedExtendedJaggedTensor(kw["keys"], kw["values"], kw["weights"], kw["lengths"], kw["offsets"],
                                                                         kw["stride"], extra=kw["counts"]))[0]
    assert isinstance(as_ext, KeyedExtendedJaggedTensor) and as_ext.extra.tolist() == [7, 8, 9]
    with pytest.raises(ValueError):
        k.split_extend([1, 1, 1])
    p = k.permute_extend([1, 0], None, None, extra_permute_func=lambda t: t * 10)
    assert p.keys() == ["b", "a"] and p.values().tolist() == [3, 1, 2] and p.counts.tolist() == [90, 70, 80]
    if torch.cuda.is_available():
        assert k.pin_memory_extend().counts.is_pinned()
    one = ExtendedJaggedTensor(torch.tensor([1, 2]), lengths=torch.tensor([2]), extras={"ts": torch.tensor([5, 6])})
    assert one.extra.tolist() == [5, 6]
    assert ExtendedJaggedTensor(torch.tensor([1]), lengths=torch.tensor([1])).extra is None
