"""``KeyedJaggedTensor``: constructors, per-key views, split / permute / concat (values, weights, lengths and the
one-id-per-bag promise travel together), device moves and the tensors handed to the input distribution."""
import pytest
import torch

from recsdk_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor


def _kjt(weighted=False):
    # keys a, b, c; B = 2; a: [1,2],[3]   b: [],[4]   c: [5],[6,7,8]
    vals = torch.tensor([1, 2, 3, 4, 5, 6, 7, 8])
    w = torch.arange(8, dtype=torch.float32) / 10 if weighted else None
    return KeyedJaggedTensor(["a", "b", "c"], vals, w, lengths=torch.tensor([2, 1, 0, 1, 1, 3]))


def test_construction_and_per_key_views():
    k = _kjt()
    assert k.stride() == 2 and k.length_per_key() == [3, 1, 4] and k.offset_per_key() == [0, 3, 4, 8]
    assert k.offsets().tolist() == [0, 2, 3, 3, 4, 5, 8] and k.device().type == "cpu"
    assert k["c"].values().tolist() == [5, 6, 7, 8] and k["c"].lengths().tolist() == [1, 3] and k["b"].to_dense()[0].numel() == 0
    assert "nnz=8" in repr(k) and "JaggedTensor" in repr(k["a"])
    by_off = KeyedJaggedTensor(["a", "b", "c"], k.values(), offsets=k.offsets())
    assert by_off.lengths().tolist() == k.lengths().tolist() and by_off.stride() == 2
    sync = KeyedJaggedTensor.from_lengths_sync(["a", "b", "c"], k.values(), k.lengths())
    assert sync._length_per_key == [3, 1, 4]
    with pytest.raises(ValueError):
        KeyedJaggedTensor(["a"], torch.tensor([1]))
    with pytest.raises(ValueError):
        _kjt().weights()
    e = KeyedJaggedTensor.empty(is_weighted=True)
    assert e.keys() == [] and e.stride() == 0 and e.length_per_key() == [] and e.weights().numel() == 0
    je = JaggedTensor.empty(is_weighted=True)
    assert je.values().numel() == 0 and je.lengths().numel() == 0


def test_split_permute_concat_round_trip():
    k = _kjt(weighted=True)
    k.one_hot = True                                        # a promise of the producer; transforms must not drop it
    head, tail = k.split([1, 2])
    assert head.keys() == ["a"] and tail.keys() == ["b", "c"] and head.one_hot and tail.one_hot
    assert tail.values().tolist() == [4, 5, 6, 7, 8] and tail.lengths().tolist() == [0, 1, 1, 3]
    assert tail.weights().tolist() == pytest.approx([0.3, 0.4, 0.5, 0.6, 0.7]) and tail.length_per_key() == [1, 4]
    back = KeyedJaggedTensor.concat([head, tail])
    assert back.keys() == k.keys() and torch.equal(back.values(), k.values()) and torch.equal(back.lengths(), k.lengths())
    assert torch.equal(back.weights(), k.weights()) and back.one_hot and back.stride() == 2
    p = k.permute([2, 0, 0])                                # reorder and repeat
    assert p.keys() == ["c", "a", "a"] and p.values().tolist() == [5, 6, 7, 8, 1, 2, 3, 1, 2, 3] and p.one_hot
    assert p.lengths().tolist() == [1, 3, 2, 1, 2, 1] and p.length_per_key() == [4, 3, 3]
    assert p.weights().tolist() == pytest.approx([0.4, 0.5, 0.6, 0.7, 0.0, 0.1, 0.2, 0.0, 0.1, 0.2])
    same = k.permute([1, 2], indices_tensor=torch.tensor([1, 2]))
    assert same.keys() == ["b", "c"] and same.values().tolist() == [4, 5, 6, 7, 8]
    none = k.permute([])
    assert none.keys() == [] and none.values().numel() == 0
    mixed = KeyedJaggedTensor.concat([head, _kjt().split([1, 2])[1]])      # one side without weights: weights are dropped
    assert mixed.weights_or_none() is None and not mixed.one_hot


def test_moves_and_dist_tensors():
    k = _kjt(weighted=True)
    k.one_hot = True
    m = k.to(torch.device("cpu"))
    assert m.one_hot and torch.equal(m.values(), k.values()) and m.keys() == k.keys()
    assert k.dist_labels() == ["lengths", "values", "weights"] and len(k.dist_tensors()) == 3
    assert _kjt().dist_labels() == ["lengths", "values"] and _kjt().dist_tensors()[1].tolist() == list(range(1, 9))
    k.record_stream(None)                                   # host tensors: nothing to record
    d = k.to_dict()
    assert list(d) == ["a", "b", "c"] and d["a"].weights().tolist() == pytest.approx([0.0, 0.1, 0.2])
    jt = d["c"].to(torch.device("cpu"))
    assert jt.offsets().tolist() == [0, 1, 4]
    if torch.cuda.is_available():
        assert k.pin_memory().values().is_pinned()


def test_small_accessors():
    k = _kjt(weighted=True)
    assert k.index_per_key() == {"a": 0, "b": 1, "c": 2} and len(k) == 3 and not k.variable_stride_per_key()
    assert k.stride_per_key() == [2, 2, 2] and k.lengths_offset_per_key() == [0, 2, 4, 6] and k.inverse_indices_or_none() is None
    assert k.unsync()._length_per_key is None and k.sync()._offset_per_key == [0, 3, 4, 8]
    two_d = KeyedJaggedTensor(["a", "b", "c"], k.values(), lengths=k.lengths().view(3, 2), stride=2)
    assert two_d.flatten_lengths().lengths().shape == (6,) and two_d.flatten_lengths()["c"].values().tolist() == [5, 6, 7, 8]
    e = KeyedJaggedTensor.empty_like(k)
    assert e.keys() == k.keys() and e.stride() == 2 and e.values().numel() == 0 and e.lengths().tolist() == [0] * 6
    assert e.weights().numel() == 0 and e["b"].values().numel() == 0
