"""Unsharded embedding modules and their configuration on CPU: pooled, weighted, sequence and hash-mapped collections
against hand-written lookups; initialisation rules; the validation limits of hash tables."""
import pytest
import torch

from recsdk_b200.modules.embedding_configs import (DataType, EmbeddingBagConfig, EmbeddingConfig, PoolingType, data_type_to_dtype,
                                                   dtype_to_data_type, validate_hash_table_config)
from recsdk_b200.modules.embedding_modules import EmbeddingBagCollection, EmbeddingCollection
from recsdk_b200.modules.hash_embeddingbag import HashEmbeddingBagCollection, HashEmbeddingBagConfig, HashTableOption, HybridHashTable
from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor


def test_config_defaults_and_dtype_mapping():
    c = EmbeddingBagConfig(num_embeddings=400, embedding_dim=8, name="t")
    assert c.feature_names == ["t"] and c.num_features() == 1 and c.pooling == PoolingType.SUM
    assert c.get_weight_init_max() == pytest.approx(0.05) and c.get_weight_init_min() == pytest.approx(-0.05)
    d = EmbeddingBagConfig(num_embeddings=4, embedding_dim=8, name="u", feature_names=["a", "b"], weight_init_min=-1.0, weight_init_max=2.0)
    assert d.num_features() == 2 and (d.get_weight_init_min(), d.get_weight_init_max()) == (-1.0, 2.0)
    for dt in DataType:
        assert dtype_to_data_type(data_type_to_dtype(dt)) == dt
    with pytest.raises(ValueError):
        dtype_to_data_type(torch.int8)


def test_pooled_collection_matches_hand_lookup():
    ca = EmbeddingBagConfig(num_embeddings=10, embedding_dim=4, name="ta", feature_names=["a", "a2"])
    cb = EmbeddingBagConfig(num_embeddings=6, embedding_dim=2, name="tb", feature_names=["b"], pooling=PoolingType.MEAN,
                            init_fn=lambda w: w.fill_(0.5))
    ebc = EmbeddingBagCollection([ca, cb])
    assert ebc.embedding_bag_configs() == [ca, cb] and not ebc.is_weighted() and not ebc.is_meta() and ebc.device.type == "cpu"
    wa, wb = ebc.embedding_bags["ta"].weight, ebc.embedding_bags["tb"].weight
    assert float(wa.detach().abs().max()) <= (1 / 10) ** 0.5 and torch.all(wb == 0.5)
    # B = 2; a: [1,2],[3]   a2: [],[9]   b: [0,5],[4]
    kjt = KeyedJaggedTensor(["a", "a2", "b"], torch.tensor([1, 2, 3, 9, 0, 5, 4]), lengths=torch.tensor([2, 1, 0, 1, 2, 1]))
    out = ebc(kjt)
    assert out.keys() == ["a", "a2", "b"] and out.length_per_key() == [4, 4, 2]
    assert torch.allclose(out["a"], torch.stack([wa[1] + wa[2], wa[3]]))
    assert torch.allclose(out["a2"], torch.stack([torch.zeros(4), wa[9]]))
    assert torch.allclose(out["b"], torch.full((2, 2), 0.5))
    out.values().sum().backward()
    assert wa.grad[1].tolist() == [1.0] * 4 and wa.grad[0].tolist() == [0.0] * 4
    with torch.no_grad():
        wa.zero_()
    ebc.reset_parameters()
    assert float(wa.detach().abs().sum()) > 0 and torch.all(wb == 0.5)
    with pytest.raises(ValueError, match="duplicate"):
        EmbeddingBagCollection([ca, ca])
    meta = EmbeddingBagCollection([ca], device=torch.device("meta"))
    assert meta.is_meta() and meta.embedding_bags["ta"].weight.device.type == "meta"


def test_weighted_collection_applies_per_sample_weights():
    c = EmbeddingBagConfig(num_embeddings=5, embedding_dim=2, name="t", feature_names=["f"])
    ebc = EmbeddingBagCollection([c], is_weighted=True)
    w = ebc.embedding_bags["t"].weight
    kjt = KeyedJaggedTensor(["f"], torch.tensor([1, 2, 3]), weights=torch.tensor([0.5, 2.0, -1.0]), lengths=torch.tensor([2, 1]))
    out = ebc(kjt)["f"]
    assert torch.allclose(out, torch.stack([0.5 * w[1] + 2.0 * w[2], -w[3]]))


def test_sequence_collection_returns_jagged_rows():
    c1 = EmbeddingConfig(num_embeddings=7, embedding_dim=4, name="items", feature_names=["hist", "cand"])
    ec = EmbeddingCollection([c1], need_indices=True)
    assert ec.embedding_configs() == [c1] and ec.embedding_dim() == 4 and not ec.is_meta()
    w = ec.embeddings["items"].weight
    kjt = KeyedJaggedTensor(["hist", "cand"], torch.tensor([1, 2, 3, 6]), lengths=torch.tensor([3, 0, 0, 1]))
    out = ec(kjt)
    assert set(out) == {"hist", "cand"} and out["hist"].lengths().tolist() == [3, 0] and out["cand"].lengths().tolist() == [0, 1]
    assert torch.equal(out["hist"].values(), w[[1, 2, 3]]) and torch.equal(out["cand"].values(), w[[6]])
    assert out["hist"].weights().tolist() == [1, 2, 3]                     # need_indices: the ids ride along
    assert EmbeddingCollection([c1])(kjt)["hist"].weights_or_none() is None
    with pytest.raises(ValueError, match="share embedding_dim"):
        EmbeddingCollection([c1, EmbeddingConfig(num_embeddings=3, embedding_dim=8, name="other")])
    assert EmbeddingCollection([c1], device=torch.device("meta")).is_meta()


def test_hash_collection_maps_raw_ids_to_slots():
    c = HashEmbeddingBagConfig(num_embeddings=16, embedding_dim=8, name="h", feature_names=["f"])
    hbc = HashEmbeddingBagCollection([c])
    table = hbc.embedding_bags["h"]
    assert isinstance(table, HybridHashTable)
    ids = torch.tensor([10**12, 7, 10**12, 123456789])
    slots = table.slots(ids)
    assert slots[0] == slots[2] and len(set(slots.tolist())) == 3 and int(slots.max()) < 16
    kjt = KeyedJaggedTensor(["f"], ids, lengths=torch.tensor([3, 1]))
    out = hbc(kjt)["f"]
    w = table.weight
    assert torch.allclose(out[0], 2 * w[slots[0]] + w[slots[1]]) and torch.allclose(out[1], w[slots[3]])
    assert torch.equal(table.slots(torch.tensor([7])), slots[1:2])         # the mapping is stable across calls
    assert HashTableOption().max_load_factor == 0.5 and HashTableOption(dim=32).dim == 32


@pytest.mark.parametrize("kw, msg", [
    (dict(name="bad name!"), "table name"), (dict(name=""), "table name"), (dict(embedding_dim=12), "multiple of 8"),
    (dict(embedding_dim=4), "multiple of 8"), (dict(embedding_dim=8192), "multiple of 8"), (dict(num_embeddings=0), "num_embeddings"),
    (dict(num_embeddings=2_000_000_000), "num_embeddings"), (dict(data_type=DataType.FP16), "fp32 only"),
    (dict(feature_names=["ok", "not ok"]), "feature name")])
def test_hash_table_limits(kw, msg):
    base = dict(num_embeddings=100, embedding_dim=16, name="t", feature_names=["f"])
    base.update(kw)
    with pytest.raises(ValueError, match=msg):
        validate_hash_table_config(HashEmbeddingBagConfig(**base))


def test_hash_collection_rejections():
    c = HashEmbeddingBagConfig(num_embeddings=16, embedding_dim=8, name="h")
    validate_hash_table_config(c)
    with pytest.raises(ValueError, match="weighted"):
        HashEmbeddingBagCollection([c], is_weighted=True)
    with pytest.raises(ValueError, match="empty"):
        HashEmbeddingBagCollection([])
    with pytest.raises(ValueError, match="duplicate"):
        HashEmbeddingBagCollection([c, c])


def test_table_names_that_shadow_container_methods():
    """``items`` / ``keys`` / ``values`` are ordinary table names: holders are reached by subscript, the state dict uses the
    table name, and a sharded collection accepts them as well."""
    from recsdk_b200.modules.embedding_modules import TableDict
    from recsdk_b200.ops import embedding_ops as E
    from recsdk_b200.parallel.collective_embeddingbag import CollectiveShardedEmbeddingBagCollection
    from recsdk_b200.parallel.comm import ShardingEnv

    cfgs = [EmbeddingBagConfig(num_embeddings=6, embedding_dim=8, name=n, feature_names=["f_" + n]) for n in ("items", "keys", "values")]
    ebc = EmbeddingBagCollection(cfgs)
    assert sorted(ebc.state_dict()) == ["embedding_bags.items.weight", "embedding_bags.keys.weight", "embedding_bags.values.weight"]
    assert list(ebc.embedding_bags.keys()) == ["items", "keys", "values"] and "items" in ebc.embedding_bags
    other = EmbeddingBagCollection(cfgs)
    other.load_state_dict(ebc.state_dict())
    assert torch.equal(other.embedding_bags["items"].weight, ebc.embedding_bags["items"].weight)
    kjt = KeyedJaggedTensor(["f_items", "f_keys", "f_values"], torch.tensor([1, 2, 3]), lengths=torch.tensor([1, 1, 1]))
    assert torch.equal(ebc(kjt)["f_items"][0], ebc.embedding_bags["items"].weight[1])
    ec = EmbeddingCollection([EmbeddingConfig(num_embeddings=6, embedding_dim=8, name="items")])
    assert list(ec.state_dict()) == ["embeddings.items.weight"]
    sh = CollectiveShardedEmbeddingBagCollection(cfgs, {}, ShardingEnv(1, 0), torch.device("cpu"), E.OptimizerSpec(kind=E.OPT_SGD, lr=0.1),
                                                 out_dtype=torch.float32)
    sh.load_from_unsharded(ebc)
    assert torch.allclose(sh(kjt).values(), ebc(kjt).values())
    d = TableDict()
    for bad in ("", "a.b", 3):
        with pytest.raises(KeyError):
            d[bad] = torch.nn.Identity()
    with pytest.raises(TypeError):
        d["x"] = "not a module"
