"""``recsdk_b200.modules.ids_process`` (the reference's ``hybrid_torchrec.modules.ids_process`` names): the mapper module, the
bucketisation entry with de-duplication and counts, and the names of the hybrid flow's modules, stages and contexts."""
import pytest
import torch

from recsdk_b200.modules import BucketParams, HashMapBase, IdsMapper, block_bucketize_sparse_features_cpu


def test_ids_mapper_module():
    m = IdsMapper(8)
    assert isinstance(m, HashMapBase) and isinstance(m, torch.nn.Module) and m.embedding_num == 8
    slots, uniq, inv = m(torch.tensor([100, 7, 100, 9]))
    assert slots.tolist() == [0, 1, 0, 2] and uniq.tolist() == [0, 1, 2] and uniq[inv].tolist() == slots.tolist() and m.size() == 3
    again, _, _ = m(torch.tensor([9, 55]))
    assert again.tolist() == [2, 3]                                         # known ids keep their slot, new ones take the next
    # the out-variant fills one table's part of batch-wide buffers
    ids = torch.tensor([5, 6, 5, 100, 100, 7])                              # table 0: first three values, table 1: the rest
    offset = torch.tensor([0, 3, 6])
    hash_indices, unique_inverse = torch.full((6,), -1), torch.full((6,), -1)
    unique, unique_ids = torch.full((6,), -1), torch.full((6,), -1)
    unique_offset = [0, 0, 0]
    t0, t1 = IdsMapper(8), IdsMapper(8)
    t0.ids2indices_unique_out(ids, hash_indices, offset, unique, unique_ids, unique_inverse, unique_offset, 0)
    t1.ids2indices_unique_out(ids, hash_indices, offset, unique, unique_ids, unique_inverse, unique_offset, 1)
    assert hash_indices.tolist() == [0, 1, 0, 0, 0, 1] and unique_offset == [0, 2, 4]
    assert unique_ids[:4].tolist() == [5, 6, 100, 7] and unique[:4].tolist() == [0, 1, 0, 1]
    assert unique_ids[unique_inverse].tolist() == ids.tolist()              # positions index the batch-wide unique list
    with pytest.raises(RuntimeError):
        m.statistic_key_count(torch.tensor([1]), None, torch.tensor([1]), 0)

    class Mgr:
        def __init__(self):
            self.seen = []

        def statistics_key_count(self, table, keys, counts, extra):
            self.seen.append((table, keys.tolist(), counts.tolist()))

    mgr = Mgr()
    m.set_cache_mgr(mgr)
    m.statistic_key_count(torch.tensor([4, 5]), None, torch.tensor([2, 1]), 3)
    assert mgr.seen == [(3, [4, 5], [2, 1])]


def test_bucketize_entry_with_dedup_and_counts():
    # F = 2, B = 2; bags: f0b0=[0,5,5] f0b1=[2,5] f1b0=[] f1b1=[7,7,1]; two buckets (id % 2)
    lengths, ids = torch.tensor([3, 2, 0, 3]), torch.tensor([0, 5, 5, 2, 5, 7, 7, 1])
    plain = block_bucketize_sparse_features_cpu(BucketParams(lengths, ids, False, True, torch.tensor([4, 4]), 2))
    assert plain[0].tolist() == [1, 1, 0, 0, 2, 1, 0, 3] and plain[1].tolist() == [0, 2, 5, 5, 5, 7, 7, 1]     # ids keep their value
    assert plain[2] is None and plain[3] is None and plain[1][plain[4]].tolist() == ids.tolist() and len(plain) == 5
    no_perm = block_bucketize_sparse_features_cpu(BucketParams(lengths, ids, False, False, torch.tensor([4, 4]), 2))
    assert no_perm[4] is None
    nl, ni, _w, _p, perm, counts = block_bucketize_sparse_features_cpu(
        BucketParams(lengths, ids, False, True, torch.tensor([4, 4]), 2, do_unique=True, return_count=True, labels=torch.tensor([1, 0])))
    assert nl.tolist() == [1, 1, 0, 0, 1, 0, 0, 2] and ni.tolist() == [0, 2, 5, 7, 1]      # 5 stays in the bag that saw it first
    assert ni[perm].tolist() == ids.tolist() and counts.tolist() == [[1, 1], [1, 0], [3, 2], [2, 0], [1, 0]]
    only_counts = block_bucketize_sparse_features_cpu(
        BucketParams(lengths, ids, False, True, torch.tensor([4, 4]), 2, do_unique=True, return_count=True))
    assert only_counts[5].tolist() == [[1], [1], [3], [2], [1]]
    weighted = block_bucketize_sparse_features_cpu(
        BucketParams(lengths, ids, False, True, torch.tensor([4, 4]), 2, weights=torch.arange(8, dtype=torch.float32), do_unique=True))
    assert weighted[2].tolist() == [0.0, 3.0, 1.0, 5.0, 7.0] and len(weighted) == 5          # the weight of the kept copy
    with pytest.raises(NotImplementedError):
        block_bucketize_sparse_features_cpu(BucketParams(lengths, ids, False, True, torch.tensor([4, 4]), 2,
                                                         batch_size_per_feature=torch.tensor([2, 2])))


def test_hybrid_flow_names():
    from recsdk_b200.modules import EmbeddingBagCollection, EmbeddingBagConfig
    from recsdk_b200.parallel import (CollectiveShardedEmbeddingBagCollection, HybridEmbeddingBagCollectionSharder, HybridPipelineContext,
                                      HybridShardedEmbeddingBagCollection, HybridShardedHashEmbeddingBagCollection, HybridStage,
                                      HybridTrainPipelineContext, ShardingEnv, TaskType)
    from recsdk_b200.ops import embedding_ops as E
    from recsdk_b200.sparse import KeyedJaggedTensor, KeyedJaggedTensorWithLookHelper

    assert HybridShardedEmbeddingBagCollection is CollectiveShardedEmbeddingBagCollection
    assert TaskType is HybridStage and HybridTrainPipelineContext is HybridPipelineContext
    assert [s.name for s in TaskType] == ["SPLIT", "FIRST_ALL2ALL", "SECOND_ALL2ALL", "POST_INPUT", "COPY_TO_DEVICE"]
    cfgs = [EmbeddingBagConfig(num_embeddings=32, embedding_dim=8, name="t", feature_names=["f"])]
    hashed = HybridShardedHashEmbeddingBagCollection(cfgs, {}, ShardingEnv(1, 0), torch.device("cpu"), E.OptimizerSpec(kind=E.OPT_SGD, lr=0.1),
                                                     out_dtype=torch.float32)
    kjt = KeyedJaggedTensor(["f"], torch.tensor([10**12, 7, 10**12]), lengths=torch.tensor([2, 1]))
    out = hashed(kjt).values()
    assert out.shape == (2, 8) and torch.isfinite(out).all()                 # raw 64-bit ids go through the id mapper
    ebc = EmbeddingBagCollection(cfgs)
    params = HybridEmbeddingBagCollectionSharder().shardable_parameters(ebc)
    assert list(params) == ["t"] and params["t"] is ebc.embedding_bags["t"].weight
    look = KeyedJaggedTensorWithLookHelper.from_kjt(kjt, hash_indices=torch.tensor([0, 1, 0]), unique_indices=torch.tensor([0, 1]),
                                                    unique_offset=torch.tensor([0, 2]), unique_inverse=torch.tensor([0, 1, 0]),
                                                    unique_ids=torch.tensor([10**12, 7]), unique_offset_host=[0, 2])
    moved = look.to(torch.device("cpu"))
    assert moved.unique_ids.tolist() == [10**12, 7] and moved.unique_offset_host == [0, 2]
    bare = KeyedJaggedTensorWithLookHelper.from_kjt(kjt, unique_offset=torch.tensor([0, 2]))
    assert bare.unique_offset_host == [0, 2] and bare.unique_ids is None       # read from the tensor when no host copy was given


def test_operator_form_of_block_bucketize():
    """``torch.ops.hybrid.block_bucketize_sparse_features_cpu`` with the reference's argument list and 7-entry result."""
    import recsdk_b200.modules.ids_process  # noqa: F401  (registers the operator)

    lengths, ids = torch.tensor([2, 1, 1, 2]), torch.tensor([4, 7, 4, 9, 6, 7])          # 2 features x batch 2
    op = torch.ops.hybrid.block_bucketize_sparse_features_cpu
    nl, ni, nw, npos, perm, mapping, counts = op(lengths, ids, False, True, torch.tensor([1, 1]), 2, max_B=2, return_bucket_mapping=True)
    assert nl.tolist() == [1, 1, 0, 1, 1, 0, 1, 1] and ni.tolist() == [4, 4, 6, 7, 9, 7]
    assert nw is None and npos is None and torch.equal(ni[perm], ids)
    assert mapping.tolist() == [0, 1, 0, 1, 0, 1] and counts.numel() == 0
    nl, ni, _, _, perm, mapping, counts = op(lengths, ids, False, False, torch.tensor([1, 1]), 2, None, None, None, 2, None, False, False,
                                             True, True)
    assert ni.tolist() == [4, 6, 7, 9, 7] and counts[:, 0].tolist() == [2, 1, 1, 1, 1] and mapping is None
    assert torch.equal(ni[perm], ids) and int(nl.sum()) == 5
    w = torch.arange(6, dtype=torch.float32)
    _, ni, nw, _, perm, _, _ = op(lengths, ids, False, True, torch.tensor([1, 1]), 2, weights=w, max_B=2)
    assert torch.equal(nw[perm], w)
    with pytest.raises(NotImplementedError):
        op(lengths, ids, False, True, torch.tensor([1, 1]), 2, max_B=2, block_bucketize_pos=[torch.tensor([0, 5, 10])])
