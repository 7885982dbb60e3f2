"""Dynamic embedding stack on the GPU hash table: the A100 golden trajectory, caching + host tier, dump/load."""
import pytest
import torch

from recsdk_b200.dynamic import (DynamicEmbDump, DynamicEmbeddingBagCollection, DynamicEmbeddingCollection,
                                 DynamicEmbInitializerArgs, DynamicEmbInitializerMode, DynamicEmbLoad,
                                 DynamicEmbScoreStrategy, DynamicEmbTableOptions, OptimizerType)
from recsdk_b200.modules.embedding_configs import EmbeddingBagConfig, EmbeddingConfig
from recsdk_b200.ops import _lib
from recsdk_b200.parallel.comm import ShardingEnv
from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor
from tests.test_dynamic_cpu import GOLDEN, _scenario_batch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _make(opt, cls=DynamicEmbeddingBagCollection, **kw):
    cfg_cls = EmbeddingBagConfig if cls is DynamicEmbeddingBagCollection else EmbeddingConfig
    cfgs = [cfg_cls(num_embeddings=1024, embedding_dim=8, name="t_%d" % i, feature_names=["cate_%d" % i]) for i in range(2)]
    options = {c.name: DynamicEmbTableOptions(
        initializer_args=DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.DEBUG),
        score_strategy=DynamicEmbScoreStrategy.STEP, **kw) for c in cfgs}
    return cls(cfgs, options, ShardingEnv(1, 0), DEV, optimizer_type=opt, learning_rate=0.1, eps=1e-8)


@pytest.mark.parametrize("opt", list(GOLDEN))
def test_golden_trajectory_on_gpu(opt):
    m = _make(opt)
    kjt = _scenario_batch().to(DEV)
    losses = []
    for _ in range(5):
        out = m(kjt).values()
        loss = (out * out).sum()
        loss.backward()
        losses.append(loss.item())
    _lib.check_status()
    tol = 4e-5 if opt == OptimizerType.ADAM else 5e-7
    for got, want in zip(losses, GOLDEN[opt]):
        assert abs(got - want) <= tol * abs(want) + 1e-3, (losses, GOLDEN[opt])


def test_sequence_collection_caching_and_dump(tmp_path):
    m = _make(OptimizerType.ROWWISE_ADAGRAD, cls=DynamicEmbeddingCollection, caching=True, max_capacity=128, init_capacity=128)
    g = torch.Generator().manual_seed(0)
    ref = {}
    for step in range(8):
        ids = torch.randint(0, 2000, (2 * 64,), generator=g)
        kjt = KeyedJaggedTensor(["cate_0", "cate_1"], ids.to(DEV), lengths=torch.ones(128, dtype=torch.int64, device=DEV), stride=64)
        out = m(kjt)
        emb = torch.cat([out["cate_0"].values(), out["cate_1"].values()])
        assert emb.shape == (128, 8)
        (emb ** 2).sum().backward()
    _lib.check_status()
    t0 = m.table("t_0")
    assert t0.table.size() <= 128 and t0.storage.size() > 0          # the cache spilled into the host tier
    DynamicEmbDump(str(tmp_path / "ck"), m, optim=True)
    m2 = _make(OptimizerType.ROWWISE_ADAGRAD, cls=DynamicEmbeddingCollection, caching=True, max_capacity=128, init_capacity=128)
    DynamicEmbLoad(str(tmp_path / "ck"), m2, optim=True)
    m.eval(); m2.eval()
    ids = torch.arange(0, 128)
    kjt = KeyedJaggedTensor(["cate_0", "cate_1"], ids.to(DEV), lengths=torch.ones(128, dtype=torch.int64, device=DEV), stride=64)
    a, b = m(kjt), m2(kjt)
    assert torch.allclose(a["cate_0"].values(), b["cate_0"].values()) and torch.allclose(a["cate_1"].values(), b["cate_1"].values())


@pytest.mark.parametrize("cls", [DynamicEmbeddingCollection, DynamicEmbeddingBagCollection])
def test_two_features_on_one_growing_table_update_once_per_step(cls):
    """Two features that read ONE small table which grows (rehash: every slot moves) during the first steps: the features
    are looked up together, so each key is updated exactly once per step with the sum of both features' gradients.
    Oracle: the same ids as a single feature on an identical table."""
    cfg_cls = EmbeddingBagConfig if cls is DynamicEmbeddingBagCollection else EmbeddingConfig

    def make(features):
        cfgs = [cfg_cls(num_embeddings=1 << 14, embedding_dim=8, name="shared", feature_names=features)]
        opts = {"shared": DynamicEmbTableOptions(initializer_args=DynamicEmbInitializerArgs(mode=DynamicEmbInitializerMode.DEBUG),
                                                  score_strategy=DynamicEmbScoreStrategy.STEP, init_capacity=128, max_capacity=1 << 14)}
        return cls(cfgs, opts, ShardingEnv(1, 0), DEV, optimizer_type=OptimizerType.ADAM, learning_rate=0.05, eps=1e-8)

    two, one = make(["fa", "fb"]), make(["fab"])
    g = torch.Generator().manual_seed(3)
    B = 64
    for step in range(6):
        ids = torch.randint(0, 400 * (step + 1), (2 * B,), generator=g)            # overlapping ids, growing key set
        ones = torch.ones(2 * B, dtype=torch.int64, device=DEV)
        k2 = KeyedJaggedTensor(["fa", "fb"], ids.to(DEV), lengths=ones, stride=B)
        k1 = KeyedJaggedTensor(["fab"], ids.to(DEV), lengths=torch.ones(2 * B, dtype=torch.int64, device=DEV), stride=2 * B)
        o2, o1 = two(k2), one(k1)
        if cls is DynamicEmbeddingBagCollection:
            v2 = o2.values()                                   # [B, 2 * 8]: feature fa | feature fb
            v2 = torch.cat([v2[:, :8], v2[:, 8:]], 0)          # -> the single feature's sample order
            v1 = o1.values()
        else:
            v2 = torch.cat([o2["fa"].values(), o2["fb"].values()])
            v1 = o1["fab"].values()
        assert torch.allclose(v2, v1, rtol=1e-5, atol=1e-5), step
        (v2 * v2).sum().backward()
        (v1 * v1).sum().backward()
    _lib.check_status()
    assert two.table("shared").table.capacity > 128            # the table did grow on the way
    ka, va, _ = two.lookup.export_keys_values("shared")
    kb, vb, _ = one.lookup.export_keys_values("shared")
    ia, ib = torch.argsort(ka), torch.argsort(kb)
    assert torch.equal(ka[ia], kb[ib]) and torch.allclose(va[ia], vb[ib], rtol=1e-5, atol=1e-5)
