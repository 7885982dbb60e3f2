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
