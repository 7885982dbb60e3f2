"""The train pipelines on the CPU path: the prefetching pipeline gives exactly the steps of the plain loop, ends with
``StopIteration`` when the iterator is exhausted, and the dataset / batch helpers behave."""
import pytest
import torch

from recsdk_b200.models.dlrm import DLRM, DLRMTrain
from recsdk_b200.modules.embedding_configs import EmbeddingBagConfig
from recsdk_b200.modules.embedding_modules import EmbeddingBagCollection
from recsdk_b200.parallel.train_pipeline import TrainPipelineBase, TrainPipelineSparseDist
from recsdk_b200.utils.data import Batch, RandomRecDataset

ROWS = [50, 20, 30]


def _model(seed=0):
    torch.manual_seed(seed)
    cfgs = [EmbeddingBagConfig(num_embeddings=r, embedding_dim=8, name="t%d" % i, feature_names=["f%d" % i]) for i, r in enumerate(ROWS)]
    return DLRMTrain(DLRM(EmbeddingBagCollection(cfgs), 4, [16, 8], [16, 1]))


def _batches(n, **kw):
    return list(RandomRecDataset(["f0", "f1", "f2"], ROWS, 32, num_dense=4, seed=5, num_batches=n, **kw))


@pytest.mark.parametrize("one_hot", [True, False])
def test_prefetching_pipeline_equals_plain_loop(one_hot):
    data = _batches(5, one_hot=one_hot, min_len=0, max_len=3)
    runs = []
    for kind in ("loop", "base", "sparse_dist"):
        m = _model()
        opt = torch.optim.SGD(m.parameters(), lr=0.1)
        losses = []
        if kind == "loop":
            for b in data:
                opt.zero_grad()
                loss, _ = m(b)
                loss.backward()
                opt.step()
                losses.append(float(loss.detach()))
        else:
            cls = TrainPipelineBase if kind == "base" else TrainPipelineSparseDist
            pipe = cls(m, opt, torch.device("cpu"), return_loss=True)
            it = iter(data)
            for _ in range(5):
                loss, out = pipe.progress(it)
                assert out[1].shape == (32,) and not loss.requires_grad
                losses.append(float(loss))
            with pytest.raises(StopIteration):
                pipe.progress(it)
        runs.append((losses, [p.detach().clone() for p in m.parameters()]))
    for losses, params in runs[1:]:
        assert losses == runs[0][0]
        assert all(torch.equal(a, b) for a, b in zip(params, runs[0][1]))
    assert runs[0][0][-1] < runs[0][0][0] + 0.5


def test_pipeline_returns_outputs_only_by_default():
    m = _model()
    pipe = TrainPipelineSparseDist(m, torch.optim.SGD(m.parameters(), lr=0.1), torch.device("cpu"))
    out = pipe.progress(iter(_batches(2)))
    assert isinstance(out, tuple) and len(out) == 3 and out[2].shape == (32,)
    assert pipe._status is None                                             # the device status word exists on CUDA only


def test_dataset_shapes_pinning_and_batch_helpers():
    ds = RandomRecDataset(["a", "b"], [10, 1000], 16, num_dense=3, one_hot=False, min_len=1, max_len=4, pos_rate=0.5, seed=1,
                          ids_dtype=torch.int32)
    b = ds.make_batch()
    kjt = b.sparse_features
    assert b.dense_features.shape == (16, 3) and b.labels.shape == (16,) and set(b.labels.tolist()) <= {0.0, 1.0}
    assert kjt.values().dtype == torch.int32 and kjt.stride() == 16 and kjt.lengths().numel() == 32
    assert 1 <= int(kjt.lengths().min()) and int(kjt.lengths().max()) <= 4
    assert int(kjt["a"].values().max()) < 10 and int(kjt["b"].values().max()) < 1000 and kjt.one_hot is False
    want = b.dense_features.numel() * 4 + 16 * 4 + kjt.values().numel() * 4 + kjt.lengths().numel() * 8
    assert b.nbytes() == want
    moved = b.to(torch.device("cpu"))
    assert isinstance(moved, Batch) and torch.equal(moved.labels, b.labels)
    b.record_stream(None)                                                   # host tensors: nothing to record
    again = RandomRecDataset(["a", "b"], [10, 1000], 16, num_dense=3, one_hot=False, min_len=1, max_len=4, pos_rate=0.5, seed=1,
                             ids_dtype=torch.int32).make_batch()
    assert torch.equal(again.sparse_features.values(), kjt.values())        # same seed, same stream of batches
    assert len(list(RandomRecDataset(["a"], [10], 4, num_batches=3))) == 3
