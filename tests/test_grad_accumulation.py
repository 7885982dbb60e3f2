"""Sparse gradient accumulation: with ``use_accumulate`` and ``accumulate_step=2`` two half batches update the tables
exactly like one step on their union."""
import torch

from recsdk_b200.modules.embedding_configs import EmbeddingBagConfig
from recsdk_b200.modules.embedding_modules import EmbeddingBagCollection
from recsdk_b200.optim import AccumulateSGD, apply_optimizer_in_backward
from recsdk_b200.parallel import DistributedModelParallel
from recsdk_b200.sparse.jagged_tensor import KeyedJaggedTensor


def _dmp(opt_cls, kw):
    torch.manual_seed(0)
    ebc = EmbeddingBagCollection([EmbeddingBagConfig(num_embeddings=50, embedding_dim=8, name="t", feature_names=["f"])])
    apply_optimizer_in_backward(opt_cls, ebc.parameters(), kw)

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.ebc = ebc

        def forward(self, kjt):
            return self.ebc(kjt).values().pow(2).sum()

    return DistributedModelParallel(M(), device=torch.device("cpu"), backend="collective")


def test_two_accumulated_passes_equal_one_step_on_the_union():
    a = KeyedJaggedTensor(["f"], torch.tensor([1, 2, 2, 7]), lengths=torch.tensor([2, 2]))
    b = KeyedJaggedTensor(["f"], torch.tensor([2, 9, 7]), lengths=torch.tensor([1, 2]))
    both = KeyedJaggedTensor(["f"], torch.tensor([1, 2, 2, 7, 2, 9, 7]), lengths=torch.tensor([2, 2, 1, 2]))
    acc = _dmp(AccumulateSGD, {"lr": 0.1, "use_accumulate": True, "accumulate_step": 2})
    ref = _dmp(torch.optim.SGD, {"lr": 0.1})
    w0 = acc.module.ebc.table_weight("t").clone()
    acc(a).backward()
    assert torch.equal(acc.module.ebc.table_weight("t"), w0)          # nothing applied after the first pass
    acc(b).backward()
    ref(both).backward()
    assert torch.allclose(acc.module.ebc.table_weight("t"), ref.module.ebc.table_weight("t"), atol=1e-6)
    assert not torch.equal(acc.module.ebc.table_weight("t"), w0)
