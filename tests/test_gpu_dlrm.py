"""Fused bf16 DLRM step on the GPU vs the fp32 PyTorch reference model with identical weights."""
import pytest
import torch

from recsdk_b200.models.dlrm import DLRM, DLRMTrain
from recsdk_b200.modules.embedding_configs import DataType, EmbeddingBagConfig
from recsdk_b200.modules.embedding_modules import EmbeddingBagCollection
from recsdk_b200.ops import _lib
from recsdk_b200.ops import embedding_ops as E
from recsdk_b200.optim import CombinedOptimizer, FusedDenseOptimizer
from recsdk_b200.parallel.comm import ShardingEnv
from recsdk_b200.parallel.model_parallel import DistributedModelParallel
from recsdk_b200.parallel.train_pipeline import TrainPipelineSparseDist
from recsdk_b200.utils.data import RandomRecDataset

pytestmark = pytest.mark.gpu


def _build(rows, D, bottom, top, one_hot=True):
    cfgs = [EmbeddingBagConfig(num_embeddings=r, embedding_dim=D, name="t%d" % i, feature_names=["f%d" % i],
                               data_type=DataType.FP32) for i, r in enumerate(rows)]
    torch.manual_seed(0)
    ref_ebc = EmbeddingBagCollection(cfgs, device=torch.device("cpu"))
    ref = DLRMTrain(DLRM(ref_ebc, 13, bottom, top, dense_device=torch.device("cpu"), fused=False))
    dev = torch.device("cuda", 0)
    ebc = EmbeddingBagCollection(cfgs, device=torch.device("cpu"))
    ebc.load_state_dict(ref_ebc.state_dict())
    fused = DLRMTrain(DLRM(ebc, 13, bottom, top, dense_device=dev))
    lin = [m for m in ref.model.dense_arch.net if isinstance(m, torch.nn.Linear)]
    fused.model.dense_arch.load_from_linears(lin)
    lin = [m for m in ref.model.over_arch.net if isinstance(m, torch.nn.Linear)]
    fused.model.over_arch.load_from_linears(lin)
    with torch.no_grad():
        fused.model.head.w32.copy_(ref.model.head.weight[0])
        fused.model.head.b32.copy_(ref.model.head.bias)
    dmp = DistributedModelParallel(fused, ShardingEnv(1, 0), dev,
                                   sparse_optimizer=E.OptimizerSpec(kind=E.OPT_SGD, lr=0.5), one_hot=one_hot,
                                   out_dtype=torch.bfloat16)
    return cfgs, ref, dmp, dev


def test_dlrm_fused_matches_reference_step():
    rows, D = [100, 2000, 50, 777, 31], 64
    cfgs, ref, dmp, dev = _build(rows, D, [128, 64], [256, 128, 64, 1])
    data = RandomRecDataset([c.feature_names[0] for c in cfgs], rows, 256, alpha=1.05, seed=3)
    batch = data.make_batch()
    loss_ref, _ = ref(batch)
    loss_ref.backward()
    opt = CombinedOptimizer([dmp.fused_optimizer, FusedDenseOptimizer(dmp.module, "sgd", lr=0.0)])
    opt.zero_grad()
    loss, (_, logits, _) = dmp(batch.to(dev))
    loss.backward()
    torch.cuda.synchronize()
    _lib.check_status()
    assert abs(loss.item() - loss_ref.item()) < 2e-2 * max(1.0, abs(loss_ref.item()))
    # dense gradients (bf16 compute vs fp32 reference)
    f = dmp.module.model
    lin = [m for m in ref.model.over_arch.net if isinstance(m, torch.nn.Linear)]
    for l, m in enumerate(lin):
        g, gr = f.over_arch.weight_grad(l).cpu(), m.weight.grad
        rel = (g - gr).norm() / (gr.norm() + 1e-12)
        assert rel < 6e-2, "top layer %d rel %g" % (l, rel)
        gb, gbr = f.over_arch.bias_grad(l).cpu(), m.bias.grad
        assert (gb - gbr).norm() / (gbr.norm() + 1e-12) < 6e-2
    lin = [m for m in ref.model.dense_arch.net if isinstance(m, torch.nn.Linear)]
    for l, m in enumerate(lin):
        g, gr = f.dense_arch.weight_grad(l).cpu(), m.weight.grad
        assert (g - gr).norm() / (gr.norm() + 1e-12) < 8e-2, "bottom layer %d" % l
    # sparse SGD update fused in backward: w_new = w - lr * grad
    for i, c in enumerate(cfgs):
        w_ref = ref.model.sparse_arch.embedding_bags[c.name].weight
        exp = w_ref.detach() - 0.5 * w_ref.grad
        got = f.sparse_arch.table_weight(c.name).detach().float().cpu()
        d = (got - exp).norm() / ((0.5 * w_ref.grad).norm() + 1e-12)
        assert d < 0.15, "table %s rel update err %g" % (c.name, d)


@pytest.mark.parametrize("cuda_graph", [False, True])
def test_dlrm_pipeline_trains(cuda_graph):
    rows, D = [1000, 5000, 300, 64], 128
    cfgs, _ref, dmp, dev = _build(rows, D, [512, 256, 128], [1024, 1024, 512, 256, 1])
    for sm in dmp.sharded_modules:
        sm.opt.kind = E.OPT_SGD
    opt = CombinedOptimizer([dmp.fused_optimizer, FusedDenseOptimizer(dmp.module, "adam", lr=2e-3)])
    data = RandomRecDataset([c.feature_names[0] for c in cfgs], rows, 1024, alpha=1.05, seed=5, pin=True)
    fixed = [data.make_batch() for _ in range(2)]

    def loop():
        while True:
            for b in fixed:
                yield b

    pipe = TrainPipelineSparseDist(dmp, opt, dev, return_loss=True, cuda_graph=cuda_graph)
    it = loop()
    losses = []
    for _ in range(40):
        loss, _ = pipe.progress(it)
        losses.append(loss.item())
    torch.cuda.synchronize()
    _lib.check_status()
    assert losses[-1] < 0.85 * losses[0], losses[::8]
