"""DCN v2 trains on CPU (fp32) with plain and dynamic embeddings; the GPU path matches the CPU path."""
import pytest
import torch

from recsdk_b200.models.dcn import DCNv2, DCNv2Train
from recsdk_b200.modules.embedding_configs import EmbeddingBagConfig
from recsdk_b200.modules.embedding_modules import EmbeddingBagCollection
from recsdk_b200.utils.data import RandomRecDataset


def _setup(device, low_rank):
    torch.manual_seed(0)
    cfgs = [EmbeddingBagConfig(num_embeddings=500, embedding_dim=16, name="t%d" % i, feature_names=["f%d" % i]) for i in range(3)]
    ebc = EmbeddingBagCollection(cfgs, device=torch.device(device))
    model = DCNv2Train(DCNv2(ebc, 13, [32, 16], cross_layers=2, low_rank=low_rank, deep_layer_sizes=[64, 32], device=device))
    data = RandomRecDataset(["f0", "f1", "f2"], [500] * 3, 128, alpha=1.05, one_hot=False, min_len=1, max_len=3, pos_rate=0.3, seed=0)
    return model, [data.make_batch() for _ in range(12)]


@pytest.mark.parametrize("low_rank", [0, 8])
def test_dcn_trains_cpu(low_rank):
    model, batches = _setup("cpu", low_rank)
    opt = torch.optim.Adam(model.parameters(), lr=3e-3)
    losses = []
    for _ in range(3):
        for b in batches:
            opt.zero_grad()
            loss, _ = model(b)
            loss.backward()
            opt.step()
            losses.append(float(loss.detach()))
    assert sum(losses[-6:]) < sum(losses[:6])


@pytest.mark.gpu
def test_dcn_gpu_matches_cpu():
    cpu, batches = _setup("cpu", 8)
    gpu, _ = _setup("cuda", 8)
    gpu.load_state_dict(cpu.state_dict())
    b = batches[0]
    lc, _ = cpu(b)
    lg, _ = gpu(b.to(torch.device("cuda")))
    assert abs(float(lc) - float(lg)) < 2e-2
    lc.backward()
    lg.backward()
    gc, gg = cpu.model.cross.u[0].weight.grad, gpu.model.cross.u[0].weight.grad.cpu()
    assert torch.allclose(gc, gg, atol=3e-3, rtol=5e-2)
