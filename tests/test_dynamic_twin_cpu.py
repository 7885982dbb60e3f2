"""A dynamic embedding collection and its static twin stay equal over several optimizer steps."""
import pytest
import torch

from recsdk_b200.dynamic import ConstructTwinModule, OptimizerType, generate_sparse_feature


@pytest.mark.parametrize("opt", [OptimizerType.SGD, OptimizerType.ROWWISE_ADAGRAD, OptimizerType.ADAGRAD, OptimizerType.ADAM])
def test_twin_models_track_each_other(opt):
    torch.manual_seed(0)
    dev = torch.device("cpu")
    twin = ConstructTwinModule(2, [8, 8], [40, 24], batch_size=16, device=dev,
                               optimizer_kwargs={"optimizer": opt, "learning_rate": 0.1, "eps": 1e-6, "initial_accumulator_value": 0.0})
    twin.init_twin_embedding_model()
    dyn, static = twin.dynamicemb_model, twin.torchrec_model
    names = ["f_0", "f_1"]
    for it in (0, 1, 0, 2):                                       # iteration 0 twice: rows with optimizer history
        kjt, ids = generate_sparse_feature(names, [40, 24], 16, it, device=dev)
        a, b = dyn(kjt), static(kjt)
        loss_a = sum((a[n].values() * (i + 1.5)).pow(2).sum() for i, n in enumerate(names))
        loss_b = sum((b[n].values() * (i + 1.5)).pow(2).sum() for i, n in enumerate(names))
        for n in names:
            torch.testing.assert_close(a[n].values(), b[n].values(), rtol=1e-5, atol=1e-6)
        loss_a.backward()
        loss_b.backward()
        static.step()
    kjt, _ = generate_sparse_feature(names, [40, 24], 16, 0, device=dev)
    a, b = dyn(kjt), static(kjt)
    for n in names:
        torch.testing.assert_close(a[n].values(), b[n].values(), rtol=1e-4, atol=1e-5)
        assert (b[n].values() - 0).abs().sum() > 0
