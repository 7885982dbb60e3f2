"""The five-stage, multi-line host pipeline (``HybridTrainPipelineSparseDist``) on one CPU rank: stage order per batch,
lookahead, draining, argument checks, and the same losses as the unpipelined loop.  The two-rank gloo run (fused lengths
exchange over a separate host group) is in test_dist_cpu_dlrm.py."""
import pytest
import torch

from recsdk_b200.models.dlrm import DLRM, DLRMTrain
from recsdk_b200.modules.hash_embeddingbag import HashEmbeddingBagCollection, HashEmbeddingBagConfig
from recsdk_b200.ops import embedding_ops as E
from recsdk_b200.optim import CombinedOptimizer, KeyedOptimizerWrapper, apply_optimizer_in_backward
from recsdk_b200.parallel import HybridTrainPipelineSparseDist, get_default_hybrid_sharders
from recsdk_b200.parallel.comm import ShardingEnv
from recsdk_b200.parallel.hybrid import HybridStage
from recsdk_b200.parallel.model_parallel import DistributedModelParallel
from recsdk_b200.parallel.train_pipeline import TrainPipelineBase
from recsdk_b200.utils.data import RandomRecDataset

T, ROWS, D, B, STEPS = 4, 5000, 16, 64, 20


def _setup(pipelined: bool, pipe_n_batch: int = 2):
    torch.manual_seed(0)
    cfgs = [HashEmbeddingBagConfig(num_embeddings=ROWS, embedding_dim=D, name="t%d" % i, feature_names=["f%d" % i],
                                   init_fn=lambda w: w.fill_(0.01)) for i in range(T)]
    ebc = HashEmbeddingBagCollection(cfgs, device=torch.device("cpu"))
    apply_optimizer_in_backward(torch.optim.Adagrad, ebc.parameters(), {"lr": 0.01})
    model = DLRMTrain(DLRM(ebc, 13, [32, D], [32, 1], dense_device=torch.device("cpu"), fused=False))
    env = ShardingEnv(1, 0, None)
    dmp = DistributedModelParallel(model, env, torch.device("cpu"), None, sharders=get_default_hybrid_sharders(env),
                                   sparse_optimizer=E.OptimizerSpec(kind=E.OPT_ROWWISE_ADAGRAD, lr=0.01, eps=1e-8))
    dense = KeyedOptimizerWrapper(dmp.dense_named_parameters(), lambda p: torch.optim.SGD(p, lr=0.1))
    opt = CombinedOptimizer([dmp.fused_optimizer, dense])
    if pipelined:
        return HybridTrainPipelineSparseDist(dmp, opt, torch.device("cpu"), return_loss=True, pipe_n_batch=pipe_n_batch)
    return TrainPipelineBase(dmp, opt, torch.device("cpu"), return_loss=True)


def _batches():
    data = RandomRecDataset(["f%d" % i for i in range(T)], [1 << 40] * T, B, alpha=1.05, one_hot=False, min_len=1, max_len=4,
                            pos_rate=0.25, seed=3)
    return [data.make_batch() for _ in range(STEPS)]


@pytest.mark.parametrize("lines", [1, 2, 3])
def test_stage_order_lookahead_and_losses(lines):
    batches = _batches()
    ref_pipe = _setup(False)
    it = iter(batches)
    ref = [float(ref_pipe.progress(it)[0]) for _ in range(STEPS)]
    pipe = _setup(True, lines)
    pipe.trace_stages = True
    it = iter(batches)
    got = []
    while True:
        try:
            got.append(float(pipe.progress(it)[0]))
        except StopIteration:
            break
        if len(got) == 1:
            assert pipe.in_flight() == min(4 * lines, STEPS - 1)           # four stages ahead on every line
    assert len(got) == STEPS
    assert got == pytest.approx(ref, rel=1e-5, abs=1e-6)
    with pytest.raises(StopIteration):
        pipe.progress(it)
    names = [s.name for s in HybridStage]
    per_batch = {}
    for step, idx, stage in pipe.stage_log:
        per_batch.setdefault(idx, []).append((step, stage))
    for idx in range(STEPS):
        stages = [s for _, s in per_batch[idx]]
        assert stages == names, (idx, stages)
        steps = [st for st, _ in per_batch[idx]]
        assert steps == sorted(steps)
    # in steady state a batch enters one stage per visit of its line: `lines` training steps apart
    steady = per_batch[STEPS - 1]
    gaps = [b[0] - a[0] for a, b in zip(steady[:3], steady[1:4])]
    assert all(g == lines for g in gaps), gaps


def test_argument_checks():
    pipe = _setup(True)
    model, opt = pipe._model, pipe._optimizer
    for bad in (0, 13, 2.0, True):
        with pytest.raises(ValueError):
            HybridTrainPipelineSparseDist(model, opt, torch.device("cpu"), pipe_n_batch=bad)
    with pytest.raises(ValueError):
        HybridTrainPipelineSparseDist(model, opt, torch.device("cpu"), apply_jit=True)
    with pytest.raises(ValueError):
        HybridTrainPipelineSparseDist(model, opt, torch.device("cpu"), execute_all_batches=False)
    with pytest.raises(TypeError):
        HybridTrainPipelineSparseDist("model", opt, torch.device("cpu"))


def test_param_check_and_enque_context():
    import pytest
    import torch

    from recsdk_b200.parallel.hybrid import HybridPipelineContext, HybridTrainPipelineSparseDist

    model = torch.nn.Linear(2, 2)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    pipe = HybridTrainPipelineSparseDist(model, opt, torch.device("cpu"), pipe_n_batch=2)
    for bad, err in ((dict(pipe_n_batch=0), ValueError), (dict(pipe_n_batch=13), ValueError), (dict(pipe_n_batch=True), ValueError),
                     (dict(apply_jit=True), ValueError), (dict(execute_all_batches=False), ValueError)):
        kw = dict(pipe_n_batch=2, apply_jit=False, execute_all_batches=True)
        kw.update(bad)
        with pytest.raises(err):
            pipe.param_check(model, torch.device("cpu"), kw["pipe_n_batch"], kw["apply_jit"], kw["execute_all_batches"])
    with pytest.raises(TypeError):
        pipe.param_check("model", torch.device("cpu"), 2, False, True)
    with pytest.raises(TypeError):
        pipe.param_check(model, "cpu", 2, False, True)
    ctx = HybridPipelineContext.__new__(HybridPipelineContext)
    pipe.enque_context(3, ctx)                               # line 3 of a two-line pipeline is line 1
    assert len(pipe._lines[1]) == 1 and pipe._lines[1][0] is ctx and len(pipe._lines[0]) == 0
