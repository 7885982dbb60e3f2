"""The invoker layer (argument records -> lookup operators) gives what a direct operator call gives."""
import pytest
import torch

from recsdk_b200.ops.hybrid_lookup_invoke import (HybridCommonArgs, HybridCommonArgsAggregation, Momentum, OptimizerArgs, VBEMetadata,
                                                  check_unique_valid, lookup_adagrad, lookup_adam, lookup_args, lookup_sgd)
from tests.test_mxrec_tbe_ops import DIMS, ROWS, _common_args, _dense_reference, _problem, _state


def _records(p, pooling_mode, cls=HybridCommonArgs, **extra):
    e = torch.empty(0)
    return cls(placeholder_autograd_tensor=torch.zeros(1, requires_grad=True), dev_weights=p["dev_weights"], host_weights=e, uvm_weights=e,
               lxu_cache_weights=e, weights_placements=e.int(), weights_offsets=p["weights_offsets"], D_offsets=p["D_offsets"],
               total_D=int(p["D_offsets"][-1]), max_D=max(DIMS), hash_size_cumsum=p["hash_size_cumsum"], rows_per_table=p["rows_per_table"],
               total_hash_size_bits=8, indices=p["idx"], offsets=p["offsets"], hash_indices=None, unique_indices=None, unique_offset=None,
               unique_inverse=None, hash_indices2address=None, pooling_mode=pooling_mode, indice_weights=None, feature_requires_grad=None,
               lxu_cache_locations=e.int(), uvm_cache_stats=None, output_dtype=0, vbe_metadata=VBEMetadata(), is_experimental=False,
               use_uniq_cache_locations_bwd=False, use_homogeneous_placements=False, learning_rate=0.05, table_grad_accumulate_offsets=None,
               grad_accumulate=None, grad_accumulate_offsets=None, use_optimize=True, **extra)


def _momentum(state_args):
    dev, uvm, placements, offsets = state_args
    return Momentum(dev=dev, host=torch.empty(0), uvm=uvm, offsets=offsets, placements=placements)


@pytest.mark.parametrize("kind", ["adagrad", "adam", "sgd"])
def test_invoke_matches_direct_call(kind):
    res = []
    for via_invoker in (True, False):
        p = _problem(torch.device("cpu"), seed=5)
        m1_buf, m1, _ = _state(p)
        m2_buf, m2, _ = _state(p)
        o = OptimizerArgs(learning_rate=123.0, eps=1e-6, beta1=0.9, beta2=0.99, weight_decay=0.01)
        if via_invoker:
            a = _records(p, 0)
            if kind == "adagrad":
                out = lookup_adagrad.invoke(a, o, _momentum(m1))
            elif kind == "adam":
                out = lookup_adam.invoke(a, o, _momentum(m1), _momentum(m2), iteration=3)
            else:
                out = lookup_sgd.invoke(a, o)
        else:
            args = _common_args(p, 0)
            kw = dict(learning_rate=0.05, rows_per_table=p["rows_per_table"])
            if kind == "adagrad":
                out = torch.ops.mxrec.split_embedding_codegen_lookup_adagrad_function(*args, *m1, eps=1e-6, **kw)
            elif kind == "adam":
                out = torch.ops.mxrec.split_embedding_codegen_lookup_adam_function(*args, *m1, *m2, eps=1e-6, beta1=0.9, beta2=0.99,
                                                                                   weight_decay=0.01, iter=3, **kw)
            else:
                out = torch.ops.mxrec.split_embedding_codegen_lookup_sgd_function(*args, **kw)
        out.backward(p["grad"])
        res.append((out.detach().clone(), p["dev_weights"].clone(), m1_buf.clone()))
    for x, y in zip(*res):
        torch.testing.assert_close(x, y)                    # the record's learning_rate (0.05) wins over OptimizerArgs'


def test_hash_indices_replace_the_ids_and_are_checked():
    p = _problem(torch.device("cpu"), seed=2)
    ref_out, _g, _t = _dense_reference(p, 0)
    a = _records(p, 0)
    a.indices = torch.zeros_like(p["idx"])                 # raw ids are ignored once hash_indices is given
    a.hash_indices = p["idx"]
    B = p["B"]
    off = p["offsets"]
    uniq, inv, uoff = [], [], [0]
    for f in range(len(p["feat_table"])):
        seg = p["idx"][int(off[f * B]):int(off[(f + 1) * B])]
        u, i = torch.unique(seg, return_inverse=True)
        uniq.append(u); inv.append(i); uoff.append(uoff[-1] + u.numel())
    a.unique_indices, a.unique_inverse, a.unique_offset = torch.cat(uniq), torch.cat(inv), torch.tensor(uoff)
    check_unique_valid(a)
    lookup_adagrad.check_unique_valid(a)
    out = lookup_sgd.invoke(a, OptimizerArgs())
    torch.testing.assert_close(out.detach(), ref_out, rtol=1e-5, atol=1e-5)
    a.unique_inverse = torch.zeros_like(a.unique_inverse)
    with pytest.raises(RuntimeError, match="do not reproduce"):
        check_unique_valid(a)
    a.host_weights = torch.ones(3)
    with pytest.raises(NotImplementedError, match="host_weights"):
        lookup_sgd.invoke(a, OptimizerArgs())
    assert lookup_args.HybridCommonArgs is HybridCommonArgs


def test_grad_aggregation_through_the_invoker():
    p = _problem(torch.device("cpu"), seed=11)
    _, dense_grads, tabs = _dense_reference(p, 0)
    acc = [torch.zeros(r * d) for r, d in zip(ROWS, DIMS)]
    a = _records(p, 0, cls=HybridCommonArgsAggregation, indices_multi_step=p["idx"], offsets_multi_step=p["offsets"])
    a.grad_accumulate, a.grad_accumulate_offsets, a.learning_rate = acc, torch.zeros(len(ROWS), dtype=torch.long), 0.1
    a.use_optimize = False
    lookup_sgd.invoke_grad_aggregation(a, OptimizerArgs()).backward(p["grad"])
    a.use_optimize, a.placeholder_autograd_tensor = True, torch.zeros(1, requires_grad=True)
    lookup_sgd.invoke_grad_aggregation(a, OptimizerArgs()).backward(p["grad"])
    for t, (s, r, d) in enumerate(zip(p["starts"], ROWS, DIMS)):
        torch.testing.assert_close(p["dev_weights"][s: s + r * d].view(r, d), tabs[t].detach() - 0.2 * dense_grads[t], rtol=1e-5, atol=1e-6)
