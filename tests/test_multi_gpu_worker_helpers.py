"""The acceptance rule of the multi-GPU worker (``tests/multi_gpu_worker.py``), checked on CPU: exact and near-exact tables
pass, a handful of outlier rows within the hard bound pass, widespread or large differences fail."""
import importlib.util
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("multi_gpu_worker", os.path.join(HERE, "multi_gpu_worker.py"))
worker = importlib.util.module_from_spec(spec)
spec.loader.exec_module(worker)


def test_exact_and_rounding_level_differences_pass():
    a = torch.randn(300, 64)
    ok, mx, bad = worker.close_up_to_outliers(a, a.clone())
    assert ok and mx == 0.0 and bad == 0
    ok, mx, bad = worker.close_up_to_outliers(a, a + 1e-6)
    assert ok and bad == 0 and mx < 1e-5


def test_few_bounded_outlier_rows_pass():
    a = torch.randn(5000, 64)
    b = a.clone()
    b[[3, 77, 4001], 5] += 9e-3                    # three rows touched by one sample whose ReLU mask flipped
    ok, mx, bad = worker.close_up_to_outliers(b, a)
    assert ok and bad == 3 and abs(mx - 9e-3) < 1e-6
    small = torch.randn(64, 64)
    t = small.clone()
    t[[1, 2]] += 5e-3                              # tiny table: two rows are always allowed
    assert worker.close_up_to_outliers(t, small)[0]


def test_widespread_or_large_differences_fail():
    a = torch.randn(5000, 64)
    b = a.clone()
    b[::4] += 5e-3                                 # a quarter of the rows: one of four ranks' gradients missing
    ok, _mx, bad = worker.close_up_to_outliers(b, a)
    assert not ok and bad == 1250
    c = a.clone()
    c[10, 0] += 0.5                                # one row, but far beyond any single update
    assert not worker.close_up_to_outliers(c, a)[0]
    small = torch.randn(64, 64)
    t = small.clone()
    t[[1, 2, 3]] += 5e-3                           # three of 64 rows: beyond the allowance
    assert not worker.close_up_to_outliers(t, small)[0]


def test_dense_vector_rule():
    w = torch.randn(60000)
    v = w.clone()
    v[:40] += 3e-3                                 # 40 of 60000 elements (< 0.1 %), within 1e-2
    assert worker.close_up_to_outliers(v, w, hard_max=1e-2, frac=1e-3)[0]
    v[:100] += 3e-3                                # 100 elements: beyond 0.1 %
    assert not worker.close_up_to_outliers(v, w, hard_max=1e-2, frac=1e-3)[0]
    assert worker.close_up_to_outliers(torch.empty(0), torch.empty(0))[0]
