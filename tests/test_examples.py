"""The quick-start examples run end to end (CPU, one process, small settings)."""
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location("example_" + name, os.path.join(ROOT, "examples", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_quick_start_hybrid():
    last = _load("quick_start_hybrid").main(["--steps", "8", "--tables", "2", "--local-batch", "32"])
    assert last == last and last < 2.0


def test_dynamic_embedding(monkeypatch):
    import torch

    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    assert _load("dynamic_embedding").main() >= 0.0


def test_embcache_multi_tier(monkeypatch):
    import torch

    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    assert _load("embcache_multi_tier").main() >= 0.0


def test_kvcache_lifecycle(monkeypatch):
    import torch

    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    assert _load("kvcache_lifecycle").main() == 440 - 256
