"""recsdk_b200: recommendation-system training and inference on B200 (sm_100a).

Sub-packages: ``modules`` (table configs, unsharded collections), ``sparse`` (jagged containers), ``parallel`` (sharding, planner,
pipelines, peer memory), ``dynamic`` (hash-table embeddings), ``embcache`` (multi-tier tables), ``inference`` (paged KV cache),
``ops`` (kernels and ``torch.ops.mxrec``), ``optim``, ``models``, ``common``, ``utils``.  The names the reference's top-level
package exports (``hybrid_torchrec/__init__.py``) resolve here as well, on first use, so that importing the package stays cheap.
"""
__version__ = "0.2.0"

_LAZY = {"HashEmbeddingBagCollection": "modules.hash_embeddingbag", "HashEmbeddingBagConfig": "modules.hash_embeddingbag",
         "HybridHashTable": "modules.hash_embeddingbag"}

__all__ = ["HashEmbeddingBagCollection", "HashEmbeddingBagConfig", "HybridHashTable", "__version__"]


def __getattr__(name):
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError("module %r has no attribute %r" % (__name__, name))
    import importlib

    return getattr(importlib.import_module("%s.%s" % (__name__, mod)), name)
