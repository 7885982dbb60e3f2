"""Jagged containers: ``JaggedTensor`` / ``KeyedJaggedTensor`` / ``KeyedTensor`` and the variants that carry per-id side tensors
through the input pipeline (reference: ``hybrid_torchrec/sparse/__init__.py``, ``torchrec_embcache/sparse/__init__.py``)."""
from .jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor, KJTList, kjt_list_to_device
from .kjt_extensions import (ExtendedJaggedTensor, JaggedTensorWithCount, JaggedTensorWithTimestamp, KeyedExtendedJaggedTensor,
                             KeyedJaggedTensorWithCount, KeyedJaggedTensorWithLookHelper, KeyedJaggedTensorWithTimestamp)

__all__ = ["JaggedTensor", "KeyedJaggedTensor", "KeyedTensor", "KJTList", "kjt_list_to_device", "ExtendedJaggedTensor", "KeyedExtendedJaggedTensor", "JaggedTensorWithCount",
           "KeyedJaggedTensorWithCount", "JaggedTensorWithTimestamp", "KeyedJaggedTensorWithTimestamp", "KeyedJaggedTensorWithLookHelper"]
