"""Inference-side components: the paged KV-cache manager (device pages + pinned host chunk tier)."""
from .kvcache_manager import (GPUKVCacheManager, HostKVStorageErrorCode, HostKVStorageManagerBase, HostKVTaskHandle,
                              HostKVTaskStatus, HostKVWaitResult, KVCacheConfig, KVCacheManager, KVCacheMetadata,
                              KVCacheOffloadMode, KVIndexMeta, KVLookupResult, NativeHostKVCacheManager, NPUKVCacheManager,
                              HostKVStorageBackend, HostKVStorageFailPolicy, copy_kvcache_metadata, get_kvcache_config,
                              get_kvcache_metadata_buffer)

__all__ = ["GPUKVCacheManager", "HostKVStorageErrorCode", "HostKVStorageManagerBase", "HostKVTaskHandle", "HostKVTaskStatus",
           "HostKVWaitResult", "KVCacheConfig", "KVCacheManager", "KVCacheMetadata", "KVCacheOffloadMode", "KVIndexMeta",
           "KVLookupResult", "NativeHostKVCacheManager", "NPUKVCacheManager", "get_kvcache_config", "HostKVStorageBackend", "HostKVStorageFailPolicy",
           "copy_kvcache_metadata", "get_kvcache_metadata_buffer"]
