"""The public names and argument orders a user of the reference's ``torch_rec`` stack relies on.  Every entry is
``(dotted path, leading parameters in the reference's order)``; this package may append parameters of its own but must not
rename, drop or reorder the reference's.  Sources: ``hybrid_torchrec`` (``modules/hash_embeddingbag.py:67-362``,
``distributed/sharding_plan.py:18-28``, ``distributed/hybrid_train_pipeline.py:216-335``), ``torchrec_embcache``
(``distributed/configs.py:33-236``, ``distributed/embedding_bag.py:229-258``, ``distributed/sharding/embedding_sharder.py:70-195``,
``distributed/train_pipeline.py:226-293``, ``saver.py:31-171``), ``dynamic_emb`` (``distributed/dynamicemb_config.py:150-453``,
``distributed/planner/planners.py:80-222``, ``distributed/dump_load.py:92-272``, ``distributed/incremental_dump.py:103-404``),
``kvcache_manager`` (``kvcache_config.py:39-105``, ``kvcache_manager.py:47-346``, ``kvcache_metadata.py:35-64``,
``host_kvstorage_manager.py:38-148``) and the TorchRec patch (``torchrec1.2.0_npu.patch:823-924``)."""
import dataclasses
import importlib
import inspect

import pytest
import torch

SIGNATURES = [
    ("recsdk_b200.modules.hash_embeddingbag.HashTableOption",
     ["init_capacity", "max_capacity", "max_npu_memory_for_vectors", "max_bucket_size", "dim", "max_load_factor", "block_size",
      "io_block_size", "device_id", "io_by_cpu"]),
    ("recsdk_b200.modules.hash_embeddingbag.HashEmbeddingBagCollection", ["tables", "is_weighted", "device"]),
    ("recsdk_b200.parallel.get_default_hybrid_sharders", ["host_env"]),
    ("recsdk_b200.parallel.HybridEmbeddingBagCollectionSharder", ["host_env"]),
    ("recsdk_b200.parallel.HybridHashEmbeddingBagCollectionSharder", ["host_env"]),
    ("recsdk_b200.parallel.HybridTrainPipelineSparseDist",
     ["model", "optimizer", "device", "execute_all_batches", "apply_jit", "return_loss", "pipe_n_batch"]),
    ("recsdk_b200.parallel.TrainPipelineSparseDist", ["model", "optimizer", "device", "execute_all_batches", "apply_jit"]),
    ("recsdk_b200.parallel.EmbeddingShardingPlanner", ["topology", "constraints", "batch_size"]),
    ("recsdk_b200.parallel.Topology", ["world_size", "compute_device", "hbm_cap", "ddr_cap", "local_world_size"]),
    ("recsdk_b200.parallel.ParameterConstraints", ["sharding_types", "compute_kernels", "min_partition", "pooling_factors"]),
    ("recsdk_b200.parallel.DistributedModelParallel", ["module", "env", "device", "plan", "sharders"]),
    ("recsdk_b200.optim.apply_optimizer_in_backward", ["optimizer_class", "params", "optimizer_kwargs"]),
    ("recsdk_b200.optim.KeyedOptimizerWrapper", ["params", "optim_factory"]),
    ("recsdk_b200.optim.CombinedOptimizer", ["optims"]),
    ("recsdk_b200.optim.AccumulateAdagrad", ["params", "use_accumulate", "accumulate_step"]),
    ("recsdk_b200.optim.AccumulateSGD", ["params", "use_accumulate", "accumulate_step"]),
    ("recsdk_b200.optim.AccumulateAdam", ["params", "use_accumulate", "accumulate_step"]),
    ("recsdk_b200.embcache.AdmitAndEvictConfig",
     ["admit_threshold", "not_admitted_default_value", "evict_threshold", "evict_step_interval", "policy_type", "show_click_params"]),
    ("recsdk_b200.embcache.ShowClickParams", ["alpha", "beta", "admit_threshold", "evict_percentage", "score_decay"]),
    ("recsdk_b200.embcache.EmbCacheEmbeddingBagCollection",
     ["tables", "world_size", "batch_size", "multi_hot_sizes", "is_weighted", "need_accumulate_offset", "device", "embedding_optimizer_cls"]),
    ("recsdk_b200.embcache.EmbCacheEmbeddingCollection", ["tables", "world_size", "batch_size", "multi_hot_sizes"]),
    ("recsdk_b200.embcache.EmbCacheEmbeddingBagCollectionSharder",
     ["cpu_device", "cpu_env", "npu_device", "npu_env", "fused_params", "qcomm_codecs_registry"]),
    ("recsdk_b200.embcache.EmbCacheEmbeddingCollectionSharder",
     ["cpu_device", "cpu_env", "npu_device", "npu_env", "fused_params", "qcomm_codecs_registry"]),
    ("recsdk_b200.embcache.EmbCacheTrainPipelineSparseDist",
     ["model", "optimizer", "cpu_device", "npu_device", "return_loss", "evict_step_interval", "execute_all_batches", "apply_jit",
      "context_type", "pipeline_postproc", "custom_model_fwd", "custom_model_zero_grad", "custom_model_bwd"]),
    ("recsdk_b200.embcache.Saver.save", ["module", "path", "incremental"]),
    ("recsdk_b200.embcache.Saver.load", ["module", "path", "incremental"]),
    ("recsdk_b200.embcache.Saver.get_latest_load_path", ["path"]),
    ("recsdk_b200.dynamic.DynamicEmbTableOptions",
     ["training", "initializer_args", "eval_initializer_args", "init_capacity", "max_load_factor", "score_strategy", "bucket_capacity",
      "safe_check_mode", "global_hbm_for_values", "caching", "external_storage", "index_type"]),
    ("recsdk_b200.dynamic.DynamicEmbInitializerArgs", ["mode", "mean", "std_dev", "lower", "upper", "value"]),
    ("recsdk_b200.dynamic.DynamicEmbeddingShardingPlanner",
     ["eb_configs", "constraints", "topology", "batch_size", "enumerator", "storage_reservation", "proposer", "partitioner",
      "performance_model", "stats", "debug"]),
    ("recsdk_b200.dynamic.DynamicEmbeddingShardingPlanner.collective_plan", ["module", "sharders", "pg"]),
    ("recsdk_b200.dynamic.DynamicEmbeddingShardingPlanner.plan", ["module", "sharders"]),
    ("recsdk_b200.dynamic.DynamicEmbeddingCollectionSharder", ["fused_params", "qcomm_codecs_registry", "use_index_dedup"]),
    ("recsdk_b200.dynamic.DynamicEmbeddingBagCollectionSharder", ["fused_params", "qcomm_codecs_registry"]),
    ("recsdk_b200.dynamic.DynamicEmbDump", ["path", "model", "table_names", "optim", "pg", "allow_overwrite"]),
    ("recsdk_b200.dynamic.DynamicEmbLoad", ["path", "model", "table_names", "optim", "pg"]),
    ("recsdk_b200.dynamic.set_score", ["model", "table_score"]),
    ("recsdk_b200.dynamic.get_score", ["model"]),
    ("recsdk_b200.dynamic.incremental_dump", ["model", "score_threshold", "pg"]),
    ("recsdk_b200.inference.KVCacheConfig",
     ["num_layers", "num_heads", "head_dim", "page_size", "offload_chunksize", "num_primary_cache_pages", "num_buffer_pages",
      "host_capacity_per_layer", "max_batch_size", "max_seq_len", "dtype", "device", "host_kvstorage_backend", "onload_timeout_ms",
      "offload_timeout_ms", "offload_mode", "host_kvstorage_fail_policy", "extra_configs"]),
    ("recsdk_b200.inference.get_kvcache_config",
     ["num_layers", "num_heads", "head_dim", "page_size", "offload_chunksize", "num_primary_cache_pages", "num_buffer_pages",
      "host_capacity_per_layer", "max_batch_size", "max_seq_len", "dtype", "device"]),
    ("recsdk_b200.inference.KVCacheManager",
     ["npu_kvcache_manager", "host_kvstorage_manager", "offload_mode", "host_kvstorage_fail_policy"]),
    ("recsdk_b200.inference.KVCacheManager.lookup_kvcache", ["user_ids", "sequence_lengths"]),
    ("recsdk_b200.inference.KVCacheManager.allocate_kvcache", ["index_meta", "lookup_results", "output_kvcache_metadata"]),
    ("recsdk_b200.inference.KVCacheManager.onboard_launch", ["index_meta", "lookup_result", "kvcache_metadata"]),
    ("recsdk_b200.inference.KVCacheManager.offload_launch", ["index_meta", "kvcache_metadata"]),
    ("recsdk_b200.inference.KVCacheManager.evict", ["user_ids", "for_npu", "for_host"]),
    ("recsdk_b200.inference.KVCacheManager.evict_all", ["for_npu", "for_host"]),
    ("recsdk_b200.inference.HostKVTaskHandle.stream_wait_layer", ["layer_idx"]),
]

DATACLASS_FIELDS = [
    ("recsdk_b200.inference.KVCacheMetadata",
     ["page_ids_npu_buffer", "metadata_npu_buffer", "kv_indices", "kv_indptr", "kv_last_page_len", "total_history_lengths",
      "total_history_offsets", "new_history_offsets", "batch_indices", "position", "new_history_nnz", "new_history_nnz_npu", "kv_seqlens",
      "kv_seqlen_offsets", "kv_cache_table", "kv_onload_handle", "max_seqlen", "onboard_slot_mappings", "onboard_task_ids"]),
    ("recsdk_b200.inference.KVLookupResult",
     ["user_ids", "cached_start_indices", "cached_lengths", "npu_cached_start_indices", "npu_cached_lengths", "host_cached_start_indices",
      "host_cached_lengths", "token_ids", "token_mask", "extra"]),
    ("recsdk_b200.dynamic.DynamicEmbTableOptions",
     ["score_type", "embedding_dtype", "dim", "max_capacity", "evict_strategy", "local_hbm_for_values", "num_aligned_embedding_per_rank",
      "device_id", "optimizer_type", "block_size", "io_block_size", "io_by_cpu", "use_constant_memory", "reserved_key_start_bit",
      "num_of_buckets_per_alloc"]),
    ("recsdk_b200.embcache.EmbCacheEmbeddingBagConfig",
     ["weight_init_mean", "weight_init_stddev", "initializer_type", "admit_and_evict_config", "is_incremental"]),
    ("recsdk_b200.embcache.EmbCacheEmbeddingConfig",
     ["weight_init_mean", "weight_init_stddev", "initializer_type", "admit_and_evict_config", "is_incremental"]),
    ("recsdk_b200.dynamic.DynamicEmbParameterConstraints", ["use_dynamicemb", "dynamicemb_options"]),
]

ENUM_MEMBERS = [
    ("recsdk_b200.modules.hash_embeddingbag.EvictStrategy", ["kLru", "kLfu", "kEpochLru", "kEpochLfu", "kCustomized"]),
    ("recsdk_b200.inference.HostKVTaskStatus",
     ["UNINITIALIZED", "SKIPPED", "LAUNCHED", "READY", "EVENT_READY", "TIMEOUT", "FAILED", "CANCELLED"]),
    ("recsdk_b200.inference.HostKVStorageErrorCode",
     ["LOOKUP_FAILED", "LOOKUP_MISSING_TOKENS", "ONBOARD_TASK_NOT_FOUND", "ONBOARD_WAIT_FAILED", "ONBOARD_TIMEOUT",
      "OFFLOAD_TASK_NOT_FOUND", "OFFLOAD_WAIT_FAILED", "OFFLOAD_TIMEOUT", "OFFLOAD_NO_SPACE", "CANCEL_FAILED"]),
    ("recsdk_b200.embcache.InitializerType", ["LINEAR", "TRUNCATED_NORMAL", "UNIFORM"]),
    ("recsdk_b200.dynamic.DynamicEmbInitializerMode", ["NORMAL", "TRUNCATED_NORMAL", "UNIFORM", "CONSTANT", "DEBUG"]),
    ("recsdk_b200.dynamic.DynamicEmbScoreStrategy", ["TIMESTAMP", "STEP", "CUSTOMIZED", "LFU"]),
]

HOST_BACKEND_METHODS = ["register_npu_cache_tables", "build_index_meta", "lookup_kvcache", "onboard_kvcache_launch", "onboard_kvcache_wait",
                        "offload_kvcache_launch", "offload_kvcache_wait", "finish_task", "cancel_task", "evict", "evict_all"]

MXREC_OPS = ["hstu_dense", "hstu_dense_backward", "hstu_jagged", "hstu_jagged_backward", "hstu_paged", "hstu_forward_v2", "hstu_backward_v2",
             "hstu_fuxi", "hstu_dense_backward_fuxi", "in_linear_silu", "distance_in_linear_silu", "in_linear_silu_backward", "relative_attn_bias_pos",
             "relative_attn_bias_time", "relative_attn_bias_time_with_index", "relative_attn_bias_time_backward", "ln_mul",
             "norm_multiply_dropout", "token_mixing", "concat_2d_jagged", "split_2d_jagged", "multislice_concat", "gather_for_rank1",
             "index_select_for_rank1_backward", "reverse_sequence", "disentangle_attention",
             "split_embedding_codegen_forward_unweighted_cuda", "split_embedding_codegen_lookup_adagrad_function",
             "split_embedding_codegen_lookup_adam_function", "split_embedding_codegen_lookup_sgd_function",
             "split_embedding_codegen_lookup_rowwise_adagrad_function"]
MXREC_OPS += ["split_embedding_codegen_lookup_%s_function_grad_aggregation" % k for k in ("adagrad", "adam", "sgd")]
MXREC_OPS += ["split_embedding_backward_codegen_%s_unweighted_exact_cuda" % k for k in ("adagrad", "adam", "sgd", "rowwise_adagrad")]
MXREC_OPS += ["split_embedding_backward_codegen_%s_unweighted_exact_cuda_grad_aggregation" % k for k in ("adagrad", "adam", "sgd")]


def _resolve(path):
    parts = path.split(".")
    for cut in range(len(parts), 0, -1):
        try:
            obj = importlib.import_module(".".join(parts[:cut]))
        except ImportError:
            continue
        for name in parts[cut:]:
            obj = getattr(obj, name)
        return obj
    raise ImportError(path)


@pytest.mark.parametrize("path, leading", SIGNATURES, ids=[p for p, _ in SIGNATURES])
def test_leading_parameters_follow_the_reference(path, leading):
    params = [p for p in inspect.signature(_resolve(path)).parameters if p not in ("self", "cls")]
    assert params[: len(leading)] == leading, "%s%s" % (path, params)


@pytest.mark.parametrize("path, fields", DATACLASS_FIELDS, ids=[p for p, _ in DATACLASS_FIELDS])
def test_record_fields(path, fields):
    have = [f.name for f in dataclasses.fields(_resolve(path))]
    assert [f for f in fields if f not in have] == []
    ordered = [f for f in have if f in fields]
    assert ordered == fields                                               # same relative order as in the reference


@pytest.mark.parametrize("path, members", ENUM_MEMBERS, ids=[p for p, _ in ENUM_MEMBERS])
def test_enum_members(path, members):
    assert [m for m in members if m not in _resolve(path).__members__] == []


def test_host_backend_contract_and_defaults():
    base = _resolve("recsdk_b200.inference.HostKVStorageManagerBase")
    assert sorted(base.__abstractmethods__) == sorted(HOST_BACKEND_METHODS)
    opts = _resolve("recsdk_b200.dynamic.DynamicEmbTableOptions")()
    assert (opts.training, opts.max_load_factor, opts.bucket_capacity, opts.caching, opts.index_type) == (True, 0.5, 128, False, torch.int64)
    assert opts.score_strategy.name == "TIMESTAMP" and opts.eval_initializer_args.mode.name == "CONSTANT" and opts.block_size == 128
    cfg = _resolve("recsdk_b200.inference.KVCacheConfig")
    d = {f.name: f.default for f in dataclasses.fields(cfg) if f.default is not dataclasses.MISSING}
    assert d == {"host_kvstorage_backend": "native_host", "onload_timeout_ms": 0.0, "offload_timeout_ms": 1000.0, "offload_mode": "lazy",
                 "host_kvstorage_fail_policy": "fail_open"}
    aec = _resolve("recsdk_b200.embcache.AdmitAndEvictConfig")()
    assert (aec.admit_threshold, aec.not_admitted_default_value, aec.evict_threshold, aec.evict_step_interval, aec.policy_type) == \
        (-1, 0.0, -1, -1, "count")
    ht = _resolve("recsdk_b200.modules.hash_embeddingbag.HashTableOption")()
    assert (ht.dim, ht.max_load_factor, ht.block_size, ht.io_block_size, ht.device_id, ht.io_by_cpu) == (64, 0.5, 128, 1024, -1, False)
    sharders = _resolve("recsdk_b200.parallel.get_default_hybrid_sharders")(_resolve("recsdk_b200.parallel.ShardingEnv")(1, 0))
    assert [type(s).__name__ for s in sharders] == ["HybridEmbeddingBagCollectionSharder", "HybridHashEmbeddingBagCollectionSharder"]
    pipe = inspect.signature(_resolve("recsdk_b200.parallel.HybridTrainPipelineSparseDist")).parameters
    assert pipe["pipe_n_batch"].default == 6 and pipe["execute_all_batches"].default is True and pipe["return_loss"].default is False
    assert issubclass(_resolve("recsdk_b200.modules.hash_embeddingbag.HashEmbeddingBagConfig"),
                      _resolve("recsdk_b200.modules.embedding_configs.EmbeddingBagConfig"))
    with pytest.raises(ValueError):                                        # only SGD / Adam / Adagrad may run inside the backward
        _resolve("recsdk_b200.optim.apply_optimizer_in_backward")(torch.optim.RMSprop, [], {})


def test_operator_names_are_registered():
    import recsdk_b200.ops.mxrec  # noqa: F401  (registers torch.ops.mxrec.*)
    import recsdk_b200.ops.mxrec_tbe  # noqa: F401

    missing = [n for n in MXREC_OPS if not hasattr(torch.ops.mxrec, n)]
    assert missing == []
    assert hasattr(torch.ops.mxrec.hstu_jagged, "equal") and hasattr(torch.ops.mxrec.hstu_jagged, "delta")
    assert hasattr(torch.ops.mxrec.hstu_jagged_backward, "equal") and hasattr(torch.ops.mxrec.hstu_jagged_backward, "delta")


# Operator -> (argument names in the reference's order, return type), taken from the ``m.def`` strings under
# ``cust_op/framework/torch_plugin/torch_library/`` of the reference.
OPERATOR_ARGUMENTS = {
    'concat_2d_jagged': ('maxSeqlen valuesA valuesB offsetA offsetB isReplace nPrefixFromRight', 'Tensor'),
    'disentangle_attention': (
        'query_layer key_layer value_layer pos_key_layer pos_query_layer relative_pos attn_mask pos_attr_type '
        'score_scale',
        '(Tensor,Tensor,Tensor'),
    'distance_in_linear_silu': ('x weight bias attr_dict', 'Tensor[]'),
    'gather_for_rank1': ('x index', 'Tensor'),
    'hstu_backward_v2': (
        'grad q k v max_seqlen_q max_seqlen_k seq_offset_q seq_offset_k rab num_context num_target scale '
        'target_group_size alpha window_size_left window_size_right',
        '(Tensor,Tensor,Tensor,Tensor'),
    'hstu_dense': ('q k v mask attn_bias mask_type max_seq_len silu_scale', 'Tensor'),
    'hstu_dense_backward': ('grad q k v mask attn_bias mask_type max_seq_len silu_scale', '(Tensor,Tensor,Tensor,Tensor)'),
    'hstu_dense_backward_fuxi': (
        'grad q k v mask biasPosition biasTimestamp layout maskType maxSeqLen siluScale seqOffset',
        '(Tensor,Tensor,Tensor,Tensor,Tensor'),
    'hstu_forward_v2': (
        'q k v mask rab mask_type max_seq_len max_seq_len_k silu_scale seq_offset seq_offset_k num_context '
        'num_target target_group_size alpha',
        'Tensor'),
    'hstu_fuxi': ('q k v timestampBias positionBias mask maskType maxSeqLen siluScale layout seqOffset', 'Tensor'),
    'hstu_jagged.delta': (
        'q k v mask attn_bias mask_type max_seq_len max_seq_len_k silu_scale seq_offset seq_offset_k '
        'num_context num_target target_group_size alpha deterministic',
        'Tensor'),
    'hstu_jagged.equal': (
        'q k v mask attn_bias mask_type max_seq_len silu_scale seq_offset num_context num_target '
        'target_group_size alpha deterministic',
        'Tensor'),
    'hstu_jagged_backward.delta': (
        'grad q k v mask attn_bias mask_type max_seq_len max_seq_len_k silu_scale seq_offset seq_offset_k '
        'num_context num_target target_group_size alpha',
        '(Tensor,Tensor,Tensor,Tensor'),
    'hstu_jagged_backward.equal': (
        'grad q k v mask attn_bias mask_type max_seq_len silu_scale seq_offset num_context num_target '
        'target_group_size alpha',
        '(Tensor,Tensor,Tensor,Tensor'),
    'hstu_paged': (
        'q k v kv_cache mask attn_bias mask_type max_seq_len max_seq_len_k silu_scale seq_offset seq_offset_k '
        'seq_offset_t page_offsets page_ids last_page_len num_target target_group_size alpha deterministic',
        'Tensor'),
    'in_linear_silu': ('x weight bias attr_dict', 'Tensor[]'),
    'in_linear_silu_backward': ('x weight bias user_grad value_grad query_grad key_grad linear_output attr_dict', 'Tensor[]'),
    'index_select_for_rank1_backward': ('grad x index', 'Tensor[]'),
    'ln_mul': ('x u gamma beta', 'Tensor'),
    'multislice_concat': ('input concat_num concat_size slice_begin slice_length', '(Tensor[])'),
    'norm_multiply_dropout': ('x u weight bias eps dropout_ratio', 'Tensor[]'),
    'relative_attn_bias_pos': ('rel_pos_bias identity past_valid_lens', 'Tensor'),
    'relative_attn_bias_time': ('timestamps timestamps_weights bucket_divisor', 'Tensor'),
    'relative_attn_bias_time_backward': ('rab_time_grad bucket_timestamps num_buckets', 'Tensor'),
    'relative_attn_bias_time_with_index': ('timestamps timestamps_weights bucket_divisor', 'Tensor[]'),
    'reverse_sequence': ('input seq_lengths', '(Tensor)'),
    'split_2d_jagged': ('values maxSeqlen offsetA offsetB dense_size nPrefixToRight', '(Tensor,Tensor)'),
    'split_embedding_backward_codegen_adagrad_unweighted_exact_cuda': (
        'grad_output dev_weights uvm_weights lxu_cache_weights weights_placements weights_offsets D_offsets '
        'max_D hash_size_cumsum total_hash_size_bits indices offsets pooling_mode lxu_cache_locations unused_ '
        'max_segment_length_per_warp stochastic_rounding info_B_num_bits info_B_mask_int64 '
        'use_uniq_cache_locations use_homogeneous_placements momentum1_dev momentum1_uvm momentum1_placements '
        'momentum1_offsets grad_accumulate grad_accumulate_offsets hash_indices unique_ids unique_offsets '
        'unique_inverse offset_per_key table_grad_accumulate_offsets eps learning_rate use_optimize',
        'Tensor'),
    'split_embedding_backward_codegen_adagrad_unweighted_exact_cuda_grad_aggregation': (
        'grad_output dev_weights uvm_weights lxu_cache_weights weights_placements weights_offsets D_offsets '
        'max_D hash_size_cumsum total_hash_size_bits indices offsets indices_multi_step offsets_multi_step '
        'pooling_mode lxu_cache_locations unused_ max_segment_length_per_warp stochastic_rounding '
        'info_B_num_bits info_B_mask_int64 use_uniq_cache_locations use_homogeneous_placements momentum1_dev '
        'momentum1_uvm momentum1_placements momentum1_offsets grad_accumulate grad_accumulate_offsets '
        'hash_indices unique_ids unique_offsets unique_inverse offset_per_key table_grad_accumulate_offsets '
        'table_offsets_multi unique_multi_step unique_offset_multi_step unique_inverse_multi_step eps '
        'learning_rate use_optimize',
        'Tensor'),
    'split_embedding_backward_codegen_adam_unweighted_exact_cuda': (
        'grad_output dev_weights uvm_weights lxu_cache_weights weights_placements weights_offsets D_offsets '
        'max_D hash_size_cumsum total_hash_size_bits indices offsets pooling_mode lxu_cache_locations unused_ '
        'max_segment_length_per_warp stochastic_rounding info_B_num_bits info_B_mask_int64 '
        'use_uniq_cache_locations use_homogeneous_placements momentum1_dev momentum1_uvm momentum1_placements '
        'momentum1_offsets momentum2_dev momentum2_uvm momentum2_placements momentum2_offsets grad_accumulate '
        'grad_accumulate_offsets hash_indices unique_ids unique_offsets unique_inverse offset_per_key '
        'table_grad_accumulate_offsets eps learning_rate beta1 beta2 iter use_optimize',
        'Tensor'),
    'split_embedding_backward_codegen_adam_unweighted_exact_cuda_grad_aggregation': (
        'grad_output dev_weights uvm_weights lxu_cache_weights weights_placements weights_offsets D_offsets '
        'max_D hash_size_cumsum total_hash_size_bits indices offsets indices_multi_step offsets_multi_step '
        'pooling_mode lxu_cache_locations unused_ max_segment_length_per_warp stochastic_rounding '
        'info_B_num_bits info_B_mask_int64 use_uniq_cache_locations use_homogeneous_placements momentum1_dev '
        'momentum1_uvm momentum1_placements momentum1_offsets momentum2_dev momentum2_uvm '
        'momentum2_placements momentum2_offsets grad_accumulate grad_accumulate_offsets hash_indices '
        'unique_ids unique_offsets unique_inverse offset_per_key table_grad_accumulate_offsets '
        'table_offsets_multi unique_multi_step unique_offset_multi_step unique_inverse_multi_step eps '
        'learning_rate beta1 beta2 iter use_optimize',
        'Tensor'),
    'split_embedding_backward_codegen_rowwise_adagrad_unweighted_exact_cuda': (
        'grad_output dev_weights uvm_weights lxu_cache_weights weights_placements weights_offsets D_offsets '
        'max_D hash_size_cumsum total_hash_size_bits indices offsets pooling_mode lxu_cache_locations unused_ '
        'max_segment_length_per_warp stochastic_rounding info_B_num_bits info_B_mask_int64 '
        'use_uniq_cache_locations use_homogeneous_placements momentum1_dev momentum1_uvm momentum1_placements '
        'momentum1_offsets grad_accumulate grad_accumulate_offsets hash_indices unique_ids unique_offsets '
        'unique_inverse offset_per_key table_grad_accumulate_offsets eps learning_rate use_optimize',
        'Tensor'),
    'split_embedding_backward_codegen_sgd_unweighted_exact_cuda': (
        'grad_output dev_weights uvm_weights lxu_cache_weights weights_placements weights_offsets D_offsets '
        'max_D hash_size_cumsum total_hash_size_bits indices offsets pooling_mode lxu_cache_locations unused_ '
        'max_segment_length_per_warp stochastic_rounding info_B_num_bits info_B_mask_int64 '
        'use_uniq_cache_locations use_homogeneous_placements grad_accumulate grad_accumulate_offsets '
        'hash_indices unique_ids unique_offsets unique_inverse offset_per_key table_grad_accumulate_offsets '
        'learning_rate use_optimize',
        'Tensor'),
    'split_embedding_backward_codegen_sgd_unweighted_exact_cuda_grad_aggregation': (
        'grad_output dev_weights uvm_weights lxu_cache_weights weights_placements weights_offsets D_offsets '
        'max_D hash_size_cumsum total_hash_size_bits indices offsets indices_multi_step offsets_multi_step '
        'pooling_mode lxu_cache_locations unused_ max_segment_length_per_warp stochastic_rounding '
        'info_B_num_bits info_B_mask_int64 use_uniq_cache_locations use_homogeneous_placements '
        'grad_accumulate grad_accumulate_offsets hash_indices unique_ids unique_offsets unique_inverse '
        'offset_per_key table_grad_accumulate_offsets table_offsets_multi unique_multi_step '
        'unique_offset_multi_step unique_inverse_multi_step learning_rate use_optimize',
        'Tensor'),
    'split_embedding_codegen_forward_unweighted_cuda': (
        'dev_weights uvm_weights lxu_cache_weights weights_placements weights_offsets D_offsets total_D max_D '
        'indices offsets pooling_mode lxu_cache_locations uvm_cache_stats output_dtype is_experimental '
        'hash_indices offset_per_key rows_per_table',
        'Tensor'),
    'split_embedding_codegen_lookup_adagrad_function': (
        'placeholder_autograd_tensor dev_weights uvm_weights lxu_cache_weights weights_placements '
        'weights_offsets D_offsets total_D max_D hash_size_cumsum total_hash_size_bits indices offsets '
        'pooling_mode indice_weights feature_requires_grad lxu_cache_locations gradient_clipping max_gradient '
        'stochastic_rounding momentum1_dev momentum1_uvm momentum1_placements momentum1_offsets '
        'grad_accumulate grad_accumulate_offsets hash_indices unique_ids unique_offsets unique_inverse '
        'table_grad_accumulate_offsets eps learning_rate output_dtype B_offsets '
        'vbe_output_offsets_feature_rank vbe_B_offsets_rank_per_feature max_B max_B_feature_rank '
        'vbe_output_size is_experimental use_uniq_cache_locations_bwd use_homogeneous_placements '
        'uvm_cache_stats prev_iter_dev iter apply_global_weight_decay gwd_lower_bound use_optimize '
        'rows_per_table',
        'Tensor'),
    'split_embedding_codegen_lookup_adagrad_function_grad_aggregation': (
        'placeholder_autograd_tensor dev_weights uvm_weights lxu_cache_weights weights_placements '
        'weights_offsets D_offsets total_D max_D hash_size_cumsum total_hash_size_bits indices offsets '
        'indices_multi_step offsets_multi_step pooling_mode indice_weights feature_requires_grad '
        'lxu_cache_locations gradient_clipping max_gradient stochastic_rounding momentum1_dev momentum1_uvm '
        'momentum1_placements momentum1_offsets grad_accumulate grad_accumulate_offsets hash_indices '
        'unique_ids unique_offsets unique_inverse table_grad_accumulate_offsets table_offsets_multi '
        'unique_multi_step unique_offset_multi_step unique_inverse_multi_step eps learning_rate output_dtype '
        'B_offsets vbe_output_offsets_feature_rank vbe_B_offsets_rank_per_feature max_B max_B_feature_rank '
        'vbe_output_size is_experimental use_uniq_cache_locations_bwd use_homogeneous_placements '
        'uvm_cache_stats prev_iter_dev iter apply_global_weight_decay gwd_lower_bound use_optimize '
        'rows_per_table',
        'Tensor'),
    'split_embedding_codegen_lookup_adam_function': (
        'placeholder_autograd_tensor dev_weights uvm_weights lxu_cache_weights weights_placements '
        'weights_offsets D_offsets total_D max_D hash_size_cumsum total_hash_size_bits indices offsets '
        'pooling_mode indice_weights feature_requires_grad lxu_cache_locations gradient_clipping max_gradient '
        'stochastic_rounding momentum1_dev momentum1_uvm momentum1_placements momentum1_offsets momentum2_dev '
        'momentum2_uvm momentum2_placements momentum2_offsets grad_accumulate grad_accumulate_offsets '
        'hash_indices unique_ids unique_offsets unique_inverse table_grad_accumulate_offsets eps '
        'learning_rate beta1 beta2 weight_decay iter output_dtype B_offsets vbe_output_offsets_feature_rank '
        'vbe_B_offsets_rank_per_feature max_B max_B_feature_rank vbe_output_size is_experimental '
        'use_uniq_cache_locations_bwd use_homogeneous_placements uvm_cache_stats prev_iter_dev '
        'apply_global_weight_decay gwd_lower_bound use_optimize rows_per_table',
        'Tensor'),
    'split_embedding_codegen_lookup_adam_function_grad_aggregation': (
        'placeholder_autograd_tensor dev_weights uvm_weights lxu_cache_weights weights_placements '
        'weights_offsets D_offsets total_D max_D hash_size_cumsum total_hash_size_bits indices offsets '
        'indices_multi_step offsets_multi_step pooling_mode indice_weights feature_requires_grad '
        'lxu_cache_locations gradient_clipping max_gradient stochastic_rounding momentum1_dev momentum1_uvm '
        'momentum1_placements momentum1_offsets momentum2_dev momentum2_uvm momentum2_placements '
        'momentum2_offsets grad_accumulate grad_accumulate_offsets hash_indices unique_ids unique_offsets '
        'unique_inverse table_grad_accumulate_offsets table_offsets_multi unique_multi_step '
        'unique_offset_multi_step unique_inverse_multi_step eps learning_rate beta1 beta2 weight_decay iter '
        'output_dtype B_offsets vbe_output_offsets_feature_rank vbe_B_offsets_rank_per_feature max_B '
        'max_B_feature_rank vbe_output_size is_experimental use_uniq_cache_locations_bwd '
        'use_homogeneous_placements uvm_cache_stats prev_iter_dev apply_global_weight_decay gwd_lower_bound '
        'use_optimize rows_per_table',
        'Tensor'),
    'split_embedding_codegen_lookup_rowwise_adagrad_function': (
        'placeholder_autograd_tensor dev_weights uvm_weights lxu_cache_weights weights_placements '
        'weights_offsets D_offsets total_D max_D hash_size_cumsum total_hash_size_bits indices offsets '
        'pooling_mode indice_weights feature_requires_grad lxu_cache_locations gradient_clipping max_gradient '
        'stochastic_rounding momentum1_dev momentum1_uvm momentum1_placements momentum1_offsets eps '
        'learning_rate weight_decay weight_decay_mode max_norm output_dtype B_offsets '
        'vbe_output_offsets_feature_rank vbe_B_offsets_rank_per_feature max_B max_B_feature_rank '
        'vbe_output_size is_experimental use_uniq_cache_locations_bwd use_homogeneous_placements '
        'uvm_cache_stats prev_iter_dev iter apply_global_weight_decay gwd_lower_bound mixed_D grad_accumulate '
        'grad_accumulate_offsets hash_indices unique_ids unique_offsets unique_inverse '
        'table_grad_accumulate_offsets rows_per_table',
        'Tensor'),
    'split_embedding_codegen_lookup_sgd_function': (
        'placeholder_autograd_tensor dev_weights uvm_weights lxu_cache_weights weights_placements '
        'weights_offsets D_offsets total_D max_D hash_size_cumsum total_hash_size_bits indices offsets '
        'pooling_mode indice_weights feature_requires_grad lxu_cache_locations gradient_clipping max_gradient '
        'stochastic_rounding grad_accumulate grad_accumulate_offsets hash_indices unique_ids unique_offsets '
        'unique_inverse table_grad_accumulate_offsets learning_rate output_dtype B_offsets '
        'vbe_output_offsets_feature_rank vbe_B_offsets_rank_per_feature max_B max_B_feature_rank '
        'vbe_output_size is_experimental use_uniq_cache_locations_bwd use_homogeneous_placements '
        'uvm_cache_stats prev_iter_dev iter apply_global_weight_decay gwd_lower_bound use_optimize '
        'rows_per_table',
        'Tensor'),
    'split_embedding_codegen_lookup_sgd_function_grad_aggregation': (
        'placeholder_autograd_tensor dev_weights uvm_weights lxu_cache_weights weights_placements '
        'weights_offsets D_offsets total_D max_D hash_size_cumsum total_hash_size_bits indices offsets '
        'indices_multi_step offsets_multi_step pooling_mode indice_weights feature_requires_grad '
        'lxu_cache_locations gradient_clipping max_gradient stochastic_rounding grad_accumulate '
        'grad_accumulate_offsets hash_indices unique_ids unique_offsets unique_inverse '
        'table_grad_accumulate_offsets table_offsets_multi unique_multi_step unique_offset_multi_step '
        'unique_inverse_multi_step learning_rate output_dtype B_offsets vbe_output_offsets_feature_rank '
        'vbe_B_offsets_rank_per_feature max_B max_B_feature_rank vbe_output_size is_experimental '
        'use_uniq_cache_locations_bwd use_homogeneous_placements uvm_cache_stats prev_iter_dev iter '
        'apply_global_weight_decay gwd_lower_bound use_optimize rows_per_table',
        'Tensor'),
    'token_mixing': ('x gamma beta epsilon', 'Tensor'),
}


@pytest.mark.parametrize("name", sorted(OPERATOR_ARGUMENTS))
def test_operator_arguments_follow_the_reference(name):
    import recsdk_b200.ops.mxrec  # noqa: F401

    base, _, overload = name.partition(".")
    op = getattr(getattr(torch.ops.mxrec, base), overload or "default")
    want, returns = OPERATOR_ARGUMENTS[name]
    want = want.split()
    have = [a.name for a in op._schema.arguments]
    assert have[: len(want)] == want
    assert all(a.has_default_value() for a in op._schema.arguments[len(want):])        # additions must be optional
    n_ret = returns.count("Tensor") if returns.startswith("(") else 1
    assert len(op._schema.returns) == n_ret
    assert ("[]" in returns) == ("List" in str(op._schema.returns[0].type))


def test_optional_scalars_accept_none():
    """``target_group_size`` and ``alpha`` are ``int?`` / ``float?`` in the reference's attention schemas."""
    import recsdk_b200.ops.mxrec  # noqa: F401

    torch.manual_seed(0)
    q, k, v = (torch.randn(7, 2, 16) for _ in range(3))
    off = torch.tensor([0, 3, 7])
    a = torch.ops.mxrec.hstu_jagged(q, k, v, None, None, 0, 4, 0.0, off, None, None, None, None)
    assert torch.equal(a, torch.ops.mxrec.hstu_jagged(q, k, v, None, None, 0, 4, 0.0, off))
    g = torch.ops.mxrec.hstu_jagged_backward(torch.ones_like(a), q, k, v, None, None, 0, 4, 0.0, off, None, None, None, None)
    g2 = torch.ops.mxrec.hstu_jagged_backward(torch.ones_like(a), q, k, v, None, None, 0, 4, 0.0, off)
    assert all(torch.equal(x, y) for x, y in zip(g, g2))


PACKAGE_EXPORTS = {
    "recsdk_b200": ["HashEmbeddingBagCollection", "HashEmbeddingBagConfig", "HybridHashTable"],
    "recsdk_b200.sparse": ["JaggedTensorWithCount", "KeyedJaggedTensorWithCount", "ExtendedJaggedTensor", "KeyedExtendedJaggedTensor",
                           "JaggedTensorWithTimestamp", "KeyedJaggedTensorWithTimestamp", "JaggedTensor", "KeyedJaggedTensor", "KeyedTensor"],
    "recsdk_b200.parallel": ["HybridTrainPipelineSparseDist", "get_default_hybrid_sharders"],
    "recsdk_b200.embcache": ["Saver", "EmbCacheEmbeddingBagConfig", "EmbCacheEmbeddingConfig", "AdmitAndEvictConfig", "InitializerType",
                             "EmbCacheEmbeddingBagCollection", "EmbCacheEmbeddingCollection", "EmbCacheTrainPipelineSparseDist",
                             "EmbCacheEmbeddingBagCollectionSharder", "EmbCacheEmbeddingCollectionSharder"],
    "recsdk_b200.dynamic": ["DynamicEmbInitializerMode", "DynamicEmbInitializerArgs", "DynamicEmbCheckMode", "DynamicEmbTableOptions",
                            "DynamicEmbScoreStrategy", "DynamicEmbeddingCollectionSharder", "DynamicEmbeddingBagCollectionSharder",
                            "DynamicEmbParameterConstraints", "DynamicEmbeddingShardingPlanner", "DynamicEmbeddingEnumerator", "DynamicEmbDump",
                            "DynamicEmbLoad", "set_score", "get_score", "EmbOptimType", "__version__"],
}


@pytest.mark.parametrize("package", sorted(PACKAGE_EXPORTS))
def test_packages_export_what_the_reference_packages_export(package):
    """``hybrid_torchrec`` / ``hybrid_torchrec.sparse`` / ``hybrid_torchrec.distributed`` / ``torchrec_embcache(.distributed, .sparse)`` /
    ``dynamic_emb`` ``__init__`` files of the reference."""
    mod = importlib.import_module(package)
    assert [n for n in PACKAGE_EXPORTS[package] if not hasattr(mod, n)] == []
    with pytest.raises(AttributeError):
        getattr(importlib.import_module("recsdk_b200"), "no_such_name")


def test_jagged_tensors_with_counts_and_timestamps():
    from recsdk_b200.sparse import (JaggedTensorWithCount, JaggedTensorWithTimestamp, KeyedJaggedTensorWithCount,
                                    KeyedJaggedTensorWithTimestamp)

    a = JaggedTensorWithCount(torch.tensor([1, 2, 3]), lengths=torch.tensor([2, 1]), counts=torch.tensor([5, 6, 7]))
    b = JaggedTensorWithCount(torch.tensor([9]), lengths=torch.tensor([0, 1]), counts=torch.tensor([1]))
    k = KeyedJaggedTensorWithCount.from_jt_dict({"a": a, "b": b})
    assert k.counts.tolist() == [5, 6, 7, 1] and k.lengths().tolist() == [2, 1, 0, 1] and k.stride() == 2
    back = k.to_dict()
    assert isinstance(back["a"], JaggedTensorWithCount) and back["b"].counts.tolist() == [1] and back["a"].values().tolist() == [1, 2, 3]
    assert isinstance(a.to(torch.device("cpu")), JaggedTensorWithCount) and JaggedTensorWithCount(torch.tensor([1]), lengths=torch.tensor([1])).counts is None
    with pytest.raises(ValueError):
        JaggedTensorWithCount(torch.tensor([1, 2]), lengths=torch.tensor([2]), counts=torch.tensor([1]))
    with pytest.raises(ValueError):
        KeyedJaggedTensorWithCount.from_jt_dict({"a": a, "b": JaggedTensorWithCount(torch.tensor([9]), lengths=torch.tensor([0, 1]))})
    t = KeyedJaggedTensorWithTimestamp(keys=["a"], values=torch.tensor([1, 2]), lengths=torch.tensor([2]), timestamps=torch.tensor([10, 11]))
    jt = t.to_dict()["a"]
    assert isinstance(jt, JaggedTensorWithTimestamp) and jt.timestamps.tolist() == [10, 11]
    again = KeyedJaggedTensorWithTimestamp.from_jt_dict({"a": jt})
    assert again.timestamps.tolist() == [10, 11] and again.keys() == ["a"]


def test_dynamic_enumerator_lists_the_placements():
    from recsdk_b200.dynamic import (DynamicEmbeddingEnumerator, DynamicEmbeddingShardingPlanner, DynamicEmbParameterConstraints,
                                     DynamicEmbTableOptions, OptimizerType)
    from recsdk_b200.modules import EmbeddingBagCollection, EmbeddingBagConfig, EmbeddingCollection, EmbeddingConfig
    from recsdk_b200.parallel import ParameterConstraints, Topology

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.z_bags = EmbeddingBagCollection([EmbeddingBagConfig(num_embeddings=1000, embedding_dim=16, name="stat"),
                                                  EmbeddingBagConfig(num_embeddings=100_000, embedding_dim=16, name="dyn")],
                                                 device=torch.device("meta"))
            self.a_seq = EmbeddingCollection([EmbeddingConfig(num_embeddings=50, embedding_dim=8, name="seq")], device=torch.device("meta"))

    cons = {"dyn": DynamicEmbParameterConstraints(use_dynamicemb=True, dynamicemb_options=DynamicEmbTableOptions()),
            "stat": ParameterConstraints(sharding_types=["table_wise", "column_wise"])}
    topo = Topology(world_size=4)
    en = DynamicEmbeddingEnumerator(topo, 512, cons)
    opts = en.enumerate(M())
    by = {}
    for o in opts:
        by.setdefault(o.name, []).append(o)
    assert [o.module_path for o in opts][0] == "a_seq"                     # sorted by module path unless the exact order is asked for
    assert [o.sharding_type for o in by["seq"]] == ["row_wise", "table_wise", "data_parallel"]
    assert [o.sharding_type for o in by["stat"]] == ["table_wise"] and by["stat"][0].rows_per_rank == 1000
    d = by["dyn"]
    assert len(d) == 1 and d[0].is_dynamic and d[0].compute_kernel == "DynamicEmb" and d[0].rows_per_rank == 32768
    assert d[0].hbm_bytes_per_rank == 32768 * (16 + 4) * 4                   # row-wise Adagrad keeps 4 floats of state per row
    exact = DynamicEmbeddingEnumerator(topo, 512, cons, use_exact_enumerate_order=True).enumerate(M())
    assert exact[0].module_path == "z_bags"
    planner = DynamicEmbeddingShardingPlanner(M().z_bags.embedding_bag_configs(), cons, topo, enumerator=DynamicEmbeddingEnumerator(topo),
                                              optimizer_type=OptimizerType.ADAM)
    assert planner.enumerator.optimizer_type == OptimizerType.ADAM and "dyn" in planner.enumerator.constraints
    dyn = [o for o in planner.enumerator.enumerate(M()) if o.name == "dyn"][0]
    assert dyn.hbm_bytes_per_rank == planner._dyn_plan["dyn"].hbm_bytes_per_rank == 32768 * 48 * 4

    class RowWiseOnly:
        module_type = EmbeddingCollection

        def sharding_types(self, compute_device_type="cuda"):
            return ["row_wise"]

    only = DynamicEmbeddingEnumerator(topo).enumerate(M(), [RowWiseOnly()])
    assert [o.sharding_type for o in only if o.name == "seq"] == ["row_wise"]
    for bad in (dict(topology="cuda"), dict(topology=topo, batch_size=0), dict(topology=topo, constraints=[1])):
        with pytest.raises((TypeError, ValueError)):
            DynamicEmbeddingEnumerator(**bad)
