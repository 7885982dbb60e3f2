"""Shared utilities: logging, validators, rank information, CPU binding."""
from .bind_cpu import (bind_cpu, bind_cpu_task, bind_current_process, bind_rank_from_env, cores_for_rank,
                       get_available_cpu_num_and_range)
from .log import LoggingProxy, logger
from .rank_info import (RankInfo, get_device_id, get_device_list, get_local_rank_size, get_min_device_id, get_rank_id, get_rank_size,
                        get_rank_to_device_dict, rank_info_from_env, rank_info_from_table)
from .validator import (DirectoryValidator, StringValidator, ValidationError, Validator, class_safe_check, dir_safe_check,
                        file_safe_check, float_safe_check, int_safe_check, path_safe_check, str_safe_check)

__all__ = ["bind_cpu_task", "get_available_cpu_num_and_range", "get_device_id", "get_device_list", "get_local_rank_size",
           "get_min_device_id", "get_rank_id", "get_rank_size", "get_rank_to_device_dict", "class_safe_check", "dir_safe_check",
           "file_safe_check", "bind_cpu", "bind_current_process", "bind_rank_from_env", "cores_for_rank", "LoggingProxy", "logger", "RankInfo", "rank_info_from_env",
           "rank_info_from_table", "DirectoryValidator", "StringValidator", "ValidationError", "Validator", "float_safe_check",
           "int_safe_check", "path_safe_check", "str_safe_check"]
