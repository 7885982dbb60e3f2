"""Shared utilities: logging, validators, rank information, CPU binding."""
from .bind_cpu import bind_cpu, bind_current_process, bind_rank_from_env, cores_for_rank
from .log import LoggingProxy, logger
from .rank_info import RankInfo, rank_info_from_env, rank_info_from_table
from .validator import (DirectoryValidator, StringValidator, ValidationError, Validator, float_safe_check, int_safe_check,
                        path_safe_check, str_safe_check)

__all__ = ["bind_cpu", "bind_current_process", "bind_rank_from_env", "cores_for_rank", "LoggingProxy", "logger", "RankInfo", "rank_info_from_env",
           "rank_info_from_table", "DirectoryValidator", "StringValidator", "ValidationError", "Validator", "float_safe_check",
           "int_safe_check", "path_safe_check", "str_safe_check"]
