"""Hard limits of the configuration checks, under the reference's names (``hybrid_torchrec/constants.py:8-16``), and its
``check`` helper (``hybrid_torchrec/utils.py``)."""
from .embcache.train_pipeline import MAX_LOCAL_UNIQUE_PARALLEL_BATCH_NUM
from .modules.embedding_configs import EMBEDDING_DIM_ALIGN as EMBEDDINGS_DIM_ALIGNMENT
from .modules.embedding_configs import MAX_EMBEDDING_DIM as MAX_EMBEDDINGS_DIM
from .modules.embedding_configs import MAX_NUM_EMBEDDINGS

MAX_NUM_TABLES = 10000
MAX_MULTI_HOT_SIZE = 102400
MAX_WORLD_SIZE = 10000
MAX_BATCH_SIZE = 102400
MAX_CACHINE_MEM_SIZE = 64 * 1024 * 1024 * 1024          # bytes of device memory a multi-tier cache may take (name as in the reference)


def check(check_flag: bool, error_msg: str) -> None:
    """Raise ``ValueError(error_msg)`` unless ``check_flag`` holds."""
    if not check_flag:
        raise ValueError(error_msg)


__all__ = ["MAX_NUM_EMBEDDINGS", "MAX_EMBEDDINGS_DIM", "EMBEDDINGS_DIM_ALIGNMENT", "MAX_NUM_TABLES", "MAX_MULTI_HOT_SIZE", "MAX_WORLD_SIZE",
           "MAX_BATCH_SIZE", "MAX_CACHINE_MEM_SIZE", "MAX_LOCAL_UNIQUE_PARALLEL_BATCH_NUM", "check"]
