"""Configuration of the multi-tier ("embcache") embedding tables: a device-memory cache of hot rows in front of
the full table in host DRAM, with optional admission and eviction of features.

Field names and defaults follow the reference (``torchrec_embcache/distributed/configs.py:33-143`` admission /
eviction, ``:164-205`` limits, ``:208-236`` table configs).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Optional

from ..modules.embedding_configs import EmbeddingBagConfig, EmbeddingConfig

POLICY_COUNT = "count"
POLICY_SHOW_CLICK = "show_click"
MIN_EVICT_STEP_INTERVAL = 10


class AdmitAndEvictPolicyType(str, enum.Enum):
    """Admission / eviction policy; members compare equal to the plain strings ``"count"`` / ``"show_click"``."""
    POLICY_COUNT = POLICY_COUNT
    POLICY_SHOWCLICK = POLICY_SHOW_CLICK


class InitializerType(enum.Enum):
    LINEAR = "linear"
    TRUNCATED_NORMAL = "truncated_normal"
    UNIFORM = "uniform"


@dataclass
class ShowClickParams:
    """score = alpha * shows + beta * clicks; a feature is admitted once its score reaches ``admit_threshold`` (> 0 turns
    admission on), the ``evict_percentage`` (> 0 turns eviction on) lowest-scored features are evicted, scores decay by
    ``score_decay`` per eviction round (``torchrec_embcache/distributed/configs.py:33-43`` of the reference)."""
    alpha: float = 1.0
    beta: float = 0.0
    admit_threshold: float = 0.0
    evict_percentage: float = 0.0
    score_decay: float = 1.0


@dataclass
class AdmitAndEvictConfig:
    admit_threshold: int = -1                 # count policy: a key is admitted once seen this many times
    not_admitted_default_value: float = 0.0
    evict_threshold: int = -1                 # seconds since the key was last seen
    evict_step_interval: int = -1
    policy_type: str = POLICY_COUNT
    show_click_params: ShowClickParams = field(default_factory=ShowClickParams)
    showclick_params: Optional[ShowClickParams] = None     # the reference's spelling of the same field; wins when given

    def __post_init__(self) -> None:
        if isinstance(self.policy_type, AdmitAndEvictPolicyType):
            self.policy_type = self.policy_type.value
        if self.policy_type not in (POLICY_COUNT, POLICY_SHOW_CLICK):
            raise ValueError("policy_type must be %r or %r" % (POLICY_COUNT, POLICY_SHOW_CLICK))
        for name in ("admit_threshold", "evict_threshold", "evict_step_interval"):
            v = getattr(self, name)
            if v is None:
                setattr(self, name, -1)
            elif not isinstance(v, int) or isinstance(v, bool):
                raise TypeError("%s must be int or None, but got %s" % (name, type(v)))
        if self.not_admitted_default_value is not None and not isinstance(self.not_admitted_default_value, float):
            raise TypeError("not_admitted_default_value must be float or None, but got %s" % type(self.not_admitted_default_value))
        if self.admit_threshold < -1 or self.evict_threshold < -1:
            raise ValueError("thresholds must be -1 / 0 (off) or positive")
        if self.evict_step_interval not in (-1, 0) and self.evict_step_interval < MIN_EVICT_STEP_INTERVAL:
            raise ValueError("evict_step_interval must be -1 / 0 (off) or >= %d" % MIN_EVICT_STEP_INTERVAL)
        if self.showclick_params is not None:
            self.show_click_params = self.showclick_params
        self.showclick_params = self.show_click_params                  # one object under both names
        p = self.show_click_params
        if not (0.0 <= p.evict_percentage <= 1.0) or not (0.0 < p.score_decay <= 1.0):
            raise ValueError("evict_percentage must be in [0, 1] and score_decay in (0, 1]")

    def is_admit_enabled(self) -> bool:
        if self.policy_type == POLICY_SHOW_CLICK:
            return self.show_click_params.admit_threshold > 0
        return self.admit_threshold > 0

    def is_evict_enabled(self) -> bool:
        if self.policy_type == POLICY_SHOW_CLICK:
            return self.show_click_params.evict_percentage > 0
        return self.evict_threshold > 0

    def is_feature_filter_enabled(self) -> bool:
        return self.is_admit_enabled() or self.is_evict_enabled()

    # the reference's names of the same predicates (``configs.py:116-143``)
    def is_feature_admit_enabled(self) -> bool:
        return self.is_admit_enabled()

    def is_feature_evict_enabled(self) -> bool:
        return self.is_evict_enabled()

    def is_showclick_policy(self) -> bool:
        return self.policy_type == POLICY_SHOW_CLICK

    def is_showclick_admit_enabled(self) -> bool:
        return self.is_showclick_policy() and self.show_click_params.admit_threshold > 0

    def is_showclick_evict_enabled(self) -> bool:
        return self.is_showclick_policy() and self.show_click_params.evict_percentage > 0

    def is_showclick_filter_enabled(self) -> bool:
        return self.is_showclick_admit_enabled() or self.is_showclick_evict_enabled()


@dataclass
class EmbCacheEmbeddingBagConfig(EmbeddingBagConfig):
    weight_init_mean: float = 0.0
    weight_init_stddev: float = 0.05
    initializer_type: InitializerType = InitializerType.LINEAR
    admit_and_evict_config: AdmitAndEvictConfig = field(default_factory=AdmitAndEvictConfig)
    is_incremental: bool = False


@dataclass
class EmbCacheEmbeddingConfig(EmbeddingConfig):
    weight_init_mean: float = 0.0
    weight_init_stddev: float = 0.05
    initializer_type: InitializerType = InitializerType.LINEAR
    admit_and_evict_config: AdmitAndEvictConfig = field(default_factory=AdmitAndEvictConfig)
    is_incremental: bool = False
