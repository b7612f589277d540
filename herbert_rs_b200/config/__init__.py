"""Typed configurations and the specs that parts are built from."""

from .base import Reader, read_config_json
from .qwen3 import Qwen3Config
from .kebisun import KebisunConfig
from .specs import (AttentionSpec, BlockSpec, GatedLinearAttentionSpec, LatentAttentionSpec, ModelSpec, NormSpec,
                    PositionSpec, RoutedFFSpec, ScaledRotarySpec, ScheduleStep, SwiGLUSpec, identity_schedule)

__all__ = [
    "Reader", "read_config_json", "Qwen3Config", "KebisunConfig", "AttentionSpec", "GatedLinearAttentionSpec",
    "LatentAttentionSpec", "RoutedFFSpec", "ScaledRotarySpec", "BlockSpec", "ModelSpec",
    "NormSpec", "PositionSpec", "ScheduleStep", "SwiGLUSpec", "identity_schedule",
]
