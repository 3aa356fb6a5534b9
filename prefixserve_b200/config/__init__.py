from .llama import Llama3RopeScaling, LlamaConfig, UnsupportedModelError
from .gekopel import BiasedAttentionConfig, DeltaConfig, DenseFF, GekopelConfig, GekopelLayer, RoutedFF
from .goganex import AttentionConfig, ClippedFF, GoganexConfig, GoganexLayer, ParallelConfig, RotationConfig
from .zomolix import ZomolixConfig, ZomolixLayer
from .nerenex import LatentAttentionConfig, NerenexConfig, NerenexLayer, RecurrentConfig
from .registry import (
    Architecture,
    UnknownArchitectureError,
    architecture_of,
    get_architecture,
    read_model_folder,
    register_architecture,
    registered_architectures,
)
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec, part, sequential_schedule

__all__ = [
    "Architecture", "AttentionConfig", "ClippedFF", "GoganexConfig", "GoganexLayer", "ParallelConfig", "RotationConfig", "BiasedAttentionConfig", "DeltaConfig", "DenseFF", "GekopelConfig", "GekopelLayer", "RoutedFF", "LatentAttentionConfig", "LayerCall", "LayerSpec", "Llama3RopeScaling", "LlamaConfig", "ModelSpec",
    "NerenexConfig", "NerenexLayer", "ZomolixConfig", "ZomolixLayer", "PartSpec", "RecurrentConfig",
    "UnknownArchitectureError", "UnsupportedModelError", "architecture_of", "get_architecture", "part",
    "read_model_folder", "register_architecture", "registered_architectures", "sequential_schedule",
]
