from .clt_config import CLTConfig, TrainingConfig, InferenceConfig, canonical_normalization
from .data_config import ActivationConfig

__all__ = ["CLTConfig", "TrainingConfig", "InferenceConfig", "ActivationConfig", "canonical_normalization"]
