"""B200-native cross-layer transcoder framework."""
from .config import CLTConfig, TrainingConfig, InferenceConfig, ActivationConfig
from .models import CrossLayerTranscoder

__version__ = "0.1.0"
__all__ = ["CLTConfig", "TrainingConfig", "InferenceConfig", "ActivationConfig", "CrossLayerTranscoder"]
