from .base_store import BaseActivationStore, LayerBatch
from .sampler import ChunkRowSampler
from .manifest_activation_store import ManifestActivationStore
from .local_activation_store import LocalActivationStore
from .remote_activation_store import RemoteActivationStore
from .memory_store import InMemoryActivationStore
from .activation_store_factory import create_activation_store

__all__ = [
    "BaseActivationStore", "LayerBatch", "ChunkRowSampler", "ManifestActivationStore", "LocalActivationStore",
    "RemoteActivationStore", "InMemoryActivationStore", "create_activation_store",
]
