from .generator import ActivationGenerator
from .synthetic import SparseDictionarySynth, SyntheticSpec, write_synthetic_dataset

__all__ = ["ActivationGenerator", "SparseDictionarySynth", "SyntheticSpec", "write_synthetic_dataset"]
