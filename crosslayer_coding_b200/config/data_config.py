"""Configuration of activation generation (reference: clt/config/data_config.py:8-99).

HDF5 output does not need h5py here: chunks are written by the framework's own
HDF5 writer (``crosslayer_coding_b200.io.hdf5``).
"""
from __future__ import annotations

import dataclasses
import logging
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

logger = logging.getLogger(__name__)


@dataclass
class ActivationConfig:
    model_name: str
    mlp_input_module_path_template: str
    mlp_output_module_path_template: str
    dataset_path: str
    model_dtype: Optional[str] = None
    activation_dtype: str = "bfloat16"
    dataset_split: str = "train"
    dataset_text_column: str = "text"
    context_size: int = 128
    inference_batch_size: int = 512
    exclude_special_tokens: bool = True
    prepend_bos: bool = False
    streaming: bool = True
    dataset_trust_remote_code: bool = False
    cache_path: Optional[str] = None
    target_total_tokens: Optional[int] = None
    activation_dir: str = "./activations"
    output_format: str = "hdf5"
    compression: Optional[str] = "gzip"
    chunk_token_threshold: int = 1_000_000
    compute_norm_stats: bool = True
    remote_server_url: Optional[str] = None
    delete_after_upload: bool = False
    upload_max_retries: int = 5
    upload_initial_backoff: float = 1.0
    upload_max_backoff: float = 30.0
    nnsight_tracer_kwargs: Dict[str, Any] = field(default_factory=dict)
    nnsight_invoker_args: Dict[str, Any] = field(default_factory=dict)
    enable_profiling: bool = False

    def __post_init__(self) -> None:
        assert self.context_size > 0, "Context size must be positive"
        assert self.inference_batch_size > 0, "Inference batch size must be positive"
        assert self.chunk_token_threshold > 0, "Chunk token threshold must be positive"
        assert self.activation_dtype in ("bfloat16", "float16", "float32"), (
            f"Invalid activation_dtype: {self.activation_dtype}"
        )
        assert self.output_format in ("hdf5", "npz"), f"Invalid output_format: {self.output_format}"
        if self.compression not in ("lz4", "gzip", None, False):
            logger.warning("Unsupported compression %r; chunks will be written uncompressed.", self.compression)

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)
