"""Small helpers shared by the training code and the scripts (reference: clt/training/utils.py)."""
from __future__ import annotations

import numpy as np
import torch

__all__ = ["format_elapsed_time", "torch_bfloat16_to_numpy_uint16", "numpy_uint16_to_torch_bfloat16"]


def format_elapsed_time(seconds: float) -> str:
    """``MM:SS`` below one hour, ``HH:MM:SS`` from there on (hours keep counting past a day)."""
    total = max(0, int(seconds))
    hours, rest = divmod(total, 3600)
    minutes, secs = divmod(rest, 60)
    return f"{hours:02d}:{minutes:02d}:{secs:02d}" if hours else f"{minutes:02d}:{secs:02d}"


def torch_bfloat16_to_numpy_uint16(x: torch.Tensor) -> np.ndarray:
    """The bit pattern of a bf16 tensor as a ``uint16`` array of the same shape (numpy has no bf16): a view of the
    tensor's own bytes, no conversion through fp32.  This is how bf16 activations are written to HDF5 chunks."""
    if x.dtype != torch.bfloat16:
        raise TypeError(f"expected a bfloat16 tensor, got {x.dtype}")
    return x.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def numpy_uint16_to_torch_bfloat16(a: np.ndarray) -> torch.Tensor:
    """Inverse of :func:`torch_bfloat16_to_numpy_uint16` (copies, so that the result owns its memory)."""
    arr = np.ascontiguousarray(a, dtype=np.uint16)
    return torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
