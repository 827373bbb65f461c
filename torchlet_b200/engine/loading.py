"""From a model folder (config.json + safetensors) to a model laid out on the device.

The model class is chosen by ``config.json`` through the architecture registry, the
tensors are read by name and checked against what the model's parts expect
(the reference: v10_triton_paged_gqa/llm.py:34-57).
"""
from __future__ import annotations

from pathlib import Path

import torch

from ..config import load_config
from ..logger import logger
from ..parts import LayeredModel, expected_tensors
from ..weights import check_and_normalise, load_checkpoint

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32}


def build_model(config, tensors: dict, dtype, device="cuda:0") -> LayeredModel:
    """A ``LayeredModel`` from a typed configuration and tensors by name (any device)."""
    spec = config.model_spec()
    tensors = check_and_normalise(tensors, expected_tensors(spec))
    torch_dtype = TORCH_DTYPES[dtype] if isinstance(dtype, str) else dtype
    if torch_dtype == torch.bfloat16:
        if hasattr(tensors, "meta"):  # a lazy checkpoint: shapes and dtypes without reading anything
            wide = [n for n in tensors if len(tensors.meta(n)[0]) >= 2 and tensors.meta(n)[1] == torch.float32]
        else:
            wide = [n for n, t in tensors.items() if t.dim() >= 2 and t.dtype == torch.float32]
        if wide:
            logger.warning("%d matrices stored in 32-bit are rounded to bfloat16 for the bfloat16 kernels", len(wide))
    model = LayeredModel(spec)
    model.load(tensors, device, torch_dtype)
    model.config = config
    return model


def load_model(model_dir: str | Path, dtype="bfloat16", device="cuda:0") -> LayeredModel:
    config = load_config(model_dir)
    spec = config.model_spec()
    tensors = load_checkpoint(model_dir, expected_tensors(spec))
    return build_model(config, tensors, dtype, device)
