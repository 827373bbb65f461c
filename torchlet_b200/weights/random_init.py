"""Random weights: writes a model folder (config.json + model.safetensors) from a
configuration and a seed, so that everything downstream goes through the loader.

Matrices, embeddings and biases are N(0, std); norm weights are 1 + N(0, norm_std)
(norm_std 0 gives exact ones).  Tensors are drawn on the CPU in float32 in the order of
the model's expected-tensor list from one ``torch.Generator(seed)``, then cast.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..parts import expected_tensors

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32}


def random_tensors(config, seed: int, std: float = 0.02, norm_std: float = 0.0, dtype="bfloat16",
                   device="cpu") -> dict:
    """Tensors by name.  ``device``: where they are drawn and left (a CUDA device draws
    other numbers than the CPU for the same seed; large models are drawn there)."""
    torch_dtype = _DTYPES[dtype] if isinstance(dtype, str) else dtype
    spec = config.model_spec()
    generator = torch.Generator(device=device).manual_seed(int(seed))
    tensors = {}
    for want in expected_tensors(spec):
        if want.optional:  # tied LM head: not stored
            continue
        if want.init == "ones":
            value = torch.ones(want.shape, dtype=torch.float32, device=device)
            if norm_std:
                value += torch.randn(want.shape, generator=generator, dtype=torch.float32, device=device) * norm_std
        else:
            value = torch.randn(want.shape, generator=generator, dtype=torch.float32, device=device) * std
        tensors[want.name] = value.to(torch_dtype)
    return tensors


def write_random_model(folder, config, seed: int, std: float = 0.02, norm_std: float = 0.0,
                       dtype="bfloat16") -> Path:
    """Write ``config.json`` and ``model.safetensors`` into ``folder``; returns it."""
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    tensors = random_tensors(config, seed, std, norm_std, dtype)
    raw = config.to_dict()
    raw["torch_dtype"] = "bfloat16" if tensors[next(iter(tensors))].dtype == torch.bfloat16 else "float32"
    (folder / "config.json").write_text(json.dumps(raw, indent=2) + "\n")
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder
