"""Weights from safetensors, by tensor name.

The reference merges every ``*.safetensors`` of the folder, sorted, later files
overwriting earlier names, and loads non-strictly (v10_triton_paged_gqa/llm.py:70-79,
src/torchlet/utils.py:5-38).  Here loading is strict: one error lists every missing
tensor, every unexpected tensor and every wrong shape.  Tensors keep the dtype they are
stored in (bfloat16 stays bfloat16, a 32-bit tensor stays 32-bit); integer tensors
become int32.
"""
from __future__ import annotations

from pathlib import Path

import torch

from ..logger import logger

# buffers some exporters write although they are recomputed at load
IGNORED_SUFFIXES = ("rotary_emb.inv_freq",)


class WeightsError(ValueError):
    """The checkpoint does not fit the model.  ``missing``, ``unexpected`` and
    ``wrong_shape`` hold the details the message lists."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = ["the checkpoint does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {tuple(got)}, expected {tuple(want)}")
        for name, got in self.wrong_dtype:
            lines.append(f"  unsupported dtype: {name} is {got}")
        super().__init__("\n".join(lines))


def read_safetensors(model_dir: str | Path) -> dict:
    """All tensors of all ``*.safetensors`` files in ``model_dir``, on the CPU."""
    from safetensors import safe_open

    files = sorted(Path(model_dir).glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors files found in {model_dir}")
    tensors = {}
    for file in files:
        with safe_open(str(file), framework="pt", device="cpu") as handle:
            for name in handle.keys():
                tensors[name] = handle.get_tensor(name)
    return tensors


def check_and_normalise(tensors: dict, expected: list) -> dict:
    """Check names and shapes against ``expected`` (``TensorSpec`` list); returns the
    tensors with integer tables as int32.  Raises ``WeightsError`` listing everything
    that is wrong at once."""
    wanted = {spec.name: spec for spec in expected}
    missing = [s.name for s in expected if s.name not in tensors and not s.optional]
    unexpected = [n for n in tensors if n not in wanted and not n.endswith(IGNORED_SUFFIXES)]
    wrong_shape, wrong_dtype, out = [], [], {}
    for name, tensor in tensors.items():
        spec = wanted.get(name)
        if spec is None:
            continue
        if tuple(tensor.shape) != tuple(spec.shape):
            wrong_shape.append((name, tensor.shape, spec.shape))
            continue
        if tensor.is_floating_point():
            if tensor.dtype not in (torch.bfloat16, torch.float32, torch.float16, torch.float64):
                wrong_dtype.append((name, tensor.dtype))
                continue
            if tensor.dtype in (torch.float16, torch.float64):
                tensor = tensor.to(torch.float32)
        elif tensor.dtype != torch.bool:
            tensor = tensor.to(torch.int32)
        out[name] = tensor
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightsError(missing, unexpected, wrong_shape, wrong_dtype)
    return out


def load_checkpoint(model_dir: str | Path, expected: list) -> dict:
    tensors = check_and_normalise(read_safetensors(model_dir), expected)
    logger.info("loaded %d tensors from %s", len(tensors), model_dir)
    if logger.isEnabledFor(10):  # DEBUG: the whole table, as the reference logs it
        from ..utils import get_weights_info

        logger.debug("weight info:\n%s", get_weights_info(tensors))
    return tensors
