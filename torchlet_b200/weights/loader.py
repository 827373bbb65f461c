"""Weights from safetensors, by tensor name.

The reference merges every ``*.safetensors`` of the folder, sorted, later files
overwriting earlier names, and loads non-strictly (v10_triton_paged_gqa/llm.py:70-79,
src/torchlet/utils.py:5-38).  Here loading is strict: one error lists every missing
tensor, every unexpected tensor and every wrong shape.  Tensors keep the dtype they are
stored in (bfloat16 stays bfloat16, a 32-bit tensor stays 32-bit); integer tensors
become int32.  A sharded checkpoint's ``*.safetensors.index.json`` is honoured, and tensors are
read one at a time when the model takes them (``LazyCheckpoint``), so that a large checkpoint
is never held twice on the host.
"""
from __future__ import annotations

from collections.abc import Mapping
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


_SAFETENSORS_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "F64": torch.float64,
                       "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
                       "BOOL": torch.bool}


def _checkpoint_files(model_dir: Path) -> dict:
    """Tensor name -> file.  A ``*.safetensors.index.json`` (the sharded layout's table of
    contents) decides where it exists; else every ``*.safetensors`` of the folder, sorted, later
    files overwriting earlier names, as the reference merges them (v10_triton_paged_gqa/llm.py:70-79)."""
    import json

    from safetensors import safe_open

    indexes = sorted(model_dir.glob("*.safetensors.index.json"))
    if indexes:
        weight_map = json.loads(indexes[0].read_text()).get("weight_map", {})
        absent = sorted({f for f in weight_map.values() if not (model_dir / f).is_file()})
        if absent:
            raise FileNotFoundError(f"{indexes[0].name} names files that are not in {model_dir}: {', '.join(absent)}")
        return {name: model_dir / file for name, file in weight_map.items()}
    files = sorted(model_dir.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors files found in {model_dir}")
    where = {}
    for file in files:
        with safe_open(str(file), framework="pt", device="cpu") as handle:
            for name in handle.keys():
                where[name] = file
    return where


def _normalise(tensor: torch.Tensor) -> torch.Tensor:
    """16- and 64-bit floats other than bfloat16 become float32, integer tables int32."""
    if tensor.is_floating_point():
        return tensor.to(torch.float32) if tensor.dtype in (torch.float16, torch.float64) else tensor
    return tensor if tensor.dtype == torch.bool else tensor.to(torch.int32)


class LazyCheckpoint(Mapping):
    """The tensors of a model folder by name, read from the (memory-mapped) files one at a time
    when asked for, so that the host never holds the checkpoint twice.  ``meta(name)`` gives
    shape and dtype without reading the tensor."""

    def __init__(self, where: dict, only=None):
        self._where = {name: file for name, file in where.items() if only is None or name in only}
        self._handles: dict = {}

    def _handle(self, name: str):
        from safetensors import safe_open

        file = self._where[name]
        handle = self._handles.get(file)
        if handle is None:
            handle = self._handles[file] = safe_open(str(file), framework="pt", device="cpu").__enter__()
        return handle

    def meta(self, name: str) -> tuple:
        piece = self._handle(name).get_slice(name)
        return tuple(piece.get_shape()), _SAFETENSORS_DTYPES.get(piece.get_dtype(), piece.get_dtype())

    def __getitem__(self, name: str) -> torch.Tensor:
        return _normalise(self._handle(name).get_tensor(name))

    def __iter__(self):
        return iter(self._where)

    def __len__(self) -> int:
        return len(self._where)

    def restricted(self, names) -> "LazyCheckpoint":
        out = LazyCheckpoint(self._where, only=set(names))
        out._handles = self._handles
        return out


def read_safetensors(model_dir: str | Path) -> dict:
    """All tensors of the folder's checkpoint, on the CPU, as an ordinary dict."""
    lazy = LazyCheckpoint(_checkpoint_files(Path(model_dir)))
    return {name: lazy._handle(name).get_tensor(name) for name in lazy}


def check_and_normalise(tensors, expected: list):
    """Check names and shapes against ``expected`` (``TensorSpec`` list); returns the
    tensors with integer tables as int32 (for a ``LazyCheckpoint``: itself, restricted to the
    expected names; nothing is read).  Raises ``WeightsError`` listing everything that is wrong
    at once."""
    lazy = isinstance(tensors, LazyCheckpoint)
    wanted = {spec.name: spec for spec in expected}
    missing = [s.name for s in expected if s.name not in tensors and not s.optional]
    unexpected = [n for n in tensors if n not in wanted and not n.endswith(IGNORED_SUFFIXES)]
    wrong_shape, wrong_dtype, out = [], [], {}
    floats = (torch.bfloat16, torch.float32, torch.float16, torch.float64)
    for name in tensors:
        spec = wanted.get(name)
        if spec is None:
            continue
        shape, dtype = tensors.meta(name) if lazy else (tuple(tensors[name].shape), tensors[name].dtype)
        if tuple(shape) != tuple(spec.shape):
            wrong_shape.append((name, shape, spec.shape))
            continue
        is_float = isinstance(dtype, torch.dtype) and dtype.is_floating_point
        if not isinstance(dtype, torch.dtype) or dtype.is_complex or (is_float and dtype not in floats):
            wrong_dtype.append((name, dtype))
            continue
        if not lazy:
            out[name] = _normalise(tensors[name])
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightsError(missing, unexpected, wrong_shape, wrong_dtype)
    return tensors.restricted(wanted) if lazy else out


def load_checkpoint(model_dir: str | Path, expected: list) -> LazyCheckpoint:
    """The folder's tensors, checked against ``expected``; each is read when the model takes it."""
    tensors = check_and_normalise(LazyCheckpoint(_checkpoint_files(Path(model_dir))), expected)
    logger.info("found %d tensors in %s", len(tensors), model_dir)
    if logger.isEnabledFor(10):  # DEBUG: the whole table, as the reference logs it
        lines = [f"{name}  {'x'.join(map(str, tensors.meta(name)[0]))}  {tensors.meta(name)[1]}" for name in tensors]
        logger.debug("weight info:\n%s", "\n".join(lines))
    return tensors
