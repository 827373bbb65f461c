"""Small helpers the entry point logs with: a table of the checkpoint's tensors and a
summary of the backend (the reference's get_weights_info / get_backend_info,
src/torchlet/utils.py:41-73)."""
from __future__ import annotations

import torch


def get_weights_info(weights: dict) -> str:
    """One line per tensor: name, shape, dtype, aligned in columns."""
    rows = [(name, str(tuple(t.shape)), str(t.dtype)) for name, t in weights.items()]
    if not rows:
        return ""
    name_width = max(len(r[0]) for r in rows)
    shape_width = max(len(r[1]) for r in rows)
    return "\n".join(f"{name:<{name_width}}\t{shape:<{shape_width}}\t{dtype}" for name, shape, dtype in rows)


def get_backend_info() -> str:
    cuda = torch.cuda.is_available()
    lines = [f"torch: {torch.__version__}", f"cuda: {cuda}"]
    if cuda:
        props = torch.cuda.get_device_properties(0)
        lines += [f"device: {props.name}", f"compute capability: {props.major}.{props.minor}",
                  f"sms: {props.multi_processor_count}", f"memory: {props.total_memory / 2**30:.1f} GiB"]
    lines.append(f"num_threads: {torch.get_num_threads()}")
    return "\n".join(lines)
