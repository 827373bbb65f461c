"""What the entry point logs about a checkpoint and about the machine.  The reference logs
the same two things (a table of the weights, a summary of the backend: src/torchlet/utils.py:41-73);
the form here is this package's own."""
from __future__ import annotations

import torch


def get_weights_info(weights: dict) -> str:
    """A table of the checkpoint's tensors (name, shape, dtype, size) and their total."""
    if not weights:
        return "(no tensors)"
    entries = []
    total = 0
    for name, tensor in weights.items():
        nbytes = tensor.numel() * tensor.element_size()
        total += nbytes
        entries.append((name, "x".join(map(str, tensor.shape)) or "scalar", str(tensor.dtype).replace("torch.", ""),
                        f"{nbytes / 2**20:.2f} MiB"))
    widths = [max(len(entry[i]) for entry in entries) for i in range(4)]
    lines = ["  ".join(cell.ljust(width) for cell, width in zip(entry, widths)).rstrip() for entry in entries]
    lines.append(f"{len(entries)} tensors, {total / 2**30:.3f} GiB")
    return "\n".join(lines)


def get_backend_info() -> str:
    """torch's version and, where there is a GPU, its name, capability, SM count and memory."""
    parts = {"torch": torch.__version__, "host threads": torch.get_num_threads()}
    if torch.cuda.is_available():
        props = torch.cuda.get_device_properties(torch.cuda.current_device())
        parts.update({"gpu": props.name, "sm": f"{props.major}{props.minor}", "sm count": props.multi_processor_count,
                      "gpu memory": f"{props.total_memory / 2**30:.0f} GiB"})
    else:
        parts["gpu"] = "none"
    return ", ".join(f"{key} {value}" for key, value in parts.items())
