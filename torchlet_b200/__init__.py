"""torchlet_b200: a small, whole LLM inference engine for one NVIDIA B200.

``LLM`` and ``SamplingParams`` are the user's entry; ``torchlet_b200.engine`` holds the
step function, scheduler and trace replay; ``torchlet_b200.parts`` the layer parts;
``torchlet_b200.cache`` the paged cache; ``torchlet_b200.csrc`` the CUDA kernels.
"""
from .sampling import SamplingParams

__all__ = ["LLM", "SamplingParams"]


def __getattr__(name):
    if name == "LLM":
        from .llm import LLM

        return LLM
    raise AttributeError(name)
